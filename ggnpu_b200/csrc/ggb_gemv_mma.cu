// Decode GEMV for Q4_K in the row-group-major layout, M <= 2 activation rows:
//   y[m][n] = sum_k x[m][k] * W[n][k]          (mul_mat_weight, src/cli/main.cpp:1367-1434)
//
// Still an HBM-bound streaming kernel (each weight byte crosses HBM once), but the products run on
// the int8 tensor-core path so that the instruction stream stays far below the issue limit:
//   * x is RMS-normalised (optional), then split into three int8 limbs per value with one scale per
//     256 values, x ~ s*(l1 + l2/128 + l3/16384), error <= 2^-22 of the block maximum.  The limbs
//     of the (at most two) rows form the 8 columns of the B operand: column 3m+p = limb p of row m.
//   * A tile is 16 weight rows x `sb` blocks of 256.  Its quant bytes arrive (bulk async copy into a
//     shared-memory ring, one mbarrier per stage) already ordered as m16n8k32 A fragments: one
//     16-byte shared load per lane feeds two mma instructions -- low nibbles as s8, high nibbles in
//     place as u8 (value 16*q, the factor 1/16 is folded into the scale).
//   * The 6-bit sub-block scales multiply the int32 mma results in the integer domain; one float
//     conversion per 256-block applies d * scale(x).  The min term dmin*m*sum(x) is formed once per
//     (row, block) from the decoded header.
//   * One consumer warp owns one tile at a time (8 tiles in flight per CTA plus the ring's
//     prefetch); tiles of the same 16 rows are combined through shared memory by whichever warp
//     finishes last, which also applies the epilogue (bias / residual / SwiGLU) and stores y.
//   * Launched with programmatic dependent launch: the producer streams weights at once, consumers
//     execute griddepcontrol.wait before reading x.
// All mbarrier waits are bounded; a timeout sets the context's device error word.
#include <stdlib.h>

#include "ggb_internal.h"

namespace ggb {

namespace {

// kWarps consumer warps (8: each keeps 166 registers and a deep private ring) plus one producer warp.
constexpr int kMaxStages = 64;
constexpr uint32_t kSpinLimit = 1u << 17;         // each poll can suspend for microseconds: about half a second in all

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err, int code) {
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(err, code);
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <int kWarps>
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory"); }

// C[16x8] = A[16x32] * B[32x8], int8 in, int32 out (C starts from zero).
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    const int z = 0;
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    const int z = 0;
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
}

// C[16x8] = A[16x16] * B[16x8], unsigned 8-bit A, signed 8-bit B
__device__ __forceinline__ void mma_u8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    const int z = 0;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(b0), "r"(z));
}

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// Optional source of x for the attention output projection: the un-normalised per-split results of
// the paged attention kernel (max, sum, acc[hd] per head and split) are merged on the fly, which
// saves the separate merge kernel.  partial == nullptr: x is read from memory as usual.
struct AttnMerge {
    const float* merged;      // with merge_below > 0: the row already merged by the attention kernel (many visible splits)
    int merge_below;
    const float* partial;     // [n_head][n_splits][hd + 2]
    const int32_t* d_pos;     // position of the token (device scalar), or nullptr -> pos0
    int pos0;
    int n_splits, keys_per_split, hd;
};

// x[k0 .. k0+7] (k0 a multiple of 8, all in one head) = merged attention output
__device__ __forceinline__ void attn_merge8(const AttnMerge& am, int k0, float (&v)[8]) {
    const int head = k0 / am.hd, d0 = k0 - head * am.hd;
    const int pos = am.d_pos ? am.d_pos[0] : am.pos0;
    const int n_active = min(am.n_splits, pos / am.keys_per_split + 1);
    const float* base = am.partial + static_cast<size_t>(head) * am.n_splits * (am.hd + 2);
    // One pass with a running maximum: every load of a split is independent of the state carried
    // from the splits before it, so the splits' loads overlap and the prologue's chain of dependent
    // round trips to L2 is position -> split data, not position -> maxima -> split data.
    float mx = -INFINITY, lsum = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.0f;
#pragma unroll 2
    for (int s = 0; s < n_active; ++s) {
        const float* ps = base + static_cast<size_t>(s) * (am.hd + 2);
        const float m_s = __ldg(ps), l_s = __ldg(ps + 1);
        float2 p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = __ldg(reinterpret_cast<const float2*>(ps + 2 + d0 + 2 * i));
        const float nm = fmaxf(mx, m_s);
        // first split: fa = exp(-inf) = 0; a split without keys (max = -inf) contributes nothing
        const float fa = mx == -INFINITY ? 0.0f : expf(mx - nm), fb = m_s == -INFINITY ? 0.0f : expf(m_s - nm);
        lsum = fmaf(l_s, fb, lsum * fa);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = fmaf(p[i].x, fb, v[2 * i] * fa);
            v[2 * i + 1] = fmaf(p[i].y, fb, v[2 * i + 1] * fa);
        }
        mx = nm;
    }
    const float r = 1.0f / lsum;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] *= r;
}

// One of up to three matrices stacked along N that share x and K (fused q/k/v projections).
struct CatMat {
    PackedW w;
    float* y;
    const float* bias;
    int ldc;
    int g_start;       // first row group of this matrix in the stacked numbering
};

struct MmaArgs {
    PackedW w, w2;
    CatMat cat[2];     // matrices 1 and 2 of a stack (matrix 0 is w / y / bias / ldc); ncat = extra count
    int ncat;
    AttnMerge attn;
    const float* x;
    float* y;
    const float* bias;
    const float* resid;
    const float* gamma;
    float eps;
    int M, lda, ldc, epi;
    int sb;            // blocks of 256 per tile
    int spr;           // tiles (k slices) per row group and matrix
    int nmat;          // 1, or 2 for the fused gate/up pair
    int groups;        // row groups of 16 (N rounded up)
    int ws;            // consumer warps that share one row group (1, 2, 4 or 8)
    int P;             // ring stages per consumer warp
    int stage_bytes;
    // routed experts (MoE): the weight holds all experts stacked along N, `sel` (device) names the chosen ones
    const int* sel;    // nullptr: none
    int sel_mode;      // 1: output rows = the chosen experts' row ranges (gate / up);  2: K = the chosen experts' K ranges side by side (down)
    int sel_groups;    // row groups of one expert's matrix
    int klog, nblog;   // logical K and blocks per row the kernel iterates over (mode 2: n_sel * the expert's)
    int64_t nlog;      // logical number of output rows
    const float* xscale;   // optional: x[i] is multiplied by xscale[i / xscale_run] (router weights folded into the activations)
    int xscale_run;
    int* err;
};

// Work split inside a CTA.  The CTA owns a contiguous range of row groups (16 rows each).  Its 8
// consumer warps form 8/ws teams of ws warps; team i takes row groups i, i + 8/ws, ... of the range;
// inside a team, member j takes tiles j, j + ws, ... of the row group's nmat*spr tiles.  Every warp
// therefore consumes a fixed sequence of tiles, which lane w of the producer warp streams into warp
// w's private ring of P stages (no stage is ever shared between warps).  A warp keeps its partial
// dot products in registers across its tiles of a row group; teams of more than one warp add their
// partials through shared memory behind a team-wide named barrier.
//
// dynamic shared memory map: [ring: 8 * P * stage_bytes][limb planes: 3*M * (K + 16) bytes]
//   [asum: M * K/32 floats][xs: M * K/256 floats][comb: 2 * 8 * nmat * 16 * M floats]
template <int kWarps>
__global__ void __launch_bounds__((kWarps + 1) * 32, 1) gemv_mma_q4k_kernel(const MmaArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages];
    __shared__ float red[2 * kWarps];
    __shared__ int x_ready;        // consumer warps that have pulled their part of x into registers
    const int K = a.klog, nb = a.nblog, M = a.M;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tprg = a.nmat * a.spr;
    const int plane_stride = K + 16;
    uint8_t* ring = smem;
    int8_t* xl = reinterpret_cast<int8_t*>(ring + static_cast<size_t>(kWarps) * a.P * a.stage_bytes);
    float* asum = reinterpret_cast<float*>(xl + static_cast<size_t>(3 * M) * plane_stride);
    float* asum16 = asum + M * (K >> 5);                  // sums of x over each 16-run
    float* xs = asum16 + M * (K >> 4);
    float* comb = xs + M * (K >> 8);
    // stacked matrices: global row group -> (matrix index, first row group of that matrix)
    auto which = [&](int64_t G_rg) -> int { return (a.ncat > 0 && G_rg >= a.cat[0].g_start) + (a.ncat > 1 && G_rg >= a.cat[1].g_start); };

    const int64_t g_begin = static_cast<int64_t>(blockIdx.x) * a.groups / gridDim.x;
    const int n_rg = static_cast<int>(static_cast<int64_t>(blockIdx.x + 1) * a.groups / gridDim.x - g_begin);
    const int n_teams = kWarps / a.ws;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWarps * a.P; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        x_ready = 0;
    }
    __syncthreads();
    pdl_launch();

    if (warp == kWarps) {
        // ---------------- producers: lane w feeds consumer warp w ----------------
        if (lane < kWarps) {
            const int team = lane / a.ws, member = lane % a.ws;
            int st = 0;
            uint32_t ph = 1;
            bool ok = true;
            // Only the first stage of each ring is requested before the activations are in: a full
            // ring of weight traffic queued ahead of the x loads would delay them by microseconds.
            bool throttled = true;
            if (a.sel) pdl_wait();                 // the expert ids are the predecessor's output
            for (int rg = team; rg < n_rg && ok; rg += n_teams) {
                const int mi = which(g_begin + rg);
                const PackedW& w0 = mi == 0 ? a.w : a.cat[mi - 1].w;
                const bool is_q6 = w0.type == T_Q6_K;
                int64_t blk0 = (g_begin + rg - (mi == 0 ? 0 : a.cat[mi - 1].g_start)) * nb;
                if (a.sel_mode == 1) {             // gathered rows: logical group -> (chosen expert, group inside it)
                    const int64_t lg = g_begin + rg;
                    const int e = a.sel[lg / a.sel_groups];
                    if (e < 0) continue;           // expert held by another rank (expert parallel): nothing to stream, the consumers skip it too
                    blk0 = (static_cast<int64_t>(e) * a.sel_groups + lg % a.sel_groups) * a.w.nb;
                }
                for (int ti = member; ti < tprg; ti += a.ws) {
                    if (a.sel_mode == 2 && a.sel[ti - (ti >= a.spr) * a.spr] < 0) continue;       // K range of an expert on another rank
                    const int s = lane * a.P + st;
                    if (throttled && (rg != team || ti != member)) {
                        uint32_t spins = 0;
                        while (*reinterpret_cast<volatile int*>(&x_ready) < kWarps && ++spins < (kSpinLimit << 6)) {}
                        if (*reinterpret_cast<volatile int*>(&x_ready) < kWarps) { atomicExch(a.err, 3); ok = false; break; }
                        throttled = false;
                    }
                    if (!(ok = mbar_wait(&empty_bar[s], ph, a.err, 1))) break;
                    const int mat = ti >= a.spr, sl = ti - mat * a.spr;
                    const int b0 = sl * a.sb, nbk = min(a.sb, nb - b0);
                    uint8_t* dst = ring + static_cast<size_t>(s) * a.stage_bytes;
                    const PackedW& w = mat ? a.w2 : w0;
                    int64_t gb = blk0 + b0;
                    if (a.sel_mode == 2)           // K ranges side by side: tile sl = all a.w.nb blocks of chosen expert sl, same row group
                        gb = (static_cast<int64_t>(a.sel[sl]) * a.sel_groups + (g_begin + rg)) * a.w.nb;
                    if (!is_q6) {
                        mbar_expect_tx(&full_bar[s], static_cast<uint32_t>(nbk) * 2304u);
                        bulk_g2s(dst, w.s[1] + gb * 2048, static_cast<uint32_t>(nbk) * 2048u, &full_bar[s]);
                        bulk_g2s(dst + a.sb * 2048, w.s[0] + gb * 256, static_cast<uint32_t>(nbk) * 256u, &full_bar[s]);
                    } else {
                        mbar_expect_tx(&full_bar[s], static_cast<uint32_t>(nbk) * 3360u);
                        bulk_g2s(dst, w.s[0] + gb * 2048, static_cast<uint32_t>(nbk) * 2048u, &full_bar[s]);
                        bulk_g2s(dst + a.sb * 2048, w.s[1] + gb * 1024, static_cast<uint32_t>(nbk) * 1024u, &full_bar[s]);
                        bulk_g2s(dst + a.sb * 3072, w.s[2] + gb * 256, static_cast<uint32_t>(nbk) * 256u, &full_bar[s]);
                        bulk_g2s(dst + a.sb * 3328, w.s[3] + gb * 32, static_cast<uint32_t>(nbk) * 32u, &full_bar[s]);
                    }
                    if (++st == a.P) { st = 0; ph ^= 1; }
                }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int tid = threadIdx.x;                          // 0 .. 255
    // lane constants of the mma fragment layout (independent of x: computed before the wait)
    const int g = lane >> 2, t = lane & 3;
    const int ncol = 3 * M;
    const int8_t* bplane = xl + static_cast<size_t>(min(g, ncol - 1)) * plane_stride + 4 * t;   // B column g (unused columns repeat the last)
    const int col0 = 2 * t, col1 = 2 * t + 1;                    // C columns this lane holds
    const int m0c = min(col0 / 3, M - 1), m1c = min(col1 / 3, M - 1);
    const float lw0 = col0 < ncol ? (col0 % 3 == 0 ? 1.0f : (col0 % 3 == 1 ? 1.0f / 128.0f : 1.0f / 16384.0f)) : 0.0f;
    const float lw1 = col1 < ncol ? (col1 % 3 == 0 ? 1.0f : (col1 % 3 == 1 ? 1.0f / 128.0f : 1.0f / 16384.0f)) : 0.0f;
    const int team = warp / a.ws, member = warp % a.ws;
    const int mshift = 16 * (t & 1);                             // this lane's two min bytes: sub-blocks 2t, 2t+1
    pdl_wait();
    // Residual epilogue of a team: the lanes that will store the first row group's rows fetch their
    // residual values now, so that the load's latency passes under the prologue and the main loop.
    const bool resid_pre = a.epi == EPI_RESIDUAL && a.ws > 1 && member == 0 && lane < 16 * M && team < n_rg && a.ncat == 0 && !a.sel;
    float resid_first = 0.0f;
    if (resid_pre) {
        const int64_t row = (g_begin + team) * 16 + (lane & 15);
        if (row < a.nlog) resid_first = a.resid[static_cast<size_t>(lane >> 4) * a.ldc + row];
    }
    // One pass over x: y = W (x * gamma) is linear in x, so the RMS factor 1/sqrt(mean(x^2)+eps) is a
    // scalar that can be applied to the finished dot products; the limbs are taken from x * gamma.
    // A warp converts 256-blocks warp, warp+8, ...; four blocks are loaded before any is converted so
    // that their memory latencies overlap.
    // attention splits: merged here while few are visible, by the attention kernel from merge_below on (the position is
    // the same for every CTA, so all take the same branch)
    bool merge_here = a.attn.partial != nullptr;
    if (merge_here && a.attn.merge_below > 0) {
        const int pos = a.attn.d_pos ? a.attn.d_pos[0] : a.attn.pos0;
        merge_here = min(a.attn.n_splits, pos / a.attn.keys_per_split + 1) < a.attn.merge_below;
    }
    for (int m = 0; m < M; ++m) {
        const float* xr = (a.attn.partial ? a.attn.merged : a.x) + static_cast<size_t>(m) * a.lda;
        float ss = 0.0f;
        for (int bb = warp; bb < (K >> 8); bb += 4 * kWarps) {
            float v[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int b = bb + u * kWarps;
                if (b < (K >> 8)) {
                    const int k0 = b * 256 + lane * 8;
                    if (merge_here) attn_merge8(a.attn, k0, v[u]);
                    else {
                        const float4 p0 = __ldg(reinterpret_cast<const float4*>(xr + k0)), p1 = __ldg(reinterpret_cast<const float4*>(xr + k0 + 4));
                        v[u][0] = p0.x; v[u][1] = p0.y; v[u][2] = p0.z; v[u][3] = p0.w; v[u][4] = p1.x; v[u][5] = p1.y; v[u][6] = p1.z; v[u][7] = p1.w;
                    }
                    if (a.xscale) {
                        const float sc = a.xscale[k0 / a.xscale_run];
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[u][i] *= sc;
                    }
                    if (a.gamma) {
                        const float4 g0 = __ldg(reinterpret_cast<const float4*>(a.gamma + k0)), g1 = __ldg(reinterpret_cast<const float4*>(a.gamma + k0 + 4));
#pragma unroll
                        for (int i = 0; i < 8; ++i) ss = fmaf(v[u][i], v[u][i], ss);
                        v[u][0] *= g0.x; v[u][1] *= g0.y; v[u][2] *= g0.z; v[u][3] *= g0.w; v[u][4] *= g1.x; v[u][5] *= g1.y; v[u][6] *= g1.z; v[u][7] *= g1.w;
                    }
                }
            }
            // the four blocks are converted side by side (independent chains interleave)
            float am[4], sm[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                am[u] = 0.0f; sm[u] = 0.0f;
                if (bb + u * kWarps < (K >> 8)) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) { am[u] = fmaxf(am[u], fabsf(v[u][i])); sm[u] += v[u][i]; }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int u = 0; u < 4; ++u) am[u] = fmaxf(am[u], __shfl_xor_sync(0xFFFFFFFFu, am[u], o));
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int b = bb + u * kWarps;
                if (b < (K >> 8)) {
                    const int k0 = b * 256 + lane * 8;
                    const float rs = am[u] > 0.0f ? 127.0f / am[u] : 0.0f;
                    uint32_t w1[2] = {0, 0}, w2[2] = {0, 0}, w3[2] = {0, 0};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        // round-to-nearest by adding 1.5 * 2^23: the integer lands in the low mantissa bits
                        // (two's complement), so no float<->int conversion instructions are needed (those
                        // issue at a quarter of the FP32 rate and dominated this loop)
                        const float kMagic = 12582912.0f;
                        const float r = fminf(fmaxf(v[u][i] * rs, -127.0f), 127.0f);
                        const float t1 = r + kMagic;
                        const float r2 = (r - (t1 - kMagic)) * 128.0f;
                        const float t2 = r2 + kMagic;
                        const float t3 = (r2 - (t2 - kMagic)) * 128.0f + kMagic;
                        w1[i >> 2] |= (__float_as_uint(t1) & 0xFFu) << (8 * (i & 3));
                        w2[i >> 2] |= (__float_as_uint(t2) & 0xFFu) << (8 * (i & 3));
                        w3[i >> 2] |= (__float_as_uint(t3) & 0xFFu) << (8 * (i & 3));
                    }
                    int8_t* pl = xl + static_cast<size_t>(3 * m) * plane_stride + k0;
                    *reinterpret_cast<uint2*>(pl) = make_uint2(w1[0], w1[1]);
                    *reinterpret_cast<uint2*>(pl + plane_stride) = make_uint2(w2[0], w2[1]);
                    *reinterpret_cast<uint2*>(pl + 2 * plane_stride) = make_uint2(w3[0], w3[1]);
                    if (lane == 0) xs[m * (K >> 8) + b] = am[u] / 127.0f;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) sm[u] += __shfl_xor_sync(0xFFFFFFFFu, sm[u], 1);      // 16-run = two lanes
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int b = bb + u * kWarps;
                if (b < (K >> 8) && (lane & 1) == 0) asum16[m * (K >> 4) + ((b * 256 + lane * 8) >> 4)] = sm[u];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) sm[u] += __shfl_xor_sync(0xFFFFFFFFu, sm[u], 2);      // 32-run = four lanes
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int b = bb + u * kWarps;
                if (b < (K >> 8) && (lane & 3) == 0) asum[m * (K >> 5) + ((b * 256 + lane * 8) >> 5)] = sm[u];
            }
        }
        ss = wsum(ss);
        if (lane == 0) red[m * kWarps + warp] = ss;
    }
    __syncwarp();
    if (lane == 0) atomicAdd(&x_ready, 1);      // this warp's x values have arrived: weight streaming may go deep
    consumer_sync<kWarps>();
    float inv[2] = {1.0f, 1.0f};
    if (a.gamma) {
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            if (m < M) {
                float tot = 0.0f;
#pragma unroll
                for (int i = 0; i < kWarps; ++i) tot += red[m * kWarps + i];
                inv[m] = 1.0f / sqrtf(tot / static_cast<float>(K) + a.eps);
            }
        }
    }

    int st = 0;
    uint32_t ph = 0;
    bool ok = true;
    int parity = 0;
    for (int rg = team; rg < n_rg; rg += n_teams, parity ^= 1) {
        if (a.sel_mode == 1 && a.sel[(g_begin + rg) / a.sel_groups] < 0) continue;      // rows of an expert on another rank: left unwritten
        const int mi = which(g_begin + rg);
        const bool is_q6 = (mi == 0 ? a.w.type : a.cat[mi - 1].w.type) == T_Q6_K;
        // accumulators in the C-fragment layout: [matrix][row g / g+8][column 2t / 2t+1], and this
        // lane's share of the min term per [matrix][row][activation row]
        // (kept as scalars selected by warp-uniform branches: no dynamically indexed register arrays)
        float F0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, F1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        float MN0[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}}, MN1[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};   // [row g / g+8][activation row]
        for (int ti = member; ti < tprg; ti += a.ws) {
            if (a.sel_mode == 2 && a.sel[ti - (ti >= a.spr) * a.spr] < 0) continue;
            const int s = warp * a.P + st;
            if (ok) ok = mbar_wait(&full_bar[s], ph, a.err, 2);
            if (++st == a.P) { st = 0; ph ^= 1; }
            if (!ok) continue;
            const int mat = ti >= a.spr, sl = ti - mat * a.spr;
            const int b0 = sl * a.sb, nbk = min(a.sb, nb - b0);
            const uint8_t* qsT = ring + static_cast<size_t>(s) * a.stage_bytes;
            const uint8_t* hdrT = qsT + a.sb * 2048;       // Q4_K: headers.  Q6_K: s1 (high bits), then s2, s3
            const uint8_t* s1T = hdrT;
            const uint8_t* s2T = s1T + a.sb * 1024;
            const uint8_t* s3T = s2T + a.sb * 256;
            float f0 = 0.0f, f1 = 0.0f, f2 = 0.0f, f3 = 0.0f;
            float mnA[2] = {0.0f, 0.0f}, mnB[2] = {0.0f, 0.0f};
            if (!is_q6) {
            for (int bl = 0; bl < nbk; ++bl) {
                // headers of rows g and g+8: 6-bit scales and mins to bytes (8 lanes share an address)
                const uint4 ha = *reinterpret_cast<const uint4*>(hdrT + (bl * 16 + g) * 16);
                const uint4 hb = *reinterpret_cast<const uint4*>(hdrT + (bl * 16 + g + 8) * 16);
                const uint32_t sa03 = ha.y & 0x3F3F3F3Fu, sa47 = (ha.w & 0x0F0F0F0Fu) | ((ha.y >> 2) & 0x30303030u);
                const uint32_t sb03 = hb.y & 0x3F3F3F3Fu, sb47 = (hb.w & 0x0F0F0F0Fu) | ((hb.y >> 2) & 0x30303030u);
                {   // min term: this lane covers sub-blocks 2t and 2t+1 of both rows
                    const uint32_t ma = (t < 2 ? (ha.z & 0x3F3F3F3Fu) : (((ha.w >> 4) & 0x0F0F0F0Fu) | ((ha.z >> 2) & 0x30303030u))) >> mshift;
                    const uint32_t mb = (t < 2 ? (hb.z & 0x3F3F3F3Fu) : (((hb.w >> 4) & 0x0F0F0F0Fu) | ((hb.z >> 2) & 0x30303030u))) >> mshift;
                    const float dmA = __half2float(__ushort_as_half(static_cast<uint16_t>(ha.x >> 16)));
                    const float dmB = __half2float(__ushort_as_half(static_cast<uint16_t>(hb.x >> 16)));
#pragma unroll
                    for (int m = 0; m < 2; ++m) {
                        if (m < M) {
                            const float2 as = *reinterpret_cast<const float2*>(asum + m * (K >> 5) + (b0 + bl) * 8 + 2 * t);
                            mnA[m] = fmaf(dmA, static_cast<float>(ma & 0xFFu) * as.x + static_cast<float>((ma >> 8) & 0xFFu) * as.y, mnA[m]);
                            mnB[m] = fmaf(dmB, static_cast<float>(mb & 0xFFu) * as.x + static_cast<float>((mb >> 8) & 0xFFu) * as.y, mnB[m]);
                        }
                    }
                }
                int lo0 = 0, lo1 = 0, lo2 = 0, lo3 = 0, hi0 = 0, hi1 = 0, hi2 = 0, hi3 = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 q = *reinterpret_cast<const uint4*>(qsT + (static_cast<size_t>(bl * 4 + j) * 32 + lane) * 16);
                    const int8_t* bp = bplane + ((b0 + bl) * 8 + 2 * j) * 32;
                    const uint32_t bl0 = *reinterpret_cast<const uint32_t*>(bp), bl1 = *reinterpret_cast<const uint32_t*>(bp + 16);
                    const uint32_t bh0 = *reinterpret_cast<const uint32_t*>(bp + 32), bh1 = *reinterpret_cast<const uint32_t*>(bp + 48);
                    int cl[4], ch[4];
                    mma_s8(cl, q.x & 0x0F0F0F0Fu, q.y & 0x0F0F0F0Fu, q.z & 0x0F0F0F0Fu, q.w & 0x0F0F0F0Fu, bl0, bl1);
                    mma_u8s8(ch, q.x & 0xF0F0F0F0u, q.y & 0xF0F0F0F0u, q.z & 0xF0F0F0F0u, q.w & 0xF0F0F0F0u, bh0, bh1);
                    const uint32_t wa = j < 2 ? sa03 : sa47, wb = j < 2 ? sb03 : sb47;   // j is a compile-time constant
                    const int sa0 = (wa >> (16 * (j & 1))) & 0xFF, sa1 = (wa >> (16 * (j & 1) + 8)) & 0xFF;
                    const int sb0 = (wb >> (16 * (j & 1))) & 0xFF, sb1 = (wb >> (16 * (j & 1) + 8)) & 0xFF;
                    lo0 += sa0 * cl[0]; lo1 += sa0 * cl[1]; lo2 += sb0 * cl[2]; lo3 += sb0 * cl[3];
                    hi0 += sa1 * ch[0]; hi1 += sa1 * ch[1]; hi2 += sb1 * ch[2]; hi3 += sb1 * ch[3];
                }
                const float dA = __half2float(__ushort_as_half(static_cast<uint16_t>(ha.x & 0xFFFF)));
                const float dB = __half2float(__ushort_as_half(static_cast<uint16_t>(hb.x & 0xFFFF)));
                const float x0 = xs[m0c * (K >> 8) + b0 + bl] * lw0, x1 = xs[m1c * (K >> 8) + b0 + bl] * lw1;
                f0 = fmaf(static_cast<float>(lo0) + static_cast<float>(hi0) * 0.0625f, dA * x0, f0);
                f1 = fmaf(static_cast<float>(lo1) + static_cast<float>(hi1) * 0.0625f, dA * x1, f1);
                f2 = fmaf(static_cast<float>(lo2) + static_cast<float>(hi2) * 0.0625f, dB * x0, f2);
                f3 = fmaf(static_cast<float>(lo3) + static_cast<float>(hi3) * 0.0625f, dB * x1, f3);
            }
            } else {
            for (int bl = 0; bl < nbk; ++bl) {
                // int8 scales (16 per block) and d of rows g and g+8
                const uint4 sa = *reinterpret_cast<const uint4*>(s2T + (bl * 16 + g) * 16);
                const uint4 sb_ = *reinterpret_cast<const uint4*>(s2T + (bl * 16 + g + 8) * 16);
                const float dA = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(s3T + (bl * 16 + g) * 2)));
                const float dB = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(s3T + (bl * 16 + g + 8) * 2)));
                const uint32_t saw[4] = {sa.x, sa.y, sa.z, sa.w}, sbw[4] = {sb_.x, sb_.y, sb_.z, sb_.w};
                {   // quants are used unsigned (0..63): remove 32 * sc * sum(x) per 16-run; this lane covers runs 4t..4t+3
                    const uint32_t wa = t == 0 ? sa.x : (t == 1 ? sa.y : (t == 2 ? sa.z : sa.w));
                    const uint32_t wb = t == 0 ? sb_.x : (t == 1 ? sb_.y : (t == 2 ? sb_.z : sb_.w));
#pragma unroll
                    for (int m = 0; m < 2; ++m) {
                        if (m < M) {
                            const float4 as = *reinterpret_cast<const float4*>(asum16 + m * (K >> 4) + (b0 + bl) * 16 + 4 * t);
                            const float ca = static_cast<float>(static_cast<int8_t>(wa)) * as.x + static_cast<float>(static_cast<int8_t>(wa >> 8)) * as.y +
                                             static_cast<float>(static_cast<int8_t>(wa >> 16)) * as.z + static_cast<float>(static_cast<int8_t>(wa >> 24)) * as.w;
                            const float cb = static_cast<float>(static_cast<int8_t>(wb)) * as.x + static_cast<float>(static_cast<int8_t>(wb >> 8)) * as.y +
                                             static_cast<float>(static_cast<int8_t>(wb >> 16)) * as.z + static_cast<float>(static_cast<int8_t>(wb >> 24)) * as.w;
                            mnA[m] = fmaf(dA * 32.0f, ca, mnA[m]);
                            mnB[m] = fmaf(dB * 32.0f, cb, mnB[m]);
                        }
                    }
                }
                int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const uint4 qh = *reinterpret_cast<const uint4*>(s1T + (static_cast<size_t>(bl * 2 + hf) * 32 + lane) * 16);
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const uint4 ql = *reinterpret_cast<const uint4*>(qsT + (static_cast<size_t>(bl * 4 + 2 * hf + c) * 32 + lane) * 16);
                        const uint32_t hA = c ? qh.z : qh.x, hB = c ? qh.w : qh.y;      // high bits of rows g, g+8
                        const uint32_t kf = 0x0F0F0F0Fu, k3 = 0x30303030u;
                        // four 16-runs: values 16c (+0, +32, +64, +96) of this half
                        const uint32_t a1g = (ql.x & kf) | ((hA << 4) & k3), a1h = (ql.z & kf) | ((hB << 4) & k3);
                        const uint32_t a2g = (ql.y & kf) | ((hA << 2) & k3), a2h = (ql.w & kf) | ((hB << 2) & k3);
                        const uint32_t a3g = ((ql.x >> 4) & kf) | (hA & k3), a3h = ((ql.z >> 4) & kf) | (hB & k3);
                        const uint32_t a4g = ((ql.y >> 4) & kf) | ((hA >> 2) & k3), a4h = ((ql.w >> 4) & kf) | ((hB >> 2) & k3);
                        const uint32_t ag[4] = {a1g, a2g, a3g, a4g}, ah[4] = {a1h, a2h, a3h, a4h};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int sidx = 8 * hf + 2 * i + c;                                  // 16-run (scale) index, compile-time
                            const uint32_t bw = *reinterpret_cast<const uint32_t*>(bplane + ((b0 + bl) * 16 + sidx) * 16);
                            int cc[4];
                            mma_u8s8_k16(cc, ag[i], ah[i], bw);
                            const int sca = static_cast<int8_t>(saw[sidx >> 2] >> (8 * (sidx & 3)));
                            const int scb = static_cast<int8_t>(sbw[sidx >> 2] >> (8 * (sidx & 3)));
                            c0 += sca * cc[0]; c1 += sca * cc[1]; c2 += scb * cc[2]; c3 += scb * cc[3];
                        }
                    }
                }
                const float x0 = xs[m0c * (K >> 8) + b0 + bl] * lw0, x1 = xs[m1c * (K >> 8) + b0 + bl] * lw1;
                f0 = fmaf(static_cast<float>(c0), dA * x0, f0); f1 = fmaf(static_cast<float>(c1), dA * x1, f1);
                f2 = fmaf(static_cast<float>(c2), dB * x0, f2); f3 = fmaf(static_cast<float>(c3), dB * x1, f3);
            }
            }
            if (mat == 0) {
                F0[0] += f0; F0[1] += f1; F0[2] += f2; F0[3] += f3;
                MN0[0][0] += mnA[0]; MN0[0][1] += mnA[1]; MN0[1][0] += mnB[0]; MN0[1][1] += mnB[1];
            } else {
                F1[0] += f0; F1[1] += f1; F1[2] += f2; F1[3] += f3;
                MN1[0][0] += mnA[0]; MN1[0][1] += mnA[1]; MN1[1][0] += mnB[0]; MN1[1][1] += mnB[1];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
        }
        // ---- per-row values: fold the limb columns (neighbouring lanes) and the min terms ----
        float va[2][2], vb[2][2];                                  // [matrix][activation row], rows g and g+8
#pragma unroll
        for (int mat = 0; mat < 2; ++mat)
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const float* F = mat ? F1 : F0;
                float pa = (col0 < ncol && col0 / 3 == m ? F[0] : 0.0f) + (col1 < ncol && col1 / 3 == m ? F[1] : 0.0f) - (mat ? MN1[0][m] : MN0[0][m]);
                float pb = (col0 < ncol && col0 / 3 == m ? F[2] : 0.0f) + (col1 < ncol && col1 / 3 == m ? F[3] : 0.0f) - (mat ? MN1[1][m] : MN0[1][m]);
                pa += __shfl_xor_sync(0xFFFFFFFFu, pa, 1); pa += __shfl_xor_sync(0xFFFFFFFFu, pa, 2);
                pb += __shfl_xor_sync(0xFFFFFFFFu, pb, 1); pb += __shfl_xor_sync(0xFFFFFFFFu, pb, 2);
                va[mat][m] = pa * inv[m]; vb[mat][m] = pb * inv[m];
            }
        const int64_t row_base = (g_begin + rg - (mi == 0 ? 0 : a.cat[mi - 1].g_start)) * 16;
        const int64_t n_rows = mi == 0 ? a.nlog : a.cat[mi - 1].w.N;
        float* const yb = mi == 0 ? a.y : a.cat[mi - 1].y;
        const float* const bb = mi == 0 ? a.bias : a.cat[mi - 1].bias;
        const int ldc = mi == 0 ? a.ldc : a.cat[mi - 1].ldc;
        auto finish = [&](float v, float v2, int64_t row, int m, bool have_resid = false, float resid_v = 0.0f) {
            if (row >= n_rows) return;
            const size_t o = static_cast<size_t>(m) * ldc + row;
            if (a.nmat == 2) v = (v / (1.0f + expf(-v))) * v2;      // silu(gate) * up
            else if (a.epi == EPI_ADD_BIAS && bb) v += __ldg(bb + row);
            else if (a.epi == EPI_RESIDUAL) v += have_resid ? resid_v : a.resid[o];
            yb[o] = v;
        };
        if (a.ws == 1) {
            if (t == 0) {
#pragma unroll
                for (int m = 0; m < 2; ++m)
                    if (m < M) { finish(va[0][m], va[1][m], row_base + g, m); finish(vb[0][m], vb[1][m], row_base + g + 8, m); }
            }
        } else {
            // team partials: comb[parity][warp][matrix][16 rows][2]
            float* cb = comb + static_cast<size_t>((parity * kWarps + warp) * 2) * 32;
            if (t == 0) {
#pragma unroll
                for (int mat = 0; mat < 2; ++mat)
#pragma unroll
                    for (int m = 0; m < 2; ++m) { cb[(mat * 16 + g) * 2 + m] = va[mat][m]; cb[(mat * 16 + g + 8) * 2 + m] = vb[mat][m]; }
            }
            asm volatile("bar.sync %0, %1;" ::"r"(2 + team), "r"(a.ws * 32) : "memory");
            if (member == 0) {
                for (int idx = lane; idx < 16 * M; idx += 32) {
                    const int r = idx & 15, m = idx >> 4;
                    float v = 0.0f, v2 = 0.0f;
                    for (int j = 0; j < a.ws; ++j) {
                        const float* cj = comb + static_cast<size_t>((parity * kWarps + team * a.ws + j) * 2) * 32;
                        v += cj[r * 2 + m]; v2 += cj[(16 + r) * 2 + m];
                    }
                    finish(v, v2, row_base + r, m, resid_pre && rg == team, resid_first);      // idx == lane on the first pass
                }
            }
        }
    }
}

template <int kWarps>
int launch_mma_t(Context* c, const GemvArgs& g, cudaStream_t s) {
    constexpr int kThreads = (kWarps + 1) * 32;
    if ((g.w.type != T_Q4_K && g.w.type != T_Q6_K) || g.w.layout != 1 || g.M < 1 || g.M > 2) return GGB_NOT_FOUND;
    if (!g.attn_partial && ((reinterpret_cast<uintptr_t>(g.x) & 15) || (g.lda & 3))) return GGB_NOT_FOUND;
    if (g.attn_partial && (g.M != 1 || g.attn_hd % 8 || g.attn_hd <= 0)) return GGB_NOT_FOUND;
    const bool dual = g.epi == EPI_SWIGLU;
    if (dual && (g.w2.layout != 1 || g.w2.type != g.w.type)) return GGB_NOT_FOUND;
    if (g.sel && (g.n_cat || g.attn_partial || g.sel_count < 1 || g.sel_rows < 16 || g.sel_rows % 16 || (g.sel_mode != 1 && g.sel_mode != 2))) return GGB_NOT_FOUND;
    if (g.sel && g.sel_mode == 2 && (dual || g.w.nb > 8)) return GGB_NOT_FOUND;
    // logical shape: with routed experts the kernel sees the chosen experts' rows (mode 1) or K ranges (mode 2)
    const int K = g.sel && g.sel_mode == 2 ? g.sel_count * g.w.K : g.w.K, nb = g.sel && g.sel_mode == 2 ? g.sel_count * g.w.nb : g.w.nb, M = g.M;
    const int64_t n_log = !g.sel ? g.w.N : (g.sel_mode == 1 ? static_cast<int64_t>(g.sel_count) * g.sel_rows : g.sel_rows);
    int groups = static_cast<int>((n_log + 15) / 16);
    bool any_q6 = g.w.type == T_Q6_K;
    if (g.n_cat < 0 || g.n_cat > 2 || (g.n_cat && dual)) return GGB_NOT_FOUND;
    int cat_start[2] = {0, 0};
    for (int i = 0; i < g.n_cat; ++i) {
        const PackedW& wc = g.cat_w[i];
        if ((wc.type != T_Q4_K && wc.type != T_Q6_K) || wc.layout != 1 || wc.K != g.w.K || !g.cat_y[i]) return GGB_NOT_FOUND;
        cat_start[i] = groups;
        groups += static_cast<int>((wc.N + 15) / 16);
        any_q6 = any_q6 || wc.type == T_Q6_K;
    }
    const int nmat = dual ? 2 : 1;
    const int gb_bytes = any_q6 ? 3360 : 2304;                   // bytes of one (row group, block), largest type
    const int G = std::min(c->sm_count, groups);
    const int gpc = (groups + G - 1) / G;                   // row groups of the busiest CTA
    // warps per row group: enough that all 8 consumer warps of the busiest CTA have work
    int ws = 1;
    while (ws < kWarps && gpc * ws < kWarps) ws <<= 1;
    // tile depth: up to 4 blocks, but at least one tile per team member
    int sb = 4;
    while (sb > 1 && nmat * ((nb + sb - 1) / sb) < ws) sb >>= 1;
    sb = std::min(sb, nb);
    if (g.sel && g.sel_mode == 2) sb = g.w.nb;            // one tile = one chosen expert's blocks of the row group
    const size_t fixed = static_cast<size_t>(3 * M) * (K + 16) + sizeof(float) * M * (K / 32 + K / 16 + K / 256) + sizeof(float) * 2 * kWarps * 2 * 32 + 64;
    const size_t budget = 200 * 1024;                       // shared memory per CTA given to rings + activations
    int spr, stage_bytes, P;
    for (;;) {
        spr = (nb + sb - 1) / sb;
        stage_bytes = sb * gb_bytes;
        const int tiles_per_warp = ((gpc + kWarps / ws - 1) / (kWarps / ws)) * ((nmat * spr + ws - 1) / ws);
        P = std::min(kMaxStages / kWarps, std::max(1, tiles_per_warp));
        while (P > 1 && static_cast<size_t>(kWarps) * P * stage_bytes + fixed > budget) --P;
        // a warp with a single stage cannot overlap copy and use: shallower tiles, more stages
        if (P > 1 || tiles_per_warp <= 1 || sb == 1 || (g.sel && g.sel_mode == 2)) break;
        sb >>= 1;
    }
    const size_t smem = static_cast<size_t>(kWarps) * P * stage_bytes + fixed;
    if (smem > 220 * 1024) return GGB_NOT_FOUND;

    MmaArgs a{};
    a.w = g.w; a.w2 = g.w2; a.x = g.x; a.y = g.y; a.bias = g.bias; a.resid = g.resid; a.gamma = g.gamma; a.eps = g.eps;
    a.M = M; a.lda = g.lda; a.ldc = g.ldc; a.epi = g.epi;
    a.ncat = g.n_cat;
    for (int i = 0; i < g.n_cat; ++i) { a.cat[i].w = g.cat_w[i]; a.cat[i].y = g.cat_y[i]; a.cat[i].bias = g.cat_bias[i]; a.cat[i].ldc = g.cat_ldc[i]; a.cat[i].g_start = cat_start[i]; }
    a.attn.partial = g.attn_partial; a.attn.d_pos = g.attn_d_pos; a.attn.pos0 = g.attn_pos0; a.attn.n_splits = g.attn_n_splits;
    a.attn.keys_per_split = g.attn_keys_per_split; a.attn.hd = g.attn_hd;
    a.attn.merge_below = g.attn_merged ? g.attn_merge_below : 0; a.attn.merged = g.attn_merged;
    a.sb = sb; a.spr = spr; a.nmat = nmat; a.groups = groups; a.ws = ws; a.P = P; a.stage_bytes = stage_bytes;
    a.sel = g.sel; a.sel_mode = g.sel ? g.sel_mode : 0; a.sel_groups = g.sel ? g.sel_rows / 16 : 0;
    a.klog = K; a.nblog = nb; a.nlog = n_log; a.xscale = g.xscale; a.xscale_run = g.xscale_run > 0 ? g.xscale_run : 1;
    a.err = c->d_err;

    {
        const cudaError_t e = ensure_dynamic_smem(c, gemv_mma_q4k_kernel<kWarps>, smem);
        if (e != cudaSuccess) return cuda_status(c, e, "gemv_mma attr");
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(G));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = c->use_pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_mma_q4k_kernel<kWarps>, a);
    c->launches++;
    return cuda_status(c, e, "gemv_mma launch");
}

}  // namespace

int launch_gemv_mma(Context* c, const GemvArgs& g, cudaStream_t s) { return launch_mma_t<8>(c, g, s); }

}  // namespace ggb
