// One decode step of the generic decoder graph as ONE persistent kernel (src/cli/main.cpp:3235-3512 for a single
// token): per layer  q/k/v projections -> RoPE + KV append + attention -> output projection (+ residual) ->
// gate/up + SwiGLU -> down (+ residual),  then the final norm and the logits GEMV.
//
// Why one kernel: at batch 1 every matrix of a 1B..8B model streams in 1-5 us, so a step made of one launch per
// matrix spends most of its time in launch gaps, prologues and pipeline ramps with the HBM idle.  Here one CTA per
// SM lives for the whole step:
//   * every warp owns a ring of shared-memory stages and a fixed sequence of weight tiles that runs through ALL
//     phases and layers in schedule order.  When a warp has consumed a tile it requests, into the stage it just
//     freed, the tile that lies one ring length ahead in its sequence (cp.async.bulk -> mbarrier).  Weights need no
//     activations, so the requests run ahead of the computation across phase boundaries and layers (the rings hold
//     ~166 KB per SM, 24 MB over the GPU) and the weight stream does not wait for a dependency.  (A dedicated
//     producer warp whose lanes poll one "stage free" barrier per ring was measured first: the polls of one lane held
//     up the refills of the others and every phase ran about twice as long.)
//   * the eight warps run the phases.  A phase = wait at a grid-wide barrier for the previous phase's output,
//     read the activation vector (L2), split it into int8 limbs, run the int8 tensor-core tiles that are already in
//     shared memory, reduce, apply the epilogue, store, arrive at the next barrier;
//   * the attention phase (the split-KV kernel's body, four warps per (KV head, split)) runs inside the same kernel;
//     its per-split results are merged by the output projection's prologue.
// The arithmetic of a tile is that of gemv_mma_q4k_kernel (ggb_gemv_mma.cu), specialised to one activation row.
//
// Grid-wide barrier: one monotonically increasing counter in global memory (zeroed by a memset node before the
// launch); barrier k is passed when the counter reaches k * gridDim.x.  All CTAs must be co-resident, which the
// cooperative launch guarantees.  Every wait (mbarrier, grid barrier) is bounded; on expiry the kernel records a code
// in the context's device error word, stops waiting at later barriers and runs to its end.
#include <cuda_bf16.h>

#include "ggb_attn_tile.cuh"
#include "ggb_decode_step.h"
#include "ggb_internal.h"

namespace ggb {

namespace {

constexpr int kWarps = 8;                        // warps per CTA
constexpr int kStageBytes = 6912;                // 3 Q4_K (row group, block) units of 2304 B, or 2 Q6_K units of 3360 B
constexpr int kMaxP = 4;
constexpr uint32_t kSpinLimit = 1u << 17;        // mbarrier polls (each can suspend for microseconds)
constexpr uint32_t kGridSpinLimit = 1u << 21;    // grid-barrier polls (~1 us each)

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
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory"); }
__device__ __forceinline__ void attn_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

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

// Optional time stamps (compile with -DGGB_STEP_TRACE): CTA 1, thread 0 writes %globaltimer into a device array that
// ggb_step_trace_read hands to the host.  Compiled out otherwise.
#ifdef GGB_STEP_TRACE
__device__ unsigned long long g_step_trace[4096];
__device__ int g_step_trace_n;
__device__ __forceinline__ void stamp(int tag) {
    __shared__ int n_s;                          // written by thread 0 only; stores are fire-and-forget, no load on the path
    if (blockIdx.x == 1 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        const int i = tag == 0 ? 0 : n_s;
        if (i < 2047) { g_step_trace[2 * i] = t; g_step_trace[2 * i + 1] = static_cast<unsigned long long>(tag); n_s = i + 1; g_step_trace_n = i + 1; }
    }
}
#else
__device__ __forceinline__ void stamp(int) {}
#endif

// Shared-memory views of one CTA.
struct Smem {
    uint8_t* ring;       // [kWarps][P][kStageBytes]
    int8_t* xl;          // 3 limb planes of (Kmax + 16) bytes
    float* asum;         // sums of x over each 32-run
    float* asum16;       // sums of x over each 16-run
    float* xs;           // scale of each 256-block
    float* comb;         // [2][kWarps][2][16] team partials
    int plane_stride;
};

// ---- the weight-tile sequence of one warp ---------------------------------------------------------------------------
// Layer descriptors live in a window of four shared-memory slots (layer L in slot L & 3), refreshed as the computation
// advances; a request that runs further ahead than the window reads its descriptor from global memory.
constexpr int kLayerSlots = 4;

struct Desc {                                    // what the sequence and the phases need to find their matrices
    const StepLayer* slots;                      // shared memory, kLayerSlots entries
    const StepLayer* global;                     // device array of all layers
    const StepMat* out;                          // logits matrix (shared memory)
    const StepShape* shapes;                     // shared memory, kPhaseCount entries
    int n_layer;
};

// Position in the sequence: layer L (n_layer: the logits phase), GEMV phase p (0 q/k/v, 1 o, 2 gate/up, 3 down, 4 logits),
// row group rg of this CTA's range (team-strided), tile ti of the row group (member-strided).  All warp-uniform.
struct TileIt {
    int L, p, rg, ti;
    int n_rg, n_teams, member, ws, ntiles;       // of the current phase / row group
    int g_begin;
    const StepMat* w0;                           // matrix of the current row group (gate for the pair)
    const StepMat* w1;                           // up matrix of the pair
    int is_q6, sb, spr, nb;
    int64_t blk0;
    bool rg_ready, end;
};

__device__ __forceinline__ const StepMat* phase_mat(const StepLayer* l, const StepMat* out, int p, int mi) {
    switch (p) {
    case kPhaseQkv: return mi == 0 ? &l->q : (mi == 1 ? &l->k : &l->v);
    case kPhaseO: return &l->o;
    case kPhaseGateUp: return mi == 0 ? &l->gate : &l->up;
    case kPhaseDown: return &l->down;
    default: return out;
    }
}

__device__ __forceinline__ void it_begin_phase(TileIt& it, const Desc& d, int warp) {
    const StepShape& sh = d.shapes[it.p];
    it.g_begin = sh.g_begin; it.n_rg = sh.n_rg;
    it.ws = sh.ws; it.n_teams = kWarps >> sh.log_ws; it.member = warp & (sh.ws - 1); it.nb = sh.nb;
    it.rg = warp >> sh.log_ws; it.ti = it.member; it.rg_ready = false;
}

// Moves `it` to the next existing tile at or after its position; false at the end of the step.  `window_max` = the
// highest layer whose descriptor is valid in the shared-memory window.
__device__ __noinline__ bool it_seek(TileIt& it, const Desc& d, int warp, int window_max) {
    while (!it.end) {
        if (it.rg < it.n_rg) {
            if (!it.rg_ready) {
                const StepShape& sh = d.shapes[it.p];
                const int G_rg = it.g_begin + it.rg;
                const int mi = sh.nmat == 2 ? 0 : (sh.ncat > 1 && G_rg >= sh.g_start[1]) + (sh.ncat > 2 && G_rg >= sh.g_start[2]);
                const StepLayer* l = it.L <= window_max ? d.slots + (it.L & (kLayerSlots - 1)) : d.global + it.L;
                it.w0 = phase_mat(l, d.out, it.p, mi);
                it.w1 = sh.nmat == 2 ? phase_mat(l, d.out, it.p, 1) : it.w0;
                it.is_q6 = it.w0->type == T_Q6_K;
                it.sb = it.is_q6 ? sh.sb6 : sh.sb4;
                it.spr = it.is_q6 ? sh.spr6 : sh.spr4;
                it.ntiles = sh.nmat * it.spr;
                it.blk0 = static_cast<int64_t>(G_rg - (sh.nmat == 2 ? 0 : sh.g_start[mi])) * sh.nb;
                it.rg_ready = true;
            }
            if (it.ti < it.ntiles) return true;
            it.rg += it.n_teams; it.ti = it.member; it.rg_ready = false;
            continue;
        }
        // next phase
        if (it.p == kPhaseLogits) { it.end = true; break; }
        if (it.p == kPhaseDown) { it.p = kPhaseQkv; if (++it.L >= d.n_layer) it.p = kPhaseLogits; }
        else ++it.p;
        it_begin_phase(it, d, warp);
    }
    return false;
}

// Requests the tile `it` points at into ring stage s of this warp (lane 0 issues), then steps past it.
__device__ __forceinline__ void it_issue(TileIt& it, uint8_t* stage, uint64_t* full, int lane) {
    const int mat = it.ti >= it.spr, sl = it.ti - mat * it.spr;
    const int b0 = sl * it.sb, nbk = min(it.sb, it.nb - b0);
    if (lane == 0) {
        const StepMat* wm = mat ? it.w1 : it.w0;
        const int64_t gb = it.blk0 + b0;
        const uint8_t *p0 = wm->s[0], *p1 = wm->s[1];
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the stage was last read through the generic proxy
        if (!it.is_q6) {
            mbar_expect_tx(full, static_cast<uint32_t>(nbk) * 2304u);
            bulk_g2s(stage, p1 + gb * 2048, static_cast<uint32_t>(nbk) * 2048u, full);
            bulk_g2s(stage + it.sb * 2048, p0 + gb * 256, static_cast<uint32_t>(nbk) * 256u, full);
        } else {
            const uint8_t *p2 = wm->s[2], *p3 = wm->s[3];
            mbar_expect_tx(full, static_cast<uint32_t>(nbk) * 3360u);
            bulk_g2s(stage, p0 + gb * 2048, static_cast<uint32_t>(nbk) * 2048u, full);
            bulk_g2s(stage + it.sb * 2048, p1 + gb * 1024, static_cast<uint32_t>(nbk) * 1024u, full);
            bulk_g2s(stage + it.sb * 3072, p2 + gb * 256, static_cast<uint32_t>(nbk) * 256u, full);
            bulk_g2s(stage + it.sb * 3328, p3 + gb * 32, static_cast<uint32_t>(nbk) * 32u, full);
        }
    }
    it.ti += it.ws;
}

// ---- consumers ---------------------------------------------------------------------------------------------------

// x[k0 .. k0+7] (k0 a multiple of 8, all in one head) = the attention splits of that head merged (max, sum, acc per split).
__device__ __noinline__ void attn_merge8(const AttnPagedArgs& am, int k0, float (&v)[8]) {
    const int hd = am.head_dim;
    const int head = k0 / hd, d0 = k0 - head * hd;
    const int pos = am.d_pos ? am.d_pos[0] : am.pos0;
    const int keys_per_split = am.pages_per_split * am.page;
    const int n_active = min(am.n_splits, pos / keys_per_split + 1);
    const float* base = am.partial + static_cast<size_t>(head) * am.n_splits * (hd + 2);
    float mx = -INFINITY, lsum = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.0f;
#pragma unroll 2
    for (int s = 0; s < n_active; ++s) {
        const float* ps = base + static_cast<size_t>(s) * (hd + 2);
        const float m_s = __ldcg(ps), l_s = __ldcg(ps + 1);
        float2 p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = __ldcg(reinterpret_cast<const float2*>(ps + 2 + d0 + 2 * i));
        const float nm = fmaxf(mx, m_s);
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

// One pass over the activation row: optional gamma (the RMS factor is a scalar applied to the finished dot products),
// three int8 limbs per value with one scale per 256-block, run sums for the min / offset terms.  Returns this warp's
// part of sum(x^2) in red[warp].
__device__ __noinline__ void x_to_limbs(const float* x, const AttnPagedArgs* merge, const float* gamma, int K, const Smem* smp, float* red) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const Smem sm = *smp;
    float ss = 0.0f;
    for (int bb = warp; bb < (K >> 8); bb += 4 * kWarps) {
        float v[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int b = bb + u * kWarps;
            if (b < (K >> 8)) {
                const int k0 = b * 256 + lane * 8;
                if (merge) attn_merge8(*merge, k0, v[u]);
                else {
                    const float4 p0 = __ldcg(reinterpret_cast<const float4*>(x + k0)), p1 = __ldcg(reinterpret_cast<const float4*>(x + k0 + 4));
                    v[u][0] = p0.x; v[u][1] = p0.y; v[u][2] = p0.z; v[u][3] = p0.w; v[u][4] = p1.x; v[u][5] = p1.y; v[u][6] = p1.z; v[u][7] = p1.w;
                }
                if (gamma) {
                    const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + k0)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + k0 + 4));
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss = fmaf(v[u][i], v[u][i], ss);
                    v[u][0] *= g0.x; v[u][1] *= g0.y; v[u][2] *= g0.z; v[u][3] *= g0.w; v[u][4] *= g1.x; v[u][5] *= g1.y; v[u][6] *= g1.z; v[u][7] *= g1.w;
                }
            }
        }
        float am[4], sum[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            am[u] = 0.0f; sum[u] = 0.0f;
            if (bb + u * kWarps < (K >> 8)) {
#pragma unroll
                for (int i = 0; i < 8; ++i) { am[u] = fmaxf(am[u], fabsf(v[u][i])); sum[u] += v[u][i]; }
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
                    // round to nearest by adding 1.5 * 2^23: the integer lands in the low mantissa bits
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
                int8_t* pl = sm.xl + k0;
                *reinterpret_cast<uint2*>(pl) = make_uint2(w1[0], w1[1]);
                *reinterpret_cast<uint2*>(pl + sm.plane_stride) = make_uint2(w2[0], w2[1]);
                *reinterpret_cast<uint2*>(pl + 2 * sm.plane_stride) = make_uint2(w3[0], w3[1]);
                if (lane == 0) sm.xs[b] = am[u] / 127.0f;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) sum[u] += __shfl_xor_sync(0xFFFFFFFFu, sum[u], 1);      // 16-run = two lanes
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int b = bb + u * kWarps;
            if (b < (K >> 8) && (lane & 1) == 0) sm.asum16[(b * 256 + lane * 8) >> 4] = sum[u];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) sum[u] += __shfl_xor_sync(0xFFFFFFFFu, sum[u], 2);      // 32-run = four lanes
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int b = bb + u * kWarps;
            if (b < (K >> 8) && (lane & 3) == 0) sm.asum[(b * 256 + lane * 8) >> 5] = sum[u];
        }
    }
    ss = wsum(ss);
    if (lane == 0) red[warp] = ss;
}

// Lane constants of the mma fragment layout for one activation row (B columns 0..2 = the three limbs).
struct LaneCtx {
    int g, t, mshift;
    const int8_t* bplane;
    float lw0, lw1;
};

// nbk Q4_K (row group, block) units of one tile: f0/f1 = columns 2t, 2t+1 of row g, f2/f3 of row g+8; mn = min terms.
__device__ __forceinline__ void tile_q4k(const uint8_t* qsT, const uint8_t* hdrT, int nbk, int b0, const Smem& sm, const LaneCtx& lc, int lane,
                                         float& f0, float& f1, float& f2, float& f3, float& mnA, float& mnB) {
    const int g = lc.g, t = lc.t;
    for (int bl = 0; bl < nbk; ++bl) {
        const uint4 ha = *reinterpret_cast<const uint4*>(hdrT + (bl * 16 + g) * 16);
        const uint4 hb = *reinterpret_cast<const uint4*>(hdrT + (bl * 16 + g + 8) * 16);
        const uint32_t sa03 = ha.y & 0x3F3F3F3Fu, sa47 = (ha.w & 0x0F0F0F0Fu) | ((ha.y >> 2) & 0x30303030u);
        const uint32_t sb03 = hb.y & 0x3F3F3F3Fu, sb47 = (hb.w & 0x0F0F0F0Fu) | ((hb.y >> 2) & 0x30303030u);
        {   // min term: this lane covers sub-blocks 2t and 2t+1 of both rows
            const uint32_t ma = (t < 2 ? (ha.z & 0x3F3F3F3Fu) : (((ha.w >> 4) & 0x0F0F0F0Fu) | ((ha.z >> 2) & 0x30303030u))) >> lc.mshift;
            const uint32_t mb = (t < 2 ? (hb.z & 0x3F3F3F3Fu) : (((hb.w >> 4) & 0x0F0F0F0Fu) | ((hb.z >> 2) & 0x30303030u))) >> lc.mshift;
            const float dmA = __half2float(__ushort_as_half(static_cast<uint16_t>(ha.x >> 16)));
            const float dmB = __half2float(__ushort_as_half(static_cast<uint16_t>(hb.x >> 16)));
            const float2 as = *reinterpret_cast<const float2*>(sm.asum + (b0 + bl) * 8 + 2 * t);
            mnA = fmaf(dmA, static_cast<float>(ma & 0xFFu) * as.x + static_cast<float>((ma >> 8) & 0xFFu) * as.y, mnA);
            mnB = fmaf(dmB, static_cast<float>(mb & 0xFFu) * as.x + static_cast<float>((mb >> 8) & 0xFFu) * as.y, mnB);
        }
        int lo0 = 0, lo1 = 0, lo2 = 0, lo3 = 0, hi0 = 0, hi1 = 0, hi2 = 0, hi3 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 q = *reinterpret_cast<const uint4*>(qsT + (static_cast<size_t>(bl * 4 + j) * 32 + lane) * 16);
            const int8_t* bp = lc.bplane + ((b0 + bl) * 8 + 2 * j) * 32;
            const uint32_t bl0 = *reinterpret_cast<const uint32_t*>(bp), bl1 = *reinterpret_cast<const uint32_t*>(bp + 16);
            const uint32_t bh0 = *reinterpret_cast<const uint32_t*>(bp + 32), bh1 = *reinterpret_cast<const uint32_t*>(bp + 48);
            int cl[4], ch[4];
            mma_s8(cl, q.x & 0x0F0F0F0Fu, q.y & 0x0F0F0F0Fu, q.z & 0x0F0F0F0Fu, q.w & 0x0F0F0F0Fu, bl0, bl1);
            mma_u8s8(ch, q.x & 0xF0F0F0F0u, q.y & 0xF0F0F0F0u, q.z & 0xF0F0F0F0u, q.w & 0xF0F0F0F0u, bh0, bh1);
            const uint32_t wa = j < 2 ? sa03 : sa47, wb = j < 2 ? sb03 : sb47;
            const int sa0 = (wa >> (16 * (j & 1))) & 0xFF, sa1 = (wa >> (16 * (j & 1) + 8)) & 0xFF;
            const int sb0 = (wb >> (16 * (j & 1))) & 0xFF, sb1 = (wb >> (16 * (j & 1) + 8)) & 0xFF;
            lo0 += sa0 * cl[0]; lo1 += sa0 * cl[1]; lo2 += sb0 * cl[2]; lo3 += sb0 * cl[3];
            hi0 += sa1 * ch[0]; hi1 += sa1 * ch[1]; hi2 += sb1 * ch[2]; hi3 += sb1 * ch[3];
        }
        const float dA = __half2float(__ushort_as_half(static_cast<uint16_t>(ha.x & 0xFFFF)));
        const float dB = __half2float(__ushort_as_half(static_cast<uint16_t>(hb.x & 0xFFFF)));
        const float xb = sm.xs[b0 + bl];
        const float x0 = xb * lc.lw0, x1 = xb * lc.lw1;
        f0 = fmaf(static_cast<float>(lo0) + static_cast<float>(hi0) * 0.0625f, dA * x0, f0);
        f1 = fmaf(static_cast<float>(lo1) + static_cast<float>(hi1) * 0.0625f, dA * x1, f1);
        f2 = fmaf(static_cast<float>(lo2) + static_cast<float>(hi2) * 0.0625f, dB * x0, f2);
        f3 = fmaf(static_cast<float>(lo3) + static_cast<float>(hi3) * 0.0625f, dB * x1, f3);
    }
}

// nbk Q6_K units: qsT = low nibbles, s1T = high bits, s2T = int8 scales, s3T = d (see the layout notes in ggb_formats.cuh).
__device__ __forceinline__ void tile_q6k(const uint8_t* qsT, const uint8_t* s1T, const uint8_t* s2T, const uint8_t* s3T, int nbk, int b0,
                                         const Smem& sm, const LaneCtx& lc, int lane, float& f0, float& f1, float& f2, float& f3, float& mnA,
                                         float& mnB) {
    const int g = lc.g, t = lc.t;
    for (int bl = 0; bl < nbk; ++bl) {
        const uint4 sa = *reinterpret_cast<const uint4*>(s2T + (bl * 16 + g) * 16);
        const uint4 sb_ = *reinterpret_cast<const uint4*>(s2T + (bl * 16 + g + 8) * 16);
        const float dA = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(s3T + (bl * 16 + g) * 2)));
        const float dB = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(s3T + (bl * 16 + g + 8) * 2)));
        const uint32_t saw[4] = {sa.x, sa.y, sa.z, sa.w}, sbw[4] = {sb_.x, sb_.y, sb_.z, sb_.w};
        {   // quants are used unsigned (0..63): remove 32 * sc * sum(x) per 16-run; this lane covers runs 4t..4t+3
            const uint32_t wa = t == 0 ? sa.x : (t == 1 ? sa.y : (t == 2 ? sa.z : sa.w));
            const uint32_t wb = t == 0 ? sb_.x : (t == 1 ? sb_.y : (t == 2 ? sb_.z : sb_.w));
            const float4 as = *reinterpret_cast<const float4*>(sm.asum16 + (b0 + bl) * 16 + 4 * t);
            const float ca = static_cast<float>(static_cast<int8_t>(wa)) * as.x + static_cast<float>(static_cast<int8_t>(wa >> 8)) * as.y +
                             static_cast<float>(static_cast<int8_t>(wa >> 16)) * as.z + static_cast<float>(static_cast<int8_t>(wa >> 24)) * as.w;
            const float cb = static_cast<float>(static_cast<int8_t>(wb)) * as.x + static_cast<float>(static_cast<int8_t>(wb >> 8)) * as.y +
                             static_cast<float>(static_cast<int8_t>(wb >> 16)) * as.z + static_cast<float>(static_cast<int8_t>(wb >> 24)) * as.w;
            mnA = fmaf(dA * 32.0f, ca, mnA);
            mnB = fmaf(dB * 32.0f, cb, mnB);
        }
        int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const uint4 qh = *reinterpret_cast<const uint4*>(s1T + (static_cast<size_t>(bl * 2 + hf) * 32 + lane) * 16);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const uint4 ql = *reinterpret_cast<const uint4*>(qsT + (static_cast<size_t>(bl * 4 + 2 * hf + c) * 32 + lane) * 16);
                const uint32_t hA = c ? qh.z : qh.x, hB = c ? qh.w : qh.y;
                const uint32_t kf = 0x0F0F0F0Fu, k3 = 0x30303030u;
                const uint32_t a1g = (ql.x & kf) | ((hA << 4) & k3), a1h = (ql.z & kf) | ((hB << 4) & k3);
                const uint32_t a2g = (ql.y & kf) | ((hA << 2) & k3), a2h = (ql.w & kf) | ((hB << 2) & k3);
                const uint32_t a3g = ((ql.x >> 4) & kf) | (hA & k3), a3h = ((ql.z >> 4) & kf) | (hB & k3);
                const uint32_t a4g = ((ql.y >> 4) & kf) | ((hA >> 2) & k3), a4h = ((ql.w >> 4) & kf) | ((hB >> 2) & k3);
                const uint32_t ag[4] = {a1g, a2g, a3g, a4g}, ah[4] = {a1h, a2h, a3h, a4h};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int sidx = 8 * hf + 2 * i + c;
                    const uint32_t bw = *reinterpret_cast<const uint32_t*>(lc.bplane + ((b0 + bl) * 16 + sidx) * 16);
                    int cc[4];
                    mma_u8s8_k16(cc, ag[i], ah[i], bw);
                    const int sca = static_cast<int8_t>(saw[sidx >> 2] >> (8 * (sidx & 3)));
                    const int scb = static_cast<int8_t>(sbw[sidx >> 2] >> (8 * (sidx & 3)));
                    c0 += sca * cc[0]; c1 += sca * cc[1]; c2 += scb * cc[2]; c3 += scb * cc[3];
                }
            }
        }
        const float xb = sm.xs[b0 + bl];
        const float x0 = xb * lc.lw0, x1 = xb * lc.lw1;
        f0 = fmaf(static_cast<float>(c0), dA * x0, f0); f1 = fmaf(static_cast<float>(c1), dA * x1, f1);
        f2 = fmaf(static_cast<float>(c2), dB * x0, f2); f3 = fmaf(static_cast<float>(c3), dB * x1, f3);
    }
}

// Per-warp state that lives across phases (kept in shared memory between calls).
struct WarpState {
    TileIt iss;              // the next tile to request
    int st; uint32_t ph;     // ring stage and barrier parity of the next tile to consume
    bool ok;
};

enum : int { kEpiStore = 0, kEpiResidual = 1, kEpiSwiglu = 2 };

// One GEMV phase.  x: the activation row (nullptr with merge != nullptr: the merged attention splits); the residual
// epilogue adds onto y in place.  m0..m2: the phase's matrices (shared-memory descriptors).
__device__ __noinline__ void consume_phase(int p, const StepMat* m0, const StepMat* m1, const StepMat* m2, const float* x, const AttnPagedArgs* merge,
                                           const float* gamma, float eps, int epi, const Desc* dp, const Smem* smp, uint64_t* full_bar, float* red,
                                           int P, WarpState* wsp, int window_max, int* err) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const Desc d = *dp;
    stamp(1);
    x_to_limbs(x, merge, gamma, d.shapes[p].K, smp, red);
    consumer_sync();
    stamp(2);
    const StepShape sh = d.shapes[p];
    const Smem sm = *smp;
    const StepMat* const mats[3] = {m0, m1, m2};
    WarpState st = *wsp;
    const int K = sh.K, nb = sh.nb;
    float inv = 1.0f;
    if (gamma) {
        float tot = 0.0f;
#pragma unroll
        for (int i = 0; i < kWarps; ++i) tot += red[i];
        inv = 1.0f / sqrtf(tot / static_cast<float>(K) + eps);
    }
    LaneCtx lc;
    lc.g = lane >> 2; lc.t = lane & 3; lc.mshift = 16 * (lc.t & 1);
    lc.bplane = sm.xl + static_cast<size_t>(min(lc.g, 2)) * sm.plane_stride + 4 * lc.t;      // B column g (unused columns repeat the last)
    const int col0 = 2 * lc.t, col1 = 2 * lc.t + 1;
    lc.lw0 = col0 == 0 ? 1.0f : (col0 == 2 ? 1.0f / 16384.0f : 0.0f);
    lc.lw1 = col1 == 1 ? 1.0f / 128.0f : 0.0f;

    const int g_begin = sh.g_begin, n_rg = sh.n_rg;
    const int n_teams = kWarps >> sh.log_ws, team = warp >> sh.log_ws, member = warp & (sh.ws - 1);
    int parity = 0;
    for (int rg = team; rg < n_rg; rg += n_teams, parity ^= 1) {
        const int G_rg = g_begin + rg;
        const int mi = sh.nmat == 2 ? 0 : (sh.ncat > 1 && G_rg >= sh.g_start[1]) + (sh.ncat > 2 && G_rg >= sh.g_start[2]);
        const StepMat* w0 = mats[mi];
        const bool is_q6 = w0->type == T_Q6_K;
        const int sb = is_q6 ? sh.sb6 : sh.sb4, spr = is_q6 ? sh.spr6 : sh.spr4;
        float F0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, F1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        float MN0[2] = {0.0f, 0.0f}, MN1[2] = {0.0f, 0.0f};                  // [row g / g+8]
        for (int ti = member; ti < sh.nmat * spr; ti += sh.ws) {
            const int s = warp * P + st.st;
            if (st.ok) st.ok = mbar_wait(&full_bar[s], st.ph, err, 2);
            if (++st.st == P) { st.st = 0; st.ph ^= 1; }
            if (!st.ok) continue;
            stamp(6);
            const int mat = ti >= spr, sl = ti - mat * spr;
            const int b0 = sl * sb, nbk = min(sb, nb - b0);
            const uint8_t* qsT = sm.ring + static_cast<size_t>(s) * kStageBytes;
            const uint8_t* s1T = qsT + sb * 2048;
            float f0 = 0.0f, f1 = 0.0f, f2 = 0.0f, f3 = 0.0f, mnA = 0.0f, mnB = 0.0f;
            if (!is_q6) tile_q4k(qsT, s1T, nbk, b0, sm, lc, lane, f0, f1, f2, f3, mnA, mnB);
            else tile_q6k(qsT, s1T, s1T + sb * 1024, s1T + sb * 1280, nbk, b0, sm, lc, lane, f0, f1, f2, f3, mnA, mnB);
            if (mat == 0) { F0[0] += f0; F0[1] += f1; F0[2] += f2; F0[3] += f3; MN0[0] += mnA; MN0[1] += mnB; }
            else { F1[0] += f0; F1[1] += f1; F1[2] += f2; F1[3] += f3; MN1[0] += mnA; MN1[1] += mnB; }
            stamp(7);
            __syncwarp();
            // the stage is free: request the tile one ring length ahead in this warp's sequence
            if (it_seek(st.iss, d, warp, window_max)) it_issue(st.iss, sm.ring + static_cast<size_t>(s) * kStageBytes, &full_bar[s], lane);
        }
        // fold the limb columns (lanes t = 0..3 of a row) and the min terms
        float va[2], vb[2];
#pragma unroll
        for (int mat = 0; mat < 2; ++mat) {
            const float* F = mat ? F1 : F0;
            float pa = (col0 < 3 ? F[0] : 0.0f) + (col1 < 3 ? F[1] : 0.0f) - (mat ? MN1[0] : MN0[0]);
            float pb = (col0 < 3 ? F[2] : 0.0f) + (col1 < 3 ? F[3] : 0.0f) - (mat ? MN1[1] : MN0[1]);
            pa += __shfl_xor_sync(0xFFFFFFFFu, pa, 1); pa += __shfl_xor_sync(0xFFFFFFFFu, pa, 2);
            pb += __shfl_xor_sync(0xFFFFFFFFu, pb, 1); pb += __shfl_xor_sync(0xFFFFFFFFu, pb, 2);
            va[mat] = pa * inv; vb[mat] = pb * inv;
        }
        const int64_t row_base = static_cast<int64_t>(G_rg - (sh.nmat == 2 ? 0 : sh.g_start[mi])) * 16;
        const int64_t n_rows = w0->N;
        float* const yb = w0->y;
        auto finish = [&](float v, float v2, int64_t row) {
            if (row >= n_rows) return;
            if (epi == kEpiSwiglu) v = (v / (1.0f + expf(-v))) * v2;
            else if (epi == kEpiResidual) v += __ldcg(yb + row);
            yb[row] = v;
        };
        if (sh.ws == 1) {
            if (lc.t == 0) { finish(va[0], va[1], row_base + lc.g); finish(vb[0], vb[1], row_base + lc.g + 8); }
        } else {
            float* cb = sm.comb + (parity * kWarps + warp) * 32;
            if (lc.t == 0) {
#pragma unroll
                for (int mat = 0; mat < 2; ++mat) { cb[mat * 16 + lc.g] = va[mat]; cb[mat * 16 + lc.g + 8] = vb[mat]; }
            }
            asm volatile("bar.sync %0, %1;" ::"r"(3 + team), "r"(sh.ws * 32) : "memory");
            if (member == 0 && lane < 16) {
                float v = 0.0f, v2 = 0.0f;
                for (int j = 0; j < sh.ws; ++j) {
                    const float* cj = sm.comb + (parity * kWarps + team * sh.ws + j) * 32;
                    v += cj[lane]; v2 += cj[16 + lane];
                }
                finish(v, v2, row_base + lane);
            }
        }
    }
    if (lane == 0) *wsp = st;
    stamp(3);
}

// Attention phase of one layer: warps 0..3 of each CTA take the (KV head, split) items blockIdx.x, blockIdx.x + gridDim.x, ...
// over the splits that hold visible keys; the other warps pass through.
template <int HD>
__device__ __noinline__ void attn_phase(const AttnPagedArgs* atp, uint32_t* tile_smem) {
    const AttnPagedArgs& at = *atp;
    if ((threadIdx.x >> 5) >= 4) return;
    const int pos = at.d_pos ? at.d_pos[0] : at.pos0;
    const int n_active = min(at.n_splits, pos / (at.pages_per_split * at.page) + 1);
    for (int item = blockIdx.x; item < at.n_kv * n_active; item += gridDim.x) {
        const int h = item % at.n_kv, split = item / at.n_kv;
        attn_tile_body<HD, true>(at, h, split, 0, threadIdx.x, tile_smem, [] { attn_sync(); });
        attn_sync();                       // the next item reuses the shared-memory tiles
    }
}

// Grid-wide barrier number `k` (1, 2, ...): arrive, then wait until all CTAs have arrived k times.
__device__ __noinline__ void grid_barrier(unsigned* bar, unsigned k, bool& failed, int* err) {
    consumer_sync();                                   // this CTA's stores of the phase are done (all consumer warps)
    stamp(4);
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(bar, 1u);
        if (!failed) {
            const unsigned target = k * gridDim.x;
            uint32_t spins = 0;
            while (*reinterpret_cast<volatile unsigned*>(bar) < target) {
                if (++spins >= kGridSpinLimit) { atomicExch(err, 6); failed = true; break; }
                if ((spins & 255u) == 0 && *reinterpret_cast<volatile int*>(err) != 0) { failed = true; break; }
            }
        }
        __threadfence();
    }
    consumer_sync();
    stamp(5);
}

template <int HD>
__global__ void __launch_bounds__(kWarps * 32, 1) decode_step_kernel(const StepArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[kWarps * kMaxP];
    __shared__ float red[kWarps];
    __shared__ AttnPagedArgs at_s;
    __shared__ StepShape sh_s[kPhaseCount];
    __shared__ StepMat out_mat_s;
    __shared__ StepLayer layer_s[kLayerSlots];
    __shared__ Smem sm_s;
    __shared__ Desc desc_s;
    __shared__ WarpState ws_s[kWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int P = a.P;
    Smem sm;
    sm.ring = smem;
    sm.xl = reinterpret_cast<int8_t*>(smem + static_cast<size_t>(kWarps) * P * kStageBytes);
    sm.plane_stride = a.k_max + 16;
    sm.asum = reinterpret_cast<float*>(sm.xl + a.fixed_bytes - sizeof(float) * (a.k_max / 32 + a.k_max / 16 + a.k_max / 256 + 2 * kWarps * 32));
    sm.asum16 = sm.asum + a.k_max / 32;
    sm.xs = sm.asum16 + a.k_max / 16;
    sm.comb = sm.xs + a.k_max / 256;
    auto load_layer = [&](int L) {               // all threads: descriptor of layer L into its window slot
        const uint32_t* src = reinterpret_cast<const uint32_t*>(a.layers + L);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&layer_s[L & (kLayerSlots - 1)]);
        for (int i = threadIdx.x; i < static_cast<int>(sizeof(StepLayer) / 4); i += kWarps * 32) dst[i] = src[i];
    };
    for (int L = 0; L < kLayerSlots && L < a.n_layer; ++L) load_layer(L);
    if (threadIdx.x == 0) {
        sm_s = sm;
        out_mat_s = a.out;
        for (int i = 0; i < kPhaseCount; ++i) {
            sh_s[i] = a.shape[i];
            const int64_t g0 = static_cast<int64_t>(blockIdx.x) * sh_s[i].groups / gridDim.x;
            sh_s[i].g_begin = static_cast<int>(g0);
            sh_s[i].n_rg = static_cast<int>(static_cast<int64_t>(blockIdx.x + 1) * sh_s[i].groups / gridDim.x - g0);
        }
        desc_s.slots = layer_s; desc_s.global = a.layers; desc_s.out = &out_mat_s; desc_s.shapes = sh_s; desc_s.n_layer = a.n_layer;
        for (int s = 0; s < kWarps * P; ++s) mbar_init(&full_bar[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    stamp(0);
    {   // fill this warp's ring with the first P tiles of its sequence
        WarpState st{};
        st.iss.L = 0; st.iss.p = a.n_layer > 0 ? kPhaseQkv : kPhaseLogits; st.iss.end = false;
        it_begin_phase(st.iss, desc_s, warp);
        for (int i = 0; i < P; ++i)
            if (it_seek(st.iss, desc_s, warp, kLayerSlots - 1)) it_issue(st.iss, sm.ring + static_cast<size_t>(warp * P + i) * kStageBytes, &full_bar[warp * P + i], lane);
        st.st = 0; st.ph = 0u; st.ok = true;
        if (lane == 0) ws_s[warp] = st;
        __syncwarp();
    }

    bool failed = false;
    unsigned bar_k = 0;
    const StepMat* const out_m = &out_mat_s;
    WarpState* const wsp = &ws_s[warp];
    for (int L = 0; L < a.n_layer; ++L) {
        const StepLayer* l = &layer_s[L & (kLayerSlots - 1)];
        // the window moves on: layer L + 2 replaces layer L - 2 (published by the next barrier)
        if (L >= 2 && L + 2 < a.n_layer) load_layer(L + 2);
        const int win_a = max(kLayerSlots - 1, L + 1), win_b = max(kLayerSlots - 1, L + 2);
        // q / k / v projections of the normalised hidden row
        consume_phase(kPhaseQkv, &l->q, &l->k, &l->v, a.x, nullptr, l->attn_norm, a.eps, kEpiStore, &desc_s, &sm_s, full_bar, red, P, wsp, win_a, a.err);
        if (threadIdx.x == 0) {      // this layer's attention arguments (published by the barrier below; last read two barriers ago)
            at_s = a.attn;
            at_s.k_cache = l->k_cache; at_s.v_cache = l->v_cache; at_s.k_cache_w = l->k_cache; at_s.v_cache_w = l->v_cache;
        }
        grid_barrier(a.bar, ++bar_k, failed, a.err);
        attn_phase<HD>(&at_s, reinterpret_cast<uint32_t*>(sm.xl));      // RoPE + KV append + attention; warps 0..3 run the (KV head, split) items
        grid_barrier(a.bar, ++bar_k, failed, a.err);
        // output projection of the merged splits, + residual
        consume_phase(kPhaseO, &l->o, &l->o, &l->o, nullptr, &at_s, nullptr, a.eps, kEpiResidual, &desc_s, &sm_s, full_bar, red, P, wsp, win_b, a.err);
        grid_barrier(a.bar, ++bar_k, failed, a.err);
        // silu(gate x) * (up x) of the normalised row
        consume_phase(kPhaseGateUp, &l->gate, &l->up, &l->up, a.x, nullptr, l->ffn_norm, a.eps, kEpiSwiglu, &desc_s, &sm_s, full_bar, red, P, wsp, win_b, a.err);
        grid_barrier(a.bar, ++bar_k, failed, a.err);
        // down projection + residual
        consume_phase(kPhaseDown, &l->down, &l->down, &l->down, a.act, nullptr, nullptr, a.eps, kEpiResidual, &desc_s, &sm_s, full_bar, red, P, wsp, win_b, a.err);
        grid_barrier(a.bar, ++bar_k, failed, a.err);
    }
    // final norm + logits
    consume_phase(kPhaseLogits, out_m, out_m, out_m, a.x, nullptr, a.out_norm, a.eps, kEpiStore, &desc_s, &sm_s, full_bar, red, P, wsp, a.n_layer, a.err);
}

// Team width and tile depth of a phase, as launch_gemv_mma chooses them for a single launch.
void plan_shape(StepShape& sh, int n_cta) {
    const int gpc = (sh.groups + n_cta - 1) / n_cta;                // row groups of the busiest CTA
    int ws = 1;
    while (ws < kWarps && gpc * ws < kWarps) ws <<= 1;
    sh.ws = ws;
    auto depth = [&](int cap) {
        int sb = cap;
        while (sb > 1 && sh.nmat * ((sh.nb + sb - 1) / sb) < ws) --sb;
        return std::min(sb, sh.nb);
    };
    sh.sb4 = depth(3);
    sh.sb6 = depth(2);
    sh.log_ws = ws == 1 ? 0 : (ws == 2 ? 1 : (ws == 4 ? 2 : 3));
    sh.spr4 = (sh.nb + sh.sb4 - 1) / sh.sb4;
    sh.spr6 = (sh.nb + sh.sb6 - 1) / sh.sb6;
}

}  // namespace

bool step_mat_ok(const PackedW& w) { return (w.type == T_Q4_K || w.type == T_Q6_K) && w.layout == 1 && w.K % 256 == 0; }

StepMat step_mat(const PackedW& w, float* y) {
    StepMat m{};
    for (int i = 0; i < 4; ++i) m.s[i] = w.s[i];
    m.type = w.type; m.nb = w.nb; m.N = w.N; m.y = y;
    return m;
}

void step_shape_init(StepShape& sh, int K, int64_t n0, int64_t n1, int64_t n2, bool dual, int n_cta) {
    sh = StepShape{};
    sh.K = K; sh.nb = K / 256;
    sh.nmat = dual ? 2 : 1;
    const int g0 = static_cast<int>((n0 + 15) / 16);
    sh.g_start[0] = 0; sh.groups = g0; sh.ncat = 1;
    if (!dual && n1 > 0) { sh.g_start[1] = sh.groups; sh.groups += static_cast<int>((n1 + 15) / 16); sh.ncat = 2; }
    if (!dual && n2 > 0) { sh.g_start[2] = sh.groups; sh.groups += static_cast<int>((n2 + 15) / 16); sh.ncat = 3; }
    plan_shape(sh, n_cta);
}

// Shared memory after the rings: limb planes + run sums + team partials, or the attention tiles, whichever is larger.
size_t step_fixed_bytes(int k_max, int head_dim) {
    const size_t tail = sizeof(float) * (k_max / 32 + k_max / 16 + k_max / 256 + 2 * kWarps * 32);
    const size_t limbs = static_cast<size_t>(3) * (k_max + 16);
    const size_t attn = head_dim == 64 ? attn_tile_smem(64) : attn_tile_smem(128);
    return ((std::max(limbs, attn) + 15) / 16) * 16 + tail;
}

int launch_decode_step(Context* c, StepArgs& a, int head_dim, cudaStream_t s) {
    const int n_cta = a.n_cta;
    const size_t fixed = step_fixed_bytes(a.k_max, head_dim);
    int P = kMaxP;
    while (P > 1 && static_cast<size_t>(kWarps) * P * kStageBytes + fixed > 220 * 1024) --P;
    const size_t smem = static_cast<size_t>(kWarps) * P * kStageBytes + fixed;
    if (smem > 227 * 1024 || P < 2) return GGB_NOT_FOUND;
    a.P = P; a.fixed_bytes = static_cast<int>(fixed);
    void (*kern)(const StepArgs) = head_dim == 64 ? decode_step_kernel<64> : decode_step_kernel<128>;
    cudaError_t e = ensure_dynamic_smem(c, kern, smem);
    if (e != cudaSuccess) return cuda_status(c, e, "decode_step attr");
    e = cudaMemsetAsync(a.bar, 0, sizeof(unsigned), s);
    if (e != cudaSuccess) return cuda_status(c, e, "decode_step barrier reset");
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(n_cta));
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;       // all CTAs co-resident: the grid-wide barriers depend on it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kern, a);
    c->launches++;
    return cuda_status(c, e, "decode_step launch");
}

}  // namespace ggb

#ifdef GGB_STEP_TRACE
// Copies out and clears the stamps: pairs (time in ns, tag); tags 1 phase start, 2 limbs done, 6 tile arrived, 7 tile
// computed, 3 phase done, 4 at the barrier (all warps of the CTA arrived), 5 barrier passed.
extern "C" __attribute__((visibility("default"))) int ggb_step_trace_read(unsigned long long* out, int cap) {
    int n = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(&n, ggb::g_step_trace_n, sizeof(int));
    n = n < cap ? n : cap;
    cudaMemcpyFromSymbol(out, ggb::g_step_trace, sizeof(unsigned long long) * 2 * n);
    const int zero = 0;
    cudaMemcpyToSymbol(ggb::g_step_trace_n, &zero, sizeof(int));
    return n;
}
#endif
