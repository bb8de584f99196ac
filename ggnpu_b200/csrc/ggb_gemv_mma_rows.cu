// Small-batch GEMV for Q4_K / Q6_K in the row-group-major layout, 3 <= M <= 16 activation rows in ONE pass over the
// weights:   y[m][n] = sum_k x[m][k] * W[n][k]          (mul_mat_weight, src/cli/main.cpp:1367-1434, at M <= 16: the
// reference's small-M decode kernel that its speculative verification relies on, src/cli/main.cpp:2295-2297).
//
// gemv_mma_q4k_kernel (ggb_gemv_mma.cu) carries two activation rows per pass, so 16 rows streamed a matrix eight times.
// Here the three int8 limbs of up to 16 rows form up to 48 columns of the B operand = CG column groups of 8; a weight
// fragment is loaded from shared memory once and feeds 2 * CG tensor-core instructions:
//   column c = 3 m + p  (m activation row, p limb, weight 1, 1/128, 1/16384), column group c / 8, lane pair (c % 8) / 2.
// The min term of Q4_K (dmin * m_sub * sum of x over the sub-block) and the -32 offset of Q6_K are float products per
// (weight row, activation row); lane (g, t) accumulates those of rows g, g + 8 and activation rows t, t + 4, ... and adds
// them to the limb-0 column of the row (its weight is 1) in the slab, so the three columns of a row simply add up.  At the end of a row group
// every warp drops its column sums into a shared-memory slab; the team's first warp adds slabs and limb columns, applies
// the epilogue and stores.
// Shared memory bounds rows x K: 3 planes of K + 16 bytes per row (16 rows at K = 2048, 8 at 4096).  A longer K is cut
// into slices of whole 256-blocks along grid.y: CTA (x, y) covers its row groups over slice y only, so the matrix is
// still streamed once; the slices' partial sums go to a workspace [slice][matrix][m][N] and a small second kernel adds
// them in slice order and applies the epilogue.  Eight warps, each with its own ring of bulk-copy stages: a warp requests the tile one
// ring length ahead whenever it has consumed one (no producer warp, so 256 threads and the full register file per thread).
#include "ggb_internal.h"
#include "ggb_limbs.h"

namespace ggb {

namespace {

constexpr int kWarps = 8;
constexpr int kMaxStages = 64;
constexpr uint32_t kSpinLimit = 1u << 17;

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
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory"); }

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

// grid (M), 256 threads: row m.  Warp w converts the 256-blocks w, w + 8, ...: limbs of x * gamma, run sums, the block's
// sum of squares; thread 0 then adds the sums of squares in block order (so the factor does not depend on timing).
__global__ void __launch_bounds__(256) rows_prep_kernel(const float* __restrict__ x, int lda, int M, int K, const float* __restrict__ gamma, float eps,
                                                         uint8_t* __restrict__ img) {
    extern __shared__ float ssb[];                      // [K / 256]
    const LimbImage L(M, K);
    const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nblk = K >> 8;
    int8_t* planes = reinterpret_cast<int8_t*>(img + L.planes) + static_cast<size_t>(3 * m) * K;
    float* asum = reinterpret_cast<float*>(img + L.asum) + static_cast<size_t>(m) * (K >> 5);
    float* asum16 = reinterpret_cast<float*>(img + L.asum16) + static_cast<size_t>(m) * (K >> 4);
    float* xs = reinterpret_cast<float*>(img + L.xs) + static_cast<size_t>(m) * nblk;
    pdl_wait();                                         // x is the predecessor's output; the image may still be read by it
    pdl_launch();
    for (int b0 = warp; b0 < nblk; b0 += 4 * 8) {       // four blocks per warp in flight
        float v[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int b = b0 + 8 * u;
            if (b < nblk) {
                const float* xr = x + static_cast<size_t>(m) * lda + b * 256 + lane * 8;
                const float4 p0 = __ldg(reinterpret_cast<const float4*>(xr)), p1 = __ldg(reinterpret_cast<const float4*>(xr + 4));
                v[u][0] = p0.x; v[u][1] = p0.y; v[u][2] = p0.z; v[u][3] = p0.w; v[u][4] = p1.x; v[u][5] = p1.y; v[u][6] = p1.z; v[u][7] = p1.w;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int b = b0 + 8 * u;
            if (b >= nblk) continue;
            const int k0 = b * 256 + lane * 8;
            if (gamma) {
                float ss = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(v[u][i], v[u][i], ss);
                ss = wsum(ss);
                if (lane == 0) ssb[b] = ss;
                const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + k0)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + k0 + 4));
                v[u][0] *= g0.x; v[u][1] *= g0.y; v[u][2] *= g0.z; v[u][3] *= g0.w; v[u][4] *= g1.x; v[u][5] *= g1.y; v[u][6] *= g1.z; v[u][7] *= g1.w;
            }
            float am = 0.0f, sm = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) { am = fmaxf(am, fabsf(v[u][i])); sm += v[u][i]; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, o));
            const float rs = am > 0.0f ? 127.0f / am : 0.0f;
            uint32_t w1[2] = {0, 0}, w2[2] = {0, 0}, w3[2] = {0, 0};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float kMagic = 12582912.0f;           // 1.5 * 2^23: round to nearest, the integer lands in the low mantissa bits
                const float r = fminf(fmaxf(v[u][i] * rs, -127.0f), 127.0f);
                const float t1 = r + kMagic;
                const float r2 = (r - (t1 - kMagic)) * 128.0f;
                const float t2 = r2 + kMagic;
                const float t3 = (r2 - (t2 - kMagic)) * 128.0f + kMagic;
                w1[i >> 2] |= (__float_as_uint(t1) & 0xFFu) << (8 * (i & 3));
                w2[i >> 2] |= (__float_as_uint(t2) & 0xFFu) << (8 * (i & 3));
                w3[i >> 2] |= (__float_as_uint(t3) & 0xFFu) << (8 * (i & 3));
            }
            *reinterpret_cast<uint2*>(planes + k0) = make_uint2(w1[0], w1[1]);
            *reinterpret_cast<uint2*>(planes + K + k0) = make_uint2(w2[0], w2[1]);
            *reinterpret_cast<uint2*>(planes + 2 * static_cast<size_t>(K) + k0) = make_uint2(w3[0], w3[1]);
            if (lane == 0) xs[b] = am / 127.0f;
            sm += __shfl_xor_sync(0xFFFFFFFFu, sm, 1);
            if ((lane & 1) == 0) asum16[k0 >> 4] = sm;
            sm += __shfl_xor_sync(0xFFFFFFFFu, sm, 2);
            if ((lane & 3) == 0) asum[k0 >> 5] = sm;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.0f;
        if (gamma) for (int b = 0; b < nblk; ++b) tot += ssb[b];
        reinterpret_cast<float*>(img + L.inv_s)[m] = gamma ? 1.0f / sqrtf(tot / static_cast<float>(K) + eps) : 1.0f;
    }
}

struct RowsArgs {
    PackedW w, w2;
    const float* x;
    float* y;
    const float* bias;
    const float* resid;
    const float* gamma;
    float eps;
    int M, lda, ldc, epi;
    int sb, nmat, groups, ws, P, stage_bytes;
    const uint8_t* img;   // activation image written by rows_prep_kernel (layout: LimbImage)
    int kbs;              // 256-blocks of K per slice (grid.y slices); nb when K is not cut
    float* part;          // K cut into slices: partial sums [slice][matrix][m][N], epilogue in rows_reduce_kernel; else nullptr
    int* err;
    // stream kernel only: up to two more matrices stacked along N behind w (q | k | v of one layer): they share x, K and the
    // format; row groups from cat_g0[i] on belong to matrix i + 1, which has its own streams, output, bias and row count
    int ncat;
    int cat_g0[2];
    PackedW cat_w[2];
    float* cat_y[2];
    const float* cat_bias[2];
    int cat_ldc[2];
};

// dynamic shared memory: [ring: 8 * P * stage_bytes][limb planes: 3 M (K + 16)][asum: M K/32][asum16: M K/16][xs: M K/256]
//                        [slab: 8 warps * nmat * 16 rows * 8 CG columns floats]
template <int CG, int NMAT>
__global__ void __launch_bounds__(kWarps * 32, 1) gemv_mma_rows_kernel(const RowsArgs a) {
    constexpr int NC = 8 * CG;                         // B columns
    constexpr int MI = CG == 2 ? 2 : (CG == 3 ? 2 : 4);   // activation rows per lane in the min / offset term: m = t + 4 i < M
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages], x_bar;
    __shared__ float inv_s[16];
    const int nb = a.w.nb, M = a.M;
    const int kb0 = blockIdx.y * a.kbs, nbs = min(a.kbs, nb - kb0);      // this CTA's slice of K: blocks [kb0, kb0 + nbs)
    const int K = a.kbs * 256;                         // capacity of the slice-local activation arrays
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int spr = (nbs + a.sb - 1) / a.sb;           // tiles per row group and matrix
    const int tprg = NMAT * spr;
    const int plane_stride = K + 16;
    uint8_t* ring = smem;
    int8_t* xl = reinterpret_cast<int8_t*>(ring + static_cast<size_t>(kWarps) * a.P * a.stage_bytes);
    float* asum = reinterpret_cast<float*>(xl + static_cast<size_t>(3 * M) * plane_stride);
    float* asum16 = asum + M * (K >> 5);
    float* xs = asum16 + M * (K >> 4);
    float* slab = xs + ((M * (K >> 8) + 3) & ~3);      // [warp][mat][16][NC], 16-byte aligned (float2 stores)

    const int64_t g_begin = static_cast<int64_t>(blockIdx.x) * a.groups / gridDim.x;
    const int n_rg = static_cast<int>(static_cast<int64_t>(blockIdx.x + 1) * a.groups / gridDim.x - g_begin);
    const int n_teams = kWarps / a.ws;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWarps * a.P; ++s) mbar_init(&full_bar[s], 1);
        mbar_init(&x_bar, kWarps);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch();

    // ---------------- every warp requests its own tiles: the one a ring length ahead whenever it frees a stage ----------------
    const int team = warp / a.ws, member = warp % a.ws;
    const bool is_q6 = a.w.type == T_Q6_K;
    int rg_i = team, ti_i = member, st_i = 0;          // next tile to request, and the stage it goes to
    auto issue_next = [&]() {
        while (rg_i < n_rg && ti_i >= tprg) { rg_i += n_teams; ti_i = member; }
        if (rg_i >= n_rg) return;
        const int s = warp * a.P + st_i;
        if (lane == 0) {
            const int mat = ti_i >= spr, sl = ti_i - mat * spr;
            const int b0 = sl * a.sb, nbk = min(a.sb, nbs - b0);
            uint8_t* dst = ring + static_cast<size_t>(s) * a.stage_bytes;
            const PackedW& w = mat ? a.w2 : a.w;
            const int64_t gb = (g_begin + rg_i) * nb + kb0 + b0;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the stage was last read through the generic proxy
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
        }
        ti_i += a.ws;
        if (++st_i == a.P) st_i = 0;
    };
    for (int i = 0; i < a.P; ++i) issue_next();        // weights do not depend on the predecessor kernel: before the wait

    // ---------------- consumers ----------------
    const int g = lane >> 2, t = lane & 3;
    const int ncol = 3 * M;
    // per column group: this lane's B column (plane), its two C columns, their activation row and limb weight
    const int8_t* bplane[CG];
    int mrow[CG][2];
    float lw[CG][2];
#pragma unroll
    for (int q = 0; q < CG; ++q) {
        bplane[q] = xl + static_cast<size_t>(min(8 * q + g, ncol - 1)) * plane_stride + 4 * t;
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
            const int col = 8 * q + 2 * t + sl;
            const bool valid = col < ncol;
            mrow[q][sl] = valid ? col / 3 : M - 1;
            const int p = col % 3;
            lw[q][sl] = valid ? (p == 0 ? 1.0f : (p == 1 ? 1.0f / 128.0f : 1.0f / 16384.0f)) : 0.0f;
        }
    }
    pdl_wait();
    // The activation image of this CTA's slice of K: 5 bulk copies per row (3 limb planes, 2 run-sum arrays), dealt to the
    // warps' first lanes and counted on one barrier; block scales and RMS factors by plain loads.
    bool ok = true;
    {
        const LimbImage L(M, a.w.K);
        const int Kf = a.w.K, Ks = nbs * 256;
        if (lane == 0) {
            uint32_t bytes = 0;
            for (int it = warp; it < 5 * M; it += kWarps) bytes += it % 5 < 3 ? Ks : (it % 5 == 3 ? Ks >> 3 : Ks >> 2);
            mbar_expect_tx(&x_bar, bytes);
            for (int it = warp; it < 5 * M; it += kWarps) {
                const int m = it / 5, p = it - 5 * m;
                if (p < 3) bulk_g2s(xl + static_cast<size_t>(3 * m + p) * plane_stride, a.img + L.planes + (static_cast<size_t>(3 * m + p) * Kf + kb0 * 256), Ks, &x_bar);
                else if (p == 3) bulk_g2s(asum + m * (K >> 5), a.img + L.asum + sizeof(float) * (static_cast<size_t>(m) * (Kf >> 5) + kb0 * 8), Ks >> 3, &x_bar);
                else bulk_g2s(asum16 + m * (K >> 4), a.img + L.asum16 + sizeof(float) * (static_cast<size_t>(m) * (Kf >> 4) + kb0 * 16), Ks >> 2, &x_bar);
            }
        }
        const float* gxs = reinterpret_cast<const float*>(a.img + L.xs);
        for (int i = threadIdx.x; i < M * nbs; i += kWarps * 32) { const int m = i / nbs, b = i - m * nbs; xs[m * (K >> 8) + b] = gxs[m * nb + kb0 + b]; }
        if (threadIdx.x < M) inv_s[threadIdx.x] = reinterpret_cast<const float*>(a.img + L.inv_s)[threadIdx.x];
        ok = mbar_wait(&x_bar, 0, a.err, 3);
    }
    consumer_sync();

    int st = 0;
    uint32_t ph = 0;
    float* my_slab = slab + static_cast<size_t>(warp) * NMAT * 16 * NC;
    for (int rg = team; rg < n_rg; rg += n_teams) {
        // column sums of this warp's share of the row group: [matrix][column group][row g: slots 0, 1 | row g + 8: slots 2, 3]
        float F[NMAT][CG][4], Fm[NMAT][2][MI];
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat) {
#pragma unroll
            for (int q = 0; q < CG; ++q)
#pragma unroll
                for (int i = 0; i < 4; ++i) F[mat][q][i] = 0.0f;
#pragma unroll
            for (int i = 0; i < MI; ++i) { Fm[mat][0][i] = 0.0f; Fm[mat][1][i] = 0.0f; }
        }
        for (int ti = member; ti < tprg; ti += a.ws) {
            const int s = warp * a.P + st;
            if (ok) ok = mbar_wait(&full_bar[s], ph, a.err, 2);
            if (++st == a.P) { st = 0; ph ^= 1; }
            if (!ok) continue;
            const int mat = ti >= spr, sl = ti - mat * spr;
            const int b0 = sl * a.sb, nbk = min(a.sb, nbs - b0);      // b, b0: block index inside the slice
            const uint8_t* qsT = ring + static_cast<size_t>(s) * a.stage_bytes;
            const uint8_t* s1T = qsT + a.sb * 2048;
            float f[CG][4];
#pragma unroll
            for (int q = 0; q < CG; ++q)
#pragma unroll
                for (int i = 0; i < 4; ++i) f[q][i] = 0.0f;
            float fmA[MI], fmB[MI];                      // min / offset terms: rows g, g + 8 x activation rows t + 4 i
#pragma unroll
            for (int i = 0; i < MI; ++i) { fmA[i] = 0.0f; fmB[i] = 0.0f; }
            if (!is_q6) {
                for (int bl = 0; bl < nbk; ++bl) {
                    const int b = b0 + bl;
                    const uint4 ha = *reinterpret_cast<const uint4*>(s1T + (bl * 16 + g) * 16);
                    const uint4 hb = *reinterpret_cast<const uint4*>(s1T + (bl * 16 + g + 8) * 16);
                    const uint32_t sa03 = ha.y & 0x3F3F3F3Fu, sa47 = (ha.w & 0x0F0F0F0Fu) | ((ha.y >> 2) & 0x30303030u);
                    const uint32_t sb03 = hb.y & 0x3F3F3F3Fu, sb47 = (hb.w & 0x0F0F0F0Fu) | ((hb.y >> 2) & 0x30303030u);
                    const float dA = __half2float(__ushort_as_half(static_cast<uint16_t>(ha.x & 0xFFFF)));
                    const float dB = __half2float(__ushort_as_half(static_cast<uint16_t>(hb.x & 0xFFFF)));
                    {   // min term of each (weight row, activation row): dmin * sum_sub m_sub * sum(x over sub)
                        const uint32_t ma03 = ha.z & 0x3F3F3F3Fu, ma47 = ((ha.w >> 4) & 0x0F0F0F0Fu) | ((ha.z >> 2) & 0x30303030u);
                        const uint32_t mb03 = hb.z & 0x3F3F3F3Fu, mb47 = ((hb.w >> 4) & 0x0F0F0F0Fu) | ((hb.z >> 2) & 0x30303030u);
                        const float dmA = __half2float(__ushort_as_half(static_cast<uint16_t>(ha.x >> 16)));
                        const float dmB = __half2float(__ushort_as_half(static_cast<uint16_t>(hb.x >> 16)));
                        float mAf[8], mBf[8];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            mAf[i] = dmA * static_cast<float>((ma03 >> (8 * i)) & 0xFFu); mAf[4 + i] = dmA * static_cast<float>((ma47 >> (8 * i)) & 0xFFu);
                            mBf[i] = dmB * static_cast<float>((mb03 >> (8 * i)) & 0xFFu); mBf[4 + i] = dmB * static_cast<float>((mb47 >> (8 * i)) & 0xFFu);
                        }
                        // lane (g, t) owns the terms of weight rows g, g + 8 and activation rows t, t + 4, ...: every lane does
                        // the same amount, nothing diverges; the sums join the limb-0 columns in the slab
#pragma unroll
                        for (int i = 0; i < MI; ++i) {
                            const int mm = t + 4 * i;
                            if (mm < M) {
                                const float* as = asum + mm * (K >> 5) + b * 8;
                                const float4 a0 = *reinterpret_cast<const float4*>(as), a1 = *reinterpret_cast<const float4*>(as + 4);
                                fmA[i] -= mAf[0] * a0.x + mAf[1] * a0.y + mAf[2] * a0.z + mAf[3] * a0.w + mAf[4] * a1.x + mAf[5] * a1.y + mAf[6] * a1.z + mAf[7] * a1.w;
                                fmB[i] -= mBf[0] * a0.x + mBf[1] * a0.y + mBf[2] * a0.z + mBf[3] * a0.w + mBf[4] * a1.x + mBf[5] * a1.y + mBf[6] * a1.z + mBf[7] * a1.w;
                            }
                        }
                    }
                    int lo[CG][4], hi[CG][4];
#pragma unroll
                    for (int q = 0; q < CG; ++q)
#pragma unroll
                        for (int i = 0; i < 4; ++i) { lo[q][i] = 0; hi[q][i] = 0; }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 qv = *reinterpret_cast<const uint4*>(qsT + (static_cast<size_t>(bl * 4 + j) * 32 + lane) * 16);
                        const uint32_t l0 = qv.x & 0x0F0F0F0Fu, l1 = qv.y & 0x0F0F0F0Fu, l2 = qv.z & 0x0F0F0F0Fu, l3 = qv.w & 0x0F0F0F0Fu;
                        const uint32_t h0 = qv.x & 0xF0F0F0F0u, h1 = qv.y & 0xF0F0F0F0u, h2 = qv.z & 0xF0F0F0F0u, h3 = qv.w & 0xF0F0F0F0u;
                        const uint32_t wa = j < 2 ? sa03 : sa47, wb = j < 2 ? sb03 : sb47;
                        const int sa0 = (wa >> (16 * (j & 1))) & 0xFF, sa1 = (wa >> (16 * (j & 1) + 8)) & 0xFF;
                        const int sb0 = (wb >> (16 * (j & 1))) & 0xFF, sb1 = (wb >> (16 * (j & 1) + 8)) & 0xFF;
#pragma unroll
                        for (int q = 0; q < CG; ++q) {
                            const int8_t* bp = bplane[q] + (b * 8 + 2 * j) * 32;
                            const uint32_t bl0 = *reinterpret_cast<const uint32_t*>(bp), bl1 = *reinterpret_cast<const uint32_t*>(bp + 16);
                            const uint32_t bh0 = *reinterpret_cast<const uint32_t*>(bp + 32), bh1 = *reinterpret_cast<const uint32_t*>(bp + 48);
                            int cl[4], ch[4];
                            mma_s8(cl, l0, l1, l2, l3, bl0, bl1);
                            mma_u8s8(ch, h0, h1, h2, h3, bh0, bh1);
                            lo[q][0] += sa0 * cl[0]; lo[q][1] += sa0 * cl[1]; lo[q][2] += sb0 * cl[2]; lo[q][3] += sb0 * cl[3];
                            hi[q][0] += sa1 * ch[0]; hi[q][1] += sa1 * ch[1]; hi[q][2] += sb1 * ch[2]; hi[q][3] += sb1 * ch[3];
                        }
                    }
#pragma unroll
                    for (int q = 0; q < CG; ++q) {
                        const float x0 = xs[mrow[q][0] * (K >> 8) + b] * lw[q][0], x1 = xs[mrow[q][1] * (K >> 8) + b] * lw[q][1];
                        f[q][0] = fmaf(static_cast<float>(lo[q][0]) + static_cast<float>(hi[q][0]) * 0.0625f, dA * x0, f[q][0]);
                        f[q][1] = fmaf(static_cast<float>(lo[q][1]) + static_cast<float>(hi[q][1]) * 0.0625f, dA * x1, f[q][1]);
                        f[q][2] = fmaf(static_cast<float>(lo[q][2]) + static_cast<float>(hi[q][2]) * 0.0625f, dB * x0, f[q][2]);
                        f[q][3] = fmaf(static_cast<float>(lo[q][3]) + static_cast<float>(hi[q][3]) * 0.0625f, dB * x1, f[q][3]);
                    }
                }
            } else {
                const uint8_t* s2T = s1T + a.sb * 1024;
                const uint8_t* s3T = s2T + a.sb * 256;
                for (int bl = 0; bl < nbk; ++bl) {
                    const int b = b0 + bl;
                    const uint4 sa = *reinterpret_cast<const uint4*>(s2T + (bl * 16 + g) * 16);
                    const uint4 sb_ = *reinterpret_cast<const uint4*>(s2T + (bl * 16 + g + 8) * 16);
                    const float dA = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(s3T + (bl * 16 + g) * 2)));
                    const float dB = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(s3T + (bl * 16 + g + 8) * 2)));
                    const uint32_t saw[4] = {sa.x, sa.y, sa.z, sa.w}, sbw[4] = {sb_.x, sb_.y, sb_.z, sb_.w};
                    // quants are used unsigned (0..63): 32 * d * sum_run sc_run * sum(x over run) comes off each (weight row,
                    // activation row); lane (g, t) owns rows g, g + 8 and activation rows t, t + 4, ... (see the Q4_K branch)
                    {
                        float scA[16], scB[16];
#pragma unroll
                        for (int w4 = 0; w4 < 4; ++w4)
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                scA[4 * w4 + k] = static_cast<float>(static_cast<int8_t>(saw[w4] >> (8 * k)));
                                scB[4 * w4 + k] = static_cast<float>(static_cast<int8_t>(sbw[w4] >> (8 * k)));
                            }
#pragma unroll
                        for (int i = 0; i < MI; ++i) {
                            const int mm = t + 4 * i;
                            if (mm < M) {
                                const float* as = asum16 + mm * (K >> 4) + b * 16;
                                float ca = 0.0f, cb = 0.0f;
#pragma unroll
                                for (int w4 = 0; w4 < 4; ++w4) {
                                    const float4 av = *reinterpret_cast<const float4*>(as + 4 * w4);
                                    ca += scA[4 * w4] * av.x + scA[4 * w4 + 1] * av.y + scA[4 * w4 + 2] * av.z + scA[4 * w4 + 3] * av.w;
                                    cb += scB[4 * w4] * av.x + scB[4 * w4 + 1] * av.y + scB[4 * w4 + 2] * av.z + scB[4 * w4 + 3] * av.w;
                                }
                                fmA[i] -= dA * 32.0f * ca;
                                fmB[i] -= dB * 32.0f * cb;
                            }
                        }
                    }
                    int c[CG][4];
#pragma unroll
                    for (int q = 0; q < CG; ++q)
#pragma unroll
                        for (int i = 0; i < 4; ++i) c[q][i] = 0;
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        const uint4 qh = *reinterpret_cast<const uint4*>(s1T + (static_cast<size_t>(bl * 2 + hf) * 32 + lane) * 16);
#pragma unroll
                        for (int cc2 = 0; cc2 < 2; ++cc2) {
                            const uint4 ql = *reinterpret_cast<const uint4*>(qsT + (static_cast<size_t>(bl * 4 + 2 * hf + cc2) * 32 + lane) * 16);
                            const uint32_t hA = cc2 ? qh.z : qh.x, hB = cc2 ? qh.w : qh.y;
                            const uint32_t kf = 0x0F0F0F0Fu, k3 = 0x30303030u;
                            const uint32_t ag[4] = {(ql.x & kf) | ((hA << 4) & k3), (ql.y & kf) | ((hA << 2) & k3), ((ql.x >> 4) & kf) | (hA & k3),
                                                    ((ql.y >> 4) & kf) | ((hA >> 2) & k3)};
                            const uint32_t ah[4] = {(ql.z & kf) | ((hB << 4) & k3), (ql.w & kf) | ((hB << 2) & k3), ((ql.z >> 4) & kf) | (hB & k3),
                                                    ((ql.w >> 4) & kf) | ((hB >> 2) & k3)};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int sidx = 8 * hf + 2 * i + cc2;
                                const int sca = static_cast<int8_t>(saw[sidx >> 2] >> (8 * (sidx & 3)));
                                const int scb = static_cast<int8_t>(sbw[sidx >> 2] >> (8 * (sidx & 3)));
#pragma unroll
                                for (int q = 0; q < CG; ++q) {
                                    const uint32_t bw = *reinterpret_cast<const uint32_t*>(bplane[q] + (b * 16 + sidx) * 16);
                                    int cc[4];
                                    mma_u8s8_k16(cc, ag[i], ah[i], bw);
                                    c[q][0] += sca * cc[0]; c[q][1] += sca * cc[1]; c[q][2] += scb * cc[2]; c[q][3] += scb * cc[3];
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int q = 0; q < CG; ++q) {
                        const float x0 = xs[mrow[q][0] * (K >> 8) + b] * lw[q][0], x1 = xs[mrow[q][1] * (K >> 8) + b] * lw[q][1];
                        f[q][0] = fmaf(static_cast<float>(c[q][0]), dA * x0, f[q][0]); f[q][1] = fmaf(static_cast<float>(c[q][1]), dA * x1, f[q][1]);
                        f[q][2] = fmaf(static_cast<float>(c[q][2]), dB * x0, f[q][2]); f[q][3] = fmaf(static_cast<float>(c[q][3]), dB * x1, f[q][3]);
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < CG; ++q)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (NMAT == 1 || mat == 0) F[0][q][i] += f[q][i]; else F[NMAT - 1][q][i] += f[q][i];
                }
#pragma unroll
            for (int i = 0; i < MI; ++i) {
                if (NMAT == 1 || mat == 0) { Fm[0][0][i] += fmA[i]; Fm[0][1][i] += fmB[i]; }
                else { Fm[NMAT - 1][0][i] += fmA[i]; Fm[NMAT - 1][1][i] += fmB[i]; }
            }
            __syncwarp();
            issue_next();                               // the stage is free again
        }
        // ---- column sums into this warp's slab: [matrix][row 0..15][column 0..NC) ----
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat) {
            {
#pragma unroll
                for (int q = 0; q < CG; ++q) {
                    float* r0 = my_slab + (static_cast<size_t>(mat) * 16 + g) * NC + 8 * q + 2 * t;
                    *reinterpret_cast<float2*>(r0) = make_float2(F[mat][q][0], F[mat][q][1]);
                    *reinterpret_cast<float2*>(r0 + 8 * NC) = make_float2(F[mat][q][2], F[mat][q][3]);
                }
            }
        }
        __syncwarp();
        // the min / offset terms join the limb-0 column (3 m) of their activation row: (row, m) pairs are unique per lane
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat)
#pragma unroll
            for (int i = 0; i < MI; ++i) {
                const int mm = t + 4 * i;
                if (mm < M) {
                    my_slab[(static_cast<size_t>(mat) * 16 + g) * NC + 3 * mm] += Fm[mat][0][i];
                    my_slab[(static_cast<size_t>(mat) * 16 + g + 8) * NC + 3 * mm] += Fm[mat][1][i];
                }
            }
        asm volatile("bar.sync %0, %1;" ::"r"(2 + team), "r"(a.ws * 32) : "memory");
        if (member == 0) {
            // the team's first warp: (row r, activation row m) = sum over the team's slabs of columns 3m, 3m+1, 3m+2
            for (int idx = lane; idx < 16 * M; idx += 32) {
                const int r = idx & 15, m = idx >> 4;
                float v = 0.0f, v2 = 0.0f;
                for (int j = 0; j < a.ws; ++j) {
                    const float* sj = slab + static_cast<size_t>(team * a.ws + j) * NMAT * 16 * NC + static_cast<size_t>(r) * NC + 3 * m;
                    v += sj[0] + sj[1] + sj[2];
                    if (NMAT == 2) { const float* s2 = sj + 16 * NC; v2 += s2[0] + s2[1] + s2[2]; }
                }
                v *= inv_s[m]; v2 *= inv_s[m];
                const int64_t row = (g_begin + rg) * 16 + r;
                if (row < a.w.N && a.part) {              // a slice of K: bare partial sums, the epilogue follows the reduction
                    const size_t plane = static_cast<size_t>(M) * a.w.N;
                    float* pz = a.part + static_cast<size_t>(blockIdx.y) * NMAT * plane + static_cast<size_t>(m) * a.w.N + row;
                    pz[0] = v;
                    if (NMAT == 2) pz[plane] = v2;
                } else if (row < a.w.N) {
                    const size_t o = static_cast<size_t>(m) * a.ldc + row;
                    if (NMAT == 2) v = (v / (1.0f + expf(-v))) * v2;
                    else if (a.epi == EPI_ADD_BIAS && a.bias) v += __ldg(a.bias + row);
                    else if (a.epi == EPI_RESIDUAL) v += a.resid[o];
                    a.y[o] = v;
                }
            }
        }
        // the slabs are reused by the next row group: wait until the first warp has read them
        asm volatile("bar.sync %0, %1;" ::"r"(2 + team), "r"(a.ws * 32) : "memory");
    }
}

// y = epilogue(sum over the K slices, in slice order, of the partial sums); one thread per output element.
__global__ void rows_reduce_kernel(const float* __restrict__ part, int slices, int nmat, int M, int64_t N, int epi,
                                   const float* __restrict__ bias, const float* resid, float* y, int ldc) {
    pdl_wait();
    pdl_launch();
    const size_t plane = static_cast<size_t>(M) * N;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < plane; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int m = static_cast<int>(i / N);
        const int64_t n = static_cast<int64_t>(i - static_cast<size_t>(m) * N);
        float v = 0.0f, v2 = 0.0f;
        for (int z = 0; z < slices; ++z) {
            const float* p = part + static_cast<size_t>(z) * nmat * plane;
            v += p[i];
            if (nmat == 2) v2 += p[plane + i];
        }
        const size_t o = static_cast<size_t>(m) * ldc + n;
        if (nmat == 2) v = (v / (1.0f + expf(-v))) * v2;
        else if (epi == EPI_ADD_BIAS && bias) v += __ldg(bias + n);
        else if (epi == EPI_RESIDUAL) v += resid[o];
        y[o] = v;
    }
}

// Shared memory of one CTA for mc rows over kbs blocks of K, without the ring.
size_t rows_fixed_bytes(int mc, int kbs, int nmat, int cg) {
    const int K = kbs * 256;
    return static_cast<size_t>(3 * mc) * (K + 16) + sizeof(float) * (mc * (K / 32 + K / 16) + ((mc * (K / 256) + 3) & ~3)) +
           sizeof(float) * kWarps * nmat * 16 * 8 * cg + 64;
}
constexpr size_t kRowsBudget = 216 * 1024;

// Slices of K: the fewest whose activation arrays leave room for a ring of three 1-block stages per warp.
int rows_slices(int nb, int mc, int nmat, int cg) {
    for (int S = 1; S <= nb; ++S) {
        const int kbs = (nb + S - 1) / S;
        if (rows_fixed_bytes(mc, kbs, nmat, cg) + static_cast<size_t>(kWarps) * 3 * 3360 <= kRowsBudget) return S;
    }
    return 0;
}

template <int CG>
int launch_rows_t(Context* c, const GemvArgs& g, float* d_part, size_t part_floats, void* d_limbs, size_t limbs_bytes, cudaStream_t s) {
    const int m0 = 0, mc = g.M;
    constexpr int kThreads = kWarps * 32;
    const int K = g.w.K, nb = g.w.nb;
    const bool dual = g.epi == EPI_SWIGLU;
    const bool q6 = g.w.type == T_Q6_K;
    const int nmat = dual ? 2 : 1;
    const int groups = static_cast<int>((g.w.N + 15) / 16);
    const int gb_bytes = q6 ? 3360 : 2304;
    const int S = rows_slices(nb, mc, nmat, CG);
    if (S < 1) return GGB_NOT_FOUND;
    const int kbs = (nb + S - 1) / S;
    const int slices = (nb + kbs - 1) / kbs;
    if (slices > 1 && static_cast<size_t>(slices) * nmat * mc * g.w.N > part_floats) return GGB_NOT_FOUND;
    if (LimbImage(mc, K).bytes > limbs_bytes || nb * sizeof(float) > 48 * 1024 || d_limbs != c->d_limbs) return GGB_NOT_FOUND;
    const int G = std::min(std::max(1, c->sm_count / slices), groups);
    const int gpc = (groups + G - 1) / G;
    int ws = 1;
    while (ws < kWarps && gpc * ws < kWarps) ws <<= 1;
    const size_t fixed = rows_fixed_bytes(mc, kbs, nmat, CG);
    const size_t budget = kRowsBudget;
    // tile depth 1..2 blocks, ring as deep as the rest of shared memory allows (at least two stages per warp)
    int sb = 2;
    while (sb > 1 && nmat * ((kbs + sb - 1) / sb) < ws) sb >>= 1;
    sb = std::min(sb, kbs);
    int spr, stage_bytes, P;
    for (;;) {
        spr = (kbs + sb - 1) / sb;
        stage_bytes = sb * gb_bytes;
        const int tiles_per_warp = ((gpc + kWarps / ws - 1) / (kWarps / ws)) * ((nmat * spr + ws - 1) / ws);
        P = std::min(kMaxStages / kWarps, std::max(2, tiles_per_warp));
        while (P > 2 && static_cast<size_t>(kWarps) * P * stage_bytes + fixed > budget) --P;
        if (static_cast<size_t>(kWarps) * P * stage_bytes + fixed <= budget || sb == 1) break;
        sb >>= 1;
    }
    const size_t smem = static_cast<size_t>(kWarps) * P * stage_bytes + fixed;
    if (smem > budget) return GGB_NOT_FOUND;

    RowsArgs a{};
    a.w = g.w; a.w2 = g.w2; a.x = g.x + static_cast<size_t>(m0) * g.lda; a.y = g.y + static_cast<size_t>(m0) * g.ldc;
    a.bias = g.bias; a.resid = g.resid ? g.resid + static_cast<size_t>(m0) * g.ldc : nullptr; a.gamma = g.gamma; a.eps = g.eps;
    a.M = mc; a.lda = g.lda; a.ldc = g.ldc; a.epi = g.epi;
    a.sb = sb; a.nmat = nmat; a.groups = groups; a.ws = ws; a.P = P; a.stage_bytes = stage_bytes;
    a.kbs = kbs; a.part = slices > 1 ? d_part : nullptr;
    a.img = static_cast<const uint8_t*>(d_limbs);
    a.err = c->d_err;
    {
        const int sp = limb_image_prepare(c, g, s);
        if (sp != GGB_OK) return sp;
    }
    void (*kern)(const RowsArgs) = dual ? gemv_mma_rows_kernel<CG, 2> : gemv_mma_rows_kernel<CG, 1>;
    cudaError_t e = ensure_dynamic_smem(c, kern, smem);
    if (e != cudaSuccess) return cuda_status(c, e, "gemv_mma_rows attr");
    e = launch_pdl(c, kern, dim3(static_cast<unsigned>(G), static_cast<unsigned>(slices)), dim3(kThreads), smem, s, a);
    c->launches++;
    if (e != cudaSuccess || slices == 1) return cuda_status(c, e, "gemv_mma_rows launch");
    const size_t elems = static_cast<size_t>(mc) * g.w.N;
    e = launch_pdl(c, rows_reduce_kernel, dim3(static_cast<unsigned>(std::min<size_t>((elems + 255) / 256, 148 * 8))), dim3(256), 0, s,
                   static_cast<const float*>(d_part), slices, nmat, mc, g.w.N, g.epi, g.bias, g.resid, g.y, g.ldc);
    c->launches++;
    return cuda_status(c, e, "gemv_mma_rows reduce");
}

// ---- stream-layout formats (Q8_0, Q4_0, IQ4_NL) on the tensor cores ------------------------------------------------
// The weights stay in the stream layout ([row][32-block]: quants and fp16 scales in two streams).  A tile is 16 weight rows
// x one 256-run of K, brought by one bulk copy per row and stream into rows PADDED by 16 bytes, so that ldmatrix reads eight
// rows without a bank conflict; ldmatrix delivers exactly the int8 A fragment of mma.m16n8k32 (Q8_0: the 32 bytes of a
// block = four 8 x 16-byte matrices; Q4_0 / IQ4_NL: the 16 bytes hold elements 0..15 in the low and 16..31 in the high
// nibbles, which are the two K halves of the fragment).  Everything else is the K-quant kernel above: limb image of the
// activations, column c = 3 m + p, slabs, K slices.  The block scale d is applied to the int32 sums per 32-block.
// IQ4_XS (256-blocks: an 8-byte header d | scales_h | scales_l[4], then eight 16-byte sub-blocks) runs the same path: the
// scale of sub-block kb is d * (ls_kb - 32); a tile brings the aligned 16-byte pair of headers that holds its block's.
enum : int { SF_Q80 = 0, SF_Q40 = 1, SF_IQ4NL = 2, SF_IQ4XS = 3 };

__device__ __forceinline__ uint32_t iq4_codes_u(uint32_t idx) {      // four codebook indices (one per byte) -> four int8 codes (src/quant/iq4_nl.cpp:16-18)
    const uint32_t x = idx | (idx >> 4);
    const uint32_t p = __byte_perm(x, 0u, 0x4420);
    const uint32_t sel = p & 0x7777u;
    const uint32_t lo = __byte_perm(0xBFAD9881u, 0xF6EADDCFu, sel);
    const uint32_t hi = __byte_perm(0x26190D01u, 0x71594535u, sel);
    return __byte_perm(lo, hi, 0x3210u | ((p & 0x8888u) >> 1));
}

template <int SF> struct StreamGeom {
    static constexpr int QB = SF == SF_Q80 ? 32 : 16;      // quant bytes per 32-block
    static constexpr int QROW = 8 * QB + 16;               // padded bytes of one row's 256-run in a stage
    static constexpr int STAGE = 16 * QROW + 256;          // + 16 rows x 8 fp16 scales
    static constexpr int TX = 16 * (8 * QB + 16);          // bytes a tile's copies deliver
};

// INLINE_X (one or two rows, K not cut): the CTA converts the activations itself in its prologue instead of copying the
// image -- a decode step cannot afford a second launch per matrix.
template <int SF, int CG, int NMAT, bool INLINE_X>
__global__ void __launch_bounds__(kWarps * 32, 1) gemv_mma_stream_kernel(const RowsArgs a) {
    using G = StreamGeom<SF>;
    constexpr int NC = 8 * CG;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages], x_bar;
    __shared__ float inv_s[16];
    __shared__ float ssb[2][64];                        // INLINE_X: sums of squares per (row, 256-run)
    const int nb = a.w.K >> 8, nb32 = a.w.K >> 5, M = a.M;        // 256-runs and 32-blocks per row
    const int kb0 = blockIdx.y * a.kbs, nbs = min(a.kbs, nb - kb0);
    const int K = a.kbs * 256;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tprg = NMAT * nbs;                        // tiles per row group: one per 256-run and matrix
    const int plane_stride = K + 16;
    uint8_t* ring = smem;
    int8_t* xl = reinterpret_cast<int8_t*>(ring + static_cast<size_t>(kWarps) * a.P * G::STAGE);
    float* xs = reinterpret_cast<float*>(xl + static_cast<size_t>(3 * M) * plane_stride);
    float* slab = xs + ((M * (K >> 8) + 3) & ~3);

    const int64_t g_begin = static_cast<int64_t>(blockIdx.x) * a.groups / gridDim.x;
    const int n_rg = static_cast<int>(static_cast<int64_t>(blockIdx.x + 1) * a.groups / gridDim.x - g_begin);
    const int n_teams = kWarps / a.ws;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWarps * a.P; ++s) mbar_init(&full_bar[s], 1);
        mbar_init(&x_bar, kWarps);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch();

    const int team = warp / a.ws, member = warp % a.ws;
    int rg_i = team, ti_i = member, st_i = 0;
    // stacked matrices: which matrix a row group of the stacked numbering belongs to, and its first group
    auto cat_of = [&](int64_t gi, int& first) -> int {
        int j = 0; first = 0;
        if (a.ncat > 0 && gi >= a.cat_g0[0]) { j = 1; first = a.cat_g0[0]; }
        if (a.ncat > 1 && gi >= a.cat_g0[1]) { j = 2; first = a.cat_g0[1]; }
        return j;
    };
    // the whole warp issues a tile: lane r < 16 copies row r's quants, lane 16 + r its scales
    auto issue_next = [&]() {
        while (rg_i < n_rg && ti_i >= tprg) { rg_i += n_teams; ti_i = member; }
        if (rg_i >= n_rg) return;
        const int s = warp * a.P + st_i;
        const int mat = ti_i >= nbs, bl = ti_i - mat * nbs;
        uint8_t* dst = ring + static_cast<size_t>(s) * G::STAGE;
        int gfirst;
        const int cj = cat_of(g_begin + rg_i, gfirst);
        const PackedW& w = mat ? a.w2 : (cj == 0 ? a.w : a.cat_w[cj - 1]);
        const int r = lane & 15;
        const int64_t lrow = (g_begin + rg_i - gfirst) * 16 + r;          // row inside its matrix
        const int64_t blk = lrow * nb32 + static_cast<int64_t>(kb0 + bl) * 8;      // first 32-block of the row's run
        // IQ4_XS: the row's 256-block headers are 8 bytes each; the aligned pair that contains this block's
        const int64_t hdr = (lrow * nb + ((kb0 + bl) & ~1)) * 8;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the stage was last read through the generic proxy
        if (lane == 0) mbar_expect_tx(&full_bar[s], G::TX);
        __syncwarp();
        if (lane < 16) bulk_g2s(dst + r * G::QROW, w.s[1] + blk * G::QB, 8 * G::QB, &full_bar[s]);
        else bulk_g2s(dst + 16 * G::QROW + r * 16, w.s[0] + (SF == SF_IQ4XS ? hdr : blk * 2), 16, &full_bar[s]);
        ti_i += a.ws;
        if (++st_i == a.P) st_i = 0;
    };
    for (int i = 0; i < a.P; ++i) issue_next();

    const int g = lane >> 2, t = lane & 3;
    const int ncol = 3 * M;
    const int8_t* bplane[CG];
    int mrow[CG][2];
    float lw[CG][2];
#pragma unroll
    for (int q = 0; q < CG; ++q) {
        bplane[q] = xl + static_cast<size_t>(min(8 * q + g, ncol - 1)) * plane_stride + 4 * t;
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
            const int col = 8 * q + 2 * t + sl;
            const bool valid = col < ncol;
            mrow[q][sl] = valid ? col / 3 : M - 1;
            const int p = col % 3;
            lw[q][sl] = valid ? (p == 0 ? 1.0f : (p == 1 ? 1.0f / 128.0f : 1.0f / 16384.0f)) : 0.0f;
        }
    }
    pdl_wait();
    bool ok = true;
    if (INLINE_X) {
        // one or two rows, the whole K: limbs of x * gamma and block scales straight into shared memory (as rows_prep_kernel)
        // a warp's 256-runs are converted four at a time, their loads issued together: one run per trip pays the
        // memory latency once per run, which at K = 8192 was a third of the kernel
        constexpr int XB = 4;
        for (int m = 0; m < M; ++m)
            for (int b0 = warp; b0 < nb; b0 += kWarps * XB) {
                float4 xp[XB][2], gp[XB][2];
#pragma unroll
                for (int u = 0; u < XB; ++u) {
                    const int b = b0 + u * kWarps;
                    if (b >= nb) continue;
                    const int k0 = b * 256 + lane * 8;
                    const float* xr = a.x + static_cast<size_t>(m) * a.lda + k0;
                    xp[u][0] = __ldg(reinterpret_cast<const float4*>(xr)); xp[u][1] = __ldg(reinterpret_cast<const float4*>(xr + 4));
                    if (a.gamma) { gp[u][0] = __ldg(reinterpret_cast<const float4*>(a.gamma + k0)); gp[u][1] = __ldg(reinterpret_cast<const float4*>(a.gamma + k0 + 4)); }
                }
#pragma unroll
                for (int u = 0; u < XB; ++u) {
                    const int b = b0 + u * kWarps;
                    if (b >= nb) continue;
                    const int k0 = b * 256 + lane * 8;
                    const float4 p0 = xp[u][0], p1 = xp[u][1];
                    float v[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
                    if (a.gamma) {
                        float ss = 0.0f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
                        ss = wsum(ss);
                        if (lane == 0) ssb[m][b] = ss;
                        const float4 g0 = gp[u][0], g1 = gp[u][1];
                        v[0] *= g0.x; v[1] *= g0.y; v[2] *= g0.z; v[3] *= g0.w; v[4] *= g1.x; v[5] *= g1.y; v[6] *= g1.z; v[7] *= g1.w;
                    }
                    float am = 0.0f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) am = fmaxf(am, fabsf(v[i]));
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, o));
                    const float rs = am > 0.0f ? 127.0f / am : 0.0f;
                    uint32_t w1[2] = {0, 0}, w2[2] = {0, 0}, w3[2] = {0, 0};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float kMagic = 12582912.0f;
                        const float r = fminf(fmaxf(v[i] * rs, -127.0f), 127.0f);
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
                    if (lane == 0) xs[m * (K >> 8) + b] = am / 127.0f;
                }
            }
        consumer_sync();
        if (threadIdx.x < M) {
            float tot = 0.0f;
            if (a.gamma) for (int b = 0; b < nb; ++b) tot += ssb[threadIdx.x][b];
            inv_s[threadIdx.x] = a.gamma ? 1.0f / sqrtf(tot / static_cast<float>(a.w.K) + a.eps) : 1.0f;
        }
    } else {
        const LimbImage L(M, a.w.K);
        const int Kf = a.w.K, Ks = nbs * 256;
        if (lane == 0) {
            uint32_t bytes = 0;
            for (int it = warp; it < 3 * M; it += kWarps) bytes += Ks;
            mbar_expect_tx(&x_bar, bytes);
            for (int it = warp; it < 3 * M; it += kWarps)
                bulk_g2s(xl + static_cast<size_t>(it) * plane_stride, a.img + L.planes + (static_cast<size_t>(it) * Kf + kb0 * 256), Ks, &x_bar);
        }
        const float* gxs = reinterpret_cast<const float*>(a.img + L.xs);
        for (int i = threadIdx.x; i < M * nbs; i += kWarps * 32) { const int m = i / nbs, b = i - m * nbs; xs[m * (K >> 8) + b] = gxs[m * nb + kb0 + b]; }
        if (threadIdx.x < M) inv_s[threadIdx.x] = reinterpret_cast<const float*>(a.img + L.inv_s)[threadIdx.x];
        ok = mbar_wait(&x_bar, 0, a.err, 3);
    }
    consumer_sync();

    // ldmatrix row address of this lane inside a stage: matrix lane / 8 -> rows (0..7 | 8..15), K half (bytes 0..15 | 16..31)
    const int lm_row = (lane & 7) + 8 * ((lane >> 3) & 1);
    const int lm_off = lm_row * G::QROW + (SF == SF_Q80 ? 16 * (lane >> 4) : 0);

    int st = 0;
    uint32_t ph = 0;
    float* my_slab = slab + static_cast<size_t>(warp) * NMAT * 16 * NC;
    for (int rg = team; rg < n_rg; rg += n_teams) {
        float F[NMAT][CG][4];
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat)
#pragma unroll
            for (int q = 0; q < CG; ++q)
#pragma unroll
                for (int i = 0; i < 4; ++i) F[mat][q][i] = 0.0f;
        for (int ti = member; ti < tprg; ti += a.ws) {
            const int s = warp * a.P + st;
            if (ok) ok = mbar_wait(&full_bar[s], ph, a.err, 2);
            if (++st == a.P) { st = 0; ph ^= 1; }
            if (!ok) continue;
            const int mat = ti >= nbs, b = ti - mat * nbs;           // b: 256-run inside the slice
            const uint8_t* qsT = ring + static_cast<size_t>(s) * G::STAGE;
            const uint4 dAv = *reinterpret_cast<const uint4*>(qsT + 16 * G::QROW + g * 16);            // the 8 block scales of rows g, g + 8
            const uint4 dBv = *reinterpret_cast<const uint4*>(qsT + 16 * G::QROW + (g + 8) * 16);
            const uint32_t dAw[4] = {dAv.x, dAv.y, dAv.z, dAv.w}, dBw[4] = {dBv.x, dBv.y, dBv.z, dBv.w};
            // IQ4_XS: this block's header is the first or second half of the pair
            const int hsel = 2 * ((kb0 + b) & 1);
            const uint32_t hAx = dAw[hsel], hAy = dAw[hsel + 1], hBx = dBw[hsel], hBy = dBw[hsel + 1];
            const float dA0 = __half2float(__ushort_as_half(static_cast<uint16_t>(hAx & 0xFFFFu))), dB0 = __half2float(__ushort_as_half(static_cast<uint16_t>(hBx & 0xFFFFu)));
            float f[CG][4];
#pragma unroll
            for (int q = 0; q < CG; ++q)
#pragma unroll
                for (int i = 0; i < 4; ++i) f[q][i] = 0.0f;
#pragma unroll
            for (int kb = 0; kb < 8; ++kb) {
                uint32_t a0, a1, a2, a3;
                const uint32_t addr = smem_u32(qsT + lm_off + kb * G::QB);
                if (SF == SF_Q80) {
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(addr));
                } else {
                    uint32_t w0, w1;
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(w0), "=r"(w1) : "r"(addr));
                    if (SF == SF_Q40) {
                        a0 = __vsub4(w0 & 0x0F0F0F0Fu, 0x08080808u); a1 = __vsub4(w1 & 0x0F0F0F0Fu, 0x08080808u);
                        a2 = __vsub4((w0 >> 4) & 0x0F0F0F0Fu, 0x08080808u); a3 = __vsub4((w1 >> 4) & 0x0F0F0F0Fu, 0x08080808u);
                    } else {
                        a0 = iq4_codes_u(w0 & 0x0F0F0F0Fu); a1 = iq4_codes_u(w1 & 0x0F0F0F0Fu);
                        a2 = iq4_codes_u((w0 >> 4) & 0x0F0F0F0Fu); a3 = iq4_codes_u((w1 >> 4) & 0x0F0F0F0Fu);
                    }
                }
                float dA, dB;
                if (SF == SF_IQ4XS) {
                    const int lsA = static_cast<int>(((hAy >> (4 * kb)) & 15u) | (((hAx >> (16 + 2 * kb)) & 3u) << 4));
                    const int lsB = static_cast<int>(((hBy >> (4 * kb)) & 15u) | (((hBx >> (16 + 2 * kb)) & 3u) << 4));
                    dA = dA0 * static_cast<float>(lsA - 32); dB = dB0 * static_cast<float>(lsB - 32);
                } else {
                    dA = __half2float(__ushort_as_half(static_cast<uint16_t>(dAw[kb >> 1] >> (16 * (kb & 1)))));
                    dB = __half2float(__ushort_as_half(static_cast<uint16_t>(dBw[kb >> 1] >> (16 * (kb & 1)))));
                }
#pragma unroll
                for (int q = 0; q < CG; ++q) {
                    const int8_t* bp = bplane[q] + (b * 8 + kb) * 32;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(bp), b1 = *reinterpret_cast<const uint32_t*>(bp + 16);
                    int c[4];
                    mma_s8(c, a0, a1, a2, a3, b0, b1);
                    f[q][0] = fmaf(static_cast<float>(c[0]), dA, f[q][0]); f[q][1] = fmaf(static_cast<float>(c[1]), dA, f[q][1]);
                    f[q][2] = fmaf(static_cast<float>(c[2]), dB, f[q][2]); f[q][3] = fmaf(static_cast<float>(c[3]), dB, f[q][3]);
                }
            }
#pragma unroll
            for (int q = 0; q < CG; ++q) {
                // the activations' block scale (one per 256-run = per tile) and limb weight of the lane's two columns
                const float x0 = xs[mrow[q][0] * (K >> 8) + b] * lw[q][0], x1 = xs[mrow[q][1] * (K >> 8) + b] * lw[q][1];
                if (NMAT == 1 || mat == 0) { F[0][q][0] += f[q][0] * x0; F[0][q][1] += f[q][1] * x1; F[0][q][2] += f[q][2] * x0; F[0][q][3] += f[q][3] * x1; }
                else { F[NMAT - 1][q][0] += f[q][0] * x0; F[NMAT - 1][q][1] += f[q][1] * x1; F[NMAT - 1][q][2] += f[q][2] * x0; F[NMAT - 1][q][3] += f[q][3] * x1; }
            }
            __syncwarp();
            issue_next();
        }
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat)
#pragma unroll
            for (int q = 0; q < CG; ++q) {
                float* r0 = my_slab + (static_cast<size_t>(mat) * 16 + g) * NC + 8 * q + 2 * t;
                *reinterpret_cast<float2*>(r0) = make_float2(F[mat][q][0], F[mat][q][1]);
                *reinterpret_cast<float2*>(r0 + 8 * NC) = make_float2(F[mat][q][2], F[mat][q][3]);
            }
        asm volatile("bar.sync %0, %1;" ::"r"(2 + team), "r"(a.ws * 32) : "memory");
        if (member == 0) {
            for (int idx = lane; idx < 16 * M; idx += 32) {
                const int r = idx & 15, m = idx >> 4;
                float v = 0.0f, v2 = 0.0f;
                for (int j = 0; j < a.ws; ++j) {
                    const float* sj = slab + static_cast<size_t>(team * a.ws + j) * NMAT * 16 * NC + static_cast<size_t>(r) * NC + 3 * m;
                    v += sj[0] + sj[1] + sj[2];
                    if (NMAT == 2) { const float* s2 = sj + 16 * NC; v2 += s2[0] + s2[1] + s2[2]; }
                }
                v *= inv_s[m]; v2 *= inv_s[m];
                int gfirst;
                const int cj = cat_of(g_begin + rg, gfirst);
                const int64_t row = (g_begin + rg - gfirst) * 16 + r;        // row inside its matrix
                const int64_t Nj = cj == 0 ? a.w.N : a.cat_w[cj - 1].N;
                float* yj = cj == 0 ? a.y : a.cat_y[cj - 1];
                const float* bj = cj == 0 ? a.bias : a.cat_bias[cj - 1];
                const int ldj = cj == 0 ? a.ldc : a.cat_ldc[cj - 1];
                if (row < Nj && a.part) {
                    const size_t plane = static_cast<size_t>(M) * a.w.N;
                    float* pz = a.part + static_cast<size_t>(blockIdx.y) * NMAT * plane + static_cast<size_t>(m) * a.w.N + row;
                    pz[0] = v;
                    if (NMAT == 2) pz[plane] = v2;
                } else if (row < Nj) {
                    const size_t o = static_cast<size_t>(m) * ldj + row;
                    if (NMAT == 2) v = (v / (1.0f + expf(-v))) * v2;
                    else if (a.epi == EPI_ADD_BIAS && bj) v += __ldg(bj + row);
                    else if (a.epi == EPI_RESIDUAL) v += a.resid[o];
                    yj[o] = v;
                }
            }
        }
        asm volatile("bar.sync %0, %1;" ::"r"(2 + team), "r"(a.ws * 32) : "memory");
    }
}

template <int SF, int CG>
int launch_stream_t(Context* c, const GemvArgs& g, float* d_part, size_t part_floats, cudaStream_t s) {
    using G = StreamGeom<SF>;
    constexpr int kThreads = kWarps * 32;
    const int K = g.w.K, nb = K >> 8, mc = g.M;
    const bool dual = g.epi == EPI_SWIGLU;
    const int nmat = dual ? 2 : 1;
    int groups = static_cast<int>(g.w.N / 16);
    int cat_g0[2] = {0, 0};
    for (int i = 0; i < g.n_cat; ++i) { cat_g0[i] = groups; groups += static_cast<int>(g.cat_w[i].N / 16); }
    const bool inline_x = mc <= 2;                      // decode steps: no second launch for the activations
    // K slices: activation arrays (planes, scales, slabs) beside a ring of at least two stages per warp
    auto fixed_bytes = [&](int kbs) {
        return static_cast<size_t>(3 * mc) * (kbs * 256 + 16) + sizeof(float) * ((mc * kbs + 3) & ~3) + sizeof(float) * kWarps * nmat * 16 * 8 * CG + 64;
    };
    int S = 0;
    for (int cand = 1; cand <= nb; ++cand) {
        const int kbs = (nb + cand - 1) / cand;
        if (fixed_bytes(kbs) + static_cast<size_t>(kWarps) * 2 * G::STAGE <= kRowsBudget) { S = cand; break; }
    }
    if (S < 1) return GGB_NOT_FOUND;
    const int kbs = (nb + S - 1) / S, slices = (nb + kbs - 1) / kbs;
    if (slices > 1 && (g.n_cat || inline_x)) return GGB_NOT_FOUND;
    if (slices > 1 && static_cast<size_t>(slices) * nmat * mc * g.w.N > part_floats) return GGB_NOT_FOUND;
    if (inline_x && nb > 64) return GGB_NOT_FOUND;
    if (!inline_x && (LimbImage(mc, K).bytes > c->d_limbs_bytes || nb * sizeof(float) > 48 * 1024)) return GGB_NOT_FOUND;
    const int Gx = std::min(std::max(1, c->sm_count / slices), groups);
    const int gpc = (groups + Gx - 1) / Gx;
    int ws = 1;
    while (ws < kWarps && gpc * ws < kWarps) ws <<= 1;
    const size_t fixed = fixed_bytes(kbs);
    const int tiles_per_warp = ((gpc + kWarps / ws - 1) / (kWarps / ws)) * ((nmat * kbs + ws - 1) / ws);
    int P = std::min(kMaxStages / kWarps, std::max(2, tiles_per_warp));
    while (P > 2 && static_cast<size_t>(kWarps) * P * G::STAGE + fixed > kRowsBudget) --P;
    const size_t smem = static_cast<size_t>(kWarps) * P * G::STAGE + fixed;
    if (smem > kRowsBudget) return GGB_NOT_FOUND;
    if (!inline_x) {
        const int sp = limb_image_prepare(c, g, s);
        if (sp != GGB_OK) return sp;
    }
    RowsArgs a{};
    a.w = g.w; a.w2 = g.w2; a.x = g.x; a.y = g.y; a.bias = g.bias; a.resid = g.resid; a.gamma = g.gamma; a.eps = g.eps;
    a.M = mc; a.lda = g.lda; a.ldc = g.ldc; a.epi = g.epi;
    a.sb = 1; a.nmat = nmat; a.groups = groups; a.ws = ws; a.P = P; a.stage_bytes = G::STAGE;
    a.kbs = kbs; a.part = slices > 1 ? d_part : nullptr;
    a.img = static_cast<const uint8_t*>(c->d_limbs);
    a.err = c->d_err;
    a.ncat = g.n_cat;
    for (int i = 0; i < g.n_cat; ++i) { a.cat_g0[i] = cat_g0[i]; a.cat_w[i] = g.cat_w[i]; a.cat_y[i] = g.cat_y[i]; a.cat_bias[i] = g.cat_bias[i]; a.cat_ldc[i] = g.cat_ldc[i]; }
    void (*kern)(const RowsArgs);
    if constexpr (CG == 1) kern = dual ? gemv_mma_stream_kernel<SF, 1, 2, true> : gemv_mma_stream_kernel<SF, 1, 1, true>;
    else kern = dual ? gemv_mma_stream_kernel<SF, CG, 2, false> : gemv_mma_stream_kernel<SF, CG, 1, false>;
    cudaError_t e = ensure_dynamic_smem(c, kern, smem);
    if (e != cudaSuccess) return cuda_status(c, e, "gemv_mma_stream attr");
    e = launch_pdl(c, kern, dim3(static_cast<unsigned>(Gx), static_cast<unsigned>(slices)), dim3(kThreads), smem, s, a);
    c->launches++;
    if (e != cudaSuccess || slices == 1) return cuda_status(c, e, "gemv_mma_stream launch");
    const size_t elems = static_cast<size_t>(mc) * g.w.N;
    e = launch_pdl(c, rows_reduce_kernel, dim3(static_cast<unsigned>(std::min<size_t>((elems + 255) / 256, 148 * 8))), dim3(256), 0, s,
                   static_cast<const float*>(d_part), slices, nmat, mc, g.w.N, g.epi, g.bias, g.resid, g.y, g.ldc);
    c->launches++;
    return cuda_status(c, e, "gemv_mma_stream reduce");
}

template <int SF>
int launch_stream_f(Context* c, const GemvArgs& g, float* d_part, size_t part_floats, cudaStream_t s) {
    if (g.M <= 2) return launch_stream_t<SF, 1>(c, g, d_part, part_floats, s);
    if (g.M <= 5) return launch_stream_t<SF, 2>(c, g, d_part, part_floats, s);
    if (g.M <= 8) return launch_stream_t<SF, 3>(c, g, d_part, part_floats, s);
    return launch_stream_t<SF, 6>(c, g, d_part, part_floats, s);
}

}  // namespace

static int rows_cg(int M) { return M <= 5 ? 2 : (M <= 8 ? 3 : 6); }

static bool rows_covered(const GemvArgs& g) {
    if ((g.w.type != T_Q4_K && g.w.type != T_Q6_K) || g.w.layout != 1 || g.M < 3 || g.M > 16 || g.w.K % 256) return false;
    if ((reinterpret_cast<uintptr_t>(g.x) & 15) || (g.lda & 3)) return false;
    const bool dual = g.epi == EPI_SWIGLU;
    if (dual && (g.w2.layout != 1 || g.w2.type != g.w.type)) return false;
    if (g.n_cat || g.attn_partial || g.sel || g.xscale || g.x_img || g.y_img) return false;
    return true;
}

// Floats of workspace launch_gemv_mma_rows needs for g (0: K is not cut, or the shape is not covered).
size_t gemv_mma_rows_ws_floats(const GemvArgs& g) {
    if (!rows_covered(g)) return 0;
    const int nmat = g.epi == EPI_SWIGLU ? 2 : 1;
    const int S = rows_slices(g.w.nb, g.M, nmat, rows_cg(g.M));
    if (S <= 1) return 0;
    const int kbs = (g.w.nb + S - 1) / S, slices = (g.w.nb + kbs - 1) / kbs;
    return static_cast<size_t>(slices) * nmat * g.M * g.w.N;
}

// 3 <= M <= 16 rows of a Q4_K / Q6_K matrix in the row-group-major layout in one pass over the weights.
// d_part: workspace of at least gemv_mma_rows_ws_floats(g) floats.  GGB_NOT_FOUND: shape not covered (the caller falls
// back to two rows per pass).
int launch_gemv_mma_rows(Context* c, const GemvArgs& g, float* d_part, size_t part_floats, void* d_limbs, size_t limbs_bytes, cudaStream_t s) {
    if (!rows_covered(g)) return GGB_NOT_FOUND;
    switch (rows_cg(g.M)) {
    case 2: return launch_rows_t<2>(c, g, d_part, part_floats, d_limbs, limbs_bytes, s);
    case 3: return launch_rows_t<3>(c, g, d_part, part_floats, d_limbs, limbs_bytes, s);
    default: return launch_rows_t<6>(c, g, d_part, part_floats, d_limbs, limbs_bytes, s);
    }
}

size_t gemv_mma_rows_limbs_bytes(int M, int K) { return LimbImage(M, K).bytes; }

static bool stream_covered(const GemvArgs& g) {
    if (g.w.layout != 0 || (g.w.type != T_Q8_0 && g.w.type != T_Q4_0 && g.w.type != T_IQ4_NL && g.w.type != T_IQ4_XS)) return false;
    if (g.w.type == T_IQ4_XS && (g.w.K % 512)) return false;       // block headers are fetched as aligned 16-byte pairs
    if (g.M < 1 || g.M > 16 || g.w.K % 256 || g.w.N % 16 || !g.x || (reinterpret_cast<uintptr_t>(g.x) & 15) || (g.lda & 3)) return false;
    const bool dual = g.epi == EPI_SWIGLU;
    if (dual && (g.w2.layout != 0 || g.w2.type != g.w.type)) return false;
    if (g.attn_partial || g.sel || g.xscale || g.x_img || g.y_img) return false;
    if (g.n_cat && (dual || g.n_cat > 2 || g.M > 2 || (g.epi != EPI_STORE && g.epi != EPI_ADD_BIAS))) return false;
    for (int i = 0; i < g.n_cat; ++i)
        if (g.cat_w[i].type != g.w.type || g.cat_w[i].K != g.w.K || g.cat_w[i].layout != 0 || g.cat_w[i].N % 16 || !g.cat_y[i]) return false;
    return true;
}

// Workspace floats (K slices) of launch_gemv_mma_stream: an upper bound, one slice per 256-run.
size_t gemv_mma_stream_ws_floats(const GemvArgs& g) {
    if (!stream_covered(g)) return 0;
    return static_cast<size_t>(g.w.K >> 8) * (g.epi == EPI_SWIGLU ? 2 : 1) * g.M * g.w.N > (size_t(64) << 20) ? 0
           : static_cast<size_t>(g.w.K >> 8) * (g.epi == EPI_SWIGLU ? 2 : 1) * g.M * g.w.N;
}

// 1 <= M <= 16 rows of a Q8_0 / Q4_0 / IQ4_NL / IQ4_XS matrix (stream layout; at M <= 2 also q | k | v stacked) on the int8 tensor cores, one pass over the weights.
// c->d_limbs holds room for the activation image (the caller grew it).  GGB_NOT_FOUND: not covered.
int launch_gemv_mma_stream(Context* c, const GemvArgs& g, float* d_part, size_t part_floats, cudaStream_t s) {
    if (!stream_covered(g)) return GGB_NOT_FOUND;
    switch (g.w.type) {
    case T_Q8_0: return launch_stream_f<SF_Q80>(c, g, d_part, part_floats, s);
    case T_Q4_0: return launch_stream_f<SF_Q40>(c, g, d_part, part_floats, s);
    case T_IQ4_XS: return launch_stream_f<SF_IQ4XS>(c, g, d_part, part_floats, s);
    default: return launch_stream_f<SF_IQ4NL>(c, g, d_part, part_floats, s);
    }
}

int limb_image_prepare(Context* c, const GemvArgs& g, cudaStream_t s) {
    const int M = g.M, K = g.w.K, nb = K >> 8;
    if (LimbImage(M, K).bytes > c->d_limbs_bytes || nb * sizeof(float) > 48 * 1024) return set_status(c, GGB_ERROR, "activation image: workspace too small");
    const bool reuse = g.limbs_reuse && c->limbs_x == g.x && c->limbs_gamma == g.gamma && c->limbs_M == M && c->limbs_K == K &&
                       c->limbs_lda == g.lda && c->limbs_eps == g.eps && c->limbs_call + 1 == c->gemv_calls;
    c->limbs_x = g.x; c->limbs_gamma = g.gamma; c->limbs_M = M; c->limbs_K = K; c->limbs_lda = g.lda; c->limbs_eps = g.eps;
    c->limbs_call = c->gemv_calls;
    if (reuse) return GGB_OK;
    const cudaError_t e = launch_pdl(c, rows_prep_kernel, dim3(static_cast<unsigned>(M)), dim3(256), nb * sizeof(float), s,
                                     static_cast<const float*>(g.x), g.lda, M, K, g.gamma, g.eps, static_cast<uint8_t*>(c->d_limbs));
    c->launches++;
    return cuda_status(c, e, "activation image");
}

}  // namespace ggb
