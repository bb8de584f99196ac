// Decode GEMV, M == 1: y[N] = W[N][K] x[K], the kernel the batch-1 token loop spends its time in
// (mul_mat_weight M==1, src/cli/main.cpp:1379-1388; logits, src/cli/main.cpp:270-327).
//
// HBM-bound by design: every weight byte crosses HBM once, nothing else of size does.
//   * One persistent CTA per SM.  A producer thread streams this CTA's row tiles (contiguous byte
//     ranges of each packed stream) into a shared-memory ring with bulk async copies
//     (cp.async.bulk global->shared, completion counted on an mbarrier).  The ring, not the register
//     file, holds the bytes in flight, so HBM stays busy whatever the consumers are doing.
//   * Weights do not depend on the previous kernel, activations do.  The kernel is launched with
//     programmatic dependent launch: the producer starts copying at once, the consumers execute
//     griddepcontrol.wait before they touch x.  The weight stream therefore runs across the kernel
//     boundary, which is what keeps a token loop made of ~0.5-3 us GEMVs near the HBM roofline.
//   * Activations are normalised (optional fused RMSNorm), then split once per CTA into three int8
//     limbs per value with one scale per 256 values, x ~ s * (l1 + l2/128 + l3/16384), |err| <=
//     2^-22 * max|x| of the block.  Each lane keeps the limbs of the k-range it owns in registers for
//     the whole kernel.  Inner products are integer (dp4a): 4 weights per instruction per limb,
//     exact; the block scales are applied per sub-block in fp32.  This keeps the instruction count
//     near 2 per weight (a float pipeline needs 4+ and cannot reach the HBM rate on 4-bit formats).
//   * Consumer warps are arranged WK x WR: WK slices of K, WR rows of the tile in parallel.  Slices
//     are combined through shared memory once per tile.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the waiter records an error word in
// global memory, stops consuming and the CTA drains and exits; the host turns the word into
// Status::ERROR.  No kernel here can spin forever.
#include "ggb_internal.h"
#include "ggb_limbs.h"

namespace ggb {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr uint32_t kSpinLimit = 1u << 17;         // each poll can suspend for microseconds: about half a second in all
constexpr int kMaxStages = 8;

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
// Bounded wait.  Returns false (and records `code`) if the barrier never flips.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err, int code) {
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(err, code);
    return false;
}
// Bulk async copy global -> this CTA's shared memory; bytes and both addresses multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory"); }

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

// The three limb planes of a 16-value run: 4 words per limb.
struct Limbs16 { int l1[4], l2[4], l3[4]; };
// What a lane keeps per unit: two 16-runs, their fp32 sums, the block scale of x.
struct XUnit { Limbs16 a, b; float sum_a, sum_b, scale; };

// T = sum_k q_k * (l1_k * 2^14 + l2_k * 2^7 + l3_k) over 16 values; q words hold 4 small ints each.
__device__ __forceinline__ int dot16_limbs(const int (&q)[4], const Limbs16& x) {
    int s1 = 0, s2 = 0, s3 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) { s1 = __dp4a(q[i], x.l1[i], s1); s2 = __dp4a(q[i], x.l2[i], s2); s3 = __dp4a(q[i], x.l3[i], s3); }
    return (s1 * 128 + s2) * 128 + s3;        // |s1| <= 16*127*127 -> fits int32 with room
}

// ---- formats ----------------------------------------------------------------------------------
// A format describes: the streams of one tile in shared memory, how unit u of a row maps to two
// 16-runs of k, and the contribution of one (row, unit) given the lane's XUnit.

struct TQ4K {
    static constexpr uint32_t TYPE = T_Q4_K;
    static constexpr int NS = 2;                                   // streams: hdr[16], qs[128] per block
    __device__ static void runs(int u, int& ka, int& kb) { ka = (u >> 3) * 256 + ((u & 7) >> 1) * 64 + (u & 1) * 16; kb = ka + 32; }
    // s0 = hdr stream of the tile, s1 = qs stream; rb = row_in_tile * nb
    __device__ static float unit(const uint8_t* const (&s)[4], int rb, int u, const XUnit& x) {
        const uint4 q = *reinterpret_cast<const uint4*>(s[1] + (static_cast<size_t>(rb) * 8 + u) * 16);
        const uint4 h = *reinterpret_cast<const uint4*>(s[0] + static_cast<size_t>(rb + (u >> 3)) * 16);
        const int lo[4] = {int(q.x & 0x0F0F0F0Fu), int(q.y & 0x0F0F0F0Fu), int(q.z & 0x0F0F0F0Fu), int(q.w & 0x0F0F0F0Fu)};
        const int hi[4] = {int((q.x >> 4) & 0x0F0F0F0Fu), int((q.y >> 4) & 0x0F0F0F0Fu), int((q.z >> 4) & 0x0F0F0F0Fu), int((q.w >> 4) & 0x0F0F0F0Fu)};
        const int t_lo = dot16_limbs(lo, x.a), t_hi = dot16_limbs(hi, x.b);
        const float d = __half2float(__ushort_as_half(static_cast<uint16_t>(h.x & 0xFFFF)));
        const float dmin = __half2float(__ushort_as_half(static_cast<uint16_t>(h.x >> 16)));
        const int j = (u & 7) >> 1;
        int sc0, m0, sc1, m1;
        if (j < 2) {
            const uint32_t a = h.y >> (16 * j), b = h.z >> (16 * j);
            sc0 = a & 63; sc1 = (a >> 8) & 63; m0 = b & 63; m1 = (b >> 8) & 63;
        } else {
            const uint32_t c = h.w >> (16 * (j - 2)), a = h.y >> (16 * (j - 2)), b = h.z >> (16 * (j - 2));
            sc0 = (c & 15) | (((a >> 6) & 3) << 4); m0 = ((c >> 4) & 15) | (((b >> 6) & 3) << 4);
            sc1 = ((c >> 8) & 15) | (((a >> 14) & 3) << 4); m1 = ((c >> 12) & 15) | (((b >> 14) & 3) << 4);
        }
        const float dot = static_cast<float>(sc0) * static_cast<float>(t_lo) + static_cast<float>(sc1) * static_cast<float>(t_hi);
        return d * x.scale * dot - dmin * (static_cast<float>(m0) * x.sum_a + static_cast<float>(m1) * x.sum_b);
    }
};

struct TQ6K {
    static constexpr uint32_t TYPE = T_Q6_K;
    static constexpr int NS = 4;                                   // ql[128], qh[64], scales[16], d[2]
    __device__ static void runs(int u, int& ka, int& kb) {
        const int t8 = u & 7;
        ka = (u >> 3) * 256 + (t8 >> 2) * 128 + ((t8 >> 1) & 1) * 32 + (t8 & 1) * 16; kb = ka + 64;
    }
    __device__ static float unit(const uint8_t* const (&s)[4], int rb, int u, const XUnit& x) {
        const int blk = rb + (u >> 3), t8 = u & 7, hf = t8 >> 2, p = (t8 >> 1) & 1, c = t8 & 1;
        const uint4 ql = *reinterpret_cast<const uint4*>(s[0] + (static_cast<size_t>(rb) * 8 + u) * 16);
        const uint4 qh = *reinterpret_cast<const uint4*>(s[1] + static_cast<size_t>(blk) * 64 + hf * 32 + c * 16);
        const int8_t* sc = reinterpret_cast<const int8_t*>(s[2] + static_cast<size_t>(blk) * 16 + 8 * hf + 2 * p + c);
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(s[3] + static_cast<size_t>(blk) * 2)));
        const int s_lo = 2 * p, s_hi = 2 * p + 4;
        const uint32_t kf = 0x0F0F0F0Fu, k3 = 0x03030303u, k32 = 0x20202020u;
        const uint32_t w[4] = {ql.x, ql.y, ql.z, ql.w}, g[4] = {qh.x, qh.y, qh.z, qh.w};
        int lo[4], hi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lo[i] = int(__vsub4((w[i] & kf) | (((g[i] >> s_lo) & k3) << 4), k32));          // q - 32, per byte
            hi[i] = int(__vsub4(((w[i] >> 4) & kf) | (((g[i] >> s_hi) & k3) << 4), k32));
        }
        const int t_lo = dot16_limbs(lo, x.a), t_hi = dot16_limbs(hi, x.b);
        return d * x.scale * (static_cast<float>(sc[0]) * static_cast<float>(t_lo) + static_cast<float>(sc[4]) * static_cast<float>(t_hi));
    }
};

struct TQ80 {
    static constexpr uint32_t TYPE = T_Q8_0;
    static constexpr int NS = 2;                                   // d[2], qs[32] per 32-block
    __device__ static void runs(int u, int& ka, int& kb) { ka = u * 32; kb = ka + 16; }
    __device__ static float unit(const uint8_t* const (&s)[4], int rb, int u, const XUnit& x) {
        const uint4 q0 = *reinterpret_cast<const uint4*>(s[1] + static_cast<size_t>(rb + u) * 32);
        const uint4 q1 = *reinterpret_cast<const uint4*>(s[1] + static_cast<size_t>(rb + u) * 32 + 16);
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(s[0] + static_cast<size_t>(rb + u) * 2)));
        const int a[4] = {int(q0.x), int(q0.y), int(q0.z), int(q0.w)}, b[4] = {int(q1.x), int(q1.y), int(q1.z), int(q1.w)};
        // |q| <= 127 and 16 values: s1 <= 16*127*127 = 258064, (s1*128 + s2)*128 < 2^33 overflows int32,
        // so the two runs are combined in float.
        int s1 = 0, s2 = 0, s3 = 0, r1 = 0, r2 = 0, r3 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            s1 = __dp4a(a[i], x.a.l1[i], s1); s2 = __dp4a(a[i], x.a.l2[i], s2); s3 = __dp4a(a[i], x.a.l3[i], s3);
            r1 = __dp4a(b[i], x.b.l1[i], r1); r2 = __dp4a(b[i], x.b.l2[i], r2); r3 = __dp4a(b[i], x.b.l3[i], r3);
        }
        const float t = static_cast<float>(s1 + r1) * 16384.0f + static_cast<float>(s2 + r2) * 128.0f + static_cast<float>(s3 + r3);
        return d * x.scale * t;
    }
};

struct TQ40 {
    static constexpr uint32_t TYPE = T_Q4_0;
    static constexpr int NS = 2;                                   // d[2], qs[16] per 32-block
    __device__ static void runs(int u, int& ka, int& kb) { ka = u * 32; kb = ka + 16; }
    __device__ static float unit(const uint8_t* const (&s)[4], int rb, int u, const XUnit& x) {
        const uint4 q = *reinterpret_cast<const uint4*>(s[1] + static_cast<size_t>(rb + u) * 16);
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(s[0] + static_cast<size_t>(rb + u) * 2)));
        const uint32_t k8 = 0x08080808u, kf = 0x0F0F0F0Fu;
        const int lo[4] = {int(__vsub4(q.x & kf, k8)), int(__vsub4(q.y & kf, k8)), int(__vsub4(q.z & kf, k8)), int(__vsub4(q.w & kf, k8))};
        const int hi[4] = {int(__vsub4((q.x >> 4) & kf, k8)), int(__vsub4((q.y >> 4) & kf, k8)), int(__vsub4((q.z >> 4) & kf, k8)),
                           int(__vsub4((q.w >> 4) & kf, k8))};
        const int t = dot16_limbs(lo, x.a) + dot16_limbs(hi, x.b);
        return d * x.scale * static_cast<float>(t);
    }
};

// The non-linear 4-bit codebook (src/quant/iq4_nl.cpp:16-18) by byte-permute: four indices (one per byte, each < 16)
// -> their four signed code bytes.
__device__ __forceinline__ int iq4_codes(uint32_t idx) {
    const uint32_t x = idx | (idx >> 4);
    const uint32_t p = __byte_perm(x, 0u, 0x4420);                     // the four nibbles in the low 16 bits
    const uint32_t sel = p & 0x7777u;
    const uint32_t lo = __byte_perm(0xBFAD9881u, 0xF6EADDCFu, sel);    // -127 -104 -83 -65 | -49 -35 -22 -10
    const uint32_t hi = __byte_perm(0x26190D01u, 0x71594535u, sel);    //    1   13  25  38 |  53  69  89 113
    return static_cast<int>(__byte_perm(lo, hi, 0x3210u | ((p & 0x8888u) >> 1)));
}
// sum over the 32 values of one sub-block: low nibbles against run a, high nibbles against run b (|code| <= 127, so
// the limb sums are combined in float as for Q8_0)
__device__ __forceinline__ float iq4_dot32(const uint4 q, const XUnit& x) {
    const uint32_t kf = 0x0F0F0F0Fu;
    const int a[4] = {iq4_codes(q.x & kf), iq4_codes(q.y & kf), iq4_codes(q.z & kf), iq4_codes(q.w & kf)};
    const int b[4] = {iq4_codes((q.x >> 4) & kf), iq4_codes((q.y >> 4) & kf), iq4_codes((q.z >> 4) & kf), iq4_codes((q.w >> 4) & kf)};
    int s1 = 0, s2 = 0, s3 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        s1 = __dp4a(a[i], x.a.l1[i], s1); s2 = __dp4a(a[i], x.a.l2[i], s2); s3 = __dp4a(a[i], x.a.l3[i], s3);
        s1 = __dp4a(b[i], x.b.l1[i], s1); s2 = __dp4a(b[i], x.b.l2[i], s2); s3 = __dp4a(b[i], x.b.l3[i], s3);
    }
    return static_cast<float>(s1) * 16384.0f + static_cast<float>(s2) * 128.0f + static_cast<float>(s3);
}

struct TIQ4NL {
    static constexpr uint32_t TYPE = T_IQ4_NL;
    static constexpr int NS = 2;                                   // d[2], qs[16] per 32-block
    __device__ static void runs(int u, int& ka, int& kb) { ka = u * 32; kb = ka + 16; }
    __device__ static float unit(const uint8_t* const (&s)[4], int rb, int u, const XUnit& x) {
        const uint4 q = *reinterpret_cast<const uint4*>(s[1] + static_cast<size_t>(rb + u) * 16);
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(s[0] + static_cast<size_t>(rb + u) * 2)));
        return d * x.scale * iq4_dot32(q, x);
    }
};

struct TIQ4XS {
    static constexpr uint32_t TYPE = T_IQ4_XS;
    static constexpr int NS = 2;                                   // header d | scales_h | scales_l[4] (8 bytes), qs[128] per 256-block
    __device__ static void runs(int u, int& ka, int& kb) { ka = u * 32; kb = ka + 16; }
    __device__ static float unit(const uint8_t* const (&s)[4], int rb, int u, const XUnit& x) {
        const uint4 q = *reinterpret_cast<const uint4*>(s[1] + (static_cast<size_t>(rb) * 8 + u) * 16);
        const uint2 h = *reinterpret_cast<const uint2*>(s[0] + static_cast<size_t>(rb + (u >> 3)) * 8);
        const int ib = u & 7;
        const int ls = static_cast<int>(((h.y >> (4 * ib)) & 15u) | (((h.x >> (16 + 2 * ib)) & 3u) << 4));
        const float d = __half2float(__ushort_as_half(static_cast<uint16_t>(h.x & 0xFFFFu)));
        return d * static_cast<float>(ls - 32) * x.scale * iq4_dot32(q, x);
    }
};

// ---- kernel -----------------------------------------------------------------------------------

struct TmaGemvArgs {
    PackedW w, w2;
    const float* x;
    float* y;
    const float* bias;
    const float* resid;
    const float* gamma;
    float eps;
    int epi;
    int tile_rows;        // rows per tile (multiple of 8)
    int n_tiles;
    int stages;
    int stage_bytes;      // bytes of one ring stage (all streams of one tile, both weights if dual)
    int wk;               // K slices
    int units_per_slice;
    int left_begin;       // >= 0: units [left_begin, K / 32) are a leftover slice that the warps take in turn, one row each (see launch_tma)
    int* err;
    // stacked matrices (q, k, v of one layer): tiles [tile_first[i], tile_first[i + 1]) belong to matrix
    // i + 1, which has its own streams, row count, output and bias; all share K, the format and x
    int n_cat;
    int tile_first[2];
    const uint8_t* cat_s[2][kMaxStreams];
    int64_t cat_N[2];
    float* cat_y[2];
    const float* cat_bias[2];
    // multi-row kernel: rows [m0, m0 + M) of the activation image (full image: M_img rows)
    int M, M_img, m0, ldc;
    const uint8_t* img;
};

// Matrix and first row of tile t.
struct TileRef {
    const uint8_t* const* s;
    int64_t N, row0;
    float* y;
    const float* bias;
};
__device__ __forceinline__ TileRef tile_ref(const TmaGemvArgs& a, int t) {
    TileRef r;
    if (a.n_cat == 0 || t < a.tile_first[0]) {
        r.s = a.w.s; r.N = a.w.N; r.y = a.y; r.bias = a.bias; r.row0 = static_cast<int64_t>(t) * a.tile_rows;
    } else {
        const int i = (a.n_cat > 1 && t >= a.tile_first[1]) ? 1 : 0;
        r.s = a.cat_s[i]; r.N = a.cat_N[i]; r.y = a.cat_y[i]; r.bias = a.cat_bias[i];
        r.row0 = static_cast<int64_t>(t - a.tile_first[i]) * a.tile_rows;
    }
    return r;
}

// Shared-memory map (dynamic): [ring: stages * stage_bytes][x limb planes 3*K][x run sums K/16 floats]
// [block scales K/256 floats][slice partials 2 * tile_rows * wk * (dual ? 2 : 1) floats]
template <class F, bool DUAL>
__global__ void __launch_bounds__(kThreads, 1) gemv_tma_kernel(const TmaGemvArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages];
    __shared__ float red[kConsumerWarps];
    const int K = a.w.K, nb = a.w.nb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const FormatInfo fi = format_info(F::TYPE);
    uint8_t* ring = smem;
    int8_t* xl = reinterpret_cast<int8_t*>(ring + static_cast<size_t>(a.stages) * a.stage_bytes);
    float* xsum = reinterpret_cast<float*>(xl + 3 * static_cast<size_t>(K));
    float* xscale = xsum + (K >> 4);
    float* part = xscale + (K >> 8);

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], kConsumerWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch();       // the next kernel may start streaming its own weights

    // per-stream byte offsets inside a stage (full tile); streams of w2 follow those of w
    int soff[2 * kMaxStreams];
    {
        int acc = 0;
        for (int i = 0; i < F::NS; ++i) { soff[i] = acc; acc += a.tile_rows * nb * fi.size[i]; }
        for (int i = 0; i < F::NS; ++i) { soff[kMaxStreams + i] = acc; if (DUAL) acc += a.tile_rows * nb * fi.size[i]; }
    }

    if (warp == kConsumerWarps) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int n = 0;
            for (int t = blockIdx.x; t < a.n_tiles; t += gridDim.x, ++n) {
                const int s = n % a.stages;
                const uint32_t ph = (n / a.stages) & 1;
                if (!mbar_wait(&empty_bar[s], ph ^ 1, a.err, 1)) break;
                const TileRef tr = tile_ref(a, t);
                const int64_t row0 = tr.row0;
                const int rows = static_cast<int>(min(static_cast<int64_t>(a.tile_rows), tr.N - row0));
                uint32_t bytes = 0;
                for (int i = 0; i < F::NS; ++i) bytes += rows * nb * fi.size[i];
                mbar_expect_tx(&full_bar[s], DUAL ? 2 * bytes : bytes);
                uint8_t* dst = ring + static_cast<size_t>(s) * a.stage_bytes;
                for (int i = 0; i < F::NS; ++i) {
                    const uint32_t sz = rows * nb * fi.size[i];
                    bulk_g2s(dst + soff[i], tr.s[i] + row0 * nb * fi.size[i], sz, &full_bar[s]);
                    if (DUAL) bulk_g2s(dst + soff[kMaxStreams + i], a.w2.s[i] + row0 * nb * fi.size[i], sz, &full_bar[s]);
                }
            }
        }
    } else {
        // ---------------- consumers ----------------
        const int tid = threadIdx.x;                      // 0 .. 255
        pdl_wait();                                       // x (and resid) come from the previous kernel
        // 1. optional RMSNorm scale
        float inv = 1.0f;
        if (a.gamma) {
            float ss = 0.0f;
            for (int i = tid; i < (K >> 2); i += kConsumerWarps * 32) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(a.x) + i);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
            ss = wsum(ss);
            if (lane == 0) red[warp] = ss;
            consumer_sync();
            float tot = 0.0f;
#pragma unroll
            for (int i = 0; i < kConsumerWarps; ++i) tot += red[i];
            inv = 1.0f / sqrtf(tot / static_cast<float>(K) + a.eps);
        }
        // 2. limbs: one warp per 256-block, 8 values per lane
        for (int b = warp; b < (K >> 8); b += kConsumerWarps) {
            const int k0 = b * 256 + lane * 8;
            float v[8];
            {
                const float4 p0 = __ldg(reinterpret_cast<const float4*>(a.x + k0)), p1 = __ldg(reinterpret_cast<const float4*>(a.x + k0 + 4));
                v[0] = p0.x; v[1] = p0.y; v[2] = p0.z; v[3] = p0.w; v[4] = p1.x; v[5] = p1.y; v[6] = p1.z; v[7] = p1.w;
            }
            if (a.gamma) {
                const float4 g0 = __ldg(reinterpret_cast<const float4*>(a.gamma + k0)), g1 = __ldg(reinterpret_cast<const float4*>(a.gamma + k0 + 4));
                v[0] = v[0] * inv * g0.x; v[1] = v[1] * inv * g0.y; v[2] = v[2] * inv * g0.z; v[3] = v[3] * inv * g0.w;
                v[4] = v[4] * inv * g1.x; v[5] = v[5] * inv * g1.y; v[6] = v[6] * inv * g1.z; v[7] = v[7] * inv * g1.w;
            }
            float am = 0.0f, sm = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) { am = fmaxf(am, fabsf(v[i])); sm += v[i]; }
            am = wmax(am);
            const float scale = am / 127.0f;
            const float rs = am > 0.0f ? 127.0f / am : 0.0f;
            uint32_t w1[2] = {0, 0}, w2[2] = {0, 0}, w3[2] = {0, 0};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float r = v[i] * rs;
                const float l1 = rintf(r);
                const float r2 = (r - l1) * 128.0f;
                const float l2 = rintf(r2);
                const float l3 = rintf((r2 - l2) * 128.0f);
                w1[i >> 2] |= (static_cast<uint32_t>(static_cast<int>(l1)) & 0xFFu) << (8 * (i & 3));
                w2[i >> 2] |= (static_cast<uint32_t>(static_cast<int>(l2)) & 0xFFu) << (8 * (i & 3));
                w3[i >> 2] |= (static_cast<uint32_t>(static_cast<int>(l3)) & 0xFFu) << (8 * (i & 3));
            }
            *reinterpret_cast<uint2*>(xl + k0) = make_uint2(w1[0], w1[1]);
            *reinterpret_cast<uint2*>(xl + K + k0) = make_uint2(w2[0], w2[1]);
            *reinterpret_cast<uint2*>(xl + 2 * K + k0) = make_uint2(w3[0], w3[1]);
            const float pair = sm + __shfl_xor_sync(0xFFFFFFFFu, sm, 1);      // 16-run = two lanes
            if ((lane & 1) == 0) xsum[(k0 >> 4)] = pair;
            if (lane == 0) xscale[b] = scale * (1.0f / 16384.0f);
        }
        consumer_sync();
        // 3. this lane's units: slice wk_i of K, units u = slice_begin + lane + 32 i
        const int wk_i = warp % a.wk, wr_i = warp / a.wk, wr_n = kConsumerWarps / a.wk;
        const int units = K >> 5;
        const int u_begin = wk_i * a.units_per_slice, u_end = min(a.left_begin >= 0 ? a.left_begin : units, u_begin + a.units_per_slice);
        XUnit xu[2];
        int my_u[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            // leftover mode: the lane's second unit is its unit of the leftover slice (the same in every warp)
            const int u = (i == 1 && a.left_begin >= 0) ? a.left_begin + lane : u_begin + lane + 32 * i;
            my_u[i] = u < ((i == 1 && a.left_begin >= 0) ? units : u_end) ? u : -1;
            if (my_u[i] >= 0) {
                int ka, kb;
                F::runs(u, ka, kb);
#pragma unroll
                for (int p = 0; p < 3; ++p) {
                    const int4 va = *reinterpret_cast<const int4*>(xl + p * K + ka), vb = *reinterpret_cast<const int4*>(xl + p * K + kb);
                    int* da = p == 0 ? xu[i].a.l1 : (p == 1 ? xu[i].a.l2 : xu[i].a.l3);
                    int* db = p == 0 ? xu[i].b.l1 : (p == 1 ? xu[i].b.l2 : xu[i].b.l3);
                    da[0] = va.x; da[1] = va.y; da[2] = va.z; da[3] = va.w; db[0] = vb.x; db[1] = vb.y; db[2] = vb.z; db[3] = vb.w;
                }
                xu[i].sum_a = xsum[ka >> 4]; xu[i].sum_b = xsum[kb >> 4]; xu[i].scale = xscale[ka >> 8];
            }
        }
        // 4. tiles
        bool ok = true;
        int n = 0;
        for (int t = blockIdx.x; t < a.n_tiles; t += gridDim.x, ++n) {
            // After a timed-out wait a warp stops computing but keeps iterating, so that the
            // consumer-wide barriers below stay matched and the CTA always runs to its end.
            const int s = n % a.stages;
            const uint32_t ph = (n / a.stages) & 1;
            if (ok) ok = mbar_wait(&full_bar[s], ph, a.err, 2);
            const TileRef tr = tile_ref(a, t);
            const int64_t row0 = tr.row0;
            const int rows = static_cast<int>(min(static_cast<int64_t>(a.tile_rows), tr.N - row0));
            const uint8_t* base = ring + static_cast<size_t>(s) * a.stage_bytes;
            // stream bases of this tile (a partial last tile fills only the head of each stream slot)
            const uint8_t* sa[4] = {nullptr, nullptr, nullptr, nullptr};
            const uint8_t* sb[4] = {nullptr, nullptr, nullptr, nullptr};
#pragma unroll
            for (int i = 0; i < F::NS; ++i) { sa[i] = base + soff[i]; sb[i] = base + soff[kMaxStreams + i]; }
            float* pp = part + (n & 1) * (a.tile_rows * a.wk * (DUAL ? 2 : 1));
            for (int r = wr_i; r < rows && ok; r += wr_n) {
                float acc = 0.0f, acc2 = 0.0f;
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    if (my_u[i] >= 0 && (i == 0 || a.left_begin < 0 || (r & (kConsumerWarps - 1)) == warp)) {
                        acc += F::unit(sa, r * nb, my_u[i], xu[i]);
                        if constexpr (DUAL) acc2 += F::unit(sb, r * nb, my_u[i], xu[i]);
                    }
                acc = wsum(acc);
                if constexpr (DUAL) acc2 = wsum(acc2);
                if (a.wk > 1) {
                    if (lane == 0) { pp[r * a.wk + wk_i] = acc; if constexpr (DUAL) pp[(a.tile_rows + r) * a.wk + wk_i] = acc2; }
                } else if (lane == 0) {
                    const int64_t nrow = row0 + r;
                    float v = acc;
                    if constexpr (DUAL) v = (v / (1.0f + expf(-v))) * acc2;
                    else if (a.epi == EPI_ADD_BIAS) v += __ldg(tr.bias + nrow);
                    else if (a.epi == EPI_RESIDUAL) v += a.resid[nrow];
                    tr.y[nrow] = v;
                }
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&empty_bar[s]);     // this warp is done reading the stage
            if (a.wk > 1) {
                consumer_sync();                           // partials of every slice are in shared memory
                for (int r = tid; r < rows && ok; r += kConsumerWarps * 32) {
                    float v = 0.0f, v2 = 0.0f;
                    for (int k = 0; k < a.wk; ++k) { v += pp[r * a.wk + k]; if constexpr (DUAL) v2 += pp[(a.tile_rows + r) * a.wk + k]; }
                    const int64_t nrow = row0 + r;
                    if constexpr (DUAL) v = (v / (1.0f + expf(-v))) * v2;
                    else if (a.epi == EPI_ADD_BIAS) v += __ldg(tr.bias + nrow);
                    else if (a.epi == EPI_RESIDUAL) v += a.resid[nrow];
                    tr.y[nrow] = v;
                }
            }
        }
    }
}

template <class F, bool DUAL>
int launch_tma(Context* c, const GemvArgs& g, cudaStream_t s) {
    const FormatInfo fi = format_info(F::TYPE);
    const int K = g.w.K, nb = g.w.nb;
    const int64_t N = g.w.N;
    const int units = K / 32;
    if (K % 256 || N % 8 || units > 8 * 64) return GGB_NOT_FOUND;
    if (g.n_cat && (DUAL || g.n_cat > 2 || (g.epi != EPI_STORE && g.epi != EPI_ADD_BIAS))) return GGB_NOT_FOUND;
    int64_t n_all = N;
    for (int i = 0; i < g.n_cat; ++i) {
        const PackedW& w = g.cat_w[i];
        if (w.type != g.w.type || w.K != K || w.layout != 0 || w.N % 8 || !g.cat_y[i] || (g.epi == EPI_ADD_BIAS && !g.cat_bias[i])) return GGB_NOT_FOUND;
        n_all += w.N;
    }
    int wk = 1;
    while (wk < kConsumerWarps && (units + wk - 1) / wk > 64) wk *= 2;
    int ups = (units + wk - 1) / wk;
    // A few units more than one per lane (K = 8960: 280 units = 8 x 32 + 24) would cost every warp a second, nearly empty
    // pass per row.  Then the slices take 32 units each and the rest forms a leftover slice that the eight warps take in
    // turn, one row each: 9 warp passes per row instead of 16.
    int left_begin = -1;
    if (wk == kConsumerWarps && ups > 32 && units - 32 * kConsumerWarps <= 32) { ups = 32; left_begin = 32 * kConsumerWarps; }
    const int row_bytes = nb * fi.block_bytes * (DUAL ? 2 : 1);
    // Tile height: every stream slice of a tile must be a multiple of 16 bytes (granule g rows), a
    // tile should carry roughly 8-24 KB, and the busiest CTA should get as few bytes as possible.
    int gran = 1;
    for (int i = 0; i < fi.n_streams; ++i) while ((gran * nb * fi.size[i]) % 16) ++gran;
    if (N % gran) return GGB_NOT_FOUND;
    for (int i = 0; i < g.n_cat; ++i) if (g.cat_w[i].N % gran) return GGB_NOT_FOUND;
    const int G = c->sm_count;
    int tile_rows = gran;
    double best = 1e30;
    for (int tr = gran; tr <= 512 && static_cast<int64_t>(tr) * row_bytes <= 24 * 1024 + (tr == gran ? (1 << 30) : 0); tr += gran) {
        int64_t nt = (N + tr - 1) / tr;
        for (int i = 0; i < g.n_cat; ++i) nt += (g.cat_w[i].N + tr - 1) / tr;
        const double cost = static_cast<double>((nt + G - 1) / G) * (static_cast<double>(tr) * row_bytes + 3072.0);
        if (cost < best * 0.999) { best = cost; tile_rows = tr; }
    }
    const int stage_bytes = (tile_rows * row_bytes + 127) / 128 * 128;
    const size_t fixed = static_cast<size_t>(3) * K + sizeof(float) * (K / 16 + K / 256) + sizeof(float) * 2 * tile_rows * wk * (DUAL ? 2 : 1) + 256;
    const size_t budget = 100 * 1024;          // two such CTAs fit one SM: this kernel and the next one's prefetch
    if (fixed + 2 * static_cast<size_t>(stage_bytes) > 200 * 1024) return GGB_NOT_FOUND;
    int stages = static_cast<int>((std::max(budget, fixed + 2 * stage_bytes) - fixed) / stage_bytes);
    stages = std::max(2, std::min(stages, kMaxStages));
    int n_tiles = static_cast<int>((N + tile_rows - 1) / tile_rows);
    int tile_first[2] = {0, 0};
    for (int i = 0; i < g.n_cat; ++i) { tile_first[i] = n_tiles; n_tiles += static_cast<int>((g.cat_w[i].N + tile_rows - 1) / tile_rows); }
    stages = std::min(stages, std::max(2, (n_tiles + c->sm_count - 1) / c->sm_count));
    const size_t smem = static_cast<size_t>(stages) * stage_bytes + fixed;

    TmaGemvArgs a{};
    a.w = g.w; a.w2 = g.w2; a.x = g.x; a.y = g.y; a.bias = g.bias; a.resid = g.resid; a.gamma = g.gamma; a.eps = g.eps; a.epi = g.epi;
    a.tile_rows = tile_rows; a.n_tiles = n_tiles; a.stages = stages; a.stage_bytes = stage_bytes; a.wk = wk; a.units_per_slice = ups;
    a.left_begin = left_begin;
    a.err = c->d_err;
    a.n_cat = g.n_cat;
    for (int i = 0; i < g.n_cat; ++i) {
        a.tile_first[i] = tile_first[i];
        for (int j = 0; j < kMaxStreams; ++j) a.cat_s[i][j] = g.cat_w[i].s[j];
        a.cat_N[i] = g.cat_w[i].N; a.cat_y[i] = g.cat_y[i]; a.cat_bias[i] = g.cat_bias[i];
    }

    auto kern = gemv_tma_kernel<F, DUAL>;
    {
        const cudaError_t e = ensure_dynamic_smem(c, kern, smem);
        if (e != cudaSuccess) return cuda_status(c, e, "gemv_tma attr");
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(std::min(n_tiles, c->sm_count)));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = c->use_pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
    c->launches++;
    return cuda_status(c, e, "gemv_tma launch");
}


// ---- 2..16 activation rows, stream layout ---------------------------------------------------------
// The same tiles, ring and per-unit arithmetic as gemv_tma_kernel, for a.M rows of activations taken from the limb
// image (ggb_limbs.h): all rows' limb planes, 16-run sums and block scales sit in shared memory, a tile is consumed
// once per row (the lane's two units of that row are re-read from the planes, then every weight row of the tile is
// multiplied), so the weights are streamed once for the whole chunk of rows.
// Shared-memory map: [ring][planes 3 * M * K][asum16 M * K / 16 floats][xs M * K / 256 floats (padded to 16 B)]
// [slice partials 2 * M * tile_rows * wk * (dual ? 2 : 1) floats]
template <class F, bool DUAL>
__global__ void __launch_bounds__(kThreads, 1) gemv_tma_rows_kernel(const TmaGemvArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], x_bar;
    __shared__ float inv_s[16];
    const int K = a.w.K, nb = a.w.nb, M = a.M;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const FormatInfo fi = format_info(F::TYPE);
    uint8_t* ring = smem;
    int8_t* xl = reinterpret_cast<int8_t*>(ring + static_cast<size_t>(a.stages) * a.stage_bytes);
    float* xsum = reinterpret_cast<float*>(xl + static_cast<size_t>(3) * M * K);
    float* xscale = xsum + static_cast<size_t>(M) * (K >> 4);
    float* part = xscale + ((M * (K >> 8) + 3) & ~3);

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], kConsumerWarps); }
        mbar_init(&x_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch();

    int soff[2 * kMaxStreams];
    {
        int acc = 0;
        for (int i = 0; i < F::NS; ++i) { soff[i] = acc; acc += a.tile_rows * nb * fi.size[i]; }
        for (int i = 0; i < F::NS; ++i) { soff[kMaxStreams + i] = acc; if (DUAL) acc += a.tile_rows * nb * fi.size[i]; }
    }

    if (warp == kConsumerWarps) {
        // ---------------- producer (as in gemv_tma_kernel) ----------------
        if (lane == 0) {
            int n = 0;
            for (int t = blockIdx.x; t < a.n_tiles; t += gridDim.x, ++n) {
                const int s = n % a.stages;
                const uint32_t ph = (n / a.stages) & 1;
                if (!mbar_wait(&empty_bar[s], ph ^ 1, a.err, 1)) break;
                const int64_t row0 = static_cast<int64_t>(t) * a.tile_rows;
                const int rows = static_cast<int>(min(static_cast<int64_t>(a.tile_rows), a.w.N - row0));
                uint32_t bytes = 0;
                for (int i = 0; i < F::NS; ++i) bytes += rows * nb * fi.size[i];
                mbar_expect_tx(&full_bar[s], DUAL ? 2 * bytes : bytes);
                uint8_t* dst = ring + static_cast<size_t>(s) * a.stage_bytes;
                for (int i = 0; i < F::NS; ++i) {
                    const uint32_t sz = rows * nb * fi.size[i];
                    bulk_g2s(dst + soff[i], a.w.s[i] + row0 * nb * fi.size[i], sz, &full_bar[s]);
                    if (DUAL) bulk_g2s(dst + soff[kMaxStreams + i], a.w2.s[i] + row0 * nb * fi.size[i], sz, &full_bar[s]);
                }
            }
        }
    } else {
        // ---------------- consumers ----------------
        const int tid = threadIdx.x;
        pdl_wait();                                       // the image (and resid) come from the previous kernels
        bool ok = true;
        {
            const LimbImage L(a.M_img, K);
            if (tid == 0) {                               // rows m0 .. m0 + M of the planes and of the 16-run sums are contiguous
                const uint32_t pb = static_cast<uint32_t>(3) * M * K, sb16 = static_cast<uint32_t>(M) * (K >> 4) * 4;
                mbar_expect_tx(&x_bar, pb + sb16);
                bulk_g2s(xl, a.img + L.planes + static_cast<size_t>(3) * a.m0 * K, pb, &x_bar);
                bulk_g2s(xsum, a.img + L.asum16 + sizeof(float) * static_cast<size_t>(a.m0) * (K >> 4), sb16, &x_bar);
            }
            const float* gxs = reinterpret_cast<const float*>(a.img + L.xs) + static_cast<size_t>(a.m0) * (K >> 8);
            for (int i = tid; i < M * (K >> 8); i += kConsumerWarps * 32) xscale[i] = gxs[i] * (1.0f / 16384.0f);
            if (tid < M) inv_s[tid] = reinterpret_cast<const float*>(a.img + L.inv_s)[a.m0 + tid];
            ok = mbar_wait(&x_bar, 0, a.err, 3);
        }
        consumer_sync();
        const int wk_i = warp % a.wk, wr_i = warp / a.wk, wr_n = kConsumerWarps / a.wk;
        const int units = K >> 5;
        const int u_begin = wk_i * a.units_per_slice, u_end = min(units, u_begin + a.units_per_slice);
        int my_u[2], ka[2], kb[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int u = u_begin + lane + 32 * i;
            my_u[i] = u < u_end ? u : -1;
            ka[i] = 0; kb[i] = 0;
            if (my_u[i] >= 0) F::runs(u, ka[i], kb[i]);
        }
        const int pstride = a.tile_rows * a.wk;           // partials of one activation row
        int n = 0;
        for (int t = blockIdx.x; t < a.n_tiles; t += gridDim.x, ++n) {
            const int s = n % a.stages;
            const uint32_t ph = (n / a.stages) & 1;
            if (ok) ok = mbar_wait(&full_bar[s], ph, a.err, 2);
            const int64_t row0 = static_cast<int64_t>(t) * a.tile_rows;
            const int rows = static_cast<int>(min(static_cast<int64_t>(a.tile_rows), a.w.N - row0));
            const uint8_t* base = ring + static_cast<size_t>(s) * a.stage_bytes;
            const uint8_t* sa[4] = {nullptr, nullptr, nullptr, nullptr};
            const uint8_t* sb[4] = {nullptr, nullptr, nullptr, nullptr};
#pragma unroll
            for (int i = 0; i < F::NS; ++i) { sa[i] = base + soff[i]; sb[i] = base + soff[kMaxStreams + i]; }
            float* pp = part + (n & 1) * (M * pstride * (DUAL ? 2 : 1));
            for (int m = 0; m < M && ok; ++m) {
                XUnit xu[2];
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    if (my_u[i] >= 0) {
                        const int8_t* pl = xl + static_cast<size_t>(3 * m) * K;
#pragma unroll
                        for (int p = 0; p < 3; ++p) {
                            const int4 va = *reinterpret_cast<const int4*>(pl + p * K + ka[i]), vb = *reinterpret_cast<const int4*>(pl + p * K + kb[i]);
                            int* da = p == 0 ? xu[i].a.l1 : (p == 1 ? xu[i].a.l2 : xu[i].a.l3);
                            int* db = p == 0 ? xu[i].b.l1 : (p == 1 ? xu[i].b.l2 : xu[i].b.l3);
                            da[0] = va.x; da[1] = va.y; da[2] = va.z; da[3] = va.w; db[0] = vb.x; db[1] = vb.y; db[2] = vb.z; db[3] = vb.w;
                        }
                        xu[i].sum_a = xsum[m * (K >> 4) + (ka[i] >> 4)]; xu[i].sum_b = xsum[m * (K >> 4) + (kb[i] >> 4)];
                        xu[i].scale = xscale[m * (K >> 8) + (ka[i] >> 8)];
                    }
                for (int r = wr_i; r < rows; r += wr_n) {
                    float acc = 0.0f, acc2 = 0.0f;
#pragma unroll
                    for (int i = 0; i < 2; ++i)
                        if (my_u[i] >= 0) {
                            acc += F::unit(sa, r * nb, my_u[i], xu[i]);
                            if constexpr (DUAL) acc2 += F::unit(sb, r * nb, my_u[i], xu[i]);
                        }
                    acc = wsum(acc);
                    if constexpr (DUAL) acc2 = wsum(acc2);
                    if (a.wk > 1) {
                        if (lane == 0) { pp[m * pstride + r * a.wk + wk_i] = acc; if constexpr (DUAL) pp[(M + m) * pstride + r * a.wk + wk_i] = acc2; }
                    } else if (lane == 0) {
                        const int64_t nrow = row0 + r;
                        const size_t o = static_cast<size_t>(m) * a.ldc + nrow;
                        float v = acc * inv_s[m];
                        if constexpr (DUAL) { const float u2 = acc2 * inv_s[m]; v = (v / (1.0f + expf(-v))) * u2; }
                        else if (a.epi == EPI_ADD_BIAS) v += __ldg(a.bias + nrow);
                        else if (a.epi == EPI_RESIDUAL) v += a.resid[o];
                        a.y[o] = v;
                    }
                }
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&empty_bar[s]);     // this warp is done reading the stage
            if (a.wk > 1) {
                consumer_sync();                           // partials of every slice are in shared memory
                for (int idx = tid; idx < rows * M && ok; idx += kConsumerWarps * 32) {
                    const int m = idx / rows, r = idx - m * rows;
                    float v = 0.0f, v2 = 0.0f;
                    for (int k = 0; k < a.wk; ++k) { v += pp[m * pstride + r * a.wk + k]; if constexpr (DUAL) v2 += pp[(M + m) * pstride + r * a.wk + k]; }
                    const int64_t nrow = row0 + r;
                    const size_t o = static_cast<size_t>(m) * a.ldc + nrow;
                    v *= inv_s[m];
                    if constexpr (DUAL) { v2 *= inv_s[m]; v = (v / (1.0f + expf(-v))) * v2; }
                    else if (a.epi == EPI_ADD_BIAS) v += __ldg(a.bias + nrow);
                    else if (a.epi == EPI_RESIDUAL) v += a.resid[o];
                    a.y[o] = v;
                }
                // the partial buffers alternate between tiles (n & 1): the next tile writes the other one, and the one after
                // that passes another consumer_sync first
            }
        }
    }
}

// Rows of activations per pass: the limb planes, 16-run sums and scales of a chunk must fit beside the ring.
static int tma_rows_chunk(int K, int M) {
    const size_t per_row = static_cast<size_t>(3) * K + sizeof(float) * ((K >> 4) + (K >> 8));
    const int fit = static_cast<int>((112 * 1024) / per_row);
    return std::min(M, fit);
}

template <class F, bool DUAL>
int launch_tma_rows(Context* c, const GemvArgs& g, cudaStream_t s) {
    const FormatInfo fi = format_info(F::TYPE);
    const int K = g.w.K, nb = g.w.nb;
    const int64_t N = g.w.N;
    const int units = K / 32;
    if (K % 256 || N % 8 || units > 8 * 64) return GGB_NOT_FOUND;
    const int Mc = tma_rows_chunk(K, g.M);
    if (Mc < 1 || (Mc < 2 && g.M > 4)) return GGB_NOT_FOUND;        // K so long that a pass would carry one row: the general kernel's M tiles do better
    int wk = 1;
    while (wk < kConsumerWarps && (units + wk - 1) / wk > 64) wk *= 2;
    const int ups = (units + wk - 1) / wk;
    const int row_bytes = nb * fi.block_bytes * (DUAL ? 2 : 1);
    int gran = 1;
    for (int i = 0; i < fi.n_streams; ++i) while ((gran * nb * fi.size[i]) % 16) ++gran;
    if (N % gran) return GGB_NOT_FOUND;
    const int G = c->sm_count;
    int tile_rows = gran;
    double best = 1e30;
    for (int tr = gran; tr <= 512 && static_cast<int64_t>(tr) * row_bytes <= 24 * 1024 + (tr == gran ? (1 << 30) : 0); tr += gran) {
        const int64_t nt = (N + tr - 1) / tr;
        const double cost = static_cast<double>((nt + G - 1) / G) * (static_cast<double>(tr) * row_bytes + 3072.0);
        if (cost < best * 0.999) { best = cost; tile_rows = tr; }
    }
    const int stage_bytes = (tile_rows * row_bytes + 127) / 128 * 128;
    const int n_tiles = static_cast<int>((N + tile_rows - 1) / tile_rows);
    {
        const int sp = limb_image_prepare(c, g, s);
        if (sp != GGB_OK) return sp;
    }
    for (int m0 = 0; m0 < g.M; m0 += Mc) {
        const int mc = std::min(Mc, g.M - m0);
        const size_t fixed = static_cast<size_t>(3) * mc * K + sizeof(float) * (static_cast<size_t>(mc) * (K >> 4) + ((mc * (K >> 8) + 3) & ~3)) +
                             sizeof(float) * 2 * mc * tile_rows * wk * (DUAL ? 2 : 1) + 256;
        if (fixed + 2 * static_cast<size_t>(stage_bytes) > 216 * 1024) return m0 == 0 ? GGB_NOT_FOUND : set_status(c, GGB_ERROR, "gemv_tma_rows: a later pass did not fit");
        int stages = static_cast<int>((216 * 1024 - fixed) / stage_bytes);
        stages = std::max(2, std::min(stages, kMaxStages));
        stages = std::min(stages, std::max(2, (n_tiles + c->sm_count - 1) / c->sm_count));
        const size_t smem = static_cast<size_t>(stages) * stage_bytes + fixed;

        TmaGemvArgs a{};
        a.w = g.w; a.w2 = g.w2; a.x = nullptr; a.y = g.y + static_cast<size_t>(m0) * g.ldc; a.bias = g.bias;
        a.resid = g.resid ? g.resid + static_cast<size_t>(m0) * g.ldc : nullptr; a.gamma = g.gamma; a.eps = g.eps; a.epi = g.epi;
        a.tile_rows = tile_rows; a.n_tiles = n_tiles; a.stages = stages; a.stage_bytes = stage_bytes; a.wk = wk; a.units_per_slice = ups;
        a.left_begin = -1;
        a.err = c->d_err;
        a.M = mc; a.M_img = g.M; a.m0 = m0; a.ldc = g.ldc; a.img = static_cast<const uint8_t*>(c->d_limbs);
        auto kern = gemv_tma_rows_kernel<F, DUAL>;
        cudaError_t e = ensure_dynamic_smem(c, kern, smem);
        if (e != cudaSuccess) return cuda_status(c, e, "gemv_tma_rows attr");
        e = launch_pdl(c, kern, dim3(static_cast<unsigned>(std::min(n_tiles, c->sm_count))), dim3(kThreads), smem, s, a);
        c->launches++;
        if (e != cudaSuccess) return cuda_status(c, e, "gemv_tma_rows launch");
    }
    return GGB_OK;
}

}  // namespace

// M == 1 fast path.  Returns GGB_NOT_FOUND when the shape or format is not covered (the caller then
// uses the general kernel), GGB_OK or an error otherwise.
int launch_gemv_tma(Context* c, const GemvArgs& g, cudaStream_t s) {
    if (g.M != 1 || g.w.layout != 0 || (reinterpret_cast<uintptr_t>(g.x) & 15)) return GGB_NOT_FOUND;
    const bool dual = g.epi == EPI_SWIGLU;
    switch (g.w.type) {
    case T_Q4_K: return dual ? launch_tma<TQ4K, true>(c, g, s) : launch_tma<TQ4K, false>(c, g, s);
    case T_Q6_K: return dual ? launch_tma<TQ6K, true>(c, g, s) : launch_tma<TQ6K, false>(c, g, s);
    case T_Q8_0: return dual ? launch_tma<TQ80, true>(c, g, s) : launch_tma<TQ80, false>(c, g, s);
    case T_Q4_0: return dual ? launch_tma<TQ40, true>(c, g, s) : launch_tma<TQ40, false>(c, g, s);
    case T_IQ4_NL: return dual ? launch_tma<TIQ4NL, true>(c, g, s) : launch_tma<TIQ4NL, false>(c, g, s);
    case T_IQ4_XS: return dual ? launch_tma<TIQ4XS, true>(c, g, s) : launch_tma<TIQ4XS, false>(c, g, s);
    default: return GGB_NOT_FOUND;
    }
}

// 2 <= M <= 16 rows of a stream-layout matrix (Q8_0, Q4_0, IQ4_NL, IQ4_XS, and Q4_K / Q6_K when they are kept in that
// layout): exact int8-limb activations as at M = 1, the weights streamed once per chunk of rows that fits shared memory.
// The caller has made c->d_limbs large enough.  GGB_NOT_FOUND: shape or format not covered.
int launch_gemv_tma_rows(Context* c, const GemvArgs& g, cudaStream_t s) {
    if (g.M < 2 || g.M > 16 || g.w.layout != 0 || !g.x || (reinterpret_cast<uintptr_t>(g.x) & 15) || (g.lda & 3)) return GGB_NOT_FOUND;
    if (g.n_cat || g.attn_partial || g.sel || g.xscale || g.x_img || g.y_img) return GGB_NOT_FOUND;
    const bool dual = g.epi == EPI_SWIGLU;
    if (dual && g.w2.layout != 0) return GGB_NOT_FOUND;
    if (g.epi == EPI_ADD_BIAS && !g.bias) return GGB_NOT_FOUND;
    switch (g.w.type) {
    case T_Q4_K: return dual ? launch_tma_rows<TQ4K, true>(c, g, s) : launch_tma_rows<TQ4K, false>(c, g, s);
    case T_Q6_K: return dual ? launch_tma_rows<TQ6K, true>(c, g, s) : launch_tma_rows<TQ6K, false>(c, g, s);
    case T_Q8_0: return dual ? launch_tma_rows<TQ80, true>(c, g, s) : launch_tma_rows<TQ80, false>(c, g, s);
    case T_Q4_0: return dual ? launch_tma_rows<TQ40, true>(c, g, s) : launch_tma_rows<TQ40, false>(c, g, s);
    case T_IQ4_NL: return dual ? launch_tma_rows<TIQ4NL, true>(c, g, s) : launch_tma_rows<TIQ4NL, false>(c, g, s);
    case T_IQ4_XS: return dual ? launch_tma_rows<TIQ4XS, true>(c, g, s) : launch_tma_rows<TIQ4XS, false>(c, g, s);
    default: return GGB_NOT_FOUND;
    }
}

}  // namespace ggb
