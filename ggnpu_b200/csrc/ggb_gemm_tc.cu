// Prefill GEMM on the 5th-generation tensor cores: Y[M tokens][N] = X[M][K] * W[N][K]^T with W a
// quantised GGUF matrix (any supported format) and M >= 17 (smaller M uses the GEMV kernels).
// Replaces the batched-prefill use of mul_mat_weight (src/cli/main.cpp:3256-3267, M <= 256 chunks).
//
// Computed as D^T: weight rows are the UMMA "M" operand (one or two 128-row tiles per CTA), tokens
// the "N" operand (up to 256 per CTA); the accumulators D[128 rows][tokens] live in tensor memory
// (TMEM, fp32).  Operands are fp16: the quantised formats carry fp16 block scales, so Q8_0 / Q4_0
// weights are reproduced exactly and K-quant sub-block scales lose 2^-12; activations are rounded to
// fp16 once (clamped to the finite range).  Warp roles, K step 64, ring of `stages` stages:
//   * warps 0-15 (dequant): read the quantised fragments with 128-bit loads, expand them with byte
//     permutes + packed half arithmetic (integer -> fp16 through the 0x6400 | q trick, exact), scale,
//     and store the 128 x 64 tiles into shared memory in the K-major 128-byte-swizzled layout
//     tcgen05.mma reads; fence.proxy.async, then one arrive per warp on the stage's `full` barrier;
//   * warp 17 lane 0 (activation producer): one cp.async.bulk per stage brings the token tile, which
//     x_prep_kernel wrote once per call already in the swizzled tile image (RMS norm fused there);
//   * warp 16 lane 0 (MMA issuer): waits for both, issues four tcgen05.mma (K = 16) per weight tile
//     accumulating in TMEM, and tcgen05.commit to the stage's `free` barrier, so the tensor cores run
//     stage s while the other warps fill the next stages.
// Inside every 32-run of K both operands use the same permutation (position 8t + 4h + i holds
// element 16h + 4t + i): a dot product does not depend on the order of its terms, and this order is
// the one in which the row-group-major Q4_K / Q6_K fragments deliver 16-byte chunks.
// Epilogue: tcgen05.ld brings the accumulators to registers (one weight row per lane); bias /
// residual / SwiGLU are applied and 32 lanes store 32 consecutive n of one token.
// No cluster launch is used and every copy targets one CTA.  Every mbarrier wait is bounded.
#include <cuda_fp16.h>

#include <stdio.h>
#include <stdlib.h>

#include <algorithm>

#include "ggb_internal.h"

namespace ggb {

namespace {

constexpr int kBK = 64;                // K per pipeline step (128 bytes of fp16: one swizzle row)
constexpr int kDequantWarps = 16;
constexpr int kThreadsG = (kDequantWarps + 2) * 32;      // dequant warps + MMA warp + producer warp
constexpr int kMaxStagesG = 8;
constexpr uint32_t kSpin = 1u << 17;
enum : int { F_GEN = 0, F_Q4K = 1, F_Q6K = 2, F_Q80 = 3, F_Q40 = 4, F_IQ4NL = 5, F_IQ4XS = 6 };

__device__ __forceinline__ uint32_t s_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(s_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err) {
    for (uint32_t i = 0; i < kSpin; ++i)
        if (mbar_try(bar, parity)) return true;
    atomicExch(err, 4);
    return false;
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(s_u32(dst)), "l"(src), "r"(bytes), "r"(s_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor of a K-major 16-bit tile whose rows are 128 bytes, swizzled in
// 8-row / 1024-byte atoms (tile base 1024-byte aligned): bits 0-13 address / 16, bits 16-29 leading
// byte offset / 16 (unused for swizzled K-major, set to 1), bits 32-45 stride between 8-row groups / 16
// (1024 B -> 64), bits 46-47 descriptor version 1 (sm_100), bits 61-63 swizzle mode 2 (128 bytes).
// The MMA thread keeps the constant high word (0x40004040) and advances the low word.
// Instruction descriptor, kind::f16: D fp32 (bits 4-5 = 1), A and B fp16 (format 0), both K-major,
// N / 8 in bits 17-22, M / 16 in bits 24-28.
__device__ __forceinline__ uint32_t umma_idesc(int M, int N) {
    return (1u << 4) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

struct GemmArgs {
    PackedW w, w2;                // w2: second matrix of the fused gate/up pair (dual)
    const __half* xb;             // activation tile images, see x_prep_kernel
    float* y;                     // [M][ldc]
    const float* bias;
    const float* resid;
    int M, K, ldc, epi, dual;
    int tn;                       // tokens per CTA tile (multiple of 64, <= 256)
    int tmem_cols;                // power of two >= accumulator columns, >= 32
    int stages;
    int steps_per_split;          // K steps per CTA (= K / 64 without split-K)
    float* ws;                    // split-K partial sums, nullptr without split-K
    __half* y_img;                // dual only: write silu(gate) * up as the fp16 tile image of the next GEMM (K = N) instead of y
    int* err;
};

// byte offset of 16-byte chunk c (0..7) of row r inside a K-major 128-byte-swizzled tile
__host__ __device__ __forceinline__ uint32_t swz_off(int r, int c) { return static_cast<uint32_t>(r) * 128u + (static_cast<uint32_t>(c ^ (r & 7)) << 4); }
// Byte offset, inside an activation image with n_steps K steps, of the 8 KB piece that holds the 64 tokens
// starting at `tok` (a multiple of 64) of K step ks: [256-token block][K step][4 pieces of 64 tokens], so
// that a token tile of 64 / 128 / 256 tokens (aligned to its size) is one contiguous range per K step.
__host__ __device__ __forceinline__ size_t img_piece(int tok, int ks, int n_steps) {
    return ((static_cast<size_t>(tok >> 8) * n_steps + ks) * 4 + ((tok >> 6) & 3)) * 8192;
}
// element of a 64-wide K step held by slot e (0..7) of chunk c (0..7)
__host__ __device__ __forceinline__ int perm_k(int c, int e) { return 32 * (c >> 2) + 16 * (e >> 2) + 4 * (c & 3) + (e & 3); }

// ---- activations: fp32 -> fp16 tile images with the fused RMS norm -------------------------------
// out[256-token block][k_step][4 x (64 rows x 128 B)]: each 8 KB piece is exactly the shared-memory image
// of 64 token rows of one pipeline step (swizzled, K permuted), and the pieces of a token tile of 64,
// 128 or 256 tokens are adjacent, so the GEMM fetches its tile with one bulk copy whatever the tile
// size.  Rows >= M are zero (they only feed output columns nobody stores).  v = sum(x^2)/K + eps, y = x * (1/sqrt(v)) * gamma (src/backends/cpu_ref/cpu_ref.cpp:139-156).
__global__ void x_prep_kernel(const float* __restrict__ x, int lda, int M, int K, const float* __restrict__ gamma, float eps,
                              __half* __restrict__ out) {
    __shared__ float red[32];
    pdl_wait();          // x comes from the previous kernel; the image may still be read by the GEMM before it
    pdl_trigger();       // the GEMM may start: its dequant warps need nothing from this kernel
    const int row = blockIdx.x, r = row & 63;
    const int n_steps = K / kBK;
    uint8_t* img = reinterpret_cast<uint8_t*>(out);
    const bool live = row < M;
    const float* xr = x + static_cast<size_t>(live ? row : 0) * lda;
    float inv = 1.0f;
    if (gamma && live) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < K; i += blockDim.x) ss += xr[i] * xr[i];
#pragma unroll
        for (int of = 16; of > 0; of >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, of);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.0f;
        for (int i = 0; i < (blockDim.x >> 5); ++i) tot += red[i];
        inv = 1.0f / sqrtf(tot / static_cast<float>(K) + eps);
    }
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {          // one 16-byte chunk per iteration
        const int ks = i >> 3, c = i & 7;
        uint32_t p[4] = {0u, 0u, 0u, 0u};
        if (live) {
#pragma unroll
            for (int hv = 0; hv < 2; ++hv) {
                const int k = ks * kBK + perm_k(c, 4 * hv);
                float4 v = *reinterpret_cast<const float4*>(xr + k);
                if (gamma) {
                    const float4 gm = *reinterpret_cast<const float4*>(gamma + k);
                    v.x = v.x * inv * gm.x; v.y = v.y * inv * gm.y; v.z = v.z * inv * gm.z; v.w = v.w * inv * gm.w;
                }
                const float lim = 65504.0f;
                const __half2 a = __floats2half2_rn(fminf(fmaxf(v.x, -lim), lim), fminf(fmaxf(v.y, -lim), lim));
                const __half2 b = __floats2half2_rn(fminf(fmaxf(v.z, -lim), lim), fminf(fmaxf(v.w, -lim), lim));
                p[2 * hv] = *reinterpret_cast<const uint32_t*>(&a);
                p[2 * hv + 1] = *reinterpret_cast<const uint32_t*>(&b);
            }
        }
        *reinterpret_cast<uint4*>(img + img_piece(row & ~63, ks, n_steps) + swz_off(r, c)) = make_uint4(p[0], p[1], p[2], p[3]);
    }
}

// ---- dequantisation into fp16 --------------------------------------------------------------------
__device__ __forceinline__ __half2 as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ uint32_t pack_h2(float a, float b) { return as_u32(__floats2half2_rn(a, b)); }
// The four bytes of n (each <= 255) as exact halves minus `bias`: 0x6400 | b is the half 1024 + b.
__device__ __forceinline__ void bytes_to_half(uint32_t n, __half2 bias, __half2& p01, __half2& p23) {
    p01 = __hsub2(as_h2(__byte_perm(n, 0x64646464u, 0x4140)), bias);
    p23 = __hsub2(as_h2(__byte_perm(n, 0x64646464u, 0x4342)), bias);
}

// Q4_K, row-group-major layout.  Table row (16 words): words 2 sb, 2 sb + 1 = half2(d * sc_sb) x 2, half2(-dmin * m_sb) x 2.
__device__ __forceinline__ void q4k_table_words(const uint4 h, uint32_t* dst) {     // h: the row's 16-byte block header
    const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(h.x & 0xFFFFu)));
    const float dmin = __half2float(__ushort_as_half(static_cast<unsigned short>(h.x >> 16)));
    auto B = [&](int i) -> int { const uint32_t wd = i < 4 ? h.y : (i < 8 ? h.z : h.w); return static_cast<int>((wd >> (8 * (i & 3))) & 0xFFu); };
#pragma unroll
    for (int sb = 0; sb < 8; ++sb) {
        int sc, mn;
        if (sb < 4) { sc = B(sb) & 63; mn = B(sb + 4) & 63; }
        else { sc = (B(sb + 4) & 15) | ((B(sb - 4) >> 6) << 4); mn = (B(sb + 4) >> 4) | ((B(sb) >> 6) << 4); }
        const float sv = d * static_cast<float>(sc), ov = -(dmin * static_cast<float>(mn));
        dst[2 * sb] = pack_h2(sv, sv);
        dst[2 * sb + 1] = pack_h2(ov, ov);
    }
}
// one 16-byte chunk: slots 0-3 from the nibbles in na, 4-7 from nb_; w = q * ss + oo
__device__ __forceinline__ uint4 q4k_chunk(uint32_t na, uint32_t nb_, const __half2 ss, const __half2 oo) {
    const __half2 k1024 = as_h2(0x64006400u);
    __half2 p0, p1, p2, p3;
    bytes_to_half(na, k1024, p0, p1);
    bytes_to_half(nb_, k1024, p2, p3);
    return make_uint4(as_u32(__hfma2(p0, ss, oo)), as_u32(__hfma2(p1, ss, oo)), as_u32(__hfma2(p2, ss, oo)), as_u32(__hfma2(p3, ss, oo)));
}

// Q6_K, row-group-major layout.  Table row (16 words): word i = half2(d * sc_i) x 2, i = 0..15.
__device__ __forceinline__ void q6k_table_words(const uint4 sc, const float d, uint32_t* dst) {     // sc: the row's 16 int8 scales
    const uint32_t wd[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int a = static_cast<int8_t>((wd[i >> 1] >> (16 * (i & 1))) & 0xFFu), c = static_cast<int8_t>((wd[i >> 1] >> (16 * (i & 1) + 8)) & 0xFFu);
        dst[2 * i] = pack_h2(d * static_cast<float>(a), d * static_cast<float>(a));
        dst[2 * i + 1] = pack_h2(d * static_cast<float>(c), d * static_cast<float>(c));
    }
}
// one chunk: slots 0-3 = 6-bit values (nib0 | hb0 << 4) with scale s0, slots 4-7 = (nib1 | hb1 << 4) with s1
__device__ __forceinline__ uint4 q6k_chunk(uint32_t nib0, uint32_t hb0, uint32_t nib1, uint32_t hb1, const __half2 s0, const __half2 s1) {
    const __half2 k1056 = as_h2(0x64206420u);     // 1024 + 32
    __half2 p0, p1, p2, p3;
    bytes_to_half(nib0 + (hb0 << 4), k1056, p0, p1);
    bytes_to_half(nib1 + (hb1 << 4), k1056, p2, p3);
    return make_uint4(as_u32(__hmul2(p0, s0)), as_u32(__hmul2(p1, s0)), as_u32(__hmul2(p2, s1)), as_u32(__hmul2(p3, s1)));
}
// Q8_0 (stream layout): signed bytes wa (slots 0-3) and wb (4-7) times the block's fp16 scale -- exact up to the final rounding
__device__ __forceinline__ uint4 q80_chunk(uint32_t wa, uint32_t wb, __half2 dd) {
    const __half2 k1152 = as_h2(0x64806480u);     // 1024 + 128
    __half2 p0, p1, p2, p3;
    bytes_to_half(wa ^ 0x80808080u, k1152, p0, p1);
    bytes_to_half(wb ^ 0x80808080u, k1152, p2, p3);
    return make_uint4(as_u32(__hmul2(p0, dd)), as_u32(__hmul2(p1, dd)), as_u32(__hmul2(p2, dd)), as_u32(__hmul2(p3, dd)));
}
// Q4_0 (stream layout): the four bytes of wq hold elements 4 cc .. 4 cc + 3 (low nibbles, slots 0-3) and 16 + 4 cc ..
// (high nibbles, slots 4-7) of the block; (q - 8) * d is exact in fp32, so the one fp16 rounding is the only one.
__device__ __forceinline__ uint4 q40_chunk(uint32_t wq, __half2 dd) {
    const __half2 k1032 = as_h2(0x64086408u);     // 1024 + 8
    __half2 p0, p1, p2, p3;
    bytes_to_half(wq & 0x0F0F0F0Fu, k1032, p0, p1);
    bytes_to_half((wq >> 4) & 0x0F0F0F0Fu, k1032, p2, p3);
    return make_uint4(as_u32(__hmul2(p0, dd)), as_u32(__hmul2(p1, dd)), as_u32(__hmul2(p2, dd)), as_u32(__hmul2(p3, dd)));
}
// The non-linear 4-bit codebook (src/quant/iq4_nl.cpp:16-18) as a byte-permute: four indices (one per byte of idx,
// each < 16) -> their four signed code bytes.  The 16 codes sit in four registers; bit 3 of an index picks the pair.
__device__ __forceinline__ uint32_t iq4_codes(uint32_t idx) {
    const uint32_t x = idx | (idx >> 4);
    const uint32_t p = __byte_perm(x, 0u, 0x4420);                     // the four nibbles in the low 16 bits
    const uint32_t sel = p & 0x7777u;
    const uint32_t lo = __byte_perm(0xBFAD9881u, 0xF6EADDCFu, sel);    // -127 -104 -83 -65 | -49 -35 -22 -10
    const uint32_t hi = __byte_perm(0x26190D01u, 0x71594535u, sel);    //    1   13  25  38 |  53  69  89 113
    return __byte_perm(lo, hi, 0x3210u | ((p & 0x8888u) >> 1));
}
// IQ4_NL / IQ4_XS (stream layout): codes of the low nibbles (slots 0-3) and high nibbles (4-7) times the scale.
// IQ4_NL: dd = the block's fp16 d, code * d exact before the one rounding.  IQ4_XS: dd = d * (ls - 32) rounded to fp16.
__device__ __forceinline__ uint4 iq4_chunk(uint32_t wq, __half2 dd) {
    return q80_chunk(iq4_codes(wq & 0x0F0F0F0Fu), iq4_codes((wq >> 4) & 0x0F0F0F0Fu), dd);
}
// Store chunks t (lo) and 4 + t (hi) of row r.  A quarter warp (lanes g, g + 1; t = 0..3) stores in one
// wavefront when its eight 16-byte slots differ: even g writes lo first, odd g hi first.
__device__ __forceinline__ void store_pair(uint8_t* tile, int r, int t, int odd, const uint4 lo, const uint4 hi) {
    const uint4 first = odd ? hi : lo, second = odd ? lo : hi;
    *reinterpret_cast<uint4*>(tile + swz_off(r, t + 4 * odd)) = first;
    *reinterpret_cast<uint4*>(tile + swz_off(r, t + 4 * (odd ^ 1))) = second;
}
// any format: exact fp32 decode (the decoder the dequant kernel uses), one rounding to fp16
__device__ __forceinline__ uint4 generic_chunk(const PackedW& w, int64_t row, int k0, int c, int block_elems) {
    uint32_t p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float v[2] = {0.0f, 0.0f};
        if (row < w.N) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int k = k0 + perm_k(c, 2 * i + u);
                v[u] = block_elems == 1 ? decode_elem(w, row * w.nb + k, 0) : decode_elem(w, row * w.nb + k / block_elems, k % block_elems);
            }
        }
        p[i] = pack_h2(v[0], v[1]);
    }
    return make_uint4(p[0], p[1], p[2], p[3]);
}

// ---- the GEMM --------------------------------------------------------------------------------------
// RT = weight tiles of 128 rows per CTA.  Non-dual: tile i covers rows n0 + 128 i of w.  Dual (RT == 2):
// tile 0 = rows n0.. of w (gate), tile 1 = the same rows of w2 (up); the epilogue combines them.
// Dynamic shared memory (1024-byte aligned): stages x RT weight tiles of 16 KB, stages token tiles of tn x 128 B,
// then the scale table 2 x 128 rows x 64 B (Q4_K / Q6_K; each warp owns the rows it fills).
// 16 dequant warps, warp w on row group w % 8 (16 rows): with RT == 2 warp w fills tile w / 8 at every
// step; with RT == 1 the warps form two sets (w / 8) that fill alternate steps, so that one set's
// load / convert / fence / arrive chain overlaps the other's.  Warp 16 issues the MMAs, warp 17 the
// activation copies.
template <int FMT, int RT>
__global__ void __launch_bounds__(kThreadsG, 1) gemm_tc_kernel(const GemmArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStagesG], free_bar[kMaxStagesG], done_bar;
    __shared__ uint32_t tmem_base_s;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // One ring of S stages.  Stage s = weight tiles at smem + s * a_bytes and the token tile at
    // smem_b + s * b_bytes.  full_bar[s] completes when the stage's dequant warps have arrived AND the
    // activation copy's bytes have landed (one wait for the MMA thread); free_bar[s] by tcgen05.commit.
    const int S = a.stages;
    const int b_bytes = a.tn * 128;
    constexpr int a_bytes = RT * 16384;
    constexpr int kFillWarps = RT == 2 ? kDequantWarps : kDequantWarps / 2;      // warps that fill one stage
    uint8_t* smem_b = smem + static_cast<size_t>(S) * a_bytes;
    uint32_t* table = reinterpret_cast<uint32_t*>(smem_b + static_cast<size_t>(S) * b_bytes);      // [2][128][16]
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * (a.dual ? 128 : 128 * RT);
    const int n_steps = a.K / kBK;
    // split-K: this CTA covers K steps [kw0, kw1) (a multiple of 4 steps, so K-quant blocks stay whole)
    const int kw0 = blockIdx.z * a.steps_per_split, kw1 = kw0 + a.steps_per_split;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full_bar[s], kFillWarps + 1); mbar_init(&free_bar[s], 1); }
        mbar_init(&done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kDequantWarps) {       // the MMA warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_u32(&tmem_base_s)), "r"(static_cast<uint32_t>(a.tmem_cols)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_s;
    bool ok = true;

    if (warp == kDequantWarps + 1) {
        // ---------------- activation producer ----------------
        if (lane == 0) {
            const uint8_t* src = reinterpret_cast<const uint8_t*>(a.xb);
            const int tok0 = blockIdx.y * a.tn;
            int s = 0; uint32_t par = 1;          // parity of the `free` phase that releases the stage (first round: none)
            pdl_wait();                           // the activation image is the predecessor's output
            for (int ks = kw0; ks < kw1; ++ks) {
                if (ks - kw0 >= S && ok) ok = mbar_wait(&free_bar[s], par, a.err);
                mbar_expect_tx(&full_bar[s], static_cast<uint32_t>(b_bytes));
                bulk_g2s(smem_b + static_cast<size_t>(s) * b_bytes, src + img_piece(tok0, ks, n_steps), static_cast<uint32_t>(b_bytes), &full_bar[s]);
                if (++s == S) { s = 0; par ^= 1; }
            }
        }
    } else if (warp == kDequantWarps) {
        // ---------------- MMA issuer ----------------
        // This one thread's instruction chain paces the whole CTA (its warp shares a scheduler with
        // dequant warps), so the loop is kept to one wait, the MMAs and one commit: descriptors are a
        // constant high word and a low word that advances by a fixed amount per stage.
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(128, a.tn);
            const uint64_t desc_hi = static_cast<uint64_t>(0x40004040u) << 32;       // stride 1024 B, version 1, 128-byte swizzle
            const uint32_t a_lo0 = ((s_u32(smem) & 0x3FFFFu) >> 4) | 0x10000u, b_lo0 = ((s_u32(smem_b) & 0x3FFFFu) >> 4) | 0x10000u;
            const uint32_t a_step = a_bytes >> 4, b_step = static_cast<uint32_t>(b_bytes) >> 4;
            uint32_t a_lo = a_lo0, b_lo = b_lo0, accumulate = 0u;
            int s = 0; uint32_t par = 0;
            for (int ks = kw0; ks < kw1; ++ks) {
                ok = mbar_wait(&full_bar[s], par, a.err);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int i = 0; i < RT; ++i) {
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; ++kk)      // +32 bytes along K per instruction, +16 KB per weight tile
                        umma_f16(tmem_d + i * a.tn, desc_hi | (a_lo + i * 1024 + 2 * kk), desc_hi | (b_lo + 2 * kk), idesc, (kk == 0) ? accumulate : 1u);
                }
                umma_commit(&free_bar[s]);
                accumulate = 1u;
                a_lo += a_step; b_lo += b_step;
                if (++s == S) { s = 0; par ^= 1; a_lo = a_lo0; b_lo = b_lo0; }
            }
            if (ok) umma_commit(&done_bar);
        }
        pdl_trigger();                            // main loop issued: the next kernel in the stream may be scheduled
    } else {
        // ---------------- dequant warps ----------------
        // Fragments are fetched two steps ahead into three register sets that rotate by name (DRAM
        // latency is longer than one step); K-quant sub-block scales are expanded once per 256-block
        // into the warp's own rows of the scale table.
        const int g = lane >> 2, t = lane & 3;
        const int grp_w = warp & 7;
        const int set = warp >> 3;                       // RT == 2: weight tile; RT == 1: which alternate steps
        const int tile = RT == 2 ? set : 0;
        const int stride = RT == 2 ? 1 : 2, ks_first = RT == 2 ? 0 : set;      // ks_first: relative to kw0
        const PackedW& w = (a.dual && tile == 1) ? a.w2 : a.w;
        const int64_t row0 = a.dual ? n0 : n0 + 128 * tile;
        const FormatInfo fi = format_info(a.w.type);
        constexpr int NQ = FMT == F_Q6K ? 3 : (FMT == F_Q80 ? 2 : 1);
        constexpr bool ROWF = FMT == F_Q80 || FMT == F_Q40 || FMT == F_IQ4NL || FMT == F_IQ4XS;     // thread = (row, 32-block of the step)
        struct Frag { uint4 v[NQ]; uint32_t d, e; };
        struct Hdr { uint4 v; float d; };
        // per-thread stream positions
        const int64_t grp = (row0 >> 4) + grp_w;
        const bool grp_live = grp < ((w.N + 15) >> 4);
        const uint8_t* q_base = nullptr;      // Q4_K: qs fragments; Q6_K: ql fragments; row formats: qs of this thread's row
        const uint8_t* q_base2 = nullptr;     // Q6_K: qh fragments; row formats: block scales / headers
        int q80_r = 0, q80_hh = 0;
        bool q80_live = false;
        if (FMT == F_Q4K) q_base = w.s[1] + (grp * w.nb * 4 * 32 + lane) * 16;
        if (FMT == F_Q6K) { q_base = w.s[0] + (grp * w.nb * 4 * 32 + lane) * 16; q_base2 = w.s[1] + (grp * w.nb * 2 * 32 + lane) * 16; }
        if (ROWF) {
            const int lt = tid & 255;
            q80_r = lt >> 1; q80_hh = lt & 1;
            const int64_t row = row0 + q80_r;
            q80_live = row < w.N;
            if (FMT == F_Q80) { q_base = w.s[1] + (row * w.nb + q80_hh) * 32; q_base2 = w.s[0] + (row * w.nb + q80_hh) * 2; }
            else if (FMT == F_IQ4XS) { q_base = w.s[1] + row * w.nb * 128 + q80_hh * 16; q_base2 = w.s[0] + row * w.nb * 8; }
            else { q_base = w.s[1] + (row * w.nb + q80_hh) * 16; q_base2 = w.s[0] + (row * w.nb + q80_hh) * 2; }
        }
        auto load_frag = [&](int ks, Frag& f) {
#pragma unroll
            for (int j = 0; j < NQ; ++j) f.v[j] = make_uint4(0u, 0u, 0u, 0u);
            f.d = 0u; f.e = 0u;
            if (FMT == F_Q4K) {
                if (grp_live) f.v[0] = __ldg(reinterpret_cast<const uint4*>(q_base + static_cast<size_t>(ks) * 512));
            } else if (FMT == F_Q6K) {
                if (grp_live) {
                    f.v[0] = __ldg(reinterpret_cast<const uint4*>(q_base + static_cast<size_t>(ks & ~1) * 512));
                    f.v[1] = __ldg(reinterpret_cast<const uint4*>(q_base + static_cast<size_t>((ks & ~1) + 1) * 512));
                    f.v[NQ - 1] = __ldg(reinterpret_cast<const uint4*>(q_base2 + static_cast<size_t>(ks >> 1) * 512));
                }
            } else if (FMT == F_Q80) {
                if (q80_live) {
                    const uint8_t* p = q_base + static_cast<size_t>(ks) * 64;
                    f.v[0] = __ldg(reinterpret_cast<const uint4*>(p));
                    f.v[NQ - 1] = __ldg(reinterpret_cast<const uint4*>(p + 16));
                    f.d = __ldg(reinterpret_cast<const unsigned short*>(q_base2 + static_cast<size_t>(ks) * 4));
                }
            } else if (FMT == F_Q40 || FMT == F_IQ4NL) {
                if (q80_live) {
                    f.v[0] = __ldg(reinterpret_cast<const uint4*>(q_base + static_cast<size_t>(ks) * 32));
                    f.d = __ldg(reinterpret_cast<const unsigned short*>(q_base2 + static_cast<size_t>(ks) * 4));
                }
            } else if (FMT == F_IQ4XS) {
                if (q80_live) {      // the 256-block's 8-byte header: d | scales_h, scales_l[4]
                    f.v[0] = __ldg(reinterpret_cast<const uint4*>(q_base + static_cast<size_t>(ks) * 32));
                    const uint2 h = __ldg(reinterpret_cast<const uint2*>(q_base2 + static_cast<size_t>(ks >> 2) * 8));
                    f.d = h.x; f.e = h.y;
                }
            }
        };
        // K-quant header of this lane's table row (row r16 of the group), block b
        const int hdr_lanes = 16;
        const int r16 = lane & 15;
        auto load_hdr = [&](int b) -> Hdr {
            Hdr h; h.v = make_uint4(0u, 0u, 0u, 0u); h.d = 0.0f;
            if ((FMT == F_Q4K || FMT == F_Q6K) && lane < hdr_lanes && b < w.nb && grp_live) {
                const int64_t slot = (grp * w.nb + b) * 16 + r16;
                if (FMT == F_Q4K) h.v = __ldg(reinterpret_cast<const uint4*>(w.s[0] + slot * 16));
                else { h.v = __ldg(reinterpret_cast<const uint4*>(w.s[2] + slot * 16)); h.d = ld_f16(w.s[3] + slot * 2); }
            }
            return h;
        };
        uint32_t* tb = table + set * 128 * 16;          // this warp set's own copy of the scale table
        uint8_t* stage_ptr = smem + tile * 16384;
        int s_cur = ks_first; uint32_t par_free = 1;
        Frag f0, f1, f2;
        Hdr h0 = load_hdr(kw0 >> 2), h1 = load_hdr((kw0 >> 2) + 1);
        if (kw0 + ks_first < kw1) load_frag(kw0 + ks_first, f0);
        if (kw0 + ks_first + stride < kw1) load_frag(kw0 + ks_first + stride, f1);
        // one pipeline step: fetch the fragments two of this warp's steps ahead into `ahead`, fill stage s_cur from `cur`
        auto step = [&](const int ks, const Frag& cur, Frag& ahead) {
            uint8_t* At = stage_ptr + static_cast<size_t>(s_cur) * a_bytes;
            if (FMT != F_GEN && ks + 2 * stride < kw1) load_frag(ks + 2 * stride, ahead);
            if ((FMT == F_Q4K || FMT == F_Q6K) && (ks & 3) == ks_first) {
                // the previous block's readers are past their __syncwarp; expand this block's scales
                if (lane < hdr_lanes) {
                    uint32_t* dst = tb + (grp_w * 16 + r16) * 16;
                    if (FMT == F_Q4K) q4k_table_words(h0.v, dst); else q6k_table_words(h0.v, h0.d, dst);
                }
                h0 = h1;
                h1 = load_hdr((ks >> 2) + 2);
                __syncwarp();
            }
            if (ks - kw0 >= S && ok) ok = mbar_wait(&free_bar[s_cur], par_free, a.err);
            if (FMT == F_Q4K || FMT == F_Q6K) {
#pragma unroll
                for (int hi = 0; hi < 2; ++hi) {                       // 0: row g, 1: row g + 8
                    const int r = grp_w * 16 + g + 8 * hi;
                    const uint4 e = *reinterpret_cast<const uint4*>(tb + r * 16 + 4 * (ks & 3));
                    if (FMT == F_Q4K) {
                        const uint32_t wa = hi ? cur.v[0].y : cur.v[0].x, wb = hi ? cur.v[0].w : cur.v[0].z;
                        store_pair(At, r, t, g & 1, q4k_chunk(wa & 0x0F0F0F0Fu, wb & 0x0F0F0F0Fu, as_h2(e.x), as_h2(e.y)),
                                   q4k_chunk((wa >> 4) & 0x0F0F0F0Fu, (wb >> 4) & 0x0F0F0F0Fu, as_h2(e.z), as_h2(e.w)));
                    } else {
                        const uint4 c0 = cur.v[0], c1 = cur.v[1], qh = cur.v[NQ - 1];
                        const uint32_t a0 = hi ? c0.z : c0.x, b0 = hi ? c0.w : c0.y;      // c = 0: ql_a, ql_b
                        const uint32_t a1 = hi ? c1.z : c1.x, b1 = hi ? c1.w : c1.y;      // c = 1
                        const uint32_t q0 = hi ? qh.y : qh.x, q1 = hi ? qh.w : qh.z;      // qh of c = 0, 1
                        const int sh = 4 * (ks & 1);
                        store_pair(At, r, t, g & 1,
                                   q6k_chunk((a0 >> sh) & 0x0F0F0F0Fu, (q0 >> sh) & 0x03030303u, (a1 >> sh) & 0x0F0F0F0Fu, (q1 >> sh) & 0x03030303u, as_h2(e.x), as_h2(e.y)),
                                   q6k_chunk((b0 >> sh) & 0x0F0F0F0Fu, (q0 >> (sh + 2)) & 0x03030303u, (b1 >> sh) & 0x0F0F0F0Fu, (q1 >> (sh + 2)) & 0x03030303u, as_h2(e.z), as_h2(e.w)));
                    }
                }
            } else if (FMT == F_Q80) {
                const uint4 lo = cur.v[0], hi4 = cur.v[NQ - 1];
                const __half2 dd = __half2half2(__ushort_as_half(static_cast<unsigned short>(cur.d)));
                const int c0 = 4 * q80_hh;
                *reinterpret_cast<uint4*>(At + swz_off(q80_r, c0 + 0)) = q80_chunk(lo.x, hi4.x, dd);
                *reinterpret_cast<uint4*>(At + swz_off(q80_r, c0 + 1)) = q80_chunk(lo.y, hi4.y, dd);
                *reinterpret_cast<uint4*>(At + swz_off(q80_r, c0 + 2)) = q80_chunk(lo.z, hi4.z, dd);
                *reinterpret_cast<uint4*>(At + swz_off(q80_r, c0 + 3)) = q80_chunk(lo.w, hi4.w, dd);
            } else if (FMT == F_Q40 || FMT == F_IQ4NL || FMT == F_IQ4XS) {
                const uint4 q = cur.v[0];
                __half2 dd;
                if (FMT == F_IQ4XS) {
                    const int ib = 2 * (ks & 3) + q80_hh;
                    const int ls = static_cast<int>(((cur.e >> (4 * ib)) & 15u) | (((cur.d >> (16 + 2 * ib)) & 3u) << 4));
                    dd = __float2half2_rn(__half2float(__ushort_as_half(static_cast<unsigned short>(cur.d & 0xFFFFu))) * static_cast<float>(ls - 32));
                } else {
                    dd = __half2half2(__ushort_as_half(static_cast<unsigned short>(cur.d)));
                }
                const int c0 = 4 * q80_hh;
                if (FMT == F_Q40) {
                    *reinterpret_cast<uint4*>(At + swz_off(q80_r, c0 + 0)) = q40_chunk(q.x, dd);
                    *reinterpret_cast<uint4*>(At + swz_off(q80_r, c0 + 1)) = q40_chunk(q.y, dd);
                    *reinterpret_cast<uint4*>(At + swz_off(q80_r, c0 + 2)) = q40_chunk(q.z, dd);
                    *reinterpret_cast<uint4*>(At + swz_off(q80_r, c0 + 3)) = q40_chunk(q.w, dd);
                } else {
                    *reinterpret_cast<uint4*>(At + swz_off(q80_r, c0 + 0)) = iq4_chunk(q.x, dd);
                    *reinterpret_cast<uint4*>(At + swz_off(q80_r, c0 + 1)) = iq4_chunk(q.y, dd);
                    *reinterpret_cast<uint4*>(At + swz_off(q80_r, c0 + 2)) = iq4_chunk(q.z, dd);
                    *reinterpret_cast<uint4*>(At + swz_off(q80_r, c0 + 3)) = iq4_chunk(q.w, dd);
                }
            } else {
                uint8_t* As = smem + static_cast<size_t>(s_cur) * a_bytes;
                for (int it = (RT == 2 ? tid : (tid & 255)); it < RT * 128 * 8; it += RT * 256) {
                    const int i = it >> 10, r = (it >> 3) & 127, c = it & 7;
                    *reinterpret_cast<uint4*>(As + i * 16384 + swz_off(r, c)) =
                        generic_chunk((a.dual && i == 1) ? a.w2 : a.w, (a.dual ? n0 : n0 + 128 * i) + r, ks * kBK, c, fi.block_elems);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy stores -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_bar[s_cur]);
            s_cur += stride;
            if (s_cur >= S) { s_cur -= S; par_free ^= 1; }
        };
        for (int ks = kw0 + ks_first; ks < kw1; ks += 3 * stride) {
            step(ks, f0, f2);
            if (ks + stride < kw1) step(ks + stride, f1, f0);
            if (ks + 2 * stride < kw1) step(ks + 2 * stride, f2, f1);
        }
        // ---------------- epilogue (the same 16 warps) ----------------
        pdl_trigger();
        if (ok) ok = mbar_wait(&done_bar, 0, a.err);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        pdl_wait();                               // first global write / residual read of this kernel
        if (ok) {
            const int q = warp & 3, part = warp >> 2;
            const int t0 = blockIdx.y * a.tn;
            // non-dual RT == 2: two warps per weight tile and lane quarter, each half the columns;
            // otherwise four warps per lane quarter, each a quarter of the columns
            const bool by_tile = (RT == 2 && !a.dual);
            const int tile_e = by_tile ? (part & 1) : 0;
            const int c_len = by_tile ? a.tn / 2 : a.tn / 4;
            const int c_begin = (by_tile ? (part >> 1) : part) * c_len;
            const int64_t n = n0 + 128 * tile_e + q * 32 + lane;
            for (int c0 = c_begin; c0 < c_begin + c_len; c0 += 16) {
                float v[16], v2[16];
                const uint32_t taddr = tmem_d + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(tile_e * a.tn + c0);
                tmem_ld16(taddr, v);
                if (a.dual) tmem_ld16(taddr + a.tn, v2);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int tok = t0 + c0 + i;
                    if (tok < a.M && n < a.w.N && a.ws) {
                        // split-K: bare partial sums [split][gate | up][M][N]; splitk_reduce_kernel applies the epilogue
                        const size_t plane = static_cast<size_t>(a.M) * a.w.N, o = static_cast<size_t>(tok) * a.w.N + n;
                        float* wsz = a.ws + static_cast<size_t>(blockIdx.z) * plane * (a.dual ? 2 : 1);
                        wsz[o] = v[i];
                        if (a.dual) wsz[plane + o] = v2[i];
                    } else if (tok < a.M && n < a.w.N) {
                        const size_t o = static_cast<size_t>(tok) * a.ldc + n;
                        float r = v[i];
                        if (a.dual) r = __fdividef(r, 1.0f + __expf(-r)) * v2[i];
                        else if (a.epi == EPI_ADD_BIAS) r += __ldg(a.bias + n);
                        else if (a.epi == EPI_RESIDUAL) r += a.resid[o];
                        if (a.y_img) {
                            // element (token tok, k = n) of an image with N / 64 steps; kl = 32 h + 16 hi + 4 t + i -> chunk 4 h + t, slot 4 hi + i
                            const int kl = static_cast<int>(n & 63), ch = ((kl >> 5) << 2) | ((kl >> 2) & 3), sl = (((kl >> 4) & 1) << 2) | (kl & 3);
                            uint8_t* img = reinterpret_cast<uint8_t*>(a.y_img) + img_piece(tok & ~63, static_cast<int>(n >> 6), static_cast<int>(a.w.N >> 6));
                            *reinterpret_cast<__half*>(img + swz_off(tok & 63, ch) + 2 * sl) = __float2half_rn(fminf(fmaxf(r, -65504.0f), 65504.0f));
                        } else a.y[o] = r;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kDequantWarps) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(static_cast<uint32_t>(a.tmem_cols)) : "memory");
    }
}

// Split-K tail: y = epilogue(sum over splits of the partial sums).  One thread per output element.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, int splits, int M, int64_t N, int dual, int epi,
                                     const float* __restrict__ bias, const float* resid, float* y, int ldc, __half* y_img) {
    pdl_wait();
    pdl_trigger();
    const size_t plane = static_cast<size_t>(M) * N;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < plane; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int tok = static_cast<int>(i / N);
        const int64_t n = static_cast<int64_t>(i - static_cast<size_t>(tok) * N);
        float g = 0.0f, u = 0.0f;
        for (int z = 0; z < splits; ++z) {
            const float* p = ws + static_cast<size_t>(z) * plane * (dual ? 2 : 1);
            g += p[i];
            if (dual) u += p[plane + i];
        }
        const size_t o = static_cast<size_t>(tok) * ldc + n;
        float r = g;
        if (dual) r = __fdividef(g, 1.0f + __expf(-g)) * u;
        else if (epi == EPI_ADD_BIAS) r += __ldg(bias + n);
        else if (epi == EPI_RESIDUAL) r += resid[o];
        if (y_img) {
            const int kl = static_cast<int>(n & 63), ch = ((kl >> 5) << 2) | ((kl >> 2) & 3), sl = (((kl >> 4) & 1) << 2) | (kl & 3);
            uint8_t* img = reinterpret_cast<uint8_t*>(y_img) + img_piece(tok & ~63, static_cast<int>(n >> 6), static_cast<int>(N >> 6));
            *reinterpret_cast<__half*>(img + swz_off(tok & 63, ch) + 2 * sl) = __float2half_rn(fminf(fmaxf(r, -65504.0f), 65504.0f));
        } else y[o] = r;
    }
}

template <int FMT, int RT>
int launch_one(Context* c, const GemmArgs& a, dim3 grid, size_t smem, cudaStream_t s) {
    const cudaError_t ea = ensure_dynamic_smem(c, gemm_tc_kernel<FMT, RT>, smem);
    if (ea != cudaSuccess) return cuda_status(c, ea, "gemm_tc attr");
    const cudaError_t e = launch_pdl(c, gemm_tc_kernel<FMT, RT>, grid, dim3(kThreadsG), smem, s, a);
    c->launches++;
    return cuda_status(c, e != cudaSuccess ? e : cudaGetLastError(), "gemm_tc launch");
}

// How many ways K is split when the (row tile x token tile) grid would leave most SMs idle: each CTA
// then takes a K window that is a whole number of 256-blocks and writes bare partial sums; a small
// kernel adds them and applies the epilogue.  1 = no split.
int k_splits(const GemvArgs& g, int tn) {
    const int64_t ctas = (g.w.N + 127) / 128 * ((g.M + tn - 1) / tn);
    const int n_steps = g.w.K / kBK;
    if (ctas >= 96 || n_steps % 4) return 1;
    int best = 1;
    for (int sp = 2; sp <= 16; ++sp)
        if (n_steps % (4 * sp) == 0 && n_steps / sp >= 16 && ctas * sp <= 160) best = sp;
    return best;
}
// tokens per CTA tile: a multiple of 64 (the epilogue reads the columns 16 at a time per warp), at most
// 256.  The largest tile whose grid (with split-K) covers about one CTA per SM; every token tile repeats
// the dequantisation of its weight rows, so bigger is cheaper.
int tile_tokens(const GemvArgs& g) {
    const int cap = std::min(256, (g.M + 63) / 64 * 64);
    const int64_t row_tiles = (g.w.N + 127) / 128;
    for (int tn = 256; tn > 64; tn >>= 1)
        if (tn <= cap && row_tiles * ((g.M + tn - 1) / tn) * k_splits(g, tn) >= 96) return tn;
    return std::min(cap, 64);
}

}  // namespace

size_t gemm_tc_ws_floats(const GemvArgs& g) {
    const int sp = k_splits(g, tile_tokens(g));
    return sp > 1 ? static_cast<size_t>(sp) * (g.epi == EPI_SWIGLU ? 2 : 1) * g.M * g.w.N : 0;
}
size_t gemm_tc_xb_elems(const GemvArgs& g) { return static_cast<size_t>((g.M + 255) / 256) * 256 * g.w.K; }

// Prefill GEMM.  Returns GGB_NOT_FOUND when the shape is not covered (caller falls back).
// d_xb_v: scratch for the fp16 activation tile images, at least gemm_tc_xb_elems(g) elements.
int launch_gemm_tc(Context* c, const GemvArgs& g, void* d_xb_v, size_t xb_elems, float* d_ws, size_t ws_floats, cudaStream_t s) {
    __half* d_xb = static_cast<__half*>(d_xb_v);
    const int K = g.w.K;
    const FormatInfo fi = format_info(g.w.type);
    if (!fi.block_elems || K % kBK || g.M < 1 || (!g.x && !g.x_img) || g.n_cat || g.attn_partial) return GGB_NOT_FOUND;
    if (g.y_img && (g.epi != EPI_SWIGLU || g.w.N % 64)) return GGB_NOT_FOUND;
    const bool dual = g.epi == EPI_SWIGLU;
    if (dual && g.w2.layout != g.w.layout) return GGB_NOT_FOUND;
    const int tn = tile_tokens(g);
    const int m_tiles = (g.M + tn - 1) / tn;
    if (!g.x_img && gemm_tc_xb_elems(g) > xb_elems) return GGB_NOT_FOUND;

    const int splits = k_splits(g, tn);
    if (splits > 1 && gemm_tc_ws_floats(g) > ws_floats) return GGB_NOT_FOUND;

    int fmt = F_GEN;
    if (g.w.type == T_Q4_K && g.w.layout == 1) fmt = F_Q4K;
    else if (g.w.type == T_Q6_K && g.w.layout == 1) fmt = F_Q6K;
    else if (g.w.type == T_Q8_0 && g.w.layout == 0) fmt = F_Q80;
    else if (g.w.type == T_Q4_0 && g.w.layout == 0) fmt = F_Q40;
    else if (g.w.type == T_IQ4_NL && g.w.layout == 0) fmt = F_IQ4NL;
    else if (g.w.type == T_IQ4_XS && g.w.layout == 0) fmt = F_IQ4XS;
    // two weight tiles per CTA halve the activation traffic per flop; one tile doubles the CTA count
    int rt = 2;
    if (!dual) {
        const int64_t ctas2 = (g.w.N + 255) / 256 * m_tiles * splits;
        if (g.w.N <= 128 || ctas2 < (c->sm_count * 3) / 4) rt = 1;
    }
    int cols = 32;
    while (cols < tn * rt) cols <<= 1;
    const size_t a_stage = static_cast<size_t>(rt) * 16384, b_stage = static_cast<size_t>(tn) * 128;
    const size_t table_bytes = static_cast<size_t>(2) * 128 * 64;      // one copy per weight tile (two tiles) or per warp set (one tile)
    const size_t budget = 227 * 1024 - 1024 - table_bytes - 2048;      // alignment slack, table, static barriers
    // (a shallower weight ring with a deeper, separate token ring measured slower than one ring)
    const int stages = static_cast<int>(std::min<size_t>(kMaxStagesG, budget / (a_stage + b_stage)));
    if (stages < 2) return GGB_NOT_FOUND;
    const size_t smem = stages * (a_stage + b_stage) + table_bytes + 1024;

    if (!g.x_img) {
        cudaError_t e = launch_pdl(c, x_prep_kernel, dim3(m_tiles * tn), dim3(256), 0, s, g.x, g.lda, g.M, K, g.gamma, g.eps, d_xb);
        c->launches++;
        if (e == cudaSuccess) e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_status(c, e, "x_prep");
    }

    GemmArgs a{};
    a.w = g.w; a.w2 = g.w2; a.xb = g.x_img ? static_cast<const __half*>(g.x_img) : d_xb; a.y = g.y; a.y_img = static_cast<__half*>(g.y_img); a.bias = g.bias; a.resid = g.resid;
    a.M = g.M; a.K = K; a.ldc = g.ldc; a.epi = g.epi; a.dual = dual ? 1 : 0; a.tn = tn; a.tmem_cols = cols; a.stages = stages; a.err = c->d_err;
    a.steps_per_split = K / kBK / splits; a.ws = splits > 1 ? d_ws : nullptr;
    dim3 grid(static_cast<unsigned>((g.w.N + (dual ? 128 : 128 * rt) - 1) / (dual ? 128 : 128 * rt)), static_cast<unsigned>(m_tiles), static_cast<unsigned>(splits));
    int st;
    switch (fmt * 2 + (rt - 1)) {
    case F_GEN * 2 + 0: st = launch_one<F_GEN, 1>(c, a, grid, smem, s); break;
    case F_GEN * 2 + 1: st = launch_one<F_GEN, 2>(c, a, grid, smem, s); break;
    case F_Q4K * 2 + 0: st = launch_one<F_Q4K, 1>(c, a, grid, smem, s); break;
    case F_Q4K * 2 + 1: st = launch_one<F_Q4K, 2>(c, a, grid, smem, s); break;
    case F_Q6K * 2 + 0: st = launch_one<F_Q6K, 1>(c, a, grid, smem, s); break;
    case F_Q6K * 2 + 1: st = launch_one<F_Q6K, 2>(c, a, grid, smem, s); break;
    case F_Q80 * 2 + 0: st = launch_one<F_Q80, 1>(c, a, grid, smem, s); break;
    case F_Q80 * 2 + 1: st = launch_one<F_Q80, 2>(c, a, grid, smem, s); break;
    case F_Q40 * 2 + 0: st = launch_one<F_Q40, 1>(c, a, grid, smem, s); break;
    case F_Q40 * 2 + 1: st = launch_one<F_Q40, 2>(c, a, grid, smem, s); break;
    case F_IQ4NL * 2 + 0: st = launch_one<F_IQ4NL, 1>(c, a, grid, smem, s); break;
    case F_IQ4NL * 2 + 1: st = launch_one<F_IQ4NL, 2>(c, a, grid, smem, s); break;
    case F_IQ4XS * 2 + 0: st = launch_one<F_IQ4XS, 1>(c, a, grid, smem, s); break;
    default: st = launch_one<F_IQ4XS, 2>(c, a, grid, smem, s); break;
    }
    if (st != GGB_OK || splits == 1) return st;
    const size_t elems = static_cast<size_t>(g.M) * g.w.N;
    const cudaError_t e = launch_pdl(c, splitk_reduce_kernel, dim3(static_cast<unsigned>(std::min<size_t>((elems + 255) / 256, 148 * 8))), dim3(256), 0, s,
                                     static_cast<const float*>(d_ws), splits, g.M, g.w.N, dual ? 1 : 0, g.epi, g.bias, g.resid, g.y, g.ldc, static_cast<__half*>(g.y_img));
    c->launches++;
    return cuda_status(c, e != cudaSuccess ? e : cudaGetLastError(), "gemm_tc split-K reduce");
}

}  // namespace ggb
