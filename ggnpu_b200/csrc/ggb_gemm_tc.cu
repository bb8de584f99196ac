// Prefill GEMM on the 5th-generation tensor cores: Y[M tokens][N] = X[M][K] * W[N][K]^T with W a
// quantised GGUF matrix (any supported format) and M >= 17 (smaller M uses the GEMV kernels).
// Replaces the batched-prefill use of mul_mat_weight (src/cli/main.cpp:3256-3267, M <= 256 chunks).
//
// Computed as D^T: the weight rows are the UMMA "M" operand (128 per CTA), the tokens the "N" operand
// (up to 256 per CTA), the accumulator D[128 rows][tokens] lives in tensor memory (TMEM, fp32).
// Per K step of 64:
//   * all 8 warps dequantise the CTA's 128 x 64 weight tile with the same exact fp32 decoder the
//     dequant kernel uses (decode_elem), round to bf16 and store it into shared memory in the K-major
//     128-byte-swizzled layout tcgen05.mma reads; they also copy the 64-wide bf16 activation slice
//     (prepared once per call by x_to_bf16_kernel, RMS norm fused) in the same layout;
//   * after fence.proxy.async + a CTA barrier one thread issues four tcgen05.mma (K = 16 each) that
//     accumulate into TMEM, then tcgen05.commit to the stage's mbarrier; the MMAs run asynchronously,
//     so the tensor cores work on stage s while the warps dequantise stage s^1.
// Epilogue: tcgen05.ld brings the accumulator to registers (one weight row per lane), bias / residual
// / SwiGLU are applied and rows are stored so that 32 lanes write 32 consecutive n of one token.
// No cluster launch and no multicast copy is used.  Every mbarrier wait is bounded.
#include <cuda_bf16.h>

#include "ggb_internal.h"

namespace ggb {

namespace {

constexpr int kTileN = 128;            // weight rows per CTA (UMMA M)
constexpr int kBK = 64;                // K per pipeline step (128 bytes of bf16: one swizzle row)
constexpr int kThreadsG = 256;
constexpr uint32_t kSpin = 1u << 17;

__device__ __forceinline__ uint32_t s_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_u32(bar)), "r"(count) : "memory");
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

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes, swizzled in
// 8-row / 1024-byte atoms (tile base 1024-byte aligned): start address, stride between 8-row groups
// 1024 bytes, descriptor version 1 (sm_100), swizzle mode 2 (128 bytes).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);          // bits 0-13: address / 16
    d |= static_cast<uint64_t>(1) << 16;                               // bits 16-29: leading byte offset / 16 (unused for swizzled K-major)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                       // bits 32-45: stride byte offset / 16
    d |= static_cast<uint64_t>(1) << 46;                               // bits 46-47: descriptor version
    d |= static_cast<uint64_t>(2) << 61;                               // bits 61-63: 128-byte swizzle
    return d;
}
// Instruction descriptor, kind::f16: D fp32, A and B bf16, both K-major, shape M x N.
__device__ __forceinline__ uint32_t umma_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                   "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
                   "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

struct GemmArgs {
    PackedW w, w2;                // w2: second matrix of the fused gate/up pair (dual)
    const __nv_bfloat16* xb;      // [M_pad][K] activations in bf16
    float* y;                     // [M][ldc]
    const float* bias;
    const float* resid;
    int M, K, ldc, epi, dual;
    int tn;                       // tokens per CTA tile (multiple of 16, <= 256)
    int tmem_cols;                // power of two >= tn * (dual ? 2 : 1), >= 32
    int* err;
};

// ---- activations: fp32 -> bf16 with the fused RMS norm ------------------------------------------
// One CTA per token row; rows M .. M_pad-1 are zero.  v = sum(x^2)/K + eps, y = x * (1/sqrt(v)) * gamma
// (src/backends/cpu_ref/cpu_ref.cpp:139-156), then round to nearest even bf16.
__global__ void x_to_bf16_kernel(const float* __restrict__ x, int lda, int M, int K, const float* __restrict__ gamma, float eps,
                                 __nv_bfloat16* __restrict__ out) {
    __shared__ float red[32];
    const int row = blockIdx.x;
    __nv_bfloat16* o = out + static_cast<size_t>(row) * K;
    if (row >= M) { for (int i = threadIdx.x; i < K; i += blockDim.x) o[i] = __float2bfloat16_rn(0.0f); return; }
    const float* xr = x + static_cast<size_t>(row) * lda;
    float inv = 1.0f;
    if (gamma) {
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
    for (int i = threadIdx.x; i < K; i += blockDim.x) o[i] = __float2bfloat16_rn(gamma ? xr[i] * inv * gamma[i] : xr[i]);
}

// byte offset of 16-byte chunk c (0..7) of row r inside a K-major 128-byte-swizzled tile
__device__ __forceinline__ uint32_t swz_off(int r, int c) { return static_cast<uint32_t>(r) * 128u + (static_cast<uint32_t>(c ^ (r & 7)) << 4); }

// Dequantise 8 consecutive weights k0..k0+7 of `row` to bf16 (exact fp32 decode, then one rounding).
__device__ __forceinline__ uint4 dequant8_bf16(const PackedW& w, int64_t row, int k0, int block_elems) {
    uint32_t p[4];
    const bool valid = row < w.N;
    const int64_t blk = row * w.nb + k0 / block_elems;
    const int j0 = k0 % block_elems;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float a = 0.0f, b = 0.0f;
        if (valid) {
            if (block_elems == 1) { a = decode_elem(w, row * w.nb + k0 + 2 * i, 0); b = decode_elem(w, row * w.nb + k0 + 2 * i + 1, 0); }
            else { a = decode_elem(w, blk, j0 + 2 * i); b = decode_elem(w, blk, j0 + 2 * i + 1); }
        }
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        p[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(p[0], p[1], p[2], p[3]);
}

// dynamic shared memory (1024-byte aligned): 2 stages x [A: 128 x 128 B][A2 (dual): 16 KB][B: tn x 128 B]
__global__ void __launch_bounds__(kThreadsG, 1) gemm_tc_kernel(const GemmArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t free_bar[2], done_bar;
    __shared__ uint32_t tmem_base_s;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int a_bytes = kTileN * 128, b_bytes = a.tn * 128;
    const int stage_bytes = a_bytes * (a.dual ? 2 : 1) + b_bytes;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kTileN;
    const int t0 = blockIdx.y * a.tn;
    const FormatInfo fi = format_info(a.w.type);

    if (tid == 0) {
        mbar_init(&free_bar[0], 1); mbar_init(&free_bar[1], 1); mbar_init(&done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {       // one warp allocates the accumulator columns in tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_u32(&tmem_base_s)), "r"(static_cast<uint32_t>(a.tmem_cols)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_s;
    const uint32_t idesc = umma_idesc(kTileN, a.tn);

    const int n_steps = a.K / kBK;
    bool ok = true;
    for (int ks = 0; ks < n_steps; ++ks) {
        const int s = ks & 1;
        // the MMAs that last read this stage (step ks-2) must have finished
        if (ks >= 2 && ok) ok = mbar_wait(&free_bar[s], ((ks >> 1) - 1) & 1, a.err);
        uint8_t* As = smem + static_cast<size_t>(s) * stage_bytes;
        uint8_t* A2s = As + a_bytes;
        uint8_t* Bs = As + a_bytes * (a.dual ? 2 : 1);
        const int k0 = ks * kBK;
        // weights: 128 rows x 8 chunks of 8 values
        for (int i = tid; i < kTileN * 8; i += kThreadsG) {
            const int r = i >> 3, c = i & 7;
            *reinterpret_cast<uint4*>(As + swz_off(r, c)) = dequant8_bf16(a.w, n0 + r, k0 + 8 * c, fi.block_elems);
            if (a.dual) *reinterpret_cast<uint4*>(A2s + swz_off(r, c)) = dequant8_bf16(a.w2, n0 + r, k0 + 8 * c, fi.block_elems);
        }
        // activations: tn token rows x 8 chunks
        for (int i = tid; i < a.tn * 8; i += kThreadsG) {
            const int r = i >> 3, c = i & 7;
            *reinterpret_cast<uint4*>(Bs + swz_off(r, c)) =
                __ldg(reinterpret_cast<const uint4*>(a.xb + static_cast<size_t>(t0 + r) * a.K + k0 + 8 * c));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy stores -> visible to the tensor core
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0 && ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = umma_desc(s_u32(As)), da2 = umma_desc(s_u32(A2s)), db = umma_desc(s_u32(Bs));
#pragma unroll
            for (int kk = 0; kk < kBK / 16; ++kk) {
                const uint32_t acc = (ks > 0 || kk > 0) ? 1u : 0u;
                umma_bf16(tmem_d, da + 2 * kk, db + 2 * kk, idesc, acc);                   // +32 bytes along K per step
                if (a.dual) umma_bf16(tmem_d + a.tn, da2 + 2 * kk, db + 2 * kk, idesc, acc);
            }
            umma_commit(ks == n_steps - 1 ? &done_bar : &free_bar[s]);
        }
    }
    // ---- epilogue: warp w reads lane quarter (w & 3), column half (w >> 2) ----
    if (ok) ok = mbar_wait(&done_bar, 0, a.err);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
        const int q = warp & 3, half = warp >> 2;
        const int64_t n = n0 + q * 32 + lane;
        const int c_begin = half * (a.tn / 2), c_end = c_begin + a.tn / 2;
        for (int c0 = c_begin; c0 < c_end; c0 += 32) {
            float v[32], v2[32];
            const uint32_t taddr = tmem_d + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(c0);
            tmem_ld32(taddr, v);
            if (a.dual) tmem_ld32(taddr + a.tn, v2);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int tok = t0 + c0 + i;
                if (c0 + i < c_end && tok < a.M && n < a.w.N) {
                    const size_t o = static_cast<size_t>(tok) * a.ldc + n;
                    float r = v[i];
                    if (a.dual) r = (r / (1.0f + expf(-r))) * v2[i];
                    else if (a.epi == EPI_ADD_BIAS) r += __ldg(a.bias + n);
                    else if (a.epi == EPI_RESIDUAL) r += a.resid[o];
                    a.y[o] = r;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(static_cast<uint32_t>(a.tmem_cols)) : "memory");
    }
}

}  // namespace

// tokens per CTA tile: a multiple of 64 (the epilogue reads two column halves 32 at a time), at most
// 256 (one accumulator) or 128 (gate and up accumulators side by side)
static int tile_tokens(const GemvArgs& g) {
    const int cap = g.epi == EPI_SWIGLU ? 128 : 256;
    return std::min(cap, (g.M + 63) / 64 * 64);
}
size_t gemm_tc_xb_elems(const GemvArgs& g) {
    const int tn = tile_tokens(g);
    return static_cast<size_t>((g.M + tn - 1) / tn) * tn * g.w.K;
}

// Prefill GEMM.  Returns GGB_NOT_FOUND when the shape is not covered (caller falls back).
// d_xb_v: scratch for the bf16 activations, at least gemm_tc_xb_elems(g) elements.
int launch_gemm_tc(Context* c, const GemvArgs& g, void* d_xb_v, size_t xb_elems, cudaStream_t s) {
    __nv_bfloat16* d_xb = static_cast<__nv_bfloat16*>(d_xb_v);
    const int K = g.w.K;
    const FormatInfo fi = format_info(g.w.type);
    if (!fi.block_elems || K % kBK || g.M < 1 || !g.x || g.n_cat || g.attn_partial) return GGB_NOT_FOUND;
    const bool dual = g.epi == EPI_SWIGLU;
    const int tn = tile_tokens(g);
    const int m_tiles = (g.M + tn - 1) / tn;
    if (static_cast<size_t>(m_tiles) * tn * K > xb_elems) return GGB_NOT_FOUND;
    int cols = 32;
    while (cols < tn * (dual ? 2 : 1)) cols <<= 1;

    x_to_bf16_kernel<<<m_tiles * tn, 256, 0, s>>>(g.x, g.lda, g.M, K, g.gamma, g.eps, d_xb);
    c->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_status(c, e, "x_to_bf16");

    GemmArgs a{};
    a.w = g.w; a.w2 = g.w2; a.xb = d_xb; a.y = g.y; a.bias = g.bias; a.resid = g.resid;
    a.M = g.M; a.K = K; a.ldc = g.ldc; a.epi = g.epi; a.dual = dual ? 1 : 0; a.tn = tn; a.tmem_cols = cols; a.err = c->d_err;
    const size_t smem = 2 * (static_cast<size_t>(kTileN) * 128 * (dual ? 2 : 1) + static_cast<size_t>(tn) * 128) + 1024;
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
        e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return cuda_status(c, e, "gemm_tc attr");
        allowed = smem;
    }
    dim3 grid(static_cast<unsigned>((g.w.N + kTileN - 1) / kTileN), static_cast<unsigned>(m_tiles));
    gemm_tc_kernel<<<grid, kThreadsG, smem, s>>>(a);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "gemm_tc launch");
}

}  // namespace ggb
