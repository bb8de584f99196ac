// Prefill attention: causal GQA flash attention of a block of query tokens over the paged bf16 KV cache.
// Replaces, for a whole prompt chunk, the per-token loop GQA expand -> Backend::flash_attn
// (src/cli/main.cpp:3364-3383 -> src/backends/cpu_ref/cpu_ref.cpp:223-280):
//   out[t][h] = softmax_j<=pos(t)( q[t][h] . K[j][kv(h)] / sqrt(hd) ) V[j][kv(h)]
// One CTA (4 warps) = 64 query tokens x one query head; each warp owns 16 query rows.  Key tiles are
// the cache's 64-token pages: K and V of the page arrive with cp.async into double-buffered,
// XOR-swizzled shared memory, S = Q K^T and O += P V run on mma.sync m16n8k16 (bf16 operands, fp32
// accumulators), the softmax is the online (running max / running sum) form in fp32 registers.
// Q is rounded to bf16 once, P once per tile.  Rows of a page beyond the last cached token are
// zero-filled so stale cache contents cannot reach the sums.
#include <cuda_bf16.h>

#include "ggb_attn.h"
#include "ggb_internal.h"

namespace ggb {

namespace {

constexpr int kQTile = 64;      // query tokens per CTA
constexpr int kKTile = 64;      // keys per step = page size

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool pred) {
    const int sz = pred ? 16 : 0;      // src-size 0: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// A [64 keys][HD] bf16 tile: 16-byte chunk c of row r is stored at chunk c ^ (r & 7).
template <int HD> __device__ __forceinline__ uint32_t tile_off(int r, int c) { return static_cast<uint32_t>(r * HD * 2 + ((c ^ (r & 7)) << 4)); }

template <int HD>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const AttnPagedArgs a, const int n_tok) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int kTileBytes = kKTile * HD * 2;
    uint8_t* Ks = smem;                       // [2][64][HD]
    uint8_t* Vs = smem + 2 * kTileBytes;      // [2][64][HD]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int qb = gridDim.x - 1 - blockIdx.x;       // longest (latest) query blocks first
    const int h = blockIdx.y, kvh = h / (a.n_head / a.n_kv);
    const int pos0 = a.d_pos ? *a.d_pos : a.pos0;
    const int tok0 = qb * kQTile;
    const int n_keys = pos0 + n_tok;                 // cached tokens once this chunk is appended
    const int last_q = min(tok0 + kQTile, n_tok) - 1;
    const int n_tiles = (pos0 + last_q) / kKTile + 1;

    auto load_tile = [&](int j, int buf) {
        const int phys = a.block_table[j];
        const size_t base = (static_cast<size_t>(phys) * a.n_kv + kvh) * kKTile * HD;
        const __nv_bfloat16* kp = a.k_cache + base;
        const __nv_bfloat16* vp = a.v_cache + base;
        for (int i = tid; i < kKTile * (HD / 8); i += 128) {
            const int r = i / (HD / 8), c = i % (HD / 8);
            const bool live = j * kKTile + r < n_keys;
            cp_async16(Ks + buf * kTileBytes + tile_off<HD>(r, c), kp + r * HD + c * 8, live);
            cp_async16(Vs + buf * kTileBytes + tile_off<HD>(r, c), vp + r * HD + c * 8, live);
        }
        cp_async_commit();
    };
    load_tile(0, 0);

    // Q fragments of this warp's 16 rows (rows past the chunk read row 0 and are never stored)
    const int row_a = tok0 + warp * 16 + g, row_b = row_a + 8;
    const float* qa = a.q + (static_cast<size_t>(row_a < n_tok ? row_a : 0) * a.n_head + h) * HD;
    const float* qb_ = a.q + (static_cast<size_t>(row_b < n_tok ? row_b : 0) * a.n_head + h) * HD;
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
        const float2 a0 = *reinterpret_cast<const float2*>(qa + 16 * kk + 2 * t), a2 = *reinterpret_cast<const float2*>(qa + 16 * kk + 8 + 2 * t);
        const float2 a1 = *reinterpret_cast<const float2*>(qb_ + 16 * kk + 2 * t), a3 = *reinterpret_cast<const float2*>(qb_ + 16 * kk + 8 + 2 * t);
        qf[kk][0] = pack_bf16(a0.x, a0.y); qf[kk][1] = pack_bf16(a1.x, a1.y);
        qf[kk][2] = pack_bf16(a2.x, a2.y); qf[kk][3] = pack_bf16(a3.x, a3.y);
    }
    const float scale_log2 = rsqrtf(static_cast<float>(HD)) * 1.4426950408889634f;
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
    const int pos_a = pos0 + row_a, pos_b = pos0 + row_b;

    for (int j = 0; j < n_tiles; ++j) {
        const int buf = j & 1;
        if (j + 1 < n_tiles) { load_tile(j + 1, buf ^ 1); cp_async_wait<1>(); } else cp_async_wait<0>();
        __syncthreads();
        const uint32_t kbase = smem_addr(Ks + buf * kTileBytes), vbase = smem_addr(Vs + buf * kTileBytes);
        // ---- S = Q K^T : 16 rows x 64 keys per warp ----
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {            // key n-tiles 2 jp, 2 jp + 1
                const int key = 16 * jp + 8 * (lane >> 4) + (lane & 7), ch = 2 * kk + ((lane >> 3) & 1);
                uint32_t b0, b1, b2, b3;
                ldsm_x4(kbase + tile_off<HD>(key, ch), b0, b1, b2, b3);
                mma_bf16(s[2 * jp], qf[kk], b0, b1);
                mma_bf16(s[2 * jp + 1], qf[kk], b2, b3);
            }
        }
        // ---- causal mask + online softmax (rows g and g + 8; this thread holds keys 8 i + 2 t, + 1) ----
        const int key0 = j * kKTile;
        const bool need_mask = key0 + kKTile - 1 > pos0 + tok0 + warp * 16;
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (need_mask) {
                const int k0 = key0 + 8 * i + 2 * t;
                if (k0 > pos_a) s[i][0] = -INFINITY;
                if (k0 + 1 > pos_a) s[i][1] = -INFINITY;
                if (k0 > pos_b) s[i][2] = -INFINITY;
                if (k0 + 1 > pos_b) s[i][3] = -INFINITY;
            }
            mx_a = fmaxf(mx_a, fmaxf(s[i][0], s[i][1]));
            mx_b = fmaxf(mx_b, fmaxf(s[i][2], s[i][3]));
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xFFFFFFFFu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xFFFFFFFFu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xFFFFFFFFu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xFFFFFFFFu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        // a row with no visible key so far keeps m = -inf; use 0 as the reference so exp2 sees -inf, not nan
        const float ref_a = mn_a == -INFINITY ? 0.0f : mn_a * scale_log2, ref_b = mn_b == -INFINITY ? 0.0f : mn_b * scale_log2;
        const float al_a = exp2f(m_a * scale_log2 - ref_a), al_b = exp2f(m_b * scale_log2 - ref_b);
        m_a = mn_a; m_b = mn_b;
        float sum_a = 0.0f, sum_b = 0.0f;
        uint32_t pf[4][4];                               // P as A fragments: k-step kk2 covers keys 16 kk2 .. + 15
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float p0 = exp2f(s[i][0] * scale_log2 - ref_a), p1 = exp2f(s[i][1] * scale_log2 - ref_a);
            const float p2 = exp2f(s[i][2] * scale_log2 - ref_b), p3 = exp2f(s[i][3] * scale_log2 - ref_b);
            sum_a += p0 + p1; sum_b += p2 + p3;
            pf[i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);
            pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l_a = l_a * al_a + sum_a; l_b = l_b * al_b + sum_b;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) { o[i][0] *= al_a; o[i][1] *= al_a; o[i][2] *= al_b; o[i][3] *= al_b; }
        // ---- O += P V ----
#pragma unroll
        for (int kk2 = 0; kk2 < 4; ++kk2) {
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {      // dim n-tiles 2 dp, 2 dp + 1
                const int key = 16 * kk2 + 8 * ((lane >> 3) & 1) + (lane & 7), ch = 2 * dp + (lane >> 4);
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(vbase + tile_off<HD>(key, ch), b0, b1, b2, b3);
                mma_bf16(o[2 * dp], pf[kk2], b0, b1);
                mma_bf16(o[2 * dp + 1], pf[kk2], b2, b3);
            }
        }
        __syncthreads();         // everyone is done with `buf` before the next iteration's copy lands in it
    }
    // ---- normalise and store ----
    l_a += __shfl_xor_sync(0xFFFFFFFFu, l_a, 1); l_a += __shfl_xor_sync(0xFFFFFFFFu, l_a, 2);
    l_b += __shfl_xor_sync(0xFFFFFFFFu, l_b, 1); l_b += __shfl_xor_sync(0xFFFFFFFFu, l_b, 2);
    const float inv_a = 1.0f / l_a, inv_b = 1.0f / l_b;
    float* oa = a.out + (static_cast<size_t>(row_a) * a.n_head + h) * HD;
    float* ob = a.out + (static_cast<size_t>(row_b) * a.n_head + h) * HD;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        if (row_a < n_tok) *reinterpret_cast<float2*>(oa + 8 * i + 2 * t) = make_float2(o[i][0] * inv_a, o[i][1] * inv_a);
        if (row_b < n_tok) *reinterpret_cast<float2*>(ob + 8 * i + 2 * t) = make_float2(o[i][2] * inv_b, o[i][3] * inv_b);
    }
}

}  // namespace

// GGB_NOT_FOUND: geometry not covered (the caller uses the per-token kernel).
int launch_attn_prefill(Context* c, const AttnPagedArgs& a, int n_tok, cudaStream_t s) {
    if (a.page != kKTile || a.fuse || (a.head_dim != 64 && a.head_dim != 128) || a.n_head % a.n_kv) return GGB_NOT_FOUND;
    dim3 grid((n_tok + kQTile - 1) / kQTile, a.n_head);
    const size_t smem = 4 * static_cast<size_t>(kKTile) * a.head_dim * 2;
    cudaError_t e = cudaSuccess;
    if (a.head_dim == 64) {
        attn_prefill_kernel<64><<<grid, 128, smem, s>>>(a, n_tok);
    } else {
        e = ensure_dynamic_smem(c, attn_prefill_kernel<128>, smem);
        if (e == cudaSuccess) attn_prefill_kernel<128><<<grid, 128, smem, s>>>(a, n_tok);
    }
    if (e != cudaSuccess) return cuda_status(c, e, "attention prefill attr");
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "attention prefill");
}

}  // namespace ggb
