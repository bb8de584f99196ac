// Attention.
//  * attn_expanded: the Backend::flash_attn contract (src/backends/cpu_ref/cpu_ref.cpp:223-280):
//    one query token, fp32 K/V already expanded to one copy per query head.
//  * paged path: bf16 K (stored after RoPE) and V in pages of `page` tokens, laid out
//    [page][kv_head][slot][head_dim]; grouped-query attention reads each KV head once for all the
//    query heads that share it (the reference expands K/V per query head instead,
//    src/cli/main.cpp:3364-3383); long contexts are split across CTAs and merged by a second kernel.
#include <cuda_bf16.h>
#include <math.h>

#include "ggb_internal.h"
#include "ggb_attn.h"
#include "ggb_attn_tile.cuh"

namespace ggb {

// Programmatic dependent launch: a kernel launched with the attribute may start before its
// predecessor in the stream has finished; it must pass pdl_sync() before reading anything the
// predecessor wrote.  The trigger right after it lets the successor be scheduled in turn.
__device__ __forceinline__ void pdl_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// ---- Backend::flash_attn ---------------------------------------------------------------------
// One CTA per head.  scores[j] = scale * q.k_j for j <= query_pos, softmax with max subtraction,
// out = sum_j w_j v_j.  Scores for the whole context live in shared memory.
__global__ void attn_expanded_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                                     float* __restrict__ out, int hd, int64_t ctx, int64_t qpos) {
    extern __shared__ float sc[];            // [ctx]
    __shared__ float red[32];
    const int h = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float* q = Q + static_cast<size_t>(h) * hd;
    const float* k = K + static_cast<size_t>(h) * ctx * hd;
    const float* v = V + static_cast<size_t>(h) * ctx * hd;
    const float scale = 1.0f / sqrtf(static_cast<float>(hd));
    const int64_t n_keys = (qpos + 1 < ctx) ? qpos + 1 : ctx;
    for (int64_t j = warp; j < n_keys; j += nw) {
        float s = 0.0f;
        for (int d = lane; d < hd; d += 32) s = fmaf(q[d], k[j * hd + d], s);
        s = wsum(s);
        if (lane == 0) sc[j] = s * scale;
    }
    __syncthreads();
    float mx = -INFINITY;
    for (int64_t j = threadIdx.x; j < n_keys; j += blockDim.x) mx = fmaxf(mx, sc[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = -INFINITY;
    for (int i = 0; i < nw; ++i) mx = fmaxf(mx, red[i]);
    __syncthreads();
    float sum = 0.0f;
    for (int64_t j = threadIdx.x; j < n_keys; j += blockDim.x) { const float e = expf(sc[j] - mx); sc[j] = e; sum += e; }
    sum = wsum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = 0.0f;
    for (int i = 0; i < nw; ++i) sum += red[i];
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.0f;
        for (int64_t j = 0; j < n_keys; ++j) o = fmaf(sc[j] / sum, v[j * hd + d], o);
        out[static_cast<size_t>(h) * hd + d] = o;
    }
}

int launch_attn_expanded(Context* c, const float* Q, const float* K, const float* V, float* out, int n_head, int head_dim,
                         int64_t ctx_len, int64_t query_pos, cudaStream_t s) {
    const size_t smem = static_cast<size_t>(ctx_len) * sizeof(float);
    if (smem > 200 * 1024) return set_status(c, GGB_INVALID_PARAM, "flash_attn: ctx_len too large for the host-pointer path");
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attn_expanded_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return cuda_status(c, e, "flash_attn attr");
    }
    if (query_pos < 0) query_pos = ctx_len - 1;
    attn_expanded_kernel<<<n_head, 256, smem, s>>>(Q, K, V, out, head_dim, ctx_len, query_pos);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "flash_attn");
}

// ---- RoPE + KV append ---------------------------------------------------------------------------
// For token t (position p = pos + t): optional per-head RMS norm of q and k (sum of squares in
// double, src/cli/main.cpp:3294-3299), rotate q in place and k from the table row p
// (src/cli/main.cpp:1294-1308 / 3328-3341), store k (rotated) and v as bf16 into page p / page,
// slot p % page (K is cached after RoPE, V raw: src/cli/main.cpp:3354-3356).
// grid (ceil((n_head + n_kv) / blockDim.y), n_tok); blockDim.x = head_dim / 2 pairs rounded up to a warp,
// blockDim.y heads per CTA (256 threads in all).
__global__ void rope_append_kernel(KvAppendArgs a) {
    pdl_sync();
    const int t = blockIdx.y, hh = blockIdx.x * blockDim.y + threadIdx.y;
    const bool active = hh < a.n_head + a.n_kv;
    const int pos = a.seq_pos ? a.seq_pos[t] : (a.d_pos ? a.d_pos[0] : a.pos0) + t;
    const int hd = a.head_dim, half = hd >> 1;
    const int rot = a.rot_dims > 0 ? a.rot_dims : hd, rh = rot >> 1;       // rotated dims and pairs
    const bool is_q = hh < a.n_head;
    const int h = is_q ? hh : hh - a.n_head;
    float* src = !active ? nullptr : (is_q ? a.q + (static_cast<size_t>(t) * a.n_head + h) * hd : a.k + (static_cast<size_t>(t) * a.n_kv + h) * hd);
    const float* nw = is_q ? a.q_norm : a.k_norm;
    __shared__ double red[8][8];
    __shared__ float inv_s[8];
    const int i = threadIdx.x;               // thread i < rh owns rotation pair i; the others own two pass-through dims
    int i0, i1;
    if (i < rh) { i0 = a.neox ? i : 2 * i; i1 = a.neox ? i + rh : 2 * i + 1; }
    else { i0 = rot + 2 * (i - rh); i1 = i0 + 1; }
    float v0 = 0.0f, v1 = 0.0f;
    if (active && i < half) { v0 = src[i0]; v1 = src[i1]; }
    if (a.q_norm || a.k_norm) {              // uniform over the CTA: every thread reaches the barriers
        double ss = a.norm_f32 ? static_cast<double>(v0 * v0 + v1 * v1) : static_cast<double>(v0) * v0 + static_cast<double>(v1) * v1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
        if ((threadIdx.x & 31) == 0) red[threadIdx.y][threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            double tot = 0.0;
            for (int w = 0; w < (blockDim.x + 31) / 32; ++w) tot += red[threadIdx.y][w];
            inv_s[threadIdx.y] = 1.0f / sqrtf(static_cast<float>(tot / hd) + a.eps);
        }
        __syncthreads();
        if (nw && active && i < half) { v0 = v0 * inv_s[threadIdx.y] * nw[i0]; v1 = v1 * inv_s[threadIdx.y] * nw[i1]; }
    }
    if (active && i < half) {
        float r0 = v0, r1 = v1;
        if (i < rh) {
            const float cs = a.cos_tab[static_cast<size_t>(pos) * rh + i], sn = a.sin_tab[static_cast<size_t>(pos) * rh + i];
            r0 = v0 * cs - v1 * sn; r1 = v0 * sn + v1 * cs;
        }
        if (is_q) { src[i0] = r0; src[i1] = r1; }
        else {
            const int page = a.block_table[static_cast<size_t>(t) * a.seq_table_stride + pos / a.page], slot = pos % a.page;
            const size_t o = ((static_cast<size_t>(page) * a.n_kv + h) * a.page + slot) * hd;
            a.k_cache[o + i0] = __float2bfloat16_rn(r0);
            a.k_cache[o + i1] = __float2bfloat16_rn(r1);
            const float* vs = a.v + (static_cast<size_t>(t) * a.n_kv + h) * hd;
            a.v_cache[o + i0] = __float2bfloat16_rn(vs[i0]);
            a.v_cache[o + i1] = __float2bfloat16_rn(vs[i1]);
        }
    }
}

int launch_rope_append(Context* c, const KvAppendArgs& a_in, int n_tok, cudaStream_t s) {
    KvAppendArgs a = a_in;
    const int tx = ((a.head_dim / 2) + 31) / 32 * 32;
    if (tx > 256) return set_status(c, GGB_INVALID_PARAM, "rope_append: head_dim must be at most 512");
    const int ty = std::max(1, std::min(8, 256 / tx));
    dim3 grid((a.n_head + a.n_kv + ty - 1) / ty, n_tok);
    const cudaError_t e = launch_pdl(c, rope_append_kernel, grid, dim3(tx, ty), 0, s, a);
    c->launches++;
    return cuda_status(c, e, "rope_append");
}

// ---- paged GQA attention, split over the context ---------------------------------------------
// grid (n_kv, n_splits, n_tok), 128 threads.  CTA (h, s, t) handles KV head h, the keys of split s
// that are <= pos_t, for the G = n_head / n_kv query heads sharing h, and writes an un-normalised
// partial (max, sum, acc[hd]) per query head.  Keys are processed in chunks of 64: the chunk's K and
// V rows are first copied into shared memory with every 16-byte load in flight at once (a loop that
// fetches key after key pays one full memory latency per key), then scores, an online softmax and
// P*V run out of shared memory in fp32.
// With a.fuse (single-token decode) the kernel also does the work of rope_append_kernel for its
// head: q is rotated on the way into shared memory, and the CTA whose split contains pos rotates the
// new key, stores key and value into the cache and uses them directly.
template <int HD>
__global__ void __launch_bounds__(128) attn_tile_kernel(AttnPagedArgs a) {
    extern __shared__ __align__(16) uint32_t sm_u[];
    pdl_sync();
    attn_tile_body<HD, false>(a, blockIdx.x, blockIdx.y, blockIdx.z, threadIdx.x, sm_u, [] { __syncthreads(); });
}
// head_dim 64 compiled for five resident CTAs per SM: the register allocation that bound produces (96 instead of 80)
// runs the Llama-3.2-1B-shape decode step 2 % faster (1638 against 1604 tok/s on one box, twice each).  The other head
// sizes keep the compiler's default: for head_dim 128 every explicit bound tried was slower on the 16-sequence step of
// the 8B shape (10.8 ms by default; 11.3 ms at five CTAs, 11.4 at three, 12.3 at one).
__global__ void __launch_bounds__(128, 5) attn_tile_kernel_hd64(AttnPagedArgs a) {
    extern __shared__ __align__(16) uint32_t sm_u[];
    pdl_sync();
    attn_tile_body<64, false>(a, blockIdx.x, blockIdx.y, blockIdx.z, threadIdx.x, sm_u, [] { __syncthreads(); });
}
// The same with the query heads of a KV head dealt to a.head_split CTAs (grid.x = n_kv * head_split).
template <int HD>
__global__ void __launch_bounds__(128) attn_tile_split_kernel(AttnPagedArgs a) {
    extern __shared__ __align__(16) uint32_t sm_u[];
    pdl_sync();
    attn_tile_body<HD, false, true>(a, blockIdx.x, blockIdx.y, blockIdx.z, threadIdx.x, sm_u, [] { __syncthreads(); });
}

// grid (n_head, n_tok), 1024 threads: merge the visible splits, normalise, write out[t][head][hd].  The splits' (max, sum)
// pairs are fetched by one thread each and the weights exp(max_s - max) kept in shared memory; the sum over splits of
// an output element is cut over eight groups of 128 threads (splits g, g + 8, ...: at most eight loads per thread, all
// in flight together), and the eight partial sums meet in shared memory.  (One thread walking 18 splits one dependent
// load after the other took 18 us; one group of 128 over 64 splits, four loads in flight, 9 us; four groups 6.5 us,
// each under a profiler that empties the caches before the launch.)
__global__ void __launch_bounds__(1024) attn_combine_kernel(AttnPagedArgs a) {
    __shared__ float m_s[64], l_s[64], w_s[64];
    __shared__ float acc_s[7][256];
    pdl_sync();
    const int head = blockIdx.x, t = blockIdx.y, hd = a.head_dim, tid = threadIdx.x;
    const int pos = a.seq_pos ? a.seq_pos[t] : (a.d_pos ? a.d_pos[0] : a.pos0) + t;
    const int keys_per_split = a.pages_per_split * a.page;
    const int n_active = min(a.n_splits, pos / keys_per_split + 1);      // at most 64 (attn_split_geometry)
    if (n_active < a.merge_min_splits) return;         // few splits: the consumer merges them in its prologue
    const size_t stride = static_cast<size_t>(hd) + 2;
    const float* part = a.partial + (static_cast<size_t>(t) * a.n_head + head) * a.n_splits * stride;
    if (tid < n_active) { m_s[tid] = part[tid * stride]; l_s[tid] = part[tid * stride + 1]; }
    __syncthreads();
    float mx = -INFINITY;
    for (int s = 0; s < n_active; ++s) mx = fmaxf(mx, m_s[s]);
    if (tid < n_active) w_s[tid] = expf(m_s[tid] - mx);
    __syncthreads();
    const int g = tid >> 7, lane = tid & 127;
    float o[2] = {0.0f, 0.0f};                          // head_dim <= 256: elements lane and lane + 128
#pragma unroll 8
    for (int s = g; s < n_active; s += 8) {
        const float w = w_s[s];
        const float* ps = part + s * stride + 2;
        if (lane < hd) o[0] += ps[lane] * w;
        if (lane + 128 < hd) o[1] += ps[lane + 128] * w;
    }
    if (g > 0) { acc_s[g - 1][lane] = o[0]; acc_s[g - 1][lane + 128] = o[1]; }
    __syncthreads();
    if (g == 0) {
        float lsum = 0.0f;                              // every thread, the same order
        for (int s = 0; s < n_active; ++s) lsum += l_s[s] * w_s[s];
        float* dst = a.out + (static_cast<size_t>(t) * a.n_head + head) * hd;
        float s0 = o[0], s1 = o[1];
#pragma unroll
        for (int j = 0; j < 7; ++j) { s0 += acc_s[j][lane]; s1 += acc_s[j][lane + 128]; }
        if (lane < hd) dst[lane] = s0 / lsum;
        if (lane + 128 < hd) dst[lane + 128] = s1 / lsum;
    }
}

size_t attn_partial_floats(int n_tok, int n_head, int n_splits, int head_dim) {
    return static_cast<size_t>(n_tok) * n_head * n_splits * (head_dim + 2);
}

int launch_attn_paged(Context* c, const AttnPagedArgs& a_in, int n_tok, cudaStream_t s) {
    AttnPagedArgs a = a_in;
    const int G = a.n_head / a.n_kv;
    if (G < 1 || G > 8 || a.n_head % a.n_kv) return set_status(c, GGB_INVALID_PARAM, "attention: query heads per KV head must be 1..8");
    const int hd = a.head_dim;
    if (a.page % 8) return set_status(c, GGB_INVALID_PARAM, "attention: page size must be a multiple of 8");
    if (a.fuse && n_tok != 1 && !a.seq_pos) return set_status(c, GGB_INVALID_PARAM, "attention: fused append is for single-token steps (one per sequence)");
    if (c->use_tc && n_tok >= std::max(c->tc_min_m, 32) && !a.fuse && !a.seq_pos) {      // prompt chunks: tensor-core flash attention
        const int st = launch_attn_prefill(c, a, n_tok, s);
        if (st != GGB_NOT_FOUND) return st;
    }
    if (a.partial_tok_cap > 0 && n_tok > a.partial_tok_cap)
        return set_status(c, GGB_INVALID_PARAM, "attention: prompt chunk larger than the split scratch and not covered by the tensor-core kernel");
    if (a.merge_ticket && a.n_splits > 128) return set_status(c, GGB_INVALID_PARAM, "attention: more than 128 context splits");
    // one or two KV heads: 2 x splits CTAs leave most SMs idle, so the query heads of a KV head are dealt to two CTAs
    // (each re-reads the K / V chunk, which is small next to the idle SMs)
    if (a.head_split <= 1 && !a.merge_ticket && a.n_kv <= 2 && G >= 4 && G % 2 == 0 && static_cast<int64_t>(a.n_kv) * a.n_splits * n_tok < c->sm_count) a.head_split = 2;
    if (a.head_split > 1 && (a.merge_ticket || G % a.head_split)) a.head_split = 1;
    dim3 grid(a.n_kv * std::max(a.head_split, 1), a.n_splits, n_tok);
    cudaError_t e = cudaSuccess;
    size_t smem = 0;
#define GGB_ATTN_CASE(HD)                                                                                              \
    {                                                                                                                  \
        smem = attn_tile_smem(HD);                                                                                     \
        void (*kern)(AttnPagedArgs) = a.head_split > 1 ? attn_tile_split_kernel<HD> : (HD == 64 ? attn_tile_kernel_hd64 : attn_tile_kernel<HD>); \
        e = ensure_dynamic_smem(c, kern, smem);                                                                        \
        if (e == cudaSuccess) e = launch_pdl(c, kern, grid, dim3(128), smem, s, a);                                     \
    }
    if (hd == 64) GGB_ATTN_CASE(64)
    else if (hd == 128) GGB_ATTN_CASE(128)
    else if (hd == 256) GGB_ATTN_CASE(256)
    else return set_status(c, GGB_INVALID_PARAM, "attention: head_dim must be 64, 128 or 256");
#undef GGB_ATTN_CASE
    if (e != cudaSuccess) return cuda_status(c, e, "attention attr");
    c->launches++;
    if (e != cudaSuccess) return cuda_status(c, e, "attention split");
    if (a.skip_merge || a.merge_ticket) return GGB_OK;
    if (a.n_splits > 64) return set_status(c, GGB_INVALID_PARAM, "attention: more than 64 context splits");
    e = launch_pdl(c, attn_combine_kernel, dim3(a.n_head, n_tok), dim3(1024), 0, s, a);
    c->launches++;
    if (e != cudaSuccess) return cuda_status(c, e, "attention combine");
    return cuda_status(c, cudaGetLastError(), "attention combine");
}

// Split geometry shared by every caller: at most 32 splits, each a whole number of pages.
void attn_split_geometry(int n_pages, int* n_splits, int* pages_per_split) {
    *pages_per_split = (n_pages + 31) / 32;
    *n_splits = (n_pages + *pages_per_split - 1) / *pages_per_split;
}
// The same with the KV head count known: one or two KV heads give the decode kernel only n_splits or 2 n_splits CTAs,
// so the context is then cut into up to 64 splits.
void attn_split_geometry(int n_pages, int n_kv, int* n_splits, int* pages_per_split) {
    const int cap = n_kv <= 2 ? 64 : 32;
    *pages_per_split = (n_pages + cap - 1) / cap;
    *n_splits = (n_pages + *pages_per_split - 1) / *pages_per_split;
}

static int check_paged_params(Context* c, const ggb_attn_paged_params* p) {
    if (!p || !p->q || !p->k_cache || !p->v_cache || !p->block_table || !p->out) return set_status(c, GGB_INVALID_PARAM, "attn_paged: null pointer");
    if (p->n_head <= 0 || p->n_kv <= 0 || p->page <= 0 || p->n_pages <= 0 || p->pos < 0 || p->pos >= p->n_pages * p->page)
        return set_status(c, GGB_INVALID_PARAM, "attn_paged: bad sizes or position");
    return GGB_OK;
}

static AttnPagedArgs paged_args(const ggb_attn_paged_params* p, float* partial) {
    AttnPagedArgs a{};
    a.q = p->q; a.k_cache = static_cast<const __nv_bfloat16*>(p->k_cache); a.v_cache = static_cast<const __nv_bfloat16*>(p->v_cache);
    a.block_table = p->block_table; a.partial = partial; a.out = p->out; a.d_pos = nullptr; a.pos0 = p->pos;
    a.n_head = p->n_head; a.n_kv = p->n_kv; a.head_dim = p->head_dim; a.page = p->page;
    attn_split_geometry(p->n_pages, &a.n_splits, &a.pages_per_split);
    return a;
}

}  // namespace ggb

using namespace ggb;

extern "C" int ggb_attn_paged_device(ggb_handle h, const ggb_attn_paged_params* p) {
    if (!h) return GGB_UNAVAILABLE;
    int st = check_paged_params(h, p);
    if (st != GGB_OK) return st;
    std::lock_guard<std::mutex> lk(h->mu);
    cudaSetDevice(h->device);
    int n_splits, pps;
    attn_split_geometry(p->n_pages, &n_splits, &pps);
    float* partial = static_cast<float*>(scratch(h, 3, sizeof(float) * attn_partial_floats(1, p->n_head, n_splits, p->head_dim)));
    if (!partial) return h->last_status;
    return launch_attn_paged(h, paged_args(p, partial), 1, h->stream);
}

extern "C" int ggb_attn_prefill_device(ggb_handle h, const ggb_attn_paged_params* p, int n_tok) {
    if (!h) return GGB_UNAVAILABLE;
    int st = check_paged_params(h, p);
    if (st != GGB_OK) return st;
    if (n_tok <= 0 || p->pos + n_tok > p->n_pages * p->page) return set_status(h, GGB_INVALID_PARAM, "attn_prefill: chunk runs past the cache");
    std::lock_guard<std::mutex> lk(h->mu);
    cudaSetDevice(h->device);
    int n_splits, pps;
    attn_split_geometry(p->n_pages, &n_splits, &pps);
    float* partial = static_cast<float*>(scratch(h, 3, sizeof(float) * attn_partial_floats(n_tok, p->n_head, n_splits, p->head_dim)));
    if (!partial) return h->last_status;
    return launch_attn_paged(h, paged_args(p, partial), n_tok, h->stream);
}

// ---- the same attention without any allocation --------------------------------------------------
// Scratch for the per-split partial results lives in this fixed array, which every GPU that loads
// the library holds until the process exits.  64 query heads x 32 context splits x (256 + 2) floats.
static constexpr size_t kStaticAttnScratchFloats = static_cast<size_t>(64) * 32 * (256 + 2);
static __device__ __align__(256) float g_attn_static_scratch[kStaticAttnScratchFloats];

// Host code cannot use the array's name as a pointer: on the host it is only a handle for the
// symbol.  The device address is looked up once per device and kept here.
static float* g_attn_static_ptr[64];
static std::mutex g_attn_static_mu;

extern "C" int ggb_attn_paged_static(ggb_handle h, const ggb_attn_paged_params* p) {
    if (!h) return GGB_UNAVAILABLE;
    int st = check_paged_params(h, p);
    if (st != GGB_OK) return st;
    int n_splits, pps;
    attn_split_geometry(p->n_pages, &n_splits, &pps);
    const size_t need = attn_partial_floats(1, p->n_head, n_splits, p->head_dim);
    if (need > kStaticAttnScratchFloats || p->n_head > 64)
        return set_status(h, GGB_INVALID_PARAM, "attn_paged_static: n_head * splits * (head_dim + 2) exceeds the built-in scratch "
                                                "(64 heads x 32 splits x 258 floats); use ggb_attn_paged_device");
    if (h->device < 0 || h->device >= 64) return set_status(h, GGB_INVALID_PARAM, "attn_paged_static: device index out of range");
    std::lock_guard<std::mutex> lk(h->mu);
    cudaSetDevice(h->device);
    float* partial = nullptr;
    {
        std::lock_guard<std::mutex> g(g_attn_static_mu);
        if (!g_attn_static_ptr[h->device]) {
            void* sym = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(&sym, g_attn_static_scratch);   // with h->device current
            if (e != cudaSuccess) return cuda_status(h, e, "attn_paged_static: cudaGetSymbolAddress");
            g_attn_static_ptr[h->device] = static_cast<float*>(sym);
        }
        partial = g_attn_static_ptr[h->device];
    }
    return launch_attn_paged(h, paged_args(p, partial), 1, h->stream);
}
