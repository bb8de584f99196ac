// Small operators of the Backend set: RMSNorm, SiLU, GELU, softmax, RoPE, F32 matmul, argmax.
// Arithmetic follows src/backends/cpu_ref/cpu_ref.cpp (cited per kernel); reductions run in
// parallel, so sums differ from the sequential reference only in fp32 summation order.
#include <math.h>

#include "ggb_internal.h"

namespace ggb {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ float block_sum(float v, float* red) {
    v = warp_sum_f(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < (blockDim.x + 31) / 32; ++i) t += red[i];
    return t;
}
__device__ float block_max(float v, float* red) {
    v = warp_max_f(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = -INFINITY;
    for (int i = 0; i < (blockDim.x + 31) / 32; ++i) t = fmaxf(t, red[i]);
    return t;
}

// cpu_ref.cpp:139-156: v = sum(x^2)/n + eps; y = x * (1/sqrt(v)) * w.  One CTA per row.
__global__ void rms_norm_kernel(const float* __restrict__ x, float* __restrict__ y, int n, float eps, const float* __restrict__ gamma) {
    __shared__ float red[32];
    const float* xr = x + static_cast<size_t>(blockIdx.x) * n;
    float* yr = y + static_cast<size_t>(blockIdx.x) * n;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += xr[i] * xr[i];
    const float tot = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(tot / static_cast<float>(n) + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) yr[i] = xr[i] * inv * (gamma ? gamma[i] : 1.0f);
}

int launch_rms_norm(Context* c, const float* x, float* y, int rows, int n, float eps, const float* gamma, cudaStream_t s) {
    rms_norm_kernel<<<rows, 256, 0, s>>>(x, y, n, eps, gamma);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "rms_norm");
}

// cpu_ref.cpp:200-209: x / (1 + exp(-x)), with the correctly rounded expf and IEEE division.
__global__ void silu_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        y[i] = x[i] / (1.0f + expf(-x[i]));
}
// cpu_ref.cpp:211-221
__global__ void gelu_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n) {
    const float k = 0.7978845608f;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const float v = x[i];
        y[i] = 0.5f * v * (1.0f + tanhf(k * (v + 0.044715f * v * v * v)));
    }
}
static int ew_grid(int64_t n) { return static_cast<int>(std::min<int64_t>((n + 255) / 256, 148 * 8)); }

int launch_silu(Context* c, const float* x, float* y, int64_t n, cudaStream_t s) {
    silu_kernel<<<ew_grid(n), 256, 0, s>>>(x, y, n);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "silu");
}
int launch_gelu(Context* c, const float* x, float* y, int64_t n, cudaStream_t s) {
    gelu_kernel<<<ew_grid(n), 256, 0, s>>>(x, y, n);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "gelu");
}

// cpu_ref.cpp:176-198: max-subtracted exp, divide by the sum.  One CTA per row.
__global__ void softmax_kernel(const float* __restrict__ x, float* __restrict__ y, int cols) {
    __shared__ float red[32];
    const float* xr = x + static_cast<size_t>(blockIdx.x) * cols;
    float* yr = y + static_cast<size_t>(blockIdx.x) * cols;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) mx = fmaxf(mx, xr[i]);
    mx = block_max(mx, red);
    float sum = 0.0f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) { const float e = expf(xr[i] - mx); yr[i] = e; sum += e; }
    sum = block_sum(sum, red);
    for (int i = threadIdx.x; i < cols; i += blockDim.x) yr[i] = yr[i] / sum;
}
int launch_softmax(Context* c, const float* x, float* y, int rows, int cols, cudaStream_t s) {
    softmax_kernel<<<rows, 256, 0, s>>>(x, y, cols);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "softmax");
}

// RoPE from a host-built table (RopeCache, src/cli/main.cpp:665-692): x is [n_tok][n_heads][head_dim],
// token t sits at position d_pos[0]+t (or pos0+t when d_pos is null).  neox=0 rotates adjacent pairs
// (apply_rope_cpu, main.cpp:1294-1308), neox=1 the split halves (main.cpp:3328-3341); only the first
// rot_dims of each head are rotated (main.cpp:906-920).
__global__ void rope_kernel(float* __restrict__ x, int n_heads, int head_dim, int rot_dims, const float* __restrict__ cos_tab,
                            const float* __restrict__ sin_tab, const int32_t* __restrict__ d_pos, int pos0, int neox, int tab_pairs) {
    const int t = blockIdx.y;
    const int pos = (d_pos ? d_pos[0] : pos0) + t;
    const int half = rot_dims >> 1;
    const int total = n_heads * half;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        const float cs = cos_tab[static_cast<size_t>(pos) * tab_pairs + i], sn = sin_tab[static_cast<size_t>(pos) * tab_pairs + i];
        float* xh = x + (static_cast<size_t>(t) * n_heads + h) * head_dim;
        const int i0 = neox ? i : 2 * i, i1 = neox ? i + half : 2 * i + 1;
        const float v0 = xh[i0], v1 = xh[i1];
        xh[i0] = v0 * cs - v1 * sn;
        xh[i1] = v0 * sn + v1 * cs;
    }
}
// Small F32 matrices applied to a (normalised) row: y[n] = (rms_norm(x) * gamma) . W[n][:].  The reference computes
// F32 weight matrices on the host in fp32 (src/cli/main.cpp:1390-1406: qwen35moe's ssm_alpha / ssm_beta).  One warp per
// output row, eight rows per CTA; each warp forms the row statistic itself (K is a few thousand floats, in L2).
__global__ void f32_rows_kernel(const float* __restrict__ x, const float* __restrict__ gamma, float eps, const float* __restrict__ W,
                                int N, int K, float* __restrict__ y) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= N) return;
    const float* wr = W + static_cast<size_t>(n) * K;
    float acc = 0.0f, ss = 0.0f;
    if ((K & 127) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(gamma)) & 15) == 0) {
        // 16-byte loads, four per lane in flight: a loop of one dependent load per step pays a memory latency per step
        // (64 of them at K = 2048)
        for (int i0 = lane * 4; i0 < K; i0 += 512) {
            float4 wv[4], xv[4], gv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + 128 * u;
                if (i < K) {
                    wv[u] = __ldg(reinterpret_cast<const float4*>(wr + i));
                    xv[u] = *reinterpret_cast<const float4*>(x + i);
                    gv[u] = gamma ? __ldg(reinterpret_cast<const float4*>(gamma + i)) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (i0 + 128 * u < K) {
                    const float4 a = xv[u], g = gv[u], b = wv[u];
                    if (gamma) ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
                    acc += (a.x * g.x) * b.x + (a.y * g.y) * b.y + (a.z * g.z) * b.z + (a.w * g.w) * b.w;
                }
            }
        }
    } else {
        for (int i = lane; i < K; i += 32) {
            float v = x[i];
            if (gamma) { ss = fmaf(v, v, ss); v *= gamma[i]; }
            acc = fmaf(v, __ldg(wr + i), acc);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o); ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o); }
    if (gamma) acc *= 1.0f / sqrtf(ss / static_cast<float>(K) + eps);
    if (lane == 0) y[n] = acc;
}

int launch_f32_rows(Context* c, const float* x, const float* gamma, float eps, const float* W, int N, int K, float* y, cudaStream_t s) {
    const cudaError_t e = launch_pdl(c, f32_rows_kernel, dim3((N + 7) / 8), dim3(256), 0, s, x, gamma, eps, W, N, K, y);
    c->launches++;
    return cuda_status(c, e, "f32 rows");
}

int launch_rope(Context* c, float* x, int n_tok, int n_heads, int head_dim, int rot_dims, const float* cos_tab,
                const float* sin_tab, const int32_t* d_pos, int pos0, int neox, cudaStream_t s) {
    const int total = n_heads * (rot_dims / 2);
    dim3 grid((total + 127) / 128, n_tok);
    rope_kernel<<<grid, 128, 0, s>>>(x, n_heads, head_dim, rot_dims, cos_tab, sin_tab, d_pos, pos0, neox, rot_dims / 2);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "rope");
}

// Backend::rope without tables.  Angles as the CPU reference backend computes them
// (cpu_ref.cpp:158-174): ratio = 1 / base^(i/n_dims), angle = offset * ratio * freq_scale, for even i.
// The reference CPU backend hard-codes base 10000; here freq_base is honoured (10000 reproduces it).
__global__ void rope_angles_kernel(float* __restrict__ x, int n_heads, int n_dims, int rope_dims, float offset, float freq_scale,
                                   float freq_base, int neox) {
    const int half = rope_dims >> 1;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < n_heads * half; idx += gridDim.x * blockDim.x) {
        const int h = idx / half, p = idx - h * half;
        const float ratio = 1.0f / powf(freq_base, static_cast<float>(2 * p) / static_cast<float>(n_dims));
        const float ang = offset * ratio * freq_scale;
        const float cs = cosf(ang), sn = sinf(ang);
        float* xh = x + static_cast<size_t>(h) * n_dims;
        const int i0 = neox ? p : 2 * p, i1 = neox ? p + half : 2 * p + 1;
        const float v0 = xh[i0], v1 = xh[i1];
        xh[i0] = v0 * cs - v1 * sn;
        xh[i1] = v0 * sn + v1 * cs;
    }
}
int launch_rope_angles(Context* c, float* x, int n_heads, int n_dims, int64_t rope_dims, int64_t offset, float freq_scale,
                       float freq_base, int neox, cudaStream_t s) {
    const int total = n_heads * static_cast<int>(rope_dims / 2);
    rope_angles_kernel<<<(total + 127) / 128, 128, 0, s>>>(x, n_heads, n_dims, static_cast<int>(rope_dims), static_cast<float>(offset),
                                                           freq_scale, freq_base, neox);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "rope_angles");
}

// C[M][N] = A[M][K] * B[K][N], all fp32 (cpu_ref.cpp:119-133 and Backend::matmul_bf16's contract,
// include/ggnpu/backend.h:142-150).  Shared-memory tiled; a correctness path, not a hot one.
__global__ void matmul_f32_kn_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N, int K,
                                     int lda, int ldc) {
    __shared__ float As[16][17], Bs[16][17];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int m = blockIdx.y * 16 + ty, n = blockIdx.x * 16 + tx;
    float acc = 0.0f;
    for (int k0 = 0; k0 < K; k0 += 16) {
        As[ty][tx] = (m < M && k0 + tx < K) ? A[static_cast<size_t>(m) * lda + k0 + tx] : 0.0f;
        Bs[ty][tx] = (k0 + ty < K && n < N) ? B[static_cast<size_t>(k0 + ty) * N + n] : 0.0f;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) acc = fmaf(As[ty][k], Bs[k][tx], acc);
        __syncthreads();
    }
    if (m < M && n < N) C[static_cast<size_t>(m) * ldc + n] = acc;
}
int launch_matmul_f32_kn(Context* c, const float* A, const float* B, float* C, int M, int N, int K, int lda, int ldc, cudaStream_t s) {
    dim3 grid((N + 15) / 16, (M + 15) / 16), block(16, 16);
    matmul_f32_kn_kernel<<<grid, block, 0, s>>>(A, B, C, M, N, K, lda, ldc);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "matmul_f32");
}

// Greedy sampling (sample_token, src/cli/main.cpp:827-838): the FIRST index holding the maximum.
// Two passes: per-CTA (max, first index) into d_partial, then one CTA combines.
// blockIdx.y = row of a [rows][ld] matrix (one row: ld unused); partials of row r at [r * gridDim.x ..).
__global__ void argmax_pass1(const float* __restrict__ x, int n, int64_t ld, float* __restrict__ pmax, int32_t* __restrict__ pidx) {
    __shared__ float smax[32];
    __shared__ int sidx[32];
    x += static_cast<size_t>(blockIdx.y) * ld;
    pmax += blockIdx.y * gridDim.x; pidx += blockIdx.y * gridDim.x;
    float best = -INFINITY; int bi = 0x7FFFFFFF;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = x[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { smax[threadIdx.x >> 5] = best; sidx[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (blockDim.x >> 5); ++w)
            if (smax[w] > best || (smax[w] == best && sidx[w] < bi)) { best = smax[w]; bi = sidx[w]; }
        pmax[blockIdx.x] = best; pidx[blockIdx.x] = bi;
    }
}
__global__ void argmax_pass2(const float* __restrict__ pmax, const int32_t* __restrict__ pidx, int parts, int32_t* __restrict__ out) {
    pmax += blockIdx.x * parts; pidx += blockIdx.x * parts; out += blockIdx.x;
    float best = -INFINITY; int bi = 0x7FFFFFFF;
    for (int i = threadIdx.x; i < parts; i += 32) {
        const float v = pmax[i]; const int ix = pidx[i];
        if (v > best || (v == best && ix < bi)) { best = v; bi = ix; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (threadIdx.x == 0) out[0] = (bi == 0x7FFFFFFF) ? 0 : bi;
}
// d_partial must hold 2 * 256 words.
int launch_argmax(Context* c, const float* x, int n, int32_t* d_out, float* d_partial, cudaStream_t s) {
    const int parts = std::min(256, (n + 1023) / 1024);
    argmax_pass1<<<parts, 256, 0, s>>>(x, n, 0, d_partial, reinterpret_cast<int32_t*>(d_partial) + 256);
    argmax_pass2<<<1, 32, 0, s>>>(d_partial, reinterpret_cast<const int32_t*>(d_partial) + 256, parts, d_out);
    c->launches += 2;
    return cuda_status(c, cudaGetLastError(), "argmax");
}
// The same for each of `rows` (<= 16) rows of a [rows][ld] matrix in one pair of launches: d_out[r] = first maximum of row r.
int launch_argmax_rows(Context* c, const float* x, int n, int64_t ld, int rows, int32_t* d_out, float* d_partial, cudaStream_t s) {
    if (rows < 1 || rows > 16) return set_status(c, GGB_INVALID_PARAM, "argmax: 1 to 16 rows");
    const int parts = std::min(16, (n + 1023) / 1024);
    argmax_pass1<<<dim3(parts, rows), 256, 0, s>>>(x, n, ld, d_partial, reinterpret_cast<int32_t*>(d_partial) + 256);
    argmax_pass2<<<rows, 32, 0, s>>>(d_partial, reinterpret_cast<const int32_t*>(d_partial) + 256, parts, d_out);
    c->launches += 2;
    return cuda_status(c, cudaGetLastError(), "argmax");
}

// ---- gated short convolution (lfm2) ---------------------------------------------------------------
// src/cli/main.cpp:2704-2724, per channel: bx = B * x; acc = w[taps - 1] * bx + sum_k w[k] * state[k] (k ascending, the
// products and sums rounded one by one as the reference's loop does); y = C * acc; the state drops its oldest value and
// takes bx.  bcx [n_tok][3 hidden] = [B | C | x] rows of the in_proj output, conv_w [hidden][taps] (tap-contiguous),
// state [taps - 1][hidden] oldest first.  One thread per channel walks the rows in order with the state in registers.
template <int TAPS>
__global__ void __launch_bounds__(128) shortconv_kernel(const float* __restrict__ bcx, const float* __restrict__ conv_w, float* __restrict__ state,
                                                        float* __restrict__ y, int n_tok, int H) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int ch = blockIdx.x * 128 + threadIdx.x;
    if (ch >= H) return;
    float w[TAPS], st[TAPS > 1 ? TAPS - 1 : 1];
#pragma unroll
    for (int k = 0; k < TAPS; ++k) w[k] = conv_w[static_cast<size_t>(ch) * TAPS + k];
#pragma unroll
    for (int k = 0; k < TAPS - 1; ++k) st[k] = state[static_cast<size_t>(k) * H + ch];
    for (int t = 0; t < n_tok; ++t) {
        const float* row = bcx + static_cast<size_t>(t) * 3 * H;
        const float bx = __fmul_rn(row[ch], row[2 * H + ch]);
        float acc = __fmul_rn(w[TAPS - 1], bx);
#pragma unroll
        for (int k = 0; k < TAPS - 1; ++k) acc = __fadd_rn(acc, __fmul_rn(w[k], st[k]));
        y[static_cast<size_t>(t) * H + ch] = __fmul_rn(row[H + ch], acc);
#pragma unroll
        for (int k = 0; k < TAPS - 2; ++k) st[k] = st[k + 1];
        if (TAPS > 1) st[TAPS - 2] = bx;
    }
#pragma unroll
    for (int k = 0; k < TAPS - 1; ++k) state[static_cast<size_t>(k) * H + ch] = st[k];
}

int launch_shortconv(Context* c, const float* bcx, const float* conv_w, float* state, float* y, int n_tok, int hidden, int taps, cudaStream_t s) {
    const dim3 grid((hidden + 127) / 128), block(128);
    cudaError_t e = cudaErrorInvalidValue;
    switch (taps) {
#define GGB_SC_CASE(T) case T: e = launch_pdl(c, shortconv_kernel<T>, grid, block, 0, s, bcx, conv_w, state, y, n_tok, hidden); break;
        GGB_SC_CASE(1) GGB_SC_CASE(2) GGB_SC_CASE(3) GGB_SC_CASE(4) GGB_SC_CASE(5) GGB_SC_CASE(6) GGB_SC_CASE(7) GGB_SC_CASE(8)
#undef GGB_SC_CASE
    default: return set_status(c, GGB_INVALID_PARAM, "shortconv: 1 to 8 taps");
    }
    c->launches++;
    return cuda_status(c, e, "shortconv");
}

// ---- gated attention (qwen35 full-attention layers) -----------------------------------------------
// The attn_q projection emits, per query head, [query(hd) | gate(hd)] (src/cli/main.cpp:3054-3060).
// qgate_split: q_out[h][i] = qg[h][i] (contiguous heads for the attention kernels; the gate stays in qg).
// attn_gate:   out[h][i] *= sigmoid(qg[h][hd + i])  (main.cpp:3098), read in place from the projection.
__global__ void qgate_split_kernel(const float* __restrict__ qg, float* __restrict__ q_out, int n, int hd) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int h = i / hd, d = i - h * hd;
        q_out[i] = qg[static_cast<size_t>(h) * 2 * hd + d];
    }
}
__global__ void attn_gate_kernel(float* __restrict__ out, const float* __restrict__ qg, int n, int hd) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int h = i / hd, d = i - h * hd;
        out[i] *= 1.0f / (1.0f + expf(-qg[static_cast<size_t>(h) * 2 * hd + hd + d]));
    }
}
int launch_qgate_split(Context* c, const float* qg, float* q_out, int n_head, int hd, cudaStream_t s) {
    qgate_split_kernel<<<ew_grid(static_cast<int64_t>(n_head) * hd), 256, 0, s>>>(qg, q_out, n_head * hd, hd);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "qgate_split");
}
int launch_attn_gate(Context* c, float* out, const float* qg, int n_head, int hd, cudaStream_t s) {
    attn_gate_kernel<<<ew_grid(static_cast<int64_t>(n_head) * hd), 256, 0, s>>>(out, qg, n_head * hd, hd);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "attn_gate");
}

}  // namespace ggb
