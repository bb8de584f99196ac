// C ABI, part 1: handle lifetime and the Backend operator set on HOST pointers
// (include/ggnpu/backend.h:113-160).  Each call stages its operands in device scratch, runs the
// kernels on the handle's stream and returns after the results are back in the caller's buffers,
// which is what the reference's NPU backend does (run.wait() inside each op,
// src/backends/amd_xdna/amd_xdna.cpp:865-897); sync() is then only a stream synchronise.
#include <stdio.h>

#include <algorithm>
#include <map>
#include <stdlib.h>
#include <string.h>

#include "ggb_internal.h"


namespace ggb {

int set_status(Context* c, int status, const char* msg) {
    if (c && status != GGB_OK) { c->last_status = status; c->last_message = msg ? msg : ""; }
    return status;
}

int cuda_status(Context* c, cudaError_t e, const char* what) {
    if (e == cudaSuccess) return GGB_OK;
    std::string m = std::string(what) + ": " + cudaGetErrorString(e);
    cudaGetLastError();   // clear the sticky-free error slot
    return set_status(c, e == cudaErrorMemoryAllocation ? GGB_OUT_OF_MEMORY : GGB_ERROR, m.c_str());
}

// FNV-1a over 64 evenly spaced 64-byte samples (the whole buffer when it is small)
static uint64_t weight_fingerprint(const void* data, size_t bytes) {
    const uint8_t* b = static_cast<const uint8_t*>(data);
    uint64_t h = 1469598103934665603ull;
    auto eat = [&](size_t from, size_t n) { for (size_t i = 0; i < n; ++i) { h ^= b[from + i]; h *= 1099511628211ull; } };
    if (bytes <= 64 * 64) { eat(0, bytes); return h; }
    const size_t stride = (bytes - 64) / 63;
    for (int i = 0; i < 64; ++i) eat(static_cast<size_t>(i) * stride, 64);
    return h;
}

void* scratch(Context* c, int slot, size_t bytes) {
    if (bytes <= c->d_scratch_bytes[slot]) return c->d_scratch[slot];
    if (c->d_scratch[slot]) { cudaStreamSynchronize(c->stream); cudaFree(c->d_scratch[slot]); c->d_scratch[slot] = nullptr; c->d_scratch_bytes[slot] = 0; }
    const size_t want = std::max(bytes, size_t(1) << 20);
    void* p = nullptr;
    if (cuda_status(c, cudaMalloc(&p, want), "cudaMalloc(scratch)") != GGB_OK) return nullptr;
    c->d_scratch[slot] = p; c->d_scratch_bytes[slot] = want;
    return p;
}

static int h2d(Context* c, void* d, const void* h, size_t n) { return cuda_status(c, cudaMemcpyAsync(d, h, n, cudaMemcpyHostToDevice, c->stream), "H2D copy"); }
static int d2h_sync(Context* c, void* h, const void* d, size_t n) {
    int st = cuda_status(c, cudaMemcpyAsync(h, d, n, cudaMemcpyDeviceToHost, c->stream), "D2H copy");
    if (st != GGB_OK) return st;
    return cuda_status(c, cudaStreamSynchronize(c->stream), "stream sync");
}

cudaError_t ensure_dynamic_smem(Context* c, const void* func, size_t smem) {
    // 48 KB is the limit without the opt-in for static + dynamic shared memory together: kernels here hold up to a few KB
    // of static arrays (barriers, small tables), so the opt-in is taken from 40 KB of dynamic memory on
    if (smem <= 40 * 1024) return cudaSuccess;
    static std::mutex mu;
    static std::map<std::pair<int, const void*>, size_t> granted;
    std::lock_guard<std::mutex> lk(mu);
    size_t& have = granted[{c->device, func}];
    if (smem <= have) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e == cudaSuccess) have = smem;
    return e;
}

// Device error word -> status.  Each bounded device-side wait records its own code when it gives up.
static const char* device_error_text(int v) {
    switch (v) {
    case 1: return "device: weight producer timed out waiting for a free ring stage";
    case 2: return "device: consumers timed out waiting for a weight tile";
    case 3: return "device: weight producer timed out waiting for the activations (x_ready)";
    case 4: return "device: tcgen05 GEMM timed out on an mbarrier (operand stage or accumulator)";
    case 5: return "device: one-shot all-reduce timed out waiting for a peer rank's flag; the buffer was left unsummed";
    case 6: return "device: decode step kernel timed out at a grid-wide phase barrier";
    default: return "device: a bounded wait gave up (unknown code)";
    }
}

int check_device_error(Context* c) {
    int v = 0;
    cudaError_t e = cudaMemcpy(&v, c->d_err, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_status(c, e, "read device error word");
    if (v == 0) return GGB_OK;
    cudaMemset(c->d_err, 0, sizeof(int));
    return set_status(c, GGB_ERROR, device_error_text(v));
}

}  // namespace ggb

using namespace ggb;

#define GGB_LOCK(h) std::lock_guard<std::mutex> _lk((h)->mu); cudaSetDevice((h)->device)
#define GGB_TRY(expr) do { int _st = (expr); if (_st != GGB_OK) return _st; } while (0)

extern "C" {

int ggb_create(int device, ggb_handle* out) {
    if (!out) return GGB_INVALID_PARAM;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0 || device < 0 || device >= n) { cudaGetLastError(); return GGB_UNAVAILABLE; }
    if (cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); return GGB_UNAVAILABLE; }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { cudaGetLastError(); return GGB_UNAVAILABLE; }
    if (prop.major < 10) return GGB_UNAVAILABLE;      // kernels are built for sm_100a only
    ggb_context* c = new ggb_context();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); delete c; return GGB_UNAVAILABLE; }
    if (cudaMalloc(&c->d_err, sizeof(int)) != cudaSuccess || cudaMemset(c->d_err, 0, sizeof(int)) != cudaSuccess) {
        cudaGetLastError(); cudaStreamDestroy(c->stream); delete c; return GGB_OUT_OF_MEMORY;
    }
    c->use_pdl = getenv("GGB_NO_PDL") == nullptr;
    c->use_tma = getenv("GGB_NO_TMA") == nullptr;
    c->use_mma = getenv("GGB_NO_MMA") == nullptr;
    c->use_tc = getenv("GGB_NO_TC") == nullptr;
    *out = c;
    return GGB_OK;
}

void ggb_destroy(ggb_handle h) {
    if (!h) return;
    cudaSetDevice(h->device);
    cudaStreamSynchronize(h->stream);
    tp_destroy(h);
    for (auto& kv : h->weight_cache) free_weight(kv.second);
    for (int i = 0; i < 4; ++i) if (h->d_scratch[i]) cudaFree(h->d_scratch[i]);
    if (h->d_xb) cudaFree(h->d_xb);
    if (h->d_ws) cudaFree(h->d_ws);
    if (h->d_limbs) cudaFree(h->d_limbs);
    if (h->h_pinned) cudaFreeHost(h->h_pinned);
    if (h->d_err) cudaFree(h->d_err);
    cudaStreamDestroy(h->stream);
    delete h;
}

void ggb_sync(ggb_handle h) {
    if (!h) return;
    GGB_LOCK(h);
    // Backend::sync returns nothing: a failure (CUDA error, or a device-side wait that gave up in any
    // kernel launched through the asynchronous entry points) lands in last_error / last_error_message.
    if (cuda_status(h, cudaStreamSynchronize(h->stream), "sync") == GGB_OK) check_device_error(h);
}
int ggb_is_available(ggb_handle h) { return h != nullptr; }
const char* ggb_name(ggb_handle) { return "cuda_b200"; }
int ggb_last_error(ggb_handle h) { return h ? h->last_status : GGB_UNAVAILABLE; }
const char* ggb_last_error_message(ggb_handle h) { return h ? h->last_message.c_str() : "no handle"; }
void* ggb_stream(ggb_handle h) { return h ? static_cast<void*>(h->stream) : nullptr; }
uint64_t ggb_launch_count(ggb_handle h) { return h ? h->launches : 0; }

int ggb_mul_mat_q(ggb_handle h, const ggb_mul_mat_params* p) {
    if (!h) return GGB_UNAVAILABLE;
    if (!p || !p->A || !p->B || !p->C) return set_status(h, GGB_INVALID_PARAM, "mul_mat_q: null pointer");
    if (p->M <= 0 || p->N <= 0 || p->K <= 0) return set_status(h, GGB_INVALID_PARAM, "mul_mat_q: non-positive size");
    GGB_LOCK(h);
    const int M = p->M, N = p->N, K = p->K;
    const int lda = p->lda >= K ? p->lda : K, ldc = p->ldc >= N ? p->ldc : N;
    float* dA = static_cast<float*>(scratch(h, 0, sizeof(float) * static_cast<size_t>(M) * K));
    float* dC = static_cast<float*>(scratch(h, 1, sizeof(float) * static_cast<size_t>(M) * N));
    if (!dA || !dC) return h->last_status;
    GGB_TRY(cuda_status(h, cudaMemcpy2DAsync(dA, sizeof(float) * K, p->A, sizeof(float) * lda, sizeof(float) * K, M, cudaMemcpyHostToDevice, h->stream), "A upload"));
    if (p->B_type == GGB_F32) {
        float* dB = static_cast<float*>(scratch(h, 2, sizeof(float) * static_cast<size_t>(K) * N));
        if (!dB) return h->last_status;
        GGB_TRY(h2d(h, dB, p->B, sizeof(float) * static_cast<size_t>(K) * N));
        GGB_TRY(launch_matmul_f32_kn(h, dA, dB, dC, M, N, K, K, N, h->stream));
    } else {
        const FormatInfo f = format_info(p->B_type);
        if (!f.block_elems) return set_status(h, GGB_INVALID_PARAM, "mul_mat_q: unsupported B_type");
        if (K % f.block_elems) return set_status(h, GGB_INVALID_PARAM, "mul_mat_q: K is not a multiple of the block length");
        Context::Key key{p->B, N, K, p->B_type};
        const uint64_t fp = weight_fingerprint(p->B, static_cast<size_t>(N) * (K / f.block_elems) * f.block_bytes);
        DeviceWeight* dw = nullptr;
        auto it = h->weight_cache.find(key);
        if (it != h->weight_cache.end() && it->second->fingerprint == fp) dw = it->second;
        else {
            if (it != h->weight_cache.end()) {            // same address and shape, other contents: replace
                cudaStreamSynchronize(h->stream);
                free_weight(it->second);
                h->weight_cache.erase(it);
            }
            GGB_TRY(upload_weight(h, p->B_type, N, K, p->B, &dw));
            dw->fingerprint = fp;
            h->weight_cache[key] = dw;
        }
        GemvArgs a{};
        a.w = dw->w; a.x = dA; a.M = M; a.lda = K; a.y = dC; a.ldc = N; a.epi = EPI_STORE;
        GGB_TRY(launch_gemv(h, a, h->stream));
    }
    GGB_TRY(cuda_status(h, cudaMemcpy2DAsync(p->C, sizeof(float) * ldc, dC, sizeof(float) * N, sizeof(float) * N, M, cudaMemcpyDeviceToHost, h->stream), "C download"));
    GGB_TRY(cuda_status(h, cudaStreamSynchronize(h->stream), "mul_mat_q"));
    return check_device_error(h);
}

int ggb_rms_norm(ggb_handle h, const ggb_rms_norm_params* p) {
    if (!h) return GGB_UNAVAILABLE;
    if (!p || !p->input || !p->output) return set_status(h, GGB_INVALID_PARAM, "rms_norm: null pointer");
    if (p->size <= 0) return set_status(h, GGB_INVALID_PARAM, "rms_norm: non-positive size");
    GGB_LOCK(h);
    const size_t nb = sizeof(float) * p->size;
    float* dx = static_cast<float*>(scratch(h, 0, nb));
    float* dy = static_cast<float*>(scratch(h, 1, nb));
    float* dw = p->weight ? static_cast<float*>(scratch(h, 2, nb)) : nullptr;
    if (!dx || !dy || (p->weight && !dw)) return h->last_status;
    GGB_TRY(h2d(h, dx, p->input, nb));
    if (dw) GGB_TRY(h2d(h, dw, p->weight, nb));
    GGB_TRY(launch_rms_norm(h, dx, dy, 1, p->size, p->eps, dw, h->stream));
    return d2h_sync(h, p->output, dy, nb);
}

static int rope_common(ggb_handle h, float* data, int n_heads, int n_dims, int64_t offset, float freq_scale, float freq_base,
                       int64_t rope_dims, const float* cos_t, const float* sin_t, int neox) {
    if (!data) return set_status(h, GGB_INVALID_PARAM, "rope: null pointer");
    if (n_heads <= 0 || n_dims <= 0 || rope_dims <= 0 || rope_dims > n_dims || (rope_dims & 1)) return set_status(h, GGB_INVALID_PARAM, "rope: bad dims");
    GGB_LOCK(h);
    const size_t nb = sizeof(float) * static_cast<size_t>(n_heads) * n_dims;
    float* dx = static_cast<float*>(scratch(h, 0, nb));
    if (!dx) return h->last_status;
    GGB_TRY(h2d(h, dx, data, nb));
    if (cos_t && sin_t) {
        const size_t tb = sizeof(float) * (rope_dims / 2);
        float* dc = static_cast<float*>(scratch(h, 1, tb));
        float* ds = static_cast<float*>(scratch(h, 2, tb));
        if (!dc || !ds) return h->last_status;
        GGB_TRY(h2d(h, dc, cos_t, tb));
        GGB_TRY(h2d(h, ds, sin_t, tb));
        GGB_TRY(launch_rope(h, dx, 1, n_heads, n_dims, static_cast<int>(rope_dims), dc, ds, nullptr, 0, neox, h->stream));
    } else {
        GGB_TRY(launch_rope_angles(h, dx, n_heads, n_dims, rope_dims, offset, freq_scale, freq_base, neox, h->stream));
    }
    return d2h_sync(h, data, dx, nb);
}

int ggb_rope(ggb_handle h, const ggb_rope_params* p) {
    if (!h) return GGB_UNAVAILABLE;
    if (!p) return set_status(h, GGB_INVALID_PARAM, "rope: null params");
    return rope_common(h, p->data, 1, p->n_dims, p->offset, p->freq_scale, p->freq_base, p->rope_dims, p->cos_table, p->sin_table, p->neox_split_half);
}

int ggb_rope_batched(ggb_handle h, const ggb_rope_batched_params* p) {
    if (!h) return GGB_UNAVAILABLE;
    if (!p) return set_status(h, GGB_INVALID_PARAM, "rope_batched: null params");
    return rope_common(h, p->data, p->n_heads, p->n_dims, p->offset, p->freq_scale, p->freq_base, p->rope_dims, p->cos_table, p->sin_table, p->neox_split_half);
}

int ggb_matmul_bf16(ggb_handle h, const float* A, const float* B, float* C, int M, int N, int K) {
    if (!h) return GGB_UNAVAILABLE;
    if (!A || !B || !C) return set_status(h, GGB_INVALID_PARAM, "matmul_bf16: null pointer");
    if (M <= 0 || N <= 0 || K <= 0) return set_status(h, GGB_INVALID_PARAM, "matmul_bf16: non-positive size");
    GGB_LOCK(h);
    float* dA = static_cast<float*>(scratch(h, 0, sizeof(float) * static_cast<size_t>(M) * K));
    float* dB = static_cast<float*>(scratch(h, 2, sizeof(float) * static_cast<size_t>(K) * N));
    float* dC = static_cast<float*>(scratch(h, 1, sizeof(float) * static_cast<size_t>(M) * N));
    if (!dA || !dB || !dC) return h->last_status;
    GGB_TRY(h2d(h, dA, A, sizeof(float) * static_cast<size_t>(M) * K));
    GGB_TRY(h2d(h, dB, B, sizeof(float) * static_cast<size_t>(K) * N));
    GGB_TRY(launch_matmul_f32_kn(h, dA, dB, dC, M, N, K, K, N, h->stream));
    return d2h_sync(h, C, dC, sizeof(float) * static_cast<size_t>(M) * N);
}

int ggb_softmax(ggb_handle h, const ggb_softmax_params* p) {
    if (!h) return GGB_UNAVAILABLE;
    if (!p || !p->input || !p->output) return set_status(h, GGB_INVALID_PARAM, "softmax: null pointer");
    if (p->rows <= 0 || p->cols <= 0) return set_status(h, GGB_INVALID_PARAM, "softmax: non-positive size");
    GGB_LOCK(h);
    const size_t nb = sizeof(float) * static_cast<size_t>(p->rows) * p->cols;
    float* dx = static_cast<float*>(scratch(h, 0, nb));
    float* dy = static_cast<float*>(scratch(h, 1, nb));
    if (!dx || !dy) return h->last_status;
    GGB_TRY(h2d(h, dx, p->input, nb));
    GGB_TRY(launch_softmax(h, dx, dy, p->rows, p->cols, h->stream));
    return d2h_sync(h, p->output, dy, nb);
}

static int unary(ggb_handle h, const ggb_unary_params* p, bool gelu) {
    if (!h) return GGB_UNAVAILABLE;
    if (!p || !p->input || !p->output) return set_status(h, GGB_INVALID_PARAM, "activation: null pointer");
    if (p->size <= 0) return set_status(h, GGB_INVALID_PARAM, "activation: non-positive size");
    GGB_LOCK(h);
    const size_t nb = sizeof(float) * p->size;
    float* dx = static_cast<float*>(scratch(h, 0, nb));
    float* dy = static_cast<float*>(scratch(h, 1, nb));
    if (!dx || !dy) return h->last_status;
    GGB_TRY(h2d(h, dx, p->input, nb));
    GGB_TRY(gelu ? launch_gelu(h, dx, dy, p->size, h->stream) : launch_silu(h, dx, dy, p->size, h->stream));
    return d2h_sync(h, p->output, dy, nb);
}
int ggb_silu(ggb_handle h, const ggb_unary_params* p) { return unary(h, p, false); }
int ggb_gelu(ggb_handle h, const ggb_unary_params* p) { return unary(h, p, true); }

int ggb_flash_attn(ggb_handle h, const ggb_attn_params* p) {
    if (!h) return GGB_UNAVAILABLE;
    if (!p || !p->Q || !p->K || !p->V || !p->output) return set_status(h, GGB_INVALID_PARAM, "flash_attn: null pointer");
    if (p->n_head <= 0 || p->head_dim <= 0 || p->ctx_len <= 0) return set_status(h, GGB_INVALID_PARAM, "flash_attn: non-positive size");
    GGB_LOCK(h);
    const size_t qb = sizeof(float) * static_cast<size_t>(p->n_head) * p->head_dim;
    const size_t kb = qb * static_cast<size_t>(p->ctx_len);
    float* dq = static_cast<float*>(scratch(h, 0, 2 * qb));
    float* dk = static_cast<float*>(scratch(h, 2, kb));
    float* dv = static_cast<float*>(scratch(h, 3, kb));
    if (!dq || !dk || !dv) return h->last_status;
    float* dout = dq + static_cast<size_t>(p->n_head) * p->head_dim;
    GGB_TRY(h2d(h, dq, p->Q, qb));
    GGB_TRY(h2d(h, dk, p->K, kb));
    GGB_TRY(h2d(h, dv, p->V, kb));
    GGB_TRY(launch_attn_expanded(h, dq, dk, dv, dout, p->n_head, p->head_dim, p->ctx_len, p->query_pos, h->stream));
    return d2h_sync(h, p->output, dout, qb);
}

// ---- part 2: packed weights and device-pointer GEMV -------------------------------------------

int ggb_dequant_rows(ggb_handle h, uint32_t type, const void* host_bytes, int64_t N, int K, int64_t row0, int64_t n_rows, float* host_out) {
    if (!h) return GGB_UNAVAILABLE;
    if (!host_bytes || !host_out) return set_status(h, GGB_INVALID_PARAM, "dequant_rows: null pointer");
    if (N <= 0 || K <= 0 || row0 < 0 || n_rows < 0 || row0 + n_rows > N) return set_status(h, GGB_INVALID_PARAM, "dequant_rows: bad range");
    if (n_rows == 0) return GGB_OK;
    GGB_LOCK(h);
    DeviceWeight* dw = nullptr;
    GGB_TRY(upload_weight(h, type, N, K, host_bytes, &dw));
    const size_t ob = sizeof(float) * static_cast<size_t>(n_rows) * K;
    float* dout = static_cast<float*>(scratch(h, 1, ob));
    int st = dout ? launch_dequant_rows(h, dw->w, row0, n_rows, dout, h->stream) : h->last_status;
    if (st == GGB_OK) st = d2h_sync(h, host_out, dout, ob);
    else cudaStreamSynchronize(h->stream);
    free_weight(dw);
    return st;
}

int ggb_weight_upload(ggb_handle h, uint32_t type, int64_t N, int K, const void* host_rows, ggb_weight* out) {
    if (!h) return GGB_UNAVAILABLE;
    if (!out) return set_status(h, GGB_INVALID_PARAM, "weight_upload: null out");
    GGB_LOCK(h);
    DeviceWeight* dw = nullptr;
    GGB_TRY(upload_weight(h, type, N, K, host_rows, &dw));
    *out = static_cast<ggb_weight>(dw);
    return GGB_OK;
}

void ggb_weight_free(ggb_handle h, ggb_weight w) {
    if (!h || !w) return;
    GGB_LOCK(h);
    cudaStreamSynchronize(h->stream);
    free_weight(w);
}

size_t ggb_weight_bytes(ggb_weight w) { return w ? w->bytes : 0; }

int ggb_gemv_device(ggb_handle h, ggb_weight w, const float* d_x, int M, int lda, float* d_y, int ldc, int epilogue,
                    const float* d_extra, const float* d_gamma, float eps) {
    if (!h) return GGB_UNAVAILABLE;
    if (!w || !d_x || !d_y) return set_status(h, GGB_INVALID_PARAM, "gemv_device: null pointer");
    if (epilogue < 0 || epilogue > 2 || (epilogue != 0 && !d_extra)) return set_status(h, GGB_INVALID_PARAM, "gemv_device: bad epilogue");
    GGB_LOCK(h);
    GemvArgs a{};
    a.w = w->w; a.x = d_x; a.M = M; a.lda = lda; a.y = d_y; a.ldc = ldc; a.epi = epilogue;
    a.bias = epilogue == EPI_ADD_BIAS ? d_extra : nullptr;
    a.resid = epilogue == EPI_RESIDUAL ? d_extra : nullptr;
    a.gamma = d_gamma; a.eps = eps;
    return launch_gemv(h, a, h->stream);
}

int ggb_gemv_swiglu_device(ggb_handle h, ggb_weight wg, ggb_weight wu, const float* d_x, int M, int lda, float* d_y, int ldc,
                           const float* d_gamma, float eps) {
    if (!h) return GGB_UNAVAILABLE;
    if (!wg || !wu || !d_x || !d_y) return set_status(h, GGB_INVALID_PARAM, "gemv_swiglu_device: null pointer");
    GGB_LOCK(h);
    GemvArgs a{};
    a.w = wg->w; a.w2 = wu->w; a.x = d_x; a.M = M; a.lda = lda; a.y = d_y; a.ldc = ldc; a.epi = EPI_SWIGLU;
    a.gamma = d_gamma; a.eps = eps;
    return launch_gemv(h, a, h->stream);
}

int ggb_qgate_split_device(ggb_handle h, const float* d_qg, float* d_q, int n_head, int head_dim) {
    if (!h) return GGB_UNAVAILABLE;
    if (!d_qg || !d_q || n_head <= 0 || head_dim <= 0) return set_status(h, GGB_INVALID_PARAM, "qgate_split: bad arguments");
    GGB_LOCK(h);
    return launch_qgate_split(h, d_qg, d_q, n_head, head_dim, h->stream);
}

int ggb_attn_gate_device(ggb_handle h, float* d_out, const float* d_qg, int n_head, int head_dim) {
    if (!h) return GGB_UNAVAILABLE;
    if (!d_out || !d_qg || n_head <= 0 || head_dim <= 0) return set_status(h, GGB_INVALID_PARAM, "attn_gate: bad arguments");
    GGB_LOCK(h);
    return launch_attn_gate(h, d_out, d_qg, n_head, head_dim, h->stream);
}

}  // extern "C"
