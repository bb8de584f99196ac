// Internal declarations shared by the translation units of libggb200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/ggb200.h"
#include "ggb_formats.cuh"

namespace ggb {

// Epilogue of a GEMV: what happens to y = W x before it is stored.
enum : int { EPI_STORE = 0, EPI_ADD_BIAS = 1, EPI_RESIDUAL = 2, EPI_SWIGLU = 3 };

struct GemvArgs {
    PackedW w;            // main weight
    PackedW w2;           // second weight of the same shape/type (SwiGLU: w = gate, w2 = up)
    const float* x;       // [M][lda] activations (device)
    int M, lda;
    float* y;             // [M][ldc]
    int ldc;
    int epi;
    const float* bias;    // EPI_ADD_BIAS: [N]
    const float* resid;   // EPI_RESIDUAL: [M][ldc], y = resid + W x (may alias y)
    // optional fused RMSNorm prologue: x is normalised with gamma before the product
    const float* gamma;   // nullptr => no norm
    float eps;
    // optional (tensor-core kernel, M == 1): x is the merge of paged-attention split results
    const float* attn_partial = nullptr;
    const int32_t* attn_d_pos = nullptr;
    int attn_pos0 = 0, attn_n_splits = 0, attn_keys_per_split = 0, attn_hd = 0;
    // attn_merge_below > 0: the kernel merges the partials only while fewer than that many splits are visible at the
    // current position; from there on the attention kernel has merged them itself (AttnPagedArgs::merge_min_splits) and
    // the merged row is read from attn_merged
    int attn_merge_below = 0;
    const float* attn_merged = nullptr;
    // optional (tensor-core kernel): up to two more matrices stacked along N sharing x, K, M, epilogue kind
    int n_cat = 0;
    PackedW cat_w[2];
    float* cat_y[2] = {nullptr, nullptr};
    const float* cat_bias[2] = {nullptr, nullptr};
    int cat_ldc[2] = {0, 0};
    // optional (tensor-core GEMV, Q4_K / Q6_K): routed experts.  w (and w2) hold all experts stacked along N
    // ([n_expert * sel_rows][K]); sel (device, sel_count ids) names the chosen ones.  sel_mode 1: the output
    // is the chosen experts' rows one after the other (gate / up);  sel_mode 2: K is the chosen experts' K
    // ranges side by side, x has sel_count * K values (down).  xscale multiplies x in runs of xscale_run.
    const int* sel = nullptr;
    int sel_mode = 0, sel_count = 0, sel_rows = 0;
    const float* xscale = nullptr;
    int xscale_run = 0;
    // optional (tcgen05 GEMM, M >= tc_min_m): x_img = activations already in the fp16 tile-image form
    // (x, gamma are then ignored); y_img (SwiGLU pair only) = write the result in that form, for a
    // following GEMM whose K is this N, instead of fp32 y.  gemm_tc_image_elems gives the buffer size.
    const void* x_img = nullptr;
    void* y_img = nullptr;
    // optional (multi-row tensor-core GEMV, 3 <= M <= 16): the previous launch_gemv call on this stream had the same
    // x, M, K, gamma and eps, so its int8-limb image of the activations is still in the workspace and is used again
    // (q, k and v projections of one layer)
    bool limbs_reuse = false;
};

struct DeviceWeight {
    PackedW w{};
    void* base = nullptr;     // one allocation holding all streams
    size_t bytes = 0;
    // fingerprint of sampled host bytes (weight cache): a freed host buffer whose address is reused
    // for other weights of the same shape must not hit the stale copy
    uint64_t fingerprint = 0;
};

struct Context {
    int device = 0;
    cudaStream_t stream = nullptr;
    std::mutex mu;
    int last_status = GGB_OK;
    std::string last_message;
    int sm_count = 148;
    // scratch buffers for the host-pointer operator path (grown on demand)
    void* d_scratch[4] = {nullptr, nullptr, nullptr, nullptr};
    size_t d_scratch_bytes[4] = {0, 0, 0, 0};
    void* h_pinned = nullptr;
    size_t h_pinned_bytes = 0;
    // host weight pointer -> packed device copy (first sight uploads)
    struct Key { const void* p; int64_t n; int k; uint32_t t; bool operator==(const Key& o) const { return p == o.p && n == o.n && k == o.k && t == o.t; } };
    struct KeyHash { size_t operator()(const Key& k) const { return std::hash<const void*>()(k.p) ^ (std::hash<int64_t>()(k.n * 1315423911u + k.k) << 1) ^ k.t; } };
    std::unordered_map<Key, DeviceWeight*, KeyHash> weight_cache;
    uint64_t launches = 0;    // kernels launched by this library on this context
    int* d_err = nullptr;     // device word: non-zero after a bounded device-side wait gave up
    bool use_pdl = true;      // launch the streaming kernels with programmatic dependent launch
    bool use_tma = true;      // M == 1 GEMV through the bulk-copy ring kernel
    bool use_mma = true;      // Q4_K in the row-group-major layout + int8 tensor-core GEMV (M <= 2)
    bool use_tc = true;       // M >= tc_min_m through the tcgen05 GEMM (fp16 operands, fp32 accumulation in TMEM)
    // 17: up to 16 rows keep fp32 activations (two rows per GEMV pass, rel-L2 1e-5 against the exact
    // product); from 17 rows on one pass of the tensor-core GEMM (~19 us for a 9-14 MB matrix whatever
    // M <= 64) beats nine and more GEMV passes (~3.5 us per row)
    int tc_min_m = 17;
    // tensor-parallel group (ggb_tp.cu); tp_size == 1: none
    void* tp_comm = nullptr;
    int tp_rank = 0, tp_size = 1;
    void* tp_region[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};   // peer-mapped exchange regions (own at tp_rank)
    bool tp_peers_attached = false;
    void* d_xb = nullptr;     // fp16 activation tile images of the tcgen05 GEMM (grown on demand, never during graph capture)
    size_t d_xb_elems = 0;
    float* d_ws = nullptr;    // split-K partial sums of the tcgen05 GEMM (grown on demand)
    size_t d_ws_floats = 0;
    void* d_limbs = nullptr;     // int8-limb image of up to 16 activation rows (multi-row GEMV), grown on demand
    size_t d_limbs_bytes = 0;
    // what the image holds and which launch_gemv call wrote or last used it: a reuse request is honoured only by the
    // very next call with the same source
    const void *limbs_x = nullptr, *limbs_gamma = nullptr;
    int limbs_M = 0, limbs_K = 0, limbs_lda = 0;
    float limbs_eps = 0.0f;
    uint64_t limbs_call = 0, gemv_calls = 0;
};

int set_status(Context* c, int status, const char* msg);
int cuda_status(Context* c, cudaError_t e, const char* what);
void* scratch(Context* c, int slot, size_t bytes);           // nullptr on failure (status set)

// ggb_pack.cu
int upload_weight(Context* c, uint32_t type, int64_t N, int K, const void* host_rows, DeviceWeight** out);
void free_weight(DeviceWeight* w);
size_t packed_bytes(uint32_t type, int64_t N, int K);
// ggb_pack_cache.cu: upload through the packed-weight disk cache (hit: 1 when the packed file was used)
int upload_weight_cached(Context* c, const char* cache_dir, const char* model_id, const char* tensor_name, uint32_t type, int64_t N, int K,
                         const void* host_rows, DeviceWeight** out, int* hit);
int launch_dequant_rows(Context* c, const PackedW& w, int64_t row0, int64_t n_rows, float* d_out, cudaStream_t s);
int launch_gather_rows(Context* c, const PackedW& w, const int32_t* d_rows, int n_rows, float* d_out, int ld, cudaStream_t s);

// ggb_gemv.cu / ggb_gemv_tma.cu
int launch_gemv(Context* c, const GemvArgs& a, cudaStream_t s);
int launch_gemv_tma(Context* c, const GemvArgs& a, cudaStream_t s);   // GGB_NOT_FOUND: shape not covered
int launch_gemv_mma(Context* c, const GemvArgs& a, cudaStream_t s);   // GGB_NOT_FOUND: shape not covered
// 3..16 rows in one pass over the weights; d_part: gemv_mma_rows_ws_floats(a) floats of workspace (K cut into slices).
// GGB_NOT_FOUND: shape not covered
int launch_gemv_mma_rows(Context* c, const GemvArgs& a, float* d_part, size_t part_floats, void* d_limbs, size_t limbs_bytes, cudaStream_t s);
size_t gemv_mma_rows_ws_floats(const GemvArgs& a);
size_t gemv_mma_rows_limbs_bytes(int M, int K);
// the same for Q8_0 / Q4_0 / IQ4_NL in the stream layout (ldmatrix on padded rows), 2..16 rows
int launch_gemv_mma_stream(Context* c, const GemvArgs& a, float* d_part, size_t part_floats, cudaStream_t s);
size_t gemv_mma_stream_ws_floats(const GemvArgs& a);
int launch_gemv_tma_rows(Context* c, const GemvArgs& a, cudaStream_t s);   // 2..16 rows, stream layout; needs c->d_limbs sized by the caller
int check_device_error(Context* c);
// ggb_gemm_tc.cu: prefill GEMM on tcgen05; GGB_NOT_FOUND: shape not covered
int launch_gemm_tc(Context* c, const GemvArgs& a, void* d_xb, size_t xb_elems, float* d_ws, size_t ws_floats, cudaStream_t s);
size_t gemm_tc_xb_elems(const GemvArgs& a);
size_t gemm_tc_ws_floats(const GemvArgs& a);       // split-K partial sums (0: no split)
inline size_t gemm_tc_image_elems(int M, int K) { return static_cast<size_t>((M + 255) / 256) * 256 * K; }

// Opt a kernel into `smem` bytes of dynamic shared memory (above the 48 KB default) on the context's
// device.  The attribute belongs to the (device, function) pair, so the bytes already granted are kept
// per pair behind one process-wide mutex: a second handle on another GPU gets its own call.
cudaError_t ensure_dynamic_smem(Context* c, const void* func, size_t smem);
template <class... KArgs>
static inline cudaError_t ensure_dynamic_smem(Context* c, void (*kern)(KArgs...), size_t smem) {
    return ensure_dynamic_smem(c, reinterpret_cast<const void*>(kern), smem);
}

// ggb_tp.cu: collectives over the handle's tensor-parallel group, on stream s (no-ops for a single rank)
int tp_all_reduce(Context* c, float* d_buf, size_t count, cudaStream_t s);               // sum, in place
int tp_all_gather_in_place(Context* c, float* d_recv, size_t count, cudaStream_t s);     // rank r's piece sits at d_recv + r * count
void tp_destroy(Context* c);

// Launch with programmatic dependent launch (when enabled on the context): the kernel may begin while its
// predecessor in the stream drains, and must execute griddepcontrol.wait before it touches anything
// an earlier kernel wrote or still reads.
template <class... KArgs, class... Args>
static inline cudaError_t launch_pdl(Context* c, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = c->use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

// ggb_ops.cu
int launch_rms_norm(Context* c, const float* x, float* y, int rows, int n, float eps, const float* gamma, cudaStream_t s);
int launch_silu(Context* c, const float* x, float* y, int64_t n, cudaStream_t s);
int launch_gelu(Context* c, const float* x, float* y, int64_t n, cudaStream_t s);
int launch_softmax(Context* c, const float* x, float* y, int rows, int cols, cudaStream_t s);
int launch_rope(Context* c, float* x, int n_tok, int n_heads, int head_dim, int rot_dims, const float* cos_tab,
                const float* sin_tab, const int32_t* d_pos, int pos0, int neox, cudaStream_t s);
int launch_rope_angles(Context* c, float* x, int n_heads, int n_dims, int64_t rope_dims, int64_t offset, float freq_scale,
                       float freq_base, int neox, cudaStream_t s);
int launch_matmul_f32_kn(Context* c, const float* A, const float* B, float* C, int M, int N, int K, int lda, int ldc, cudaStream_t s);
int launch_qgate_split(Context* c, const float* qg, float* q_out, int n_head, int hd, cudaStream_t s);
int launch_attn_gate(Context* c, float* out, const float* qg, int n_head, int hd, cudaStream_t s);
int launch_shortconv(Context* c, const float* bcx, const float* conv_w, float* state, float* y, int n_tok, int hidden, int taps, cudaStream_t s);
int launch_argmax(Context* c, const float* x, int n, int32_t* d_out, float* d_partial, cudaStream_t s);
int launch_argmax_rows(Context* c, const float* x, int n, int64_t ld, int rows, int32_t* d_out, float* d_partial, cudaStream_t s);

// ggb_sample.cu: temperature sampling (src/cli/main.cpp:839-864) on logits in HBM
size_t sample_scratch_bytes(int n);
int sample_enqueue(Context* c, const float* d_logits, int n, const int32_t* d_argmax, const float* d_temp, const double* d_u, const int32_t* d_step,
                   void* scratch, int32_t* d_out, cudaStream_t s);
double sample_next_uniform(uint64_t* seed);

// ggb_moe.cu / ggb_deltanet.cu: the operators of the qwen35moe layers with caller-owned scratch
size_t moe_scratch_floats(const ggb_moe_params* p);
struct MoeStacked { const DeviceWeight *gate, *up, *down; };      // expert tensors with the shared expert appended as one more expert
int moe_ffn_enqueue(Context* c, const ggb_moe_params* p, float* scr, cudaStream_t s, const MoeStacked* stacked = nullptr);
// ggb_pack.cu: a new weight whose rows are a's followed by b's (both Q4_K or both Q6_K in the row-group-major layout, the
// same K, a.N a multiple of 16); device-to-device copies on the context's stream
int concat_weight_rows(Context* c, const DeviceWeight* a, const DeviceWeight* b, DeviceWeight** out);
int deltanet_step_enqueue(Context* c, const ggb_deltanet_params* p, float* conv, cudaStream_t s);
// y[n] = (rms_norm(x) * gamma) . W[n][:] for small F32 matrices (a warp per row); gamma may be nullptr
int launch_f32_rows(Context* c, const float* x, const float* gamma, float eps, const float* W, int N, int K, float* y, cudaStream_t s);

// ggb_attn.cu
int launch_attn_expanded(Context* c, const float* Q, const float* K, const float* V, float* out, int n_head, int head_dim,
                         int64_t ctx_len, int64_t query_pos, cudaStream_t s);

}  // namespace ggb

// The opaque C handles are thin names for the internal structs.
struct ggb_context : ggb::Context {};
struct ggb_weight_s : ggb::DeviceWeight {};
