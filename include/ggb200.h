/*
 * ggb200.h -- C ABI of libggb200.so, a CUDA (sm_100a) implementation of the
 * ggnpu Backend operator set.
 *
 * Part 1 mirrors ggnpu's plugin boundary one to one: every function takes the
 * same parameter block, with the same field order, types and meaning, as the
 * C++ method it stands in for (include/ggnpu/backend.h), uses HOST pointers
 * owned by the caller, and returns the integer value of ggnpu::Status.
 * Part 2 is the device-resident path (weights packed once into HBM, paged bf16
 * KV cache, whole decode step as one CUDA graph); it has no counterpart in the
 * reference, whose only caller keeps every activation in host memory.
 *
 * No function throws, aborts, or falls back to the CPU.  Every failure is a
 * status code plus a message kept per handle (ggb_last_error_message).
 */
#ifndef GGB200_H
#define GGB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define GGB_API __attribute__((visibility("default")))
#else
#define GGB_API
#endif

/* ggnpu::Status, include/ggnpu/backend.h:12-19 (same integer values). */
enum ggb_status {
    GGB_OK = 0,
    GGB_ERROR = 1,
    GGB_NOT_FOUND = 2,
    GGB_INVALID_PARAM = 3,
    GGB_UNAVAILABLE = 4, /* NPU_UNAVAILABLE: no usable CUDA device */
    GGB_OUT_OF_MEMORY = 5
};

/* ggml type ids as in ggnpu::GgmlType, include/ggnpu/tensor.h:11-42. */
enum ggb_type {
    GGB_F32 = 0, GGB_F16 = 1, GGB_Q4_0 = 2, GGB_Q4_1 = 3, GGB_Q8_0 = 8, GGB_Q2_K = 10, GGB_Q3_K = 11,
    GGB_Q4_K = 12, GGB_Q5_K = 13, GGB_Q6_K = 14, GGB_IQ4_NL = 20, GGB_IQ4_XS = 23, GGB_BF16 = 30,
    /* grid-coded formats (src/quant/iquants.cpp:37-203).  Their codebooks are generated when the library
     * is built (ggnpu_b200/iq_tables.py, from the gguf package); a library built without them answers
     * GGB_INVALID_PARAM for these ids. */
    GGB_IQ2_XXS = 16, GGB_IQ2_XS = 17, GGB_IQ3_XXS = 18, GGB_IQ1_S = 19, GGB_IQ3_S = 21, GGB_IQ2_S = 22, GGB_IQ1_M = 29
};

typedef struct ggb_context* ggb_handle;

/* ---------------------------------------------------------------------------
 * Part 1: the Backend operator set (host pointers, f32 activations)
 * ------------------------------------------------------------------------- */

/* ggnpu::MulMatParams, include/ggnpu/backend.h:21-35.  C[M,N] = A[M,K] * W^T.
 * For a quantised B_type, B is raw GGUF bytes: N rows of ceil(K/blk) blocks
 * (what the reference hands any backend whose name is not "amd_xdna",
 * src/cli/main.cpp:1430-1432).  For F32, B is [K][N] as in
 * src/backends/cpu_ref/cpu_ref.cpp:119-133.  ldb, scales, n_weight_scales and
 * n_batches are accepted and ignored, as both reference backends do for
 * quantised weights.  B is cached by (pointer, N, K, type): the first call
 * uploads and packs it, later calls reuse the HBM copy, so B must stay valid
 * and unchanged while the handle lives (the reference passes mmap'd weights). */
typedef struct ggb_mul_mat_params {
    const void* A;
    const void* B;
    void* C;
    int M, N, K;
    int lda, ldb, ldc;
    int32_t n_batches;
    const void* scales;
    int n_weight_scales;
    uint32_t B_type;
} ggb_mul_mat_params;

/* ggnpu::RmsNormParams, include/ggnpu/backend.h:37-43. */
typedef struct ggb_rms_norm_params {
    const float* input;
    float* output;
    int size;
    float eps;
    const float* weight; /* may be NULL */
} ggb_rms_norm_params;

/* ggnpu::RopeParams, include/ggnpu/backend.h:45-62.  Rotates data in place. */
typedef struct ggb_rope_params {
    float* data;
    int n_dims;
    int64_t offset;
    float freq_scale;
    float freq_base;
    int64_t rope_dims;
    const float* cos_table; /* optional [rope_dims/2]; with sin_table overrides the angles */
    const float* sin_table;
    uint8_t neox_split_half;
} ggb_rope_params;

/* ggnpu::RopeBatchedParams, include/ggnpu/backend.h:68-79. */
typedef struct ggb_rope_batched_params {
    float* data; /* [n_heads][n_dims] */
    int n_heads;
    int n_dims;
    int64_t offset;
    float freq_scale;
    float freq_base;
    int64_t rope_dims;
    const float* cos_table;
    const float* sin_table;
    uint8_t neox_split_half;
} ggb_rope_batched_params;

/* ggnpu::SoftmaxParams / SiluParams / GeluParams, include/ggnpu/backend.h:81-98. */
typedef struct ggb_softmax_params { const float* input; float* output; int rows; int cols; } ggb_softmax_params;
typedef struct ggb_unary_params { const float* input; float* output; int size; } ggb_unary_params;

/* ggnpu::AttnParams, include/ggnpu/backend.h:100-111.  Q [n_head][head_dim];
 * K,V [n_head][ctx_len][head_dim] already expanded per query head; keys after
 * query_pos are masked; query_pos < 0 means ctx_len-1; scale 1/sqrt(head_dim). */
typedef struct ggb_attn_params {
    const float* Q;
    const float* K;
    const float* V;
    float* output;
    int batch_size;
    int n_head;
    int head_dim;
    int64_t ctx_len;
    int64_t query_pos;
    const float* freq_factors; /* unused, as in the reference */
} ggb_attn_params;

/* Factory + lifetime.  Replaces ggnpu::create_amd_xdna_backend(int),
 * include/ggnpu/backend.h:162-165 (defined src/backends/amd_xdna/amd_xdna.cpp:3104-3111).
 * Returns GGB_UNAVAILABLE when the device cannot be used. */
GGB_API int ggb_create(int device, ggb_handle* out);
GGB_API void ggb_destroy(ggb_handle h);

/* Backend::mul_mat_q, include/ggnpu/backend.h:117. */
GGB_API int ggb_mul_mat_q(ggb_handle h, const ggb_mul_mat_params* p);
/* Backend::rms_norm, include/ggnpu/backend.h:118. */
GGB_API int ggb_rms_norm(ggb_handle h, const ggb_rms_norm_params* p);
/* Backend::rope, include/ggnpu/backend.h:119. */
GGB_API int ggb_rope(ggb_handle h, const ggb_rope_params* p);
/* Backend::rope_batched, include/ggnpu/backend.h:123-140. */
GGB_API int ggb_rope_batched(ggb_handle h, const ggb_rope_batched_params* p);
/* Backend::matmul_bf16, include/ggnpu/backend.h:146-150: C[M,N] = A[M,K] B[K,N],
 * f32 host buffers. */
GGB_API int ggb_matmul_bf16(ggb_handle h, const float* A, const float* B, float* C, int M, int N, int K);
/* Backend::softmax / silu / gelu / flash_attn, include/ggnpu/backend.h:152-155. */
GGB_API int ggb_softmax(ggb_handle h, const ggb_softmax_params* p);
GGB_API int ggb_silu(ggb_handle h, const ggb_unary_params* p);
GGB_API int ggb_gelu(ggb_handle h, const ggb_unary_params* p);
GGB_API int ggb_flash_attn(ggb_handle h, const ggb_attn_params* p);
/* Backend::sync / is_available / name / last_error, include/ggnpu/backend.h:156-160. */
GGB_API void ggb_sync(ggb_handle h);
GGB_API int ggb_is_available(ggb_handle h);
GGB_API const char* ggb_name(ggb_handle h); /* "cuda_b200" */
GGB_API int ggb_last_error(ggb_handle h);
GGB_API const char* ggb_last_error_message(ggb_handle h);

/* ---------------------------------------------------------------------------
 * Part 2: device-resident path
 * ------------------------------------------------------------------------- */

/* Block decode on the GPU (the role of dequant_*_block, include/ggnpu/quant/kquant.h:70-202
 * and src/quant/q*.cpp, and of dequant_tensor_row, src/cli/main.cpp:36-261): host bytes of
 * N rows x K values in, fp32 [n_rows][K] out for rows row0..row0+n_rows-1.  The bytes go
 * through the same pack-into-HBM step as every weight, so this also checks the re-layout. */
GGB_API int ggb_dequant_rows(ggb_handle h, uint32_t type, const void* host_bytes, int64_t N, int K,
                             int64_t row0, int64_t n_rows, float* host_out);

typedef struct ggb_weight_s* ggb_weight;

/* Pack a [N][K] matrix of the given type into HBM (what src/quant's decode_*_for_npu plus the
 * WeightCache of include/ggnpu/weight_cache.h:34-158 do for the NPU: one-time conversion of
 * GGUF bytes into the device's layout).  host_rows may be freed after the call returns. */
GGB_API int ggb_weight_upload(ggb_handle h, uint32_t type, int64_t N, int K, const void* host_rows, ggb_weight* out);
GGB_API void ggb_weight_free(ggb_handle h, ggb_weight w);
GGB_API size_t ggb_weight_bytes(ggb_weight w);

/* Packed-weight disk cache: the role of the reference's WeightCache + CompileCache for its NPU backend
 * (include/ggnpu/weight_cache.h:34-158, src/cache/cache.cpp:16-58): what is expensive to derive from the GGUF bytes is
 * kept in a file per tensor under cache_dir and found again by a key built as WeightCache::make_key does
 * (weight_cache.h:141-152): layout version, hash of model_id + tensor name, type, data size.  model_id is the caller's
 * fingerprint of the model file, e.g. "<path>:<file size>" (src/cli/main.cpp:1203-1210).  Here the file holds the tensor
 * in this library's HBM layout, so a hit is one read + one host-to-device copy, no repack kernels.  A file whose recorded
 * fingerprint of the source bytes differs from host_rows is treated as a miss and rewritten.  host_rows == NULL loads
 * from the cache only (GGB_NOT_FOUND on a miss).  *hit (optional) = 1 when the file was used. */
GGB_API int ggb_weight_upload_cached(ggb_handle h, const char* cache_dir, const char* model_id, const char* tensor_name,
                                     uint32_t type, int64_t N, int K, const void* host_rows, ggb_weight* out, int* hit);
/* The cache's key and file format, usable without a GPU (tools, tests). */
GGB_API int ggb_pack_cache_key(const char* model_id, const char* tensor_name, uint32_t type, uint64_t data_size, char* out, int cap);
GGB_API int ggb_pack_file_write(const char* path, uint32_t type, int64_t N, int K, int nb, int layout, const uint64_t* stream_off,
                                uint64_t src_fingerprint, const void* blob, uint64_t bytes);
GGB_API int ggb_pack_file_read(const char* path, uint32_t type, int64_t N, int K, uint64_t src_fingerprint, int* nb, int* layout,
                               uint64_t* stream_off, void* blob, uint64_t cap, uint64_t* bytes);

/* y[M][ldc] = x[M][lda] * W^T with DEVICE pointers on the handle's stream.  M <= 16: the exact-activation GEMVs
 * (rel-L2 <= 1e-5 against the reference's exact fp32 product; M of 3..16 streams the weights once for all rows);
 * M >= 17: the tcgen05 GEMM (fp16 operands).  epilogue: 0 store; 1 + bias[N]; 2 + resid[M][ldc].  gamma != NULL applies RMSNorm
 * (eps) to each x row first.  Asynchronous. */
GGB_API int ggb_gemv_device(ggb_handle h, ggb_weight w, const float* d_x, int M, int lda, float* d_y, int ldc,
                            int epilogue, const float* d_extra, const float* d_gamma, float eps);
/* Fused SwiGLU pair: y = silu(Wg x) * (Wu x)  (src/cli/main.cpp:3449-3479 in one pass). */
GGB_API int ggb_gemv_swiglu_device(ggb_handle h, ggb_weight w_gate, ggb_weight w_up, const float* d_x, int M, int lda,
                                   float* d_y, int ldc, const float* d_gamma, float eps);

/* Grouped-query attention of ONE query token over a paged bf16 KV cache, DEVICE pointers: the
 * GPU-native form of Backend::flash_attn (include/ggnpu/backend.h:155) plus the caller's GQA expand
 * (src/cli/main.cpp:3364-3383), which it makes unnecessary: each KV head is read once for all the
 * query heads that share it.  q [n_head][head_dim] f32 already rotated; k_cache / v_cache are bf16
 * [pages][n_kv][page][head_dim] (K stored after RoPE); block_table[logical page] = physical page;
 * keys 0..pos are attended with scale 1/sqrt(head_dim); out [n_head][head_dim] f32.  The context is
 * split across CTAs and merged by a second kernel through a scratch buffer owned by the handle
 * (allocated with cudaMalloc on first need and when it must grow).  Asynchronous on the handle's
 * stream. */
typedef struct ggb_attn_paged_params {
    const float* q;
    const void* k_cache;
    const void* v_cache;
    const int32_t* block_table;
    float* out;
    int n_head, n_kv, head_dim;
    int page;      /* tokens per page */
    int n_pages;   /* logical pages in block_table */
    int pos;       /* position of the query token; attends keys 0..pos */
} ggb_attn_paged_params;
GGB_API int ggb_attn_paged_device(ggb_handle h, const ggb_attn_paged_params* p);

/* Causal attention of a prompt chunk: n_tok query tokens at positions p->pos .. p->pos + n_tok - 1,
 * q and out are [n_tok][n_head][head_dim]; token t attends keys 0 .. p->pos + t, all of which must
 * already be in the cache (p->pos + n_tok <= n_pages * page).  Replaces the per-token loop GQA expand
 * -> Backend::flash_attn (src/cli/main.cpp:3364-3383 -> cpu_ref.cpp:223-280) over the chunk.  With
 * page == 64 and head_dim 64 or 128 this is a tensor-core flash-attention kernel (Q and the softmax
 * weights rounded to bf16, fp32 accumulation); other geometries run the per-token kernel. */
GGB_API int ggb_attn_prefill_device(ggb_handle h, const ggb_attn_paged_params* p, int n_tok);

/* The same computation as ggb_attn_paged_device for callers that must not cause a device
 * allocation.  (No counterpart in the reference: its backends allocate buffers as they please.)
 * Who needs it: a host that gave all of the GPU's memory to its own pool at start-up, so a
 * cudaMalloc made by this library would fail or fight that pool; and a serving loop that cannot
 * afford the device-wide stall an allocation may bring.  This entry point calls neither cudaMalloc
 * nor cudaFree nor any routine that does: the per-split partial results go to a fixed array inside
 * the library (2.1 MB of device memory on every GPU that loads the library, held until the process
 * exits).  Limits: n_head <= 64 and n_head * splits * (head_dim + 2) <= 64 * 32 * 258 floats, where
 * splits = min(32, n_pages) rounded to whole pages; larger requests are refused with
 * GGB_INVALID_PARAM and a message.  The first call on each device looks up the array's device
 * address (a one-time set-up step): make that first call before any stream capture begins.  All
 * calls share the one array and it keeps whatever the previous call left; the kernels overwrite
 * every slot they later read, so nothing has to be cleared, but two calls whose kernels overlap on
 * the GPU (different handles or streams) would race on it -- keep them ordered. */
GGB_API int ggb_attn_paged_static(ggb_handle h, const ggb_attn_paged_params* p);

/* Mixture-of-experts FFN of ONE token (the qwen35moe branch of the reference's layer loop,
 * src/cli/main.cpp:3110-3193): router logits = router[n_expert][hidden] . x; the top_k experts by logit;
 * weights = softmax over just those; y = (resid +) sum_j w_j * down_j(silu(gate_j x) * up_j x)
 * (+ sigmoid(sh_gate_inp . x) * shared expert).  x is the FFN-normed hidden row.  The expert tensors are
 * the GGUF 3-D tensors uploaded whole with ggb_weight_upload as 2-D matrices: gate_exps / up_exps as
 * [n_expert * eff][hidden], down_exps as [n_expert * hidden][eff] (Q4_K or Q6_K); top_k <= 15, hidden <= 8192.
 * The chosen ids stay on the device: five launches (router + top-k in one), no host round trip.  All pointers are device memory; asynchronous on the
 * handle's stream.  sel_out / w_out (optional) receive the chosen ids [top_k] and weights [top_k + 1,
 * the last one the shared expert's gate]. */
typedef struct ggb_moe_params {
    const float* x;
    const float* resid;          /* optional [hidden]; may alias y */
    float* y;
    const float* router;         /* F32 [n_expert][hidden] */
    ggb_weight gate_exps, up_exps, down_exps;
    ggb_weight sh_gate, sh_up, sh_down;     /* shared expert: all three or none */
    const float* sh_gate_inp;    /* optional F32 [hidden] */
    int hidden, eff, eff_sh, n_expert, top_k;
    int32_t* sel_out;
    float* w_out;
    /* Expert parallel (ep_local > 0; the handle must belong to a group, ggb_tp_init): this rank's expert tensors
     * hold experts [ep_first, ep_first + ep_local) only; the router (replicated) still scores all n_expert.  Each
     * rank streams just the chosen experts it holds, rank 0 adds the residual and the shared expert, and the
     * partial rows are summed over the group (the batch-1 form of dispatch / combine), so every rank ends with
     * the same y.  sel_out / w_out report the global choice on every rank. */
    int ep_first, ep_local;
    /* Optional fused FFN norm: with gamma != NULL, x is the RAW hidden row and the operator works on
     * rms_norm(x, eps) * gamma (src/cli/main.cpp:3109), applied inside the router and expert kernels.  x must not
     * alias y when a shared expert is given (the shared expert reads x after the routed experts wrote y). */
    const float* gamma;
    float eps;
} ggb_moe_params;
GGB_API int ggb_moe_ffn_device(ggb_handle h, const ggb_moe_params* p);

/* One token of a Gated DeltaNet (linear attention) layer after its projections, the qwen35 / qwen35moe
 * branch of the reference's layer loop, src/cli/main.cpp:2925-3023: causal depthwise conv (conv_k taps) +
 * SiLU over mixed = [q: n_khead*sk | k: n_khead*sk | v: n_vhead*sk] with a rolling state of the previous
 * conv_k - 1 inputs; per key head L2 norm of q and k (q also / sqrt(sk)); per value head h (key head
 * h % n_khead): beta = sigmoid(braw), g = exp(ssm_a * softplus(araw + dt_bias)), S *= g, pred = S^T k,
 * delta = beta (v - pred), S += k (x) delta, o = S^T q; out = rms_norm(o) * ssm_norm * silu(zgate).
 * All pointers are device memory (F32); conv_state [(conv_k-1)][conv_dim] and rec_state
 * [n_vhead][sk][sk] are updated in place; asynchronous on the handle's stream.  sk is 64 or 128. */
typedef struct ggb_deltanet_params {
    const float* mixed;
    const float* zgate;
    const float* araw;
    const float* braw;
    const float* conv_w;     /* [conv_dim][conv_k], newest tap last */
    const float* ssm_a;      /* [n_vhead], stored as -exp(A_log) */
    const float* dt_bias;
    const float* ssm_norm;   /* [sk] */
    float* conv_state;
    float* rec_state;
    float* out;              /* [n_vhead * sk] */
    int n_khead, n_vhead, sk, conv_k;
    float rms_eps;
} ggb_deltanet_params;
GGB_API int ggb_deltanet_step_device(ggb_handle h, const ggb_deltanet_params* p);

/* Gated full attention (qwen35 / qwen35moe attention layers, src/cli/main.cpp:3035-3105): the attn_q projection
 * emits per query head [query(head_dim) | gate(head_dim)].  ggb_qgate_split_device copies the query halves into
 * contiguous heads d_q[n_head][head_dim] for the attention entry points (:3054-3060; the gate halves stay where
 * they are); ggb_attn_gate_device multiplies the attention output by sigmoid(gate), reading the gate in place
 * from the projection (:3098).  QK-norm, the partial NeoX rotation and head_dim 256 are covered by ggb_rms_norm,
 * ggb_rope (rope_dims < n_dims) and the paged attention entry points.  Device pointers, asynchronous. */
GGB_API int ggb_qgate_split_device(ggb_handle h, const float* d_qg, float* d_q, int n_head, int head_dim);
GGB_API int ggb_attn_gate_device(ggb_handle h, float* d_out, const float* d_qg, int n_head, int head_dim);

/* The handle's CUDA stream (a cudaStream_t), for callers that time or order work on it. */
GGB_API void* ggb_stream(ggb_handle h);
/* Number of kernels this library has launched on the handle so far. */
GGB_API uint64_t ggb_launch_count(ggb_handle h);

/* ---- tensor parallel group (no counterpart in the reference, which drives one device) ----
 * One process per GPU.  Rank 0 obtains a 128-byte id with ggb_tp_unique_id and hands it to the other
 * ranks by any host channel; every rank then calls ggb_tp_init on its handle (a collective call: it
 * returns when all `size` ranks have joined; NCCL over NVLink / NVSwitch underneath).  A model created
 * on such a handle is one shard of a tensor-parallel model: see ggb_model_desc. */
GGB_API int ggb_tp_unique_id(void* id128);
GGB_API int ggb_tp_init(ggb_handle h, const void* id128, int rank, int size);
/* Optional, after ggb_tp_init: a one-shot all-reduce over peer memory for small messages (the 16 KB partial
 * rows of a decode step, where NCCL's latency dominates).  Every rank calls ggb_tp_ipc_handle (allocates
 * its exchange region, returns a 64-byte CUDA IPC handle), the ranks exchange the handles over the host
 * channel, and every rank calls ggb_tp_attach_peers with all `size` handles in rank order (its own entry is
 * ignored).  From then on, in groups of 4 or more ranks (where it is faster than NCCL; GGB_TP_ONE_SHOT=1 in the
 * environment lowers that to 2), sums of up to 16384 floats use the peer-memory kernel, larger ones NCCL.
 * All ranks of a group must be processes on one machine whose GPUs can reach each other (NVLink / NVSwitch). */
GGB_API int ggb_tp_ipc_handle(ggb_handle h, void* handle64);
GGB_API int ggb_tp_attach_peers(ggb_handle h, const void* handles);
/* Sum of d_buf[0..count) over the group, in place, asynchronous on the handle's stream. */
GGB_API int ggb_tp_all_reduce_device(ggb_handle h, float* d_buf, int64_t count);

/* ---- whole-model path (generic llama / qwen2 / qwen3 graph, src/cli/main.cpp:3235-3512) ---- */

typedef struct ggb_model_desc {
    int n_layer, hidden, n_head, n_kv, head_dim, ffn, vocab, ctx;
    float rms_eps, rope_base, rope_scale;
    int rope_neox;   /* 1: split-half pairs (qwen3); 0: adjacent pairs (llama, qwen2) */
    int kv_page;     /* tokens per KV page; 0 = default (64) */
    int conv_taps;   /* lfm2 only: taps of the gated short convolution (lfm2.shortconv.l_cache, src/cli/main.cpp:2146-2147);
                        0 = the reference's default (3); at most 8 */
} ggb_model_desc;
/* lfm2 (src/cli/main.cpp:2145-2167, 2680-2856): a layer that is given GGB_T_SC_IN_PROJ / GGB_T_SC_OUT_PROJ / GGB_T_SC_CONV
 * instead of the attention tensors runs the gated short convolution: [B | C | x] = in_proj(norm(h)); bx = B * x; y = C *
 * (causal depthwise convolution over the last conv_taps values of bx); h += out_proj(y).  The layer's state (the previous
 * conv_taps - 1 values of bx) lives in device memory and returns to zero whenever a call starts at position 0.  Attention
 * layers take GGB_T_Q_NORM / GGB_T_K_NORM; the final norm (token_embd_norm) goes to GGB_T_OUTPUT_NORM.  rope_neox = 1 and
 * rope_base = lfm2.rope.freq_base give the rotation the branch asks its backend for (:2250-2268); the reference's CPU
 * backend ignores both (cpu_ref.cpp:158-174: adjacent pairs, base 10000), which rope_neox = 0, rope_base = 10000
 * reproduces.  Such a model runs one sequence on one GPU; ggb_model_generate_spec refuses it as the reference does (:2299-2301). */
/* On a handle that belongs to a tensor-parallel group of `size` ranks the description and the tensors
 * are those of ONE SHARD (Megatron-style): n_head, n_kv and ffn are the full model's divided by size;
 * attn_q/k/v, ffn_gate/up and their biases hold this rank's rows (column parallel); attn_output and
 * ffn_down hold this rank's K range of every row (row parallel, a whole number of quant blocks);
 * GGB_T_OUTPUT holds rows [rank * vocab / size, (rank + 1) * vocab / size) of the output matrix and must
 * be given explicitly (also for tied embeddings); token_embd, the norms, hidden, vocab and ctx are the
 * full model's.  The library sums the partial results of attn_output and ffn_down over the group
 * (all-reduce) and gathers the logits slices (all-gather), so every rank ends a step with the full
 * logits and the same next token.  ggnpu_b200/tp.py cuts a full GGUF tensor set into such shards. */

typedef struct ggb_model_s* ggb_model;

enum ggb_tensor_slot {
    GGB_T_TOKEN_EMBD = 0, GGB_T_OUTPUT = 1, GGB_T_OUTPUT_NORM = 2, GGB_T_ROPE_FREQS = 3,
    GGB_T_ATTN_NORM = 10, GGB_T_ATTN_Q = 11, GGB_T_ATTN_K = 12, GGB_T_ATTN_V = 13, GGB_T_ATTN_OUT = 14,
    GGB_T_FFN_NORM = 15, GGB_T_FFN_GATE = 16, GGB_T_FFN_UP = 17, GGB_T_FFN_DOWN = 18,
    GGB_T_BIAS_Q = 19, GGB_T_BIAS_K = 20, GGB_T_BIAS_V = 21, GGB_T_Q_NORM = 22, GGB_T_K_NORM = 23,
    /* lfm2 short-convolution layers: in_proj [3 hidden][hidden], out_proj [hidden][hidden], conv F32 [hidden][conv_taps] */
    GGB_T_SC_IN_PROJ = 24, GGB_T_SC_OUT_PROJ = 25, GGB_T_SC_CONV = 26
};

GGB_API int ggb_model_create(ggb_handle h, const ggb_model_desc* desc, ggb_model* out);
GGB_API void ggb_model_destroy(ggb_model m);
/* Optional, before the tensors are set: route the model's matrices through the packed-weight disk cache
 * (ggb_weight_upload_cached) under cache_dir, keyed by model_id = the caller's fingerprint of the model file
 * (src/cli/main.cpp:1203-1210).  ggb_model_cache_stats reports how many matrices came from packed files. */
GGB_API int ggb_model_set_cache(ggb_model m, const char* cache_dir, const char* model_id);
GGB_API int ggb_model_cache_stats(ggb_model m, int* hits, int* misses);
/* One tensor of the model: matrices as GGUF rows ([N][K] of `type`), vectors as F32. */
GGB_API int ggb_model_set_tensor(ggb_model m, int slot, int layer, uint32_t type, int64_t N, int K, const void* host_data);
/* Allocate KV pages, build the RoPE table (RopeCache::build, src/cli/main.cpp:665-692) and
 * capture the decode graph.  Call once after all tensors are set. */
GGB_API int ggb_model_finalize(ggb_model m);
/* Forward over n_tok prompt tokens at positions pos0.. (writes KV); logits of the LAST row to
 * host_logits (may be NULL), greedy token to *next_token (may be NULL). */
GGB_API int ggb_model_prefill(ggb_model m, const int32_t* host_tokens, int n_tok, int pos0, float* host_logits, int32_t* next_token);
/* One decode step from host buffers: token in, logits (optional) and greedy next token out.  A host_logits buffer in
 * page-locked memory (cudaHostAlloc / cudaHostRegister) receives the device copy directly; any other buffer is filled
 * through the model's own page-locked staging buffer and one host copy. */
GGB_API int ggb_model_decode(ggb_model m, int32_t token, int pos, float* host_logits, int32_t* next_token);
/* n greedy decode steps with the token fed back on the device (no host round trip inside);
 * the n generated ids land in host_out afterwards. */
GGB_API int ggb_model_generate(ggb_model m, int32_t first_token, int pos0, int n, int32_t* host_out);
/* Greedy generation with prompt-lookup speculative decoding, the reference's GGNPU_SPEC_DECODE mode (drafter
 * lookup_draft, src/cli/main.cpp:397-415; block building :2343-2349; verification :3531-3588).  history holds all
 * tokens so far (prompt + generated), its last element is the token to feed at position pos0.  Each step drafts up
 * to draft_k (1..15) tokens by matching the last 3, 2 or 1 tokens against the history, runs the block
 * [last, drafts] as ONE forward, takes the arg-max of every row and commits the longest matching draft prefix plus
 * one token, so the stream equals plain greedy decoding wherever the two forwards agree on the arg-max.  n tokens
 * land in host_out; stats (optional, 4 ints) = steps, drafted, accepted, generated.  One GPU only. */
GGB_API int ggb_model_generate_spec(ggb_model m, const int32_t* history, int n_history, int pos0, int n, int draft_k,
                                    int32_t* host_out, int32_t* stats);
/* n decode steps with temperature sampling and device-side feedback: sample_token of the reference CLI
 * (src/cli/main.cpp:827-864) applied to each step's logits where they lie in HBM.  *seed is the CLI's rng_seed:
 * it advances exactly as the reference's does (one std::mt19937 per call, re-seeded from its own first output), so
 * a run split over several calls continues the same stream.  temp <= 0 is greedy decoding (ggb_model_generate). */
GGB_API int ggb_model_generate_sampled(ggb_model m, int32_t first_token, int pos0, int n, float temp, uint64_t* seed, int32_t* host_out);
/* Several sequences on one set of weights (no counterpart in the reference, whose CLI runs one sequence: the
 * batch-16 decode scenario needs it).  ggb_model_set_sequences(n_seq <= 16), before finalize, reserves n_seq KV
 * streams of ctx tokens each.  ggb_model_select_sequence picks the stream that prefill / decode / read_kv work on
 * (default 0; ggb_model_generate and ggb_model_generate_spec run on stream 0 only).
 * ggb_model_decode_batch: ONE forward in which row r is the next token of sequence r at position pos[r]; every
 * matrix is streamed once for all rows, each row attends to its own KV stream.  Logits [n_seq][vocab] to host_logits
 * (may be NULL), greedy tokens to next_tokens (may be NULL).  ggb_model_generate_batch: n such steps with tokens and
 * positions fed back on the device (one CUDA graph per step); host_out[step * n_seq + r]. */
GGB_API int ggb_model_set_sequences(ggb_model m, int n_seq);
GGB_API int ggb_model_select_sequence(ggb_model m, int seq);
GGB_API int ggb_model_decode_batch(ggb_model m, const int32_t* tokens, const int32_t* pos, int n_seq, float* host_logits, int32_t* next_tokens);
GGB_API int ggb_model_generate_batch(ggb_model m, const int32_t* first_tokens, const int32_t* pos0, int n_seq, int n, int32_t* host_out);
/* Read back one KV row [n_kv][head_dim] as f32 (tests). */
GGB_API int ggb_model_read_kv(ggb_model m, int layer, int pos, int want_v, float* host_out);
/* Algorithmic HBM bytes one decode step at position pos reads+writes (weights once + KV). */
GGB_API uint64_t ggb_model_decode_bytes(ggb_model m, int pos);

/* ---- sampling ----
 * sample_token, src/cli/main.cpp:827-864 (the CLI's sampler; not a Backend member).  temp <= 0: index of the first
 * maximum.  temp > 0: softmax((v - max) / temp) in float, then std::discrete_distribution driven by
 * std::mt19937(*seed); *seed becomes the generator's first output, as in the reference.  The exponentials, both
 * normalisations and the search run on the GPU; the chosen index equals the reference's unless the uniform draw lies
 * within float rounding (~1e-7 relative) of the boundary between two tokens' cumulative probabilities.
 * ggb_sample takes host logits, ggb_sample_device logits already in HBM. */
GGB_API int ggb_sample(ggb_handle h, const float* host_logits, int n, float temp, uint64_t* seed, int32_t* token);
GGB_API int ggb_sample_device(ggb_handle h, const float* d_logits, int n, float temp, uint64_t* seed, int32_t* token);

/* ---- whole-model path, qwen35 / qwen35moe graph (src/cli/main.cpp:2859-3232) ----
 * Gated DeltaNet layers (those given an ssm_conv1d tensor, :2207-2213) and gated full-attention layers, a
 * mixture-of-experts FFN in every layer.  The architecture is a recurrence, so the reference feeds it one token
 * per forward, the prompt included (:2327); so does this path: one CUDA graph per token, a prompt being the graph
 * replayed over a device-resident token list (no host round trip between tokens).  Metadata as the reference
 * reads it (:2181-2200): head_dim = attention.key_length, rope_dim = rope.dimension_count (leading dims of a head
 * that rotate, NeoX pairs), sk = ssm.state_size, n_vhead = ssm.inner_size / sk, n_khead = ssm.group_count,
 * eff = expert_feed_forward_length (routed and shared experts alike). */
typedef struct ggb_q35_desc {
    int n_layer, hidden, n_head, n_kv, head_dim, rope_dim, conv_k, sk, n_vhead, n_khead, n_expert, top_k, eff, vocab, ctx;
    float rms_eps, rope_base;
    int kv_page;     /* tokens per KV page; 0 = default (64) */
} ggb_q35_desc;
/* On a handle that belongs to a group of `size` ranks (ggb_tp_init) the model is EXPERT parallel: the three
 * *_exps tensors hold this rank's n_expert / size experts, rank r owning experts [r n_expert / size, ...); every
 * other tensor is replicated and n_expert in the description stays the full count.  Each rank runs the mixers,
 * streams only the chosen experts it owns, and the partial FFN rows are summed over the group, so every rank ends
 * a step with the same logits and token. */
typedef struct ggb_q35_model_s* ggb_q35_model;
enum ggb_q35_slot {
    GGB_Q35_TOKEN_EMBD = 0, GGB_Q35_OUTPUT = 1, GGB_Q35_OUTPUT_NORM = 2,
    GGB_Q35_ATTN_NORM = 10, GGB_Q35_POST_NORM = 11,
    /* DeltaNet layers: attn_qkv [2 n_khead sk + n_vhead sk][hidden], attn_gate [n_vhead sk][hidden], ssm_alpha / ssm_beta
     * F32 [n_vhead][hidden], ssm_conv1d F32 [conv_dim][conv_k] (newest tap last), ssm_a / ssm_dt.bias F32 [n_vhead],
     * ssm_norm F32 [sk], ssm_out [hidden][n_vhead sk] */
    GGB_Q35_SSM_QKV = 20, GGB_Q35_SSM_GATE = 21, GGB_Q35_SSM_ALPHA = 22, GGB_Q35_SSM_BETA = 23, GGB_Q35_SSM_CONV = 24,
    GGB_Q35_SSM_A = 25, GGB_Q35_SSM_DT_BIAS = 26, GGB_Q35_SSM_NORM = 27, GGB_Q35_SSM_OUT = 28,
    /* attention layers: attn_q [2 n_head head_dim][hidden] (per head query | gate), attn_k / attn_v, attn_output, QK norms */
    GGB_Q35_ATTN_Q = 30, GGB_Q35_ATTN_K = 31, GGB_Q35_ATTN_V = 32, GGB_Q35_ATTN_OUT = 33, GGB_Q35_Q_NORM = 34, GGB_Q35_K_NORM = 35,
    /* every layer: ffn_gate_inp F32 [n_expert][hidden], ffn_{gate,up}_exps [n_expert eff][hidden], ffn_down_exps
     * [n_expert hidden][eff], the shared expert's three matrices and its gate vector F32 [hidden] */
    GGB_Q35_ROUTER = 40, GGB_Q35_GATE_EXPS = 41, GGB_Q35_UP_EXPS = 42, GGB_Q35_DOWN_EXPS = 43, GGB_Q35_SH_GATE = 44,
    GGB_Q35_SH_UP = 45, GGB_Q35_SH_DOWN = 46, GGB_Q35_SH_GATE_INP = 47
};
GGB_API int ggb_q35_create(ggb_handle h, const ggb_q35_desc* desc, ggb_q35_model* out);
GGB_API void ggb_q35_destroy(ggb_q35_model m);
/* Matrices as GGUF rows ([N][K] of `type`; expert tensors whole, experts stacked along N); F32 tensors with N * K
 * equal to their element count (vectors: K = 1). */
GGB_API int ggb_q35_set_tensor(ggb_q35_model m, int slot, int layer, uint32_t type, int64_t N, int K, const void* host_data);
GGB_API int ggb_q35_finalize(ggb_q35_model m);
/* Zero the recurrent and convolution states (a new sequence; the KV cache needs no clearing). */
GGB_API int ggb_q35_reset(ggb_q35_model m);
/* n_tok prompt tokens at positions pos0.., one graph replay each; logits of the last (optional) and the greedy token. */
GGB_API int ggb_q35_prefill(ggb_q35_model m, const int32_t* host_tokens, int n_tok, int pos0, float* host_logits, int32_t* next_token);
GGB_API int ggb_q35_decode(ggb_q35_model m, int32_t token, int pos, float* host_logits, int32_t* next_token);
/* n greedy steps with the token fed back on the device. */
GGB_API int ggb_q35_generate(ggb_q35_model m, int32_t first_token, int pos0, int n, int32_t* host_out);
/* Recurrent state [n_vhead][sk][sk] of a DeltaNet layer (tests). */
GGB_API int ggb_q35_read_state(ggb_q35_model m, int layer, float* host_out);
/* Algorithmic HBM bytes of one decode step at position pos (mixer weights, router, the top_k + shared experts,
 * recurrent and conv states read and written, KV of the attention layers, logits matrix). */
GGB_API uint64_t ggb_q35_decode_bytes(ggb_q35_model m, int pos);

#ifdef __cplusplus
}
#endif
#endif /* GGB200_H */
