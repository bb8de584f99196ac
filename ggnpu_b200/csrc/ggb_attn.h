// Argument blocks of the paged-KV attention kernels (ggb_attn.cu).
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace ggb {

struct Context;

struct KvAppendArgs {
    float* q;                 // [n_tok][n_head][hd]  rotated in place
    float* k;                 // [n_tok][n_kv][hd]    pre-RoPE keys (read)
    const float* v;           // [n_tok][n_kv][hd]
    __nv_bfloat16* k_cache;   // one layer: [pages][n_kv][page][hd]
    __nv_bfloat16* v_cache;
    const int32_t* block_table;   // logical page -> physical page
    const float* cos_tab;     // [ctx][hd/2]
    const float* sin_tab;
    const float* q_norm;      // optional [hd]
    const float* k_norm;
    const int32_t* d_pos;     // device scalar: position of token 0 (nullptr => pos0)
    int pos0;
    int n_head, n_kv, head_dim, page, neox;
    float eps;
    // batched sequences (row t is the next token of sequence t): seq_pos[t] is row t's position and its block table
    // starts at block_table + t * seq_table_stride; null / 0: one sequence, rows at consecutive positions
    const int32_t* seq_pos;
    int seq_table_stride;
    int rot_dims;             // leading dims of each head that rotate (0: all head_dim); tables hold rot_dims / 2 entries per position
    int norm_f32;             // 1: QK-norm sum of squares in float (qwen35: src/cli/main.cpp:896-901) instead of double
};

struct AttnPagedArgs {
    const float* q;           // [n_tok][n_head][hd] post-RoPE
    const __nv_bfloat16* k_cache;
    const __nv_bfloat16* v_cache;
    const int32_t* block_table;
    float* partial;           // [n_tok][n_head][n_splits][hd + 2] scratch
    int partial_tok_cap;      // tokens `partial` has room for (0: the caller sized it for this call)
    float* out;               // [n_tok][n_head][hd]
    const int32_t* d_pos;
    int pos0;
    const int32_t* seq_pos;   // batched sequences: position of row t (then d_pos / pos0 are unused) ...
    int seq_table_stride;     // ... and row t's block table = block_table + t * seq_table_stride
    int n_head, n_kv, head_dim, page, n_splits, pages_per_split;
    // fused RoPE + KV append for a single-token step (fuse != 0): q is then PRE-RoPE, k_new / v_new are
    // this token's projections [n_kv][hd]; the kernel rotates, stores into the cache and attends.
    int fuse, neox;
    int skip_merge;           // 1: leave the per-split partials for the consumer (the output projection merges them)
    // optional: one counter per (token, KV head), zero before the first launch.  The CTA of a (token, KV head) that
    // finishes last merges the splits of its query heads itself and writes `out`, so neither the merge kernel nor a
    // merging consumer is needed (the counter is back at zero when the launch ends)
    int head_split;           // > 1: the query heads of a KV head are dealt to this many CTAs (grid.x = n_kv * head_split); no merge_ticket then
    int* merge_ticket;
    int merge_min_splits;     // merge (in the kernel with merge_ticket, else in the merge kernel) only when at least this many splits are visible (0: always)
    const float* k_new;
    const float* v_new;
    __nv_bfloat16* k_cache_w;
    __nv_bfloat16* v_cache_w;
    const float* cos_tab;
    const float* sin_tab;
    const float* q_norm;
    const float* k_norm;
    float eps;
};

int launch_rope_append(Context* c, const KvAppendArgs& a, int n_tok, cudaStream_t s);
int launch_attn_paged(Context* c, const AttnPagedArgs& a, int n_tok, cudaStream_t s);
int launch_attn_prefill(Context* c, const AttnPagedArgs& a, int n_tok, cudaStream_t s);   // ggb_attn_prefill.cu; GGB_NOT_FOUND: geometry not covered
size_t attn_partial_floats(int n_tok, int n_head, int n_splits, int head_dim);
void attn_split_geometry(int n_pages, int* n_splits, int* pages_per_split);
void attn_split_geometry(int n_pages, int n_kv, int* n_splits, int* pages_per_split);      // up to 64 splits when n_kv <= 2

}  // namespace ggb
