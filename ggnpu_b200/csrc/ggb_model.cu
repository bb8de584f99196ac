// C ABI, part 2: the generic decoder graph of the reference CLI (src/cli/main.cpp:2367-2375 embed,
// :3235-3500 layer loop, :3504-3512 final norm, :3593-3599 logits, :827-838 greedy) kept entirely in
// HBM: packed weights, paged bf16 KV cache, f32 activations, one CUDA graph per decode step.
#include <cuda_bf16.h>
#include <math.h>

#include <stdio.h>
#include <stdlib.h>

#include <cmath>
#include <map>
#include <memory>

#include "ggb_attn.h"
#include "ggb_decode_step.h"
#include "ggb_internal.h"

using namespace ggb;


namespace {

struct Layer {
    DeviceWeight *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr, *gate = nullptr, *up = nullptr, *down = nullptr;
    float *attn_norm = nullptr, *ffn_norm = nullptr, *bq = nullptr, *bk = nullptr, *bv = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    // lfm2 gated short-convolution layer (instead of q / k / v / o): projections, taps [hidden][conv_taps], state [conv_taps - 1][hidden]
    DeviceWeight *sc_in = nullptr, *sc_out = nullptr;
    float *sc_conv = nullptr, *sc_state = nullptr;
    bool conv() const { return sc_in != nullptr; }
};

// Prompt tokens per forward pass.  The reference chunks at 256 (main.cpp:2326); results do not depend
// on the chunking.  With the tensor-core attention available a chunk is up to 2048 tokens (each GEMM
// then dequantises its weights once per 2048 tokens); otherwise 256, which bounds the per-token
// attention kernel's split scratch.
constexpr int kSmallChunk = 256, kLargeChunk = 2048;
constexpr int kMergeInAttn = 12;    // visible context splits from which the attention kernel merges them itself
constexpr int kSpecRows = 16;       // a verified block: the fed token + up to 15 drafted ones (src/cli/main.cpp:2305-2308)

}  // namespace

struct ggb_model_s {
    int chunk = kSmallChunk;
    Context* c = nullptr;
    ggb_model_desc d{};
    DeviceWeight *tok_embd = nullptr, *output = nullptr;
    float* output_norm = nullptr;
    std::vector<float> rope_ff;
    std::vector<Layer> layers;
    std::vector<void*> owned;            // cudaMalloc'd vectors and buffers
    bool finalized = false;
    // KV cache
    __nv_bfloat16 *k_cache = nullptr, *v_cache = nullptr;
    int32_t* block_table = nullptr;
    int page = 64, n_pages = 0, n_splits = 1, pages_per_split = 1;
    // single-token steps of a long context cut it finer (up to 128 splits, one 64-key chunk per CTA where possible: every
    // CTA's K/V loads are then in flight from its first instruction); several rows per step keep the coarser cut
    int n_splits1 = 1, pages_per_split1 = 1;
    size_t kv_layer_elems = 0;
    float *cos_tab = nullptr, *sin_tab = nullptr;
    // activations
    float *x = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *act = nullptr, *logits = nullptr;
    float *partial = nullptr, *amax_partial = nullptr;
    int* attn_ticket = nullptr;          // per (token, KV head): the split that finishes last merges (AttnPagedArgs::merge_ticket)
    uint16_t* act_img = nullptr;         // SwiGLU output of a prompt chunk as the down projection's fp16 tile image
    bool tc_images = false;              // prompt chunks pass activations between GEMMs as tile images
    int32_t *d_tokens = nullptr, *d_pos = nullptr, *d_next = nullptr, *d_gen = nullptr, *d_step = nullptr;
    // pinned host staging
    int32_t* h_io = nullptr;             // [0]=token [1]=pos [2]=next
    float* h_logits = nullptr;
    cudaGraphExec_t decode_graph = nullptr;
    uint64_t launches_per_step = 0;
    std::string cache_dir, cache_model_id;     // packed-weight disk cache for the matrices (empty: none)
    int cache_hits = 0, cache_misses = 0;
    // speculative verification: logits and greedy token of every row of a block of up to kSpecRows tokens
    float* logits_rows = nullptr;
    int32_t* d_rows_next = nullptr;
    // batched sequences: n_seq KV streams of n_pages pages each (sequence b owns logical pages [b * n_pages, (b + 1) * n_pages)
    // of the block table); cur_seq is the stream the single-sequence entry points work on
    int n_seq = 1, cur_seq = 0;
    int32_t *d_seq_pos = nullptr, *d_gen_batch = nullptr;
    std::map<int, cudaGraphExec_t> batch_graphs;       // one captured step per batch size
    std::map<int, uint64_t> batch_launches;
    // temperature sampling (ggb_model_generate_sampled): scratch, the step's uniform draws, the captured step
    void* samp_scratch = nullptr;
    float* d_temp = nullptr;
    double* d_u = nullptr;
    int32_t* d_sampled = nullptr;
    cudaGraphExec_t sample_graph = nullptr;
    uint64_t sample_launches = 0;
    // lfm2: any short-convolution layer; [B | C | x] rows of its in_proj and the convolution's output rows
    bool has_conv = false;
    int conv_taps = 3;
    float *bcx = nullptr, *yconv = nullptr;
    // persistent decode-step kernel (single-token steps of an all-Q4_K / Q6_K model on one GPU)
    bool use_step = false;
    StepArgs step{};
    StepLayer* d_step_layers = nullptr;
    unsigned* d_step_bar = nullptr;
};

namespace {

template <class T>
int dev_alloc(ggb_model m, T** p, size_t count) {
    void* v = nullptr;
    int st = cuda_status(m->c, cudaMalloc(&v, sizeof(T) * std::max<size_t>(count, 1)), "cudaMalloc(model)");
    if (st != GGB_OK) return st;
    m->owned.push_back(v);
    *p = static_cast<T*>(v);
    return GGB_OK;
}

// One thread per sequence: the greedy token becomes the sequence's next input, its position advances.
__global__ void feedback_batch_kernel(const int32_t* next, int32_t* tokens, int32_t* seq_pos, int32_t* gen, int32_t* step, int n_seq, int gen_cap) {
    const int r = threadIdx.x, s = step[0];
    if (r < n_seq) {
        if (s < gen_cap) gen[static_cast<size_t>(s) * n_seq + r] = next[r];
        tokens[r] = next[r];
        seq_pos[r] += 1;
    }
    __syncthreads();
    if (r == 0) step[0] = s + 1;
}

__global__ void feedback_kernel(const int32_t* next, int32_t* tokens, int32_t* pos, int32_t* gen, int32_t* step, int gen_cap) {
    const int s = step[0];
    if (s < gen_cap) gen[s] = next[0];
    tokens[0] = next[0];
    pos[0] += 1;
    step[0] = s + 1;
}

GemvArgs gemv_args(const DeviceWeight* w, const float* x, int M, int lda, float* y, int ldc) {
    GemvArgs a{};
    a.w = w->w; a.x = x; a.M = M; a.lda = lda; a.y = y; a.ldc = ldc; a.epi = EPI_STORE;
    return a;
}

#define M_TRY(expr) do { int _st = (expr); if (_st != GGB_OK) return _st; } while (0)

// Enqueue one forward over n_tok tokens whose ids are in m->d_tokens.  Positions start at
// d_pos[0] when dev_pos, else at pos0.  Ends with logits of the last row and its argmax in d_next.
// batch: row r is instead the next token of sequence r at position d_seq_pos[r] (its own KV stream), and the
// pass ends with the logits and greedy token of every row (logits_rows, d_rows_next).
int enqueue_forward(ggb_model m, int n_tok, bool dev_pos, int pos0, bool all_rows = false, bool batch = false) {
    Context* c = m->c;
    cudaStream_t s = c->stream;
    const ggb_model_desc& d = m->d;
    const int H = d.hidden, hd = d.head_dim, qd = d.n_head * hd, kvd = d.n_kv * hd, F = d.ffn;
    const int32_t* dpos = dev_pos ? m->d_pos : nullptr;
    const int32_t* table = m->block_table + (batch ? 0 : static_cast<size_t>(m->cur_seq) * m->n_pages);
    const bool single = n_tok == 1 && !batch;
    if (batch) all_rows = true;
    M_TRY(launch_gather_rows(c, m->tok_embd->w, m->d_tokens, n_tok, m->x, H, s));
    if (m->use_step && single && m->cur_seq == 0) {
        // all layers and the logits in one persistent kernel
        m->step.attn.d_pos = dpos; m->step.attn.pos0 = pos0;
        M_TRY(launch_decode_step(c, m->step, hd, s));
        return launch_argmax(c, m->logits, d.vocab, m->d_next, m->amax_partial, s);
    }
    for (int L = 0; L < d.n_layer; ++L) {
        const Layer& l = m->layers[L];
        const bool tp = c->tp_size > 1;
        const int resid_epi = (!tp || c->tp_rank == 0) ? EPI_RESIDUAL : EPI_STORE;
        GemvArgs a{};
        if (l.conv()) {
            // gated short convolution (src/cli/main.cpp:2693-2732): in_proj with the norm in its prologue, the per-channel
            // convolution over the rows in order, out_proj with the residual in its epilogue
            a = gemv_args(l.sc_in, m->x, n_tok, H, m->bcx, 3 * H);
            a.gamma = l.attn_norm; a.eps = d.rms_eps;
            M_TRY(launch_gemv(c, a, s));
            M_TRY(launch_shortconv(c, m->bcx, l.sc_conv, l.sc_state, m->yconv, n_tok, H, m->conv_taps, s));
            a = gemv_args(l.sc_out, m->yconv, n_tok, H, m->x, H);
            a.epi = EPI_RESIDUAL; a.resid = m->x;
            M_TRY(launch_gemv(c, a, s));
        } else {
        a = gemv_args(l.q, m->x, n_tok, H, m->q, qd);
        a.gamma = l.attn_norm; a.eps = d.rms_eps;
        if (l.bq) { a.epi = EPI_ADD_BIAS; a.bias = l.bq; }
        const bool biases_agree = (l.bq != nullptr) == (l.bk != nullptr) && (l.bq != nullptr) == (l.bv != nullptr);
        const bool same_kind = l.q->w.type == l.k->w.type && l.q->w.type == l.v->w.type && l.q->w.layout == l.k->w.layout && l.q->w.layout == l.v->w.layout;
        if (biases_agree && ((n_tok <= 2 && l.q->w.layout == 1 && l.k->w.layout == 1 && l.v->w.layout == 1) || (n_tok == 1 && same_kind))) {
            // q, k and v in one launch: three matrices stacked along N share the normalised x
            a.n_cat = 2;
            a.cat_w[0] = l.k->w; a.cat_y[0] = m->k; a.cat_bias[0] = l.bk; a.cat_ldc[0] = kvd;
            a.cat_w[1] = l.v->w; a.cat_y[1] = m->v; a.cat_bias[1] = l.bv; a.cat_ldc[1] = kvd;
            M_TRY(launch_gemv(c, a, s));
        } else {
            // prompt chunk on the tensor-core GEMM: the q projection prepares the normalised fp16 tile
            // image of x, the k and v projections read the same image
            const bool img = m->tc_images && n_tok >= c->tc_min_m;
            M_TRY(launch_gemv(c, a, s));
            a = gemv_args(l.k, m->x, n_tok, H, m->k, kvd);
            a.gamma = l.attn_norm; a.eps = d.rms_eps;
            if (l.bk) { a.epi = EPI_ADD_BIAS; a.bias = l.bk; }
            if (img) a.x_img = c->d_xb;
            a.limbs_reuse = true;                 // 3..16 rows: the q projection's int8-limb image of the normalised x
            M_TRY(launch_gemv(c, a, s));
            a = gemv_args(l.v, m->x, n_tok, H, m->v, kvd);
            a.gamma = l.attn_norm; a.eps = d.rms_eps;
            if (l.bv) { a.epi = EPI_ADD_BIAS; a.bias = l.bv; }
            if (img) a.x_img = c->d_xb;
            a.limbs_reuse = true;
            M_TRY(launch_gemv(c, a, s));
        }

        KvAppendArgs ka{};
        ka.q = m->q; ka.k = m->k; ka.v = m->v;
        ka.k_cache = m->k_cache + static_cast<size_t>(L) * m->kv_layer_elems;
        ka.v_cache = m->v_cache + static_cast<size_t>(L) * m->kv_layer_elems;
        ka.block_table = table; ka.cos_tab = m->cos_tab; ka.sin_tab = m->sin_tab;
        ka.q_norm = l.q_norm; ka.k_norm = l.k_norm; ka.d_pos = dpos; ka.pos0 = pos0;
        ka.n_head = d.n_head; ka.n_kv = d.n_kv; ka.head_dim = hd; ka.page = m->page; ka.neox = d.rope_neox; ka.eps = d.rms_eps;
        if (!single && !batch) M_TRY(launch_rope_append(c, ka, n_tok, s));   // single-token steps (one per sequence) fuse this into attention

        AttnPagedArgs aa{};
        if (batch) { aa.seq_pos = m->d_seq_pos; aa.seq_table_stride = m->n_pages; }
        if (single || batch) {
            aa.fuse = 1; aa.neox = d.rope_neox; aa.k_new = m->k; aa.v_new = m->v;
            aa.k_cache_w = ka.k_cache; aa.v_cache_w = ka.v_cache; aa.cos_tab = m->cos_tab; aa.sin_tab = m->sin_tab;
            aa.q_norm = l.q_norm; aa.k_norm = l.k_norm; aa.eps = d.rms_eps;
        }
        aa.q = m->q; aa.k_cache = ka.k_cache; aa.v_cache = ka.v_cache; aa.block_table = table;
        aa.partial = m->partial; aa.partial_tok_cap = kSmallChunk; aa.out = m->att; aa.d_pos = dpos; aa.pos0 = pos0;
        static const bool no_ticket = getenv("GGB_NO_ATTN_MERGE") != nullptr;      // keep every merge out of the attention kernel
        const bool merge_in_attn = d.n_kv >= 4 && !no_ticket;
        const bool fine = single && merge_in_attn;                      // the fine cut relies on the in-kernel merge
        const int n_splits = fine ? m->n_splits1 : m->n_splits, pps = fine ? m->pages_per_split1 : m->pages_per_split;
        aa.n_head = d.n_head; aa.n_kv = d.n_kv; aa.head_dim = hd; aa.page = m->page; aa.n_splits = n_splits;
        aa.pages_per_split = pps;
        // Who merges the context splits.  Single-token step with the output projection in the tensor-core layout: that
        // projection's prologue while few splits are visible (0.6 us per split, overlapped with its other loads).  From
        // kMergeInAttn visible splits on, and for several rows, the attention kernel itself (its last CTA per KV head:
        // ~3 us whatever the count; 8B shape at position 4100, 23 splits: 3.27 ms per step against 3.32) -- but only with
        // four or more KV heads: with one or two, two CTAs would merge everything (measured on the 12 / 2-head shape:
        // 1.74 ms per step against 1.55 with the merge kernel, whose grid is one CTA per query head).
        const bool merge_in_gemv = single && l.o->w.layout == 1;
        aa.merge_ticket = merge_in_attn ? m->attn_ticket : nullptr;
        // below kMergeInAttn visible splits the projection merges; from there on the attention kernel (four or more KV
        // heads) or the merge kernel does, which then returns at once while few splits are visible
        aa.merge_min_splits = merge_in_gemv ? kMergeInAttn : 0;
        aa.skip_merge = 0;
        M_TRY(launch_attn_paged(c, aa, n_tok, s));

        // Tensor parallel: attn_output and ffn_down are row parallel (this rank's K range), so their
        // results are partial sums.  Rank 0 adds the residual stream, the other ranks overwrite their
        // copy of it with the bare partial product, and the all-reduce leaves resid + sum on every rank.
        a = gemv_args(l.o, m->att, n_tok, qd, m->x, H);
        a.epi = resid_epi; a.resid = resid_epi == EPI_RESIDUAL ? m->x : nullptr;
        if (merge_in_gemv) {
            a.x = nullptr; a.attn_partial = m->partial; a.attn_d_pos = dpos; a.attn_pos0 = pos0; a.attn_n_splits = n_splits;
            a.attn_merged = m->att; a.attn_merge_below = kMergeInAttn;
            a.attn_keys_per_split = pps * m->page; a.attn_hd = hd;
        }
        M_TRY(launch_gemv(c, a, s));
        if (tp) M_TRY(tp_all_reduce(c, m->x, static_cast<size_t>(n_tok) * H, s));
        }

        // prompt chunks: silu(gate) * up goes straight into the down projection's fp16 tile image
        const bool act_as_image = m->tc_images && n_tok >= c->tc_min_m;
        a = gemv_args(l.gate, m->x, n_tok, H, m->act, F);
        a.w2 = l.up->w; a.epi = EPI_SWIGLU; a.gamma = l.ffn_norm; a.eps = d.rms_eps;
        if (act_as_image) a.y_img = m->act_img;
        M_TRY(launch_gemv(c, a, s));

        a = gemv_args(l.down, m->act, n_tok, F, m->x, H);
        a.epi = resid_epi; a.resid = resid_epi == EPI_RESIDUAL ? m->x : nullptr;
        if (act_as_image) a.x_img = m->act_img;
        M_TRY(launch_gemv(c, a, s));
        if (tp) M_TRY(tp_all_reduce(c, m->x, static_cast<size_t>(n_tok) * H, s));
    }
    // final norm fused into the logits GEMV; only the last row feeds sampling (main.cpp:3593-3598)
    // tensor parallel: each rank computes its slice of the vocabulary, then the slices are gathered
    const int vocab_l = d.vocab / c->tp_size;
    if (all_rows) {
        // logits and greedy token of EVERY row (compute_logits_rows, src/cli/main.cpp:347-391): the verification of a
        // speculative block, or one step of a batch of sequences.  Tensor parallel: each rank fills its slice of the
        // vocabulary in every row, then the slices are gathered row by row.
        GemvArgs a = gemv_args(m->output ? m->output : m->tok_embd, m->x, n_tok, H, m->logits_rows + static_cast<size_t>(c->tp_rank) * vocab_l, d.vocab);
        a.gamma = m->output_norm; a.eps = d.rms_eps;
        M_TRY(launch_gemv(c, a, s));
        if (c->tp_size > 1)
            for (int r = 0; r < n_tok; ++r) M_TRY(tp_all_gather_in_place(c, m->logits_rows + static_cast<size_t>(r) * d.vocab, static_cast<size_t>(vocab_l), s));
        return launch_argmax_rows(c, m->logits_rows, d.vocab, d.vocab, n_tok, m->d_rows_next, m->amax_partial, s);
    }
    GemvArgs a = gemv_args(m->output ? m->output : m->tok_embd, m->x + static_cast<size_t>(n_tok - 1) * H, 1, H,
                           m->logits + static_cast<size_t>(c->tp_rank) * vocab_l, vocab_l);
    a.gamma = m->output_norm; a.eps = d.rms_eps;
    M_TRY(launch_gemv(c, a, s));
    M_TRY(tp_all_gather_in_place(c, m->logits, static_cast<size_t>(vocab_l), s));
    M_TRY(launch_argmax(c, m->logits, d.vocab, m->d_next, m->amax_partial, s));
    return GGB_OK;
}

// A call that starts at position 0 starts a new sequence: the short-convolution states return to zero
// (lconv_state, src/cli/main.cpp:2159).  The KV cache needs no such step (a position is written before it is read).
int conv_reset(ggb_model m, int pos0) {
    if (!m->has_conv || pos0 != 0) return GGB_OK;
    for (Layer& l : m->layers)
        if (l.conv())
            M_TRY(cuda_status(m->c, cudaMemsetAsync(l.sc_state, 0, sizeof(float) * static_cast<size_t>(std::max(m->conv_taps - 1, 1)) * m->d.hidden, m->c->stream), "conv state reset"));
    return GGB_OK;
}

}  // namespace

#define GGB_LOCK(h) std::lock_guard<std::mutex> _lk((h)->mu); cudaSetDevice((h)->device)

extern "C" {

int ggb_model_create(ggb_handle h, const ggb_model_desc* desc, ggb_model* out) {
    if (!h) return GGB_UNAVAILABLE;
    if (!desc || !out) return set_status(h, GGB_INVALID_PARAM, "model_create: null pointer");
    const ggb_model_desc& d = *desc;
    if (d.n_layer <= 0 || d.hidden <= 0 || d.n_head <= 0 || d.n_kv <= 0 || d.head_dim <= 0 || d.ffn <= 0 || d.vocab <= 0 || d.ctx <= 0 ||
        d.n_head % d.n_kv || (d.head_dim != 64 && d.head_dim != 128 && d.head_dim != 256) || d.hidden % 32 || d.ffn % 32)
        return set_status(h, GGB_INVALID_PARAM, "model_create: unsupported dimensions");
    ggb_model m = new ggb_model_s();
    m->c = h; m->d = d;
    if (m->d.rope_scale == 0.0f) m->d.rope_scale = 1.0f;
    m->page = d.kv_page > 0 ? d.kv_page : 64;
    m->conv_taps = d.conv_taps > 0 ? d.conv_taps : 3;          // lfm2.shortconv.l_cache, default as src/cli/main.cpp:2146-2147
    if (m->conv_taps > 8) { delete m; return set_status(h, GGB_INVALID_PARAM, "model_create: at most 8 convolution taps"); }
    m->layers.resize(d.n_layer);
    *out = m;
    return GGB_OK;
}

void ggb_model_destroy(ggb_model m) {
    if (!m) return;
    {
        GGB_LOCK(m->c);
        cudaStreamSynchronize(m->c->stream);
        if (m->decode_graph) cudaGraphExecDestroy(m->decode_graph);
        for (auto& g : m->batch_graphs) cudaGraphExecDestroy(g.second);
        if (m->sample_graph) cudaGraphExecDestroy(m->sample_graph);
        for (void* p : m->owned) cudaFree(p);
        if (m->h_io) cudaFreeHost(m->h_io);
        if (m->h_logits) cudaFreeHost(m->h_logits);
        free_weight(m->tok_embd); free_weight(m->output);
        for (Layer& l : m->layers) { free_weight(l.q); free_weight(l.k); free_weight(l.v); free_weight(l.o); free_weight(l.gate); free_weight(l.up); free_weight(l.down); free_weight(l.sc_in); free_weight(l.sc_out); }
    }
    delete m;
}

int ggb_model_set_cache(ggb_model m, const char* cache_dir, const char* model_id) {
    if (!m) return GGB_INVALID_PARAM;
    if (m->finalized) return set_status(m->c, GGB_INVALID_PARAM, "set_cache: model already finalized");
    m->cache_dir = cache_dir ? cache_dir : "";
    m->cache_model_id = model_id ? model_id : "";
    return GGB_OK;
}

int ggb_model_cache_stats(ggb_model m, int* hits, int* misses) {
    if (!m) return GGB_INVALID_PARAM;
    if (hits) *hits = m->cache_hits;
    if (misses) *misses = m->cache_misses;
    return GGB_OK;
}

int ggb_model_set_tensor(ggb_model m, int slot, int layer, uint32_t type, int64_t N, int K, const void* host) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (!host) return set_status(c, GGB_INVALID_PARAM, "set_tensor: null data");
    if (m->finalized) return set_status(c, GGB_INVALID_PARAM, "set_tensor: model already finalized");
    GGB_LOCK(c);
    const ggb_model_desc& d = m->d;
    const int qd = d.n_head * d.head_dim, kvd = d.n_kv * d.head_dim;
    auto mat = [&](DeviceWeight** dst, int64_t wantN, int wantK) -> int {
        if (N != wantN || K != wantK) return set_status(c, GGB_INVALID_PARAM, "set_tensor: shape does not match the model description");
        if (*dst) { free_weight(*dst); *dst = nullptr; }
        if (m->cache_dir.empty()) return upload_weight(c, type, N, K, host, dst);
        char name[48];
        snprintf(name, sizeof(name), "slot%d.layer%d.rank%dof%d", slot, layer, c->tp_rank, c->tp_size);
        int hit = 0;
        const int st = upload_weight_cached(c, m->cache_dir.c_str(), m->cache_model_id.c_str(), name, type, N, K, host, dst, &hit);
        if (st == GGB_OK) (hit ? m->cache_hits : m->cache_misses)++;
        return st;
    };
    auto vec = [&](float** dst, int64_t wantN) -> int {
        if (type != GGB_F32 || N != wantN) return set_status(c, GGB_INVALID_PARAM, "set_tensor: vectors must be F32 of the model's size");
        int st = dev_alloc(m, dst, static_cast<size_t>(N));
        if (st != GGB_OK) return st;
        st = cuda_status(c, cudaMemcpyAsync(*dst, host, sizeof(float) * N, cudaMemcpyHostToDevice, c->stream), "vector upload");
        if (st != GGB_OK) return st;
        return cuda_status(c, cudaStreamSynchronize(c->stream), "vector upload");
    };
    if (slot < 10) {
        switch (slot) {
        case GGB_T_TOKEN_EMBD: return mat(&m->tok_embd, d.vocab, d.hidden);
        case GGB_T_OUTPUT: return mat(&m->output, d.vocab / c->tp_size, d.hidden);
        case GGB_T_OUTPUT_NORM: return vec(&m->output_norm, d.hidden);
        case GGB_T_ROPE_FREQS:
            if (type != GGB_F32 || N <= 0) return set_status(c, GGB_INVALID_PARAM, "set_tensor: rope_freqs must be F32");
            m->rope_ff.assign(static_cast<const float*>(host), static_cast<const float*>(host) + N);
            return GGB_OK;
        default: return set_status(c, GGB_NOT_FOUND, "set_tensor: unknown slot");
        }
    }
    if (layer < 0 || layer >= d.n_layer) return set_status(c, GGB_INVALID_PARAM, "set_tensor: layer out of range");
    Layer& l = m->layers[layer];
    switch (slot) {
    case GGB_T_ATTN_NORM: return vec(&l.attn_norm, d.hidden);
    case GGB_T_FFN_NORM: return vec(&l.ffn_norm, d.hidden);
    case GGB_T_ATTN_Q: return mat(&l.q, qd, d.hidden);
    case GGB_T_ATTN_K: return mat(&l.k, kvd, d.hidden);
    case GGB_T_ATTN_V: return mat(&l.v, kvd, d.hidden);
    case GGB_T_ATTN_OUT: return mat(&l.o, d.hidden, qd);
    case GGB_T_FFN_GATE: return mat(&l.gate, d.ffn, d.hidden);
    case GGB_T_FFN_UP: return mat(&l.up, d.ffn, d.hidden);
    case GGB_T_FFN_DOWN: return mat(&l.down, d.hidden, d.ffn);
    case GGB_T_BIAS_Q: return vec(&l.bq, qd);
    case GGB_T_BIAS_K: return vec(&l.bk, kvd);
    case GGB_T_BIAS_V: return vec(&l.bv, kvd);
    case GGB_T_Q_NORM: return vec(&l.q_norm, d.head_dim);
    case GGB_T_K_NORM: return vec(&l.k_norm, d.head_dim);
    case GGB_T_SC_IN_PROJ: return mat(&l.sc_in, 3 * static_cast<int64_t>(d.hidden), d.hidden);
    case GGB_T_SC_OUT_PROJ: return mat(&l.sc_out, d.hidden, d.hidden);
    case GGB_T_SC_CONV: return vec(&l.sc_conv, static_cast<int64_t>(d.hidden) * m->conv_taps);
    default: return set_status(c, GGB_NOT_FOUND, "set_tensor: unknown slot");
    }
}

int ggb_model_finalize(ggb_model m) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (m->finalized) return GGB_OK;
    GGB_LOCK(c);
    const ggb_model_desc& d = m->d;
    if (!m->tok_embd || !m->output_norm) return set_status(c, GGB_INVALID_PARAM, "finalize: token_embd / output_norm missing");
    if (c->tp_size > 1 && (!m->output || d.vocab % c->tp_size))
        return set_status(c, GGB_INVALID_PARAM, "finalize: a tensor-parallel shard needs its slice of the output matrix (vocab divisible by the group size)");
    for (const Layer& l : m->layers) {
        // a layer carries the short convolution or attention, told apart by tensor presence (src/cli/main.cpp:2155-2164)
        const bool mixer_ok = l.conv() ? (l.sc_out && l.sc_conv && !l.q && !l.k && !l.v && !l.o) : (l.q && l.k && l.v && l.o && !l.sc_out && !l.sc_conv);
        if (!mixer_ok || !l.gate || !l.up || !l.down || !l.attn_norm || !l.ffn_norm)
            return set_status(c, GGB_INVALID_PARAM, "finalize: a layer tensor is missing");
        if (l.gate->w.type != l.up->w.type) return set_status(c, GGB_INVALID_PARAM, "finalize: ffn_gate and ffn_up must share a type");
        m->has_conv = m->has_conv || l.conv();
    }
    if (m->has_conv && (c->tp_size > 1 || m->n_seq > 1))
        return set_status(c, GGB_INVALID_PARAM, "finalize: a model with short-convolution layers runs one sequence on one GPU");
    const int hd = d.head_dim, qd = d.n_head * hd, kvd = d.n_kv * hd;
    // RoPE table exactly as RopeCache::build (src/cli/main.cpp:665-692): float pow/cos/sin on the host.
    {
        const int pairs = hd / 2;
        std::vector<float> cs(static_cast<size_t>(d.ctx) * pairs), sn(cs.size());
        for (int64_t p = 0; p < d.ctx; ++p)
            for (int i = 0; i < pairs; ++i) {
                float ff = i < static_cast<int>(m->rope_ff.size()) ? m->rope_ff[i] : 1.0f;
                if (ff == 0.0f) ff = 1.0f;
                const float wavelength = std::pow(d.rope_base, 2.0f * static_cast<float>(i) / static_cast<float>(hd));
                const float angle = m->d.rope_scale * static_cast<float>(p) / (wavelength * ff);
                cs[p * pairs + i] = std::cos(angle);
                sn[p * pairs + i] = std::sin(angle);
            }
        M_TRY(dev_alloc(m, &m->cos_tab, cs.size()));
        M_TRY(dev_alloc(m, &m->sin_tab, sn.size()));
        M_TRY(cuda_status(c, cudaMemcpy(m->cos_tab, cs.data(), sizeof(float) * cs.size(), cudaMemcpyHostToDevice), "rope table"));
        M_TRY(cuda_status(c, cudaMemcpy(m->sin_tab, sn.data(), sizeof(float) * sn.size(), cudaMemcpyHostToDevice), "rope table"));
    }
    // paged KV
    m->n_pages = (d.ctx + m->page - 1) / m->page;
    attn_split_geometry(m->n_pages, d.n_kv, &m->n_splits, &m->pages_per_split);
    m->pages_per_split1 = (m->n_pages + 127) / 128;
    m->n_splits1 = (m->n_pages + m->pages_per_split1 - 1) / m->pages_per_split1;
    m->kv_layer_elems = static_cast<size_t>(m->n_seq) * m->n_pages * d.n_kv * m->page * hd;
    M_TRY(dev_alloc(m, &m->k_cache, m->kv_layer_elems * d.n_layer));
    M_TRY(dev_alloc(m, &m->v_cache, m->kv_layer_elems * d.n_layer));
    M_TRY(cuda_status(c, cudaMemset(m->k_cache, 0, sizeof(__nv_bfloat16) * m->kv_layer_elems * d.n_layer), "kv memset"));
    M_TRY(cuda_status(c, cudaMemset(m->v_cache, 0, sizeof(__nv_bfloat16) * m->kv_layer_elems * d.n_layer), "kv memset"));
    {
        std::vector<int32_t> bt(static_cast<size_t>(m->n_seq) * m->n_pages);
        for (size_t i = 0; i < bt.size(); ++i) bt[i] = static_cast<int32_t>(i);
        M_TRY(dev_alloc(m, &m->block_table, bt.size()));
        M_TRY(cuda_status(c, cudaMemcpy(m->block_table, bt.data(), sizeof(int32_t) * bt.size(), cudaMemcpyHostToDevice), "block table"));
    }
    const bool tensor_attn = c->use_tc && c->tc_min_m <= kSmallChunk && m->page == 64 && (hd == 64 || hd == 128);
    m->chunk = tensor_attn ? std::min(kLargeChunk, std::max(d.ctx, kSmallChunk)) : kSmallChunk;
    const size_t T = m->chunk;
    M_TRY(dev_alloc(m, &m->x, T * d.hidden));
    M_TRY(dev_alloc(m, &m->q, T * qd));
    M_TRY(dev_alloc(m, &m->k, T * kvd));
    M_TRY(dev_alloc(m, &m->v, T * kvd));
    M_TRY(dev_alloc(m, &m->att, T * qd));
    M_TRY(dev_alloc(m, &m->act, T * d.ffn));
    if (m->has_conv) {
        M_TRY(dev_alloc(m, &m->bcx, T * 3 * d.hidden));
        M_TRY(dev_alloc(m, &m->yconv, T * d.hidden));
        for (Layer& l : m->layers)
            if (l.conv()) M_TRY(dev_alloc(m, &l.sc_state, static_cast<size_t>(std::max(m->conv_taps - 1, 1)) * d.hidden));
    }
    m->tc_images = tensor_attn && d.hidden % 64 == 0 && d.ffn % 64 == 0;
    if (m->tc_images) M_TRY(dev_alloc(m, &m->act_img, gemm_tc_image_elems(m->chunk, d.ffn)));
    M_TRY(dev_alloc(m, &m->logits, static_cast<size_t>(d.vocab)));
    M_TRY(dev_alloc(m, &m->partial, std::max(attn_partial_floats(kSmallChunk, d.n_head, m->n_splits, hd), attn_partial_floats(1, d.n_head, m->n_splits1, hd))));
    M_TRY(dev_alloc(m, &m->amax_partial, 512));
    M_TRY(dev_alloc(m, &m->attn_ticket, static_cast<size_t>(kSmallChunk) * d.n_kv));
    M_TRY(cuda_status(c, cudaMemset(m->attn_ticket, 0, sizeof(int) * kSmallChunk * d.n_kv), "memset"));
    M_TRY(dev_alloc(m, &m->logits_rows, static_cast<size_t>(kSpecRows) * d.vocab));
    M_TRY(dev_alloc(m, &m->d_rows_next, kSpecRows));
    M_TRY(dev_alloc(m, &m->d_seq_pos, kSpecRows));
    M_TRY(cuda_status(c, cudaMemset(m->d_seq_pos, 0, 4 * kSpecRows), "memset"));
    if (m->n_seq > 1) M_TRY(dev_alloc(m, &m->d_gen_batch, static_cast<size_t>(d.ctx) * m->n_seq));
    M_TRY(dev_alloc(m, &m->d_tokens, T));
    M_TRY(dev_alloc(m, &m->d_pos, 1));
    M_TRY(dev_alloc(m, &m->d_next, 1));
    M_TRY(dev_alloc(m, &m->d_step, 1));
    M_TRY(dev_alloc(m, &m->d_gen, static_cast<size_t>(d.ctx)));
    M_TRY(cuda_status(c, cudaMemset(m->d_pos, 0, 4), "memset"));
    M_TRY(cuda_status(c, cudaMemset(m->d_step, 0, 4), "memset"));
    M_TRY(cuda_status(c, cudaMemset(m->d_tokens, 0, 4 * T), "memset"));
    M_TRY(cuda_status(c, cudaMallocHost(&m->h_io, 64), "pinned alloc"));
    M_TRY(cuda_status(c, cudaMallocHost(&m->h_logits, sizeof(float) * d.vocab), "pinned alloc"));

    // Persistent decode-step kernel (opt-in, GGB_STEP_KERNEL=1): every layer matrix and the logits matrix Q4_K / Q6_K in the
    // tensor-core layout, no biases or QK norms, head_dim 64 / 128, one GPU.  Measured on the Llama-3.2-1B shape it takes
    // 0.93 ms per step against 0.61 ms for the kernel-per-matrix graph (grid-wide barriers of ~2 us each, and a code
    // footprint of ~140 KB that is fetched anew in every phase), so the graph stays the default.
    {
        bool ok = !m->has_conv && c->use_mma && c->tp_size == 1 && (hd == 64 || hd == 128) && m->page % 8 == 0 && getenv("GGB_STEP_KERNEL") != nullptr &&
                  d.hidden % 256 == 0 && d.ffn % 256 == 0 && qd % 256 == 0;
        const DeviceWeight* outw = m->output ? m->output : m->tok_embd;
        ok = ok && step_mat_ok(outw->w);
        for (const Layer& l : m->layers)
            ok = ok && !l.conv() && step_mat_ok(l.q->w) && step_mat_ok(l.k->w) && step_mat_ok(l.v->w) && step_mat_ok(l.o->w) && step_mat_ok(l.gate->w) &&
                 step_mat_ok(l.up->w) && step_mat_ok(l.down->w) && l.gate->w.type == l.up->w.type && !l.bq && !l.bk && !l.bv && !l.q_norm && !l.k_norm;
        if (ok) {
            const int n_cta = c->sm_count;
            std::vector<StepLayer> hl(d.n_layer);
            for (int L = 0; L < d.n_layer; ++L) {
                const Layer& l = m->layers[L];
                StepLayer& t = hl[L];
                t.q = step_mat(l.q->w, m->q); t.k = step_mat(l.k->w, m->k); t.v = step_mat(l.v->w, m->v); t.o = step_mat(l.o->w, m->x);
                t.gate = step_mat(l.gate->w, m->act); t.up = step_mat(l.up->w, m->act); t.down = step_mat(l.down->w, m->x);
                t.attn_norm = l.attn_norm; t.ffn_norm = l.ffn_norm;
                t.k_cache = m->k_cache + static_cast<size_t>(L) * m->kv_layer_elems;
                t.v_cache = m->v_cache + static_cast<size_t>(L) * m->kv_layer_elems;
            }
            M_TRY(dev_alloc(m, &m->d_step_layers, hl.size()));
            M_TRY(dev_alloc(m, &m->d_step_bar, 1));
            M_TRY(cuda_status(c, cudaMemcpy(m->d_step_layers, hl.data(), sizeof(StepLayer) * hl.size(), cudaMemcpyHostToDevice), "step layers"));
            StepArgs& a = m->step;
            a.layers = m->d_step_layers; a.n_layer = d.n_layer;
            a.out = step_mat(outw->w, m->logits); a.out_norm = m->output_norm;
            step_shape_init(a.shape[kPhaseQkv], d.hidden, qd, kvd, kvd, false, n_cta);
            step_shape_init(a.shape[kPhaseO], qd, d.hidden, 0, 0, false, n_cta);
            step_shape_init(a.shape[kPhaseGateUp], d.hidden, d.ffn, 0, 0, true, n_cta);
            step_shape_init(a.shape[kPhaseDown], d.ffn, d.hidden, 0, 0, false, n_cta);
            step_shape_init(a.shape[kPhaseLogits], d.hidden, outw->w.N, 0, 0, false, n_cta);
            a.x = m->x; a.act = m->act; a.eps = d.rms_eps; a.n_cta = n_cta;
            a.k_max = std::max(std::max(d.hidden, qd), d.ffn);
            a.bar = m->d_step_bar; a.err = c->d_err;
            AttnPagedArgs& aa = a.attn;
            aa = AttnPagedArgs{};
            aa.q = m->q; aa.block_table = m->block_table; aa.partial = m->partial; aa.out = m->att;
            aa.n_head = d.n_head; aa.n_kv = d.n_kv; aa.head_dim = hd; aa.page = m->page; aa.n_splits = m->n_splits;
            aa.pages_per_split = m->pages_per_split;
            aa.fuse = 1; aa.neox = d.rope_neox; aa.skip_merge = 1; aa.k_new = m->k; aa.v_new = m->v;
            aa.cos_tab = m->cos_tab; aa.sin_tab = m->sin_tab; aa.eps = d.rms_eps;
            m->use_step = true;
        }
    }
    // One eager step first: it sets every kernel's shared-memory attribute outside capture
    // (and faults early, if anything is wrong, where the error is attributable).
    {
        int st = enqueue_forward(m, 1, true, 0);
        if (st == GGB_OK) st = cuda_status(c, cudaStreamSynchronize(c->stream), "warm-up step");
        if (st != GGB_OK && m->use_step) {      // shapes outside the step kernel's shared memory, or no cooperative launch
            m->use_step = false;
            cudaStreamSynchronize(c->stream);
            M_TRY(enqueue_forward(m, 1, true, 0));
            M_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "warm-up step"));
        } else if (st != GGB_OK) return st;
        M_TRY(check_device_error(c));
    }
    // Capture the decode step: forward + token/position feedback.  Should the capture refuse the cooperative launch of
    // the persistent kernel, the kernel-per-matrix graph is captured instead.
    auto capture = [&]() -> int {
        const uint64_t before = c->launches;
        M_TRY(cuda_status(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal), "begin capture"));
        int st = enqueue_forward(m, 1, true, 0);
        if (st == GGB_OK) {
            feedback_kernel<<<1, 1, 0, c->stream>>>(m->d_next, m->d_tokens, m->d_pos, m->d_gen, m->d_step, d.ctx);
            c->launches++;
            st = cuda_status(c, cudaGetLastError(), "feedback kernel");
        }
        cudaGraph_t graph = nullptr;
        cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
        m->launches_per_step = c->launches - before;
        c->launches = before;    // captured launches are counted when the graph is replayed
        if (st != GGB_OK) { if (graph) cudaGraphDestroy(graph); return st; }
        M_TRY(cuda_status(c, e, "end capture"));
        e = cudaGraphInstantiate(&m->decode_graph, graph, 0);
        cudaGraphDestroy(graph);
        return cuda_status(c, e, "graph instantiate");
    };
    {
        int st = capture();
        if (st != GGB_OK && m->use_step) {
            m->use_step = false;
            cudaGetLastError();
            st = capture();
        }
        if (st != GGB_OK) return st;
    }
    M_TRY(cuda_status(c, cudaMemset(m->k_cache, 0, sizeof(__nv_bfloat16) * m->kv_layer_elems * d.n_layer), "kv memset"));
    M_TRY(cuda_status(c, cudaMemset(m->v_cache, 0, sizeof(__nv_bfloat16) * m->kv_layer_elems * d.n_layer), "kv memset"));
    M_TRY(conv_reset(m, 0));              // the warm-up step advanced the convolution states
    M_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "finalize"));
    m->finalized = true;
    return GGB_OK;
}

int ggb_model_prefill(ggb_model m, const int32_t* host_tokens, int n_tok, int pos0, float* host_logits, int32_t* next_token) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (!m->finalized) return set_status(c, GGB_INVALID_PARAM, "prefill: model not finalized");
    if (!host_tokens || n_tok <= 0 || pos0 < 0 || pos0 + n_tok > m->d.ctx) return set_status(c, GGB_INVALID_PARAM, "prefill: bad arguments");
    GGB_LOCK(c);
    M_TRY(conv_reset(m, pos0));
    for (int t0 = 0; t0 < n_tok; t0 += m->chunk) {
        const int n = std::min(m->chunk, n_tok - t0);
        M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_tokens, host_tokens + t0, sizeof(int32_t) * n, cudaMemcpyHostToDevice, c->stream), "token upload"));
        M_TRY(enqueue_forward(m, n, false, pos0 + t0));
    }
    if (host_logits) M_TRY(cuda_status(c, cudaMemcpyAsync(host_logits, m->logits, sizeof(float) * m->d.vocab, cudaMemcpyDeviceToHost, c->stream), "logits download"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->h_io + 2, m->d_next, 4, cudaMemcpyDeviceToHost, c->stream), "token download"));
    M_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "prefill"));
    if (next_token) *next_token = m->h_io[2];
    return check_device_error(c);
}

int ggb_model_decode(ggb_model m, int32_t token, int pos, float* host_logits, int32_t* next_token) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (!m->finalized) return set_status(c, GGB_INVALID_PARAM, "decode: model not finalized");
    if (pos < 0 || pos >= m->d.ctx || token < 0 || token >= m->d.vocab) return set_status(c, GGB_INVALID_PARAM, "decode: token or position out of range");
    GGB_LOCK(c);
    M_TRY(conv_reset(m, pos));
    m->h_io[0] = token; m->h_io[1] = pos;
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_tokens, m->h_io, 4, cudaMemcpyHostToDevice, c->stream), "token upload"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_pos, m->h_io + 1, 4, cudaMemcpyHostToDevice, c->stream), "pos upload"));
    if (m->cur_seq == 0) {
        M_TRY(cuda_status(c, cudaGraphLaunch(m->decode_graph, c->stream), "graph launch"));
        c->launches += m->launches_per_step;
    } else {
        M_TRY(enqueue_forward(m, 1, true, 0));       // the captured step is bound to sequence 0's block table
    }
    // a caller's buffer in page-locked memory takes the logits directly; any other goes through the model's own pinned
    // buffer and one host copy (0.5 MB at a 128 K vocabulary: some 20 us of a 0.7 ms step)
    bool direct = false;
    if (host_logits) {
        cudaPointerAttributes pa{};
        direct = cudaPointerGetAttributes(&pa, host_logits) == cudaSuccess && pa.type == cudaMemoryTypeHost;
        cudaGetLastError();
        M_TRY(cuda_status(c, cudaMemcpyAsync(direct ? host_logits : m->h_logits, m->logits, sizeof(float) * m->d.vocab, cudaMemcpyDeviceToHost, c->stream), "logits download"));
    }
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->h_io + 2, m->d_next, 4, cudaMemcpyDeviceToHost, c->stream), "token download"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->h_io + 4, c->d_err, 4, cudaMemcpyDeviceToHost, c->stream), "error word download"));
    M_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "decode"));
    if (m->h_io[4] != 0) return check_device_error(c);
    if (host_logits && !direct) memcpy(host_logits, m->h_logits, sizeof(float) * m->d.vocab);
    if (next_token) *next_token = m->h_io[2];
    return GGB_OK;
}

int ggb_model_generate(ggb_model m, int32_t first_token, int pos0, int n, int32_t* host_out) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (!m->finalized) return set_status(c, GGB_INVALID_PARAM, "generate: model not finalized");
    if (n <= 0 || pos0 < 0 || pos0 + n > m->d.ctx || first_token < 0 || first_token >= m->d.vocab || !host_out)
        return set_status(c, GGB_INVALID_PARAM, "generate: bad arguments");
    if (m->cur_seq != 0) return set_status(c, GGB_INVALID_PARAM, "generate: the device-resident loop runs on sequence 0 (use ggb_model_generate_batch for several)");
    GGB_LOCK(c);
    M_TRY(conv_reset(m, pos0));
    m->h_io[0] = first_token; m->h_io[1] = pos0; m->h_io[3] = 0;
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_tokens, m->h_io, 4, cudaMemcpyHostToDevice, c->stream), "token upload"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_pos, m->h_io + 1, 4, cudaMemcpyHostToDevice, c->stream), "pos upload"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_step, m->h_io + 3, 4, cudaMemcpyHostToDevice, c->stream), "step upload"));
    for (int i = 0; i < n; ++i) M_TRY(cuda_status(c, cudaGraphLaunch(m->decode_graph, c->stream), "graph launch"));
    c->launches += m->launches_per_step * n;
    M_TRY(cuda_status(c, cudaMemcpyAsync(host_out, m->d_gen, sizeof(int32_t) * n, cudaMemcpyDeviceToHost, c->stream), "tokens download"));
    M_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "generate"));
    return check_device_error(c);
}

// Prompt-lookup drafter, src/cli/main.cpp:397-415: the most recent earlier occurrence of the last `ng` tokens (longest
// n-gram first) and up to k tokens that followed it.
static std::vector<int32_t> lookup_draft(const std::vector<int32_t>& seq, int ngram_max, int ngram_min, int k) {
    const int n = static_cast<int>(seq.size());
    for (int ng = ngram_max; ng >= ngram_min; --ng) {
        if (n < ng + 1) continue;
        for (int i = n - ng - 1; i >= 0; --i) {
            bool match = true;
            for (int j = 0; j < ng && match; ++j) match = seq[i + j] == seq[n - ng + j];
            if (!match) continue;
            std::vector<int32_t> draft;
            for (int j = 0; j < k && i + ng + j < n; ++j) draft.push_back(seq[i + ng + j]);
            if (!draft.empty()) return draft;
        }
    }
    return {};
}

int ggb_model_generate_spec(ggb_model m, const int32_t* history, int n_history, int pos0, int n, int draft_k, int32_t* host_out, int32_t* stats) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (!m->finalized) return set_status(c, GGB_INVALID_PARAM, "generate_spec: model not finalized");
    if (c->tp_size > 1) return set_status(c, GGB_INVALID_PARAM, "generate_spec: one GPU only");
    // a rejected draft cannot be taken back out of a recurrent state; the reference keeps lfm2 off this path too (src/cli/main.cpp:2299-2301)
    if (m->has_conv) return set_status(c, GGB_INVALID_PARAM, "generate_spec: not for models with short-convolution layers");
    if (m->cur_seq != 0) return set_status(c, GGB_INVALID_PARAM, "generate_spec: runs on sequence 0");
    if (!history || n_history < 1 || n <= 0 || pos0 < 0 || pos0 + n > m->d.ctx || !host_out)
        return set_status(c, GGB_INVALID_PARAM, "generate_spec: bad arguments");
    for (int i = 0; i < n_history; ++i)
        if (history[i] < 0 || history[i] >= m->d.vocab) return set_status(c, GGB_INVALID_PARAM, "generate_spec: token out of range");
    GGB_LOCK(c);
    const int k = std::max(1, std::min(kSpecRows - 1, draft_k));          // k + 1 rows per block (src/cli/main.cpp:2305-2308)
    std::vector<int32_t> seq(history, history + n_history);
    int32_t last = seq.back();
    int pos = pos0, generated = 0;
    long steps = 0, proposed = 0, accepted = 0;
    std::vector<int32_t> block, rows(kSpecRows);
    while (generated < n) {
        // the block [last, draft_1 .. draft_k]: ngrams of 3 down to 1, as the reference (src/cli/main.cpp:2303-2304, 2343-2349)
        std::vector<int32_t> draft = lookup_draft(seq, 3, 1, k);
        const int room = m->d.ctx - pos - 1;                              // positions left after the fed token
        if (static_cast<int>(draft.size()) > room) draft.resize(std::max(room, 0));
        block.assign(1, last);
        block.insert(block.end(), draft.begin(), draft.end());
        const int n_tok = static_cast<int>(block.size()), n_draft = n_tok - 1;
        M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_tokens, block.data(), sizeof(int32_t) * n_tok, cudaMemcpyHostToDevice, c->stream), "token upload"));
        M_TRY(enqueue_forward(m, n_tok, false, pos, true));
        M_TRY(cuda_status(c, cudaMemcpyAsync(rows.data(), m->d_rows_next, sizeof(int32_t) * n_tok, cudaMemcpyDeviceToHost, c->stream), "tokens download"));
        M_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "generate_spec"));
        // greedy verification (src/cli/main.cpp:3531-3588): accept the longest draft prefix whose token equals the row's
        // arg-max; commit the accepted tokens plus one (the correction, or the bonus token after a full match)
        int matched = 0;
        std::vector<int32_t> committed;
        for (;;) {
            const int32_t t = rows[matched];
            committed.push_back(t);
            if (matched < n_draft && t == block[matched + 1]) ++matched; else break;
        }
        pos += 1 + matched;            // rows of rejected drafts are overwritten by the next block
        ++steps; proposed += n_draft; accepted += matched;
        for (int32_t t : committed) {
            host_out[generated++] = t;
            seq.push_back(t);
            last = t;
            if (generated >= n || pos >= m->d.ctx) break;
        }
        if (pos >= m->d.ctx) break;
    }
    if (stats) { stats[0] = static_cast<int32_t>(steps); stats[1] = static_cast<int32_t>(proposed); stats[2] = static_cast<int32_t>(accepted); stats[3] = generated; }
    return check_device_error(c);
}

int ggb_model_generate_sampled(ggb_model m, int32_t first_token, int pos0, int n, float temp, uint64_t* seed, int32_t* host_out) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (!m->finalized) return set_status(c, GGB_INVALID_PARAM, "generate_sampled: model not finalized");
    if (n <= 0 || pos0 < 0 || pos0 + n > m->d.ctx || first_token < 0 || first_token >= m->d.vocab || !host_out || !seed)
        return set_status(c, GGB_INVALID_PARAM, "generate_sampled: bad arguments");
    if (m->cur_seq != 0) return set_status(c, GGB_INVALID_PARAM, "generate_sampled: runs on sequence 0");
    if (temp <= 0.0f) return ggb_model_generate(m, first_token, pos0, n, host_out);      // greedy (src/cli/main.cpp:828-837)
    GGB_LOCK(c);
    M_TRY(conv_reset(m, pos0));
    if (!m->samp_scratch) {
        uint8_t* sc = nullptr;
        M_TRY(dev_alloc(m, &sc, sample_scratch_bytes(m->d.vocab)));
        M_TRY(dev_alloc(m, &m->d_temp, 1));
        M_TRY(dev_alloc(m, &m->d_u, static_cast<size_t>(m->d.ctx)));
        M_TRY(dev_alloc(m, &m->d_sampled, 1));
        m->samp_scratch = sc;
    }
    auto step = [&]() -> int {
        M_TRY(enqueue_forward(m, 1, true, 0));           // ends with the index of the first maximum in d_next
        M_TRY(sample_enqueue(c, m->logits, m->d.vocab, m->d_next, m->d_temp, m->d_u, m->d_step, m->samp_scratch, m->d_sampled, c->stream));
        feedback_kernel<<<1, 1, 0, c->stream>>>(m->d_sampled, m->d_tokens, m->d_pos, m->d_gen, m->d_step, m->d.ctx);
        c->launches++;
        return cuda_status(c, cudaGetLastError(), "feedback kernel");
    };
    // every step's uniform draw: the generator is re-seeded from its own first output at each call
    // (src/cli/main.cpp:841,862), so the draws depend on the seed alone
    std::vector<double> u(n);
    for (int i = 0; i < n; ++i) u[i] = sample_next_uniform(seed);
    m->h_io[0] = first_token; m->h_io[1] = pos0; m->h_io[3] = 0;
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_tokens, m->h_io, 4, cudaMemcpyHostToDevice, c->stream), "token upload"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_pos, m->h_io + 1, 4, cudaMemcpyHostToDevice, c->stream), "pos upload"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_step, m->h_io + 3, 4, cudaMemcpyHostToDevice, c->stream), "step upload"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_temp, &temp, 4, cudaMemcpyHostToDevice, c->stream), "temperature upload"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_u, u.data(), sizeof(double) * n, cudaMemcpyHostToDevice, c->stream), "draws upload"));
    int done = 0;
    if (!m->sample_graph) {
        // the first step runs eagerly (kernel attributes are set outside capture), then the step is captured
        M_TRY(step());
        M_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "generate_sampled"));
        done = 1;
        const uint64_t before = c->launches;
        M_TRY(cuda_status(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal), "begin capture"));
        const int st = step();
        cudaGraph_t graph = nullptr;
        cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
        m->sample_launches = c->launches - before;
        c->launches = before;
        if (st != GGB_OK) { if (graph) cudaGraphDestroy(graph); return st; }
        M_TRY(cuda_status(c, e, "end capture"));
        e = cudaGraphInstantiate(&m->sample_graph, graph, 0);
        cudaGraphDestroy(graph);
        M_TRY(cuda_status(c, e, "graph instantiate"));
    }
    for (int i = done; i < n; ++i) M_TRY(cuda_status(c, cudaGraphLaunch(m->sample_graph, c->stream), "graph launch"));
    c->launches += m->sample_launches * (n - done);
    M_TRY(cuda_status(c, cudaMemcpyAsync(host_out, m->d_gen, sizeof(int32_t) * n, cudaMemcpyDeviceToHost, c->stream), "tokens download"));
    M_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "generate_sampled"));
    return check_device_error(c);
}

int ggb_model_set_sequences(ggb_model m, int n_seq) {
    if (!m) return GGB_INVALID_PARAM;
    if (m->finalized) return set_status(m->c, GGB_INVALID_PARAM, "set_sequences: model already finalized");
    if (n_seq < 1 || n_seq > kSpecRows) return set_status(m->c, GGB_INVALID_PARAM, "set_sequences: 1 to 16 sequences");
    m->n_seq = n_seq;
    return GGB_OK;
}

int ggb_model_select_sequence(ggb_model m, int seq) {
    if (!m) return GGB_INVALID_PARAM;
    if (seq < 0 || seq >= m->n_seq) return set_status(m->c, GGB_INVALID_PARAM, "select_sequence: no such sequence");
    m->cur_seq = seq;
    return GGB_OK;
}

namespace {

int check_batch(ggb_model m, const int32_t* tokens, const int32_t* pos, int n_seq, int n_steps, const char* who) {
    Context* c = m->c;
    auto fail = [&](const char* what) { return set_status(c, GGB_INVALID_PARAM, (std::string(who) + ": " + what).c_str()); };
    if (!m->finalized) return fail("model not finalized");
    if (m->has_conv) return fail("not for models with short-convolution layers (one sequence, its state inside the model)");
    if (!tokens || !pos || n_seq < 1 || n_seq > m->n_seq) return fail("bad arguments (more sequences than ggb_model_set_sequences reserved?)");
    for (int r = 0; r < n_seq; ++r)
        if (tokens[r] < 0 || tokens[r] >= m->d.vocab || pos[r] < 0 || pos[r] + n_steps > m->d.ctx) return fail("token or position out of range");
    return GGB_OK;
}

// The captured step of a batch of n_seq sequences: forward + feedback.  The first call for a batch size runs one eager
// step on scratch inputs first (kernel attributes are set outside capture), so the caller uploads its inputs afterwards.
int batch_graph(ggb_model m, int n_seq, cudaGraphExec_t* out) {
    Context* c = m->c;
    auto it = m->batch_graphs.find(n_seq);
    if (it != m->batch_graphs.end()) { *out = it->second; return GGB_OK; }
    // The warm-up step runs at the LAST position of each stream: the only cache slot it writes is one that a real
    // step rewrites before reading (a step at position p stores slot p first), so prefilled streams stay intact.
    std::vector<int32_t> pos(n_seq, m->d.ctx - 1), tok(n_seq, 0);
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_tokens, tok.data(), 4 * n_seq, cudaMemcpyHostToDevice, c->stream), "token upload"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_seq_pos, pos.data(), 4 * n_seq, cudaMemcpyHostToDevice, c->stream), "pos upload"));
    M_TRY(enqueue_forward(m, n_seq, false, 0, true, true));
    M_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "batch warm-up step"));
    M_TRY(check_device_error(c));
    const uint64_t before = c->launches;
    M_TRY(cuda_status(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal), "begin capture"));
    int st = enqueue_forward(m, n_seq, false, 0, true, true);
    if (st == GGB_OK) {
        feedback_batch_kernel<<<1, 32, 0, c->stream>>>(m->d_rows_next, m->d_tokens, m->d_seq_pos, m->d_gen_batch, m->d_step, n_seq, m->d.ctx);
        c->launches++;
        st = cuda_status(c, cudaGetLastError(), "feedback kernel");
    }
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
    m->batch_launches[n_seq] = c->launches - before;
    c->launches = before;
    if (st != GGB_OK) { if (graph) cudaGraphDestroy(graph); return st; }
    M_TRY(cuda_status(c, e, "end capture"));
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    M_TRY(cuda_status(c, e, "graph instantiate"));
    m->batch_graphs[n_seq] = exec;
    *out = exec;
    return GGB_OK;
}

}  // namespace

int ggb_model_decode_batch(ggb_model m, const int32_t* tokens, const int32_t* pos, int n_seq, float* host_logits, int32_t* next_tokens) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    M_TRY(check_batch(m, tokens, pos, n_seq, 1, "decode_batch"));
    GGB_LOCK(c);
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_tokens, tokens, 4 * n_seq, cudaMemcpyHostToDevice, c->stream), "token upload"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_seq_pos, pos, 4 * n_seq, cudaMemcpyHostToDevice, c->stream), "pos upload"));
    M_TRY(enqueue_forward(m, n_seq, false, 0, true, true));
    std::vector<int32_t> next(n_seq);
    if (host_logits)
        M_TRY(cuda_status(c, cudaMemcpyAsync(host_logits, m->logits_rows, sizeof(float) * static_cast<size_t>(n_seq) * m->d.vocab, cudaMemcpyDeviceToHost, c->stream), "logits download"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(next.data(), m->d_rows_next, 4 * n_seq, cudaMemcpyDeviceToHost, c->stream), "token download"));
    M_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "decode_batch"));
    if (next_tokens) memcpy(next_tokens, next.data(), 4 * n_seq);
    return check_device_error(c);
}

int ggb_model_generate_batch(ggb_model m, const int32_t* first_tokens, const int32_t* pos0, int n_seq, int n, int32_t* host_out) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (n <= 0 || !host_out) return set_status(c, GGB_INVALID_PARAM, "generate_batch: bad arguments");
    M_TRY(check_batch(m, first_tokens, pos0, n_seq, n, "generate_batch"));
    if (m->n_seq < 2) return set_status(c, GGB_INVALID_PARAM, "generate_batch: reserve the sequences with ggb_model_set_sequences before finalize");
    GGB_LOCK(c);
    cudaGraphExec_t g = nullptr;
    M_TRY(batch_graph(m, n_seq, &g));
    const int32_t zero = 0;
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_tokens, first_tokens, 4 * n_seq, cudaMemcpyHostToDevice, c->stream), "token upload"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_seq_pos, pos0, 4 * n_seq, cudaMemcpyHostToDevice, c->stream), "pos upload"));
    M_TRY(cuda_status(c, cudaMemcpyAsync(m->d_step, &zero, 4, cudaMemcpyHostToDevice, c->stream), "step upload"));
    for (int i = 0; i < n; ++i) M_TRY(cuda_status(c, cudaGraphLaunch(g, c->stream), "graph launch"));
    c->launches += m->batch_launches[n_seq] * n;
    M_TRY(cuda_status(c, cudaMemcpyAsync(host_out, m->d_gen_batch, sizeof(int32_t) * static_cast<size_t>(n) * n_seq, cudaMemcpyDeviceToHost, c->stream), "tokens download"));
    M_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "generate_batch"));
    return check_device_error(c);
}

int ggb_model_read_kv(ggb_model m, int layer, int pos, int want_v, float* host_out) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (!m->finalized || !host_out || layer < 0 || layer >= m->d.n_layer || pos < 0 || pos >= m->d.ctx) return set_status(c, GGB_INVALID_PARAM, "read_kv: bad arguments");
    GGB_LOCK(c);
    const int hd = m->d.head_dim;
    std::vector<__nv_bfloat16> tmp(hd);
    const __nv_bfloat16* base = (want_v ? m->v_cache : m->k_cache) + static_cast<size_t>(layer) * m->kv_layer_elems;
    const int page = m->cur_seq * m->n_pages + pos / m->page, slot = pos % m->page;   // identity block table
    for (int h = 0; h < m->d.n_kv; ++h) {
        const size_t o = ((static_cast<size_t>(page) * m->d.n_kv + h) * m->page + slot) * hd;
        M_TRY(cuda_status(c, cudaMemcpy(tmp.data(), base + o, sizeof(__nv_bfloat16) * hd, cudaMemcpyDeviceToHost), "kv download"));
        for (int i = 0; i < hd; ++i) host_out[h * hd + i] = __bfloat162float(tmp[i]);
    }
    return GGB_OK;
}

uint64_t ggb_model_decode_bytes(ggb_model m, int pos) {
    if (!m || !m->finalized) return 0;
    const ggb_model_desc& d = m->d;
    auto wb = [](const DeviceWeight* w) -> uint64_t {
        if (!w) return 0;
        const FormatInfo f = format_info(w->w.type);
        return static_cast<uint64_t>(w->w.N) * w->w.nb * f.block_bytes;
    };
    uint64_t b = wb(m->output ? m->output : m->tok_embd);
    int n_attn = 0;
    for (const Layer& l : m->layers) {
        b += wb(l.q) + wb(l.k) + wb(l.v) + wb(l.o) + wb(l.gate) + wb(l.up) + wb(l.down) + wb(l.sc_in) + wb(l.sc_out);
        if (l.conv()) b += static_cast<uint64_t>(d.hidden) * 4 * (m->conv_taps + 2 * (m->conv_taps - 1));   // taps, state read and written
        else ++n_attn;
    }
    b += static_cast<uint64_t>(d.hidden) * 4 * (2 * d.n_layer + 1);                        // norm gammas
    b += static_cast<uint64_t>(2) * n_attn * (pos + 1) * d.n_kv * d.head_dim * 2;          // K and V read, bf16
    const FormatInfo fe = format_info(m->tok_embd->w.type);
    b += static_cast<uint64_t>(m->tok_embd->w.nb) * fe.block_bytes;                        // one embedding row
    return b;
}

}  // extern "C"
