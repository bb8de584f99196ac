// C ABI, part 2: the qwen35 / qwen35moe decoder graph of the reference CLI (src/cli/main.cpp:2859-3232) kept
// entirely in HBM.  Per layer: attn_norm -> Gated DeltaNet mixer (layers that carry ssm_conv1d, :2900-3034) or
// gated full attention (:3035-3105) -> residual -> post_attention_norm -> mixture-of-experts FFN (:3110-3193)
// -> residual; then output_norm, logits (:3504-3512, :3593-3598) and the greedy token (:827-838).
//
// The architecture is a recurrence (conv state, delta-rule state), so the reference feeds it one token per
// forward, prompt included (:2327).  This file does the same: one CUDA graph = one token; a prompt is the graph
// replayed over a device-resident list of forced tokens, with no host round trip between tokens.
//
// Launches per token and layer.  DeltaNet layer (12): stacked qkv | z-gate GEMV (attn_norm fused) - alpha | beta
// F32 rows - conv + SiLU - delta-rule step - ssm_out GEMV (+ residual) - MoE (7: router logits, top-k, routed
// gate/up, routed down, shared gate/up, shared down; the FFN norm is fused into the router and expert kernels).
// Attention layer (14): stacked q|gate, k, v GEMV - query split - QK-norm + partial NeoX RoPE + KV append -
// attention splits - merge - sigmoid gate - attn_output GEMV (+ residual) - MoE.
#include <cuda_bf16.h>
#include <math.h>
#include <string.h>

#include <cmath>

#include "ggb_attn.h"
#include "ggb_internal.h"

using namespace ggb;

namespace {

struct Q35Layer {
    bool is_ssm = false;
    float *attn_norm = nullptr, *post_norm = nullptr;
    // DeltaNet
    DeviceWeight *qkv = nullptr, *zgate = nullptr, *ssm_out = nullptr;
    float *alpha_beta = nullptr;                 // F32 [2 * n_vhead][hidden]: alpha rows, then beta rows
    bool have_alpha = false, have_beta = false;
    float *conv_w = nullptr, *ssm_a = nullptr, *dt_bias = nullptr, *ssm_norm = nullptr;
    float *conv_state = nullptr, *rec_state = nullptr;
    // full attention
    DeviceWeight *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr;
    float *q_norm = nullptr, *k_norm = nullptr;
    int kv_slot = -1;                            // index among the attention layers (KV cache slab)
    // MoE
    float* router = nullptr;
    DeviceWeight *gate_exps = nullptr, *up_exps = nullptr, *down_exps = nullptr, *sh_gate = nullptr, *sh_up = nullptr, *sh_down = nullptr;
    // finalize appends the shared expert to the expert tensors as one more expert (stacked) when the types agree: it then
    // rides in the routed experts' launches; bytes of the routed experts and of the shared expert for the traffic figure
    bool stacked = false, has_shared = false;
    uint64_t bytes_experts = 0, bytes_shared = 0;
    float* sh_gate_inp = nullptr;
};

}  // namespace

struct ggb_q35_model_s {
    Context* c = nullptr;
    ggb_q35_desc d{};
    DeviceWeight *tok_embd = nullptr, *output = nullptr;
    float* output_norm = nullptr;
    std::vector<Q35Layer> layers;
    std::vector<void*> owned;
    bool finalized = false;
    int n_local_expert = 0, ep_first = 0;        // expert parallel: this rank's experts
    // paged KV of the attention layers
    __nv_bfloat16 *k_cache = nullptr, *v_cache = nullptr;
    int32_t* block_table = nullptr;
    int page = 64, n_pages = 0, n_splits = 1, pages_per_split = 1, n_attn_layers = 0;
    size_t kv_layer_elems = 0;
    float *cos_tab = nullptr, *sin_tab = nullptr;
    // activations
    float *xa = nullptr, *xb = nullptr;          // residual stream, ping-pong (the MoE reads one and writes the other)
    float *mixed = nullptr, *zgate = nullptr, *ab = nullptr, *conv = nullptr, *o_all = nullptr;
    float *qg = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *partial = nullptr;
    float *moe_scr = nullptr, *logits = nullptr, *amax_partial = nullptr;
    int* attn_ticket = nullptr;
    int32_t *d_tokens = nullptr, *d_pos = nullptr, *d_next = nullptr, *d_gen = nullptr, *d_step = nullptr, *d_forced = nullptr, *d_n_forced = nullptr;
    int32_t* h_io = nullptr;
    float* h_logits = nullptr;
    cudaGraphExec_t graph = nullptr;
    uint64_t launches_per_step = 0;
};

namespace {

template <class T>
int q_alloc(ggb_q35_model m, T** p, size_t count, bool zero = false) {
    void* v = nullptr;
    int st = cuda_status(m->c, cudaMalloc(&v, sizeof(T) * std::max<size_t>(count, 1)), "cudaMalloc(q35 model)");
    if (st != GGB_OK) return st;
    m->owned.push_back(v);
    *p = static_cast<T*>(v);
    if (zero) return cuda_status(m->c, cudaMemset(v, 0, sizeof(T) * std::max<size_t>(count, 1)), "memset(q35 model)");
    return GGB_OK;
}

// After a step: record the greedy token, choose the next input (the next forced prompt token while there is one,
// else the token just produced), advance position and step.
__global__ void q35_feedback_kernel(const int32_t* next, int32_t* tokens, int32_t* pos, int32_t* gen, int32_t* step, const int32_t* forced,
                                    const int32_t* n_forced, int gen_cap) {
    const int s = step[0];
    if (s < gen_cap) gen[s] = next[0];
    tokens[0] = (s + 1 < n_forced[0]) ? forced[s + 1] : next[0];
    pos[0] += 1;
    step[0] = s + 1;
}

#define Q_TRY(expr) do { int _st = (expr); if (_st != GGB_OK) return _st; } while (0)

GemvArgs q_gemv(const DeviceWeight* w, const float* x, int lda, float* y, int ldc) {
    GemvArgs a{};
    a.w = w->w; a.x = x; a.M = 1; a.lda = lda; a.y = y; a.ldc = ldc; a.epi = EPI_STORE;
    return a;
}

// One token (id in d_tokens[0], position in d_pos[0]) through all layers; logits and greedy token at the end.
int q35_enqueue_step(ggb_q35_model m) {
    Context* c = m->c;
    cudaStream_t s = c->stream;
    const ggb_q35_desc& d = m->d;
    const int H = d.hidden, Hd = d.head_dim, qdim = d.n_head * Hd, kvdim = d.n_kv * Hd;
    const int key_dim = d.n_khead * d.sk, value_dim = d.n_vhead * d.sk, conv_dim = 2 * key_dim + value_dim;
    float *x = m->xa, *x2 = m->xb;
    Q_TRY(launch_gather_rows(c, m->tok_embd->w, m->d_tokens, 1, x, H, s));
    for (int L = 0; L < d.n_layer; ++L) {
        const Q35Layer& l = m->layers[L];
        if (l.is_ssm) {
            GemvArgs a = q_gemv(l.qkv, x, H, m->mixed, conv_dim);
            a.gamma = l.attn_norm; a.eps = d.rms_eps;
            a.n_cat = 1; a.cat_w[0] = l.zgate->w; a.cat_y[0] = m->zgate; a.cat_ldc[0] = value_dim;
            Q_TRY(launch_gemv(c, a, s));
            Q_TRY(launch_f32_rows(c, x, l.attn_norm, d.rms_eps, l.alpha_beta, 2 * d.n_vhead, H, m->ab, s));
            ggb_deltanet_params dp{};
            dp.mixed = m->mixed; dp.zgate = m->zgate; dp.araw = m->ab; dp.braw = m->ab + d.n_vhead; dp.conv_w = l.conv_w; dp.ssm_a = l.ssm_a;
            dp.dt_bias = l.dt_bias; dp.ssm_norm = l.ssm_norm; dp.conv_state = l.conv_state; dp.rec_state = l.rec_state; dp.out = m->o_all;
            dp.n_khead = d.n_khead; dp.n_vhead = d.n_vhead; dp.sk = d.sk; dp.conv_k = d.conv_k; dp.rms_eps = d.rms_eps;
            Q_TRY(deltanet_step_enqueue(c, &dp, m->conv, s));
            a = q_gemv(l.ssm_out, m->o_all, value_dim, x, H);
            a.epi = EPI_RESIDUAL; a.resid = x;
            Q_TRY(launch_gemv(c, a, s));
        } else {
            GemvArgs a = q_gemv(l.q, x, H, m->qg, 2 * qdim);
            a.gamma = l.attn_norm; a.eps = d.rms_eps;
            a.n_cat = 2;
            a.cat_w[0] = l.k->w; a.cat_y[0] = m->k; a.cat_ldc[0] = kvdim;
            a.cat_w[1] = l.v->w; a.cat_y[1] = m->v; a.cat_ldc[1] = kvdim;
            Q_TRY(launch_gemv(c, a, s));
            Q_TRY(launch_qgate_split(c, m->qg, m->q, d.n_head, Hd, s));
            KvAppendArgs ka{};
            ka.q = m->q; ka.k = m->k; ka.v = m->v;
            ka.k_cache = m->k_cache + static_cast<size_t>(l.kv_slot) * m->kv_layer_elems;
            ka.v_cache = m->v_cache + static_cast<size_t>(l.kv_slot) * m->kv_layer_elems;
            ka.block_table = m->block_table; ka.cos_tab = m->cos_tab; ka.sin_tab = m->sin_tab;
            ka.q_norm = l.q_norm; ka.k_norm = l.k_norm; ka.d_pos = m->d_pos; ka.pos0 = 0;
            ka.n_head = d.n_head; ka.n_kv = d.n_kv; ka.head_dim = Hd; ka.page = m->page; ka.neox = 1; ka.eps = d.rms_eps;
            ka.rot_dims = d.rope_dim; ka.norm_f32 = 1;
            Q_TRY(launch_rope_append(c, ka, 1, s));
            AttnPagedArgs aa{};
            aa.q = m->q; aa.k_cache = ka.k_cache; aa.v_cache = ka.v_cache; aa.block_table = m->block_table;
            aa.partial = m->partial; aa.partial_tok_cap = 1; aa.out = m->att; aa.d_pos = m->d_pos; aa.pos0 = 0;
            aa.n_head = d.n_head; aa.n_kv = d.n_kv; aa.head_dim = Hd; aa.page = m->page; aa.n_splits = m->n_splits;
            aa.pages_per_split = m->pages_per_split;
            aa.merge_ticket = d.n_kv >= 4 ? m->attn_ticket : nullptr;      // enough KV heads: the last split of each merges, no merge launch
            Q_TRY(launch_attn_paged(c, aa, 1, s));
            Q_TRY(launch_attn_gate(c, m->att, m->qg, d.n_head, Hd, s));
            a = q_gemv(l.o, m->att, qdim, x, H);
            a.epi = EPI_RESIDUAL; a.resid = x;
            Q_TRY(launch_gemv(c, a, s));
        }
        ggb_moe_params mp{};
        mp.x = x; mp.resid = x; mp.y = x2; mp.router = l.router;
        mp.gate_exps = static_cast<ggb_weight>(l.gate_exps); mp.up_exps = static_cast<ggb_weight>(l.up_exps);
        mp.down_exps = static_cast<ggb_weight>(l.down_exps);
        mp.sh_gate = static_cast<ggb_weight>(l.sh_gate); mp.sh_up = static_cast<ggb_weight>(l.sh_up); mp.sh_down = static_cast<ggb_weight>(l.sh_down);
        mp.sh_gate_inp = l.sh_gate_inp;
        mp.hidden = H; mp.eff = d.eff; mp.eff_sh = l.has_shared ? d.eff : 0; mp.n_expert = d.n_expert; mp.top_k = d.top_k;
        mp.gamma = l.post_norm; mp.eps = d.rms_eps;
        if (c->tp_size > 1) { mp.ep_first = m->ep_first; mp.ep_local = m->n_local_expert; }
        const MoeStacked stacked{l.gate_exps, l.up_exps, l.down_exps};
        Q_TRY(moe_ffn_enqueue(c, &mp, m->moe_scr, s, l.stacked ? &stacked : nullptr));
        std::swap(x, x2);
    }
    GemvArgs a = q_gemv(m->output ? m->output : m->tok_embd, x, H, m->logits, d.vocab);
    a.gamma = m->output_norm; a.eps = d.rms_eps;
    Q_TRY(launch_gemv(c, a, s));
    Q_TRY(launch_argmax(c, m->logits, d.vocab, m->d_next, m->amax_partial, s));
    q35_feedback_kernel<<<1, 1, 0, s>>>(m->d_next, m->d_tokens, m->d_pos, m->d_gen, m->d_step, m->d_forced, m->d_n_forced, d.ctx);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "feedback kernel");
}

// Runs n_steps tokens: the first n_forced come from `forced` (host), the rest are fed back on the device.
int q35_run(ggb_q35_model m, const int32_t* forced, int n_forced, int pos0, int n_steps) {
    Context* c = m->c;
    m->h_io[0] = forced[0]; m->h_io[1] = pos0; m->h_io[3] = 0; m->h_io[5] = n_forced;
    Q_TRY(cuda_status(c, cudaMemcpyAsync(m->d_forced, forced, sizeof(int32_t) * n_forced, cudaMemcpyHostToDevice, c->stream), "token upload"));
    Q_TRY(cuda_status(c, cudaMemcpyAsync(m->d_tokens, m->h_io, 4, cudaMemcpyHostToDevice, c->stream), "token upload"));
    Q_TRY(cuda_status(c, cudaMemcpyAsync(m->d_pos, m->h_io + 1, 4, cudaMemcpyHostToDevice, c->stream), "pos upload"));
    Q_TRY(cuda_status(c, cudaMemcpyAsync(m->d_step, m->h_io + 3, 4, cudaMemcpyHostToDevice, c->stream), "step upload"));
    Q_TRY(cuda_status(c, cudaMemcpyAsync(m->d_n_forced, m->h_io + 5, 4, cudaMemcpyHostToDevice, c->stream), "count upload"));
    for (int i = 0; i < n_steps; ++i) Q_TRY(cuda_status(c, cudaGraphLaunch(m->graph, c->stream), "graph launch"));
    c->launches += m->launches_per_step * n_steps;
    return GGB_OK;
}

}  // namespace

#define GGB_LOCK(h) std::lock_guard<std::mutex> _lk((h)->mu); cudaSetDevice((h)->device)

extern "C" {

int ggb_q35_create(ggb_handle h, const ggb_q35_desc* desc, ggb_q35_model* out) {
    if (!h) return GGB_UNAVAILABLE;
    if (!desc || !out) return set_status(h, GGB_INVALID_PARAM, "q35_create: null pointer");
    const ggb_q35_desc& d = *desc;
    if (d.n_layer <= 0 || d.hidden <= 0 || d.hidden % 256 || d.n_head <= 0 || d.n_kv <= 0 || d.n_head % d.n_kv || d.n_head / d.n_kv > 8 ||
        (d.head_dim != 64 && d.head_dim != 128 && d.head_dim != 256) || d.rope_dim <= 0 || d.rope_dim > d.head_dim || (d.rope_dim & 1) ||
        (d.sk != 64 && d.sk != 128) || d.n_vhead <= 0 || d.n_khead <= 0 || d.conv_k < 1 || d.conv_k > 8 || d.n_expert < 1 || d.n_expert > 1024 ||
        d.top_k < 1 || d.top_k > 16 || d.top_k > d.n_expert || d.eff <= 0 || d.eff % 256 || d.vocab <= 0 || d.ctx <= 0 ||
        (d.n_vhead * d.sk) % 256)
        return set_status(h, GGB_INVALID_PARAM, "q35_create: unsupported dimensions");
    if (h->tp_size > 1 && d.n_expert % h->tp_size) return set_status(h, GGB_INVALID_PARAM, "q35_create: n_expert must divide over the group");
    ggb_q35_model m = new ggb_q35_model_s();
    m->c = h; m->d = d;
    m->page = d.kv_page > 0 ? d.kv_page : 64;
    m->n_local_expert = d.n_expert / h->tp_size;
    m->ep_first = h->tp_rank * m->n_local_expert;
    m->layers.resize(d.n_layer);
    *out = m;
    return GGB_OK;
}

void ggb_q35_destroy(ggb_q35_model m) {
    if (!m) return;
    {
        GGB_LOCK(m->c);
        cudaStreamSynchronize(m->c->stream);
        if (m->graph) cudaGraphExecDestroy(m->graph);
        for (void* p : m->owned) cudaFree(p);
        if (m->h_io) cudaFreeHost(m->h_io);
        if (m->h_logits) cudaFreeHost(m->h_logits);
        free_weight(m->tok_embd); free_weight(m->output);
        for (Q35Layer& l : m->layers)
            for (DeviceWeight* w : {l.qkv, l.zgate, l.ssm_out, l.q, l.k, l.v, l.o, l.gate_exps, l.up_exps, l.down_exps, l.sh_gate, l.sh_up, l.sh_down}) free_weight(w);
    }
    delete m;
}

int ggb_q35_set_tensor(ggb_q35_model m, int slot, int layer, uint32_t type, int64_t N, int K, const void* host) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (!host) return set_status(c, GGB_INVALID_PARAM, "q35_set_tensor: null data");
    if (m->finalized) return set_status(c, GGB_INVALID_PARAM, "q35_set_tensor: model already finalized");
    GGB_LOCK(c);
    const ggb_q35_desc& d = m->d;
    const int H = d.hidden, qdim = d.n_head * d.head_dim, kvdim = d.n_kv * d.head_dim;
    const int key_dim = d.n_khead * d.sk, value_dim = d.n_vhead * d.sk, conv_dim = 2 * key_dim + value_dim;
    auto mat = [&](DeviceWeight** dst, int64_t wantN, int wantK) -> int {
        if (N != wantN || K != wantK) return set_status(c, GGB_INVALID_PARAM, "q35_set_tensor: shape does not match the model description");
        if (*dst) { free_weight(*dst); *dst = nullptr; }
        return upload_weight(c, type, N, K, host, dst);
    };
    auto vec_at = [&](float* dst, int64_t count) -> int {
        int st = cuda_status(c, cudaMemcpyAsync(dst, host, sizeof(float) * count, cudaMemcpyHostToDevice, c->stream), "vector upload");
        if (st != GGB_OK) return st;
        return cuda_status(c, cudaStreamSynchronize(c->stream), "vector upload");
    };
    auto vec = [&](float** dst, int64_t want) -> int {
        if (type != GGB_F32 || N * static_cast<int64_t>(K > 0 ? K : 1) != want) return set_status(c, GGB_INVALID_PARAM, "q35_set_tensor: F32 tensor of the wrong size");
        if (!*dst) Q_TRY(q_alloc(m, dst, static_cast<size_t>(want)));
        return vec_at(*dst, want);
    };
    if (slot < 10) {
        switch (slot) {
        case GGB_Q35_TOKEN_EMBD: return mat(&m->tok_embd, d.vocab, H);
        case GGB_Q35_OUTPUT: return mat(&m->output, d.vocab, H);
        case GGB_Q35_OUTPUT_NORM: return vec(&m->output_norm, H);
        default: return set_status(c, GGB_NOT_FOUND, "q35_set_tensor: unknown slot");
        }
    }
    if (layer < 0 || layer >= d.n_layer) return set_status(c, GGB_INVALID_PARAM, "q35_set_tensor: layer out of range");
    Q35Layer& l = m->layers[layer];
    const int64_t nl = m->n_local_expert;
    switch (slot) {
    case GGB_Q35_ATTN_NORM: return vec(&l.attn_norm, H);
    case GGB_Q35_POST_NORM: return vec(&l.post_norm, H);
    case GGB_Q35_SSM_QKV: return mat(&l.qkv, conv_dim, H);
    case GGB_Q35_SSM_GATE: return mat(&l.zgate, value_dim, H);
    case GGB_Q35_SSM_ALPHA:
    case GGB_Q35_SSM_BETA: {
        if (type != GGB_F32 || N != d.n_vhead || K != H) return set_status(c, GGB_INVALID_PARAM, "q35_set_tensor: ssm_alpha / ssm_beta must be F32 [n_vhead][hidden]");
        if (!l.alpha_beta) Q_TRY(q_alloc(m, &l.alpha_beta, static_cast<size_t>(2) * d.n_vhead * H));
        const bool beta = slot == GGB_Q35_SSM_BETA;
        (beta ? l.have_beta : l.have_alpha) = true;
        return vec_at(l.alpha_beta + (beta ? static_cast<size_t>(d.n_vhead) * H : 0), static_cast<int64_t>(d.n_vhead) * H);
    }
    case GGB_Q35_SSM_CONV: l.is_ssm = true; return vec(&l.conv_w, static_cast<int64_t>(conv_dim) * d.conv_k);
    case GGB_Q35_SSM_A: return vec(&l.ssm_a, d.n_vhead);
    case GGB_Q35_SSM_DT_BIAS: return vec(&l.dt_bias, d.n_vhead);
    case GGB_Q35_SSM_NORM: return vec(&l.ssm_norm, d.sk);
    case GGB_Q35_SSM_OUT: return mat(&l.ssm_out, H, value_dim);
    case GGB_Q35_ATTN_Q: return mat(&l.q, 2 * qdim, H);
    case GGB_Q35_ATTN_K: return mat(&l.k, kvdim, H);
    case GGB_Q35_ATTN_V: return mat(&l.v, kvdim, H);
    case GGB_Q35_ATTN_OUT: return mat(&l.o, H, qdim);
    case GGB_Q35_Q_NORM: return vec(&l.q_norm, d.head_dim);
    case GGB_Q35_K_NORM: return vec(&l.k_norm, d.head_dim);
    case GGB_Q35_ROUTER: return vec(&l.router, static_cast<int64_t>(d.n_expert) * H);
    case GGB_Q35_GATE_EXPS: return mat(&l.gate_exps, nl * d.eff, H);
    case GGB_Q35_UP_EXPS: return mat(&l.up_exps, nl * d.eff, H);
    case GGB_Q35_DOWN_EXPS: return mat(&l.down_exps, nl * H, d.eff);
    case GGB_Q35_SH_GATE: return mat(&l.sh_gate, d.eff, H);
    case GGB_Q35_SH_UP: return mat(&l.sh_up, d.eff, H);
    case GGB_Q35_SH_DOWN: return mat(&l.sh_down, H, d.eff);
    case GGB_Q35_SH_GATE_INP: return vec(&l.sh_gate_inp, H);
    default: return set_status(c, GGB_NOT_FOUND, "q35_set_tensor: unknown slot");
    }
}

int ggb_q35_finalize(ggb_q35_model m) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (m->finalized) return GGB_OK;
    GGB_LOCK(c);
    const ggb_q35_desc& d = m->d;
    if (!m->tok_embd || !m->output_norm) return set_status(c, GGB_INVALID_PARAM, "q35_finalize: token_embd / output_norm missing");
    const int H = d.hidden, Hd = d.head_dim, qdim = d.n_head * Hd, kvdim = d.n_kv * Hd;
    const int key_dim = d.n_khead * d.sk, value_dim = d.n_vhead * d.sk, conv_dim = 2 * key_dim + value_dim;
    m->n_attn_layers = 0;
    for (Q35Layer& l : m->layers) {
        const bool moe_ok = l.router && l.gate_exps && l.up_exps && l.down_exps && ((l.sh_gate != nullptr) == (l.sh_up != nullptr)) &&
                            ((l.sh_gate != nullptr) == (l.sh_down != nullptr));
        if (!l.attn_norm || !l.post_norm || !moe_ok) return set_status(c, GGB_INVALID_PARAM, "q35_finalize: a layer's norm or MoE tensor is missing");
        if (l.gate_exps->w.layout != 1 || l.up_exps->w.layout != 1 || l.down_exps->w.layout != 1)
            return set_status(c, GGB_INVALID_PARAM, "q35_finalize: expert tensors must be Q4_K or Q6_K");
        {
            auto wbytes = [](const DeviceWeight* w) -> uint64_t {
                return w ? static_cast<uint64_t>(w->w.N) * w->w.nb * format_info(w->w.type).block_bytes : 0;
            };
            l.bytes_experts = wbytes(l.gate_exps) + wbytes(l.up_exps) + wbytes(l.down_exps);
            l.bytes_shared = wbytes(l.sh_gate) + wbytes(l.sh_up) + wbytes(l.sh_down);
            l.has_shared = l.sh_gate != nullptr;
            if (l.has_shared && !l.stacked && d.top_k + 1 < 16 && l.sh_gate->w.layout == 1 && l.sh_up->w.layout == 1 && l.sh_down->w.layout == 1 &&
                l.sh_gate->w.type == l.gate_exps->w.type && l.sh_up->w.type == l.up_exps->w.type && l.sh_down->w.type == l.down_exps->w.type) {
                DeviceWeight *g2 = nullptr, *u2 = nullptr, *d2 = nullptr;
                int st = concat_weight_rows(c, l.gate_exps, l.sh_gate, &g2);
                if (st == GGB_OK) st = concat_weight_rows(c, l.up_exps, l.sh_up, &u2);
                if (st == GGB_OK) st = concat_weight_rows(c, l.down_exps, l.sh_down, &d2);
                if (st != GGB_OK) { free_weight(g2); free_weight(u2); free_weight(d2); return st; }
                for (DeviceWeight* w : {l.gate_exps, l.up_exps, l.down_exps, l.sh_gate, l.sh_up, l.sh_down}) free_weight(w);
                l.gate_exps = g2; l.up_exps = u2; l.down_exps = d2;
                l.sh_gate = l.sh_up = l.sh_down = nullptr;
                l.stacked = true;
            }
        }
        if (l.is_ssm) {
            if (!l.qkv || !l.zgate || !l.ssm_out || !l.have_alpha || !l.have_beta || !l.conv_w || !l.ssm_a || !l.dt_bias || !l.ssm_norm)
                return set_status(c, GGB_INVALID_PARAM, "q35_finalize: a DeltaNet layer tensor is missing");
            Q_TRY(q_alloc(m, &l.conv_state, static_cast<size_t>(std::max(d.conv_k - 1, 1)) * conv_dim, true));
            Q_TRY(q_alloc(m, &l.rec_state, static_cast<size_t>(d.n_vhead) * d.sk * d.sk, true));
        } else {
            if (!l.q || !l.k || !l.v || !l.o || !l.q_norm || !l.k_norm) return set_status(c, GGB_INVALID_PARAM, "q35_finalize: an attention layer tensor is missing");
            l.kv_slot = m->n_attn_layers++;
        }
    }
    // cos / sin rows exactly as rope_neox_partial forms them (src/cli/main.cpp:906-920): theta = pos * base^(-2i / rope_dim), float
    {
        const int rh = d.rope_dim / 2;
        std::vector<float> cs(static_cast<size_t>(d.ctx) * rh), sn(cs.size());
        for (int64_t p = 0; p < d.ctx; ++p)
            for (int i = 0; i < rh; ++i) {
                const float theta = static_cast<float>(p) * std::pow(d.rope_base, -2.0f * static_cast<float>(i) / static_cast<float>(d.rope_dim));
                cs[p * rh + i] = std::cos(theta);
                sn[p * rh + i] = std::sin(theta);
            }
        Q_TRY(q_alloc(m, &m->cos_tab, cs.size()));
        Q_TRY(q_alloc(m, &m->sin_tab, sn.size()));
        Q_TRY(cuda_status(c, cudaMemcpy(m->cos_tab, cs.data(), sizeof(float) * cs.size(), cudaMemcpyHostToDevice), "rope table"));
        Q_TRY(cuda_status(c, cudaMemcpy(m->sin_tab, sn.data(), sizeof(float) * sn.size(), cudaMemcpyHostToDevice), "rope table"));
    }
    m->n_pages = (d.ctx + m->page - 1) / m->page;
    attn_split_geometry(m->n_pages, d.n_kv, &m->n_splits, &m->pages_per_split);
    m->kv_layer_elems = static_cast<size_t>(m->n_pages) * d.n_kv * m->page * Hd;
    Q_TRY(q_alloc(m, &m->k_cache, m->kv_layer_elems * std::max(m->n_attn_layers, 1), true));
    Q_TRY(q_alloc(m, &m->v_cache, m->kv_layer_elems * std::max(m->n_attn_layers, 1), true));
    {
        std::vector<int32_t> bt(m->n_pages);
        for (int i = 0; i < m->n_pages; ++i) bt[i] = i;
        Q_TRY(q_alloc(m, &m->block_table, bt.size()));
        Q_TRY(cuda_status(c, cudaMemcpy(m->block_table, bt.data(), sizeof(int32_t) * bt.size(), cudaMemcpyHostToDevice), "block table"));
    }
    Q_TRY(q_alloc(m, &m->xa, H)); Q_TRY(q_alloc(m, &m->xb, H));
    Q_TRY(q_alloc(m, &m->mixed, conv_dim)); Q_TRY(q_alloc(m, &m->zgate, value_dim)); Q_TRY(q_alloc(m, &m->ab, 2 * d.n_vhead));
    Q_TRY(q_alloc(m, &m->conv, conv_dim)); Q_TRY(q_alloc(m, &m->o_all, value_dim));
    Q_TRY(q_alloc(m, &m->qg, 2 * qdim)); Q_TRY(q_alloc(m, &m->q, qdim)); Q_TRY(q_alloc(m, &m->k, kvdim)); Q_TRY(q_alloc(m, &m->v, kvdim));
    Q_TRY(q_alloc(m, &m->att, qdim));
    Q_TRY(q_alloc(m, &m->partial, attn_partial_floats(1, d.n_head, m->n_splits, Hd)));
    {
        ggb_moe_params mp{};
        mp.top_k = d.top_k; mp.eff = d.eff; mp.eff_sh = d.eff; mp.n_expert = d.n_expert;
        Q_TRY(q_alloc(m, &m->moe_scr, moe_scratch_floats(&mp), true));      // zeroed: the router kernel's ticket counter lives there
    }
    Q_TRY(q_alloc(m, &m->logits, static_cast<size_t>(d.vocab)));
    Q_TRY(q_alloc(m, &m->amax_partial, 512));
    Q_TRY(q_alloc(m, &m->attn_ticket, static_cast<size_t>(std::max(d.n_kv, 1)), true));
    Q_TRY(q_alloc(m, &m->d_tokens, 1, true)); Q_TRY(q_alloc(m, &m->d_pos, 1, true)); Q_TRY(q_alloc(m, &m->d_next, 1, true));
    Q_TRY(q_alloc(m, &m->d_step, 1, true)); Q_TRY(q_alloc(m, &m->d_n_forced, 1, true));
    Q_TRY(q_alloc(m, &m->d_gen, static_cast<size_t>(d.ctx), true));
    Q_TRY(q_alloc(m, &m->d_forced, static_cast<size_t>(d.ctx), true));
    Q_TRY(cuda_status(c, cudaMallocHost(&m->h_io, 64), "pinned alloc"));
    Q_TRY(cuda_status(c, cudaMallocHost(&m->h_logits, sizeof(float) * d.vocab), "pinned alloc"));

    // One eager step (sets the kernels' shared-memory attributes outside capture), then the capture.
    Q_TRY(q35_enqueue_step(m));
    Q_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "warm-up step"));
    const uint64_t before = c->launches;
    Q_TRY(cuda_status(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal), "begin capture"));
    const int st = q35_enqueue_step(m);
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
    if (st != GGB_OK) { if (graph) cudaGraphDestroy(graph); return st; }
    Q_TRY(cuda_status(c, e, "end capture"));
    m->launches_per_step = c->launches - before;
    c->launches = before;
    e = cudaGraphInstantiate(&m->graph, graph, 0);
    cudaGraphDestroy(graph);
    Q_TRY(cuda_status(c, e, "graph instantiate"));
    // the warm-up step wrote states and KV: start from zero
    for (Q35Layer& l : m->layers)
        if (l.is_ssm) {
            Q_TRY(cuda_status(c, cudaMemset(l.conv_state, 0, sizeof(float) * std::max(d.conv_k - 1, 1) * conv_dim), "state reset"));
            Q_TRY(cuda_status(c, cudaMemset(l.rec_state, 0, sizeof(float) * d.n_vhead * d.sk * d.sk), "state reset"));
        }
    Q_TRY(cuda_status(c, cudaMemset(m->k_cache, 0, sizeof(__nv_bfloat16) * m->kv_layer_elems * std::max(m->n_attn_layers, 1)), "kv reset"));
    Q_TRY(cuda_status(c, cudaMemset(m->v_cache, 0, sizeof(__nv_bfloat16) * m->kv_layer_elems * std::max(m->n_attn_layers, 1)), "kv reset"));
    m->finalized = true;
    return GGB_OK;
}

int ggb_q35_reset(ggb_q35_model m) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (!m->finalized) return set_status(c, GGB_INVALID_PARAM, "q35_reset: model not finalized");
    GGB_LOCK(c);
    const ggb_q35_desc& d = m->d;
    const size_t conv_dim = static_cast<size_t>(2) * d.n_khead * d.sk + static_cast<size_t>(d.n_vhead) * d.sk;
    for (Q35Layer& l : m->layers)
        if (l.is_ssm) {
            Q_TRY(cuda_status(c, cudaMemsetAsync(l.conv_state, 0, sizeof(float) * std::max(d.conv_k - 1, 1) * conv_dim, c->stream), "state reset"));
            Q_TRY(cuda_status(c, cudaMemsetAsync(l.rec_state, 0, sizeof(float) * d.n_vhead * d.sk * d.sk, c->stream), "state reset"));
        }
    return cuda_status(c, cudaStreamSynchronize(c->stream), "q35_reset");
}

int ggb_q35_prefill(ggb_q35_model m, const int32_t* host_tokens, int n_tok, int pos0, float* host_logits, int32_t* next_token) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (!m->finalized) return set_status(c, GGB_INVALID_PARAM, "q35_prefill: model not finalized");
    if (!host_tokens || n_tok <= 0 || pos0 < 0 || pos0 + n_tok > m->d.ctx) return set_status(c, GGB_INVALID_PARAM, "q35_prefill: bad arguments");
    for (int i = 0; i < n_tok; ++i)
        if (host_tokens[i] < 0 || host_tokens[i] >= m->d.vocab) return set_status(c, GGB_INVALID_PARAM, "q35_prefill: token out of range");
    GGB_LOCK(c);
    Q_TRY(q35_run(m, host_tokens, n_tok, pos0, n_tok));
    if (host_logits) Q_TRY(cuda_status(c, cudaMemcpyAsync(m->h_logits, m->logits, sizeof(float) * m->d.vocab, cudaMemcpyDeviceToHost, c->stream), "logits download"));
    Q_TRY(cuda_status(c, cudaMemcpyAsync(m->h_io + 2, m->d_next, 4, cudaMemcpyDeviceToHost, c->stream), "token download"));
    Q_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "q35_prefill"));
    if (host_logits) memcpy(host_logits, m->h_logits, sizeof(float) * m->d.vocab);
    if (next_token) *next_token = m->h_io[2];
    return check_device_error(c);
}

int ggb_q35_decode(ggb_q35_model m, int32_t token, int pos, float* host_logits, int32_t* next_token) {
    return ggb_q35_prefill(m, &token, 1, pos, host_logits, next_token);
}

int ggb_q35_generate(ggb_q35_model m, int32_t first_token, int pos0, int n, int32_t* host_out) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (!m->finalized) return set_status(c, GGB_INVALID_PARAM, "q35_generate: model not finalized");
    if (n <= 0 || pos0 < 0 || pos0 + n > m->d.ctx || first_token < 0 || first_token >= m->d.vocab || !host_out)
        return set_status(c, GGB_INVALID_PARAM, "q35_generate: bad arguments");
    GGB_LOCK(c);
    Q_TRY(q35_run(m, &first_token, 1, pos0, n));
    Q_TRY(cuda_status(c, cudaMemcpyAsync(host_out, m->d_gen, sizeof(int32_t) * n, cudaMemcpyDeviceToHost, c->stream), "tokens download"));
    Q_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "q35_generate"));
    return check_device_error(c);
}

int ggb_q35_read_state(ggb_q35_model m, int layer, float* host_out) {
    if (!m) return GGB_INVALID_PARAM;
    Context* c = m->c;
    if (!m->finalized || !host_out || layer < 0 || layer >= m->d.n_layer || !m->layers[layer].is_ssm)
        return set_status(c, GGB_INVALID_PARAM, "q35_read_state: not a finalized DeltaNet layer");
    GGB_LOCK(c);
    Q_TRY(cuda_status(c, cudaStreamSynchronize(c->stream), "q35_read_state"));
    return cuda_status(c, cudaMemcpy(host_out, m->layers[layer].rec_state, sizeof(float) * m->d.n_vhead * m->d.sk * m->d.sk, cudaMemcpyDeviceToHost), "state download");
}

uint64_t ggb_q35_decode_bytes(ggb_q35_model m, int pos) {
    if (!m || !m->finalized) return 0;
    const ggb_q35_desc& d = m->d;
    auto wb = [](const DeviceWeight* w) -> uint64_t {
        if (!w) return 0;
        const FormatInfo f = format_info(w->w.type);
        return static_cast<uint64_t>(w->w.N) * w->w.nb * f.block_bytes;
    };
    const uint64_t conv_dim = static_cast<uint64_t>(2) * d.n_khead * d.sk + static_cast<uint64_t>(d.n_vhead) * d.sk;
    uint64_t b = wb(m->output ? m->output : m->tok_embd);
    for (const Q35Layer& l : m->layers) {
        if (l.is_ssm) {
            b += wb(l.qkv) + wb(l.zgate) + wb(l.ssm_out) + static_cast<uint64_t>(2) * d.n_vhead * d.hidden * 4 + conv_dim * d.conv_k * 4;
            b += static_cast<uint64_t>(2) * d.n_vhead * d.sk * d.sk * 4;                       // recurrent state read + written
            b += static_cast<uint64_t>(2) * std::max(d.conv_k - 1, 0) * conv_dim * 4;          // conv state read + written
        } else {
            b += wb(l.q) + wb(l.k) + wb(l.v) + wb(l.o);
            b += static_cast<uint64_t>(2) * (pos + 1) * d.n_kv * d.head_dim * 2;               // K and V read, bf16
        }
        // router + the top_k chosen experts of this rank's share (all of them on one GPU) + the shared expert
        const uint64_t per_expert = l.bytes_experts / std::max(m->n_local_expert, 1);
        b += static_cast<uint64_t>(d.n_expert) * d.hidden * 4 + per_expert * d.top_k / m->c->tp_size + l.bytes_shared;
        b += static_cast<uint64_t>(d.hidden) * 4 * 3;                                          // norms, shared-gate vector
    }
    b += static_cast<uint64_t>(d.hidden) * 4;
    const FormatInfo fe = format_info(m->tok_embd->w.type);
    b += static_cast<uint64_t>(m->tok_embd->w.nb) * fe.block_bytes;
    return b;
}

}  // extern "C"
