// Mixture-of-experts FFN of one token on device pointers: router, top-k, softmax over the chosen
// experts, routed SwiGLU experts, sigmoid-gated shared expert.  Replaces the qwen35moe branch of the
// reference's layer loop, src/cli/main.cpp:3110-3193, which runs 9 experts x 3 host-pointer matmuls
// with a sync after each.
//
// Five launches (three when the shared expert is stacked behind the routed ones), no host round trip (the chosen expert ids never leave the GPU):
//   1. moe_route_kernel: logits = router[n_expert][hidden] . x (a warp per expert), then, in the CTA that finishes
//      last, k rounds of block-wide arg-max (lowest index wins a tie), weights exp(l - max) / sum over the
//      chosen, shared-expert gate sigmoid(g . x);
//   2. gate/up of the k chosen experts as ONE tensor-core GEMV over gathered row ranges (the expert
//      tensors are uploaded whole, [n_expert * eff][hidden]; the kernel's producer maps its row groups
//      through the id list) with the SwiGLU epilogue -> act[k][eff];
//   3. down of the k experts as ONE GEMV whose K axis is the k experts' K ranges side by side, the
//      router weights folded into the activations (x scale per run of eff), residual added in the
//      epilogue;
//   4. the shared expert: the ordinary fused gate/up GEMV and a down GEMV that accumulates onto y.
#include "ggb_internal.h"

namespace ggb {

namespace {

constexpr int kMaxTopK = 16;

// k rounds of block-wide arg-max over the logits (n_expert <= 1024; lowest index wins a tie), softmax over the chosen,
// shared-expert gate.  256 threads of one CTA.
// Expert parallel: sel / w describe this rank's share -- experts outside [ep_first, ep_first + ep_local) get
// id -1 (the GEMV kernels skip them) and weight 0; sel_glob / w_glob (optional) keep the global choice.
// shared_slot >= 0: the shared expert is stacked behind the routed ones in the expert tensors; it then becomes choice
// number top_k with id shared_slot (-2: stacked, but held by another rank -> id -1) and its sigmoid gate as weight.
__device__ void moe_topk_body(const float* __restrict__ logits, int n_expert, int top_k, int has_gate, int ep_first, int ep_local, int shared_slot,
                              int32_t* __restrict__ sel, float* __restrict__ w, int32_t* __restrict__ sel_glob, float* __restrict__ w_glob) {
    __shared__ float logit[1024];
    __shared__ float chosen[kMaxTopK];
    __shared__ int picked[kMaxTopK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) logit[e] = __ldcg(logits + e);      // written by other CTAs of this launch
    if (threadIdx.x == 0) {
        w[top_k] = has_gate ? 1.0f / (1.0f + expf(-__ldcg(logits + n_expert))) : 1.0f;
        if (shared_slot != -1) sel[top_k] = shared_slot >= 0 ? shared_slot : -1;
    }
    __syncthreads();
    if (warp != 0) return;
    // one warp, no block-wide barrier: k rounds of (each lane scans its strided share, warp arg-max by shuffles)
    for (int j = 0; j < top_k; ++j) {
        float bv = -INFINITY; int bi = 0x7FFFFFFF;
        for (int e = lane; e < n_expert; e += 32) {
            const float v = logit[e];
            if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            int e = bi;
            float ev = bv;
            bool none = e < 0 || e >= n_expert;
            for (int r = 0; r < j && !none; ++r) none = picked[r] == e;      // an exhausted (-inf) entry won the tie
            if (none) {
                // no candidate compared greater or equal (every remaining logit is NaN): take the lowest
                // index not chosen yet, so that the ids stay valid rows of the expert tensors and the NaN
                // reaches the output through the weights instead of through a wild index
                e = 0;
                for (int q = 0; q < n_expert; ++q) {
                    bool taken = false;
                    for (int r = 0; r < j; ++r) taken = taken || picked[r] == q;
                    if (!taken) { e = q; break; }
                }
                ev = logit[e];
            }
            picked[j] = e;
            if (sel_glob) sel_glob[j] = e;
            sel[j] = (e >= ep_first && e < ep_first + ep_local) ? e - ep_first : -1;
            chosen[j] = ev;
            logit[e] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0) {
        const float mx = chosen[0];
        float sum = 0.0f;
        for (int j = 0; j < top_k; ++j) { chosen[j] = expf(chosen[j] - mx); sum += chosen[j]; }
        for (int j = 0; j < top_k; ++j) {
            const float wj = chosen[j] / sum;
            if (w_glob) w_glob[j] = wj;
            w[j] = sel[j] >= 0 ? wj : 0.0f;
        }
        if (w_glob) w_glob[top_k] = w[top_k];
    }
}

struct MoeRouteArgs {
    const float* x; const float* gamma; float eps; const float* router; int hidden, n_expert; const float* sh_gate_inp; float* logits;
    unsigned* ticket;          // counts finished CTAs over all launches (starts at a multiple of the grid size)
    int top_k, ep_first, ep_local, shared_slot;
    int32_t* sel; float* w; int32_t* sel_glob; float* w_glob;
};

// Router logits and the choice in one launch.  One warp per expert row (row n_expert = the shared expert's gate vector),
// 8 rows per CTA, so the 2 MB router matrix is read by dozens of SMs rather than one; the CTA that finishes last
// (a ticket counter behind a fence) then holds all logits and runs the top-k.
__global__ void __launch_bounds__(256) moe_route_kernel(const MoeRouteArgs a) {
    __shared__ int is_last;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * 8 + warp;
    const float* wr = e < a.n_expert ? a.router + static_cast<size_t>(e) * a.hidden : (e == a.n_expert ? a.sh_gate_inp : nullptr);
    // x * gamma once per CTA into shared memory (hidden <= 8192), the sum of squares with it; a warp then has all the
    // 16-byte loads of its router row in flight at once (sixteen at a time)
    __shared__ __align__(16) float xg[8192];
    __shared__ float ss_w[8];
    {
        float ss = 0.0f;
        for (int i = threadIdx.x * 4; i < a.hidden; i += 1024) {
            float4 v = *reinterpret_cast<const float4*>(a.x + i);
            if (a.gamma) {
                const float4 g = __ldg(reinterpret_cast<const float4*>(a.gamma + i));
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                v.x *= g.x; v.y *= g.y; v.z *= g.z; v.w *= g.w;
            }
            *reinterpret_cast<float4*>(xg + i) = v;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
        if (lane == 0) ss_w[warp] = ss;
    }
    __syncthreads();
    if (wr) {
        float acc = 0.0f;
        for (int i0 = lane * 4; i0 < a.hidden; i0 += 2048) {
            float4 wv[16];
#pragma unroll
            for (int u = 0; u < 16; ++u)
                if (i0 + 128 * u < a.hidden) wv[u] = __ldg(reinterpret_cast<const float4*>(wr + i0 + 128 * u));
#pragma unroll
            for (int u = 0; u < 16; ++u)
                if (i0 + 128 * u < a.hidden) {
                    const float4 v = *reinterpret_cast<const float4*>(xg + i0 + 128 * u), b = wv[u];
                    acc += v.x * b.x + v.y * b.y + v.z * b.z + v.w * b.w;
                }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
        if (a.gamma) {
            float ss = 0.0f;
#pragma unroll
            for (int q = 0; q < 8; ++q) ss += ss_w[q];
            acc *= 1.0f / sqrtf(ss / static_cast<float>(a.hidden) + a.eps);
        }
        if (lane == 0) a.logits[e] = acc;
    }
    __threadfence();                       // this CTA's logits are visible before its ticket is
    __syncthreads();
    if (threadIdx.x == 0) is_last = (atomicAdd(a.ticket, 1u) + 1u) % gridDim.x == 0u;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    moe_topk_body(a.logits, a.n_expert, a.top_k, a.sh_gate_inp ? 1 : 0, a.ep_first, a.ep_local, a.shared_slot, a.sel, a.w, a.sel_glob, a.w_glob);
}

}  // namespace

size_t moe_scratch_floats(const ggb_moe_params* p) {
    return 64 + static_cast<size_t>(p->top_k + 1) * p->eff + static_cast<size_t>(p->eff_sh > 0 ? p->eff_sh : 0) + p->n_expert + 1;
}

// Validates and enqueues on stream s; `scr` holds moe_scratch_floats(p) floats whose first 64 words were zero when the
// scratch was first used (the ticket counter of moe_route_kernel lives there).  The caller holds the handle's lock.
// stacked (optional): the expert tensors with the shared expert's matrices appended as expert number n_local
// (concat_weight_rows); the shared expert then rides in the routed experts' two launches as choice number top_k.
int moe_ffn_enqueue(Context* h, const ggb_moe_params* p, float* scr, cudaStream_t s, const MoeStacked* stacked) {
    if (!p || !p->x || !p->y || !p->router || !p->gate_exps || !p->up_exps || !p->down_exps)
        return set_status(h, GGB_INVALID_PARAM, "moe_ffn: null pointer");
    if (p->hidden <= 0 || p->hidden % 256 || p->eff <= 0 || p->eff % 256 || p->n_expert < 1 || p->n_expert > 1024 || p->top_k < 1 ||
        p->top_k > kMaxTopK - 1 || p->top_k > p->n_expert || p->hidden > 8192)
        return set_status(h, GGB_INVALID_PARAM, "moe_ffn: hidden (<= 8192) and eff must be multiples of 256, n_expert <= 1024, top_k <= 15");
    // expert parallel: this rank holds experts [ep_first, ep_first + ep_local) of the n_expert the router knows
    const bool ep = p->ep_local > 0;
    const int n_local = ep ? p->ep_local : p->n_expert, ep_first = ep ? p->ep_first : 0;
    if (ep && (p->ep_first < 0 || p->ep_first + p->ep_local > p->n_expert || h->tp_size < 2))
        return set_status(h, GGB_INVALID_PARAM, "moe_ffn: expert-parallel range outside the router's experts, or the handle is not in a group");
    const DeviceWeight *ge = reinterpret_cast<const DeviceWeight*>(p->gate_exps), *ue = reinterpret_cast<const DeviceWeight*>(p->up_exps),
                       *de = reinterpret_cast<const DeviceWeight*>(p->down_exps);
    const int n_rows = stacked ? n_local + 1 : n_local;          // experts in the tensors
    if (stacked) { ge = stacked->gate; ue = stacked->up; de = stacked->down; }
    if (ge->w.N != static_cast<int64_t>(n_rows) * p->eff || ue->w.N != ge->w.N || ge->w.K != p->hidden || ue->w.K != p->hidden ||
        de->w.N != static_cast<int64_t>(n_rows) * p->hidden || de->w.K != p->eff || ge->w.type != ue->w.type)
        return set_status(h, GGB_INVALID_PARAM, "moe_ffn: expert tensors must be [n_expert * eff][hidden] (gate, up) and [n_expert * hidden][eff] (down)");
    if (ge->w.layout != 1 || ue->w.layout != 1 || de->w.layout != 1)
        return set_status(h, GGB_INVALID_PARAM, "moe_ffn: expert tensors must be Q4_K or Q6_K in the tensor-core layout");
    // expert parallel: rank 0 alone adds the residual and the shared expert; the all-reduce spreads them
    const bool lead = !ep || h->tp_rank == 0;
    const bool shared = !stacked && p->sh_gate && p->sh_up && p->sh_down && lead;
    const DeviceWeight *sg = reinterpret_cast<const DeviceWeight*>(p->sh_gate), *su = reinterpret_cast<const DeviceWeight*>(p->sh_up),
                       *sd = reinterpret_cast<const DeviceWeight*>(p->sh_down);
    if (shared && (sg->w.N != p->eff_sh || su->w.N != p->eff_sh || sg->w.K != p->hidden || su->w.K != p->hidden || sd->w.N != p->hidden ||
                   sd->w.K != p->eff_sh || p->eff_sh <= 0 || p->eff_sh % 256))
        return set_status(h, GGB_INVALID_PARAM, "moe_ffn: shared expert shapes do not match");
    if (stacked && p->eff_sh != p->eff) return set_status(h, GGB_INVALID_PARAM, "moe_ffn: a stacked shared expert must have the routed experts' width");
    // scratch: [sel: 16 ints][w: 17 floats][ticket at word 40][act: (top_k + 1) * eff][act_sh: eff_sh][logits: n_expert + 1]
    int32_t* sel = reinterpret_cast<int32_t*>(scr);
    float* w = scr + 16;
    float* act = scr + 64;
    float* act_sh = act + static_cast<size_t>(p->top_k + 1) * p->eff;
    float* logits = act_sh + (p->eff_sh > 0 ? p->eff_sh : 0);
    const bool gate = (shared || stacked) && p->sh_gate_inp;
    const int n_sel = stacked ? p->top_k + 1 : p->top_k;

    MoeRouteArgs ra{};
    ra.x = p->x; ra.gamma = p->gamma; ra.eps = p->eps; ra.router = p->router; ra.hidden = p->hidden; ra.n_expert = p->n_expert;
    ra.sh_gate_inp = gate ? p->sh_gate_inp : nullptr; ra.logits = logits; ra.ticket = reinterpret_cast<unsigned*>(scr + 40);
    ra.top_k = p->top_k; ra.ep_first = ep_first; ra.ep_local = n_local; ra.shared_slot = stacked ? (lead ? n_local : -2) : -1;
    ra.sel = sel; ra.w = w; ra.sel_glob = p->sel_out; ra.w_glob = p->w_out;
    cudaError_t e = launch_pdl(h, moe_route_kernel, dim3((p->n_expert + 1 + 7) / 8), dim3(256), 0, s, ra);
    h->launches++;
    if (e != cudaSuccess) return cuda_status(h, e, "moe router");

    GemvArgs a{};
    a.w = ge->w; a.w2 = ue->w; a.x = p->x; a.M = 1; a.lda = p->hidden; a.y = act; a.ldc = n_sel * p->eff; a.epi = EPI_SWIGLU;
    a.gamma = p->gamma; a.eps = p->eps;
    a.sel = sel; a.sel_mode = 1; a.sel_count = n_sel; a.sel_rows = p->eff;
    int st = launch_gemv_mma(h, a, s);
    if (st != GGB_OK) return st == GGB_NOT_FOUND ? set_status(h, GGB_INVALID_PARAM, "moe_ffn: expert gate/up shape not covered") : st;

    a = GemvArgs{};
    a.w = de->w; a.x = act; a.M = 1; a.lda = n_sel * p->eff; a.y = p->y; a.ldc = p->hidden;
    a.epi = (p->resid && lead) ? EPI_RESIDUAL : EPI_STORE; a.resid = lead ? p->resid : nullptr;
    a.sel = sel; a.sel_mode = 2; a.sel_count = n_sel; a.sel_rows = p->hidden; a.xscale = w; a.xscale_run = p->eff;
    st = launch_gemv_mma(h, a, s);
    if (st != GGB_OK) return st == GGB_NOT_FOUND ? set_status(h, GGB_INVALID_PARAM, "moe_ffn: expert down shape not covered") : st;

    if (shared) {
        a = GemvArgs{};
        a.w = sg->w; a.w2 = su->w; a.x = p->x; a.M = 1; a.lda = p->hidden; a.y = act_sh; a.ldc = p->eff_sh; a.epi = EPI_SWIGLU;
        a.gamma = p->gamma; a.eps = p->eps;
        st = launch_gemv(h, a, s);
        if (st != GGB_OK) return st;
        a = GemvArgs{};
        a.w = sd->w; a.x = act_sh; a.M = 1; a.lda = p->eff_sh; a.y = p->y; a.ldc = p->hidden; a.epi = EPI_RESIDUAL; a.resid = p->y;
        a.xscale = w + p->top_k; a.xscale_run = p->eff_sh;
        st = launch_gemv(h, a, s);
        if (st != GGB_OK) return st;
    }
    if (ep) return tp_all_reduce(h, p->y, static_cast<size_t>(p->hidden), s);      // sum of the ranks' expert shares (+ rank 0's residual, shared expert)
    return GGB_OK;
}

}  // namespace ggb

using namespace ggb;

extern "C" int ggb_moe_ffn_device(ggb_handle h, const ggb_moe_params* p) {
    if (!h) return GGB_UNAVAILABLE;
    if (!p) return set_status(h, GGB_INVALID_PARAM, "moe_ffn: null pointer");
    std::lock_guard<std::mutex> lk(h->mu);
    cudaSetDevice(h->device);
    float* scr = static_cast<float*>(scratch(h, 3, sizeof(float) * moe_scratch_floats(p)));
    if (!scr) return h->last_status;
    const int st = cuda_status(h, cudaMemsetAsync(scr, 0, 64 * sizeof(float), h->stream), "moe_ffn scratch");      // ticket counter
    if (st != GGB_OK) return st;
    return moe_ffn_enqueue(h, p, scr, h->stream, nullptr);
}
