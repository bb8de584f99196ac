// Mixture-of-experts FFN of one token on device pointers: router, top-k, softmax over the chosen
// experts, routed SwiGLU experts, sigmoid-gated shared expert.  Replaces the qwen35moe branch of the
// reference's layer loop, src/cli/main.cpp:3110-3193, which runs 9 experts x 3 host-pointer matmuls
// with a sync after each.
//
// Six launches, no host round trip (the chosen expert ids never leave the GPU):
//   1. moe_logits_kernel: logits = router[n_expert][hidden] . x (a warp per expert); moe_topk_kernel: k
//      rounds of block-wide arg-max (lowest index wins a tie), weights exp(l - max) / sum over the
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

// Router logits: one warp per expert row (row n_expert = the shared expert's gate vector), 8 rows per CTA,
// so the 2 MB router matrix is read by dozens of SMs rather than one.
__global__ void moe_logits_kernel(const float* __restrict__ x, const float* __restrict__ gamma, float eps, const float* __restrict__ router,
                                  int hidden, int n_expert, const float* __restrict__ sh_gate_inp, float* __restrict__ logits) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * 8 + warp;
    if (e > n_expert) return;
    const float* wr = e < n_expert ? router + static_cast<size_t>(e) * hidden : sh_gate_inp;
    if (!wr) return;
    // with gamma: the logit of rms_norm(x) * gamma, formed as (x * gamma) . w times the row's 1 / rms
    float acc = 0.0f, ss = 0.0f;
    for (int i = lane * 4; i < hidden; i += 128) {
        float4 a = *reinterpret_cast<const float4*>(x + i);
        const float4 b = __ldg(reinterpret_cast<const float4*>(wr + i));
        if (gamma) {
            const float4 g = __ldg(reinterpret_cast<const float4*>(gamma + i));
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            a.x *= g.x; a.y *= g.y; a.z *= g.z; a.w *= g.w;
        }
        acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o); ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o); }
    if (gamma) acc *= 1.0f / sqrtf(ss / static_cast<float>(hidden) + eps);
    if (lane == 0) logits[e] = acc;
}

// grid 1, block 256: k rounds of block-wide arg-max over the logits (n_expert <= 1024), softmax over the chosen,
// shared-expert gate.
// Expert parallel: sel / w describe this rank's share -- experts outside [ep_first, ep_first + ep_local) get
// id -1 (the GEMV kernels skip them) and weight 0; sel_glob / w_glob (optional) keep the global choice.
__global__ void moe_topk_kernel(const float* __restrict__ logits, int n_expert, int top_k, int has_gate, int ep_first, int ep_local,
                                int32_t* __restrict__ sel, float* __restrict__ w, int32_t* __restrict__ sel_glob, float* __restrict__ w_glob) {
    __shared__ float logit[1024];
    __shared__ float red_v[8];
    __shared__ int red_i[8];
    __shared__ float chosen[kMaxTopK];
    __shared__ int picked[kMaxTopK];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) logit[e] = logits[e];
    if (threadIdx.x == 0) w[top_k] = has_gate ? 1.0f / (1.0f + expf(-logits[n_expert])) : 1.0f;
    __syncthreads();
    for (int j = 0; j < top_k; ++j) {
        float bv = -INFINITY; int bi = 0x7FFFFFFF;
        for (int e = threadIdx.x; e < n_expert; e += blockDim.x) {
            const float v = logit[e];
            if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { red_v[warp] = bv; red_i[warp] = bi; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int q = 1; q < 8; ++q)
                if (red_v[q] > red_v[0] || (red_v[q] == red_v[0] && red_i[q] < red_i[0])) { red_v[0] = red_v[q]; red_i[0] = red_i[q]; }
            int e = red_i[0];
            float ev = red_v[0];
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
        __syncthreads();
    }
    if (threadIdx.x == 0) {
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

}  // namespace

size_t moe_scratch_floats(const ggb_moe_params* p) {
    return 64 + static_cast<size_t>(p->top_k) * p->eff + static_cast<size_t>(p->eff_sh > 0 ? p->eff_sh : 0) + p->n_expert + 1;
}

// Validates and enqueues on stream s; `scr` holds moe_scratch_floats(p) floats.  The caller holds the handle's lock.
int moe_ffn_enqueue(Context* h, const ggb_moe_params* p, float* scr, cudaStream_t s) {
    if (!p || !p->x || !p->y || !p->router || !p->gate_exps || !p->up_exps || !p->down_exps)
        return set_status(h, GGB_INVALID_PARAM, "moe_ffn: null pointer");
    if (p->hidden <= 0 || p->hidden % 256 || p->eff <= 0 || p->eff % 256 || p->n_expert < 1 || p->n_expert > 1024 || p->top_k < 1 ||
        p->top_k > kMaxTopK || p->top_k > p->n_expert)
        return set_status(h, GGB_INVALID_PARAM, "moe_ffn: hidden and eff must be multiples of 256, n_expert <= 1024, top_k <= 16");
    // expert parallel: this rank holds experts [ep_first, ep_first + ep_local) of the n_expert the router knows
    const bool ep = p->ep_local > 0;
    const int n_local = ep ? p->ep_local : p->n_expert, ep_first = ep ? p->ep_first : 0;
    if (ep && (p->ep_first < 0 || p->ep_first + p->ep_local > p->n_expert || h->tp_size < 2))
        return set_status(h, GGB_INVALID_PARAM, "moe_ffn: expert-parallel range outside the router's experts, or the handle is not in a group");
    const DeviceWeight *ge = reinterpret_cast<const DeviceWeight*>(p->gate_exps), *ue = reinterpret_cast<const DeviceWeight*>(p->up_exps),
                       *de = reinterpret_cast<const DeviceWeight*>(p->down_exps);
    if (ge->w.N != static_cast<int64_t>(n_local) * p->eff || ue->w.N != ge->w.N || ge->w.K != p->hidden || ue->w.K != p->hidden ||
        de->w.N != static_cast<int64_t>(n_local) * p->hidden || de->w.K != p->eff || ge->w.type != ue->w.type)
        return set_status(h, GGB_INVALID_PARAM, "moe_ffn: expert tensors must be [n_expert * eff][hidden] (gate, up) and [n_expert * hidden][eff] (down)");
    if (ge->w.layout != 1 || ue->w.layout != 1 || de->w.layout != 1)
        return set_status(h, GGB_INVALID_PARAM, "moe_ffn: expert tensors must be Q4_K or Q6_K in the tensor-core layout");
    // expert parallel: rank 0 alone adds the residual and the shared expert; the all-reduce spreads them
    const bool lead = !ep || h->tp_rank == 0;
    const bool shared = p->sh_gate && p->sh_up && p->sh_down && lead;
    const DeviceWeight *sg = reinterpret_cast<const DeviceWeight*>(p->sh_gate), *su = reinterpret_cast<const DeviceWeight*>(p->sh_up),
                       *sd = reinterpret_cast<const DeviceWeight*>(p->sh_down);
    if (shared && (sg->w.N != p->eff_sh || su->w.N != p->eff_sh || sg->w.K != p->hidden || su->w.K != p->hidden || sd->w.N != p->hidden ||
                   sd->w.K != p->eff_sh || p->eff_sh <= 0 || p->eff_sh % 256))
        return set_status(h, GGB_INVALID_PARAM, "moe_ffn: shared expert shapes do not match");
    // scratch: [sel: 16 ints][w: 17 floats][act: top_k * eff][act_sh: eff_sh][logits: n_expert + 1]
    int32_t* sel = reinterpret_cast<int32_t*>(scr);
    float* w = scr + 16;
    float* act = scr + 64;
    float* act_sh = act + static_cast<size_t>(p->top_k) * p->eff;
    float* logits = act_sh + (shared ? p->eff_sh : 0);
    const float* gate_vec = shared ? p->sh_gate_inp : static_cast<const float*>(nullptr);

    cudaError_t e = launch_pdl(h, moe_logits_kernel, dim3((p->n_expert + 1 + 7) / 8), dim3(256), 0, s, p->x, p->gamma, p->eps, p->router, p->hidden,
                               p->n_expert, gate_vec, logits);
    h->launches++;
    if (e != cudaSuccess) return cuda_status(h, e, "moe router logits");
    e = launch_pdl(h, moe_topk_kernel, dim3(1), dim3(256), 0, s, static_cast<const float*>(logits), p->n_expert, p->top_k, gate_vec ? 1 : 0,
                   ep_first, n_local, sel, w, p->sel_out, p->w_out);
    h->launches++;
    if (e != cudaSuccess) return cuda_status(h, e, "moe top-k");

    GemvArgs a{};
    a.w = ge->w; a.w2 = ue->w; a.x = p->x; a.M = 1; a.lda = p->hidden; a.y = act; a.ldc = p->top_k * p->eff; a.epi = EPI_SWIGLU;
    a.gamma = p->gamma; a.eps = p->eps;
    a.sel = sel; a.sel_mode = 1; a.sel_count = p->top_k; a.sel_rows = p->eff;
    int st = launch_gemv_mma(h, a, s);
    if (st != GGB_OK) return st == GGB_NOT_FOUND ? set_status(h, GGB_INVALID_PARAM, "moe_ffn: expert gate/up shape not covered") : st;

    a = GemvArgs{};
    a.w = de->w; a.x = act; a.M = 1; a.lda = p->top_k * p->eff; a.y = p->y; a.ldc = p->hidden;
    a.epi = (p->resid && lead) ? EPI_RESIDUAL : EPI_STORE; a.resid = lead ? p->resid : nullptr;
    a.sel = sel; a.sel_mode = 2; a.sel_count = p->top_k; a.sel_rows = p->hidden; a.xscale = w; a.xscale_run = p->eff;
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
    return moe_ffn_enqueue(h, p, scr, h->stream);
}
