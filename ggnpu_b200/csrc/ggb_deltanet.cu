// One token of a Gated DeltaNet (linear attention) layer after its projections: causal depthwise conv +
// SiLU with a rolling state, per-head L2 norm of q and k, the gated delta-rule recurrence on a
// [sk x sk] fp32 state per value head, and the gated RMS norm of the output.  Replaces
// src/cli/main.cpp:2925-3023 (the qwen35 / qwen35moe branch of the reference's layer loop, host loops
// over 32 heads x 128 x 128 state entries).  The projections around it (attn_qkv, attn_gate, ssm_alpha,
// ssm_beta, ssm_out) are ordinary quantised GEMVs.
//
// Two kernels, both HBM-bound (the recurrent state, sk * sk * 4 bytes per value head, is read and written
// once per token: 4 MB per layer at 32 heads x 128 x 128):
//   dn_conv_kernel  one thread per channel: conv over the conv_k - 1 stored inputs and this token's,
//                   SiLU, state roll.
//   dn_step_kernel  one CTA per value head, thread = (group of sk / 8 state rows, column v): the state
//                   tile lives in registers across the two passes (decay + prediction, then correction +
//                   read-out), partial sums over the row groups meet in shared memory, and the head's
//                   RMS statistic is a block reduction; state columns are independent, state rows are
//                   read and written with 128-byte coalesced accesses.
#include "ggb_internal.h"

namespace ggb {

namespace {

__global__ void dn_conv_kernel(const float* __restrict__ mixed, const float* __restrict__ conv_w, float* __restrict__ conv_state,
                               float* __restrict__ conv_out, int conv_dim, int conv_k) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= conv_dim) return;
    const int ckm1 = conv_k - 1;
    const float x = mixed[ch];
    float acc = conv_w[ch * conv_k + ckm1] * x;
    for (int t = 0; t < ckm1; ++t) acc += conv_w[ch * conv_k + t] * conv_state[static_cast<size_t>(t) * conv_dim + ch];
    conv_out[ch] = acc / (1.0f + expf(-acc));
    for (int t = 0; t < ckm1 - 1; ++t) conv_state[static_cast<size_t>(t) * conv_dim + ch] = conv_state[static_cast<size_t>(t + 1) * conv_dim + ch];
    if (ckm1 > 0) conv_state[static_cast<size_t>(ckm1 - 1) * conv_dim + ch] = x;
}

struct StepArgs {
    const float* conv;       // [2 * n_khead * sk + n_vhead * sk]  q | k | v after conv + SiLU
    const float* zgate;      // [n_vhead * sk]
    const float* araw;
    const float* braw;
    const float* ssm_a;
    const float* dt_bias;
    const float* ssm_norm;   // [sk]
    float* rec_state;        // [n_vhead][sk][sk]
    float* out;              // [n_vhead * sk]
    int n_khead, n_vhead;
    float rms_eps;
};

// SK = head size (64 or 128); block = 8 * SK threads; thread (kg, v) owns state rows kg * SK/8 .. of column v.
template <int SK>
__global__ void __launch_bounds__(8 * SK) dn_step_kernel(const StepArgs a) {
    constexpr int RPT = SK / 8;                       // state rows per thread
    __shared__ float qn[SK], kn[SK], part[8][SK], red[2][32];
    __shared__ float bcast[4];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int h = blockIdx.x, tid = threadIdx.x, v = tid % SK, kg = tid / SK;
    const int kh = h % a.n_khead;                     // value head h reads key / query head h % n_khead (main.cpp:2982)
    const int key_dim = a.n_khead * SK;
    const float* qc = a.conv + kh * SK;
    const float* kc = a.conv + key_dim + kh * SK;
    const float* vc = a.conv + 2 * key_dim + h * SK;
    float* S = a.rec_state + static_cast<size_t>(h) * SK * SK;

    // the state tile first: its loads are the long-latency part
    float s[RPT];
#pragma unroll
    for (int r = 0; r < RPT; ++r) s[r] = S[static_cast<size_t>(kg * RPT + r) * SK + v];

    // L2 norms of q and k over the head (eps 1e-6), q also times 1 / sqrt(sk)  (main.cpp:2956-2968)
    if (tid < SK) {
        const float qv = qc[tid], kv = kc[tid];
        float sq = qv * qv, s2 = kv * kv;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { sq += __shfl_xor_sync(0xFFFFFFFFu, sq, o); s2 += __shfl_xor_sync(0xFFFFFFFFu, s2, o); }
        if ((tid & 31) == 0) { red[0][tid >> 5] = sq; red[1][tid >> 5] = s2; }
    }
    __syncthreads();
    if (tid == 0) {
        float sq = 0.0f, s2 = 0.0f;
        for (int i = 0; i < SK / 32; ++i) { sq += red[0][i]; s2 += red[1][i]; }
        bcast[0] = (1.0f / sqrtf(sq + 1e-6f)) / sqrtf(static_cast<float>(SK));
        bcast[1] = 1.0f / sqrtf(s2 + 1e-6f);
        const float al = a.araw[h] + a.dt_bias[h];
        const float sp = al > 20.0f ? al : log1pf(expf(al));                 // softplus
        bcast[2] = expf(a.ssm_a[h] * sp);                                    // decay g
        bcast[3] = 1.0f / (1.0f + expf(-a.braw[h]));                         // beta
    }
    __syncthreads();
    if (tid < SK) { qn[tid] = qc[tid] * bcast[0]; kn[tid] = kc[tid] * bcast[1]; }
    const float g = bcast[2], beta = bcast[3];
    __syncthreads();

    // pass 1: S *= g, pred[v] = sum_k S[k][v] k[k]
    float p = 0.0f;
#pragma unroll
    for (int r = 0; r < RPT; ++r) { s[r] *= g; p = fmaf(s[r], kn[kg * RPT + r], p); }
    part[kg][v] = p;
    __syncthreads();
    float pred = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) pred += part[i][v];
    const float delta = beta * (vc[v] - pred);
    __syncthreads();
    // pass 2: S += k (x) delta, o[v] = sum_k S[k][v] q[k]
    float o = 0.0f;
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
        s[r] = fmaf(kn[kg * RPT + r], delta, s[r]);
        o = fmaf(s[r], qn[kg * RPT + r], o);
        S[static_cast<size_t>(kg * RPT + r) * SK + v] = s[r];
    }
    part[kg][v] = o;
    __syncthreads();
    if (tid < SK) {
        float oh = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) oh += part[i][tid];
        // gated RMS norm: norm first, then the gate (main.cpp:3016-3023)
        float ss = oh * oh;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, off);
        if ((tid & 31) == 0) red[0][tid >> 5] = ss;
        // (all SK threads reach the barrier below)
        asm volatile("bar.sync 1, %0;" ::"n"(SK) : "memory");
        float tot = 0.0f;
        for (int i = 0; i < SK / 32; ++i) tot += red[0][i];
        const float r = 1.0f / sqrtf(tot / static_cast<float>(SK) + a.rms_eps);
        const float z = a.zgate[h * SK + tid];
        a.out[h * SK + tid] = (oh * r * a.ssm_norm[tid]) * (z / (1.0f + expf(-z)));
    }
}

}  // namespace

// Validates and enqueues on stream s; `conv` holds 2 * n_khead * sk + n_vhead * sk floats.  The caller holds the handle's lock.
int deltanet_step_enqueue(Context* h, const ggb_deltanet_params* p, float* conv, cudaStream_t s) {
    if (!p || !p->mixed || !p->zgate || !p->araw || !p->braw || !p->conv_w || !p->ssm_a || !p->dt_bias || !p->ssm_norm ||
        !p->conv_state || !p->rec_state || !p->out)
        return set_status(h, GGB_INVALID_PARAM, "deltanet_step: null pointer");
    if ((p->sk != 64 && p->sk != 128) || p->n_khead < 1 || p->n_vhead < 1 || p->conv_k < 1 || p->conv_k > 8)
        return set_status(h, GGB_INVALID_PARAM, "deltanet_step: head size must be 64 or 128, conv_k 1..8");
    const int conv_dim = 2 * p->n_khead * p->sk + p->n_vhead * p->sk;
    cudaError_t e = launch_pdl(h, dn_conv_kernel, dim3((conv_dim + 255) / 256), dim3(256), 0, s, p->mixed, p->conv_w, p->conv_state, conv, conv_dim, p->conv_k);
    h->launches++;
    if (e != cudaSuccess) return cuda_status(h, e, "deltanet conv");
    StepArgs a{};
    a.conv = conv; a.zgate = p->zgate; a.araw = p->araw; a.braw = p->braw; a.ssm_a = p->ssm_a; a.dt_bias = p->dt_bias; a.ssm_norm = p->ssm_norm;
    a.rec_state = p->rec_state; a.out = p->out; a.n_khead = p->n_khead; a.n_vhead = p->n_vhead; a.rms_eps = p->rms_eps;
    if (p->sk == 128) e = launch_pdl(h, dn_step_kernel<128>, dim3(p->n_vhead), dim3(1024), 0, s, a);
    else e = launch_pdl(h, dn_step_kernel<64>, dim3(p->n_vhead), dim3(512), 0, s, a);
    h->launches++;
    return cuda_status(h, e, "deltanet step");
}

}  // namespace ggb

using namespace ggb;

extern "C" int ggb_deltanet_step_device(ggb_handle h, const ggb_deltanet_params* p) {
    if (!h) return GGB_UNAVAILABLE;
    if (!p || p->n_khead < 1 || p->n_vhead < 1 || p->sk < 1) return set_status(h, GGB_INVALID_PARAM, "deltanet_step: bad arguments");
    std::lock_guard<std::mutex> lk(h->mu);
    cudaSetDevice(h->device);
    const size_t conv_dim = static_cast<size_t>(2) * p->n_khead * p->sk + static_cast<size_t>(p->n_vhead) * p->sk;
    float* conv = static_cast<float*>(scratch(h, 3, sizeof(float) * conv_dim));
    if (!conv) return h->last_status;
    return deltanet_step_enqueue(h, p, conv, h->stream);
}
