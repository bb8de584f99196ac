// Temperature sampling: the temp > 0 branch of the reference's sample_token (src/cli/main.cpp:839-864) with the
// logits left in HBM.
//
// The reference: probs_i = exp((v_i - max) / temp) / sum_exp in float, then a std::discrete_distribution over the
// probs driven by std::mt19937(seed): the distribution normalises the probs again in double, builds their running
// sums and returns the first index whose running sum reaches a uniform double u in [0, 1); before the draw the
// caller's seed is replaced by the generator's first output.  Here the generator runs on the host (the sequence of
// (u, next seed) pairs depends on the seed alone, so the u of every step of a generation can be produced up front)
// and the 128 K-entry part runs on the GPU: exponentials, both normalisations and the search for the crossing.
// The float sum_exp and the double running sums are added in a different order than the reference's sequential
// loops; sum_exp cancels in the second normalisation, so the chosen index differs from the reference's only when u
// lies within rounding distance (about 1e-7 relative) of a boundary between two tokens.
#include <random>

#include "ggb_internal.h"

namespace ggb {

namespace {

constexpr int kSampleChunk = 4096;       // elements per CTA: 256 threads x 16
constexpr int kSampleMaxParts = 1024;

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// e_i = exp((v_i - max) / temp), float as the reference (expf is within 1 ulp of the host's); per-CTA sums.
__global__ void __launch_bounds__(256) sample_exp_kernel(const float* __restrict__ logits, int n, const int32_t* __restrict__ d_argmax,
                                                          const float* __restrict__ d_temp, float* __restrict__ e, float* __restrict__ part) {
    __shared__ float red[8];
    const float mx = logits[d_argmax[0]], temp = d_temp[0];
    const int base = blockIdx.x * kSampleChunk;
    float s = 0.0f;
#pragma unroll 4
    for (int k = 0; k < 16; ++k) {
        const int i = base + k * 256 + threadIdx.x;
        if (i < n) { const float v = expf((logits[i] - mx) / temp); e[i] = v; s += v; }
    }
    s = warp_sum_f(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) { float t = 0.0f; for (int w = 0; w < 8; ++w) t += red[w]; part[blockIdx.x] = t; }
}

// p_i = e_i / sum_exp (float division, `p /= sum_exp`); per-CTA sums of p in double (the distribution's own normaliser).
__global__ void __launch_bounds__(256) sample_norm_kernel(float* __restrict__ e, int n, const float* __restrict__ part, int n_part, double* __restrict__ dpart) {
    __shared__ double red[8];
    float sum_exp = 0.0f;
    for (int b = 0; b < n_part; ++b) sum_exp += part[b];          // the same order in every CTA
    const int base = blockIdx.x * kSampleChunk;
    double s = 0.0;
#pragma unroll 4
    for (int k = 0; k < 16; ++k) {
        const int i = base + k * 256 + threadIdx.x;
        if (i < n) { const float p = e[i] / sum_exp; e[i] = p; s += static_cast<double>(p); }
    }
    s = warp_sum_d(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) { double t = 0.0; for (int w = 0; w < 8; ++w) t += red[w]; dpart[blockIdx.x] = t; }
}

// One CTA: the first index whose running sum of p / S reaches u (std::lower_bound over the cumulative
// probabilities, whose last entry the distribution pins to 1).  Compared as running sum >= u * S.
__global__ void __launch_bounds__(256) sample_pick_kernel(const float* __restrict__ p, int n, const double* __restrict__ dpart, int n_part,
                                                           const double* __restrict__ d_u, const int32_t* __restrict__ d_step, int32_t* __restrict__ out) {
    __shared__ double sh_pref[256];
    __shared__ double sh_target, sh_base;
    __shared__ int sh_block, sh_found;
    const int tid = threadIdx.x;
    if (tid == 0) {
        double S = 0.0;
        for (int b = 0; b < n_part; ++b) S += dpart[b];
        const double target = d_u[d_step ? d_step[0] : 0] * S;
        double run = 0.0;                      // sum of the chunks before the one that holds the crossing
        int blk = n_part - 1;                  // (the last chunk, should rounding leave the total just short of the target)
        for (int b = 0; b < n_part; ++b) {
            if (run + dpart[b] >= target || b == n_part - 1) { blk = b; break; }
            run += dpart[b];
        }
        sh_target = target; sh_base = run; sh_block = blk; sh_found = 0x7FFFFFFF;
    }
    __syncthreads();
    const int first = sh_block * kSampleChunk + tid * 16;          // 16 consecutive elements per thread
    double v[16], ls = 0.0;
#pragma unroll
    for (int k = 0; k < 16; ++k) { v[k] = first + k < n ? static_cast<double>(p[first + k]) : 0.0; ls += v[k]; }
    sh_pref[tid] = ls;
    __syncthreads();
    if (tid == 0) {                                                // exclusive running sums over the 256 threads
        double run = sh_base;
        for (int t = 0; t < 256; ++t) { const double x = sh_pref[t]; sh_pref[t] = run; run += x; }
    }
    __syncthreads();
    double run = sh_pref[tid];
    const double target = sh_target;
    if (run < target || (sh_block == 0 && tid == 0)) {
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            run += v[k];
            if (run >= target && first + k < n) { atomicMin(&sh_found, first + k); break; }
        }
    }
    __syncthreads();
    if (tid == 0) {
        int idx = sh_found;
        if (idx == 0x7FFFFFFF) idx = min(n, (sh_block + 1) * kSampleChunk) - 1;     // rounding left the crossing just past this chunk
        if (sh_block == n_part - 1 && idx >= n) idx = n - 1;
        out[0] = idx;
    }
}

}  // namespace

size_t sample_scratch_bytes(int n) { return sizeof(float) * (static_cast<size_t>(n) + kSampleMaxParts) + sizeof(double) * kSampleMaxParts + 256; }

// d_argmax: index of the first maximum of the logits (already computed); d_temp, d_u[d_step[0]]: temperature and
// the step's uniform draw in device memory, so a captured graph can be replayed with new values.
int sample_enqueue(Context* c, const float* d_logits, int n, const int32_t* d_argmax, const float* d_temp, const double* d_u, const int32_t* d_step,
                   void* scratch, int32_t* d_out, cudaStream_t s) {
    const int n_part = (n + kSampleChunk - 1) / kSampleChunk;
    if (n < 1 || n_part > kSampleMaxParts) return set_status(c, GGB_INVALID_PARAM, "sample: vocabulary size out of range");
    // scratch: doubles first (alignment), then the float partial sums, then the probabilities
    double* dpart = static_cast<double*>(scratch);
    float* part = reinterpret_cast<float*>(dpart + kSampleMaxParts);
    float* e = part + kSampleMaxParts;
    sample_exp_kernel<<<n_part, 256, 0, s>>>(d_logits, n, d_argmax, d_temp, e, part);
    sample_norm_kernel<<<n_part, 256, 0, s>>>(e, n, part, n_part, dpart);
    sample_pick_kernel<<<1, 256, 0, s>>>(e, n, dpart, n_part, d_u, d_step, d_out);
    c->launches += 3;
    return cuda_status(c, cudaGetLastError(), "sample");
}

// One draw of the reference's generator: std::mt19937 seeded with `seed`; its first output replaces the seed, the
// distribution then takes one uniform double (two 32-bit outputs) from the same generator (src/cli/main.cpp:841,862-863).
double sample_next_uniform(uint64_t* seed) {
    std::mt19937 rng(*seed);
    *seed = rng();
    return std::generate_canonical<double, 53>(rng);
}

}  // namespace ggb

using namespace ggb;

static int sample_common(ggb_handle h, const float* d_logits, int n, float temp, uint64_t* seed, int32_t* token) {
    // scratch slot 1: [argmax partials 512 words][argmax index][temp][u][sampled] then the sampler's own scratch
    uint8_t* base = static_cast<uint8_t*>(scratch(h, 1, 4096 + sample_scratch_bytes(n)));
    if (!base) return h->last_status;
    float* amax_partial = reinterpret_cast<float*>(base);
    int32_t* d_arg = reinterpret_cast<int32_t*>(base + 2048);
    float* d_temp = reinterpret_cast<float*>(base + 2048 + 16);
    double* d_u = reinterpret_cast<double*>(base + 2048 + 32);
    int32_t* d_out = reinterpret_cast<int32_t*>(base + 2048 + 48);
    cudaStream_t s = h->stream;
    int st = launch_argmax(h, d_logits, n, d_arg, amax_partial, s);
    if (st != GGB_OK) return st;
    int32_t result = 0;
    if (temp <= 0.0f) {          // greedy: first maximum (src/cli/main.cpp:828-837)
        st = cuda_status(h, cudaMemcpyAsync(&result, d_arg, 4, cudaMemcpyDeviceToHost, s), "sample download");
    } else {
        const double u = sample_next_uniform(seed);
        st = cuda_status(h, cudaMemcpyAsync(d_temp, &temp, 4, cudaMemcpyHostToDevice, s), "sample upload");
        if (st == GGB_OK) st = cuda_status(h, cudaMemcpyAsync(d_u, &u, 8, cudaMemcpyHostToDevice, s), "sample upload");
        if (st == GGB_OK) st = sample_enqueue(h, d_logits, n, d_arg, d_temp, d_u, nullptr, base + 4096, d_out, s);
        if (st == GGB_OK) st = cuda_status(h, cudaMemcpyAsync(&result, d_out, 4, cudaMemcpyDeviceToHost, s), "sample download");
    }
    if (st == GGB_OK) st = cuda_status(h, cudaStreamSynchronize(s), "sample");
    if (st == GGB_OK) *token = result;
    return st;
}

extern "C" int ggb_sample_device(ggb_handle h, const float* d_logits, int n, float temp, uint64_t* seed, int32_t* token) {
    if (!h) return GGB_UNAVAILABLE;
    if (!d_logits || n < 1 || !seed || !token) return set_status(h, GGB_INVALID_PARAM, "sample: null pointer or empty logits");
    std::lock_guard<std::mutex> lk(h->mu);
    cudaSetDevice(h->device);
    return sample_common(h, d_logits, n, temp, seed, token);
}

extern "C" int ggb_sample(ggb_handle h, const float* host_logits, int n, float temp, uint64_t* seed, int32_t* token) {
    if (!h) return GGB_UNAVAILABLE;
    if (!host_logits || n < 1 || !seed || !token) return set_status(h, GGB_INVALID_PARAM, "sample: null pointer or empty logits");
    std::lock_guard<std::mutex> lk(h->mu);
    cudaSetDevice(h->device);
    float* d = static_cast<float*>(scratch(h, 0, sizeof(float) * static_cast<size_t>(n)));
    if (!d) return h->last_status;
    int st = cuda_status(h, cudaMemcpyAsync(d, host_logits, sizeof(float) * static_cast<size_t>(n), cudaMemcpyHostToDevice, h->stream), "sample upload");
    if (st != GGB_OK) return st;
    return sample_common(h, d, n, temp, seed, token);
}
