// Pack GGUF rows into the HBM stream layout, and decode packed rows back to fp32.
#include "ggb_internal.h"

namespace ggb {

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t packed_bytes(uint32_t type, int64_t N, int K) {
    const FormatInfo f = format_info(type);
    if (!f.block_elems) return 0;
    const size_t blocks = static_cast<size_t>(N) * (K / f.block_elems);
    size_t total = 0;
    for (int i = 0; i < f.n_streams; ++i) total += align_up(blocks * f.size[i], 256);
    return total;
}

// One thread per 16 bytes of the destination stream where possible would need
// 16-byte aligned sources; GGUF blocks are not (18, 34, 210 ... bytes), so the
// permutation runs byte-wise.  It executes once per weight at load time.
__global__ void repack_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ dst, int64_t blocks,
                              int block_bytes, int off, int size) {
    const int64_t total = blocks * size;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t b = i / size;
        const int j = static_cast<int>(i - b * size);
        dst[i] = raw[b * block_bytes + off + j];
    }
}

int upload_weight(Context* c, uint32_t type, int64_t N, int K, const void* host_rows, DeviceWeight** out) {
    const FormatInfo f = format_info(type);
    if (!f.block_elems) return set_status(c, GGB_INVALID_PARAM, "unsupported weight type");
    if (!host_rows || N <= 0 || K <= 0 || K % f.block_elems) return set_status(c, GGB_INVALID_PARAM, "bad weight shape");
    const int nb = K / f.block_elems;
    const size_t blocks = static_cast<size_t>(N) * nb;
    const size_t raw_bytes = blocks * f.block_bytes;
    DeviceWeight* dw = new DeviceWeight();
    dw->bytes = packed_bytes(type, N, K);
    cudaError_t e = cudaMalloc(&dw->base, dw->bytes);
    if (e != cudaSuccess) { delete dw; return cuda_status(c, e, "cudaMalloc(weight)"); }
    dw->w.N = N; dw->w.K = K; dw->w.nb = nb; dw->w.type = type;
    uint8_t* p = static_cast<uint8_t*>(dw->base);
    for (int i = 0; i < kMaxStreams; ++i) dw->w.s[i] = nullptr;
    if (f.n_streams == 1) {
        dw->w.s[0] = p;
        e = cudaMemcpyAsync(p, host_rows, raw_bytes, cudaMemcpyHostToDevice, c->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
        if (e != cudaSuccess) { free_weight(dw); return cuda_status(c, e, "weight upload"); }
        *out = dw;
        return GGB_OK;
    }
    // stage the raw bytes in chunks of whole blocks, permute on the device
    const size_t chunk_blocks = std::max<size_t>(1, (size_t(256) << 20) / f.block_bytes);
    void* staging = nullptr;
    e = cudaMalloc(&staging, std::min(blocks, chunk_blocks) * f.block_bytes);
    if (e != cudaSuccess) { free_weight(dw); return cuda_status(c, e, "cudaMalloc(staging)"); }
    size_t stream_off[kMaxStreams];
    size_t acc = 0;
    for (int i = 0; i < f.n_streams; ++i) { stream_off[i] = acc; dw->w.s[i] = p + acc; acc += align_up(blocks * f.size[i], 256); }
    for (size_t b0 = 0; b0 < blocks && e == cudaSuccess; b0 += chunk_blocks) {
        const size_t nblk = std::min(chunk_blocks, blocks - b0);
        e = cudaMemcpyAsync(staging, static_cast<const uint8_t*>(host_rows) + b0 * f.block_bytes, nblk * f.block_bytes,
                            cudaMemcpyHostToDevice, c->stream);
        for (int i = 0; i < f.n_streams && e == cudaSuccess; ++i) {
            const int64_t total = static_cast<int64_t>(nblk) * f.size[i];
            const int grid = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 16));
            repack_kernel<<<grid, 256, 0, c->stream>>>(static_cast<const uint8_t*>(staging), p + stream_off[i] + b0 * f.size[i],
                                                        static_cast<int64_t>(nblk), f.block_bytes, f.off[i], f.size[i]);
            c->launches++;
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    }
    cudaFree(staging);
    if (e != cudaSuccess) { free_weight(dw); return cuda_status(c, e, "weight pack"); }
    *out = dw;
    return GGB_OK;
}

void free_weight(DeviceWeight* w) {
    if (!w) return;
    if (w->base) cudaFree(w->base);
    delete w;
}

// fp32 rows out of the packed layout: the GPU form of dequant_tensor_row
// (src/cli/main.cpp:36-261).  One thread per output element.
__global__ void dequant_rows_kernel(PackedW w, int64_t row0, int64_t n_rows, int block_elems, float* __restrict__ out) {
    const int64_t total = n_rows * w.K;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / w.K;
        const int k = static_cast<int>(i - r * w.K);
        const int64_t blk = (row0 + r) * w.nb + k / block_elems;
        out[i] = decode_elem(w, blk, k % block_elems);
    }
}

int launch_dequant_rows(Context* c, const PackedW& w, int64_t row0, int64_t n_rows, float* d_out, cudaStream_t s) {
    const FormatInfo f = format_info(w.type);
    const int64_t total = n_rows * w.K;
    if (total <= 0) return GGB_OK;
    const int grid = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 32));
    dequant_rows_kernel<<<grid, 256, 0, s>>>(w, row0, n_rows, f.block_elems, d_out);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "dequant_rows");
}

// Embedding lookup (src/cli/main.cpp:2367-2375): row ids live in device memory
// so the decode graph can feed the sampled token straight back in.
__global__ void gather_rows_kernel(PackedW w, const int32_t* __restrict__ rows, int n_rows, int block_elems, float* __restrict__ out, int ld) {
    const int r = blockIdx.y;
    if (r >= n_rows) return;
    int64_t row = rows[r];
    if (row < 0 || row >= w.N) row = 0;
    for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < w.K; k += gridDim.x * blockDim.x)
        out[static_cast<size_t>(r) * ld + k] = decode_elem(w, row * w.nb + k / block_elems, k % block_elems);
}

int launch_gather_rows(Context* c, const PackedW& w, const int32_t* d_rows, int n_rows, float* d_out, int ld, cudaStream_t s) {
    const FormatInfo f = format_info(w.type);
    if (n_rows <= 0) return GGB_OK;
    dim3 grid((w.K + 255) / 256, n_rows);
    gather_rows_kernel<<<grid, 256, 0, s>>>(w, d_rows, n_rows, f.block_elems, d_out, ld);
    c->launches++;
    return cuda_status(c, cudaGetLastError(), "gather_rows");
}

}  // namespace ggb
