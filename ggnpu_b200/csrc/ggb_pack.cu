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

// Q4_K into the row-group-major layout (layout 1 of ggb_formats.cuh).  `raw` holds `rows` GGUF rows
// starting at the first row of group `g0`; groups g0 .. g0+groups-1 are written; rows past the end
// of the matrix become zero blocks (d = dmin = 0 decodes to 0).
__global__ void repack_q4k_rg16_kernel(const uint8_t* __restrict__ raw, int64_t rows, int nb, int64_t groups,
                                       uint8_t* __restrict__ hdr, uint8_t* __restrict__ qs) {
    const int64_t n_hdr = groups * nb * 16 * 4;          // 32-bit words of the header stream
    const int64_t n_qs = groups * nb * 4 * 32 * 4;       // 32-bit words of the quant stream
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n_hdr + n_qs;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        int64_t row; int b, src_byte; uint8_t* dst;
        if (i < n_hdr) {
            const int word = static_cast<int>(i & 3);
            const int64_t e = i >> 2;                     // (group * nb + b) * 16 + r
            const int r = static_cast<int>(e & 15);
            const int64_t gb = e >> 4;
            b = static_cast<int>(gb % nb); row = (gb / nb) * 16 + r;
            src_byte = word * 4; dst = hdr + i * 4;
        } else {
            const int64_t k = i - n_hdr;
            const int word = static_cast<int>(k & 3), lane = static_cast<int>((k >> 2) & 31), j = static_cast<int>((k >> 7) & 3);
            const int64_t gb = k >> 9;
            b = static_cast<int>(gb % nb); row = (gb / nb) * 16 + (lane >> 2) + 8 * (word & 1);
            src_byte = 16 + 32 * j + 16 * (word >> 1) + 4 * (lane & 3); dst = qs + k * 4;
        }
        uchar4 v = make_uchar4(0, 0, 0, 0);
        if (row < rows) {
            const uint8_t* sp = raw + (row * nb + b) * 144 + src_byte;
            v = make_uchar4(sp[0], sp[1], sp[2], sp[3]);
        }
        *reinterpret_cast<uchar4*>(dst) = v;
    }
}

// Q6_K into its row-group-major layout (ggb_formats.cuh).  Same contract as the Q4_K kernel.
__global__ void repack_q6k_rg16_kernel(const uint8_t* __restrict__ raw, int64_t rows, int nb, int64_t groups,
                                       uint8_t* __restrict__ s0, uint8_t* __restrict__ s1, uint8_t* __restrict__ s2, uint8_t* __restrict__ s3) {
    const int64_t gbs = groups * nb;
    const int64_t n0 = gbs * 512, n1 = gbs * 256, n2 = gbs * 64, n3 = gbs * 16;   // 32-bit words (s3: 16-bit)
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n0 + n1 + n2 + n3;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        int64_t gb, row; int src_byte, nbytes = 4; uint8_t* dst;
        if (i < n0) {
            const int word = static_cast<int>(i & 3), lane = static_cast<int>((i >> 2) & 31), combo = static_cast<int>((i >> 7) & 3);
            gb = i >> 9;
            row = (lane >> 2) + 8 * (word >> 1);
            src_byte = 64 * (combo >> 1) + 32 * (word & 1) + 16 * (combo & 1) + 4 * (lane & 3); dst = s0 + i * 4;
        } else if (i < n0 + n1) {
            const int64_t k = i - n0;
            const int word = static_cast<int>(k & 3), lane = static_cast<int>((k >> 2) & 31), hf = static_cast<int>((k >> 7) & 1);
            gb = k >> 8;
            row = (lane >> 2) + 8 * (word & 1);
            src_byte = 128 + 32 * hf + 16 * (word >> 1) + 4 * (lane & 3); dst = s1 + k * 4;
        } else if (i < n0 + n1 + n2) {
            const int64_t k = i - n0 - n1;
            gb = k >> 6; row = (k >> 2) & 15; src_byte = 192 + 4 * static_cast<int>(k & 3); dst = s2 + k * 4;
        } else {
            const int64_t k = i - n0 - n1 - n2;
            gb = k >> 4; row = k & 15; src_byte = 208; nbytes = 2; dst = s3 + k * 2;
        }
        const int b = static_cast<int>(gb % nb);
        row += (gb / nb) * 16;
        const bool ok = row < rows;
        const uint8_t* sp = raw + (row * nb + b) * 210 + src_byte;
        for (int q = 0; q < nbytes; ++q) dst[q] = ok ? sp[q] : 0;
    }
}

// Q4_K / Q6_K in the row-group-major layouts: stage whole row groups, permute on the device.
static int upload_rg16(Context* c, uint32_t type, int64_t N, int K, const void* host_rows, DeviceWeight** out) {
    const int nb = K / 256;
    const int64_t groups = (N + 15) / 16;
    const bool q4 = type == T_Q4_K;
    // bytes of each stream per (group, block)
    const int per_gb[4] = {q4 ? 256 : 2048, q4 ? 2048 : 1024, q4 ? 0 : 256, q4 ? 0 : 32};
    const int block_bytes = q4 ? 144 : 210;
    DeviceWeight* dw = new DeviceWeight();
    size_t off[4], acc = 0;
    for (int i = 0; i < 4; ++i) { off[i] = acc; acc += align_up(static_cast<size_t>(groups) * nb * per_gb[i], 256); }
    dw->bytes = acc;
    cudaError_t e = cudaMalloc(&dw->base, dw->bytes);
    if (e != cudaSuccess) { delete dw; return cuda_status(c, e, "cudaMalloc(weight)"); }
    uint8_t* p = static_cast<uint8_t*>(dw->base);
    dw->w.N = N; dw->w.K = K; dw->w.nb = nb; dw->w.type = type; dw->w.layout = 1;
    for (int i = 0; i < 4; ++i) dw->w.s[i] = per_gb[i] ? p + off[i] : nullptr;
    const size_t row_bytes = static_cast<size_t>(nb) * block_bytes;
    const int64_t chunk_groups = std::max<int64_t>(1, static_cast<int64_t>((size_t(256) << 20) / (16 * row_bytes)));
    void* staging = nullptr;
    e = cudaMalloc(&staging, static_cast<size_t>(std::min(groups, chunk_groups)) * 16 * row_bytes);
    if (e != cudaSuccess) { free_weight(dw); return cuda_status(c, e, "cudaMalloc(staging)"); }
    for (int64_t g0 = 0; g0 < groups && e == cudaSuccess; g0 += chunk_groups) {
        const int64_t ng = std::min(chunk_groups, groups - g0);
        const int64_t rows = std::min<int64_t>(ng * 16, N - g0 * 16);
        e = cudaMemcpyAsync(staging, static_cast<const uint8_t*>(host_rows) + static_cast<size_t>(g0) * 16 * row_bytes,
                            static_cast<size_t>(rows) * row_bytes, cudaMemcpyHostToDevice, c->stream);
        if (e != cudaSuccess) break;
        const int64_t items = ng * nb * (q4 ? (16 * 4 + 4 * 32 * 4) : (512 + 256 + 64 + 16));
        const int grid = static_cast<int>(std::min<int64_t>((items + 255) / 256, 148 * 16));
        uint8_t* d[4];
        for (int i = 0; i < 4; ++i) d[i] = p + off[i] + static_cast<size_t>(g0) * nb * per_gb[i];
        if (q4) repack_q4k_rg16_kernel<<<grid, 256, 0, c->stream>>>(static_cast<const uint8_t*>(staging), rows, nb, ng, d[0], d[1]);
        else repack_q6k_rg16_kernel<<<grid, 256, 0, c->stream>>>(static_cast<const uint8_t*>(staging), rows, nb, ng, d[0], d[1], d[2], d[3]);
        c->launches++;
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    }
    cudaFree(staging);
    if (e != cudaSuccess) { free_weight(dw); return cuda_status(c, e, "weight pack (row groups)"); }
    *out = dw;
    return GGB_OK;
}

int upload_weight(Context* c, uint32_t type, int64_t N, int K, const void* host_rows, DeviceWeight** out) {
    const FormatInfo f = format_info(type);
    if (!f.block_elems) return set_status(c, GGB_INVALID_PARAM, "unsupported weight type");
    if (!host_rows || N <= 0 || K <= 0 || K % f.block_elems) return set_status(c, GGB_INVALID_PARAM, "bad weight shape");
    if ((type == T_Q4_K || type == T_Q6_K) && c->use_mma) return upload_rg16(c, type, N, K, host_rows, out);
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

int concat_weight_rows(Context* c, const DeviceWeight* a, const DeviceWeight* b, DeviceWeight** out) {
    if (!a || !b || a->w.layout != 1 || b->w.layout != 1 || a->w.type != b->w.type || a->w.K != b->w.K || a->w.N % 16 ||
        (a->w.type != T_Q4_K && a->w.type != T_Q6_K))
        return set_status(c, GGB_INVALID_PARAM, "concat_weight_rows: both weights must be Q4_K or Q6_K in the row-group-major layout with the same K");
    const bool q4 = a->w.type == T_Q4_K;
    const int per_gb[4] = {q4 ? 256 : 2048, q4 ? 2048 : 1024, q4 ? 0 : 256, q4 ? 0 : 32};
    const int nb = a->w.nb;
    const int64_t ga = a->w.N / 16, gb = (b->w.N + 15) / 16;
    DeviceWeight* dw = new DeviceWeight();
    size_t off[4], acc = 0;
    for (int i = 0; i < 4; ++i) { off[i] = acc; acc += align_up(static_cast<size_t>(ga + gb) * nb * per_gb[i], 256); }
    dw->bytes = acc;
    cudaError_t e = cudaMalloc(&dw->base, dw->bytes);
    if (e != cudaSuccess) { delete dw; return cuda_status(c, e, "cudaMalloc(weight)"); }
    uint8_t* p = static_cast<uint8_t*>(dw->base);
    dw->w = a->w;
    dw->w.N = a->w.N + b->w.N;
    for (int i = 0; i < 4 && e == cudaSuccess; ++i) {
        dw->w.s[i] = per_gb[i] ? p + off[i] : nullptr;
        if (!per_gb[i]) continue;
        const size_t na = static_cast<size_t>(ga) * nb * per_gb[i], nbb = static_cast<size_t>(gb) * nb * per_gb[i];
        e = cudaMemcpyAsync(p + off[i], a->w.s[i], na, cudaMemcpyDeviceToDevice, c->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(p + off[i] + na, b->w.s[i], nbb, cudaMemcpyDeviceToDevice, c->stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) { free_weight(dw); return cuda_status(c, e, "concat_weight_rows"); }
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
