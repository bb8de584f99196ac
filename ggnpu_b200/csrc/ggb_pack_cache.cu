// Packed-weight disk cache: the role the reference's WeightCache + CompileCache play for its NPU backend
// (include/ggnpu/weight_cache.h:34-158: decode once, keep in memory, persist on disk; src/cache/cache.cpp:16-58: one file
// per key under the cache directory).  There the persisted object is the int8 decode of a tensor; here it is the tensor
// in this library's HBM layout (the byte permutation ggb_pack.cu makes), so a later process uploads the file as it is and
// skips the repack kernels.
//
// Key, as WeightCache::make_key builds it (weight_cache.h:141-152): a layout-version prefix, a hash of
// model_id + 0x1f + tensor name (model_id = the caller's fingerprint of the model file, e.g. "<path>:<file size>",
// src/cli/main.cpp:1203-1210, so that two models with the same tensor names never collide), the type and the data size.
// A file also records a fingerprint of the source bytes: a stale entry (same key, other contents) is a miss.
#include <errno.h>
#include <stdio.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "ggb_internal.h"

namespace ggb {

namespace {

constexpr char kMagic[8] = {'G', 'G', 'B', '2', '0', '0', 'P', 'K'};
constexpr uint32_t kVersion = 1;            // bump when a packed layout changes: old files then miss

struct PackHeader {
    char magic[8];
    uint32_t version, type;
    int64_t N;
    int32_t K, nb, layout, n_streams;
    uint64_t stream_off[kMaxStreams];       // offset of each stream inside the blob; UINT64_MAX: absent
    uint64_t bytes;                         // blob size
    uint64_t src_fingerprint;               // of the GGUF bytes the blob was packed from
};

uint64_t fnv1a(const void* data, size_t n, uint64_t h = 1469598103934665603ull) {
    const uint8_t* b = static_cast<const uint8_t*>(data);
    for (size_t i = 0; i < n; ++i) { h ^= b[i]; h *= 1099511628211ull; }
    return h;
}

// FNV-1a over 64 evenly spaced 64-byte samples (the whole buffer when it is small) and the length
uint64_t source_fingerprint(const void* data, size_t bytes) {
    const uint8_t* b = static_cast<const uint8_t*>(data);
    uint64_t h = fnv1a(&bytes, sizeof(bytes));
    if (bytes <= 64 * 64) return fnv1a(b, bytes, h);
    const size_t stride = (bytes - 64) / 63;
    for (int i = 0; i < 64; ++i) h = fnv1a(b + static_cast<size_t>(i) * stride, 64, h);
    return h;
}

}  // namespace

std::string pack_cache_key(const char* model_id, const char* tensor_name, uint32_t type, uint64_t data_size) {
    const std::string id = std::string(model_id ? model_id : "") + "\x1f" + (tensor_name ? tensor_name : "");
    char buf[96];
    snprintf(buf, sizeof(buf), "p%u_%016llx_t%u_%llu", kVersion, static_cast<unsigned long long>(fnv1a(id.data(), id.size())), type,
             static_cast<unsigned long long>(data_size));
    return buf;
}

// 0 on success.  Written to a temporary name and renamed, so a reader never sees half a file.
int pack_file_write(const char* path, uint32_t type, int64_t N, int K, int nb, int layout, const uint64_t* stream_off, uint64_t src_fingerprint,
                    const void* blob, uint64_t bytes) {
    PackHeader h{};
    memcpy(h.magic, kMagic, 8);
    h.version = kVersion; h.type = type; h.N = N; h.K = K; h.nb = nb; h.layout = layout; h.n_streams = kMaxStreams;
    for (int i = 0; i < kMaxStreams; ++i) h.stream_off[i] = stream_off[i];
    h.bytes = bytes; h.src_fingerprint = src_fingerprint;
    const std::string tmp = std::string(path) + ".tmp." + std::to_string(static_cast<long>(getpid()));
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) return errno ? errno : -1;
    const bool ok = fwrite(&h, sizeof(h), 1, f) == 1 && (bytes == 0 || fwrite(blob, 1, bytes, f) == bytes);
    const bool closed = fclose(f) == 0;
    if (!ok || !closed || rename(tmp.c_str(), path) != 0) { remove(tmp.c_str()); return -1; }
    return 0;
}

// 0: header and blob read and consistent with (type, N, K) and, when src_fingerprint != 0, with the source bytes;
// 1: no such file; -1: a file that does not match (stale, truncated, other version).
int pack_file_read(const char* path, uint32_t type, int64_t N, int K, uint64_t src_fingerprint, int* nb, int* layout, uint64_t* stream_off,
                   std::vector<uint8_t>* blob) {
    FILE* f = fopen(path, "rb");
    if (!f) return 1;
    PackHeader h{};
    int rc = -1;
    if (fread(&h, sizeof(h), 1, f) == 1 && memcmp(h.magic, kMagic, 8) == 0 && h.version == kVersion && h.type == type && h.N == N && h.K == K &&
        h.n_streams == kMaxStreams && (src_fingerprint == 0 || h.src_fingerprint == src_fingerprint) && h.bytes < (uint64_t(1) << 40)) {
        bool sane = true;
        for (int i = 0; i < kMaxStreams; ++i) sane = sane && (h.stream_off[i] == UINT64_MAX || h.stream_off[i] < std::max<uint64_t>(h.bytes, 1));
        if (sane) {
            blob->resize(h.bytes);
            if (h.bytes == 0 || fread(blob->data(), 1, h.bytes, f) == h.bytes) {
                // nothing may follow the blob
                uint8_t extra;
                if (fread(&extra, 1, 1, f) == 0) {
                    *nb = h.nb; *layout = h.layout;
                    for (int i = 0; i < kMaxStreams; ++i) stream_off[i] = h.stream_off[i];
                    rc = 0;
                }
            }
        }
    }
    fclose(f);
    return rc;
}

// Upload through the cache directory.  hit (optional): 1 when the packed file was used, 0 when the tensor was packed and
// the file written.  host_rows == nullptr: load from the cache only (GGB_NOT_FOUND on a miss).
int upload_weight_cached(Context* c, const char* cache_dir, const char* model_id, const char* tensor_name, uint32_t type, int64_t N, int K,
                         const void* host_rows, DeviceWeight** out, int* hit) {
    const FormatInfo fi = format_info(type);
    if (!fi.block_elems || N <= 0 || K <= 0 || K % fi.block_elems) return set_status(c, GGB_INVALID_PARAM, "bad weight shape");
    if (!cache_dir || !*cache_dir) return set_status(c, GGB_INVALID_PARAM, "weight cache: no directory");
    const uint64_t data_size = static_cast<uint64_t>(N) * (K / fi.block_elems) * fi.block_bytes;
    mkdir(cache_dir, 0755);
    const std::string path = std::string(cache_dir) + "/" + pack_cache_key(model_id, tensor_name, type, data_size) + ".ggbpack";
    const uint64_t fp = host_rows ? source_fingerprint(host_rows, data_size) : 0;
    if (hit) *hit = 0;
    std::vector<uint8_t> blob;
    int nb = 0, layout = 0;
    uint64_t off[kMaxStreams];
    const int rc = pack_file_read(path.c_str(), type, N, K, fp, &nb, &layout, off, &blob);
    // a file packed for the other Q4_K / Q6_K layout (library run with the tensor-core GEMV switched off, or on) is a miss
    const int want_layout = ((type == T_Q4_K || type == T_Q6_K) && c->use_mma) ? 1 : 0;
    if (rc == 0 && layout == want_layout) {
        DeviceWeight* dw = new DeviceWeight();
        dw->bytes = blob.size();
        cudaError_t e = cudaMalloc(&dw->base, std::max<size_t>(dw->bytes, 1));
        if (e != cudaSuccess) { delete dw; return cuda_status(c, e, "cudaMalloc(weight)"); }
        e = cudaMemcpyAsync(dw->base, blob.data(), dw->bytes, cudaMemcpyHostToDevice, c->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
        if (e != cudaSuccess) { free_weight(dw); return cuda_status(c, e, "weight upload (packed file)"); }
        dw->w.N = N; dw->w.K = K; dw->w.nb = nb; dw->w.type = type; dw->w.layout = layout;
        for (int i = 0; i < kMaxStreams; ++i) dw->w.s[i] = off[i] == UINT64_MAX ? nullptr : static_cast<uint8_t*>(dw->base) + off[i];
        dw->fingerprint = fp;
        *out = dw;
        if (hit) *hit = 1;
        return GGB_OK;
    }
    if (!host_rows) return set_status(c, GGB_NOT_FOUND, "weight cache: no packed file for this tensor");
    DeviceWeight* dw = nullptr;
    const int st = upload_weight(c, type, N, K, host_rows, &dw);
    if (st != GGB_OK) return st;
    dw->fingerprint = fp;
    // persist: the packed bytes come back once; a failed write only costs the next process the repack
    blob.resize(dw->bytes);
    if (cudaMemcpy(blob.data(), dw->base, dw->bytes, cudaMemcpyDeviceToHost) == cudaSuccess) {
        for (int i = 0; i < kMaxStreams; ++i)
            off[i] = dw->w.s[i] ? static_cast<uint64_t>(dw->w.s[i] - static_cast<const uint8_t*>(dw->base)) : UINT64_MAX;
        pack_file_write(path.c_str(), type, N, K, dw->w.nb, dw->w.layout, off, fp, blob.data(), dw->bytes);
    } else cudaGetLastError();
    *out = dw;
    return GGB_OK;
}

}  // namespace ggb

using namespace ggb;

extern "C" {

int ggb_pack_cache_key(const char* model_id, const char* tensor_name, uint32_t type, uint64_t data_size, char* out, int cap) {
    if (!out || cap <= 0) return GGB_INVALID_PARAM;
    const std::string k = pack_cache_key(model_id, tensor_name, type, data_size);
    if (static_cast<int>(k.size()) + 1 > cap) return GGB_INVALID_PARAM;
    memcpy(out, k.c_str(), k.size() + 1);
    return GGB_OK;
}

int ggb_pack_file_write(const char* path, uint32_t type, int64_t N, int K, int nb, int layout, const uint64_t* stream_off, uint64_t src_fingerprint,
                        const void* blob, uint64_t bytes) {
    if (!path || !stream_off || (!blob && bytes)) return GGB_INVALID_PARAM;
    return pack_file_write(path, type, N, K, nb, layout, stream_off, src_fingerprint, blob, bytes) == 0 ? GGB_OK : GGB_ERROR;
}

int ggb_pack_file_read(const char* path, uint32_t type, int64_t N, int K, uint64_t src_fingerprint, int* nb, int* layout, uint64_t* stream_off,
                       void* blob, uint64_t cap, uint64_t* bytes) {
    if (!path || !nb || !layout || !stream_off || !bytes) return GGB_INVALID_PARAM;
    std::vector<uint8_t> v;
    const int rc = pack_file_read(path, type, N, K, src_fingerprint, nb, layout, stream_off, &v);
    if (rc == 1) return GGB_NOT_FOUND;
    if (rc != 0) return GGB_ERROR;
    *bytes = v.size();
    if (blob) {
        if (cap < v.size()) return GGB_INVALID_PARAM;
        memcpy(blob, v.data(), v.size());
    }
    return GGB_OK;
}

int ggb_weight_upload_cached(ggb_handle h, const char* cache_dir, const char* model_id, const char* tensor_name, uint32_t type, int64_t N, int K,
                             const void* host_rows, ggb_weight* out, int* hit) {
    if (!h) return GGB_UNAVAILABLE;
    if (!out) return set_status(h, GGB_INVALID_PARAM, "weight_upload_cached: null out");
    std::lock_guard<std::mutex> lk(h->mu);
    cudaSetDevice(h->device);
    DeviceWeight* dw = nullptr;
    const int st = upload_weight_cached(h, cache_dir, model_id, tensor_name, type, N, K, host_rows, &dw, hit);
    if (st != GGB_OK) return st;
    *out = static_cast<ggb_weight>(dw);
    return GGB_OK;
}

}  // extern "C"
