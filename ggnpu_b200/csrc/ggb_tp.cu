// Tensor-parallel group of a handle: one process per GPU, NCCL over NVLink / NVSwitch.
// Net-new relative to the reference, which has no multi-device path (one process, one device selected
// by --npu-device, src/cli/main.cpp:573-626).  The collectives run on the handle's stream, so they are
// ordered with the kernels around them and are captured into the decode CUDA graph with them.
//
// NCCL is bound at run time (dlopen of libnccl.so.2 -- in a process that already loaded PyTorch this
// resolves to the copy PyTorch brought), so the library has no link-time dependency on it and
// single-GPU users never touch it.
#include <dlfcn.h>
#include <string.h>

#include "ggb_internal.h"

namespace ggb {

namespace {

struct NcclId { char bytes[128]; };
typedef int (*fn_get_unique_id)(NcclId*);
typedef int (*fn_comm_init_rank)(void**, int, NcclId, int);
typedef int (*fn_comm_destroy)(void*);
typedef int (*fn_all_reduce)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*fn_all_gather)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef const char* (*fn_error_string)(int);

struct Nccl {
    void* lib = nullptr;
    fn_get_unique_id get_unique_id = nullptr;
    fn_comm_init_rank comm_init_rank = nullptr;
    fn_comm_destroy comm_destroy = nullptr;
    fn_all_reduce all_reduce = nullptr;
    fn_all_gather all_gather = nullptr;
    fn_error_string error_string = nullptr;
};

constexpr int kNcclFloat32 = 7, kNcclSum = 0;      // ncclFloat32, ncclSum in nccl.h

Nccl* nccl() {
    static Nccl n;
    static std::once_flag once;
    std::call_once(once, [] {
        for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
            n.lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (n.lib) break;
        }
        if (!n.lib) return;
        n.get_unique_id = reinterpret_cast<fn_get_unique_id>(dlsym(n.lib, "ncclGetUniqueId"));
        n.comm_init_rank = reinterpret_cast<fn_comm_init_rank>(dlsym(n.lib, "ncclCommInitRank"));
        n.comm_destroy = reinterpret_cast<fn_comm_destroy>(dlsym(n.lib, "ncclCommDestroy"));
        n.all_reduce = reinterpret_cast<fn_all_reduce>(dlsym(n.lib, "ncclAllReduce"));
        n.all_gather = reinterpret_cast<fn_all_gather>(dlsym(n.lib, "ncclAllGather"));
        n.error_string = reinterpret_cast<fn_error_string>(dlsym(n.lib, "ncclGetErrorString"));
        if (!n.get_unique_id || !n.comm_init_rank || !n.comm_destroy || !n.all_reduce || !n.all_gather) { dlclose(n.lib); n.lib = nullptr; }
    });
    return n.lib ? &n : nullptr;
}

int nccl_status(Context* c, int rc, const char* what) {
    if (rc == 0) return GGB_OK;
    Nccl* n = nccl();
    std::string msg = std::string(what) + ": NCCL error " + std::to_string(rc);
    if (n && n->error_string) msg += std::string(" (") + n->error_string(rc) + ")";
    return set_status(c, GGB_ERROR, msg.c_str());
}

}  // namespace

int tp_all_reduce(Context* c, float* d_buf, size_t count, cudaStream_t s) {
    if (c->tp_size <= 1) return GGB_OK;
    Nccl* n = nccl();
    if (!n || !c->tp_comm) return set_status(c, GGB_UNAVAILABLE, "tensor parallel group not initialised");
    c->launches++;
    return nccl_status(c, n->all_reduce(d_buf, d_buf, count, kNcclFloat32, kNcclSum, c->tp_comm, s), "all-reduce");
}

// recv holds tp_size consecutive pieces of `count` floats; this rank's piece is already at recv + rank * count
int tp_all_gather_in_place(Context* c, float* d_recv, size_t count, cudaStream_t s) {
    if (c->tp_size <= 1) return GGB_OK;
    Nccl* n = nccl();
    if (!n || !c->tp_comm) return set_status(c, GGB_UNAVAILABLE, "tensor parallel group not initialised");
    c->launches++;
    return nccl_status(c, n->all_gather(d_recv + static_cast<size_t>(c->tp_rank) * count, d_recv, count, kNcclFloat32, c->tp_comm, s), "all-gather");
}

void tp_destroy(Context* c) {
    Nccl* n = nccl();
    if (n && c->tp_comm) n->comm_destroy(c->tp_comm);
    c->tp_comm = nullptr; c->tp_size = 1; c->tp_rank = 0;
}

}  // namespace ggb

using namespace ggb;

extern "C" int ggb_tp_unique_id(void* id128) {
    Nccl* n = nccl();
    if (!n || !id128) return GGB_UNAVAILABLE;
    NcclId id;
    if (n->get_unique_id(&id) != 0) return GGB_ERROR;
    memcpy(id128, id.bytes, sizeof(id.bytes));
    return GGB_OK;
}

extern "C" int ggb_tp_init(ggb_handle h, const void* id128, int rank, int size) {
    if (!h) return GGB_UNAVAILABLE;
    if (!id128 || size < 1 || rank < 0 || rank >= size) return set_status(h, GGB_INVALID_PARAM, "tp_init: bad rank / size");
    std::lock_guard<std::mutex> lk(h->mu);
    cudaSetDevice(h->device);
    if (h->tp_comm) return set_status(h, GGB_INVALID_PARAM, "tp_init: the handle already belongs to a group");
    if (size == 1) { h->tp_rank = 0; h->tp_size = 1; return GGB_OK; }
    Nccl* n = nccl();
    if (!n) return set_status(h, GGB_UNAVAILABLE, "tp_init: libnccl.so.2 could not be loaded");
    NcclId id;
    memcpy(id.bytes, id128, sizeof(id.bytes));
    void* comm = nullptr;
    const int rc = n->comm_init_rank(&comm, size, id, rank);
    if (rc != 0) return nccl_status(h, rc, "tp_init");
    h->tp_comm = comm; h->tp_rank = rank; h->tp_size = size;
    return GGB_OK;
}

extern "C" int ggb_tp_all_reduce_device(ggb_handle h, float* d_buf, int64_t count) {
    if (!h) return GGB_UNAVAILABLE;
    if (!d_buf || count <= 0) return set_status(h, GGB_INVALID_PARAM, "tp_all_reduce: bad arguments");
    std::lock_guard<std::mutex> lk(h->mu);
    cudaSetDevice(h->device);
    return tp_all_reduce(h, d_buf, static_cast<size_t>(count), h->stream);
}
