// Tensor-parallel group of a handle: one process per GPU, NCCL over NVLink / NVSwitch.
// Net-new relative to the reference, which has no multi-device path (one process, one device selected
// by --npu-device, src/cli/main.cpp:573-626).  The collectives run on the handle's stream, so they are
// ordered with the kernels around them and are captured into the decode CUDA graph with them.
//
// NCCL is bound at run time (dlopen of libnccl.so.2 -- in a process that already loaded PyTorch this
// resolves to the copy PyTorch brought), so the library has no link-time dependency on it and
// single-GPU users never touch it.
#include <dlfcn.h>
#include <stdlib.h>
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

// ---- one-shot all-reduce over peer memory (small messages: the 16 KB partial rows of a decode step) ----
// Every rank owns a region {buf[2][ranks][kCap] floats, flag[2][ranks][kMaxBlocks], counter[kMaxBlocks]}
// that its peers map through CUDA IPC.  A call = one kernel of count / 1024 CTAs per rank: CTA b copies
// its 1024-float slice of the local partial row into slot (parity, my rank) of every peer's buf with
// plain NVLink stores, fences system-wide, then raises flag (parity, my rank, b) = epoch in every peer;
// it then waits for the size - 1 flags its peers raise in ITS region and adds the slices in rank order
// (the same order on every rank, so all ranks end with bit-identical sums).  Epochs come from a counter
// in device memory (replay-safe under CUDA graphs); consecutive calls alternate between the two halves
// of buf, which is enough because a rank cannot finish call e before every peer has sent for call e,
// i.e. has finished reading call e - 1.  The wait is bounded by a %globaltimer deadline; on expiry the
// kernel records an error and returns (no trap, the context stays usable).
constexpr int kCap = 16384;            // floats per slot (64 KB)
constexpr int kMaxBlocks = kCap / 1024;
constexpr int kMaxRanks = 8;
constexpr unsigned long long kWaitNs = 4000000000ull;     // 4 s: a peer's kernel may start late, never this late (GGB_TP_WAIT_MS overrides)

struct PeerRegion {                    // device layout of one rank's region
    float buf[2][kMaxRanks][kCap];
    unsigned flag[2][kMaxRanks][kMaxBlocks];
    unsigned counter[kMaxBlocks];
};

struct OneShotArgs {
    float* x;
    int count, rank, size;
    PeerRegion* region[kMaxRanks];     // region[rank] is this rank's own
    int* err;
    unsigned long long wait_ns;        // how long to wait for a peer's flag before giving up
};

__global__ void __launch_bounds__(256) tp_oneshot_allreduce_kernel(const OneShotArgs a) {
    __shared__ unsigned epoch_s;
    __shared__ int failed;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    PeerRegion* mine = a.region[a.rank];
    const int b = blockIdx.x, i = (b * 256 + threadIdx.x) * 4;
    // after a recorded failure (a peer that never came) later calls do not wait again
    if (threadIdx.x == 0) { epoch_s = ++mine->counter[b]; failed = *reinterpret_cast<volatile int*>(a.err) != 0; }
    __syncthreads();
    if (failed) return;
    const unsigned epoch = epoch_s;
    const int par = epoch & 1;
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (i < a.count) {
        v = *reinterpret_cast<const float4*>(a.x + i);
        for (int q = 0; q < a.size; ++q)
            if (q != a.rank) *reinterpret_cast<float4*>(&a.region[q]->buf[par][a.rank][i]) = v;      // NVLink store into the peer's region
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < a.size && threadIdx.x != a.rank) {
        // raise my flag in peer threadIdx.x, then wait for that peer's flag in my region
        volatile unsigned* theirs = &a.region[threadIdx.x]->flag[par][a.rank][b];
        *theirs = epoch;
        volatile unsigned* f = &mine->flag[par][threadIdx.x][b];
        unsigned long long t0, t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        while (static_cast<int>(*f - epoch) < 0) {
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t - t0 > a.wait_ns) { failed = 1; atomicExch(a.err, 5); break; }
        }
    }
    __threadfence_system();
    __syncthreads();
    if (i < a.count && !failed) {
        float4 s = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int q = 0; q < a.size; ++q) {
            const float4 p = q == a.rank ? v : __ldcv(reinterpret_cast<const float4*>(&mine->buf[par][q][i]));
            s.x += p.x; s.y += p.y; s.z += p.z; s.w += p.w;
        }
        *reinterpret_cast<float4*>(a.x + i) = s;
    }
}

int tp_all_reduce(Context* c, float* d_buf, size_t count, cudaStream_t s) {
    if (c->tp_size <= 1) return GGB_OK;
    // measured (16 KB, launch included): 2 ranks NCCL 10 us / one-shot 19 us; 4 ranks 17 / 15; 8 ranks 26 / 16
    static const bool force_one_shot = getenv("GGB_TP_ONE_SHOT") != nullptr;
    if (c->tp_peers_attached && (c->tp_size >= 4 || force_one_shot) && count <= static_cast<size_t>(kCap) && count % 4 == 0 &&
        !(reinterpret_cast<uintptr_t>(d_buf) & 15)) {
        OneShotArgs a{};
        a.x = d_buf; a.count = static_cast<int>(count); a.rank = c->tp_rank; a.size = c->tp_size; a.err = c->d_err;
        a.wait_ns = kWaitNs;
        if (const char* w = getenv("GGB_TP_WAIT_MS")) { const long ms = atol(w); if (ms > 0 && ms <= 60000) a.wait_ns = static_cast<unsigned long long>(ms) * 1000000ull; }
        for (int q = 0; q < c->tp_size; ++q) a.region[q] = static_cast<PeerRegion*>(c->tp_region[q]);
        const cudaError_t e = launch_pdl(c, tp_oneshot_allreduce_kernel, dim3(static_cast<unsigned>((count + 1023) / 1024)), dim3(256), 0, s, a);
        c->launches++;
        return cuda_status(c, e, "one-shot all-reduce");
    }
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
    for (int q = 0; q < 8; ++q) {
        if (!c->tp_region[q]) continue;
        if (q == c->tp_rank) cudaFree(c->tp_region[q]); else cudaIpcCloseMemHandle(c->tp_region[q]);
        c->tp_region[q] = nullptr;
    }
    c->tp_peers_attached = false;
    // NCCL is only touched by handles that joined a group (no dlopen from a destructor otherwise)
    if (c->tp_comm) { Nccl* n = nccl(); if (n) n->comm_destroy(c->tp_comm); }
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

extern "C" int ggb_tp_ipc_handle(ggb_handle h, void* handle64) {
    if (!h) return GGB_UNAVAILABLE;
    if (!handle64) return set_status(h, GGB_INVALID_PARAM, "tp_ipc_handle: null pointer");
    std::lock_guard<std::mutex> lk(h->mu);
    cudaSetDevice(h->device);
    if (h->tp_size < 2 || h->tp_size > kMaxRanks) return set_status(h, GGB_INVALID_PARAM, "tp_ipc_handle: needs a group of 2..8 ranks (call ggb_tp_init first)");
    void*& mine = h->tp_region[h->tp_rank];
    if (!mine) {
        if (cuda_status(h, cudaMalloc(&mine, sizeof(PeerRegion)), "cudaMalloc(peer region)") != GGB_OK) return h->last_status;
        if (cuda_status(h, cudaMemset(mine, 0, sizeof(PeerRegion)), "memset(peer region)") != GGB_OK) return h->last_status;
    }
    cudaIpcMemHandle_t ipc;
    static_assert(sizeof(ipc) == 64, "CUDA IPC handles are 64 bytes");
    if (cuda_status(h, cudaIpcGetMemHandle(&ipc, mine), "cudaIpcGetMemHandle") != GGB_OK) return h->last_status;
    memcpy(handle64, &ipc, 64);
    return GGB_OK;
}

extern "C" int ggb_tp_attach_peers(ggb_handle h, const void* handles) {
    if (!h) return GGB_UNAVAILABLE;
    if (!handles) return set_status(h, GGB_INVALID_PARAM, "tp_attach_peers: null pointer");
    std::lock_guard<std::mutex> lk(h->mu);
    cudaSetDevice(h->device);
    if (h->tp_size < 2 || h->tp_size > kMaxRanks || !h->tp_region[h->tp_rank])
        return set_status(h, GGB_INVALID_PARAM, "tp_attach_peers: call ggb_tp_init and ggb_tp_ipc_handle first");
    if (getenv("GGB_TP_NCCL_ONLY")) return GGB_OK;
    for (int q = 0; q < h->tp_size; ++q) {
        if (q == h->tp_rank || h->tp_region[q]) continue;
        cudaIpcMemHandle_t ipc;
        memcpy(&ipc, static_cast<const char*>(handles) + 64 * q, 64);
        if (cuda_status(h, cudaIpcOpenMemHandle(&h->tp_region[q], ipc, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle") != GGB_OK)
            return h->last_status;
    }
    h->tp_peers_attached = true;
    return GGB_OK;
}

extern "C" int ggb_tp_all_reduce_device(ggb_handle h, float* d_buf, int64_t count) {
    if (!h) return GGB_UNAVAILABLE;
    if (!d_buf || count <= 0) return set_status(h, GGB_INVALID_PARAM, "tp_all_reduce: bad arguments");
    std::lock_guard<std::mutex> lk(h->mu);
    cudaSetDevice(h->device);
    return tp_all_reduce(h, d_buf, static_cast<size_t>(count), h->stream);
}
