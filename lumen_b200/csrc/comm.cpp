// The data-parallel communicator behind the C ABI: NCCL over NVLink 5 / NVSwitch, one communicator per process group,
// set up through the keyed store (store.cpp). The counterpart of lumen/distributed/nccl.rs:103-213 (library loaded at
// run time, unique id from the group's first rank, ncclCommInitRank), :387-410 (all_reduce) and :279-307 (device_wait).
//
// libnccl.so.2 is opened at the first lb_comm_create, not at load time: a single-GPU process needs no NCCL at all.
// Hosts that cannot lose a rank silently get deadlines everywhere on the host side: the store barrier before
// ncclCommInitRank (a rank that never arrives -> LB_ERR_TIMEOUT on the others), lb_comm_barrier, and
// lb_comm_synchronize, which waits for a stream with a deadline while polling ncclCommGetAsyncError and aborts the
// communicator instead of waiting forever.
#include <dlfcn.h>
#include <nccl.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <mutex>
#include <thread>

#include "device.h"

struct lb_store;
extern "C" {
int lb_store_set(lb_store* s, const char* key, const void* value, size_t n);
int lb_store_get(lb_store* s, const char* key, void* out, size_t capacity, size_t* n, int timeout_ms);
int lb_store_add(lb_store* s, const char* key, int64_t amount, int64_t* result);
int lb_store_wait(lb_store* s, const char* const* keys, int n_keys, int timeout_ms);
}

namespace lb {
namespace {

struct Nccl {
    void* handle = nullptr;
    ncclResult_t (*GetVersion)(int*) = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    int version = 0;
};

const Nccl& nccl() {
    static Nccl lib;
    static std::mutex mutex;
    std::lock_guard<std::mutex> lock(mutex);
    if (lib.handle) return lib;
    // a copy some other library of the process already loaded is reused (same soname); otherwise the system's
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) fail(LB_ERR_UNSUPPORTED, format("cannot load libnccl.so.2 (%s): collectives across GPUs need NCCL", dlerror()));
    auto sym = [&](const char* name) {
        void* p = dlsym(h, name);
        if (!p) fail(LB_ERR_UNSUPPORTED, format("libnccl.so.2 lacks %s", name));
        return p;
    };
    lib.GetVersion = (decltype(lib.GetVersion))sym("ncclGetVersion");
    lib.GetUniqueId = (decltype(lib.GetUniqueId))sym("ncclGetUniqueId");
    lib.CommInitRank = (decltype(lib.CommInitRank))sym("ncclCommInitRank");
    lib.CommDestroy = (decltype(lib.CommDestroy))sym("ncclCommDestroy");
    lib.CommAbort = (decltype(lib.CommAbort))sym("ncclCommAbort");
    lib.CommGetAsyncError = (decltype(lib.CommGetAsyncError))sym("ncclCommGetAsyncError");
    lib.AllReduce = (decltype(lib.AllReduce))sym("ncclAllReduce");
    lib.Broadcast = (decltype(lib.Broadcast))sym("ncclBroadcast");
    lib.GetErrorString = (decltype(lib.GetErrorString))sym("ncclGetErrorString");
    lib.GetVersion(&lib.version);
    lib.handle = h;
    return lib;
}

void check_nccl(ncclResult_t r, const char* what) {
    if (r == ncclSuccess) return;
    fail(LB_ERR_CUDA, format("%s: %s (ncclResult %d)", what, nccl().GetErrorString(r), (int)r));
}

ncclDataType_t nccl_dtype(int dtype) {
    switch (dtype) {
        case LB_I8: return ncclInt8;
        case LB_U8: case LB_BOOL: return ncclUint8;
        case LB_I32: return ncclInt32;
        case LB_U32: return ncclUint32;
        case LB_I64: return ncclInt64;
        case LB_U64: return ncclUint64;
        case LB_F16: return ncclFloat16;
        case LB_BF16: return ncclBfloat16;
        case LB_F32: return ncclFloat32;
        case LB_F64: return ncclFloat64;
    }
    fail(LB_ERR_UNSUPPORTED, format("collectives: no NCCL type for %s", dtype_name(dtype)));
}

}  // namespace
}  // namespace lb

struct lb_comm {
    ncclComm_t comm = nullptr;
    lb_store* store = nullptr;  // borrowed: must outlive the communicator
    int rank = 0, world = 1, device = 0, index = 0;
    int64_t barriers = 0;
    bool aborted = false;
};

namespace lb {
// queues an in-place or out-of-place all-reduce on `stream` (used by the plan's collective steps)
void comm_all_reduce(lb_comm* c, const void* send, void* recv, size_t count, int dtype, int op, void* stream) {
    if (!c || !c->comm || c->aborted) fail(LB_ERR_INVALID, "all_reduce: the communicator is gone (destroyed or aborted)");
    if (op < 0 || op > 3) fail(LB_ERR_INVALID, "all_reduce: op is 0 sum, 1 prod, 2 max or 3 min");
    if (count == 0) return;
    check_nccl(nccl().AllReduce(send, recv, count, nccl_dtype(dtype), (ncclRedOp_t)op, c->comm, (cudaStream_t)stream), "ncclAllReduce");
}
int comm_world(const lb_comm* c) { return c ? c->world : 1; }
}  // namespace lb

extern "C" {

const char* lb_nccl_version(void) {
    static char text[64];
    int rc = lb::guarded([&] {
        int v = lb::nccl().version;
        snprintf(text, sizeof(text), "%d.%d.%d", v / 10000, (v / 100) % 100, v % 100);
    });
    return rc == LB_OK ? text : "";
}

int lb_comm_barrier(lb_comm* c, int timeout_ms);

int lb_comm_create(lb_store* store, int rank, int world, int timeout_ms, lb_comm** out) {
    return lb::guarded([&] {
        if (!store || !out || world < 1 || rank < 0 || rank >= world) lb::fail(LB_ERR_INVALID, "lb_comm_create: a store, 0 <= rank < world, an out pointer");
        static std::atomic<int> created{0};  // every rank creates its communicators in the same order
        auto c = std::make_unique<lb_comm>();
        c->store = store, c->rank = rank, c->world = world, c->index = created++;
        lb::device_info();
        LB_CUDA(cudaGetDevice(&c->device));
        const lb::Nccl& n = lb::nccl();
        const std::string key = "nccl/" + std::to_string(c->index) + "/id";
        ncclUniqueId id;
        if (rank == 0) {
            lb::check_nccl(n.GetUniqueId(&id), "ncclGetUniqueId");
            if (lb_store_set(store, key.c_str(), &id, sizeof(id)) != LB_OK) lb::fail(LB_ERR_TIMEOUT, lb_last_error());
        } else {
            size_t got = 0;
            int rc = lb_store_get(store, key.c_str(), &id, sizeof(id), &got, timeout_ms);
            if (rc != LB_OK) lb::fail(rc, std::string("lb_comm_create: rank 0 never published the NCCL id: ") + lb_last_error());
            if (got != sizeof(id)) lb::fail(LB_ERR_INVALID, "lb_comm_create: malformed NCCL id in the store");
        }
        // every rank must be here and alive before the blocking ncclCommInitRank: a missing rank times out on the host
        int rc = lb_comm_barrier(c.get(), timeout_ms);
        if (rc != LB_OK) lb::fail(rc, std::string("lb_comm_create: not every rank arrived: ") + lb_last_error());
        lb::check_nccl(n.CommInitRank(&c->comm, world, id, rank), "ncclCommInitRank");
        *out = c.release();
    });
}

int lb_comm_rank(const lb_comm* c) { return c ? c->rank : -1; }
int lb_comm_size(const lb_comm* c) { return c ? c->world : -1; }

int lb_comm_all_reduce(lb_comm* c, const void* send, void* recv, size_t count, int dtype, int op, void* stream) {
    return lb::guarded([&] { lb::comm_all_reduce(c, send, recv, count, dtype, op, stream); });
}

int lb_comm_broadcast(lb_comm* c, void* buffer, size_t count, int dtype, int root, void* stream) {
    return lb::guarded([&] {
        if (!c || !c->comm || c->aborted) lb::fail(LB_ERR_INVALID, "broadcast: the communicator is gone (destroyed or aborted)");
        if (root < 0 || root >= c->world) lb::fail(LB_ERR_INVALID, "broadcast: root out of range");
        if (count == 0) return;
        lb::check_nccl(lb::nccl().Broadcast(buffer, buffer, count, lb::nccl_dtype(dtype), root, c->comm, (cudaStream_t)stream), "ncclBroadcast");
    });
}

// Host barrier through the store: every rank adds one to the round's counter and waits for the round's flag, which
// the last arrival sets. A rank that never arrives makes the others return LB_ERR_TIMEOUT after `timeout_ms`.
int lb_comm_barrier(lb_comm* c, int timeout_ms) {
    return lb::guarded([&] {
        if (!c || !c->store) lb::fail(LB_ERR_INVALID, "lb_comm_barrier: null communicator");
        const std::string round = "barrier/" + std::to_string(c->index) + "/" + std::to_string(c->barriers++);
        int64_t arrived = 0;
        if (lb_store_add(c->store, (round + "/count").c_str(), 1, &arrived) != LB_OK) lb::fail(LB_ERR_TIMEOUT, lb_last_error());
        const std::string flag = round + "/done";
        if (arrived == c->world && lb_store_set(c->store, flag.c_str(), "1", 1) != LB_OK) lb::fail(LB_ERR_TIMEOUT, lb_last_error());
        const char* keys[1] = {flag.c_str()};
        int rc = lb_store_wait(c->store, keys, 1, timeout_ms);
        if (rc != LB_OK) lb::fail(rc, lb::format("barrier: %lld of %d ranks arrived: %s", (long long)arrived, c->world, lb_last_error()));
    });
}

// The communicator's asynchronous error state: LB_OK, or LB_ERR_CUDA with NCCL's message (a peer that died, a
// network fault). Does not block.
int lb_comm_check(lb_comm* c) {
    return lb::guarded([&] {
        if (!c || !c->comm) lb::fail(LB_ERR_INVALID, "lb_comm_check: null communicator");
        if (c->aborted) lb::fail(LB_ERR_CUDA, "the communicator was aborted");
        ncclResult_t state = ncclSuccess;
        lb::check_nccl(lb::nccl().CommGetAsyncError(c->comm, &state), "ncclCommGetAsyncError");
        if (state != ncclSuccess && state != ncclInProgress) lb::check_nccl(state, "NCCL asynchronous error");
    });
}

// Waits until everything queued on `stream` has finished, for at most `timeout_ms`, polling the communicator's error
// state meanwhile. On an NCCL error or at the deadline the communicator is ABORTED (its kernels are told to quit) and
// the call returns LB_ERR_CUDA / LB_ERR_TIMEOUT: the host gets control back instead of waiting on a dead peer.
int lb_comm_synchronize(lb_comm* c, void* stream, int timeout_ms) {
    return lb::guarded([&] {
        if (!c || !c->comm) lb::fail(LB_ERR_INVALID, "lb_comm_synchronize: null communicator");
        auto until = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms > 0 ? timeout_ms : 30000);
        for (;;) {
            cudaError_t q = cudaStreamQuery((cudaStream_t)stream);
            if (q == cudaSuccess) return;
            if (q != cudaErrorNotReady) LB_CUDA(q);
            ncclResult_t state = ncclSuccess;
            ncclResult_t rc = lb::nccl().CommGetAsyncError(c->comm, &state);
            const bool failed = rc != ncclSuccess || (state != ncclSuccess && state != ncclInProgress);
            const bool late = std::chrono::steady_clock::now() >= until;
            if (failed || late) {
                lb::nccl().CommAbort(c->comm);
                c->aborted = true, c->comm = nullptr;
                if (failed) lb::fail(LB_ERR_CUDA, lb::format("NCCL reported an asynchronous error (%s); the communicator was aborted",
                                                             lb::nccl().GetErrorString(rc != ncclSuccess ? rc : state)));
                lb::fail(LB_ERR_TIMEOUT, lb::format("the stream did not finish within %d ms; the communicator was aborted", timeout_ms));
            }
            std::this_thread::sleep_for(std::chrono::microseconds(200));
        }
    });
}

int lb_comm_abort(lb_comm* c) {
    return lb::guarded([&] {
        if (!c) lb::fail(LB_ERR_INVALID, "lb_comm_abort: null communicator");
        if (c->comm) lb::nccl().CommAbort(c->comm);
        c->comm = nullptr, c->aborted = true;
    });
}

void lb_comm_destroy(lb_comm* c) {
    if (!c) return;
    if (c->comm) lb::nccl().CommDestroy(c->comm);
    delete c;
}
}
