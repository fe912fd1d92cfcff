// hk_ring.cpp -- the ring hop issued from native code (see include/hk_ring.h).
//
// NCCL is resolved with dlopen at the first call, so the library itself has no link-time dependency on it.
#include "../../include/hk_ring.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <chrono>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>

namespace {

// the handful of NCCL declarations used here (stable since NCCL 2.x)
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[HK_RING_UNIQUE_ID_BYTES]; } ncclUniqueId;
typedef int ncclResult_t;  // ncclSuccess = 0, ncclInProgress = 7
constexpr int kNcclInt8 = 0;  // ncclInt8 / ncclChar

struct Nccl {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*CommAbort)(ncclComm_t);
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    ncclResult_t (*Send)(const void*, size_t, int, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void*, size_t, int, int, ncclComm_t, cudaStream_t);
    const char* (*GetErrorString)(ncclResult_t);
    bool ok = false;
};

Nccl g_nccl;
std::once_flag g_once;
thread_local std::string g_last;

void load_nccl() {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
    auto sym = [&](const char* n) { return dlsym(h, n); };
    g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(sym("ncclGetUniqueId"));
    g_nccl.CommInitRank = reinterpret_cast<decltype(g_nccl.CommInitRank)>(sym("ncclCommInitRank"));
    g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(sym("ncclCommDestroy"));
    g_nccl.CommAbort = reinterpret_cast<decltype(g_nccl.CommAbort)>(sym("ncclCommAbort"));
    g_nccl.CommGetAsyncError = reinterpret_cast<decltype(g_nccl.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    g_nccl.GroupStart = reinterpret_cast<decltype(g_nccl.GroupStart)>(sym("ncclGroupStart"));
    g_nccl.GroupEnd = reinterpret_cast<decltype(g_nccl.GroupEnd)>(sym("ncclGroupEnd"));
    g_nccl.Send = reinterpret_cast<decltype(g_nccl.Send)>(sym("ncclSend"));
    g_nccl.Recv = reinterpret_cast<decltype(g_nccl.Recv)>(sym("ncclRecv"));
    g_nccl.GetErrorString = reinterpret_cast<decltype(g_nccl.GetErrorString)>(sym("ncclGetErrorString"));
    g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.CommDestroy && g_nccl.CommAbort &&
                g_nccl.CommGetAsyncError && g_nccl.GroupStart && g_nccl.GroupEnd && g_nccl.Send && g_nccl.Recv &&
                g_nccl.GetErrorString;
}

bool have_nccl() {
    std::call_once(g_once, load_nccl);
    return g_nccl.ok;
}

int nccl_fail(ncclResult_t r) {
    g_last = g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "NCCL error";
    return HK_RING_ERR_NCCL;
}

}  // namespace

struct hk_ring {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 0, device = 0;
    cudaEvent_t ready = nullptr;                // compute stream -> communication stream
    cudaEvent_t done[HK_RING_SLOTS] = {};       // communication stream -> compute stream / host, one per hop in flight
    bool aborted = false;
};

extern "C" {

int hk_ring_get_unique_id(void* id) {
    if (!id) return HK_RING_ERR_ARG;
    if (!have_nccl()) return HK_RING_ERR_NO_NCCL;
    ncclUniqueId u;
    const ncclResult_t r = g_nccl.GetUniqueId(&u);
    if (r != 0) return nccl_fail(r);
    std::memcpy(id, &u, sizeof(u));
    return HK_RING_OK;
}

int hk_ring_create(hk_ring_t** out, const void* id, int rank, int world) {
    if (!out || !id || world <= 0 || rank < 0 || rank >= world) return HK_RING_ERR_ARG;
    *out = nullptr;
    if (!have_nccl()) return HK_RING_ERR_NO_NCCL;
    hk_ring* r = new hk_ring;
    r->rank = rank;
    r->world = world;
    bool ev_ok = cudaGetDevice(&r->device) == cudaSuccess &&
                 cudaEventCreateWithFlags(&r->ready, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; ev_ok && i < HK_RING_SLOTS; ++i)
        ev_ok = cudaEventCreateWithFlags(&r->done[i], cudaEventDisableTiming) == cudaSuccess;
    auto drop_events = [&] {
        if (r->ready) cudaEventDestroy(r->ready);
        for (int i = 0; i < HK_RING_SLOTS; ++i)
            if (r->done[i]) cudaEventDestroy(r->done[i]);
    };
    if (!ev_ok) {
        cudaGetLastError();
        drop_events();
        delete r;
        return HK_RING_ERR_CUDA;
    }
    ncclUniqueId u;
    std::memcpy(&u, id, sizeof(u));
    const ncclResult_t rc = g_nccl.CommInitRank(&r->comm, world, u, rank);
    if (rc != 0) {
        drop_events();
        delete r;
        return nccl_fail(rc);
    }
    *out = r;
    return HK_RING_OK;
}

int hk_ring_exchange(hk_ring_t* r, int slot, const void* send, int send_peer, void* recv, int recv_peer, size_t bytes,
                     void* compute_stream, void* comm_stream) {
    if (!r || r->aborted || slot < 0 || slot >= HK_RING_SLOTS || !send || !recv || send_peer < 0 || send_peer >= r->world || recv_peer < 0 ||
        recv_peer >= r->world)
        return HK_RING_ERR_ARG;
    cudaStream_t cs = static_cast<cudaStream_t>(compute_stream), ms = static_cast<cudaStream_t>(comm_stream);
    if (cudaEventRecord(r->ready, cs) != cudaSuccess || cudaStreamWaitEvent(ms, r->ready, 0) != cudaSuccess)
        return HK_RING_ERR_CUDA;
    ncclResult_t rc = g_nccl.GroupStart();
    if (rc == 0) rc = g_nccl.Send(send, bytes, kNcclInt8, send_peer, r->comm, ms);
    if (rc == 0) rc = g_nccl.Recv(recv, bytes, kNcclInt8, recv_peer, r->comm, ms);
    const ncclResult_t re = g_nccl.GroupEnd();
    if (rc == 0) rc = re;
    if (rc != 0) return nccl_fail(rc);
    if (cudaEventRecord(r->done[slot], ms) != cudaSuccess) return HK_RING_ERR_CUDA;
    return HK_RING_OK;
}

int hk_ring_join(hk_ring_t* r, int slot, void* compute_stream) {
    if (!r || slot < 0 || slot >= HK_RING_SLOTS) return HK_RING_ERR_ARG;
    return cudaStreamWaitEvent(static_cast<cudaStream_t>(compute_stream), r->done[slot], 0) == cudaSuccess
               ? HK_RING_OK
               : HK_RING_ERR_CUDA;
}

int hk_ring_poll(hk_ring_t* r) {
    if (!r || !r->comm) return HK_RING_ERR_ARG;
    ncclResult_t async = 0;
    const ncclResult_t rc = g_nccl.CommGetAsyncError(r->comm, &async);
    if (rc != 0) return nccl_fail(rc);
    if (async != 0 && async != 7 /* ncclInProgress */) {
        nccl_fail(async);
        return HK_RING_ERR_ASYNC;
    }
    return HK_RING_OK;
}

int hk_ring_wait(hk_ring_t* r, int slot, double timeout_s) {
    if (!r || r->aborted || slot < 0 || slot >= HK_RING_SLOTS) return HK_RING_ERR_ARG;
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        const cudaError_t q = cudaEventQuery(r->done[slot]);
        if (q == cudaSuccess) return HK_RING_OK;
        int st = HK_RING_OK;
        if (q != cudaErrorNotReady) {
            cudaGetLastError();
            st = HK_RING_ERR_CUDA;
        } else if ((st = hk_ring_poll(r)) == HK_RING_OK &&
                   std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s) {
            st = HK_RING_ERR_TIMEOUT;
        }
        if (st != HK_RING_OK) {
            // the hop will never complete: take the communicator down so that its kernel leaves the stream
            if (st != HK_RING_ERR_CUDA) {
                g_nccl.CommAbort(r->comm);
                r->comm = nullptr;
                r->aborted = true;
            }
            return st;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

int hk_ring_destroy(hk_ring_t* r) {
    if (!r) return HK_RING_ERR_ARG;
    int st = HK_RING_OK;
    if (r->comm) {
        const ncclResult_t rc = g_nccl.CommDestroy(r->comm);
        if (rc != 0) st = nccl_fail(rc);
    }
    if (r->ready) cudaEventDestroy(r->ready);
    for (int i = 0; i < HK_RING_SLOTS; ++i)
        if (r->done[i]) cudaEventDestroy(r->done[i]);
    delete r;
    return st;
}

int hk_ring_abort(hk_ring_t* r) {
    if (!r) return HK_RING_ERR_ARG;
    if (r->comm) {
        g_nccl.CommAbort(r->comm);
        r->comm = nullptr;
    }
    return hk_ring_destroy(r);
}

const char* hk_ring_error_string(int status) {
    switch (status) {
        case HK_RING_OK: return "ok";
        case HK_RING_ERR_NO_NCCL: return "libnccl.so.2 could not be loaded";
        case HK_RING_ERR_NCCL: return "an NCCL call failed";
        case HK_RING_ERR_CUDA: return "a CUDA runtime call failed";
        case HK_RING_ERR_ARG: return "bad argument";
        case HK_RING_ERR_TIMEOUT: return "the hop did not complete in time";
        case HK_RING_ERR_ASYNC: return "NCCL reported an asynchronous error";
        default: return "unknown status";
    }
}

const char* hk_ring_last_nccl_error(void) { return g_last.c_str(); }

}  // extern "C"
