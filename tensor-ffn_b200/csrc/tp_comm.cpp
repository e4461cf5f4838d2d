// Tensor-parallel communicator: a thin layer over NCCL, opened at run time (dlopen) so that the library
// loads and every single-GPU path works on machines without NCCL, plus the exchange of peer-mapped
// "windows" (CUDA IPC handles of plain cudaMalloc allocations, one process per GPU) that this library's own
// kernels store into and poll. Only this GPU's own buffers are ever handed to NCCL.
// The reference is single-GPU and has no counterpart; the collectives sit where its single GPU adds the
// projections' outputs into the residual stream (inference/src/model/qwen.cu:413-419, 441-447).
#include "engine.h"
#include "kernels.h"
#include <chrono>
#include <dlfcn.h>
#include <mutex>
#include <thread>
#include <vector>
#include <nccl.h>

namespace tffn {

namespace {

struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi& api() {
    static NcclApi a;
    static std::once_flag once;
    std::call_once(once, [] {
        // inside a process that already loaded an NCCL (e.g. through torch) the same soname resolves to it
        for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
            a.lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (a.lib) break;
        }
        if (!a.lib) return;
        a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(a.lib, "ncclGetUniqueId");
        a.CommInitRank = (decltype(a.CommInitRank))dlsym(a.lib, "ncclCommInitRank");
        a.CommDestroy = (decltype(a.CommDestroy))dlsym(a.lib, "ncclCommDestroy");
        a.AllReduce = (decltype(a.AllReduce))dlsym(a.lib, "ncclAllReduce");
        a.AllGather = (decltype(a.AllGather))dlsym(a.lib, "ncclAllGather");
        a.GetErrorString = (decltype(a.GetErrorString))dlsym(a.lib, "ncclGetErrorString");
    });
    if (!a.lib || !a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.AllReduce || !a.AllGather || !a.GetErrorString)
        throw Error(kErrUnsupported, "tensor parallel needs NCCL (libnccl.so.2 could not be opened)");
    return a;
}

void nccl_check(ncclResult_t r, const char* what) {
    if (r == ncclSuccess) return;
    throw Error(kErrCuda, std::string("NCCL error in ") + what + ": " + api().GetErrorString(r));
}

}  // namespace

struct TpComm {
    ncclComm_t comm = nullptr;
    int rank = 0, size = 1, device = 0;
};

void tp_comm_unique_id(uint8_t id[128]) {
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    ncclUniqueId u;
    nccl_check(api().GetUniqueId(&u), "ncclGetUniqueId");
    memcpy(id, &u, 128);
}

TpComm* tp_comm_create(const uint8_t id[128], int rank, int size, int device) {
    if (size < 1 || rank < 0 || rank >= size) throw Error(kErrInvalid, "tensor-parallel rank / size out of range");
    TFFN_CUDA(cudaSetDevice(device));
    ncclUniqueId u;
    memcpy(&u, id, 128);
    TpComm* c = new TpComm();
    c->rank = rank;
    c->size = size;
    c->device = device;
    try {
        nccl_check(api().CommInitRank(&c->comm, size, u, rank), "ncclCommInitRank");
    } catch (...) {
        delete c;
        throw;
    }
    return c;
}

void tp_comm_free(TpComm* c) {
    if (!c) return;
    if (c->comm) api().CommDestroy(c->comm);
    delete c;
}
int tp_comm_size(const TpComm* c) { return c ? c->size : 1; }
int tp_comm_rank(const TpComm* c) { return c ? c->rank : 0; }

void tp_all_reduce_f32(TpComm* c, float* buf, size_t n, cudaStream_t s) {
    nccl_check(api().AllReduce(buf, buf, n, ncclFloat32, ncclSum, c->comm, s), "ncclAllReduce");
}
void tp_all_gather_bytes(TpComm* c, const void* send, void* recv, size_t bytes, cudaStream_t s) {
    nccl_check(api().AllGather(send, recv, bytes, ncclInt8, c->comm, s), "ncclAllGather");
}

// Collective: every rank passes its own window (a whole cudaMalloc allocation) and receives every rank's
// view of it (peers[rank] = local). The IPC handles travel through an all-gather on `s`.
void tp_window_open(TpComm* c, void* local, void* peers[kTpMaxRanks], cudaStream_t s) {
    if (c->size > kTpMaxRanks) throw Error(kErrUnsupported, "tensor-parallel groups of more than 8 ranks are not supported");
    cudaIpcMemHandle_t mine;
    TFFN_CUDA(cudaIpcGetMemHandle(&mine, local));
    void *d_send = nullptr, *d_recv = nullptr;
    TFFN_CUDA(cudaMalloc(&d_send, sizeof mine));
    TFFN_CUDA(cudaMalloc(&d_recv, sizeof mine * c->size));
    std::vector<cudaIpcMemHandle_t> all(c->size);
    try {
        TFFN_CUDA(cudaMemcpyAsync(d_send, &mine, sizeof mine, cudaMemcpyHostToDevice, s));
        tp_all_gather_bytes(c, d_send, d_recv, sizeof mine, s);
        TFFN_CUDA(cudaMemcpyAsync(all.data(), d_recv, sizeof mine * c->size, cudaMemcpyDeviceToHost, s));
        TFFN_CUDA(cudaStreamSynchronize(s));
    } catch (...) {
        cudaFree(d_send);
        cudaFree(d_recv);
        throw;
    }
    cudaFree(d_send);
    cudaFree(d_recv);
    for (int p = 0; p < kTpMaxRanks; ++p) peers[p] = nullptr;
    for (int p = 0; p < c->size; ++p) {
        if (p == c->rank) {
            peers[p] = local;
            continue;
        }
        cudaError_t e = cudaIpcOpenMemHandle(&peers[p], all[p], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int q = 0; q < p; ++q)
                if (q != c->rank && peers[q]) cudaIpcCloseMemHandle(peers[q]);
            throw Error(kErrCuda, std::string("tensor parallel: a peer's exchange window could not be mapped (") + cudaGetErrorString(e) +
                                      "); the ranks must be processes on one machine whose GPUs have peer access");
        }
    }
}

// Collective: unmaps the peers' windows, then waits (bounded) until every rank has done so; true = the
// caller may free its own window, false = a peer did not arrive in time and the window must be left alone.
bool tp_window_close(TpComm* c, void* peers[kTpMaxRanks], cudaStream_t s, double timeout_s) {
    for (int p = 0; p < c->size && p < kTpMaxRanks; ++p)
        if (p != c->rank && peers[p]) cudaIpcCloseMemHandle(peers[p]);
    float* token = nullptr;
    if (cudaMalloc((void**)&token, 4) != cudaSuccess) return false;
    cudaMemsetAsync(token, 0, 4, s);
    bool ok = api().AllReduce(token, token, 1, ncclFloat32, ncclSum, c->comm, s) == ncclSuccess;
    cudaEvent_t ev = nullptr;
    ok = ok && cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) == cudaSuccess && cudaEventRecord(ev, s) == cudaSuccess;
    if (ok) {
        const auto t0 = std::chrono::steady_clock::now();
        for (;;) {
            cudaError_t q = cudaEventQuery(ev);
            if (q == cudaSuccess) break;
            if (q != cudaErrorNotReady || std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s) {
                ok = false;
                break;
            }
            std::this_thread::sleep_for(std::chrono::microseconds(200));
        }
    }
    if (ev) cudaEventDestroy(ev);
    if (ok) cudaFree(token);  // still in use by the collective otherwise
    return ok;
}

}  // namespace tffn
