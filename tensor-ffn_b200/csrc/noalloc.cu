// tffn_op_swiglu_bs1_noalloc — the fused batch-1 SwiGLU kernel for callers that must not allocate.
//
// Who needs this: code that runs where device allocation is forbidden or impossible — a host
// thread in the middle of a latency-critical loop that may not take the allocator's lock or
// trigger an implicit device synchronisation (cudaMalloc and cudaFree can do both), a plugin
// loaded into a process whose memory pool is owned and fully reserved by someone else, or a
// caller running under a strict memory budget fixed at start-up. Such callers hand in device
// pointers for inputs and outputs that they obtained earlier; the kernel's scratch (the fixed-point
// accumulator that collects every CTA's share of the FFN output, and the status word) lives in a
// fixed array inside this library's device image instead of a buffer from cudaMalloc.
//
// Consequences the caller has to know:
//  * Every GPU that loads the library holds the array (about 33 KB) until the process exits.
//  * The size is fixed: hidden <= 2048 (a multiple of 64); larger requests are refused.
//  * All calls on one device share the array and it keeps the previous call's contents. The sums
//    must start at zero: the entry point clears them and the status word before every launch. Two
//    calls whose kernels overlap on the GPU (different streams, or different host threads) would add
//    into the same sums: serialise them.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and
//    opts the kernel into its shared-memory size.
//  * The call blocks until `cuda_stream` has finished it (it synchronises that stream only, never
//    the device), so it cannot be part of a stream capture.
//  * The caller's pointers go to the kernel as they are; bulk copies and 16-byte vector loads
//    need them 16-byte aligned, which is checked here because a misaligned access would fault.
//  * The calling thread's current device is restored before return.
#include "../../include/tffn.h"
#include "engine.h"
#include <mutex>

namespace tffn {
void set_last_error(const std::string& msg);  // c_api.cpp
}

namespace {

constexpr int kMaxHidden = 2048;
constexpr int kMaxAccWords = 2 * kMaxHidden;  // >= bs1_acc_words(kMaxHidden), checked at set-up
constexpr int kMaxDevices = 64;

struct Scratch {
    long long acc[kMaxAccWords];  // fixed-point sums of the FFN output, zero before each launch
    int status;                   // device status word of the launch
    int pad[63];
};

// In host code this name is only a handle for the runtime; the address the kernel needs comes
// from cudaGetSymbolAddress on the device that will run it.
static __device__ __align__(256) unsigned char g_scratch[sizeof(Scratch)];

std::mutex g_mu;
Scratch* g_dev_ptr[kMaxDevices] = {nullptr};
int g_dev_sms[kMaxDevices] = {0};

int fail(int code, const std::string& msg) {
    tffn::set_last_error(msg);
    return code;
}

}  // namespace

extern "C" int tffn_op_swiglu_bs1_noalloc(int device, void* h_io, const void* norm_w, const void* packed_base,
                                          const void* packed_expert, float expert_scale, float eps, int H, int I,
                                          void* cuda_stream) {
    using namespace tffn;
    if (!h_io || !norm_w || !packed_base || I < 1) return fail(TFFN_ERR_INVALID, "NULL pointer or empty intermediate size");
    if (H < 64 || H % 64 != 0 || H > kMaxHidden)
        return fail(TFFN_ERR_CAPACITY, "tffn_op_swiglu_bs1_noalloc: hidden must be a multiple of 64 and at most " +
                                           std::to_string(kMaxHidden) + " (the built-in scratch is sized for that)");
    if (device < 0 || device >= kMaxDevices) return fail(TFFN_ERR_INVALID, "device index out of range");
    for (const void* ptr : {(const void*)h_io, norm_w, packed_base, packed_expert})
        if (((uintptr_t)ptr & 15u) != 0)
            return fail(TFFN_ERR_INVALID, "tffn_op_swiglu_bs1_noalloc: every device pointer must be 16-byte aligned");
    int prev_device = -1;
    cudaError_t e = cudaGetDevice(&prev_device);
    if (e != cudaSuccess) return fail(TFFN_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    struct RestoreDevice {
        int d;
        ~RestoreDevice() { cudaSetDevice(d); }
    } restore{prev_device};
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail(TFFN_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
    Scratch* scratch = nullptr;
    int sms = 0;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_dev_ptr[device]) {  // set-up, once per device, with that device current
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_scratch);
            if (e != cudaSuccess) return fail(TFFN_ERR_CUDA, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
            int n = 0;
            e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
            if (e != cudaSuccess) return fail(TFFN_ERR_CUDA, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
            if (bs1_acc_words(kMaxHidden) > (size_t)kMaxAccWords)
                return fail(TFFN_ERR_CAPACITY, "tffn_op_swiglu_bs1_noalloc: built-in scratch smaller than the kernel's accumulator");
            const int rc = bs1_prepare(kMaxHidden, true);
            if (rc != 0) return fail(TFFN_ERR_CUDA, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString((cudaError_t)rc));
            g_dev_sms[device] = n;
            g_dev_ptr[device] = (Scratch*)p;
        }
        scratch = g_dev_ptr[device];
        sms = g_dev_sms[device];
    }
    {
        const int rc = bs1_prepare(H, true);  // shared-memory opt-in for this hidden size (no allocation)
        if (rc != 0) return fail(TFFN_ERR_CUDA, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString((cudaError_t)rc));
    }
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    // the array keeps the last call's contents: the sums and the status word must start at zero
    e = cudaMemsetAsync(scratch, 0, sizeof(scratch->acc) + sizeof(int), stream);
    if (e != cudaSuccess) return fail(TFFN_ERR_CUDA, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
    Bs1Ctx x;
    memset(&x, 0, sizeof x);
    x.H = H;
    x.I = I;
    x.eps = eps;
    x.expert_scale = expert_scale;
    x.h = (bf16*)h_io;
    x.acc_out = scratch->acc;
    x.status = &scratch->status;
    x.num_sms = sms;
    Bs1Layer ly;
    memset(&ly, 0, sizeof ly);
    ly.ffn_norm = (const bf16*)norm_w;
    ly.ffn_base = (const bf16*)packed_base;
    ly.ffn_expert = (const bf16*)packed_expert;
    launch_bs1_ffn(x, ly, stream, false);
    launch_bs1_ffn_finalize(x.h, x.acc_out, H, stream);  // h_io = bf16(h_io + sums)
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(TFFN_ERR_CUDA, std::string("kernel launch: ") + cudaGetErrorString(e));
    // status read-back on the caller's stream: a plain cudaMemcpy would run on the legacy default
    // stream and synchronise with every blocking stream of the process
    int st = 0;
    e = cudaMemcpyAsync(&st, &scratch->status, sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return fail(TFFN_ERR_CUDA, std::string("cudaMemcpyAsync: ") + cudaGetErrorString(e));
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail(TFFN_ERR_CUDA, std::string("cudaStreamSynchronize: ") + cudaGetErrorString(e));
    if (st != 0) return fail(TFFN_ERR_DEVICE, "FFN kernel reported device status " + std::to_string(st));
    return TFFN_OK;
}
