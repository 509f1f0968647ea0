// w8a8_linear_static_scratch: the W8A8 linear for callers that may not allocate device memory.
//
// Who that is: code that lives inside someone else's process and memory budget — a synthesis
// plugin loaded by a serving host that has handed all device memory to its own pool, or a
// real-time audio thread for which the implicit device-wide synchronisation of cudaMalloc /
// cudaFree is a glitch. Such callers cannot use w8a8_create (it allocates the context's scratch),
// so this entry point needs no context: the activation codes and scales that w8a8_linear keeps in
// the context's buffer go into an array that is part of the library image instead.
//
// Cost and limits of that choice:
//  * the array is kStaticScratchBytes (8 MiB) on EVERY GPU that loads this library, from load to
//    process exit, whether or not this entry point is ever called;
//  * a call needs  round_up(M*K, 256) + round_up(4*M*G, 256)  bytes of it and is refused with
//    W8A8_ERR_WORKSPACE (nothing launched) when that exceeds the array;
//  * there is ONE array per GPU, shared by every stream and every host thread: two calls that can
//    overlap on the GPU race on it. Serialise them (same stream, or an event between them);
//  * the array keeps the previous call's contents. Nothing in it has to start at zero: the
//    quantiser writes every code and every scale that the following kernel reads, and nothing
//    else is read;
//  * the first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current). Make that first call before starting any stream capture.
#include <mutex>

#include "w8a8_internal.h"

namespace {

constexpr size_t kStaticScratchBytes = size_t(8) << 20;
constexpr int kMaxDevices = 64;

// In host code these names are only handles for the runtime's symbol table, not addresses a kernel
// can use: the device addresses are fetched once per device below and passed to the kernels.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ __align__(256) int g_static_status[64];

struct DeviceSlots {
    unsigned char* scratch = nullptr;
    int* status = nullptr;
    bool ready = false;
};
DeviceSlots g_slots[kMaxDevices];
std::mutex g_slots_mu;

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

// Resolves the per-device addresses of the two arrays for the CURRENT device.
int static_slots(DeviceSlots** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return w8a8::fail(W8A8_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return w8a8::fail(W8A8_ERR_UNSUPPORTED, "device index %d", dev);
    std::lock_guard<std::mutex> lock(g_slots_mu);
    DeviceSlots& s = g_slots[dev];
    if (!s.ready) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess)
            return w8a8::fail(W8A8_ERR_CUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
        s.scratch = static_cast<unsigned char*>(p);
        e = cudaGetSymbolAddress(&p, g_static_status);
        if (e != cudaSuccess)
            return w8a8::fail(W8A8_ERR_CUDA, "cudaGetSymbolAddress(status): %s", cudaGetErrorString(e));
        s.status = static_cast<int*>(p);
        s.ready = true;
    }
    *out = &s;
    return W8A8_OK;
}

}  // namespace

extern "C" {

size_t w8a8_static_scratch_bytes(void) { return kStaticScratchBytes; }

int w8a8_linear_static_scratch(const void* W, const void* w_scale, int group_size, const void* act_scale,
                               const void* smooth_inv, const void* X, void* Y, int M, int N, int K,
                               const w8a8_linear_opts* opts, void* stream) {
    using namespace w8a8;
    if (M < 0 || N <= 0 || K <= 0) return fail(W8A8_ERR_INVALID_ARG, "bad shape M=%d N=%d K=%d", M, N, K);
    if (!W || !w_scale || (M > 0 && (!X || !Y))) return fail(W8A8_ERR_INVALID_ARG, "null W, w_scale, X or Y");
    int act_mode = W8A8_ACT_PER_TOKEN_GROUP, kernel = W8A8_KERNEL_AUTO;
    if (opts) {
        if (opts->epilogue < W8A8_EPI_NONE || opts->epilogue > W8A8_EPI_SWIGLU)
            return fail(W8A8_ERR_INVALID_ARG, "unknown epilogue %d", opts->epilogue);
        if (opts->epilogue == W8A8_EPI_RESIDUAL && !opts->residual)
            return fail(W8A8_ERR_INVALID_ARG, "W8A8_EPI_RESIDUAL needs opts->residual");
        if (opts->epilogue == W8A8_EPI_SWIGLU && N % 16 != 0)
            return fail(W8A8_ERR_INVALID_ARG, "W8A8_EPI_SWIGLU needs N %% 16 == 0 (got %d)", N);
        if (opts->act_mode != W8A8_ACT_PER_TOKEN_GROUP && opts->act_mode != W8A8_ACT_PER_TOKEN)
            return fail(W8A8_ERR_INVALID_ARG, "unknown act_mode %d", opts->act_mode);
        if (opts->kernel < W8A8_KERNEL_AUTO || opts->kernel > W8A8_KERNEL_GEMM_PAIR)
            return fail(W8A8_ERR_INVALID_ARG, "unknown kernel %d", opts->kernel);
        act_mode = opts->act_mode;
        kernel = opts->kernel;
    }
    if (M == 0) return W8A8_OK;
    const int G = num_groups(K, group_size);
    const size_t codes_bytes = align256(static_cast<size_t>(M) * K);
    const size_t need = codes_bytes + align256(static_cast<size_t>(M) * G * sizeof(float));
    if (need > kStaticScratchBytes)
        return fail(W8A8_ERR_WORKSPACE,
                    "M=%d K=%d group=%d needs %zu bytes of scratch; the built-in array holds %zu "
                    "(use w8a8_linear with a context for larger calls)",
                    M, K, group_size, need, kStaticScratchBytes);
    DeviceSlots* slots = nullptr;
    int rc = static_slots(&slots);
    if (rc) return rc;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int8_t* Xq = reinterpret_cast<int8_t*>(slots->scratch);
    float* Xs = reinterpret_cast<float*>(slots->scratch + codes_bytes);
    rc = launch_rowquant(static_cast<const __half*>(X), nullptr, nullptr, nullptr, 0.0f,
                         static_cast<const __half*>(smooth_inv), static_cast<const __half*>(act_scale), M, K,
                         group_size, act_mode, nullptr, Xq, Xs, s);
    if (rc) return rc;
    LinearArgs a = {};
    a.W = static_cast<const int8_t*>(W);
    a.w_scale = static_cast<const __half*>(w_scale);
    a.Xq = Xq;
    a.Xs = Xs;
    a.Y = static_cast<__half*>(Y);
    a.M = M;
    a.N = N;
    a.K = K;
    a.g = norm_group(K, group_size);
    a.G = G;
    a.epilogue = opts ? opts->epilogue : W8A8_EPI_NONE;
    a.residual = opts ? static_cast<const __half*>(opts->residual) : nullptr;
    a.dump = opts ? opts->dump_group_sums : nullptr;
    a.split_k = opts ? opts->split_k : 0;
    return dispatch_linear_q(a, kernel, slots->status, s);
}

int w8a8_static_scratch_check_status(void* stream) {
    using namespace w8a8;
    DeviceSlots* slots = nullptr;
    int rc = static_slots(&slots);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int host = 0;
    cudaError_t e = cudaMemcpyAsync(&host, slots->status, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "status read: %s", cudaGetErrorString(e));
    if (host != 0) {
        cudaMemsetAsync(slots->status, 0, sizeof(int), s);
        return fail(W8A8_ERR_TIMEOUT, "a kernel gave up a bounded wait (code %d)", host);
    }
    return W8A8_OK;
}

}  // extern "C"
