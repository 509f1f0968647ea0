// The reference's C++ entry points on top of the C ABI (see include/fish_kernels_shim.h).
//
// The reference keeps its scratch in a thread_local struct that grows inside the call
// (src/kernels/int8_gemm.cu:44, :97-102). The shim keeps that contract for callers that
// were written against it: one lazily created context per host thread and device, regrown
// (with a device synchronisation, as cudaFree implies in the reference too) when a call needs
// more scratch than it has. Callers that want allocation-free, capturable calls use the C ABI
// with their own context instead.
#include <stdexcept>
#include <string>

#include "../../include/fish_kernels_shim.h"
#include "../../include/w8a8.h"

namespace {

struct ThreadCtx {
    w8a8_ctx* ctx = nullptr;
    int device = -1;
    ~ThreadCtx() {
        // Deliberately not destroyed: at thread/process exit the CUDA runtime may already be gone.
    }
};
thread_local ThreadCtx t_ctx;

[[noreturn]] void raise(const char* where, int status) {
    throw std::runtime_error(std::string("w8a8 error in ") + where + ": " + w8a8_status_string(status) + ": " +
                             w8a8_last_error());
}

w8a8_ctx* context_for(size_t need_bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) raise("cudaGetDevice", W8A8_ERR_CUDA);
    if (t_ctx.ctx && (t_ctx.device != dev || w8a8_ctx_workspace_bytes(t_ctx.ctx) < need_bytes)) {
        cudaDeviceSynchronize();
        w8a8_destroy(t_ctx.ctx);
        t_ctx.ctx = nullptr;
    }
    if (!t_ctx.ctx) {
        size_t bytes = need_bytes < (size_t(1) << 20) ? (size_t(1) << 20) : need_bytes;
        int rc = w8a8_create(&t_ctx.ctx, dev, bytes);
        if (rc) raise("w8a8_create", rc);
        t_ctx.device = dev;
    }
    return t_ctx.ctx;
}

}  // namespace

namespace fish::kernels {

void int8_dequant_gemm_fp16(const int8_t* W, const __half* scale, int group_size, const __half* act_scale,
                            const __half* smooth_inv, const __half* X, __half* Y, int M, int N, int K,
                            cublasHandle_t /*cublas*/, cudaStream_t stream) {
    // Reference letters: M = weight rows, N = tokens.
    w8a8_ctx* ctx = context_for(w8a8_workspace_bytes(N, M, K, group_size));
    int rc = w8a8_linear(ctx, W, scale, group_size, act_scale, smooth_inv, X, Y, /*tokens*/ N, /*out*/ M, K,
                         nullptr, stream);
    if (rc) raise("int8_dequant_gemm_fp16", rc);
}

void rms_norm(const __half* x, const __half* weight, __half* out, int n_tokens, int dim, float eps,
              cudaStream_t stream) {
    int rc = w8a8_rms_norm(context_for(0), x, weight, out, n_tokens, dim, eps, stream);
    if (rc) raise("rms_norm", rc);
}

void silu_forward(__half* x, int n, cudaStream_t stream) {
    int rc = w8a8_silu(context_for(0), x, n, stream);
    if (rc) raise("silu_forward", rc);
}

void mul_forward(__half* a, const __half* b, int n, cudaStream_t stream) {
    int rc = w8a8_mul(context_for(0), a, b, n, stream);
    if (rc) raise("mul_forward", rc);
}

void residual_add(__half* a, const __half* b, int n, cudaStream_t stream) {
    int rc = w8a8_residual_add(context_for(0), a, b, n, stream);
    if (rc) raise("residual_add", rc);
}

}  // namespace fish::kernels

// C handles on the shim, so that tests written in Python can drive the C++ entry points
// exactly as a C++ caller would (exceptions are turned back into a status + message).
extern "C" FISH_SHIM_API int fish_shim_int8_dequant_gemm_fp16(const void* W, const void* scale, int group_size,
                                                const void* act_scale, const void* smooth_inv, const void* X,
                                                void* Y, int M, int N, int K, void* stream, char* err,
                                                int err_len) {
    try {
        fish::kernels::int8_dequant_gemm_fp16(
            static_cast<const int8_t*>(W), static_cast<const __half*>(scale), group_size,
            static_cast<const __half*>(act_scale), static_cast<const __half*>(smooth_inv),
            static_cast<const __half*>(X), static_cast<__half*>(Y), M, N, K, nullptr,
            static_cast<cudaStream_t>(stream));
        return 0;
    } catch (const std::exception& e) {
        if (err && err_len > 0) snprintf(err, err_len, "%s", e.what());
        return 1;
    }
}

namespace {
template <class F>
int shim_guard(char* err, int err_len, F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        if (err && err_len > 0) snprintf(err, err_len, "%s", e.what());
        return 1;
    }
}
}  // namespace

extern "C" FISH_SHIM_API int fish_shim_rms_norm(const void* x, const void* weight, void* out, int n_tokens, int dim,
                                                float eps, void* stream, char* err, int err_len) {
    return shim_guard(err, err_len, [&] {
        fish::kernels::rms_norm(static_cast<const __half*>(x), static_cast<const __half*>(weight),
                                static_cast<__half*>(out), n_tokens, dim, eps, static_cast<cudaStream_t>(stream));
    });
}

extern "C" FISH_SHIM_API int fish_shim_silu_forward(void* x, int n, void* stream, char* err, int err_len) {
    return shim_guard(err, err_len, [&] {
        fish::kernels::silu_forward(static_cast<__half*>(x), n, static_cast<cudaStream_t>(stream));
    });
}

extern "C" FISH_SHIM_API int fish_shim_mul_forward(void* a, const void* b, int n, void* stream, char* err,
                                                   int err_len) {
    return shim_guard(err, err_len, [&] {
        fish::kernels::mul_forward(static_cast<__half*>(a), static_cast<const __half*>(b), n,
                                   static_cast<cudaStream_t>(stream));
    });
}

extern "C" FISH_SHIM_API int fish_shim_residual_add(void* a, const void* b, int n, void* stream, char* err,
                                                    int err_len) {
    return shim_guard(err, err_len, [&] {
        fish::kernels::residual_add(static_cast<__half*>(a), static_cast<const __half*>(b), n,
                                    static_cast<cudaStream_t>(stream));
    });
}
