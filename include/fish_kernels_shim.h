// fish_kernels_shim.h — the reference's own C++ signatures, served by libw8a8.
//
// A fish-audio-cpp build that links libw8a8 instead of compiling its
// src/kernels/{int8_gemm,rms_norm}.cu and the silu/mul/residual_add part of
// ffn_activations.cu gets these five functions with unchanged names, argument
// order and error behaviour (std::runtime_error on failure, as CUDA_CHECK in
// src/utils/cuda_utils.h:9-16 throws). Nothing at the call sites
// (src/engine/dual_ar_engine.cc:327-342, :580-647; src/engine/dac_engine.cc:50-64)
// changes.
//
// Argument naming follows the reference here: M = weight rows (output
// features), N = tokens. The C ABI in w8a8.h uses the opposite letters.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

struct cublasContext;  // the handle is accepted for signature compatibility and never used
typedef struct cublasContext* cublasHandle_t;

#if defined(__GNUC__)
#define FISH_SHIM_API __attribute__((visibility("default")))
#else
#define FISH_SHIM_API
#endif

namespace fish::kernels {

// src/kernels/kernels.h:242-259
FISH_SHIM_API void int8_dequant_gemm_fp16(const int8_t* W, const __half* scale, int group_size, const __half* act_scale,
                            const __half* smooth_inv, const __half* X, __half* Y, int M, int N, int K,
                            cublasHandle_t cublas, cudaStream_t stream = 0);
// src/kernels/kernels.h:10-19
FISH_SHIM_API void rms_norm(const __half* x, const __half* weight, __half* out, int n_tokens, int dim, float eps,
              cudaStream_t stream = 0);
// src/kernels/kernels.h:111-115, :127-141
FISH_SHIM_API void silu_forward(__half* x, int n, cudaStream_t stream = 0);
FISH_SHIM_API void mul_forward(__half* a, const __half* b, int n, cudaStream_t stream = 0);
FISH_SHIM_API void residual_add(__half* a, const __half* b, int n, cudaStream_t stream = 0);

}  // namespace fish::kernels
