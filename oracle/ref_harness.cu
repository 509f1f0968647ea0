// Parity harness around the reference's own CUDA kernels — TEST INFRASTRUCTURE.
//
// The reference sources are compiled where they lie (the build passes
// -I<reference>/src); nothing of them is copied here. Including the .cu files
// into this translation unit makes the reference's file-local workspace
// (int8 codes, activation scales, int32 partial sums) visible, so tests can
// compare those intermediates bit for bit.
//
// Exposed as a C ABI so the Python tests and the benchmark's reference arm can
// drive it through ctypes. Built into oracle/_ref/libfishref.so.
#include "kernels/int8_gemm.cu"        // reference: src/kernels/int8_gemm.cu
#include "kernels/rms_norm.cu"         // reference: src/kernels/rms_norm.cu
#include "kernels/ffn_activations.cu"  // reference: src/kernels/ffn_activations.cu
#include "kernels/rope.cu"             // reference: src/kernels/rope.cu
#include "kernels/paged_attention.cu"  // reference: src/kernels/paged_attention.cu

#include <cstdio>

namespace {
cublasHandle_t g_handle = nullptr;
char g_err[512] = {0};

template <typename F>
int guarded(F&& f) {
    try {
        f();
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            snprintf(g_err, sizeof g_err, "CUDA: %s", cudaGetErrorString(e));
            return 3;
        }
        return 0;
    } catch (const std::exception& ex) {
        snprintf(g_err, sizeof g_err, "%s", ex.what());
        return 3;
    }
}
}  // namespace

extern "C" {

const char* fishref_last_error() { return g_err; }

// fish::kernels::int8_dequant_gemm_fp16 (src/kernels/kernels.h:242-259), stock path.
// M_out = weight rows, N_tok = tokens (the reference's own argument order).
int fishref_int8_dequant_gemm_fp16(const void* W, const void* scale, int group_size,
                                   const void* act_scale, const void* smooth_inv,
                                   const void* X, void* Y, int M_out, int N_tok, int K,
                                   void* stream) {
    return guarded([&] {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        if (!g_handle) CUBLAS_CHECK(cublasCreate(&g_handle));
        CUBLAS_CHECK(cublasSetStream(g_handle, s));
        fish::kernels::int8_dequant_gemm_fp16(
            static_cast<const int8_t*>(W), static_cast<const __half*>(scale), group_size,
            static_cast<const __half*>(act_scale), static_cast<const __half*>(smooth_inv),
            static_cast<const __half*>(X), static_cast<__half*>(Y), M_out, N_tok, K, g_handle, s);
    });
}

// Device pointers of the reference's workspace after the last call on this thread:
// which = 0 int8 codes [N_tok,K], 1 fp32 activation scales [N_tok,G],
//         2 int32 partial sums of the LAST group, laid out [N_tok][M_out],
//         3 fp32 accumulator [N_tok][M_out].
void* fishref_workspace_ptr(int which) {
    switch (which) {
        case 0: return fish::kernels::g_ws.x_q;
        case 1: return fish::kernels::g_ws.x_scale;
        case 2: return fish::kernels::g_ws.partial;
        case 3: return fish::kernels::g_ws.accum;
    }
    return nullptr;
}

// Copies `bytes` of workspace `which` (see above) into the device buffer dst.
int fishref_copy_workspace(int which, void* dst, size_t bytes) {
    void* src = fishref_workspace_ptr(which);
    if (!src) { snprintf(g_err, sizeof g_err, "workspace %d is empty", which); return 1; }
    cudaError_t e = cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice);
    if (e != cudaSuccess) { snprintf(g_err, sizeof g_err, "CUDA: %s", cudaGetErrorString(e)); return 3; }
    return 0;
}

int fishref_rms_norm(const void* x, const void* w, void* out, int n_tokens, int dim, float eps,
                     void* stream) {
    return guarded([&] {
        fish::kernels::rms_norm(static_cast<const __half*>(x), static_cast<const __half*>(w),
                                static_cast<__half*>(out), n_tokens, dim, eps,
                                static_cast<cudaStream_t>(stream));
    });
}

int fishref_silu(void* x, int n, void* stream) {
    return guarded([&] {
        fish::kernels::silu_forward(static_cast<__half*>(x), n, static_cast<cudaStream_t>(stream));
    });
}

int fishref_mul(void* a, const void* b, int n, void* stream) {
    return guarded([&] {
        fish::kernels::mul_forward(static_cast<__half*>(a), static_cast<const __half*>(b), n,
                                   static_cast<cudaStream_t>(stream));
    });
}

int fishref_residual_add(void* a, const void* b, int n, void* stream) {
    return guarded([&] {
        fish::kernels::residual_add(static_cast<__half*>(a), static_cast<const __half*>(b), n,
                                    static_cast<cudaStream_t>(stream));
    });
}

int fishref_rope_qk(void* q, void* k, const float* freqs, int batch, int n_q, int n_k, int seq_len, int head_dim,
                    int offset, void* stream) {
    return guarded([&] {
        fish::kernels::rope_qk(static_cast<const __half*>(q), static_cast<const __half*>(k), freqs, batch, n_q, n_k,
                               seq_len, head_dim, offset, static_cast<cudaStream_t>(stream));
    });
}

int fishref_paged_attention_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                   const int* seq_lens, void* out, int batch, int n_heads, int head_dim,
                                   int max_blocks, float sm_scale, int layer, int n_layers, int n_kv, void* stream) {
    return guarded([&] {
        fish::kernels::paged_attention_decode(static_cast<const __half*>(q), static_cast<const __half*>(k_cache),
                                              static_cast<const __half*>(v_cache), block_table, seq_lens,
                                              static_cast<__half*>(out), batch, n_heads, head_dim, max_blocks,
                                              sm_scale, layer, n_layers, n_kv, static_cast<cudaStream_t>(stream));
    });
}

}  // extern "C"
