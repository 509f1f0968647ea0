// Internal declarations shared by the .cu files of libw8a8. Not installed.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/w8a8.h"

namespace w8a8 {

// Records a message for w8a8_last_error() and returns `status`.
int fail(int status, const char* fmt, ...);
// cudaGetLastError() after a launch -> status.
int check_launch(const char* what);
// Which launches carry the programmatic-dependent-launch attribute (may start while the kernel before
// them is still running, and wait inside the kernel for its results). Classes are a bit mask so that
// the environment variable W8A8_PDL=<mask> can switch them one by one; W8A8_NO_PDL=1 switches all off.
enum { kPdlLinear = 1, kPdlRow = 2, kPdlAttn = 4 };
// Measured over the decode stack: early launch pays for the linears (weights are requested while the small kernel
// before them runs) and for the row kernels. It costs time on the attention launch: its CTAs, resident early, take
// the shared memory that the second CTA per SM of the linear before them needs.
constexpr int kPdlDefaultMask = kPdlLinear | kPdlRow;
bool pdl_enabled(int kernel_class);

inline int norm_group(int K, int group_size) {
    return (group_size <= 0 || group_size > K) ? K : group_size;
}
inline int num_groups(int K, int group_size) {
    int g = norm_group(K, group_size);
    return (K + g - 1) / g;
}

// Where a row-parallel linear sends its fp32 partial output (w8a8_tp.cu): slot [rank] of every rank's exchange buffer.
struct TpPush {
    int world, rank, max_tokens;  // world == 0: no send
    size_t ctl_off;               // control words behind the slots: [0] the epoch of the last finished exchange
    unsigned char* peers[8];      // every rank's exchange buffer as mapped here (peers[rank] is the local one)
};

struct LinearArgs {
    const int8_t* W;
    const __half* w_scale;  // [N, G]
    const int8_t* Xq;       // [M, K]   (null when X is given and the kernel quantises itself)
    const float* Xs;        // [M, G]
    const __half* X;        // [M, K]   fp16 source for kernels that quantise in their prologue
    const __half* smooth_inv;
    const __half* act_scale;
    __half* Y;
    const __half* residual;
    int32_t* dump;          // [M, N, G] or null
    int M, N, K, g, G;
    int epilogue;
    int split_k;
    const void* packed;     // the weight re-packed by launch_pack_weight (null: not packed)
    // scratch for kernels that cut K across CTAs (owned by the context; null: such kernels are not used)
    void* splitk_partials;
    size_t splitk_partial_bytes;
    int* splitk_counters;        // zero between launches
    size_t splitk_counter_count;
    // Fused prologue (packed GEMV, M <= 8): norm_weight != null means that Xq / Xs are absent and every CTA
    // forms them itself in shared memory from X: [x = half(x + norm_residual)] -> RMSNorm -> quantiser.
    const __half* norm_weight;    // [K]
    float norm_eps;
    const __half* norm_residual;  // [M, K] or null
    __half* norm_x_out;           // [M, K] or null: CTA 0 stores the updated x (must not alias X)
    int8_t* codes_out;            // [M, K] / [M, G] or null: CTA 0 stores the codes and scales it formed
    float* scales_out;
    // Tail (packed GEMV, M <= 8): work on the launch's own OUTPUT done by the CTAs that finish last, so that the
    // small kernel that would follow (and the launch edge before it) disappears. Counted in `tail_counters`
    // (context-owned, zero between launches).
    //   kTailRowNorm:  x += Y (rounded like residual_add) -> RMSNorm -> quantiser, a CTA per token row
    //   kTailGroupQuant: the quantiser alone over Y ([M, N] or, with the SwiGLU epilogue, [M, N/2]), by whichever
    //                    CTA stores the last tile of a quantisation group
    int tail_kind;
    int* tail_counters;
    __half* tail_x;               // kTailRowNorm: residual stream [M, N], updated in place
    const __half* tail_norm_weight;
    float tail_eps;
    int tail_g;                   // group size of the codes the tail produces
    int8_t* tail_Xq;              // [M, N'] (null with kTailRowNorm: no quantiser, e.g. the final norm)
    float* tail_Xs;               // [M, N'/tail_g]
    __half* tail_normed_out;      // kTailRowNorm: optional fp16 [M, N]
    TpPush tp;                    // packed GEMV, W8A8_EPI_NONE: finished tiles also go to every rank's exchange buffer
};
enum { kTailNone = 0, kTailRowNorm = 1, kTailGroupQuant = 2 };
constexpr int kTailCounterInts = 256;  // two for kTailRowNorm, one per output group for kTailGroupQuant

// w8a8_api.cu : picks the kernel for a linear whose codes and scales exist.
int dispatch_linear_q(const LinearArgs& a, int kernel, int* device_status, cudaStream_t s);
// w8a8_quant.cu
int launch_rowquant(const __half* x_in, __half* x_out, const __half* residual,
                    const __half* norm_weight, float eps, const __half* smooth_inv,
                    const __half* act_scale, int M, int K, int g, int act_mode, __half* normed_out,
                    int8_t* Xq, float* Xs, cudaStream_t stream);
// w8a8_elementwise.cu
int launch_silu(__half* a, long n, cudaStream_t s);
int launch_mul(__half* a, const __half* b, long n, cudaStream_t s);
int launch_residual_add(__half* a, const __half* b, long n, cudaStream_t s);
int launch_pack_gate_up(const int8_t* wg, const __half* sg, const int8_t* wu, const __half* su,
                        int inter, int K, int G, int8_t* Wo, __half* So, cudaStream_t s);
// w8a8_generic.cu : any shape, sequential group order.
int launch_linear_generic(const LinearArgs& a, cudaStream_t s);
// w8a8_gemv.cu : M <= 32.
bool gemv_supports(const LinearArgs& a);
int launch_linear_gemv(const LinearArgs& a, cudaStream_t s);
// w8a8_gemv_tma.cu : M <= 32, TMA-fed persistent stream-K form.
bool gemv_tma_supports(const LinearArgs& a);
int launch_linear_gemv_tma(const LinearArgs& a, int* device_status, cudaStream_t s);
// w8a8_gemv_packed.cu : M <= 32 over pre-packed weights (linear byte stream, 1-D bulk copies).
size_t packed_weight_bytes(int N, int K, int g);
int launch_pack_weight(const int8_t* W, const __half* S, int N, int K, int g, void* out, cudaStream_t s);
int gemv_packed_ctas(int tiles, int sms, bool two_per_sm);  // CTAs that share a linear's row tiles
bool gemv_packed_supports(const LinearArgs& a);  // also answers for the prologue and tail forms (fields of a set)
int launch_linear_gemv_packed(const LinearArgs& a, int* device_status, cudaStream_t s);
// w8a8_attn.cu : decode-step neighbours (qk-norm + RoPE + KV write; paged attention).
int launch_qknorm_rope_kvwrite(const __half* qkv, const __half* q_norm_w, const __half* k_norm_w, float eps,
                               const float* freqs, const int* positions, const int* block_table, int max_blocks,
                               __half* k_cache, __half* v_cache, int layer, int n_layers, int B, int n_q, int n_kv,
                               __half* q_out, cudaStream_t stream);
int launch_paged_attention_decode(const __half* q, const __half* k_cache, const __half* v_cache,
                                  const int* block_table, const int* seq_lens, int B, int n_q, int n_kv,
                                  int max_blocks, float sm_scale, int layer, int n_layers, __half* out, int g,
                                  int8_t* Xq, float* Xs, int splits, int* status, cudaStream_t stream);
int launch_qkv_attention_decode(const __half* qkv, const __half* q_norm_w, const __half* k_norm_w, float eps,
                                const float* freqs, const int* positions, __half* k_cache, __half* v_cache,
                                const int* block_table, const int* seq_lens, int B, int n_q, int n_kv, int max_blocks,
                                float sm_scale, int layer, int n_layers, __half* out, int g, int8_t* Xq, float* Xs,
                                int splits, int* status, cudaStream_t stream);
// w8a8_decode_stack.cu : a whole decode step as one persistent cooperative kernel.
size_t decode_stack_workspace_bytes(const w8a8_decode_stack& d);
int launch_decode_stack(const w8a8_decode_stack& d, unsigned char* workspace, size_t workspace_bytes, float* partials,
                        size_t partial_bytes, int* counters, size_t counter_count, int* status, cudaStream_t stream);
int decode_stack_timeline(const w8a8_decode_stack& d, const unsigned char* workspace, unsigned long long* out, int capacity,
                          cudaStream_t stream);
// w8a8_tp.cu : one-shot all-reduce over peer memory fused with residual add + RMSNorm + quantiser.
struct TpState;
int tp_create(TpState** out, int rank, int world, int max_tokens, int dim, void* ipc_handle_out64);
int tp_connect(TpState* t, const void* all_handles);
int tp_destroy(TpState* t);
int tp_push_args(const TpState* t, int M, int N, TpPush* out);
int launch_tp_allreduce_rowquant(TpState* t, __half* x, const __half* partial, const __half* norm_weight, float eps,
                                 const __half* smooth_inv, const __half* act_scale, int M, int K, int g, int act_mode,
                                 __half* normed_out, int8_t* Xq, float* Xs, int* status, cudaStream_t stream);
// w8a8_gemm_sm100.cu : tcgen05 + TMA.
bool gemm_supports(const LinearArgs& a);
// form: -1 picks between one CTA per tile (0) and a CTA pair per tile (1) by shape
int launch_linear_gemm(const LinearArgs& a, int* device_status, cudaStream_t s, int form = -1);

}  // namespace w8a8
