/*
 * CPU oracle for the INT8 W8A8 linear path — TEST INFRASTRUCTURE, NOT PRODUCT.
 *
 * A plain-C, scalar restatement of the arithmetic in the reference's
 * src/kernels/int8_gemm.cu (quantiser, per-group integer sums, fp32 promote,
 * fp16 cast), src/kernels/rms_norm.cu and the silu/mul/residual_add kernels of
 * src/kernels/ffn_activations.cu.  Only tests, the smoke check and the
 * benchmark's CPU-baseline leg may call it; the CUDA library never does.
 *
 * Parity status: the reference ships no test, golden vector or host
 * implementation for this path, so this oracle is pinned against outputs of
 * the reference's own CUDA kernels (see tests/golden/) rather than against
 * reference test fixtures.
 *
 * Naming: M = tokens, N = output features, K = input features,
 * g = group size along K, G = ceil(K / g).  fp16 values travel as uint16_t.
 */
#ifndef W8A8_ORACLE_H
#define W8A8_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { W8A8O_ACT_PER_TOKEN_GROUP = 0, W8A8O_ACT_PER_TOKEN = 1 };
enum { W8A8O_PROMOTE_FMA = 0, W8A8O_PROMOTE_MUL_ADD = 1 };
enum { W8A8O_EPI_NONE = 0, W8A8O_EPI_RESIDUAL = 1, W8A8O_EPI_SWIGLU = 2 };

float    w8a8o_half_to_float(uint16_t h);
uint16_t w8a8o_float_to_half(float f);

/* group_size <= 0 or > K means one group of K (int8_gemm.cu:396-397). */
int w8a8o_num_groups(int K, int group_size);

/* Activation quantiser (int8_gemm.cu:147-211).  Xs is [M,G] fp32. */
int w8a8o_quantize(const uint16_t* X, const uint16_t* smooth_inv,
                   const uint16_t* act_scale, int M, int K, int group_size,
                   int act_mode, int8_t* Xq, float* Xs);

/* Exact per-group integer sums P[m][n][j] (what int8_gemm.cu:470-490 asks cuBLAS for). */
int w8a8o_group_sums(const int8_t* W, const int8_t* Xq, int M, int N, int K,
                     int group_size, int32_t* P);

/* Promote + cast (int8_gemm.cu:213-243): groups ascending from 0.0f.
 * Yh fp16 [M,N]; Yf32 (optional) the fp32 accumulator before the cast;
 * Yf64 (optional) the same sum carried in double. */
int w8a8o_linear_q(const int8_t* W, const uint16_t* w_scale, const int8_t* Xq,
                   const float* Xs, int M, int N, int K, int group_size,
                   int promote, uint16_t* Yh, float* Yf32, double* Yf64);

/* Whole entry point (int8_gemm.cu:384-511) with an optional fused epilogue.
 * EPI_RESIDUAL: Y = half(float(half(acc)) + float(R[m][n]))   (GEMM, then
 *   ffn_activations.cu:41-45, with the fp16 rounding between them kept).
 * EPI_SWIGLU: W rows are interleaved in blocks of 16 (rows 16b..16b+7 = gate
 *   channels 8b..8b+7, rows 16b+8..16b+15 = up channels 8b..8b+7) and
 *   Y is [M, N/2]:  half(float(half(silu(float(half(gate))))) * float(half(up)))
 *   (GEMM, silu, GEMM, mul of dual_ar_engine.cc:640-644, all roundings kept). */
int w8a8o_linear(const int8_t* W, const uint16_t* w_scale, int group_size,
                 const uint16_t* act_scale, const uint16_t* smooth_inv,
                 const uint16_t* X, int M, int N, int K, int act_mode,
                 int promote, int epilogue, const uint16_t* R, uint16_t* Y);

/* RMSNorm (rms_norm.cu:10-58): out = half((float(x) * r) * float(w)),
 * r = 1/sqrt(mean(x^2) + eps).  The device uses an approximate rsqrt and a
 * tree-shaped fp32 sum, so device results are compared at 1 fp16 ulp. */
int w8a8o_rms_norm(const uint16_t* x, const uint16_t* w, uint16_t* out,
                   int tokens, int dim, float eps);

/* Elementwise neighbours (ffn_activations.cu:12-17, 35-45), in place on a. */
int w8a8o_silu(uint16_t* a, long n);
int w8a8o_mul(uint16_t* a, const uint16_t* b, long n);
int w8a8o_residual_add(uint16_t* a, const uint16_t* b, long n);

/* Timed leg for the benchmark's CPU baseline: runs w8a8o_linear over the first
 * n_rows output rows with `threads` host threads (<= 0: all online cores). Returns seconds, <0 on error. */
int w8a8o_host_threads(void);
double w8a8o_timed_linear(const int8_t* W, const uint16_t* w_scale, int group_size,
                          const uint16_t* X, int M, int N, int K, int n_rows,
                          int threads, uint16_t* Y);

#ifdef __cplusplus
}
#endif
#endif
