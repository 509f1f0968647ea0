/*
 * w8a8.h — C ABI of the B200 (sm_100a) INT8 W8A8 linear-layer library.
 *
 * Drop-in for the kernel-layer boundary of KBlackMeow/fish-audio-cpp: every
 * entry point names the reference interface it replaces (path:line inside
 * that project). All pointers are DEVICE pointers owned by the caller unless
 * said otherwise; `stream` is a cudaStream_t passed as void*. The calls of "the
 * path" and "decode-step neighbours" below are asynchronous on `stream`, never
 * allocate and never synchronise. Set-up and read-out calls are the exception and
 * say so: w8a8_create / w8a8_destroy / w8a8_tp_create / w8a8_tp_connect allocate
 * or map device memory, w8a8_check_device_status, w8a8_static_scratch_check_status
 * and w8a8_decode_stack_timeline synchronise the stream. Every call returns a
 * status code (no C++ exception crosses this boundary).
 *
 * Naming: M = tokens, N = output features (weight rows), K = input features,
 * group_size = quantisation group along K (<= 0 or > K means one group of K),
 * G = ceil(K / group_size). The reference's own signature calls the weight
 * rows "M" and the tokens "N"; the C++ shim (fish_kernels_shim.h) keeps that
 * order, this header does not.
 *
 * Layouts (all row-major, identical to the reference's):
 *   W        int8   [N, K]
 *   w_scale  fp16   [N] when G == 1, else [N, G]
 *   X, Y     fp16   [M, K], [M, N]
 *   Xq       int8   [M, K]      activation codes, never -128
 *   Xs       fp32   [M, G]      activation scales
 *   smooth_inv fp16 [K]  (optional)   act_scale fp16 [G] (optional, static scales)
 */
#ifndef W8A8_H
#define W8A8_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define W8A8_API __attribute__((visibility("default")))
#else
#define W8A8_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status -------------------------------------------------------------- */
enum {
    W8A8_OK = 0,
    W8A8_ERR_INVALID_ARG = 1, /* null pointer, negative size, misaligned pointer */
    W8A8_ERR_UNSUPPORTED = 2, /* shape outside what any kernel here handles */
    W8A8_ERR_CUDA = 3,        /* a CUDA call failed; see w8a8_last_error() */
    W8A8_ERR_TIMEOUT = 4,     /* a bounded device-side wait ran out */
    W8A8_ERR_WORKSPACE = 5    /* the context's scratch is too small for this call */
};
W8A8_API const char* w8a8_status_string(int status);
/* Message of the last failing call on this host thread (thread-local, never NULL).
 * Replaces the std::runtime_error text of CUDA_CHECK, src/utils/cuda_utils.h:9-16. */
W8A8_API const char* w8a8_last_error(void);

/* ---- context ------------------------------------------------------------- */
/* Owns the scratch that the reference keeps in a thread_local Workspace that
 * grows by cudaFree+cudaMalloc inside the call (src/kernels/int8_gemm.cu:31-44,
 * :97-102, :405-413). Here it is sized once, so calls are capturable and never
 * block. One context per stream: calls sharing a context must not overlap. */
typedef struct w8a8_ctx w8a8_ctx;

W8A8_API int w8a8_create(w8a8_ctx** out, int device, size_t workspace_bytes);
W8A8_API int w8a8_destroy(w8a8_ctx* ctx);
/* Scratch a w8a8_linear call of this shape needs in the context's workspace: the int8 codes
 * [M, K] and fp32 scales [M, G], each rounded up to 256 bytes (the same for every M). */
W8A8_API size_t w8a8_workspace_bytes(int M, int N, int K, int group_size);
W8A8_API size_t w8a8_ctx_workspace_bytes(const w8a8_ctx* ctx);
/* Polls the context's device error word (set by a kernel whose bounded wait ran
 * out). Synchronises `stream`. Returns W8A8_OK or W8A8_ERR_TIMEOUT and clears it. */
W8A8_API int w8a8_check_device_status(w8a8_ctx* ctx, void* stream);

/* ---- options ------------------------------------------------------------- */
enum { /* how activation scales are formed */
    W8A8_ACT_PER_TOKEN_GROUP = 0, /* one scale per (token, K-group): what the reference does,
                                     int8_gemm.cu:147-211 with grid (tokens, groups) */
    W8A8_ACT_PER_TOKEN = 1        /* one scale per token over all of K (no reference counterpart) */
};
enum { /* what happens to the fp32 accumulator after the last group */
    W8A8_EPI_NONE = 0,     /* Y = half(acc)                         int8_gemm.cu:236-243 */
    W8A8_EPI_RESIDUAL = 1, /* Y = half(float(half(acc)) + float(R)) + ffn_activations.cu:41-45 */
    W8A8_EPI_SWIGLU = 2    /* W holds gate and up rows interleaved in blocks of 16 rows
                              (8 gate rows, then the 8 up rows of the same channels; see
                              w8a8_pack_gate_up). Y is [M, N/2]:
                              half(float(half(silu(float(half(g))))) * float(half(u))),
                              i.e. the GEMM, silu, GEMM, mul chain of
                              src/engine/dual_ar_engine.cc:640-644 with every fp16 rounding kept. */
};
enum { /* forces a kernel family; default picks by shape */
    W8A8_KERNEL_AUTO = 0,
    W8A8_KERNEL_GENERIC = 1, /* scalar-order SIMT kernel, any shape */
    W8A8_KERNEL_GEMV = 2,    /* M <= 32: warp-MMA weight-streaming kernel, cluster split-K */
    W8A8_KERNEL_GEMM = 3,    /* tcgen05 + TMA kernel; picks between the two forms below by shape */
    W8A8_KERNEL_GEMV_TMA = 4, /* M <= 32: TMA-fed persistent stream-K kernel over the row-major matrix */
    W8A8_KERNEL_GEMV_PACKED = 5, /* M <= 32: the same over a weight packed by w8a8_pack_weight (the default
                                    once the weight is registered) */
    W8A8_KERNEL_GEMM_SINGLE = 6, /* tcgen05 kernel, one CTA per 128-token x 256-row tile */
    W8A8_KERNEL_GEMM_PAIR = 7    /* tcgen05 kernel, a CTA pair (cta_group::2) per 256-token x 256-row tile */
};

typedef struct w8a8_linear_opts {
    int act_mode;             /* W8A8_ACT_* (ignored by w8a8_linear_q) */
    int epilogue;             /* W8A8_EPI_* */
    const void* residual;     /* fp16 [M, N], W8A8_EPI_RESIDUAL only; may alias Y */
    int32_t* dump_group_sums; /* optional int32 [M, N, G]: the exact per-group integer sums
                                 (what int8_gemm.cu:470-490 leaves in `partial`), for parity tests */
    int kernel;               /* W8A8_KERNEL_* */
    int split_k;              /* GEMV only: 0 = choose, else 1/2/4/8 K-slices per row tile */
} w8a8_linear_opts;

/* ---- the path ------------------------------------------------------------ */

/* Replaces quantize_activation_groups_kernel, src/kernels/int8_gemm.cu:147-211. */
W8A8_API int w8a8_quantize(w8a8_ctx* ctx, const void* X, const void* smooth_inv, const void* act_scale,
                  int M, int K, int group_size, int act_mode, void* Xq, void* Xs, void* stream);

/* Replaces fish::kernels::rms_norm, src/kernels/kernels.h:10-19 (src/kernels/rms_norm.cu:10-76).
 * Same summation order as the reference kernel, so results are bit-identical to it. */
W8A8_API int w8a8_rms_norm(w8a8_ctx* ctx, const void* x, const void* weight, void* out, int tokens,
                  int dim, float eps, void* stream);

/* Fuses, per token row: [x += residual (ffn_activations.cu:41-45)] -> rms_norm
 * (rms_norm.cu:10-58) -> quantiser (int8_gemm.cu:147-211). The normed value is rounded to
 * fp16 in registers before it is quantised, so codes equal those of the unfused chain.
 * residual may be NULL; when it is not, x is updated in place. normed_out may be NULL. */
W8A8_API int w8a8_rmsnorm_quantize(w8a8_ctx* ctx, void* x, const void* residual, const void* weight,
                          float eps, const void* smooth_inv, const void* act_scale, int M, int K,
                          int group_size, int act_mode, void* normed_out, void* Xq, void* Xs,
                          void* stream);

/* Replace silu_forward / mul_forward / residual_add, src/kernels/kernels.h:111-141
 * (src/kernels/ffn_activations.cu:12-17, :35-45). In place on a. */
W8A8_API int w8a8_silu(w8a8_ctx* ctx, void* a, long n, void* stream);
W8A8_API int w8a8_mul(w8a8_ctx* ctx, void* a, const void* b, long n, void* stream);
W8A8_API int w8a8_residual_add(w8a8_ctx* ctx, void* a, const void* b, long n, void* stream);

/* Replaces fish::kernels::int8_dequant_gemm_fp16, src/kernels/kernels.h:242-259
 * (src/kernels/int8_gemm.cu:384-511): quantise X, integer GEMM per K-group, fp32 promote with
 * both scales, fp16 out. opts may be NULL (reference behaviour). */
W8A8_API int w8a8_linear(w8a8_ctx* ctx, const void* W, const void* w_scale, int group_size,
                const void* act_scale, const void* smooth_inv, const void* X, void* Y, int M,
                int N, int K, const w8a8_linear_opts* opts, void* stream);

/* w8a8_rmsnorm_quantize and the w8a8_linear_q after it as ONE call, for the decode step: per token row
 * [x_out = x + residual (ffn_activations.cu:41-45)] -> rms_norm (rms_norm.cu:10-58) -> quantiser
 * (int8_gemm.cu:147-211) -> linear (int8_gemm.cu:423-505). Replaces, in DualAREngine::decode_step, the
 * rms_norm launch and the quantized_gemm after it (src/engine/dual_ar_engine.cc:580-584, :636-641).
 * x is not modified. residual may be NULL; when it is not, x_out (a buffer other than x) receives the
 * updated residual stream. codes_out / scales_out (both or neither) receive the int8 codes [M, K] and
 * fp32 scales [M, G] the linear consumed. For M <= 8 over a weight registered with
 * w8a8_register_packed_weight this is one launch (every CTA quantises the rows itself, in shared memory,
 * while its first weight blocks are in flight); other shapes run the two kernels back to back. Results
 * are those of the two-call chain, bit for bit. opts->act_mode must be W8A8_ACT_PER_TOKEN_GROUP for the
 * one-launch form. */
W8A8_API int w8a8_rmsnorm_linear(w8a8_ctx* ctx, const void* W, const void* w_scale, int group_size,
                        const void* x, const void* residual, void* x_out, const void* norm_weight,
                        float eps, void* Y, int M, int N, int K, const w8a8_linear_opts* opts,
                        void* codes_out, void* scales_out, void* stream);

/* The same from codes and scales already formed (by w8a8_quantize or
 * w8a8_rmsnorm_quantize): int8_gemm.cu:423-505 without its first stage. */
W8A8_API int w8a8_linear_q(w8a8_ctx* ctx, const void* W, const void* w_scale, int group_size,
                  const void* Xq, const void* Xs, void* Y, int M, int N, int K,
                  const w8a8_linear_opts* opts, void* stream);

/* What the launch of a decode-time linear may do to its own output once the output is complete, in place of the
 * small kernel the engine would launch next (and of the launch edge before it):
 *   W8A8_TAIL_ROWNORM     x += Y (ffn_activations.cu:41-45), then rms_norm of x (rms_norm.cu:10-58), then the
 *                         quantiser of the next linear (int8_gemm.cu:147-211): DualAREngine::decode_step's
 *                         residual_add + rms_norm after wo and after w2 (src/engine/dual_ar_engine.cc:631-637,
 *                         :645-647, :580) plus the first stage of the quantized_gemm that follows.
 *   W8A8_TAIL_GROUPQUANT  the quantiser alone over Y (with W8A8_EPI_SWIGLU: over the [M, N/2] product): the first
 *                         stage of the w2 call after silu / mul (dual_ar_engine.cc:640-646).
 * Results are those of the separate calls, bit for bit. */
enum { W8A8_TAIL_NONE = 0, W8A8_TAIL_ROWNORM = 1, W8A8_TAIL_GROUPQUANT = 2 };
typedef struct w8a8_tail {
    int kind;                /* W8A8_TAIL_* */
    void* x;                 /* ROWNORM: the residual stream, fp16 [M, N], updated in place */
    const void* norm_weight; /* ROWNORM: fp16 [N] */
    float eps;               /* ROWNORM */
    int group_size;          /* quantisation group of the codes written (64, 128 or 256 for ROWNORM) */
    void* Xq;                /* int8 codes of the result, [M, N] (GROUPQUANT after SwiGLU: [M, N/2]); ROWNORM: may be
                                NULL (no quantiser, e.g. the final norm) */
    void* Xs;                /* fp32 scales [M, columns / group_size] */
    void* normed_out;        /* ROWNORM: optional fp16 [M, N], the normed rows */
} w8a8_tail;

/* w8a8_linear_q followed by `tail` on its output. For M <= 8 over a weight registered with
 * w8a8_register_packed_weight this is ONE launch: the CTAs of the decode kernel that finish last do the tail (a
 * CTA per token row for ROWNORM, after a bounded wait for the rest of the grid; whichever CTA completes a group
 * for GROUPQUANT). Other shapes run the separate kernels back to back. Y is written as by w8a8_linear_q and must
 * not alias tail->x. */
W8A8_API int w8a8_linear_q_tail(w8a8_ctx* ctx, const void* W, const void* w_scale, int group_size,
                       const void* Xq, const void* Xs, void* Y, int M, int N, int K,
                       const w8a8_linear_opts* opts, const w8a8_tail* tail, void* stream);

/* Diagnostic: copies the first `count` (<= 256) ints of the context's tail arrival counters to host memory
 * (synchronises the stream). Between launches every counter a tail uses is zero; a diagnostic build of the
 * library (-DW8A8_TAIL_TIMELINE) additionally leaves the device-timer stamps of the last CTA to arrive in
 * ints 128.. (nine 64-bit words). */
W8A8_API int w8a8_debug_tail_counters(w8a8_ctx* ctx, int* out, int count, void* stream);

/* No counterpart in the reference. The same computation as w8a8_linear for callers that may not
 * allocate device memory and therefore cannot create a context (w8a8_create allocates): a plugin
 * inside a host process that owns the whole device-memory budget, or a real-time audio thread that
 * cannot afford the device-wide synchronisation cudaMalloc/cudaFree imply. The activation codes and
 * scales live in an array built into the library image: w8a8_static_scratch_bytes() (8 MiB) on
 * every GPU that loads the library, until the process exits. The call needs
 * round_up(M*K, 256) + round_up(4*M*G, 256) bytes of it and returns W8A8_ERR_WORKSPACE, launching
 * nothing, when that is more than the array holds. One array per GPU is shared by all streams and
 * threads and keeps the last call's contents: calls that can overlap on the GPU race, so order
 * them; nothing needs clearing between calls (every byte read was written by the same call). The
 * first call on a device resolves the array's address on that device and should be made before any
 * stream capture begins. Calls no cudaMalloc, cudaFree or other allocating routine. */
W8A8_API size_t w8a8_static_scratch_bytes(void);
W8A8_API int w8a8_linear_static_scratch(const void* W, const void* w_scale, int group_size,
                               const void* act_scale, const void* smooth_inv, const void* X,
                               void* Y, int M, int N, int K, const w8a8_linear_opts* opts,
                               void* stream);
/* No counterpart in the reference. w8a8_check_device_status for the context-free entry point above:
 * reads (and clears) the error word that w8a8_linear_static_scratch's kernels set on the current
 * device when one of their bounded waits runs out. Synchronises `stream`; allocates nothing.
 * Returns W8A8_OK or W8A8_ERR_TIMEOUT. */
W8A8_API int w8a8_static_scratch_check_status(void* stream);

/* ---- loader side --------------------------------------------------------- */
/* ---- decode-step neighbours inside a layer ----------------------------------------------- */

/* Replaces, per layer of DualAREngine::decode_step: the three device copies that split the fused qkv
 * row, rms_norm on q and on k (qk-norm, skipped when the weight pointers are NULL), rope_qk, and the
 * 2 x n_kv cudaMemcpyAsync calls that write k and v into the paged cache
 * (src/engine/dual_ar_engine.cc:585-628; src/kernels/rope.cu:9-65; src/kernels/rms_norm.cu:10-58).
 * qkv fp16 [batch, (n_q + 2 n_kv) * head_dim] laid out [q | k | v]; positions int32 [batch] = the new
 * token's position (the reference handles batch 1 and passes it as `token_pos`); caches fp16
 * [blocks, n_layers, n_kv, 16, head_dim] (src/engine/block_manager.h:73); q_out fp16
 * [batch, n_q, head_dim]. Same rounding points and summation order as the reference chain. */
W8A8_API int w8a8_qknorm_rope_kvwrite(w8a8_ctx* ctx, const void* qkv, const void* q_norm_w,
                             const void* k_norm_w, float eps, const float* freqs, const int* positions,
                             const int* block_table, int max_blocks_per_seq, void* k_cache, void* v_cache,
                             int layer, int n_layers, int batch, int n_q_heads, int n_kv_heads,
                             int head_dim, void* q_out, void* stream);

/* Replaces fish::kernels::paged_attention_decode, src/kernels/kernels.h:51-69
 * (src/kernels/paged_attention.cu:13-150); same arguments in the same order, then three additions:
 * when Xq is not NULL the attention output is also quantised for the following o-projection
 * (int8 codes [batch, n_heads*head_dim], fp32 scales per quant_group_size channels, the arithmetic of
 * int8_gemm.cu:147-211), `out` may then be NULL; context_splits (0 = choose) is the number of CTAs
 * that share one (sequence, kv head). Needs n_heads == 4 * n_kv_heads. */
W8A8_API int w8a8_paged_attention_decode(w8a8_ctx* ctx, const void* q, const void* k_cache,
                                const void* v_cache, const int* block_table, const int* seq_lens,
                                void* out, int batch, int n_heads, int head_dim, int max_blocks_per_seq,
                                float sm_scale, int layer, int n_layers, int n_kv_heads,
                                int quant_group_size, void* Xq, void* Xs, int context_splits,
                                void* stream);

/* w8a8_qknorm_rope_kvwrite and w8a8_paged_attention_decode as ONE launch (same arguments, q never leaves the
 * chip): each (sequence, kv head) CTA group norms and rotates its four query heads itself, the CTA that attends
 * over the block the new token joins writes the new k and v rows first. Same arithmetic and rounding points as
 * the two calls, so outputs, codes, scales and cache contents are theirs bit for bit. seq_lens must count the
 * new token (positions[b] + 1 in a plain decode step). */
W8A8_API int w8a8_qkv_attention_decode(w8a8_ctx* ctx, const void* qkv, const void* q_norm_w,
                              const void* k_norm_w, float eps, const float* freqs, const int* positions,
                              void* k_cache, void* v_cache, const int* block_table, const int* seq_lens,
                              void* out, int batch, int n_heads, int head_dim, int max_blocks_per_seq,
                              float sm_scale, int layer, int n_layers, int n_kv_heads, int quant_group_size,
                              void* Xq, void* Xs, int context_splits, void* stream);

/* ---- one decode step of the whole stack as one launch ------------------------------------------ */

typedef struct w8a8_decode_layer {
    const void* attn_norm; /* fp16 [dim] */
    const void* ffn_norm;  /* fp16 [dim] */
    const void* q_norm;    /* fp16 [head_dim], NULL = no qk-norm */
    const void* k_norm;
    const void* packed[4]; /* images made by w8a8_pack_weight of: wqkv [(n_q + 2 n_kv) * head_dim, dim];
                              wo [dim, n_q * head_dim]; w1/w3 interleaved by w8a8_pack_gate_up
                              [2 * inter, dim]; w2 [dim, inter] */
} w8a8_decode_layer;

typedef struct w8a8_decode_stack {
    int n_layers, batch, dim, n_q_heads, n_kv_heads, head_dim, inter, group_size;
    float eps, sm_scale;
    const w8a8_decode_layer* layers; /* DEVICE array [n_layers] */
    const void* final_norm;          /* fp16 [dim] */
    const float* rope_freqs;         /* device fp32 [head_dim / 2] */
    const int* positions;            /* device int32 [batch]: position of the new token */
    const int* seq_lens;             /* device int32 [batch]: tokens to attend over, the new one included */
    const int* block_table;          /* device int32 [batch, max_blocks_per_seq] */
    int max_blocks_per_seq;
    void* k_cache;                   /* fp16 [blocks, n_layers, n_kv, 16, head_dim] */
    void* v_cache;
    void* x;   /* fp16 [batch, dim]: in = embeddings of the new tokens; left holding the residual stream */
    void* out; /* fp16 [batch, dim]: the final-normed hidden state */
} w8a8_decode_stack;

/* Scratch the step needs inside the context's workspace (0 = the shape is not supported). */
W8A8_API size_t w8a8_decode_stack_workspace_bytes(const w8a8_decode_stack* stack);

/* Replaces the layer loop of DualAREngine::decode_step (src/engine/dual_ar_engine.cc:560-665; LM head
 * and sampling excluded) for batch <= 8 on one GPU: per layer residual add + RMSNorm + quantiser, wqkv,
 * qk-norm + RoPE + KV write, paged attention, wo, residual add + RMSNorm + quantiser, fused gate/up with
 * SwiGLU, quantiser, w2 — then the final norm. One persistent cooperative launch (a CTA per SM) whose
 * warps stream the weights of all linears without interruption; phases are separated by grid
 * barriers with bounded waits (W8A8_ERR_TIMEOUT through w8a8_check_device_status when one runs out).
 * The arithmetic is that of this library's separate calls: int8 codes, scales and int32 group sums are
 * the same; a linear's fp32 partial sums are grouped differently (its row tiles are shared by one CTA per
 * SM here, by up to two in a separate call), so its fp16 outputs may differ from the separate calls' in
 * the last bit. The
 * descriptor is read on the host during the call; `layers` must stay valid on the device until the
 * step has run. */
W8A8_API int w8a8_decode_stack_step(w8a8_ctx* ctx, const w8a8_decode_stack* stack, void* stream);

/* Diagnostic: the device-side timeline of the last w8a8_decode_stack_step on this context. CTA 0 stamps the
 * GPU's nanosecond timer at the start, after each of the nine phases of a layer and after each of the nine
 * grid barriers, and after the final norm: 18 * n_layers + 2 stamps, copied to host memory (synchronises the
 * stream). Returns the number of stamps, or minus a status code. */
W8A8_API int w8a8_decode_stack_timeline(w8a8_ctx* ctx, const w8a8_decode_stack* stack,
                               unsigned long long* stamps_out, int capacity, void* stream);

/* ---- tensor parallelism (no counterpart in the reference, which is single-GPU) ------------- */

/* Row-parallel projections (wo, w2 with K cut at quantisation-group boundaries) leave a partial [M, dim] on every
 * rank; their sum is the projection's output. The exchange is a one-shot all-reduce over NVLink peer memory, split
 * between the two kernels around it:
 *   w8a8_tp_linear_q   is w8a8_linear_q whose output, instead of Y, is its fp32 partial sent tile by tile, from the
 *                      kernel's epilogue, into every rank's exchange buffer (plain peer stores of self-validating
 *                      {value, epoch} words: no fence, no flag, the transfer overlaps the rest of the kernel). Needs a
 *                      weight registered with w8a8_register_packed_weight, M <= 32, no epilogue.
 *   w8a8_tp_allreduce_rmsnorm_quantize   is w8a8_rmsnorm_quantize whose residual is the SUM of all ranks' partials:
 *                      it waits (bounded; W8A8_ERR_TIMEOUT through w8a8_check_device_status) for every rank's words
 *                      in its OWN buffer, adds them in rank order in fp32, rounds once to fp16, adds that to x in place
 *                      and continues with RMSNorm (weight == NULL: none) and the quantiser (Xq == NULL: none).
 *                      partial == NULL: the partials were sent by w8a8_tp_linear_q. partial != NULL (fp16 [M, K], e.g.
 *                      the output of a plain w8a8_linear_q): the kernel sends it itself first. smooth_inv / act_scale
 *                      must be NULL and act_mode W8A8_ACT_PER_TOKEN_GROUP; K % 256 == 0, K <= 4096.
 * Every rank adds the same values in the same order, so all ranks end with the same bits; against one GPU the sum
 * differs only by the association of fp32 additions (with partial != NULL: by one fp16 rounding per rank as well).
 * Set-up, once per process: w8a8_tp_create allocates the exchange buffer for at most max_tokens rows of `dim` and
 * returns a 64-byte CUDA IPC handle; the host gathers all ranks' handles (any transport) and passes the world*64
 * bytes, in rank order, to w8a8_tp_connect (NULL = loop-back onto this rank's own buffer: the other ranks' rows then
 * never arrive, which is what the time-out test uses). One process per GPU, world <= 8. */
W8A8_API int w8a8_tp_create(w8a8_ctx* ctx, int rank, int world, int max_tokens, int dim, void* ipc_handle_out);
W8A8_API int w8a8_tp_connect(w8a8_ctx* ctx, const void* all_ipc_handles);
W8A8_API int w8a8_tp_linear_q(w8a8_ctx* ctx, const void* W, const void* w_scale, int group_size, const void* Xq,
                     const void* Xs, int M, int N, int K, const w8a8_linear_opts* opts, void* stream);
W8A8_API int w8a8_tp_allreduce_rmsnorm_quantize(w8a8_ctx* ctx, void* x, const void* partial, const void* weight,
                                       float eps, const void* smooth_inv, const void* act_scale, int M,
                                       int K, int group_size, int act_mode, void* normed_out, void* Xq,
                                       void* Xs, void* stream);

/* Decode-time weight layout. The reference uploads each weight as it lies in the container
 * (src/engine/dual_ar_engine.cc:231-278) and keys its quantisation metadata by the device pointer
 * (:275). A loader built on this library does one more step per weight: it packs the row-major
 * matrix and its scales into one linear stream in the order the M <= 32 kernel consumes it
 * (blocks of 16 rows x 256 K-bytes, each followed by its scales), and registers the pair. From
 * then on w8a8_linear / w8a8_linear_q with that W pointer and M <= 32 stream the packed image;
 * larger M keeps reading the row-major matrix (which TMA feeds to the tensor cores as it is).
 * w8a8_packed_weight_bytes returns 0 for shapes that cannot be packed (needs K % 256 == 0 and a
 * group size of 64, 128 or a multiple of 256); such weights simply stay unpacked. */
W8A8_API size_t w8a8_packed_weight_bytes(int N, int K, int group_size);
W8A8_API int w8a8_pack_weight(w8a8_ctx* ctx, const void* W, const void* w_scale, int N, int K,
                     int group_size, void* packed_out, void* stream);
/* Registers the image `packed` (made by w8a8_pack_weight for exactly this N, K, group_size) under the
 * raw weight pointer W. The image is used only by calls whose N, K and group size equal the registered
 * ones: should W be freed and its address reused for another tensor before the entry is removed, a call
 * with another shape falls back to the row-major kernels instead of streaming a stale image. Remove the
 * entry (packed == NULL; N, K, group_size ignored) before freeing either buffer. */
W8A8_API int w8a8_register_packed_weight(w8a8_ctx* ctx, const void* W, const void* packed, int N, int K,
                                int group_size);

/* Pre-pack for W8A8_EPI_SWIGLU: interleaves w1 (gate) and w3 (up), both int8 [inter, K] with
 * fp16 scales [inter, G], into W_out int8 [2*inter, K] / scale_out fp16 [2*inter, G] in blocks
 * of 16 rows = 8 gate rows then the 8 up rows of the same channels. inter % 8 == 0. The
 * reference keeps w1 and w3 apart and runs two GEMMs (src/engine/dual_ar_engine.cc:640-643);
 * this is what its loader loop (dual_ar_engine.cc:231-278) would call once per layer. */
W8A8_API int w8a8_pack_gate_up(w8a8_ctx* ctx, const void* w_gate, const void* s_gate, const void* w_up,
                      const void* s_up, int inter, int K, int G, void* W_out, void* scale_out,
                      void* stream);

#ifdef __cplusplus
}
#endif
#endif /* W8A8_H */
