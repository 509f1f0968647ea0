/*
 * CPU oracle for the INT8 W8A8 linear path — TEST INFRASTRUCTURE, NOT PRODUCT.
 * See w8a8_oracle.h.  Every function cites the reference lines it restates.
 * Compile with -O2 -ffp-contract=off so that no multiply-add is fused unless
 * fmaf() is written out.
 */
#include "w8a8_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <pthread.h>
#include <unistd.h>

/* ---- a minimal pthread parallel-for (no OpenMP runtime is assumed) ------- */

typedef void (*range_fn)(int begin, int end, void* ctx);
typedef struct { range_fn fn; void* ctx; int begin, end; } range_job;

static void* range_thread(void* p) {
    range_job* j = (range_job*)p;
    j->fn(j->begin, j->end, j->ctx);
    return NULL;
}

static int host_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n < 1 ? 1 : (n > 256 ? 256 : (int)n);
}

int w8a8o_host_threads(void) { return host_threads(); }

static void parallel_for(int n, int threads, range_fn fn, void* ctx) {
    if (threads <= 0) threads = host_threads();
    if (threads > 256) threads = 256;
    if (threads > n) threads = n;
    if (threads <= 1) { fn(0, n, ctx); return; }
    pthread_t tid[256];
    int live[256];
    range_job job[256];
    int chunk = (n + threads - 1) / threads, started = 0;
    for (int t = 0; t < threads; ++t) {
        job[t].fn = fn; job[t].ctx = ctx;
        job[t].begin = t * chunk;
        job[t].end = (t + 1) * chunk < n ? (t + 1) * chunk : n;
        if (job[t].begin >= job[t].end) break;
        live[t] = pthread_create(&tid[t], NULL, range_thread, &job[t]) == 0;
        if (!live[t]) fn(job[t].begin, job[t].end, ctx); /* no thread to be had: run inline */
        started = t + 1;
    }
    for (int t = 0; t < started; ++t)
        if (live[t]) pthread_join(tid[t], NULL);
}

/* ---- fp16 <-> fp32 (IEEE binary16, round-to-nearest-even) ---------------- */

float w8a8o_half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t w8a8o_float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | (ax > 0x7f800000u ? 0x200u : 0));
    if (ax >= 0x477ff000u) /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    if (ax < 0x33000001u) /* <= 2^-25 -> 0 (tie at exactly 2^-25 rounds to even = 0) */
        return sign;
    int e = (int)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7fffffu) | 0x800000u;
    int shift = (e < -14) ? (13 + (-14 - e)) : 13; /* bits dropped */
    uint32_t kept = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (kept & 1u))) ++kept;
    uint32_t out;
    if (e < -14) {
        out = kept; /* subnormal; carry into exponent field is the right answer */
    } else {
        out = ((uint32_t)(e + 15) << 10) + (kept - 0x400u); /* carry propagates into exponent */
    }
    return (uint16_t)(sign | out);
}

int w8a8o_num_groups(int K, int group_size) {
    if (group_size <= 0 || group_size > K) group_size = K; /* int8_gemm.cu:396 */
    return (K + group_size - 1) / group_size;              /* int8_gemm.cu:397 */
}

static int norm_group(int K, int group_size) {
    return (group_size <= 0 || group_size > K) ? K : group_size;
}

/* __float2int_rn followed by the clamp of int8_gemm.cu:207-208. */
static int8_t round_clamp(float r) {
    if (r != r) return 0; /* NaN converts to 0 */
    if (r >= 127.0f) return 127;
    if (r <= -127.0f) return -127;
    return (int8_t)lrintf(r); /* default rounding mode: nearest-even */
}

/* int8_gemm.cu:147-211. One (token, group) at a time; absmax is order-free. */
int w8a8o_quantize(const uint16_t* X, const uint16_t* smooth_inv,
                   const uint16_t* act_scale, int M, int K, int group_size,
                   int act_mode, int8_t* Xq, float* Xs) {
    if (M < 0 || K <= 0) return 1;
    int g = norm_group(K, group_size);
    int G = (K + g - 1) / g;
    for (int m = 0; m < M; ++m) {
        const uint16_t* xr = X + (size_t)m * K;
        float row_scale = 0.0f;
        if (act_mode == W8A8O_ACT_PER_TOKEN && !act_scale) {
            float amax = 0.0f;
            for (int k = 0; k < K; ++k) {
                float v = w8a8o_half_to_float(xr[k]);
                if (smooth_inv) v *= w8a8o_half_to_float(smooth_inv[k]);
                amax = fmaxf(amax, fabsf(v));
            }
            row_scale = amax / 127.0f;
            if (row_scale < 1e-8f) row_scale = 1e-8f;
        }
        for (int j = 0; j < G; ++j) {
            int start = j * g;
            int end = start + g < K ? start + g : K;
            float scale;
            if (act_scale) { /* :171-176 */
                scale = w8a8o_half_to_float(act_scale[j]);
                if (scale < 1e-8f) scale = 1e-8f;
            } else if (act_mode == W8A8O_ACT_PER_TOKEN) {
                scale = row_scale;
            } else { /* :177-199 */
                float amax = 0.0f;
                for (int k = start; k < end; ++k) {
                    float v = w8a8o_half_to_float(xr[k]);
                    if (smooth_inv) v *= w8a8o_half_to_float(smooth_inv[k]);
                    amax = fmaxf(amax, fabsf(v));
                }
                scale = amax / 127.0f;
                if (scale < 1e-8f) scale = 1e-8f;
            }
            Xs[(size_t)m * G + j] = scale;
            float inv = 1.0f / scale; /* :201 */
            for (int k = start; k < end; ++k) {
                float v = w8a8o_half_to_float(xr[k]);
                if (smooth_inv) v *= w8a8o_half_to_float(smooth_inv[k]);
                Xq[(size_t)m * K + k] = round_clamp(v * inv); /* :206-209 */
            }
        }
    }
    return 0;
}

typedef struct { const int8_t* W; const int8_t* Xq; int M, N, K, g, G; int32_t* P; } gs_ctx;

static void group_sums_rows(int n0, int n1, void* p) {
    const gs_ctx* c = (const gs_ctx*)p;
    for (int n = n0; n < n1; ++n) {
        const int8_t* wr = c->W + (size_t)n * c->K;
        for (int m = 0; m < c->M; ++m) {
            const int8_t* xr = c->Xq + (size_t)m * c->K;
            for (int j = 0; j < c->G; ++j) {
                int start = j * c->g;
                int end = start + c->g < c->K ? start + c->g : c->K;
                int32_t s = 0;
                for (int k = start; k < end; ++k) s += (int32_t)wr[k] * (int32_t)xr[k];
                c->P[((size_t)m * c->N + n) * c->G + j] = s;
            }
        }
    }
}

/* The integer GEMM of int8_gemm.cu:470-490, one group at a time. */
int w8a8o_group_sums(const int8_t* W, const int8_t* Xq, int M, int N, int K,
                     int group_size, int32_t* P) {
    gs_ctx c = {W, Xq, M, N, K, norm_group(K, group_size), 0, P};
    c.G = (K + c.g - 1) / c.g;
    parallel_for(N, 0, group_sums_rows, &c);
    return 0;
}

static inline float promote_step(float acc, int32_t p, float ws, float xs, int promote) {
    float t = (float)p * ws; /* int8_gemm.cu:233, left-to-right */
    if (promote == W8A8O_PROMOTE_FMA) return fmaf(t, xs, acc);
    float u = t * xs;
    return acc + u;
}

static void linear_rows(const int8_t* W, const uint16_t* w_scale, const int8_t* Xq,
                        const float* Xs, int M, int N, int K, int g, int G,
                        int promote, int n0, int n1, uint16_t* Yh, float* Yf32,
                        double* Yf64) {
    for (int n = n0; n < n1; ++n) {
        const int8_t* wr = W + (size_t)n * K;
        for (int m = 0; m < M; ++m) {
            const int8_t* xr = Xq + (size_t)m * K;
            float acc = 0.0f; /* memset of int8_gemm.cu:423-432 */
            double acc64 = 0.0;
            for (int j = 0; j < G; ++j) {
                int start = j * g;
                int end = start + g < K ? start + g : K;
                int32_t s = 0;
                for (int k = start; k < end; ++k) s += (int32_t)wr[k] * (int32_t)xr[k];
                /* scale indexing: [N] when G == 1, else [N,G] (:225-227) */
                float ws = w8a8o_half_to_float(G == 1 ? w_scale[n] : w_scale[(size_t)n * G + j]);
                float xs = Xs[(size_t)m * G + j];
                acc = promote_step(acc, s, ws, xs, promote);
                acc64 += (double)s * (double)ws * (double)xs;
            }
            size_t o = (size_t)m * N + n;
            if (Yh) Yh[o] = w8a8o_float_to_half(acc); /* :236-243 */
            if (Yf32) Yf32[o] = acc;
            if (Yf64) Yf64[o] = acc64;
        }
    }
}

typedef struct {
    const int8_t* W; const uint16_t* w_scale; const int8_t* Xq; const float* Xs;
    int M, N, K, g, G, promote; uint16_t* Yh; float* Yf32; double* Yf64;
} lin_ctx;

static void linear_range(int n0, int n1, void* p) {
    const lin_ctx* c = (const lin_ctx*)p;
    linear_rows(c->W, c->w_scale, c->Xq, c->Xs, c->M, c->N, c->K, c->g, c->G, c->promote, n0, n1,
                c->Yh, c->Yf32, c->Yf64);
}

int w8a8o_linear_q(const int8_t* W, const uint16_t* w_scale, const int8_t* Xq,
                   const float* Xs, int M, int N, int K, int group_size,
                   int promote, uint16_t* Yh, float* Yf32, double* Yf64) {
    if (M < 0 || N <= 0 || K <= 0) return 1;
    int g = norm_group(K, group_size);
    int G = (K + g - 1) / g;
    lin_ctx c = {W, w_scale, Xq, Xs, M, N, K, g, G, promote, Yh, Yf32, Yf64};
    parallel_for(N, 0, linear_range, &c);
    return 0;
}

static float silu_f(float v) { return v / (1.0f + expf(-v)); } /* ffn_activations.cu:15-16 */

int w8a8o_linear(const int8_t* W, const uint16_t* w_scale, int group_size,
                 const uint16_t* act_scale, const uint16_t* smooth_inv,
                 const uint16_t* X, int M, int N, int K, int act_mode,
                 int promote, int epilogue, const uint16_t* R, uint16_t* Y) {
    if (M < 0 || N <= 0 || K <= 0) return 1;
    if (epilogue == W8A8O_EPI_SWIGLU && (N % 16)) return 1;
    if (epilogue == W8A8O_EPI_RESIDUAL && !R) return 1;
    int G = w8a8o_num_groups(K, group_size);
    int8_t* Xq = (int8_t*)malloc((size_t)(M > 0 ? M : 1) * K);
    float* Xs = (float*)malloc(sizeof(float) * (size_t)(M > 0 ? M : 1) * G);
    uint16_t* T = (epilogue == W8A8O_EPI_NONE)
                      ? Y
                      : (uint16_t*)malloc(sizeof(uint16_t) * (size_t)(M > 0 ? M : 1) * N);
    if (!Xq || !Xs || !T) return 2;
    int rc = w8a8o_quantize(X, smooth_inv, act_scale, M, K, group_size, act_mode, Xq, Xs);
    if (!rc) rc = w8a8o_linear_q(W, w_scale, Xq, Xs, M, N, K, group_size, promote, T, NULL, NULL);
    if (!rc && epilogue == W8A8O_EPI_RESIDUAL) {
        for (size_t i = 0; i < (size_t)M * N; ++i) /* ffn_activations.cu:41-45 */
            Y[i] = w8a8o_float_to_half(w8a8o_half_to_float(T[i]) + w8a8o_half_to_float(R[i]));
    } else if (!rc && epilogue == W8A8O_EPI_SWIGLU) {
        int H = N / 2;
        for (int m = 0; m < M; ++m)
            for (int c = 0; c < H; ++c) {
                int blk = c / 8, i = c % 8; /* rows 16*blk+i = gate, 16*blk+8+i = up */
                float gt = w8a8o_half_to_float(T[(size_t)m * N + 16 * blk + i]);
                float up = w8a8o_half_to_float(T[(size_t)m * N + 16 * blk + 8 + i]);
                uint16_t s16 = w8a8o_float_to_half(silu_f(gt));
                Y[(size_t)m * H + c] = w8a8o_float_to_half(w8a8o_half_to_float(s16) * up);
            }
    }
    free(Xq);
    free(Xs);
    if (T != Y) free(T);
    return rc;
}

/* rms_norm.cu:10-58. The sum is carried in double here: the device sums fp32
 * partials in a tree, so neither order is "the" fp32 answer; tests compare the
 * device against this at 1 fp16 ulp. */
int w8a8o_rms_norm(const uint16_t* x, const uint16_t* w, uint16_t* out,
                   int tokens, int dim, float eps) {
    if (tokens < 0 || dim <= 0) return 1;
    for (int t = 0; t < tokens; ++t) {
        const uint16_t* xr = x + (size_t)t * dim;
        double ss = 0.0;
        for (int i = 0; i < dim; ++i) {
            double v = w8a8o_half_to_float(xr[i]);
            ss += v * v;
        }
        float r = (float)(1.0 / sqrt((double)((float)ss / (float)dim + eps)));
        for (int i = 0; i < dim; ++i) {
            float v = w8a8o_half_to_float(xr[i]) * r; /* :53 */
            out[(size_t)t * dim + i] = w8a8o_float_to_half(v * w8a8o_half_to_float(w[i])); /* :55 */
        }
    }
    return 0;
}

int w8a8o_silu(uint16_t* a, long n) {
    for (long i = 0; i < n; ++i) a[i] = w8a8o_float_to_half(silu_f(w8a8o_half_to_float(a[i])));
    return 0;
}

int w8a8o_mul(uint16_t* a, const uint16_t* b, long n) { /* ffn_activations.cu:35-39 */
    for (long i = 0; i < n; ++i)
        a[i] = w8a8o_float_to_half(w8a8o_half_to_float(a[i]) * w8a8o_half_to_float(b[i]));
    return 0;
}

int w8a8o_residual_add(uint16_t* a, const uint16_t* b, long n) { /* ffn_activations.cu:41-45 */
    for (long i = 0; i < n; ++i)
        a[i] = w8a8o_float_to_half(w8a8o_half_to_float(a[i]) + w8a8o_half_to_float(b[i]));
    return 0;
}

double w8a8o_timed_linear(const int8_t* W, const uint16_t* w_scale, int group_size,
                          const uint16_t* X, int M, int N, int K, int n_rows,
                          int threads, uint16_t* Y) {
    if (M <= 0 || N <= 0 || K <= 0 || n_rows <= 0 || n_rows > N) return -1.0;
    int g = norm_group(K, group_size);
    int G = (K + g - 1) / g;
    int8_t* Xq = (int8_t*)malloc((size_t)M * K);
    float* Xs = (float*)malloc(sizeof(float) * (size_t)M * G);
    if (!Xq || !Xs) return -1.0;
    struct timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    w8a8o_quantize(X, NULL, NULL, M, K, group_size, W8A8O_ACT_PER_TOKEN_GROUP, Xq, Xs);
    lin_ctx c = {W, w_scale, Xq, Xs, M, N, K, g, G, W8A8O_PROMOTE_FMA, Y, NULL, NULL};
    parallel_for(n_rows, threads, linear_range, &c);
    clock_gettime(CLOCK_MONOTONIC, &t1);
    free(Xq);
    free(Xs);
    return (double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec);
}
