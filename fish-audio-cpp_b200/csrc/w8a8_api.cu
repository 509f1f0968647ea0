// C ABI of libw8a8 (see include/w8a8.h): argument checks, kernel choice, scratch layout.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <new>
#include <unordered_map>

#include "w8a8_internal.h"

struct w8a8_ctx {
    int device = 0;
    unsigned char* workspace = nullptr;
    size_t workspace_bytes = 0;
    int* device_status = nullptr;  // set by kernels whose bounded waits run out
    void* splitk_partials = nullptr;  // per-warp fp32 partial tiles of the stream-K GEMV
    int* splitk_counters = nullptr;   // one arrival counter per 16-row tile, zero between launches
    // raw weight pointer -> its packed image; filled by the loader (w8a8_register_packed_weight), the
    // same pointer-keyed lookup as DualAREngine::weight_quant_meta_ (src/engine/dual_ar_engine.h:105)
    struct PackedEntry {
        const void* image;
        int N, K, g;  // the shape the image was packed for: a call with another shape must not stream it
    };
    std::unordered_map<const void*, PackedEntry> packed;
    std::mutex packed_mu;
    int* tail_counters = nullptr;     // arrival counters of the decode kernel's tails, zero between launches
    w8a8::TpState* tp = nullptr;  // tensor-parallel exchange, when w8a8_tp_create was called
};

static constexpr size_t kSplitkPartialBytes = size_t(16) << 20;
static constexpr size_t kSplitkCounters = size_t(1) << 18;

namespace w8a8 {

static thread_local char g_error[512] = "";

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return status;
}

bool pdl_enabled(int kernel_class) {
    static const int mask = [] {
        const char* off = std::getenv("W8A8_NO_PDL");
        if (off && *off && *off != '0') return 0;
        const char* v = std::getenv("W8A8_PDL");
        return v && *v ? std::atoi(v) : kPdlDefaultMask;
    }();
    return (mask & kernel_class) != 0;
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return W8A8_OK;
}

static inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

static size_t quant_scratch_bytes(int M, int K, int group_size) {
    return align256(static_cast<size_t>(M) * K) + align256(static_cast<size_t>(M) * num_groups(K, group_size) * 4);
}


static int check_linear_common(const w8a8_ctx* ctx, const void* W, const void* w_scale, const void* Y,
                               int M, int N, int K, const w8a8_linear_opts* o) {
    if (!ctx) return fail(W8A8_ERR_INVALID_ARG, "null context");
    if (M < 0 || N <= 0 || K <= 0) return fail(W8A8_ERR_INVALID_ARG, "bad shape M=%d N=%d K=%d", M, N, K);
    if (!W || !w_scale || (!Y && M > 0)) return fail(W8A8_ERR_INVALID_ARG, "null W, w_scale or Y");
    if (o) {
        if (o->epilogue < W8A8_EPI_NONE || o->epilogue > W8A8_EPI_SWIGLU)
            return fail(W8A8_ERR_INVALID_ARG, "unknown epilogue %d", o->epilogue);
        if (o->epilogue == W8A8_EPI_RESIDUAL && !o->residual)
            return fail(W8A8_ERR_INVALID_ARG, "W8A8_EPI_RESIDUAL needs opts->residual");
        if (o->epilogue == W8A8_EPI_SWIGLU && N % 16 != 0)
            return fail(W8A8_ERR_INVALID_ARG, "W8A8_EPI_SWIGLU needs N %% 16 == 0 (got %d)", N);
        if (o->act_mode != W8A8_ACT_PER_TOKEN_GROUP && o->act_mode != W8A8_ACT_PER_TOKEN)
            return fail(W8A8_ERR_INVALID_ARG, "unknown act_mode %d", o->act_mode);
        if (o->kernel < W8A8_KERNEL_AUTO || o->kernel > W8A8_KERNEL_GEMM_PAIR)
            return fail(W8A8_ERR_INVALID_ARG, "unknown kernel %d", o->kernel);
    }
    return W8A8_OK;
}

static LinearArgs make_args(const void* W, const void* w_scale, int group_size, void* Y, int M, int N, int K,
                            const w8a8_linear_opts* o) {
    LinearArgs a = {};
    a.W = static_cast<const int8_t*>(W);
    a.w_scale = static_cast<const __half*>(w_scale);
    a.Y = static_cast<__half*>(Y);
    a.M = M;
    a.N = N;
    a.K = K;
    a.g = norm_group(K, group_size);
    a.G = num_groups(K, group_size);
    a.epilogue = o ? o->epilogue : W8A8_EPI_NONE;
    a.residual = o ? static_cast<const __half*>(o->residual) : nullptr;
    a.dump = o ? o->dump_group_sums : nullptr;
    a.split_k = o ? o->split_k : 0;
    return a;
}

// Runs a linear whose codes and scales exist.
int dispatch_linear_q(const LinearArgs& a, int kernel, int* device_status, cudaStream_t s) {
    if (a.M == 0) return W8A8_OK;
    switch (kernel) {
        case W8A8_KERNEL_GENERIC: return launch_linear_generic(a, s);
        case W8A8_KERNEL_GEMV: return launch_linear_gemv(a, s);
        case W8A8_KERNEL_GEMM: return launch_linear_gemm(a, device_status, s);
        case W8A8_KERNEL_GEMM_SINGLE: return launch_linear_gemm(a, device_status, s, 0);
        case W8A8_KERNEL_GEMM_PAIR: return launch_linear_gemm(a, device_status, s, 1);
        case W8A8_KERNEL_GEMV_TMA: return launch_linear_gemv_tma(a, device_status, s);
        case W8A8_KERNEL_GEMV_PACKED: return launch_linear_gemv_packed(a, device_status, s);
        default: break;
    }
    if (a.M <= 32 && gemv_packed_supports(a)) return launch_linear_gemv_packed(a, device_status, s);
    if (a.M <= 32 && gemv_tma_supports(a)) return launch_linear_gemv_tma(a, device_status, s);
    if (a.M <= 32 && gemv_supports(a)) return launch_linear_gemv(a, s);
    if (gemm_supports(a)) return launch_linear_gemm(a, device_status, s);
    return launch_linear_generic(a, s);
}

// Points the arguments at the context's split-K scratch and at the packed image of the weight, if registered.
static void fill_scratch(w8a8_ctx* ctx, LinearArgs& a) {
    a.splitk_partials = ctx->splitk_partials;
    a.splitk_partial_bytes = kSplitkPartialBytes;
    a.splitk_counters = ctx->splitk_counters;
    a.splitk_counter_count = kSplitkCounters;
    a.tail_counters = ctx->tail_counters;
    if (a.M <= 32 && !ctx->packed.empty()) {
        std::lock_guard<std::mutex> lock(ctx->packed_mu);
        auto it = ctx->packed.find(a.W);
        // A pointer may outlive its registration (the caller freed the weight and the allocator handed the
        // address to another tensor): the image is used only for the shape it was packed for.
        if (it != ctx->packed.end() && it->second.N == a.N && it->second.K == a.K && it->second.g == a.g)
            a.packed = it->second.image;
    }
}

static int dispatch_q(w8a8_ctx* ctx, const LinearArgs& args, int kernel, cudaStream_t s) {
    LinearArgs a = args;
    fill_scratch(ctx, a);
    return dispatch_linear_q(a, kernel, ctx->device_status, s);
}

}  // namespace w8a8

using namespace w8a8;

extern "C" {

const char* w8a8_status_string(int status) {
    switch (status) {
        case W8A8_OK: return "ok";
        case W8A8_ERR_INVALID_ARG: return "invalid argument";
        case W8A8_ERR_UNSUPPORTED: return "unsupported shape";
        case W8A8_ERR_CUDA: return "CUDA error";
        case W8A8_ERR_TIMEOUT: return "device-side wait timed out";
        case W8A8_ERR_WORKSPACE: return "context workspace too small";
    }
    return "unknown status";
}

const char* w8a8_last_error(void) { return g_error; }

int w8a8_create(w8a8_ctx** out, int device, size_t workspace_bytes) {
    if (!out) return fail(W8A8_ERR_INVALID_ARG, "null out");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(W8A8_ERR_CUDA, "no CUDA device: %s", cudaGetErrorString(e));
    }
    if (device < 0 || device >= count) return fail(W8A8_ERR_INVALID_ARG, "device %d of %d", device, count);
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (prop.major != 10)
        return fail(W8A8_ERR_UNSUPPORTED, "built for sm_100a only; device %d is sm_%d%d", device, prop.major,
                    prop.minor);
    int prev = 0;
    cudaGetDevice(&prev);
    if ((e = cudaSetDevice(device)) != cudaSuccess)
        return fail(W8A8_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
    w8a8_ctx* c = new (std::nothrow) w8a8_ctx;
    if (!c) return fail(W8A8_ERR_CUDA, "out of host memory");
    c->device = device;
    if (workspace_bytes == 0) workspace_bytes = quant_scratch_bytes(8192, 9728, 64);
    c->workspace_bytes = align256(workspace_bytes);
    e = cudaMalloc(&c->workspace, c->workspace_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&c->device_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(c->device_status, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&c->splitk_partials, kSplitkPartialBytes);
    if (e == cudaSuccess) e = cudaMalloc(&c->splitk_counters, kSplitkCounters * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(c->splitk_counters, 0, kSplitkCounters * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&c->tail_counters, kTailCounterInts * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(c->tail_counters, 0, kTailCounterInts * sizeof(int));
    cudaSetDevice(prev);
    if (e != cudaSuccess) {
        cudaFree(c->workspace);
        cudaFree(c->device_status);
        cudaFree(c->splitk_partials);
        cudaFree(c->splitk_counters);
        cudaFree(c->tail_counters);
        delete c;
        return fail(W8A8_ERR_CUDA, "context allocation: %s", cudaGetErrorString(e));
    }
    *out = c;
    return W8A8_OK;
}

int w8a8_destroy(w8a8_ctx* ctx) {
    if (!ctx) return W8A8_OK;
    cudaFree(ctx->workspace);
    cudaFree(ctx->device_status);
    cudaFree(ctx->splitk_partials);
    cudaFree(ctx->splitk_counters);
    cudaFree(ctx->tail_counters);
    tp_destroy(ctx->tp);
    delete ctx;
    return W8A8_OK;
}

size_t w8a8_workspace_bytes(int M, int N, int K, int group_size) {
    (void)N;
    if (M <= 0 || K <= 0) return 0;
    return quant_scratch_bytes(M, K, group_size);
}

size_t w8a8_ctx_workspace_bytes(const w8a8_ctx* ctx) { return ctx ? ctx->workspace_bytes : 0; }

int w8a8_check_device_status(w8a8_ctx* ctx, void* stream) {
    if (!ctx) return fail(W8A8_ERR_INVALID_ARG, "null context");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int host = 0;
    cudaError_t e = cudaMemcpyAsync(&host, ctx->device_status, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "status read: %s", cudaGetErrorString(e));
    if (host != 0) {
        cudaMemsetAsync(ctx->device_status, 0, sizeof(int), s);
        // a kernel that gave up may have left arrival counters half-counted
        cudaMemsetAsync(ctx->tail_counters, 0, kTailCounterInts * sizeof(int), s);
        return fail(W8A8_ERR_TIMEOUT, "a kernel gave up a bounded wait (code %d)", host);
    }
    return W8A8_OK;
}

int w8a8_quantize(w8a8_ctx* ctx, const void* X, const void* smooth_inv, const void* act_scale, int M, int K,
                  int group_size, int act_mode, void* Xq, void* Xs, void* stream) {
    if (!ctx) return fail(W8A8_ERR_INVALID_ARG, "null context");
    if (M < 0 || K <= 0) return fail(W8A8_ERR_INVALID_ARG, "bad shape M=%d K=%d", M, K);
    if (M > 0 && (!X || !Xq || !Xs)) return fail(W8A8_ERR_INVALID_ARG, "null X, Xq or Xs");
    if (act_mode != W8A8_ACT_PER_TOKEN_GROUP && act_mode != W8A8_ACT_PER_TOKEN)
        return fail(W8A8_ERR_INVALID_ARG, "unknown act_mode %d", act_mode);
    return launch_rowquant(static_cast<const __half*>(X), nullptr, nullptr, nullptr, 0.0f,
                           static_cast<const __half*>(smooth_inv), static_cast<const __half*>(act_scale), M, K,
                           group_size, act_mode, nullptr, static_cast<int8_t*>(Xq), static_cast<float*>(Xs),
                           static_cast<cudaStream_t>(stream));
}

int w8a8_rms_norm(w8a8_ctx* ctx, const void* x, const void* weight, void* out, int tokens, int dim, float eps,
                  void* stream) {
    if (!ctx) return fail(W8A8_ERR_INVALID_ARG, "null context");
    if (tokens < 0 || dim <= 0) return fail(W8A8_ERR_INVALID_ARG, "bad shape tokens=%d dim=%d", tokens, dim);
    if (tokens > 0 && (!x || !weight || !out)) return fail(W8A8_ERR_INVALID_ARG, "null x, weight or out");
    return launch_rowquant(static_cast<const __half*>(x), nullptr, nullptr, static_cast<const __half*>(weight), eps,
                           nullptr, nullptr, tokens, dim, dim, W8A8_ACT_PER_TOKEN_GROUP, static_cast<__half*>(out),
                           nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

int w8a8_rmsnorm_quantize(w8a8_ctx* ctx, void* x, const void* residual, const void* weight, float eps,
                          const void* smooth_inv, const void* act_scale, int M, int K, int group_size,
                          int act_mode, void* normed_out, void* Xq, void* Xs, void* stream) {
    if (!ctx) return fail(W8A8_ERR_INVALID_ARG, "null context");
    if (M < 0 || K <= 0) return fail(W8A8_ERR_INVALID_ARG, "bad shape M=%d K=%d", M, K);
    if (M > 0 && (!x || !weight || !Xq || !Xs)) return fail(W8A8_ERR_INVALID_ARG, "null x, weight, Xq or Xs");
    if (act_mode != W8A8_ACT_PER_TOKEN_GROUP && act_mode != W8A8_ACT_PER_TOKEN)
        return fail(W8A8_ERR_INVALID_ARG, "unknown act_mode %d", act_mode);
    return launch_rowquant(static_cast<const __half*>(x), static_cast<__half*>(x),
                           static_cast<const __half*>(residual), static_cast<const __half*>(weight), eps,
                           static_cast<const __half*>(smooth_inv), static_cast<const __half*>(act_scale), M, K,
                           group_size, act_mode, static_cast<__half*>(normed_out), static_cast<int8_t*>(Xq),
                           static_cast<float*>(Xs), static_cast<cudaStream_t>(stream));
}

int w8a8_silu(w8a8_ctx* ctx, void* a, long n, void* stream) {
    if (!ctx || (n > 0 && !a) || n < 0) return fail(W8A8_ERR_INVALID_ARG, "silu: bad arguments");
    return launch_silu(static_cast<__half*>(a), n, static_cast<cudaStream_t>(stream));
}

int w8a8_mul(w8a8_ctx* ctx, void* a, const void* b, long n, void* stream) {
    if (!ctx || (n > 0 && (!a || !b)) || n < 0) return fail(W8A8_ERR_INVALID_ARG, "mul: bad arguments");
    return launch_mul(static_cast<__half*>(a), static_cast<const __half*>(b), n, static_cast<cudaStream_t>(stream));
}

int w8a8_residual_add(w8a8_ctx* ctx, void* a, const void* b, long n, void* stream) {
    if (!ctx || (n > 0 && (!a || !b)) || n < 0) return fail(W8A8_ERR_INVALID_ARG, "residual_add: bad arguments");
    return launch_residual_add(static_cast<__half*>(a), static_cast<const __half*>(b), n,
                               static_cast<cudaStream_t>(stream));
}

int w8a8_linear_q(w8a8_ctx* ctx, const void* W, const void* w_scale, int group_size, const void* Xq,
                  const void* Xs, void* Y, int M, int N, int K, const w8a8_linear_opts* opts, void* stream) {
    int rc = check_linear_common(ctx, W, w_scale, Y, M, N, K, opts);
    if (rc) return rc;
    if (M > 0 && (!Xq || !Xs)) return fail(W8A8_ERR_INVALID_ARG, "null Xq or Xs");
    LinearArgs a = make_args(W, w_scale, group_size, Y, M, N, K, opts);
    a.Xq = static_cast<const int8_t*>(Xq);
    a.Xs = static_cast<const float*>(Xs);
    return dispatch_q(ctx, a, opts ? opts->kernel : W8A8_KERNEL_AUTO, static_cast<cudaStream_t>(stream));
}

int w8a8_linear_q_tail(w8a8_ctx* ctx, const void* W, const void* w_scale, int group_size, const void* Xq,
                       const void* Xs, void* Y, int M, int N, int K, const w8a8_linear_opts* opts,
                       const w8a8_tail* tail, void* stream) {
    if (!tail || tail->kind == W8A8_TAIL_NONE)
        return w8a8_linear_q(ctx, W, w_scale, group_size, Xq, Xs, Y, M, N, K, opts, stream);
    int rc = check_linear_common(ctx, W, w_scale, Y, M, N, K, opts);
    if (rc) return rc;
    if (M > 0 && (!Xq || !Xs)) return fail(W8A8_ERR_INVALID_ARG, "null Xq or Xs");
    const int epi = opts ? opts->epilogue : W8A8_EPI_NONE;
    const int cols = epi == W8A8_EPI_SWIGLU ? N / 2 : N;
    if (tail->kind == W8A8_TAIL_ROWNORM) {
        if (epi != W8A8_EPI_NONE) return fail(W8A8_ERR_INVALID_ARG, "W8A8_TAIL_ROWNORM goes with W8A8_EPI_NONE");
        if (!tail->x || !tail->norm_weight || tail->x == Y)
            return fail(W8A8_ERR_INVALID_ARG, "W8A8_TAIL_ROWNORM needs x (other than Y) and a norm weight");
        if (tail->Xq && !tail->Xs) return fail(W8A8_ERR_INVALID_ARG, "tail: Xq without Xs");
    } else if (tail->kind == W8A8_TAIL_GROUPQUANT) {
        if (epi == W8A8_EPI_RESIDUAL || !tail->Xq || !tail->Xs)
            return fail(W8A8_ERR_INVALID_ARG, "W8A8_TAIL_GROUPQUANT needs Xq and Xs and no residual epilogue");
    } else {
        return fail(W8A8_ERR_INVALID_ARG, "unknown tail kind %d", tail->kind);
    }
    if (M == 0) return W8A8_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int kernel = opts ? opts->kernel : W8A8_KERNEL_AUTO;
    LinearArgs a = make_args(W, w_scale, group_size, Y, M, N, K, opts);
    a.Xq = static_cast<const int8_t*>(Xq);
    a.Xs = static_cast<const float*>(Xs);
    if (kernel == W8A8_KERNEL_AUTO || kernel == W8A8_KERNEL_GEMV_PACKED) {
        LinearArgs f = a;
        fill_scratch(ctx, f);
        f.tail_kind = tail->kind == W8A8_TAIL_ROWNORM ? kTailRowNorm : kTailGroupQuant;
        f.tail_counters = ctx->tail_counters;
        f.tail_x = static_cast<__half*>(tail->x);
        f.tail_norm_weight = static_cast<const __half*>(tail->norm_weight);
        f.tail_eps = tail->eps;
        f.tail_g = norm_group(cols, tail->group_size);
        f.tail_Xq = static_cast<int8_t*>(tail->Xq);
        f.tail_Xs = static_cast<float*>(tail->Xs);
        f.tail_normed_out = static_cast<__half*>(tail->normed_out);
        if (f.packed && gemv_packed_supports(f)) return launch_linear_gemv_packed(f, ctx->device_status, s);
    }
    // the separate kernels, back to back
    rc = dispatch_q(ctx, a, kernel, s);
    if (rc) return rc;
    if (tail->kind == W8A8_TAIL_ROWNORM) {
        if (tail->Xq)
            return launch_rowquant(static_cast<const __half*>(tail->x), static_cast<__half*>(tail->x),
                                   static_cast<const __half*>(Y), static_cast<const __half*>(tail->norm_weight), tail->eps,
                                   nullptr, nullptr, M, N, tail->group_size, W8A8_ACT_PER_TOKEN_GROUP,
                                   static_cast<__half*>(tail->normed_out), static_cast<int8_t*>(tail->Xq),
                                   static_cast<float*>(tail->Xs), s);
        rc = launch_residual_add(static_cast<__half*>(tail->x), static_cast<const __half*>(Y), static_cast<long>(M) * N, s);
        if (rc || !tail->normed_out) return rc;
        return launch_rowquant(static_cast<const __half*>(tail->x), nullptr, nullptr,
                               static_cast<const __half*>(tail->norm_weight), tail->eps, nullptr, nullptr, M, N, N,
                               W8A8_ACT_PER_TOKEN_GROUP, static_cast<__half*>(tail->normed_out), nullptr, nullptr, s);
    }
    return launch_rowquant(static_cast<const __half*>(Y), nullptr, nullptr, nullptr, 0.0f, nullptr, nullptr, M, cols,
                           tail->group_size, W8A8_ACT_PER_TOKEN_GROUP, nullptr, static_cast<int8_t*>(tail->Xq),
                           static_cast<float*>(tail->Xs), s);
}

int w8a8_rmsnorm_linear(w8a8_ctx* ctx, const void* W, const void* w_scale, int group_size, const void* x,
                        const void* residual, void* x_out, const void* norm_weight, float eps, void* Y, int M, int N,
                        int K, const w8a8_linear_opts* opts, void* codes_out, void* scales_out, void* stream) {
    int rc = check_linear_common(ctx, W, w_scale, Y, M, N, K, opts);
    if (rc) return rc;
    if (M > 0 && (!x || !norm_weight)) return fail(W8A8_ERR_INVALID_ARG, "null x or norm weight");
    if (residual && (!x_out || x_out == x))
        return fail(W8A8_ERR_INVALID_ARG, "with a residual, x_out must be a buffer other than x");
    if ((codes_out == nullptr) != (scales_out == nullptr))
        return fail(W8A8_ERR_INVALID_ARG, "codes_out and scales_out go together");
    if (M == 0) return W8A8_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int kernel = opts ? opts->kernel : W8A8_KERNEL_AUTO;
    const int act_mode = opts ? opts->act_mode : W8A8_ACT_PER_TOKEN_GROUP;
    LinearArgs a = make_args(W, w_scale, group_size, Y, M, N, K, opts);
    if (act_mode == W8A8_ACT_PER_TOKEN_GROUP && (kernel == W8A8_KERNEL_AUTO || kernel == W8A8_KERNEL_GEMV_PACKED)) {
        LinearArgs f = a;
        f.X = static_cast<const __half*>(x);
        f.norm_weight = static_cast<const __half*>(norm_weight);
        f.norm_eps = eps;
        f.norm_residual = static_cast<const __half*>(residual);
        f.norm_x_out = static_cast<__half*>(x_out);
        f.codes_out = static_cast<int8_t*>(codes_out);
        f.scales_out = static_cast<float*>(scales_out);
        fill_scratch(ctx, f);
        if (gemv_packed_supports(f)) return launch_linear_gemv_packed(f, ctx->device_status, s);
    }
    // the two-launch form: row kernel into scratch (or the caller's buffers), then the integer kernel
    const size_t need = quant_scratch_bytes(M, K, group_size);
    if (!codes_out && need > ctx->workspace_bytes)
        return fail(W8A8_ERR_WORKSPACE, "need %zu bytes of scratch, context has %zu", need, ctx->workspace_bytes);
    int8_t* Xq = codes_out ? static_cast<int8_t*>(codes_out) : reinterpret_cast<int8_t*>(ctx->workspace);
    float* Xs = scales_out ? static_cast<float*>(scales_out)
                           : reinterpret_cast<float*>(ctx->workspace + align256(static_cast<size_t>(M) * K));
    rc = launch_rowquant(static_cast<const __half*>(x), static_cast<__half*>(x_out),
                         static_cast<const __half*>(residual), static_cast<const __half*>(norm_weight), eps, nullptr,
                         nullptr, M, K, group_size, act_mode, nullptr, Xq, Xs, s);
    if (rc) return rc;
    a.Xq = Xq;
    a.Xs = Xs;
    return dispatch_q(ctx, a, kernel, s);
}

int w8a8_linear(w8a8_ctx* ctx, const void* W, const void* w_scale, int group_size, const void* act_scale,
                const void* smooth_inv, const void* X, void* Y, int M, int N, int K,
                const w8a8_linear_opts* opts, void* stream) {
    int rc = check_linear_common(ctx, W, w_scale, Y, M, N, K, opts);
    if (rc) return rc;
    if (M > 0 && !X) return fail(W8A8_ERR_INVALID_ARG, "null X");
    if (M == 0) return W8A8_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    LinearArgs a = make_args(W, w_scale, group_size, Y, M, N, K, opts);
    const int act_mode = opts ? opts->act_mode : W8A8_ACT_PER_TOKEN_GROUP;
    const int kernel = opts ? opts->kernel : W8A8_KERNEL_AUTO;

    // Codes and scales into the context's scratch (row kernel), then the integer kernel; the two are
    // chained with programmatic dependent launch, so the second starts streaming weights early.
    const size_t need = quant_scratch_bytes(M, K, group_size);
    if (need > ctx->workspace_bytes)
        return fail(W8A8_ERR_WORKSPACE, "need %zu bytes of scratch, context has %zu", need, ctx->workspace_bytes);
    int8_t* Xq = reinterpret_cast<int8_t*>(ctx->workspace);
    float* Xs = reinterpret_cast<float*>(ctx->workspace + align256(static_cast<size_t>(M) * K));
    rc = launch_rowquant(static_cast<const __half*>(X), nullptr, nullptr, nullptr, 0.0f,
                         static_cast<const __half*>(smooth_inv), static_cast<const __half*>(act_scale), M, K,
                         group_size, act_mode, nullptr, Xq, Xs, s);
    if (rc) return rc;
    a.Xq = Xq;
    a.Xs = Xs;
    return dispatch_q(ctx, a, kernel, s);
}

int w8a8_qknorm_rope_kvwrite(w8a8_ctx* ctx, const void* qkv, const void* q_norm_w, const void* k_norm_w, float eps,
                             const float* freqs, const int* positions, const int* block_table,
                             int max_blocks_per_seq, void* k_cache, void* v_cache, int layer, int n_layers,
                             int batch, int n_q_heads, int n_kv_heads, int head_dim, void* q_out, void* stream) {
    if (!ctx) return fail(W8A8_ERR_INVALID_ARG, "null context");
    if (head_dim != 128) return fail(W8A8_ERR_UNSUPPORTED, "head_dim %d (only 128 is built)", head_dim);
    if (batch < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || max_blocks_per_seq <= 0 || layer < 0 || layer >= n_layers)
        return fail(W8A8_ERR_INVALID_ARG, "qknorm_rope_kvwrite: bad sizes");
    if (batch > 0 && (!qkv || !freqs || !positions || !block_table || !k_cache || !v_cache || !q_out))
        return fail(W8A8_ERR_INVALID_ARG, "qknorm_rope_kvwrite: null pointer");
    return launch_qknorm_rope_kvwrite(static_cast<const __half*>(qkv), static_cast<const __half*>(q_norm_w),
                                      static_cast<const __half*>(k_norm_w), eps, freqs, positions, block_table,
                                      max_blocks_per_seq, static_cast<__half*>(k_cache), static_cast<__half*>(v_cache),
                                      layer, n_layers, batch, n_q_heads, n_kv_heads, static_cast<__half*>(q_out),
                                      static_cast<cudaStream_t>(stream));
}

int w8a8_paged_attention_decode(w8a8_ctx* ctx, const void* q, const void* k_cache, const void* v_cache,
                                const int* block_table, const int* seq_lens, void* out, int batch, int n_heads,
                                int head_dim, int max_blocks_per_seq, float sm_scale, int layer, int n_layers,
                                int n_kv_heads, int quant_group_size, void* Xq, void* Xs, int context_splits,
                                void* stream) {
    if (!ctx) return fail(W8A8_ERR_INVALID_ARG, "null context");
    if (head_dim != 128) return fail(W8A8_ERR_UNSUPPORTED, "head_dim %d (only 128 is built)", head_dim);
    if (batch < 0 || n_heads <= 0 || n_kv_heads <= 0 || max_blocks_per_seq <= 0 || layer < 0 || layer >= n_layers)
        return fail(W8A8_ERR_INVALID_ARG, "paged_attention_decode: bad sizes");
    if (batch > 0 && (!q || !k_cache || !v_cache || !block_table || !seq_lens || (!out && !Xq) || (Xq && !Xs)))
        return fail(W8A8_ERR_INVALID_ARG, "paged_attention_decode: null pointer");
    return launch_paged_attention_decode(static_cast<const __half*>(q), static_cast<const __half*>(k_cache),
                                         static_cast<const __half*>(v_cache), block_table, seq_lens, batch, n_heads,
                                         n_kv_heads, max_blocks_per_seq, sm_scale, layer, n_layers,
                                         static_cast<__half*>(out), quant_group_size, static_cast<int8_t*>(Xq),
                                         static_cast<float*>(Xs), context_splits, ctx->device_status,
                                         static_cast<cudaStream_t>(stream));
}

int w8a8_qkv_attention_decode(w8a8_ctx* ctx, const void* qkv, const void* q_norm_w, const void* k_norm_w, float eps,
                              const float* freqs, const int* positions, void* k_cache, void* v_cache,
                              const int* block_table, const int* seq_lens, void* out, int batch, int n_heads,
                              int head_dim, int max_blocks_per_seq, float sm_scale, int layer, int n_layers,
                              int n_kv_heads, int quant_group_size, void* Xq, void* Xs, int context_splits,
                              void* stream) {
    if (!ctx) return fail(W8A8_ERR_INVALID_ARG, "null context");
    if (batch < 0 || head_dim != 128) return fail(W8A8_ERR_UNSUPPORTED, "head_dim must be 128 (got %d)", head_dim);
    if (batch > 0 && (!qkv || !freqs || !positions || !k_cache || !v_cache || !block_table || !seq_lens || (!out && !Xq)))
        return fail(W8A8_ERR_INVALID_ARG, "qkv_attention_decode: null argument");
    if ((Xq == nullptr) != (Xs == nullptr)) return fail(W8A8_ERR_INVALID_ARG, "Xq and Xs go together");
    return launch_qkv_attention_decode(static_cast<const __half*>(qkv), static_cast<const __half*>(q_norm_w),
                                       static_cast<const __half*>(k_norm_w), eps, freqs, positions,
                                       static_cast<__half*>(k_cache), static_cast<__half*>(v_cache), block_table, seq_lens,
                                       batch, n_heads, n_kv_heads, max_blocks_per_seq, sm_scale, layer, n_layers,
                                       static_cast<__half*>(out), quant_group_size, static_cast<int8_t*>(Xq),
                                       static_cast<float*>(Xs), context_splits, ctx->device_status,
                                       static_cast<cudaStream_t>(stream));
}

size_t w8a8_decode_stack_workspace_bytes(const w8a8_decode_stack* stack) {
    return stack ? decode_stack_workspace_bytes(*stack) : 0;
}

int w8a8_decode_stack_step(w8a8_ctx* ctx, const w8a8_decode_stack* stack, void* stream) {
    if (!ctx || !stack) return fail(W8A8_ERR_INVALID_ARG, "null context or stack descriptor");
    return launch_decode_stack(*stack, ctx->workspace, ctx->workspace_bytes, static_cast<float*>(ctx->splitk_partials),
                               kSplitkPartialBytes, ctx->splitk_counters, kSplitkCounters, ctx->device_status,
                               static_cast<cudaStream_t>(stream));
}

int w8a8_decode_stack_timeline(w8a8_ctx* ctx, const w8a8_decode_stack* stack, unsigned long long* stamps_out,
                               int capacity, void* stream) {
    if (!ctx || !stack || !stamps_out) return -fail(W8A8_ERR_INVALID_ARG, "null argument");
    const int n = decode_stack_timeline(*stack, ctx->workspace, stamps_out, capacity, static_cast<cudaStream_t>(stream));
    return n;
}

int w8a8_tp_create(w8a8_ctx* ctx, int rank, int world, int max_tokens, int dim, void* ipc_handle_out) {
    if (!ctx) return fail(W8A8_ERR_INVALID_ARG, "null context");
    if (ctx->tp) return fail(W8A8_ERR_INVALID_ARG, "this context already has a tensor-parallel exchange");
    return tp_create(&ctx->tp, rank, world, max_tokens, dim, ipc_handle_out);
}

int w8a8_tp_connect(w8a8_ctx* ctx, const void* all_ipc_handles) {
    if (!ctx || !ctx->tp) return fail(W8A8_ERR_INVALID_ARG, "w8a8_tp_create first");
    return tp_connect(ctx->tp, all_ipc_handles);
}

int w8a8_tp_linear_q(w8a8_ctx* ctx, const void* W, const void* w_scale, int group_size, const void* Xq, const void* Xs,
                     int M, int N, int K, const w8a8_linear_opts* opts, void* stream) {
    if (!ctx || !ctx->tp) return fail(W8A8_ERR_INVALID_ARG, "w8a8_tp_create first");
    if (M < 0 || N <= 0 || K <= 0 || !W || !w_scale || (M > 0 && (!Xq || !Xs)))
        return fail(W8A8_ERR_INVALID_ARG, "tp_linear_q: bad arguments");
    if (opts && opts->epilogue != W8A8_EPI_NONE) return fail(W8A8_ERR_INVALID_ARG, "tp_linear_q takes no epilogue");
    if (M == 0) return W8A8_OK;
    LinearArgs a = make_args(W, w_scale, group_size, nullptr, M, N, K, opts);
    a.Xq = static_cast<const int8_t*>(Xq);
    a.Xs = static_cast<const float*>(Xs);
    fill_scratch(ctx, a);
    int rc = tp_push_args(ctx->tp, M, N, &a.tp);
    if (rc) return rc;
    if (!a.packed || !gemv_packed_supports(a))
        return fail(W8A8_ERR_UNSUPPORTED, "tp_linear_q needs a weight registered with w8a8_register_packed_weight and M <= 32 "
                                          "(use w8a8_linear_q and hand its output to w8a8_tp_allreduce_rmsnorm_quantize)");
    return launch_linear_gemv_packed(a, ctx->device_status, static_cast<cudaStream_t>(stream));
}

int w8a8_tp_allreduce_rmsnorm_quantize(w8a8_ctx* ctx, void* x, const void* partial, const void* weight, float eps,
                                       const void* smooth_inv, const void* act_scale, int M, int K, int group_size,
                                       int act_mode, void* normed_out, void* Xq, void* Xs, void* stream) {
    if (!ctx || !ctx->tp) return fail(W8A8_ERR_INVALID_ARG, "w8a8_tp_create first");
    if (M < 0 || K <= 0 || (M > 0 && !x)) return fail(W8A8_ERR_INVALID_ARG, "tp row kernel: bad arguments");
    if (Xq && !Xs) return fail(W8A8_ERR_INVALID_ARG, "tp row kernel: Xq without Xs");
    return launch_tp_allreduce_rowquant(ctx->tp, static_cast<__half*>(x), static_cast<const __half*>(partial),
                                        static_cast<const __half*>(weight), eps, static_cast<const __half*>(smooth_inv),
                                        static_cast<const __half*>(act_scale), M, K, group_size, act_mode,
                                        static_cast<__half*>(normed_out), static_cast<int8_t*>(Xq),
                                        static_cast<float*>(Xs), ctx->device_status, static_cast<cudaStream_t>(stream));
}

int w8a8_debug_tail_counters(w8a8_ctx* ctx, int* out, int count, void* stream) {
    if (!ctx || !out || count < 0 || count > kTailCounterInts) return fail(W8A8_ERR_INVALID_ARG, "debug_tail_counters: bad arguments");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(out, ctx->tail_counters, count * sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "counter read: %s", cudaGetErrorString(e));
    return W8A8_OK;
}

size_t w8a8_packed_weight_bytes(int N, int K, int group_size) { return packed_weight_bytes(N, K, group_size); }

int w8a8_pack_weight(w8a8_ctx* ctx, const void* W, const void* w_scale, int N, int K, int group_size,
                     void* packed_out, void* stream) {
    if (!ctx || !W || !w_scale || !packed_out) return fail(W8A8_ERR_INVALID_ARG, "pack_weight: null argument");
    if (N <= 0 || K <= 0) return fail(W8A8_ERR_INVALID_ARG, "pack_weight: bad shape N=%d K=%d", N, K);
    return launch_pack_weight(static_cast<const int8_t*>(W), static_cast<const __half*>(w_scale), N, K, group_size,
                              packed_out, static_cast<cudaStream_t>(stream));
}

int w8a8_register_packed_weight(w8a8_ctx* ctx, const void* W, const void* packed, int N, int K, int group_size) {
    if (!ctx || !W) return fail(W8A8_ERR_INVALID_ARG, "register_packed_weight: null argument");
    std::lock_guard<std::mutex> lock(ctx->packed_mu);
    if (!packed) {
        ctx->packed.erase(W);
        return W8A8_OK;
    }
    if (N <= 0 || K <= 0 || packed_weight_bytes(N, K, group_size) == 0)
        return fail(W8A8_ERR_INVALID_ARG, "register_packed_weight: N=%d K=%d group=%d is not a packable shape", N, K,
                    group_size);
    ctx->packed[W] = w8a8_ctx::PackedEntry{packed, N, K, norm_group(K, group_size)};
    return W8A8_OK;
}

int w8a8_pack_gate_up(w8a8_ctx* ctx, const void* w_gate, const void* s_gate, const void* w_up, const void* s_up,
                      int inter, int K, int G, void* W_out, void* scale_out, void* stream) {
    if (!ctx) return fail(W8A8_ERR_INVALID_ARG, "null context");
    if (inter < 0 || inter % 8 != 0 || K <= 0 || G <= 0)
        return fail(W8A8_ERR_INVALID_ARG, "pack_gate_up: inter=%d (must be a multiple of 8) K=%d G=%d", inter, K, G);
    if (inter > 0 && (!w_gate || !s_gate || !w_up || !s_up || !W_out || !scale_out))
        return fail(W8A8_ERR_INVALID_ARG, "pack_gate_up: null pointer");
    return launch_pack_gate_up(static_cast<const int8_t*>(w_gate), static_cast<const __half*>(s_gate),
                               static_cast<const int8_t*>(w_up), static_cast<const __half*>(s_up), inter, K, G,
                               static_cast<int8_t*>(W_out), static_cast<__half*>(scale_out),
                               static_cast<cudaStream_t>(stream));
}

}  // extern "C"
