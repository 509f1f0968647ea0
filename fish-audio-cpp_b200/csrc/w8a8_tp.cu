// Tensor-parallel exchange for the row-parallel projections (wo, w2): a one-shot all-reduce fused with
// the kernel that consumes it. The reference is single-GPU; nothing there corresponds to this file.
//
// After a row-parallel linear every rank holds a partial [M, dim] fp16. Instead of handing it to a
// collective library (72 calls per decode step, each a launch with tens of microseconds of latency)
// the NEXT kernel of the layer — residual add + RMSNorm + activation quantiser — does the exchange
// itself over NVLink peer memory:
//   1. CTA m (one per token row) stores row m of its rank's partial into slot [rank] of EVERY rank's
//      exchange buffer with plain 128-bit peer stores, fences at system scope, and raises flag
//      [rank][m] on every rank to the row's new epoch number;
//   2. it waits (bounded) until all `world` flags of row m in its OWN buffer carry that epoch;
//   3. it adds the `world` partial rows from its own HBM in ascending rank order in fp32, rounds once
//      to fp16 (that is the all-reduced projection output), adds it to the residual stream, and goes
//      on with the norm and the quantiser exactly like the single-GPU kernel.
// Every rank adds the same values in the same order, so all ranks hold bit-identical activations.
// Buffers are double-buffered by epoch parity: a rank can be at most one exchange ahead of a peer.
// Peers are only ever WRITTEN to; no load, TMA or otherwise, touches another GPU's memory.
#include <cstring>

#include "w8a8_internal.h"
#include "w8a8_trace.cuh"

namespace w8a8 {

struct TpState {
    int rank = 0, world = 1, max_tokens = 0, dim = 0;
    unsigned char* local = nullptr;      // this rank's exchange region (cudaMalloc, exported over IPC)
    unsigned char* peers[8] = {nullptr}; // the same region on every rank (peers[rank] == local)
    size_t slot_bytes = 0, flags_off = 0, epochs_off = 0, total = 0;
    bool connected = false;
};

namespace {

constexpr int kWarp = 32;
constexpr int kMaxWorld = 8;
constexpr int kElems = 4;

struct TpRowParams {
    __half* x;                 // residual stream, updated in place
    const __half* partial;     // this rank's projection output [M, K]
    const __half* norm_weight;
    float eps;
    const __half* smooth_inv;
    const __half* act_scale;
    __half* normed_out;
    int8_t* Xq;
    float* Xs;
    int K, g, G, per_token;
    int rank, world, max_tokens;
    unsigned char* peers[kMaxWorld];
    size_t flags_off, epochs_off;
    int* status;
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = kWarp / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// slots: [2 parities][world][max_tokens][K] fp16; flags: [2][world][max_tokens] int; epochs: [max_tokens] int
__global__ void __launch_bounds__(1024) tp_allreduce_rowquant_kernel(const TpRowParams p) {
    __shared__ float s_red[kWarp];
    __shared__ unsigned s_gmax[160];
    __shared__ int s_epoch, s_fail;
    const int tid = threadIdx.x, T = blockDim.x, K = p.K, g = p.g, G = p.G, m = blockIdx.x;
    const int lane = tid & (kWarp - 1), warp = tid / kWarp;
    const size_t base = static_cast<size_t>(m) * K;
    W8A8_TRACE_SCOPE();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    W8A8_TRACE_WAITED();

    unsigned char* mine = p.peers[p.rank];
    int* epochs = reinterpret_cast<int*>(mine + p.epochs_off);
    if (tid == 0) { s_epoch = epochs[m] + 1; s_fail = 0; }
    for (int j = tid; j < G; j += T) s_gmax[j] = 0u;
    __syncthreads();
    const int ep = s_epoch, par = ep & 1;
    const size_t row_off = ((static_cast<size_t>(par) * p.world + p.rank) * p.max_tokens + m) * K * sizeof(__half);

    // 1. push this rank's row to every rank (16 bytes per thread and peer), then raise the flags.
    //    One system-scope fence by the flag-raising threads is enough: the block barrier orders the
    //    other threads' peer stores before it, and the fence is cumulative.
    for (int v = tid; v < K / 8; v += T) {
        const uint4 u = *reinterpret_cast<const uint4*>(p.partial + base + v * 8);
        for (int r = 0; r < p.world; ++r) *reinterpret_cast<uint4*>(p.peers[r] + row_off + v * 16) = u;
    }
    __syncthreads();
    if (tid < p.world) {
        __threadfence_system();
        int* flag = reinterpret_cast<int*>(p.peers[tid] + p.flags_off) + (par * p.world + p.rank) * p.max_tokens + m;
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(ep) : "memory");
    }
    // 2. wait for every rank's row m to have arrived here (bounded: about a second at most)
    if (tid < p.world) {
        const int* flag = reinterpret_cast<const int*>(mine + p.flags_off) + (par * p.world + tid) * p.max_tokens + m;
        int seen = 0;
        unsigned spins = 0;
        do {
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
            if (seen == ep) break;
            if (++spins > 256) __nanosleep(64);
        } while (spins < (1u << 23));
        if (seen != ep) { atomicExch(p.status, 700 + tid); s_fail = 1; }
    }
    __syncthreads();

    // 3. sum the world partial rows in rank order in fp32, round once, x += half(sum)
    //    (ffn_activations.cu:41-45 for the add). The rows were written by other GPUs straight into this
    //    GPU's L2: read them past L1 (ld.cg), 16 bytes at a time.
    for (int v = tid; v < K / 8; v += T) {
        float sum[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) sum[i] = 0.0f;
        for (int r = 0; r < p.world; ++r) {
            const unsigned char* slot = mine + ((static_cast<size_t>(par) * p.world + r) * p.max_tokens + m) * K * sizeof(__half);
            const uint4 u = __ldcg(reinterpret_cast<const uint4*>(slot) + v);
            const __half* hh = reinterpret_cast<const __half*>(&u);
#pragma unroll
            for (int i = 0; i < 8; ++i) sum[i] += __half2float(hh[i]);
        }
        uint4 xu = *reinterpret_cast<const uint4*>(p.x + base + v * 8);
        __half* xh = reinterpret_cast<__half*>(&xu);
#pragma unroll
        for (int i = 0; i < 8; ++i) xh[i] = __float2half(__half2float(xh[i]) + __half2float(__float2half(sum[i])));
        *reinterpret_cast<uint4*>(p.x + base + v * 8) = xu;
    }
    __syncthreads();
    // each thread now picks up the elements it owns in the reference's norm order: t, t+T, t+2T, ...
    __half h[kElems];
    float local_sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kElems; ++i) {
        const int e = tid + i * T;
        if (e < K) {
            h[i] = p.x[base + e];
            float val = __half2float(h[i]);
            local_sum += val * val;
        }
    }
    if (tid == 0) epochs[m] = ep;
    // ---- from here on: rowquant_fast_kernel (RMSNorm in the reference's order, then the quantiser) ----
    if (p.norm_weight) {
        for (int offset = kWarp / 2; offset > 0; offset /= 2)
            local_sum += __shfl_down_sync(0xffffffffu, local_sum, offset);
        if (lane == 0) s_red[warp] = local_sum;
        __syncthreads();
        float total_sum = 0.0f;
        const int num_warps = (T + kWarp - 1) / kWarp;
        if (tid < num_warps) total_sum = s_red[tid];
        if (warp == 0) {
            for (int offset = kWarp / 2; offset > 0; offset /= 2)
                total_sum += __shfl_down_sync(0xffffffffu, total_sum, offset);
        }
        __syncthreads();
        if (tid == 0) s_red[0] = rsqrtf(total_sum / K + p.eps);
        __syncthreads();
        const float rms = s_red[0];
#pragma unroll
        for (int i = 0; i < kElems; ++i) {
            const int e = tid + i * T;
            if (e < K) {
                float val = __half2float(h[i]) * rms;
                h[i] = __float2half(val * __half2float(p.norm_weight[e]));
                if (p.normed_out) p.normed_out[base + e] = h[i];
            }
        }
    }
    if (!p.Xq) {
        W8A8_TRACE_END(5u);
        return;
    }
    float v[kElems];
#pragma unroll
    for (int i = 0; i < kElems; ++i) {
        const int e = tid + i * T;
        v[i] = 0.0f;
        if (e < K) {
            v[i] = __half2float(h[i]);
            if (p.smooth_inv) v[i] *= __half2float(p.smooth_inv[e]);
        }
    }
    if (!p.act_scale) {
#pragma unroll
        for (int i = 0; i < kElems; ++i) {
            const int e0 = warp * kWarp + i * T;
            if (e0 < K) {
                float mx = warp_max(fabsf(v[i]));
                if (lane == 0) atomicMax(&s_gmax[p.per_token ? 0 : e0 / g], __float_as_uint(mx));
            }
        }
    }
    __syncthreads();
    for (int j = tid; j < G; j += T) {
        float sc = p.act_scale ? __half2float(p.act_scale[j]) : __uint_as_float(s_gmax[p.per_token ? 0 : j]) / 127.0f;
        if (sc < 1e-8f) sc = 1e-8f;
        p.Xs[static_cast<size_t>(m) * G + j] = sc;
    }
#pragma unroll
    for (int i = 0; i < kElems; ++i) {
        const int e = tid + i * T;
        if (e < K) {
            const int j = e / g;
            float sc = p.act_scale ? __half2float(p.act_scale[j]) : __uint_as_float(s_gmax[p.per_token ? 0 : j]) / 127.0f;
            if (sc < 1e-8f) sc = 1e-8f;
            const float inv_scale = 1.0f / sc;
            int q = __float2int_rn(v[i] * inv_scale);
            q = max(-127, min(127, q));
            p.Xq[base + e] = static_cast<int8_t>(q);
        }
    }
    W8A8_TRACE_END(5u);
}

}  // namespace

int tp_create(TpState** out, int rank, int world, int max_tokens, int dim, void* ipc_handle_out64) {
    if (!out || world < 1 || world > kMaxWorld || rank < 0 || rank >= world || max_tokens < 1 || dim < 8 || dim % 8)
        return fail(W8A8_ERR_INVALID_ARG, "tp_create: rank %d world %d tokens %d dim %d", rank, world, max_tokens, dim);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    TpState* t = new TpState;
    t->rank = rank; t->world = world; t->max_tokens = max_tokens; t->dim = dim;
    t->slot_bytes = static_cast<size_t>(2) * world * max_tokens * dim * sizeof(__half);
    t->flags_off = (t->slot_bytes + 255) & ~size_t(255);
    t->epochs_off = t->flags_off + ((static_cast<size_t>(2) * world * max_tokens * sizeof(int) + 255) & ~size_t(255));
    t->total = t->epochs_off + ((static_cast<size_t>(max_tokens) * sizeof(int) + 255) & ~size_t(255));
    cudaError_t e = cudaMalloc(&t->local, t->total);
    if (e == cudaSuccess) e = cudaMemset(t->local, 0, t->total);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, t->local);
    if (e != cudaSuccess) {
        cudaFree(t->local);
        delete t;
        return fail(W8A8_ERR_CUDA, "tp_create: %s", cudaGetErrorString(e));
    }
    if (ipc_handle_out64) std::memcpy(ipc_handle_out64, &h, 64);
    t->peers[rank] = t->local;
    t->connected = world == 1;
    *out = t;
    return W8A8_OK;
}

int tp_connect(TpState* t, const void* all_handles) {
    if (!t) return fail(W8A8_ERR_INVALID_ARG, "tp_connect: null argument");
    if (!all_handles) {
        // Loop-back for failure-detection tests on one GPU: every "peer" is this rank's own buffer, so the
        // other ranks' rows never arrive and the bounded wait must run out with an error status.
        for (int r = 0; r < t->world; ++r) t->peers[r] = t->local;
        t->connected = true;
        return W8A8_OK;
    }
    for (int r = 0; r < t->world; ++r) {
        if (r == t->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, static_cast<const unsigned char*>(all_handles) + 64 * r, 64);
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "tp_connect: rank %d cannot map rank %d: %s", t->rank, r, cudaGetErrorString(e));
        t->peers[r] = static_cast<unsigned char*>(p);
    }
    t->connected = true;
    return W8A8_OK;
}

int tp_destroy(TpState* t) {
    if (!t) return W8A8_OK;
    for (int r = 0; r < t->world; ++r)
        if (r != t->rank && t->peers[r] && t->peers[r] != t->local) cudaIpcCloseMemHandle(t->peers[r]);
    cudaFree(t->local);
    delete t;
    return W8A8_OK;
}

int launch_tp_allreduce_rowquant(TpState* t, __half* x, const __half* partial, const __half* norm_weight, float eps,
                                 const __half* smooth_inv, const __half* act_scale, int M, int K, int g, int act_mode,
                                 __half* normed_out, int8_t* Xq, float* Xs, int* status, cudaStream_t stream) {
    if (!t || !t->connected) return fail(W8A8_ERR_INVALID_ARG, "tensor-parallel state is not connected");
    if (M == 0) return W8A8_OK;
    if (M > t->max_tokens || K != t->dim)
        return fail(W8A8_ERR_INVALID_ARG, "tp exchange was created for %d x %d, got %d x %d", t->max_tokens, t->dim, M, K);
    int threads = 1;
    while (threads < K && threads < 1024) threads <<= 1;
    if (threads < 32) threads = 32;
    const int gn = norm_group(K, g), G = num_groups(K, g);
    if (K > kElems * threads || gn % 32 != 0 || G > 160 || K % 8 != 0 || (reinterpret_cast<uintptr_t>(partial) & 15u))
        return fail(W8A8_ERR_UNSUPPORTED, "tp row kernel: K=%d group=%d", K, gn);
    TpRowParams p = {};
    p.x = x; p.partial = partial; p.norm_weight = norm_weight; p.eps = eps; p.smooth_inv = smooth_inv;
    p.act_scale = act_scale; p.normed_out = normed_out; p.Xq = Xq; p.Xs = Xs;
    p.K = K; p.g = gn; p.G = G; p.per_token = act_mode == W8A8_ACT_PER_TOKEN;
    p.rank = t->rank; p.world = t->world; p.max_tokens = t->max_tokens;
    for (int r = 0; r < t->world; ++r) p.peers[r] = t->peers[r];
    p.flags_off = t->flags_off; p.epochs_off = t->epochs_off; p.status = status;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(M, 1, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled(kPdlRow) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, tp_allreduce_rowquant_kernel, p);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "tp row kernel launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}

}  // namespace w8a8

W8A8_TRACE_READER(tp)
