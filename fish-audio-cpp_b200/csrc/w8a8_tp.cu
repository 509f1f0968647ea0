// Tensor-parallel exchange for the row-parallel projections (wo, w2): a one-shot all-reduce whose SEND side is the
// epilogue of the projection's own kernel and whose RECEIVE side is the prologue of the kernel that consumes the sum.
// The reference is single-GPU; nothing there corresponds to this file.
//
// After a row-parallel linear every rank holds a partial [M, dim]. A collective library would make that 72 calls per
// decode step, each a launch with tens of microseconds of latency. Here:
//   send     the decode kernel (w8a8_gemv_packed.cu, LinearArgs::tp) stores every finished 16-row tile of its fp32
//            partial straight into slot [rank] of EVERY rank's exchange buffer over NVLink peer memory, as 8-byte words
//            {fp32 value, epoch}: the words carry their own arrival flag, so the sender needs no fence and no separate
//            flag, and the transfer of a tile overlaps the rest of the kernel. (A caller that already holds an fp16
//            partial can hand it to the receive kernel instead, which then sends it the same way first.)
//   receive  the residual add + RMSNorm + quantiser kernel: CTA m (one per token row) reads row m of all `world`
//            slots of its OWN buffer, polling (bounded) each 8-byte word until it carries this exchange's epoch, adds
//            the partials in ascending rank order in fp32, rounds once to fp16 (the all-reduced projection output),
//            adds that to the residual stream and goes on exactly like the single-GPU row kernel.
// Every rank adds the same values in the same order, so all ranks hold bit-identical activations, and the sum differs
// from the single-GPU projection output only by the association of its fp32 additions.
// The epoch lives on the device (it advances inside the kernels, so a replayed CUDA graph keeps counting); slots are
// double-buffered by epoch parity: a rank can be at most one exchange ahead of a peer. Peers are only ever WRITTEN
// to with plain stores; no load, TMA or otherwise, touches another GPU's memory, and nothing here uses multicast.
#include <cstring>

#include "w8a8_internal.h"
#include "w8a8_trace.cuh"

namespace w8a8 {

struct TpState {
    int rank = 0, world = 1, max_tokens = 0, dim = 0;
    unsigned char* local = nullptr;      // this rank's exchange region (cudaMalloc, exported over IPC)
    unsigned char* peers[8] = {nullptr}; // the same region on every rank (peers[rank] == local)
    size_t slot_bytes = 0, ctl_off = 0, total = 0;
    bool connected = false;
};

namespace {

constexpr int kMaxWorld = 8;
constexpr int kRowThreads = 256;
constexpr unsigned kSpinLimit = 1u << 22;  // polls of one word before the kernel gives up (3 to 4 seconds: a poll is an
                                            // L2 read plus a 64 ns sleep)

struct TpRowParams {
    __half* x;                 // residual stream, updated in place
    const __half* partial;     // this rank's projection output [M, K] fp16, or null: already sent by the linear
    const __half* norm_weight; // null: no norm
    float eps;
    __half* normed_out;
    int8_t* Xq;
    float* Xs;
    int M, K, g, G, T;         // T: threads of the reference's rms_norm launch for this K (summation order)
    TpPush tp;
    int* status;
};

__device__ __forceinline__ uint4 ld_volatile16(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// control words behind the slots: [0] epoch of the last finished exchange, [1] CTAs of the running receive kernel
// that are done (the last one advances the epoch and clears this)
__global__ void __launch_bounds__(kRowThreads) tp_receive_rowquant_kernel(const TpRowParams p) {
    __shared__ float s_red[32];
    __shared__ __align__(16) __half row_s[4096];
    __shared__ int s_fail;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K, m = blockIdx.x, pieces = K / 8, VW = p.T / kRowThreads;
    const size_t base = static_cast<size_t>(m) * K;
    W8A8_TRACE_SCOPE();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint4 wv[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c8 = tid + i * kRowThreads;
        wv[i] = make_uint4(0u, 0u, 0u, 0u);
        if (p.norm_weight) wv[i] = __ldg(reinterpret_cast<const uint4*>(p.norm_weight) + (c8 < pieces ? c8 : 0));
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    W8A8_TRACE_WAITED();
    if (tid == 0) s_fail = 0;
    int* ctl = reinterpret_cast<int*>(p.tp.peers[p.tp.rank] + p.tp.ctl_off);
    const int ep = *reinterpret_cast<volatile int*>(ctl) + 1, par = ep & 1;
    const int world = p.tp.world;
    const size_t row_words = (static_cast<size_t>(par) * world * p.tp.max_tokens + m) * K;  // + r * max_tokens * K
    const size_t src_stride = static_cast<size_t>(p.tp.max_tokens) * K;                     // words between sources

    // 0. (two-call form) send this rank's fp16 row to every rank as {fp32, epoch} words
    if (p.partial) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int c8 = tid + i * kRowThreads;
            if (c8 < pieces) {
                const uint4 u = *reinterpret_cast<const uint4*>(p.partial + base + c8 * 8);
                const __half* h = reinterpret_cast<const __half*>(&u);
                for (int r = 0; r < world; ++r) {
                    uint4* dst = reinterpret_cast<uint4*>(p.tp.peers[r]) +
                                 (row_words + static_cast<size_t>(p.tp.rank) * src_stride + c8 * 8) / 2;
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        dst[q] = make_uint4(__float_as_uint(__half2float(h[2 * q])), static_cast<unsigned>(ep),
                                            __float_as_uint(__half2float(h[2 * q + 1])), static_cast<unsigned>(ep));
                }
            }
        }
    }
    __syncthreads();

    // 1. + 2. poll the words of row m from every source (in this GPU's own memory), sum in rank order in fp32
    uint4 xv[2];
    float sum[2][8];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c8 = tid + i * kRowThreads;
        const int cc = c8 < pieces ? c8 : 0;
        xv[i] = *reinterpret_cast<const uint4*>(p.x + base + cc * 8);
#pragma unroll
        for (int e = 0; e < 8; ++e) sum[i][e] = 0.0f;
    }
    const unsigned char* mine = p.tp.peers[p.tp.rank];
    bool failed = false;
    for (int r = 0; r < world; ++r) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int c8 = tid + i * kRowThreads;
            if (c8 >= pieces) continue;
            const uint4* src = reinterpret_cast<const uint4*>(mine) + (row_words + static_cast<size_t>(r) * src_stride + c8 * 8) / 2;
            uint4 w[4];
            unsigned spins = 0;
            for (;;) {
#pragma unroll
                for (int q = 0; q < 4; ++q) w[q] = ld_volatile16(src + q);
                bool ok = true;
#pragma unroll
                for (int q = 0; q < 4; ++q) ok &= (w[q].y == static_cast<unsigned>(ep)) & (w[q].w == static_cast<unsigned>(ep));
                if (ok) break;
                if (++spins > kSpinLimit) { failed = true; break; }
                if (spins > 64) __nanosleep(64);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                sum[i][2 * q] += __uint_as_float(w[q].x);
                sum[i][2 * q + 1] += __uint_as_float(w[q].z);
            }
        }
        if (failed) break;
    }
    if (failed) {
        atomicExch(p.status, 700 + m);
        s_fail = 1;
    }
    // x += half(sum) (ffn_activations.cu:41-45 for the add); the row goes to shared memory for the norm's sum
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c8 = tid + i * kRowThreads;
        if (c8 < pieces) {
            __half* hx = reinterpret_cast<__half*>(&xv[i]);
#pragma unroll
            for (int e = 0; e < 8; ++e) hx[e] = __float2half(__half2float(hx[e]) + __half2float(__float2half(sum[i][e])));
            *reinterpret_cast<uint4*>(p.x + base + c8 * 8) = xv[i];
            reinterpret_cast<uint4*>(row_s)[c8] = xv[i];
        }
    }
    __syncthreads();
    // ---- from here on: rowquant_compact_kernel (RMSNorm in the reference's order, then the quantiser) ----
    float rms = 1.0f;
    if (p.norm_weight) {
#pragma unroll 1
        for (int k = 0; k < VW; ++k) {
            float local_sum = 0.0f;
#pragma unroll 1
            for (int e = (warp * VW + k) * 32 + lane; e < K; e += p.T) {
                float val = __half2float(row_s[e]);
                local_sum += val * val;
            }
            for (int offset = 16; offset > 0; offset /= 2) local_sum += __shfl_down_sync(0xffffffffu, local_sum, offset);
            if (lane == 0) s_red[warp * VW + k] = local_sum;
        }
        __syncthreads();
        float total_sum = 0.0f;
        if (warp == 0) {
            if (lane < p.T / 32) total_sum = s_red[lane];
            for (int offset = 16; offset > 0; offset /= 2) total_sum += __shfl_down_sync(0xffffffffu, total_sum, offset);
        }
        __syncthreads();
        if (tid == 0) s_red[0] = rsqrtf(total_sum / K + p.eps);
        __syncthreads();
        rms = s_red[0];
    }
    const int lanes = p.g / 8;  // threads per quantisation group
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c8 = tid + i * kRowThreads;
        const bool live = c8 < pieces;  // whole warps are live or not (pieces is a multiple of 32)
        __half* hx = reinterpret_cast<__half*>(&xv[i]);
        const __half* hw = reinterpret_cast<const __half*>(&wv[i]);
        float v[8], amax = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            if (p.norm_weight) {
                float val = __half2float(hx[e]) * rms;
                hx[e] = __float2half(val * __half2float(hw[e]));
            }
            v[e] = __half2float(hx[e]);
            amax = fmaxf(amax, fabsf(v[e]));
        }
        if (live && p.normed_out) *reinterpret_cast<uint4*>(p.normed_out + base + c8 * 8) = xv[i];
        if (!p.Xq) continue;
        for (int o = lanes / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (!live) continue;
        float scale = amax / 127.0f;
        if (scale < 1e-8f) scale = 1e-8f;
        if ((lane & (lanes - 1)) == 0) p.Xs[static_cast<size_t>(m) * p.G + (c8 * 8) / p.g] = scale;
        const float inv_scale = 1.0f / scale;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            int q = __float2int_rn(v[e] * inv_scale);
            q = max(-127, min(127, q));
            if (e < 4) lo |= (static_cast<uint32_t>(q) & 0xffu) << (8 * e);
            else hi |= (static_cast<uint32_t>(q) & 0xffu) << (8 * (e - 4));
        }
        *reinterpret_cast<uint2*>(p.Xq + base + c8 * 8) = make_uint2(lo, hi);
    }
    // The CTA that finishes last advances the epoch: by then every CTA of this launch has read it.
    if (tid == 0) {
        const int done = atomicAdd(&ctl[1], 1);
        if (done == static_cast<int>(gridDim.x) - 1) {
            ctl[1] = 0;
            __threadfence();
            ctl[0] = ep;
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
    // slots: [2 parities][world][max_tokens][dim] words of 8 bytes {fp32 value, epoch}; then the control words
    t->slot_bytes = static_cast<size_t>(2) * world * max_tokens * dim * 8;
    t->ctl_off = (t->slot_bytes + 255) & ~size_t(255);
    t->total = t->ctl_off + 256;
    cudaError_t e = cudaMalloc(&t->local, t->total);
    if (e == cudaSuccess) e = cudaMemset(t->local, 0, t->total);  // epoch 0 everywhere: the first exchange is epoch 1
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

int tp_push_args(const TpState* t, int M, int N, TpPush* out) {
    if (!t || !t->connected) return fail(W8A8_ERR_INVALID_ARG, "tensor-parallel state is not connected");
    if (M > t->max_tokens || N != t->dim)
        return fail(W8A8_ERR_INVALID_ARG, "tp exchange was created for %d x %d, got %d x %d", t->max_tokens, t->dim, M, N);
    TpPush p = {};
    p.world = t->world; p.rank = t->rank; p.max_tokens = t->max_tokens;
    p.ctl_off = t->ctl_off;
    for (int r = 0; r < t->world; ++r) p.peers[r] = t->peers[r];
    *out = p;
    return W8A8_OK;
}

int launch_tp_allreduce_rowquant(TpState* t, __half* x, const __half* partial, const __half* norm_weight, float eps,
                                 const __half* smooth_inv, const __half* act_scale, int M, int K, int g, int act_mode,
                                 __half* normed_out, int8_t* Xq, float* Xs, int* status, cudaStream_t stream) {
    if (M == 0) return W8A8_OK;
    TpRowParams p = {};
    int rc = tp_push_args(t, M, K, &p.tp);
    if (rc) return rc;
    if (smooth_inv || act_scale || act_mode != W8A8_ACT_PER_TOKEN_GROUP)
        return fail(W8A8_ERR_UNSUPPORTED, "the tensor-parallel row kernel quantises dynamically per (token, group) only");
    const int gn = norm_group(K, g), G = num_groups(K, g);
    int T = 1;
    while (T < K && T < 1024) T <<= 1;
    if (K % 256 != 0 || K > 4096 || T < kRowThreads || (Xq && !(gn == 64 || gn == 128 || gn == 256)) ||
        ((reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(normed_out) |
          reinterpret_cast<uintptr_t>(Xq)) & 15u))
        return fail(W8A8_ERR_UNSUPPORTED, "tp row kernel: K=%d group=%d", K, gn);
    p.x = x; p.partial = partial; p.norm_weight = norm_weight; p.eps = eps; p.normed_out = normed_out; p.Xq = Xq; p.Xs = Xs;
    p.M = M; p.K = K; p.g = Xq ? gn : 256; p.G = G; p.T = T; p.status = status;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(M, 1, 1);
    cfg.blockDim = dim3(kRowThreads, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled(kPdlRow) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, tp_receive_rowquant_kernel, p);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "tp row kernel launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}

}  // namespace w8a8

W8A8_TRACE_READER(tp)
