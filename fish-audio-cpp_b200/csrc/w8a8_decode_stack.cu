// One decode step of the slow-AR transformer stack (the layer loop of DualAREngine::decode_step,
// src/engine/dual_ar_engine.cc:560-665) as ONE persistent kernel: a CTA per SM, launched cooperatively,
// phases separated by grid barriers.
//
// Why one kernel. At batch 8 a layer is nine small launches; each of them pays its own ramp-up and tail
// (a few microseconds) around one to eight microseconds of streaming, so the step runs at a fraction of
// the HBM roofline although every kernel moves only its algorithmic bytes. The weights, however, do not
// depend on the activations: here every warp pulls ITS weight blocks of all 4 x n_layers linears, in the
// order in which it will consume them, through one private ring of shared-memory stages that never
// stops — while a warp waits at a barrier, normalises a row or attends, its next blocks are already
// arriving. Barriers stall arithmetic, not the HBM stream.
//
// The arithmetic of every phase is that of the stand-alone kernels (w8a8_quant.cu, w8a8_gemv_packed.cu,
// w8a8_attn.cu), operation for operation. One thing differs: how many CTAs share a linear's row tiles (one per
// SM here, up to two per SM there), hence where its K range is cut between warps and how its fp32 partial sums
// are grouped; int8 codes, scales and int32 group sums are the same.
//
//   per layer:  A  x += delta; RMSNorm; quantise            (CTA r = token row r)       | barrier
//               B  qkv = W8A8 linear(wqkv)                  (all warps, stream-K)        | barrier
//               C  qk-norm, RoPE, KV write, attention part  (CTA = sequence x kv head x context slice) | barrier
//               D  merge slices, quantise for wo            (CTA = sequence x kv head)   | barrier
//               E  delta = linear(wo)                                                    | barrier
//               F  x += delta; RMSNorm; quantise                                         | barrier
//               G  act = SwiGLU(linear(w1|w3 interleaved))                               | barrier
//               H  quantise act                             (warp = row x 256 channels)  | barrier
//               I  delta = linear(w2)                                                    | barrier
//   then        x += delta; final RMSNorm -> out
//
// Everything a phase reads that an earlier phase of the same launch wrote is read past L1 (ld.global.cg):
// L1 is not coherent between SMs. Every wait (mbarrier, grid barrier) is bounded; when one runs out the
// CTA records a code in the status word, which makes all other CTAs leave at their next barrier, waits
// (bounded) for its own copies in flight and returns.
#include "sm100_ptx.cuh"
#include "w8a8_internal.h"

namespace w8a8 {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 4;
constexpr int kBlockW = 16 * 256;
constexpr int kStagePitch = kBlockW + 128;
constexpr int kRingBytes = kStages * kStagePitch;
constexpr int kHeadDim = 128;
constexpr int kBlockTokens = 16;
constexpr int kQPerKv = 4;
// The grid barrier's fence and atomic are issued by a thread other than the one that requests the bulk copies.
constexpr int kFenceLane = 1;
constexpr int kLocalTiles = 128;  // row tiles per CTA whose arrival counters live in shared memory
constexpr int kPartStride = 4 + kHeadDim;  // floats per head of an attention partial: m, l, 2 pad, acc[128]

struct GemvShape {
    int N, K, G, upt, epilogue;
    unsigned U;   // units (16 rows x 256 K-bytes) in all
    unsigned NW;  // warps that take part
};

struct StackParams {
    const w8a8_decode_layer* layers;
    int n_layers, B, dim, n_q, n_kv, inter, g;
    int norm_threads;  // block size of the reference's rms_norm launch for `dim`: min(1024, pow2 >= dim)
    int block_bytes;   // packed block: 4096 + 32 * groups per 256
    int S;             // context slices per (sequence, kv head)
    float eps, sm_scale;
    const __half* final_norm;
    const float* freqs;
    const int* positions;
    const int* seq_lens;
    const int* block_table;
    int max_blocks;
    __half* k_cache;
    __half* v_cache;
    __half* x;
    __half* out;
    // scratch
    __half* qkv;
    int8_t* xq;
    float* xs;
    int8_t* aq;
    float* as_;
    __half* act;
    int8_t* actq;
    float* acts;
    __half* delta;
    float* attn_part;
    unsigned* barrier;
    int* status;
    unsigned long long* timeline;  // CTA 0 stamps the global nanosecond timer after every phase and barrier
    GemvShape gs[4];
};

// ---- loads that bypass L1 -------------------------------------------------------------------
__device__ __forceinline__ uint4 ldcg128(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float4 ldcg_f4(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float ldcg_f(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ __half ldcg_h(const __half* p) {
    unsigned short v;
    asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return __ushort_as_half(v);
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D(16x8, fp32) += A(16x16 fp16, rows 8..15 zero) x B(16x8 fp16); only rows 0..7 of D are kept.
__device__ __forceinline__ void mma_top_rows(float& d0, float& d1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float j2, j3;
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d0), "=f"(d1), "=f"(j2), "=f"(j3)
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(d0), "f"(d1), "f"(0.0f), "f"(0.0f));
}
__device__ __forceinline__ uint32_t reg_of(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
__device__ __forceinline__ float warp_max(float v) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// The units of a linear are dealt out in whole 16-row tiles to the CTAs (tile t of T goes to CTA t * C / T) and a
// CTA's units in equal contiguous runs to its 8 warps. A tile cut by a run boundary is therefore always cut
// between warps of ONE CTA, and its partial sums meet in shared memory: no global scratch, no atomics on L2.
__device__ __forceinline__ void warp_range(const GemvShape& sh, unsigned cta, unsigned nctas, unsigned warp, unsigned& cu0,
                                           unsigned& n, unsigned& nw, unsigned& u0, unsigned& u1) {
    const unsigned tiles = sh.U / sh.upt;
    const unsigned t0 = cta * tiles / nctas, t1 = (cta + 1) * tiles / nctas;
    cu0 = t0 * sh.upt;
    n = (t1 - t0) * sh.upt;
    nw = n < kWarps ? n : kWarps;  // warps that take part: none of them with an empty run
    u0 = u1 = cu0;
    if (warp < nw) {
        u0 = cu0 + warp * n / nw;
        u1 = cu0 + (warp + 1) * n / nw;
    }
}

// ---- the weight stream of one warp ------------------------------------------------------------
struct Stream {
    uint32_t ring;
    uint64_t* bar;
    unsigned pt, ct;  // blocks requested / consumed so far, over all linears
    int pj;           // the linear the producer is in: layer * 4 + kind
    unsigned p_left;  // blocks of it still to request
    const unsigned char* p_src;
    const unsigned char* next_img;  // packed image of linear pj + 1 (fetched one linear ahead)
};

__device__ __forceinline__ const unsigned char* packed_image(const StackParams& p, int j) {
    if (j >= 4 * p.n_layers) return nullptr;
    static_assert(sizeof(void*) == sizeof(unsigned long long), "pointer width");
    return reinterpret_cast<const unsigned char*>(
        __ldg(reinterpret_cast<const unsigned long long*>(&p.layers[j >> 2].packed[j & 3])));
}

// Lane 0 only: requests the next block of this warp's sequence, if there is one.
__device__ __forceinline__ void stream_issue(Stream& s, const StackParams& p, unsigned gw) {
    while (s.p_left == 0) {
        if (s.pj + 1 >= 4 * p.n_layers) return;
        ++s.pj;
        const GemvShape& sh = p.gs[s.pj & 3];
        const unsigned char* img = s.next_img;
        s.next_img = packed_image(p, s.pj + 1);
        unsigned cu0, n, nw, u0, u1;
        warp_range(sh, blockIdx.x, gridDim.x, gw % kWarps, cu0, n, nw, u0, u1);
        s.p_left = u1 - u0;
        s.p_src = img + static_cast<size_t>(u0) * p.block_bytes;
    }
    const int slot = s.pt % kStages;
    ptx::mbar_arrive_expect_tx(&s.bar[slot], p.block_bytes);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(s.ring + slot * kStagePitch), "l"(s.p_src), "r"(p.block_bytes), "r"(ptx::smem_u32(&s.bar[slot]))
                 : "memory");
    s.p_src += p.block_bytes;
    --s.p_left;
    ++s.pt;
}

// Waits (bounded) for every requested block that has not been consumed: before leaving on an error, so
// that no copy lands in shared memory that already belongs to another CTA.
__device__ __forceinline__ void stream_drain(Stream& s) {
    const unsigned pt = __shfl_sync(0xffffffffu, s.pt, 0);
    for (unsigned c = s.ct; c < pt; ++c) ptx::mbar_wait_bounded(&s.bar[c % kStages], (c / kStages) & 1, 1u << 16);
}

__device__ __noinline__ void stamp(const StackParams& p, int& slot) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.timeline[slot] = t;
    }
    ++slot;
}

// ---- grid barrier -------------------------------------------------------------------------------
// Monotonic counter, zeroed by the host before the launch. Returns false when the step is being abandoned.
__device__ __noinline__ bool grid_barrier(const StackParams& p, unsigned& epoch, int* s_abort) {
    ++epoch;
    __syncthreads();
    if (threadIdx.x == kFenceLane) {
        __threadfence();
        atomicAdd(p.barrier, 1u);
        const unsigned target = epoch * gridDim.x;
        bool ok = false;
        for (unsigned i = 0; i < (1u << 21); ++i) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.barrier) : "memory");
            if (v >= target) { ok = true; break; }
            if ((i & 63) == 63) {
                int st;
                asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(st) : "l"(p.status) : "memory");
                if (st != 0) break;
            }
            if (i > 32) __nanosleep(32);
        }
        if (!ok) {
            atomicCAS(p.status, 0, 700 + static_cast<int>(epoch % 100));
            *s_abort = 1;
        }
        __threadfence();
    }
    __syncthreads();
    return *s_abort == 0;
}

// ---- phase A / F / final: residual add + RMSNorm (+ quantiser) of one token row by one CTA -----------------
// The row is staged in shared memory. The sum of squares follows the reference's T = norm_threads launch
// (rms_norm.cu:23-49, :69-70): real warp w plays virtual warps w*VW .. w*VW+VW-1 — thread-strided partial
// sums, a shuffle-down tree inside each (virtual) warp, a tree over the warp partials — so the normed values
// are the reference's. Normalising and quantising then go 8 elements (one 128-bit piece) per thread: the
// g/8 threads of a group find its absmax with shuffles (int8_gemm.cu:147-211 is order-free there).
// Written as plain loops on purpose: the code of a phase runs once per layer and must stay small.
template <int GM>
__device__ __noinline__ void row_phase(const StackParams& p, int row, const __half* norm_w, bool add_delta,
                                       bool final_out, float* s_red, __half* row_s) {
    constexpr int LANES = GM / 8;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.dim, T = p.norm_threads, VW = T / kThreads, G = K / GM;
    const size_t base = static_cast<size_t>(row) * K;
    const int pieces = K / 8;
    uint4 xv[2], dv[2], wv[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {  // every load first (K <= 4096: at most two pieces per thread)
        const int c8 = tid + i * kThreads;
        const int cc = c8 < pieces ? c8 : 0;
        xv[i] = ldcg128(p.x + base + cc * 8);
        dv[i] = ldcg128((add_delta ? p.delta : p.x) + base + cc * 8);
        wv[i] = __ldg(reinterpret_cast<const uint4*>(norm_w) + cc);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c8 = tid + i * kThreads;
        if (c8 < pieces) {
            if (add_delta) {
                __half* hx = reinterpret_cast<__half*>(&xv[i]);
                const __half* hd = reinterpret_cast<const __half*>(&dv[i]);
#pragma unroll
                for (int e = 0; e < 8; ++e) hx[e] = __float2half(__half2float(hx[e]) + __half2float(hd[e]));
                *reinterpret_cast<uint4*>(p.x + base + c8 * 8) = xv[i];
            }
            reinterpret_cast<uint4*>(row_s)[c8] = xv[i];
        }
    }
    __syncthreads();
#pragma unroll 1
    for (int k = 0; k < VW; ++k) {
        float local_sum = 0.0f;
#pragma unroll 1
        for (int e = (warp * VW + k) * 32 + lane; e < K; e += T) {
            float val = __half2float(row_s[e]);
            local_sum += val * val;
        }
        for (int offset = 16; offset > 0; offset /= 2) local_sum += __shfl_down_sync(0xffffffffu, local_sum, offset);
        if (lane == 0) s_red[warp * VW + k] = local_sum;
    }
    __syncthreads();
    float total_sum = 0.0f;
    if (warp == 0) {
        if (lane < T / 32) total_sum = s_red[lane];
        for (int offset = 16; offset > 0; offset /= 2) total_sum += __shfl_down_sync(0xffffffffu, total_sum, offset);
    }
    __syncthreads();
    if (tid == 0) s_red[0] = rsqrtf(total_sum / K + p.eps);
    __syncthreads();
    const float rms = s_red[0];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c8 = tid + i * kThreads;
        const bool live = c8 < pieces;  // whole warps are live or not (pieces is a multiple of 32)
        __half* hx = reinterpret_cast<__half*>(&xv[i]);
        const __half* hw = reinterpret_cast<const __half*>(&wv[i]);
        float v[8], amax = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float val = __half2float(hx[e]) * rms;
            hx[e] = __float2half(val * __half2float(hw[e]));
            v[e] = __half2float(hx[e]);
            amax = fmaxf(amax, fabsf(v[e]));
        }
        if (final_out) {
            if (live) *reinterpret_cast<uint4*>(p.out + base + c8 * 8) = xv[i];
            continue;
        }
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (!live) continue;
        float scale = amax / 127.0f;
        if (scale < 1e-8f) scale = 1e-8f;
        if ((lane & (LANES - 1)) == 0) p.xs[static_cast<size_t>(row) * G + (c8 * 8) / GM] = scale;
        const float inv_scale = 1.0f / scale;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            int q = __float2int_rn(v[e] * inv_scale);
            q = max(-127, min(127, q));
            if (e < 4) lo |= (static_cast<uint32_t>(q) & 0xffu) << (8 * e);
            else hi |= (static_cast<uint32_t>(q) & 0xffu) << (8 * (e - 4));
        }
        *reinterpret_cast<uint2*>(p.xq + base + c8 * 8) = make_uint2(lo, hi);
    }
    __syncthreads();  // s_red and the staged row may be reused
}

// Stores a finished 16-row tile held in MMA fragment layout (rows gq / gq+8, tokens 2c / 2c+1), with the
// SwiGLU epilogue for the gate/up linear. Kept out of line: it is called from several places of a phase
// and the phases must stay small enough for the instruction cache.
__device__ __noinline__ void store_tile_fn(const GemvShape& sh, __half* Y, int M, int rt, int gq, int c, float v0, float v1,
                                           float v2, float v3) {
    const float v[4] = {v0, v1, v2, v3};
    const int rA = rt * 16 + gq;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int tok = 2 * c + e;
        if (tok >= M) continue;
        if (sh.epilogue == W8A8_EPI_SWIGLU) {
            if (rA + 8 < sh.N) {
                const float g16 = __half2float(__float2half(v[e]));
                const __half s16 = __float2half(g16 / (1.0f + expf(-g16)));
                const float u16 = __half2float(__float2half(v[2 + e]));
                Y[static_cast<size_t>(tok) * (sh.N / 2) + rt * 8 + gq] = __float2half(__half2float(s16) * u16);
            }
        } else {
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int row = rA + 8 * hrow;
                if (row < sh.N) Y[static_cast<size_t>(tok) * sh.N + row] = __float2half(v[2 * hrow + e]);
            }
        }
    }
}

// ---- phases B / E / G / I: one W8A8 linear over the packed stream, M <= 8 ------------------------------------
// The consumer of w8a8_gemv_packed.cu for one token tile, fed by the warp's running stream.
// The activation codes and scales of the whole batch are first copied into shared memory (every warp reads
// all of K over its range, and a read from L2 per block would put a memory round trip on each step);
// rows are K + 64 bytes apart so that a quarter-warp's eight 16-byte reads fall into different banks.
template <int GM>
__device__ __noinline__ bool gemv_phase(const StackParams& p, Stream& s_ref, const GemvShape& sh, const int8_t* Xq,
                                           const float* Xs, __half* Y, unsigned gw, int lane, unsigned char* stage,
                                           float (*red_s)[2][4 * 32], int* cnt_s) {
    Stream s = s_ref;  // in registers for the length of the phase
    constexpr int GPU = GM == 64 ? 4 : GM == 128 ? 2 : 1;
    const int gq = lane >> 2, c = lane & 3;
    const unsigned warp = gw % kWarps;
    unsigned cu0, n_cta, nw_cta, u0, u1;
    warp_range(sh, blockIdx.x, gridDim.x, warp, cu0, n_cta, nw_cta, u0, u1);
    const int T = static_cast<int>(u1 - u0);
    const int M = p.B, upt = sh.upt;
    const int pitch = sh.K + 64;
    float* scales_s = reinterpret_cast<float*>(stage + 8 * pitch);
    {
        const uint32_t dst0 = ptx::smem_u32(stage);
        const int per_row = sh.K / 16;
        for (int i = threadIdx.x; i < M * per_row; i += kThreads) {
            const int row = i / per_row, piece = i - row * per_row;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + row * pitch + piece * 16),
                         "l"(Xq + static_cast<size_t>(row) * sh.K + piece * 16) : "memory");
        }
        for (int i = threadIdx.x; i < M * sh.G; i += kThreads) scales_s[i] = ldcg_f(Xs + i);  // past L1, like the codes
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();
    }
    const uint32_t xq_s = ptx::smem_u32(stage) + min(gq, M - 1) * pitch + c * 16;
    const float* xsp0 = scales_s + min(2 * c, M - 1) * sh.G;
    const float* xsp1 = scales_s + min(2 * c + 1, M - 1) * sh.G;

    int P[4] = {0, 0, 0, 0}, Q[4] = {0, 0, 0, 0};
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};

    auto store_tile = [&](int rt, const float (&v)[4]) { store_tile_fn(sh, Y, M, rt, gq, c, v[0], v[1], v[2], v[3]); };
    auto warp_of_unit = [&](unsigned u) -> unsigned {  // the warp of this CTA whose run holds unit u
        return ((u - cu0 + 1) * nw_cta - 1) / n_cta;
    };
    const int cta_rt0 = static_cast<int>(cu0 / upt);
    // Called when the warp has added its last unit of row tile rt into acc. A cut tile: the partial goes to the
    // warp's slot, the arrival is counted, and whichever warp arrives last adds the partials in ascending-K
    // order and stores. Nothing waits.
    auto finish_tile = [&](int rt) {
        const unsigned t_lo = static_cast<unsigned>(rt) * upt, t_hi = t_lo + upt;
        if (u0 <= t_lo && t_hi <= u1) {
            store_tile(rt, acc);
        } else {
            const unsigned first = warp_of_unit(t_lo), last = warp_of_unit(t_hi - 1);
            const int my_slot = (static_cast<int>(u0 / upt) == rt) ? 0 : 1;
            float* mine = red_s[warp][my_slot];
#pragma unroll
            for (int r = 0; r < 4; ++r) mine[r * 32 + lane] = acc[r];
            __syncwarp();
            int old = 0;
            if (lane == 0) {
                __threadfence_block();
                old = atomicAdd(&cnt_s[rt - cta_rt0], 1);
            }
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old == static_cast<int>(last - first)) {
                __threadfence_block();
                float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                for (unsigned ww = first; ww <= last; ++ww) {
                    const unsigned wu0 = cu0 + ww * n_cta / nw_cta;
                    const float* src = red_s[ww][(static_cast<int>(wu0 / upt) == rt) ? 0 : 1];
#pragma unroll
                    for (int r = 0; r < 4; ++r) sum[r] += src[r * 32 + lane];
                }
                store_tile(rt, sum);
                if (lane == 0) cnt_s[rt - cta_rt0] = 0;  // the next linear starts from zero again
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[r] = 0.0f;
    };
    auto promote = [&](__half hsa, __half hsb, float x0, float x1) {
        const float fa = __half2float(hsa), fb = __half2float(hsb);
#pragma unroll
        for (int r = 0; r < 4; ++r) { P[r] += Q[r]; Q[r] = 0; }
        acc[0] = __fmaf_rn(__fmul_rn(static_cast<float>(P[0]), fa), x0, acc[0]);
        acc[1] = __fmaf_rn(__fmul_rn(static_cast<float>(P[1]), fa), x1, acc[1]);
        acc[2] = __fmaf_rn(__fmul_rn(static_cast<float>(P[2]), fb), x0, acc[2]);
        acc[3] = __fmaf_rn(__fmul_rn(static_cast<float>(P[3]), fb), x1, acc[3]);
        P[0] = P[1] = P[2] = P[3] = 0;
    };

    int ub = static_cast<int>(u0 % upt), rt = static_cast<int>(u0 / upt);
    uint4 xc[4];
    float xsc[GPU][2];
    bool ok = true;
    for (int t = 0; t < T; ++t) {
        const int slot = s.ct % kStages;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) xc[ch] = lds128(xq_s + ub * 256 + ch * 64);
#pragma unroll
        for (int q = 0; q < GPU; ++q) {
            xsc[q][0] = xsp0[ub * GPU + q];
            xsc[q][1] = xsp1[ub * GPU + q];
        }
        if (!ptx::mbar_wait_bounded(&s.bar[slot], (s.ct / kStages) & 1)) {
            if (lane == 0) atomicCAS(p.status, 0, 600 + slot);
            ok = false;
            break;
        }
        const uint32_t st = s.ring + slot * kStagePitch;
        __half sa[GPU], sb[GPU];
#pragma unroll
        for (int q = 0; q < GPU; ++q) {
            sa[q] = __ushort_as_half(static_cast<unsigned short>(lds16(st + kBlockW + (gq * GPU + q) * 2)));
            sb[q] = __ushort_as_half(static_cast<unsigned short>(lds16(st + kBlockW + ((gq + 8) * GPU + q) * 2)));
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            const uint32_t fa = st + ch * 1024 + lane * 16;
            const uint4 wa = lds128(fa), wb = lds128(fa + 512);
            mma_s8(P, wa.x, wb.x, wa.y, wb.y, xc[ch].x, xc[ch].y);
            mma_s8(Q, wa.z, wb.z, wa.w, wb.w, xc[ch].z, xc[ch].w);
            if (GM == 64) promote(sa[ch % GPU], sb[ch % GPU], xsc[ch % GPU][0], xsc[ch % GPU][1]);
            if (GM == 128 && (ch & 1))
                promote(sa[(ch >> 1) % GPU], sb[(ch >> 1) % GPU], xsc[(ch >> 1) % GPU][0], xsc[(ch >> 1) % GPU][1]);
        }
        __syncwarp();
        ++s.ct;
        if (lane == 0) stream_issue(s, p, gw);
        if (GM == 256) promote(sa[0], sb[0], xsc[0][0], xsc[0][1]);
        // one call site for the tile end: the row tile is complete, or the range ends inside it
        ++ub;
        if (ub == upt || t + 1 == T) {
            finish_tile(rt);
            if (ub == upt) { ub = 0; ++rt; }
        }
    }
    s_ref = s;
    return ok;
}

// ---- phase C: qk-norm + RoPE + KV write + attention over one context slice ------------------------------------
struct KvFrag {
    uint4 k[2][4];
    uint4 v[4][2];
};

// One warp, one head of the new token: per-head RMSNorm in the reference's order (rms_norm.cu:23-49 with
// a 128-thread block) and interleaved-pair RoPE (rope.cu:36-45). h: elements lane, 32+lane, 64+lane, 96+lane.
__device__ __forceinline__ void head_norm_rope(__half (&h)[4], bool with_norm, const __half (&w)[4], float eps,
                                               const float (&fr)[4], int pos, int lane) {
    if (with_norm) {
        float part[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            float val = __half2float(h[v]);
            float local_sum = 0.0f;
            local_sum += val * val;
            for (int offset = 16; offset > 0; offset /= 2) local_sum += __shfl_down_sync(0xffffffffu, local_sum, offset);
            part[v] = __shfl_sync(0xffffffffu, local_sum, 0);
        }
        float total_sum = (part[0] + part[2]) + (part[1] + part[3]);
        const float rms = rsqrtf(total_sum / kHeadDim + eps);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            float val = __half2float(h[v]) * rms;
            h[v] = __float2half(val * __half2float(w[v]));
        }
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        float angle = fr[v] * static_cast<float>(pos);
        float cos_a = cosf(angle), sin_a = sinf(angle);
        const float mine = __half2float(h[v]);
        const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
        float q0 = (lane & 1) ? other : mine, q1 = (lane & 1) ? mine : other;
        h[v] = (lane & 1) ? __float2half(q0 * sin_a + q1 * cos_a) : __float2half(q0 * cos_a - q1 * sin_a);
    }
}

struct AttnSmem {
    float red_acc[kWarps][kQPerKv][kHeadDim];
    float red_m[kWarps][kQPerKv];
    float red_l[kWarps][kQPerKv];
    __half q_s[kQPerKv][kHeadDim];
    __half out_s[kQPerKv * kHeadDim];
};

// Physical numbers of the warp's first 32 KV blocks (lane i: its i-th block). They depend on the sequence and on
// the context slice only, not on the layer, so the kernel reads them once and keeps them in a register.
__device__ __forceinline__ int first_phys(const StackParams& p, int item, int warp, int lane, int seq_len) {
    const int S = p.S, s = item % S, b = item / (S * p.n_kv);
    const int n_blocks = (seq_len + kBlockTokens - 1) / kBlockTokens;
    const int bi = s + warp * S + lane * S * kWarps;
    return bi < n_blocks ? __ldg(p.block_table + static_cast<size_t>(b) * p.max_blocks + bi) : 0;
}

__device__ __noinline__ void attn_phase(const StackParams& p, const w8a8_decode_layer& L, int layer, int item,
                                           AttnSmem& sm, int pos, int seq_len, int phys_first) {
    const int S = p.S;
    const int s = item % S, kvh = (item / S) % p.n_kv, b = item / (S * p.n_kv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int total_heads = p.n_q + 2 * p.n_kv;
    // Everything the prologue reads is requested here, before the first value is used: each dependent read
    // is a round trip to L2, and a chain of five of them was longer than the attention loop itself.
    const __half* qkv_row = p.qkv + static_cast<size_t>(b) * total_heads * kHeadDim;
    const bool role_q = warp < kQPerKv, is_k = warp == kQPerKv, is_v = warp == kQPerKv + 1;
    __half hq[4], wq[4];
    float fr[4];
    const __half* norm_w = static_cast<const __half*>(role_q ? L.q_norm : L.k_norm);
    {
        const __half* src = qkv_row + (role_q ? kvh * kQPerKv + warp : p.n_q + (is_k ? 0 : p.n_kv) + kvh) * kHeadDim;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            hq[v] = (role_q || is_k || is_v) ? ldcg_h(src + v * 32 + lane) : __float2half(0.0f);
            wq[v] = norm_w ? __ldg(norm_w + v * 32 + lane) : __float2half(1.0f);
            fr[v] = __ldg(p.freqs + ((v * 32 + lane) >> 1));
        }
    }
    const int n_blocks = (seq_len + kBlockTokens - 1) / kBlockTokens;
    const bool owner = ((pos / kBlockTokens) % S) == s;  // this CTA attends over the block the new token joins

    // The K and V blocks do not depend on this step's q: the first two are requested before the new token's
    // q / k / v rows are normalised and rotated, so that the two latencies overlap. The one block that does
    // depend on this step (the block the new token joins, attended over by the owner) waits for the write.
    const int stride = S * kWarps, first = s + warp * S;
    const int n_mine = first < n_blocks ? (n_blocks - first + stride - 1) / stride : 0;
    auto fetch_phys = [&](int it0) -> int {
        const int bi = first + (it0 + lane) * stride;
        return bi < n_blocks ? __ldg(p.block_table + static_cast<size_t>(b) * p.max_blocks + bi) : 0;
    };
    int phys_mine = phys_first;
    auto load = [&](KvFrag& f, int it) {
        if ((it & 31) == 0 && it > 0) phys_mine = fetch_phys(it);
        const int phys = __shfl_sync(0xffffffffu, phys_mine, it & 31);
        const int bi = first + it * stride;
        const int tokens = min(kBlockTokens, seq_len - bi * kBlockTokens);
        const size_t base = (((static_cast<size_t>(phys) * p.n_layers + layer) * p.n_kv + kvh) * kBlockTokens) * kHeadDim;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int tok = j * 8 + g;
            const __half* row = p.k_cache + base + static_cast<size_t>(tok < tokens ? tok : 0) * kHeadDim;
#pragma unroll
            for (int i = 0; i < 4; ++i) f.k[j][i] = ldcg128(row + (i * 4 + t) * 8);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int tok = 2 * t + (q & 1) + 8 * (q >> 1);
            const __half* row = p.v_cache + base + static_cast<size_t>(tok < tokens ? tok : 0) * kHeadDim;
#pragma unroll
            for (int h = 0; h < 2; ++h) f.v[q][h] = ldcg128(row + (g + 8 * h) * 8);
        }
    };
    KvFrag fa, fb;
    const int new_bi = pos / kBlockTokens;
    const bool pre0 = n_mine > 0 && !(owner && first == new_bi);
    const bool pre1 = n_mine > 1 && !(owner && first + stride == new_bi);
    if (pre0) load(fa, 0);
    if (pre1) load(fb, 1);

    // warps 0..3: a query head each; in the owner CTA warp 4: the new k row, warp 5: the new v row
    if (role_q || ((is_k || is_v) && owner)) {
        if (!is_v) head_norm_rope(hq, norm_w != nullptr, wq, p.eps, fr, pos, lane);
        if (role_q) {
#pragma unroll
            for (int v = 0; v < 4; ++v) sm.q_s[warp][v * 32 + lane] = hq[v];
        } else {
            const int phys = __ldg(p.block_table + static_cast<size_t>(b) * p.max_blocks + new_bi);
            if (phys >= 0) {
                __half* dst = (is_k ? p.k_cache : p.v_cache) +
                              ((((static_cast<size_t>(phys) * p.n_layers + layer) * p.n_kv + kvh) * kBlockTokens) +
                               pos % kBlockTokens) * kHeadDim;
#pragma unroll
                for (int v = 0; v < 4; ++v) dst[v * 32 + lane] = hq[v];
            }
        }
    }
    __syncthreads();  // q in shared memory; the new token's k and v row written (read back past L1 below)
    if (n_mine > 0 && !pre0) load(fa, 0);
    if (n_mine > 1 && !pre1) load(fb, 1);

    uint32_t qa[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (g < kQPerKv) v = *reinterpret_cast<const uint4*>(&sm.q_s[g][(i * 4 + t) * 8]);
        qa[i][0] = v.x; qa[i][1] = v.y; qa[i][2] = v.z; qa[i][3] = v.w;
    }
    float m_run = -1e30f, l_run = 0.0f;
    float o[16][2];
#pragma unroll
    for (int n = 0; n < 16; ++n) { o[n][0] = 0.0f; o[n][1] = 0.0f; }
    auto compute = [&](const KvFrag& f, int it) {
        const int bi = first + it * stride;
        const int tokens = min(kBlockTokens, seq_len - bi * kBlockTokens);
        float sc[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            sc[j][0] = 0.0f; sc[j][1] = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    mma_top_rows(sc[j][0], sc[j][1], qa[i][2 * h], qa[i][2 * h + 1], reg_of(f.k[j][i], 2 * h),
                                 reg_of(f.k[j][i], 2 * h + 1));
        }
        float mx = -1e30f;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = j * 8 + 2 * t + e;
                sc[j][e] = tok < tokens ? sc[j][e] * p.sm_scale : -1e30f;
                mx = fmaxf(mx, sc[j][e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float new_m = fmaxf(m_run, mx);
        const float corr = __expf(m_run - new_m);
        m_run = new_m;
        const __half2 p0 = __floats2half2_rn(__expf(sc[0][0] - new_m), __expf(sc[0][1] - new_m));
        const __half2 p1 = __floats2half2_rn(__expf(sc[1][0] - new_m), __expf(sc[1][1] - new_m));
        const float2 f0 = __half22float2(p0), f1 = __half22float2(p1);
        l_run = l_run * corr + ((f0.x + f0.y) + (f1.x + f1.y));
        const uint32_t pa0 = *reinterpret_cast<const uint32_t*>(&p0), pa2 = *reinterpret_cast<const uint32_t*>(&p1);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int n = h * 8 + e;
                const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
                const uint32_t b0 = __byte_perm(reg_of(f.v[0][h], e >> 1), reg_of(f.v[1][h], e >> 1), sel);
                const uint32_t b1 = __byte_perm(reg_of(f.v[2][h], e >> 1), reg_of(f.v[3][h], e >> 1), sel);
                o[n][0] *= corr;
                o[n][1] *= corr;
                mma_top_rows(o[n][0], o[n][1], pa0, pa2, b0, b1);
            }
    };
    for (int it = 0; it < n_mine;) {  // fa holds block `it`, fb block `it + 1`
        compute(fa, it);
        if (it + 2 < n_mine) load(fa, it + 2);
        if (++it >= n_mine) break;
        compute(fb, it);
        if (it + 2 < n_mine) load(fb, it + 2);
        ++it;
    }
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (g < kQPerKv) {
        if (t == 0) { sm.red_m[warp][g] = m_run; sm.red_l[warp][g] = l_run; }
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                sm.red_acc[warp][g][(2 * t + 8 * h) * 8 + e] = o[h * 8 + e][0];
                sm.red_acc[warp][g][(2 * t + 1 + 8 * h) * 8 + e] = o[h * 8 + e][1];
            }
    }
    __syncthreads();
    if (threadIdx.x < kQPerKv * 32) {
        const int hh = threadIdx.x >> 5, d0 = (threadIdx.x & 31) * 4;
        float m = -1e30f;
        for (int w = 0; w < kWarps; ++w) m = fmaxf(m, sm.red_m[w][hh]);
        float l = 0.0f, a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int w = 0; w < kWarps; ++w) {
            const float scw = __expf(sm.red_m[w][hh] - m);
            l += sm.red_l[w][hh] * scw;
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] += sm.red_acc[w][hh][d0 + i] * scw;
        }
        float* dst = p.attn_part + (static_cast<size_t>(item) * kQPerKv + hh) * kPartStride;
        *reinterpret_cast<float4*>(dst + 4 + d0) = make_float4(a[0], a[1], a[2], a[3]);
        if ((threadIdx.x & 31) == 0) { dst[0] = m; dst[1] = l; }
    }
    __syncthreads();  // shared memory is free for the CTA's next item
}

// ---- phase D: merge the context slices of one (sequence, kv head), quantise for wo -----------------------------
__device__ __noinline__ void merge_phase(const StackParams& p, int pair, AttnSmem& sm) {
    const int S = p.S, kvh = pair % p.n_kv, b = pair / p.n_kv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq_len = __ldg(p.seq_lens + b);
    if (threadIdx.x < kQPerKv * 32) {
        const int hh = threadIdx.x >> 5, d0 = (threadIdx.x & 31) * 4;
        const float* src0 = p.attn_part + (static_cast<size_t>(pair) * S * kQPerKv + hh) * kPartStride;
        float4 ml[8], v4s[8];  // S <= 8; every load is requested before the first value is used
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const float* src = src0 + static_cast<size_t>(r < S ? r : 0) * kQPerKv * kPartStride;
            ml[r] = ldcg_f4(src);
            v4s[r] = ldcg_f4(src + 4 + d0);
        }
        float m = -1e30f;
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (r < S) m = fmaxf(m, ml[r].x);
        float l = 0.0f, a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (r < S) {
                const float scr = __expf(ml[r].x - m);
                l += ml[r].y * scr;
                a[0] += v4s[r].x * scr; a[1] += v4s[r].y * scr; a[2] += v4s[r].z * scr; a[3] += v4s[r].w * scr;
            }
        const float inv = seq_len > 0 ? 1.0f / l : 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) sm.out_s[hh * kHeadDim + d0 + i] = __float2half(seq_len > 0 ? a[i] * inv : 0.0f);
    }
    __syncthreads();
    const int gsz = p.g, K = p.n_q * kHeadDim, G = K / gsz;
    const int ch0 = kvh * kQPerKv * kHeadDim;
    const int groups_here = (kQPerKv * kHeadDim) / gsz;
    for (int j = warp; j < groups_here; j += kWarps) {
        float amax = 0.0f;
        for (int e = lane; e < gsz; e += 32) amax = fmaxf(amax, fabsf(__half2float(sm.out_s[j * gsz + e])));
        amax = warp_max(amax);
        float scale = amax / 127.0f;
        if (scale < 1e-8f) scale = 1e-8f;
        if (lane == 0) p.as_[static_cast<size_t>(b) * G + ch0 / gsz + j] = scale;
        const float inv_scale = 1.0f / scale;
        for (int e = lane; e < gsz; e += 32) {
            int qv = __float2int_rn(__half2float(sm.out_s[j * gsz + e]) * inv_scale);
            qv = max(-127, min(127, qv));
            p.aq[static_cast<size_t>(b) * K + ch0 + j * gsz + e] = static_cast<int8_t>(qv);
        }
    }
    __syncthreads();
}

// ---- phase H: quantise the SwiGLU output; one warp per (row, 256 channels) ---------------------------------------
template <int GM>
__device__ __noinline__ void actquant_phase(const StackParams& p, unsigned gw, unsigned total_warps, int lane) {
    constexpr int LANES = GM / 8;  // lanes per group
    const int chunks = p.inter / 256, G = p.inter / p.g;
    for (unsigned it = gw; it < static_cast<unsigned>(p.B * chunks); it += total_warps) {
        const int row = it / chunks, e = (it % chunks) * 256 + lane * 8;
        const uint4 u = ldcg128(p.act + static_cast<size_t>(row) * p.inter + e);
        const __half* h = reinterpret_cast<const __half*>(&u);
        float v[8], amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = __half2float(h[i]);
            amax = fmaxf(amax, fabsf(v[i]));
        }
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        float scale = amax / 127.0f;
        if (scale < 1e-8f) scale = 1e-8f;
        if ((lane & (LANES - 1)) == 0) p.acts[static_cast<size_t>(row) * G + e / GM] = scale;
        const float inv_scale = 1.0f / scale;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int q = __float2int_rn(v[i] * inv_scale);
            q = max(-127, min(127, q));
            if (i < 4) lo |= (static_cast<uint32_t>(q) & 0xffu) << (8 * i);
            else hi |= (static_cast<uint32_t>(q) & 0xffu) << (8 * (i - 4));
        }
        *reinterpret_cast<uint2*>(p.actq + static_cast<size_t>(row) * p.inter + e) = make_uint2(lo, hi);
    }
}

// ---------------------------------------------------------------------------------------------------------------
template <int GM>
__global__ void __launch_bounds__(kThreads, 1) decode_stack_kernel(const __grid_constant__ StackParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[kWarps][kStages];
    __shared__ float s_red[32];
    __shared__ int s_abort;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ float red_s[kWarps][2][4 * 32];
    __shared__ int cnt_s[kLocalTiles];
    for (int i = threadIdx.x; i < kLocalTiles; i += kThreads) cnt_s[i] = 0;
    const unsigned gw = blockIdx.x * kWarps + warp, total_warps = gridDim.x * kWarps;
    const uint32_t base_u32 = (ptx::smem_u32(smem_raw) + 127u) & ~127u;
    // after the ring: one region used by turns for the attention scratch and for the staged activation codes
    unsigned char* stage = smem_raw + (base_u32 - ptx::smem_u32(smem_raw)) + kWarps * kRingBytes;
    AttnSmem& asm_ = *reinterpret_cast<AttnSmem*>(stage);

    Stream s;
    s.ring = base_u32 + warp * kRingBytes;
    s.bar = bars[warp];
    s.pt = 0; s.ct = 0; s.pj = -1; s.p_left = 0; s.p_src = nullptr; s.next_img = nullptr;
    if (threadIdx.x == 0) s_abort = 0;
    if (lane == 0) {
        for (int i = 0; i < kStages; ++i) ptx::mbar_init(&s.bar[i], 1);
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
        s.next_img = packed_image(p, 0);
        for (int i = 0; i < kStages; ++i) stream_issue(s, p, gw);
    }
    __syncwarp();
    __syncthreads();

    // layer-invariant inputs of the attention phase, read once
    const int n_items = p.B * p.n_kv * p.S;
    int a_pos = 0, a_len = 0, a_phys = 0;
    if (static_cast<int>(blockIdx.x) < n_items) {
        const int b = blockIdx.x / (p.S * p.n_kv);
        a_pos = __ldg(p.positions + b);
        a_len = __ldg(p.seq_lens + b);
        a_phys = first_phys(p, blockIdx.x, warp, lane, a_len);
    }
    unsigned epoch = 0;
    int ts = 0;  // 19 stamps per layer: after each of the 9 phases and each of the 9 barriers, +1 at the top
    bool ok = true;
    stamp(p, ts);
    for (int l = 0; l < p.n_layers && ok; ++l) {
        const w8a8_decode_layer& L = p.layers[l];
        // A
        if (static_cast<int>(blockIdx.x) < p.B)
            row_phase<GM>(p, blockIdx.x, static_cast<const __half*>(L.attn_norm), l > 0, false, s_red,
                          reinterpret_cast<__half*>(stage));
        stamp(p, ts);
        if (!(ok = grid_barrier(p, epoch, &s_abort))) break;
        stamp(p, ts);
        // B
        ok = gemv_phase<GM>(p, s, p.gs[0], p.xq, p.xs, p.qkv, gw, lane, stage, red_s, cnt_s);
        stamp(p, ts);
        if (!grid_barrier(p, epoch, &s_abort) || !ok) { ok = false; break; }
        stamp(p, ts);
        // C
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            if (item != static_cast<int>(blockIdx.x)) {  // a CTA with more than one item looks the later ones up again
                const int b = item / (p.S * p.n_kv);
                a_pos = __ldg(p.positions + b);
                a_len = __ldg(p.seq_lens + b);
                a_phys = first_phys(p, item, warp, lane, a_len);
            }
            attn_phase(p, L, l, item, asm_, a_pos, a_len, a_phys);
        }
        if (n_items > static_cast<int>(gridDim.x)) {  // back to the first item's values for the next layer
            const int b = blockIdx.x / (p.S * p.n_kv);
            a_pos = __ldg(p.positions + b);
            a_len = __ldg(p.seq_lens + b);
            a_phys = first_phys(p, blockIdx.x, warp, lane, a_len);
        }
        stamp(p, ts);
        if (!(ok = grid_barrier(p, epoch, &s_abort))) break;
        stamp(p, ts);
        // D
        for (int pair = blockIdx.x; pair < p.B * p.n_kv; pair += gridDim.x) merge_phase(p, pair, asm_);
        stamp(p, ts);
        if (!(ok = grid_barrier(p, epoch, &s_abort))) break;
        stamp(p, ts);
        // E
        ok = gemv_phase<GM>(p, s, p.gs[1], p.aq, p.as_, p.delta, gw, lane, stage, red_s, cnt_s);
        stamp(p, ts);
        if (!grid_barrier(p, epoch, &s_abort) || !ok) { ok = false; break; }
        stamp(p, ts);
        // F
        if (static_cast<int>(blockIdx.x) < p.B)
            row_phase<GM>(p, blockIdx.x, static_cast<const __half*>(L.ffn_norm), true, false, s_red,
                          reinterpret_cast<__half*>(stage));
        stamp(p, ts);
        if (!(ok = grid_barrier(p, epoch, &s_abort))) break;
        stamp(p, ts);
        // G
        ok = gemv_phase<GM>(p, s, p.gs[2], p.xq, p.xs, p.act, gw, lane, stage, red_s, cnt_s);
        stamp(p, ts);
        if (!grid_barrier(p, epoch, &s_abort) || !ok) { ok = false; break; }
        stamp(p, ts);
        // H
        actquant_phase<GM>(p, gw, total_warps, lane);
        stamp(p, ts);
        if (!(ok = grid_barrier(p, epoch, &s_abort))) break;
        stamp(p, ts);
        // I
        ok = gemv_phase<GM>(p, s, p.gs[3], p.actq, p.acts, p.delta, gw, lane, stage, red_s, cnt_s);
        stamp(p, ts);
        if (!grid_barrier(p, epoch, &s_abort) || !ok) { ok = false; break; }
        stamp(p, ts);
    }
    if (ok) {
        if (static_cast<int>(blockIdx.x) < p.B)
            row_phase<GM>(p, blockIdx.x, p.final_norm, true, true, s_red, reinterpret_cast<__half*>(stage));
        stamp(p, ts);
    } else {
        stream_drain(s);
    }
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

struct Scratch {
    size_t qkv, xq, xs, aq, as_, act, actq, acts, delta, attn_part, barrier, timeline, total;
};

Scratch layout(const w8a8_decode_stack& d, int S) {
    Scratch sc;
    const size_t B = d.batch, g = d.group_size;
    const size_t qkv_n = static_cast<size_t>(d.n_q_heads + 2 * d.n_kv_heads) * kHeadDim;
    const size_t attn_k = static_cast<size_t>(d.n_q_heads) * kHeadDim;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align256(bytes); return o; };
    sc.qkv = take(B * qkv_n * 2);
    sc.xq = take(B * d.dim);
    sc.xs = take(B * (d.dim / g) * 4);
    sc.aq = take(B * attn_k);
    sc.as_ = take(B * (attn_k / g) * 4);
    sc.act = take(B * d.inter * 2);
    sc.actq = take(B * d.inter);
    sc.acts = take(B * (d.inter / g) * 4);
    sc.delta = take(B * d.dim * 2);
    sc.attn_part = take(B * d.n_kv_heads * S * kQPerKv * kPartStride * 4);
    sc.barrier = take(256);
    sc.timeline = take(static_cast<size_t>(18 * d.n_layers + 2) * 8);
    sc.total = off;
    return sc;
}

int num_sms() {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        v <= 0)
        v = 148;
    return v;
}

int slices_for(const w8a8_decode_stack& d, int sms) {
    const int want = sms / (d.batch * d.n_kv_heads);
    return want >= 8 ? 8 : want >= 4 ? 4 : want >= 2 ? 2 : 1;  // the stand-alone attention launch picks the same
}

const char* check(const w8a8_decode_stack& d) {
    if (!d.layers || !d.final_norm || !d.rope_freqs || !d.positions || !d.seq_lens || !d.block_table || !d.k_cache ||
        !d.v_cache || !d.x || !d.out)
        return "null pointer in the stack descriptor";
    if (d.n_layers < 1 || d.batch < 1 || d.batch > 8) return "batch must be 1..8";
    if (d.head_dim != kHeadDim || d.n_kv_heads < 1 || d.n_q_heads != kQPerKv * d.n_kv_heads)
        return "needs head_dim 128 and 4 query heads per kv head";
    if (d.group_size != 64 && d.group_size != 128 && d.group_size != 256) return "group size must be 64, 128 or 256";
    if (d.dim % 256 != 0 || d.dim < 256 || d.dim > 4096) return "dim must be a multiple of 256 in 256..4096";
    if (d.inter % 256 != 0 || d.inter < 256) return "inter must be a multiple of 256";
    return nullptr;
}

}  // namespace

size_t decode_stack_workspace_bytes(const w8a8_decode_stack& d) {
    if (check(d)) return 0;
    return layout(d, slices_for(d, num_sms())).total;
}

int decode_stack_timeline(const w8a8_decode_stack& d, const unsigned char* workspace, unsigned long long* out, int capacity,
                          cudaStream_t stream) {
    if (const char* why = check(d)) return fail(W8A8_ERR_UNSUPPORTED, "decode stack: %s", why);
    const Scratch sc = layout(d, slices_for(d, num_sms()));
    const int n = 18 * d.n_layers + 2;
    if (capacity < n) return fail(W8A8_ERR_INVALID_ARG, "timeline needs room for %d stamps", n);
    cudaError_t e = cudaMemcpyAsync(out, workspace + sc.timeline, static_cast<size_t>(n) * 8, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "decode stack timeline: %s", cudaGetErrorString(e));
    return n;
}

int launch_decode_stack(const w8a8_decode_stack& d, unsigned char* workspace, size_t workspace_bytes, float* partials,
                        size_t partial_bytes, int* counters, size_t counter_count, int* status, cudaStream_t stream) {
    if (const char* why = check(d)) return fail(W8A8_ERR_UNSUPPORTED, "decode stack: %s", why);
    const int sms = num_sms();
    StackParams p = {};
    p.S = slices_for(d, sms);
    const Scratch sc = layout(d, p.S);
    if (sc.total > workspace_bytes)
        return fail(W8A8_ERR_WORKSPACE, "decode stack needs %zu bytes of scratch, context has %zu", sc.total, workspace_bytes);
    p.layers = d.layers;
    p.n_layers = d.n_layers; p.B = d.batch; p.dim = d.dim; p.n_q = d.n_q_heads; p.n_kv = d.n_kv_heads;
    p.inter = d.inter; p.g = d.group_size;
    int T = 1;
    while (T < d.dim && T < 1024) T <<= 1;
    p.norm_threads = T;
    p.block_bytes = kBlockW + 32 * (256 / d.group_size);
    p.eps = d.eps; p.sm_scale = d.sm_scale;
    p.final_norm = static_cast<const __half*>(d.final_norm);
    p.freqs = d.rope_freqs; p.positions = d.positions; p.seq_lens = d.seq_lens; p.block_table = d.block_table;
    p.max_blocks = d.max_blocks_per_seq;
    p.k_cache = static_cast<__half*>(d.k_cache); p.v_cache = static_cast<__half*>(d.v_cache);
    p.x = static_cast<__half*>(d.x); p.out = static_cast<__half*>(d.out);
    p.qkv = reinterpret_cast<__half*>(workspace + sc.qkv);
    p.xq = reinterpret_cast<int8_t*>(workspace + sc.xq);
    p.xs = reinterpret_cast<float*>(workspace + sc.xs);
    p.aq = reinterpret_cast<int8_t*>(workspace + sc.aq);
    p.as_ = reinterpret_cast<float*>(workspace + sc.as_);
    p.act = reinterpret_cast<__half*>(workspace + sc.act);
    p.actq = reinterpret_cast<int8_t*>(workspace + sc.actq);
    p.acts = reinterpret_cast<float*>(workspace + sc.acts);
    p.delta = reinterpret_cast<__half*>(workspace + sc.delta);
    p.attn_part = reinterpret_cast<float*>(workspace + sc.attn_part);
    p.barrier = reinterpret_cast<unsigned*>(workspace + sc.barrier);
    p.timeline = reinterpret_cast<unsigned long long*>(workspace + sc.timeline);
    p.status = status;
    (void)partials; (void)partial_bytes; (void)counters; (void)counter_count;  // the step adds cut tiles in shared memory
    const int Ns[4] = {(d.n_q_heads + 2 * d.n_kv_heads) * kHeadDim, d.dim, 2 * d.inter, d.dim};
    const int Ks[4] = {d.dim, d.n_q_heads * kHeadDim, d.dim, d.inter};
    const unsigned warps = static_cast<unsigned>(sms) * kWarps;
    for (int i = 0; i < 4; ++i) {
        GemvShape& sh = p.gs[i];
        sh.N = Ns[i]; sh.K = Ks[i]; sh.G = Ks[i] / d.group_size; sh.upt = Ks[i] / 256;
        sh.epilogue = i == 2 ? W8A8_EPI_SWIGLU : W8A8_EPI_NONE;
        if (Ks[i] % 256 != 0 || Ns[i] % 16 != 0) return fail(W8A8_ERR_UNSUPPORTED, "decode stack: linear %d is %d x %d", i, Ns[i], Ks[i]);
        const unsigned long long U = static_cast<unsigned long long>(Ns[i] / 16) * sh.upt;
        if ((U + 1) * warps >= (1ull << 32)) return fail(W8A8_ERR_UNSUPPORTED, "decode stack: linear %d too large", i);
        sh.U = static_cast<unsigned>(U);
        sh.NW = warps;
        if (Ns[i] / 16 / sms + 2 > kLocalTiles) return fail(W8A8_ERR_UNSUPPORTED, "decode stack: linear %d has too many row tiles per CTA", i);
    }

    cudaError_t e = cudaMemsetAsync(p.barrier, 0, 256, stream);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "decode stack: memset: %s", cudaGetErrorString(e));
    size_t region = sizeof(AttnSmem);
    for (int i = 0; i < 4; ++i) {
        const size_t need = static_cast<size_t>(8) * (Ks[i] + 64) + static_cast<size_t>(8) * (Ks[i] / d.group_size) * 4;
        region = need > region ? need : region;
    }
    const size_t smem = static_cast<size_t>(kWarps) * kRingBytes + region + 128;
    if (smem > 227 * 1024) return fail(W8A8_ERR_UNSUPPORTED, "decode stack: K = %d does not fit shared memory", d.inter);
    auto launch = [&](auto kern) -> int {
        cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess) return fail(W8A8_ERR_CUDA, "decode stack: shared memory attribute: %s", cudaGetErrorString(err));
        int per_sm = 0;
        err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem);
        if (err != cudaSuccess || per_sm < 1)
            return fail(W8A8_ERR_UNSUPPORTED, "decode stack: the kernel does not fit an SM (%s)", cudaGetErrorString(err));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(sms, 1, 1);
        cfg.blockDim = dim3(kThreads, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once: they wait on one another
        attr[0].val.cooperative = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        err = cudaLaunchKernelEx(&cfg, kern, p);
        if (err != cudaSuccess) return fail(W8A8_ERR_CUDA, "decode stack launch: %s", cudaGetErrorString(err));
        return W8A8_OK;
    };
    switch (d.group_size) {
        case 64: return launch(decode_stack_kernel<64>);
        case 128: return launch(decode_stack_kernel<128>);
        default: return launch(decode_stack_kernel<256>);
    }
}

}  // namespace w8a8
