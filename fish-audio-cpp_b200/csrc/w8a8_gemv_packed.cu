// Small-M (decode) W8A8 linear over PRE-PACKED weights: the HBM-roofline form.
//
// Same arithmetic as the other GEMV kernels (exact int32 sum per K-group from mma.sync.m16n8k32.s8
// with the weights as the A operand, acc = fma(float(P) * ws, xs, acc) over ascending groups, fp32
// partial tiles of a cut row tile added in ascending-K order). What changes is the weight layout.
//
// A row-major [N,K] matrix makes every 16-row tile 16 separate runs in DRAM, 256 bytes at a time per
// run; measured, that streams at about half of what a linear copy reaches. The loader therefore
// re-packs each weight once (w8a8_pack_weight) into the order in which this kernel consumes it:
//
//   block (rt, kb) = 16 rows x 256 bytes of K      rt = row tile, kb = 256-byte K block
//     [4 chunks of 64 K-bytes][2 halves][32 lanes][16 bytes]   a lane's MMA A-fragment pieces: half 0 =
//                                                   row gq, half 1 = row gq+8 (gq = lane / 4)
//     [16 rows][groups per block] fp16              the block's weight scales (32, 64 or 128 bytes)
//   blocks ordered rt-major, kb ascending, one after another with no gaps.
//
// Work split: whole 16-row tiles per CTA (tile t of T goes to CTA t * C / T), the CTA's units of 256 K-bytes
// in equal contiguous runs to its eight warps. A warp's run is then ONE contiguous byte range: the warp
// pulls it through a private ring of shared-memory stages with 1-D bulk copies (cp.async.bulk, one
// block per copy, completion on an mbarrier), reads its fragments back with conflict-free 128-bit
// shared loads, and finds the scales in the same stage — no strided access, no separate scale
// traffic, no tensor map. Rows past N are stored as zeros, so no tail handling is needed on loads.
// A row tile cut by a run boundary is always cut between warps of one CTA: its fp32 partial tiles meet in
// shared memory and the warp that arrives last adds them in ascending-K order. (An earlier form cut one
// global range over all warps of the grid and fixed cut tiles up through global scratch and L2 atomics:
// perfectly balanced, but two to three L2 round trips at the tail of every launch; measured 2 us slower
// per launch on the decode shapes than the at most one-tile imbalance of this form.)
//
// Launched with programmatic dependent launch: the first kStages blocks are requested before
// griddepcontrol.wait. Every mbarrier wait is bounded; on expiry the warp records an error word.
#include <cstdlib>

#include "sm100_ptx.cuh"
#include "w8a8_internal.h"
#include "w8a8_trace.cuh"

namespace w8a8 {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kBlockW = 16 * 256;        // weight bytes of a block
constexpr int kStagePitch = kBlockW + 128;  // room for the largest scale tail, keeps stages 128-byte aligned
constexpr int kLocalTiles = 128;  // row tiles per CTA whose arrival counters live in shared memory
// How the activations arrive (template parameter PRO):
enum { kProCodes = 0,   // int8 codes + fp32 scales made by an earlier launch (Xq, Xs)
       kProNorm = 1 };  // fp16 rows: every CTA does [x + residual] -> RMSNorm -> quantiser itself, in its prologue

struct GemvPackedParams {
    LinearArgs a;
    const unsigned char* packed;
    int block_bytes;  // kBlockW + 32 * groups per block
    int upt;          // units per 16-row tile
    int bpu;          // blocks per unit (1, or g / 256 when g > 256)
    unsigned U;       // units in all
    int* status;
#ifdef W8A8_TRACE
    int ablate;       // diagnostic build: bit mask of pieces of the kernel to leave out (timing experiments only)
#endif
};
#ifdef W8A8_TRACE
#define W8A8_ABLATED(bit) ((p.ablate & (bit)) != 0)
#else
#define W8A8_ABLATED(bit) false
#endif

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint4 ld_cg16(const __half* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ float ld_cg(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];\n" : "=f"(v) : "l"(p));
    return v;
}

#ifdef W8A8_TAIL_TIMELINE
// Diagnostic build only: the last CTA to arrive leaves nanosecond stamps of its launch in tail_counters[128..].
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define W8A8_STAMP(slot) do { if (threadIdx.x == 0) tl[slot] = now_ns(); } while (0)
#define W8A8_STAMP_FLUSH(counters, is_last) do { if (threadIdx.x == 0 && (is_last)) { \
    unsigned long long* o = reinterpret_cast<unsigned long long*>((counters) + 128); \
    for (int i_ = 0; i_ < 8; ++i_) o[i_] = tl[i_]; o[8] = blockIdx.x; } } while (0)
#else
#define W8A8_STAMP(slot) do {} while (0)
#define W8A8_STAMP_FLUSH(counters, is_last) do {} while (0)
#endif

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Tail, kind kTailRowNorm. Called by all 256 threads of a CTA after its last tile is stored. The CTA takes a ticket;
// the last min(M, grid) CTAs to arrive each wait (bounded) until every CTA of the grid has arrived, i.e. until the
// whole output Y = [M, N] is in L2, and then run, for the token rows they own, exactly what the kernel launched next
// would have run (rowquant_compact_kernel): x = half(x + Y) (ffn_activations.cu:41-45), RMSNorm with the
// reference's 1024-thread summation order (rms_norm.cu:23-49), the group quantiser (int8_gemm.cu:147-211).
// N % 256 == 0, 512 < N <= 4096. The last row CTA to finish puts the counters back to zero.
__device__ __forceinline__ void tail_row_norm(const LinearArgs& a, unsigned char* scratch, int* status,
                                              unsigned long long (&tl)[8]) {
    __shared__ int s_ticket, s_fail;
    __shared__ float s_red[32];
    __half* row_s = reinterpret_cast<__half*>(scratch);  // [N]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int total = gridDim.x, n_row = a.M < total ? a.M : total, first = total - n_row;
    if (tid == 0) {
        __threadfence();  // this CTA's tiles (stored by all its warps, ordered by the barrier before the call)
        s_ticket = atomicAdd(&a.tail_counters[0], 1);
        s_fail = 0;
    }
    __syncthreads();
    const int ticket = s_ticket;
    W8A8_STAMP(3);
    if (ticket < first) return;
    if (tid == 0) {
        unsigned spins = 0;
        while (ld_acquire_gpu(&a.tail_counters[0]) < total) {
            if (++spins > (1u << 22)) { atomicExch(status, 610); s_fail = 1; break; }
            if (spins > 32) __nanosleep(32);
        }
    }
    __syncthreads();
    W8A8_STAMP(4);
    const int K = a.N, T = 1024, VW = T / kThreads, pieces = K / 8;
    const int G = K / a.tail_g;
    if (!s_fail) {
        for (int row = ticket - first; row < a.M; row += n_row) {
            const size_t base = static_cast<size_t>(row) * K;
            uint4 xv[2], dv[2], wv[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {  // every load first (at most two pieces per thread)
                const int c8 = tid + i * kThreads;
                const int cc = c8 < pieces ? c8 : 0;
                wv[i] = __ldg(reinterpret_cast<const uint4*>(a.tail_norm_weight) + cc);
                xv[i] = __ldcg(reinterpret_cast<const uint4*>(a.tail_x + base) + cc);
                dv[i] = __ldcg(reinterpret_cast<const uint4*>(a.Y + base) + cc);  // written by other SMs: past L1
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int c8 = tid + i * kThreads;
                if (c8 < pieces) {
                    __half* hx = reinterpret_cast<__half*>(&xv[i]);
                    const __half* hd = reinterpret_cast<const __half*>(&dv[i]);
#pragma unroll
                    for (int e = 0; e < 8; ++e) hx[e] = __float2half(__half2float(hx[e]) + __half2float(hd[e]));
                    *reinterpret_cast<uint4*>(a.tail_x + base + c8 * 8) = xv[i];
                    reinterpret_cast<uint4*>(row_s)[c8] = xv[i];
                }
            }
            __syncthreads();
            W8A8_STAMP(5);
#pragma unroll 1
            for (int k = 0; k < VW; ++k) {  // real warp w plays the reference's warps w*VW .. w*VW + VW - 1
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
                total_sum = s_red[lane];
                for (int offset = 16; offset > 0; offset /= 2) total_sum += __shfl_down_sync(0xffffffffu, total_sum, offset);
            }
            __syncthreads();
            if (tid == 0) s_red[0] = rsqrtf(total_sum / K + a.tail_eps);
            __syncthreads();
            const float rms = s_red[0];
            const int lanes = a.tail_g / 8;  // threads per quantisation group: 8, 16 or 32
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
                if (live && a.tail_normed_out) *reinterpret_cast<uint4*>(a.tail_normed_out + base + c8 * 8) = xv[i];
                if (!a.tail_Xq) continue;
                for (int o = lanes / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                if (!live) continue;
                float scale = amax / 127.0f;
                if (scale < 1e-8f) scale = 1e-8f;
                if ((lane & (lanes - 1)) == 0) a.tail_Xs[static_cast<size_t>(row) * G + (c8 * 8) / a.tail_g] = scale;
                const float inv_scale = 1.0f / scale;
                uint32_t lo = 0, hi = 0;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    int q = __float2int_rn(v[e] * inv_scale);
                    q = max(-127, min(127, q));
                    if (e < 4) lo |= (static_cast<uint32_t>(q) & 0xffu) << (8 * e);
                    else hi |= (static_cast<uint32_t>(q) & 0xffu) << (8 * (e - 4));
                }
                *reinterpret_cast<uint2*>(a.tail_Xq + base + c8 * 8) = make_uint2(lo, hi);
            }
            __syncthreads();  // row_s and s_red are reused by the next row of this CTA
        }
    }
    W8A8_STAMP(6);
    W8A8_STAMP_FLUSH(a.tail_counters, ticket == total - 1);
    if (tid == 0) {
        const int done = atomicAdd(&a.tail_counters[1], 1);
        if (done == n_row - 1) {  // every row CTA is past its wait: the counters can go back to zero
            a.tail_counters[1] = 0;
            __threadfence();
            a.tail_counters[0] = 0;
        }
    }
}

// Tail, kind kTailGroupQuant: the quantiser (int8_gemm.cu:147-211) of the launch's own output for the linear that
// follows. out = Y as stored: [M, N] (16 channels per row tile) or, with the SwiGLU epilogue, [M, N/2] (8 channels
// per tile). A CTA adds the number of its tiles in each quantisation group to that group's counter; the CTA whose
// add completes a group quantises it (one warp per token row, 8 channels per lane and step) and zeroes the counter.
// Nothing waits. tail_g % 8 == 0 and a multiple of the channels per tile.
__device__ __forceinline__ void tail_group_quant(const LinearArgs& a, int ct0, int ct1, unsigned char* scratch,
                                                 unsigned long long (&tl)[8]) {
    int* s_mine = reinterpret_cast<int*>(scratch);  // [groups this CTA touches]: 1 = this CTA completes the group
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cpt = a.epilogue == W8A8_EPI_SWIGLU ? 8 : 16;      // output channels per row tile
    const int Kout = a.epilogue == W8A8_EPI_SWIGLU ? a.N / 2 : a.N;
    const int tpg = a.tail_g / cpt;                               // tiles per group
    const int tiles = (a.N + 15) / 16, G = (Kout + a.tail_g - 1) / a.tail_g;
    if (ct1 <= ct0) return;
    const int j0 = ct0 / tpg, j1 = (ct1 - 1) / tpg;
    if (tid <= j1 - j0) {
        const int j = j0 + tid;
        const int lo = max(ct0, j * tpg), hi = min(ct1, (j + 1) * tpg);
        const int in_group = min(tiles, (j + 1) * tpg) - j * tpg;
        __threadfence();  // this CTA's tiles (ordered before by the barrier before the call)
        const int old = atomicAdd(&a.tail_counters[j], hi - lo);
        const int mine = (old + (hi - lo) == in_group) ? 1 : 0;
        if (mine) {
            a.tail_counters[j] = 0;
            __threadfence();  // acquire side: the other CTAs' tiles are visible to the loads below
        }
        s_mine[tid] = mine;
    }
    __syncthreads();
    W8A8_STAMP(3);
    bool any_mine = false;
    for (int j = j0; j <= j1; ++j) any_mine |= s_mine[j - j0] != 0;
    for (int j = j0; j <= j1; ++j) {
        if (!s_mine[j - j0]) continue;
        const int c0 = j * a.tail_g, width = min(a.tail_g, Kout - c0);
        for (int row = warp; row < a.M; row += kWarps) {
            const __half* src = a.Y + static_cast<size_t>(row) * Kout + c0;
            float amax = 0.0f;
            for (int e = lane * 8; e < width; e += 256) {
                const uint4 u = __ldcg(reinterpret_cast<const uint4*>(src + e));
                const __half* h = reinterpret_cast<const __half*>(&u);
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(__half2float(h[i])));
            }
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            float scale = amax / 127.0f;
            if (scale < 1e-8f) scale = 1e-8f;
            if (lane == 0) a.tail_Xs[static_cast<size_t>(row) * G + j] = scale;
            const float inv_scale = 1.0f / scale;
            for (int e = lane * 8; e < width; e += 256) {
                const uint4 u = __ldcg(reinterpret_cast<const uint4*>(src + e));
                const __half* h = reinterpret_cast<const __half*>(&u);
                uint32_t lo = 0, hi = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    int q = __float2int_rn(__half2float(h[i]) * inv_scale);
                    q = max(-127, min(127, q));
                    if (i < 4) lo |= (static_cast<uint32_t>(q) & 0xffu) << (8 * i);
                    else hi |= (static_cast<uint32_t>(q) & 0xffu) << (8 * (i - 4));
                }
                *reinterpret_cast<uint2*>(a.tail_Xq + static_cast<size_t>(row) * Kout + c0 + e) = make_uint2(lo, hi);
            }
        }
    }
    __syncthreads();
    W8A8_STAMP(6);
    W8A8_STAMP_FLUSH(a.tail_counters, any_mine && j1 == G - 1);
    (void)any_mine;
}

// GM: 64 or 128 = the group size itself; 256 = any group size that is a multiple of 256 (a unit is then
// one whole group = g/256 blocks).
//
// PRO == kProNorm: the activations arrive as fp16 rows and every CTA forms codes and scales itself before it
// consumes its first block (whose copy is already in flight): [x + residual] -> RMSNorm with the summation
// order of the reference's 1024-thread launch (rms_norm.cu:23-49) -> group quantiser (int8_gemm.cu:147-211).
// One warp per token row (M <= 8), the row in registers from the load to the codes; only the codes and scales
// go to shared memory. This replaces a separate launch of a kernel that runs on M CTAs and leaves the rest of
// the GPU idle, and the trip of its results through L2.
// ST: stages of a warp's ring (3; 2 for kProNorm so that two CTAs fit an SM beside the code rows).
// KI: kProNorm only, the 16-byte pieces of a row a lane holds (K <= 256 * KI): 10 for the stack's K = 2560, else 16.
template <int MT, int GM, int PRO, int ST, int KI>
__global__ void __launch_bounds__(kThreads, (PRO == kProNorm || MT == 1) ? 2 : 1)
gemv_packed_kernel(const GemvPackedParams p) {
    constexpr bool FUSED = PRO == kProNorm;
    constexpr int kStages = ST;
    constexpr int kRingBytes = kStages * kStagePitch;
    static_assert(PRO == kProCodes || MT == 1, "the fused prologue handles one row per warp");
    extern __shared__ unsigned char smem_raw[];
    W8A8_TRACE_SCOPE();
    unsigned long long tl[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    (void)tl;
    W8A8_STAMP(0);
    __shared__ __align__(8) uint64_t bars[kWarps][kStages];
    const LinearArgs& a = p.a;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gq = lane >> 2, c = lane & 3;
    constexpr int GPU = GM == 64 ? 4 : GM == 128 ? 2 : 1;  // groups per unit

    // ---- this warp's contiguous range of units; the eight ranges of a CTA are neighbours, so that most row
    // tiles cut by a range boundary are cut between warps of ONE CTA and can be added up in shared memory ----
    __shared__ float red_s[kWarps][2][MT * 4 * 32];
    __shared__ int cnt_s[kLocalTiles];
    for (int i = threadIdx.x; i < kLocalTiles; i += kThreads) cnt_s[i] = 0;
    __syncthreads();
    // Whole 16-row tiles per CTA (tile t of `tiles` goes to CTA t * C / tiles), the CTA's units in equal contiguous
    // runs to its warps (none with an empty run): a tile cut by a run boundary is always cut between warps of
    // this CTA.
    const unsigned tiles = p.U / p.upt;
    const unsigned ct0 = blockIdx.x * tiles / gridDim.x, ct1 = (blockIdx.x + 1) * tiles / gridDim.x;
    const unsigned cu0 = ct0 * p.upt, n_cta = (ct1 - ct0) * p.upt;
    const unsigned nw_cta = n_cta < kWarps ? n_cta : kWarps;
    unsigned u0 = cu0, u1 = cu0;
    if (static_cast<unsigned>(warp) < nw_cta) {
        u0 = cu0 + warp * n_cta / nw_cta;
        u1 = cu0 + (warp + 1) * n_cta / nw_cta;
    }
    const int T = static_cast<int>(u1 - u0) * p.bpu;  // blocks

    const uint32_t ring = ((ptx::smem_u32(smem_raw) + 127u) & ~127u) + warp * kRingBytes;
    uint64_t* bar = bars[warp];
    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) ptx::mbar_init(&bar[s], 1);
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
    }
    __syncwarp();

    // producer (lane 0): the range is one contiguous run of blocks in the packed image
    int pt = 0;
    const unsigned char* src = p.packed + static_cast<size_t>(u0) * p.bpu * p.block_bytes;
    auto issue = [&]() {  // lane 0 only
        const int slot = pt % kStages;
        ptx::mbar_arrive_expect_tx(&bar[slot], p.block_bytes);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(ring + slot * kStagePitch), "l"(src), "r"(p.block_bytes), "r"(ptx::smem_u32(&bar[slot]))
                     : "memory");
        src += p.block_bytes;
        ++pt;
    };
    if (lane == 0) {
        const int pre = T < kStages ? T : kStages;
        for (int i = 0; i < pre; ++i) issue();
    }
    // kProNorm shared memory behind the rings: norm weight [K] fp16 | code rows [8][K + 64] | scales [8][G] fp32
    unsigned char* const fbase = smem_raw + (ring - warp * kRingBytes - ptx::smem_u32(smem_raw)) + kWarps * kRingBytes;
    if constexpr (FUSED) {  // the norm weight is a parameter too: stage it before the wait
        __half* normw_s = reinterpret_cast<__half*>(fbase);
        for (int c8 = threadIdx.x; c8 < a.K / 8; c8 += kThreads)
            reinterpret_cast<uint4*>(normw_s)[c8] = __ldg(reinterpret_cast<const uint4*>(a.norm_weight) + c8);
        __syncthreads();  // staged by all threads, read by each warp on its own after the wait
    }
    // Everything above touches only weights. Let the next launch begin its own prologue, then wait
    // for the kernel before this one: it produces the activations.
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    W8A8_TRACE_WAITED();
    W8A8_STAMP(1);
    // tensor-parallel send: this exchange's epoch = the last finished one + 1 (advanced by the receive kernel)
    int tp_ep = 0;
    if (a.tp.world > 0)
        tp_ep = *reinterpret_cast<const volatile int*>(a.tp.peers[a.tp.rank] + a.tp.ctl_off) + 1;

    const int8_t* xq[MT];
    const float* xsp[MT][2];
    uint32_t xq_s = 0;                    // kProNorm: this lane's code row in shared memory
    const float* xsp_s[2] = {nullptr, nullptr};
    if constexpr (FUSED) {
        const int K = a.K, pitch = K + 64;  // the pitch puts rows gq and gq+1 in different bank halves
        const __half* normw_s = reinterpret_cast<const __half*>(fbase);
        int8_t* codes_s = reinterpret_cast<int8_t*>(fbase + static_cast<size_t>(K) * 2);   // [8][pitch]
        float* scales_s = reinterpret_cast<float*>(codes_s + 8 * pitch);                    // [8][G]
        const int row = warp;
        const bool writer = blockIdx.x == 0;
        // Lane l owns the 16-byte pieces c8 = l + 32 i of its row, i.e. elements e = 8 l + j + 256 i (j < 8): these
        // are ALL the elements of the reference's virtual threads vt = 8 l + j + 256 r (r = i mod 4 < 4), which sum
        // e = vt, vt + 1024, vt + 2048, ... in that order (rms_norm.cu:23-27 with a 1024-thread block).
        constexpr int kMaxI = KI;  // K <= 256 * KI
        const int iters = K / 256;
        uint4 v[kMaxI];
        if (row < a.M) {
            // All loads are requested before anything is used or stored: a load placed after a store that might
            // alias it would wait for it.
            uint4 r[kMaxI];
#pragma unroll
            for (int i = 0; i < kMaxI; ++i) {
                v[i] = make_uint4(0u, 0u, 0u, 0u);
                r[i] = make_uint4(0u, 0u, 0u, 0u);
                if (i < iters) {
                    const size_t off = static_cast<size_t>(row) * K + (lane + 32 * i) * 8;
                    v[i] = ld_cg16(a.X + off);
                    if (a.norm_residual) r[i] = ld_cg16(a.norm_residual + off);
                }
            }
            if (a.norm_residual) {
#pragma unroll
                for (int i = 0; i < kMaxI; ++i) {
                    if (i < iters) {
                        __half* hv = reinterpret_cast<__half*>(&v[i]);
                        const __half* hr = reinterpret_cast<const __half*>(&r[i]);
#pragma unroll
                        for (int e = 0; e < 8; ++e) hv[e] = __float2half(__half2float(hv[e]) + __half2float(hr[e]));
                        if (writer && a.norm_x_out)
                            *reinterpret_cast<uint4*>(a.norm_x_out + static_cast<size_t>(row) * K + (lane + 32 * i) * 8) = v[i];
                    }
                }
            }
            W8A8_STAMP(2);
            // per virtual thread (r, j): local_sum over i = r, r + 4, r + 8, r + 12 ascending
            float ls[4][8];
#pragma unroll
            for (int r4 = 0; r4 < 4; ++r4)
#pragma unroll
                for (int j = 0; j < 8; ++j) ls[r4][j] = 0.0f;
#pragma unroll
            for (int i = 0; i < kMaxI; ++i) {
                if (i < iters) {
                    const __half* hv = reinterpret_cast<const __half*>(&v[i]);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float val = __half2float(hv[j]);
                        ls[i & 3][j] += val * val;
                    }
                }
            }
            // The reference's shuffle-down tree over a virtual warp. Virtual warp (r, l / 4) is made of the
            // virtual lanes vl = 8 (l % 4) + j: offsets 16 and 8 cross real lanes (l + 2, l + 1), offsets 4, 2, 1
            // stay inside the lane's eight j. Only virtual lane 0 (l % 4 == 0, j == 0) is used afterwards, and its
            // sum takes exactly the reference's operands in the reference's order.
            float wsum[4];
#pragma unroll
            for (int r4 = 0; r4 < 4; ++r4) {
                float b8[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float local_sum = ls[r4][j];
                    local_sum += __shfl_down_sync(0xffffffffu, local_sum, 2);   // virtual offset 16
                    local_sum += __shfl_down_sync(0xffffffffu, local_sum, 1);   // virtual offset 8
                    b8[j] = local_sum;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) b8[j] += b8[j + 4];                  // virtual offset 4
                b8[0] += b8[2];                                                  // virtual offset 2
                b8[1] += b8[3];
                wsum[r4] = b8[0] + b8[1];                                        // virtual offset 1
            }
            // second tree (rms_norm.cu:36-42): lane vw takes s_red[vw]; virtual warp vw = 8 r + q lives in lane 4 q
            float total_sum = 0.0f;
#pragma unroll
            for (int r4 = 0; r4 < 4; ++r4) {
                const float t = __shfl_sync(0xffffffffu, wsum[r4], 4 * (lane & 7));
                if ((lane >> 3) == r4) total_sum = t;
            }
            for (int offset = 16; offset > 0; offset /= 2)
                total_sum += __shfl_down_sync(0xffffffffu, total_sum, offset);
            total_sum = __shfl_sync(0xffffffffu, total_sum, 0);
            const float rms = rsqrtf(total_sum / K + a.norm_eps);
            W8A8_STAMP(3);
            // normalise in registers (rounded to fp16 like rms_norm's output) and find the group maxima; a run
            // of 256 channels is one i across the warp
            constexpr int kLanesPerGroup = GM == 64 ? 8 : GM == 128 ? 16 : 32;
            const int per_group = GM == 256 ? a.g / 256 : 1;
            float gmax[kMaxI];
#pragma unroll
            for (int i = 0; i < kMaxI; ++i) {
                gmax[i] = 0.0f;
                if (i < iters) {
                    const uint4 w = reinterpret_cast<const uint4*>(normw_s)[lane + 32 * i];
                    __half* hv = reinterpret_cast<__half*>(&v[i]);
                    const __half* hw = reinterpret_cast<const __half*>(&w);
                    float m = 0.0f;
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        float val = __half2float(hv[e]) * rms;
                        hv[e] = __float2half(val * __half2float(hw[e]));
                        m = fmaxf(m, fabsf(__half2float(hv[e])));
                    }
#pragma unroll
                    for (int o = 1; o < kLanesPerGroup; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                    gmax[i] = m;
                }
            }
            W8A8_STAMP(4);
            if (GM == 256 && per_group > 1) {  // a group spans per_group consecutive runs: give each run its group's maximum
#pragma unroll
                for (int i = 1; i < kMaxI; ++i)   // forward: the last run of a group collects the maximum
                    if (i < iters && i % per_group != 0) gmax[i] = fmaxf(gmax[i], gmax[i - 1]);
#pragma unroll
                for (int i = kMaxI - 2; i >= 0; --i)  // backward: hand it to the runs before it
                    if (i + 1 < iters && (i + 1) % per_group != 0) gmax[i] = gmax[i + 1];
            }
#pragma unroll
            for (int i = 0; i < kMaxI; ++i) {
                if (i < iters) {
                    float scale = gmax[i] / 127.0f;
                    if (scale < 1e-8f) scale = 1e-8f;
                    const int j = GM == 256 ? i / per_group : i * (256 / GM) + lane / kLanesPerGroup;
                    if (lane % kLanesPerGroup == 0 && (GM != 256 || i % per_group == 0)) {
                        scales_s[row * a.G + j] = scale;
                        if (writer && a.scales_out) a.scales_out[static_cast<size_t>(row) * a.G + j] = scale;
                    }
                    const float inv_scale = 1.0f / scale;
                    const __half* hv = reinterpret_cast<const __half*>(&v[i]);
                    __align__(8) int8_t q8[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        int q = __float2int_rn(__half2float(hv[e]) * inv_scale);
                        q8[e] = static_cast<int8_t>(max(-127, min(127, q)));
                    }
                    const int c8 = lane + 32 * i;
                    *reinterpret_cast<uint2*>(codes_s + row * pitch + c8 * 8) = *reinterpret_cast<const uint2*>(q8);
                    if (writer && a.codes_out)
                        *reinterpret_cast<uint2*>(a.codes_out + static_cast<size_t>(row) * K + c8 * 8) =
                            *reinterpret_cast<const uint2*>(q8);
                }
            }
        }
        __syncthreads();  // all rows' codes and scales are in place
        W8A8_STAMP(5);
        xq_s = ptx::smem_u32(codes_s) + min(gq, a.M - 1) * pitch + c * 16;
        xsp_s[0] = scales_s + min(2 * c, a.M - 1) * a.G;
        xsp_s[1] = scales_s + min(2 * c + 1, a.M - 1) * a.G;
    } else {
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) {
            xq[nt] = a.Xq + static_cast<size_t>(min(nt * 8 + gq, a.M - 1)) * a.K + c * 16;
            xsp[nt][0] = a.Xs + static_cast<size_t>(min(nt * 8 + 2 * c, a.M - 1)) * a.G;
            xsp[nt][1] = a.Xs + static_cast<size_t>(min(nt * 8 + 2 * c + 1, a.M - 1)) * a.G;
        }
    }

    // Two integer accumulators per tile: consecutive MMAs alternate between them, so that one MMA does
    // not wait for the previous one's result (with one warp per scheduler that latency is exposed).
    int P[MT][4], Q[MT][4];
    float acc[MT][4];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int r = 0; r < 4; ++r) { P[nt][r] = 0; Q[nt][r] = 0; acc[nt][r] = 0.0f; }

    // Stores a finished 16-row tile held in fragment layout: rows gq / gq+8, tokens 2c / 2c+1.
    auto store_tile = [&](int rt, const float (&v)[MT][4]) {
        const int rA = rt * 16 + gq;
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = nt * 8 + 2 * c + e;
                if (tok >= a.M) continue;
                if (a.epilogue == W8A8_EPI_SWIGLU) {
                    if (rA + 8 < a.N) {
                        const float g16 = __half2float(__float2half(v[nt][e]));
                        const __half s16 = __float2half(g16 / (1.0f + expf(-g16)));
                        const float u16 = __half2float(__float2half(v[nt][2 + e]));
                        a.Y[static_cast<size_t>(tok) * (a.N / 2) + rt * 8 + gq] = __float2half(__half2float(s16) * u16);
                    }
                } else {
#pragma unroll
                    for (int hrow = 0; hrow < 2; ++hrow) {
                        const int row = rA + 8 * hrow;
                        if (row >= a.N) continue;
                        const size_t o = static_cast<size_t>(tok) * a.N + row;
                        if (a.tp.world > 0) {
                            // the fp32 partial as a self-validating word {value, epoch} into slot [rank] of every rank
                            const size_t word = (static_cast<size_t>((tp_ep & 1) * a.tp.world + a.tp.rank) * a.tp.max_tokens + tok) *
                                                    a.N + row;
                            const uint2 w = make_uint2(__float_as_uint(v[nt][2 * hrow + e]), static_cast<unsigned>(tp_ep));
                            for (int r = 0; r < a.tp.world; ++r) reinterpret_cast<uint2*>(a.tp.peers[r])[word] = w;
                        }
                        if (!a.Y || W8A8_ABLATED(4)) continue;
                        __half y = __float2half(v[nt][2 * hrow + e]);
                        if (a.epilogue == W8A8_EPI_RESIDUAL)
                            y = __float2half(__half2float(y) + __half2float(a.residual[o]));
                        a.Y[o] = y;
                    }
                }
            }
        }
    };

    auto warp_of_unit = [&](unsigned u) -> unsigned {  // the warp of this CTA whose run holds unit u
        return ((u - cu0 + 1) * nw_cta - 1) / n_cta;
    };
    const int cta_rt0 = static_cast<int>(ct0);

    // Called when the warp has added its last unit of row tile rt into acc. A cut tile: the fp32 partial goes to
    // the warp's slot in shared memory, the arrival is counted, and whichever warp arrives last adds the
    // partials in ascending-K order and stores. Nothing waits; nothing leaves the SM.
    auto finish_tile = [&](int rt) {
        const unsigned t_lo = static_cast<unsigned>(rt) * p.upt, t_hi = t_lo + p.upt;  // [t_lo, t_hi)
        if ((u0 <= t_lo && t_hi <= u1) || W8A8_ABLATED(8)) {
            store_tile(rt, acc);
        } else {
            const unsigned first = warp_of_unit(t_lo), last = warp_of_unit(t_hi - 1);
            const int my_slot = (static_cast<int>(u0 / p.upt) == rt) ? 0 : 1;
            float* mine = red_s[warp][my_slot];
#pragma unroll
            for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                for (int r = 0; r < 4; ++r) mine[(nt * 4 + r) * 32 + lane] = acc[nt][r];
            __syncwarp();
            int old = 0;
            if (lane == 0) {
                __threadfence_block();
                old = atomicAdd(&cnt_s[rt - cta_rt0], 1);
            }
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old == static_cast<int>(last - first)) {
                __threadfence_block();
                float sum[MT][4];
#pragma unroll
                for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                    for (int r = 0; r < 4; ++r) sum[nt][r] = 0.0f;
                for (unsigned ww = first; ww <= last; ++ww) {
                    const unsigned wu0 = cu0 + ww * n_cta / nw_cta;
                    const float* src = red_s[ww][(static_cast<int>(wu0 / p.upt) == rt) ? 0 : 1];
#pragma unroll
                    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                        for (int r = 0; r < 4; ++r) sum[nt][r] += src[(nt * 4 + r) * 32 + lane];
                }
                store_tile(rt, sum);
            }
        }
#pragma unroll
        for (int nt = 0; nt < MT; ++nt)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[nt][r] = 0.0f;
    };

    auto promote = [&](int rt, int j, __half hsa, __half hsb, const float (&xsv)[MT][2]) {
        const float fa = __half2float(hsa), fb = __half2float(hsb);
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) {
            const float x0 = xsv[nt][0], x1 = xsv[nt][1];
#pragma unroll
            for (int r = 0; r < 4; ++r) { P[nt][r] += Q[nt][r]; Q[nt][r] = 0; }
            if (a.dump) {
                const int t0 = nt * 8 + 2 * c, rA = rt * 16 + gq;
                const size_t NG = static_cast<size_t>(a.N) * a.G;
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int row = rA + 8 * (r >> 1), tok = t0 + (r & 1);
                    if (row < a.N && tok < a.M) a.dump[tok * NG + static_cast<size_t>(row) * a.G + j] = P[nt][r];
                }
            }
            acc[nt][0] = __fmaf_rn(__fmul_rn(static_cast<float>(P[nt][0]), fa), x0, acc[nt][0]);
            acc[nt][1] = __fmaf_rn(__fmul_rn(static_cast<float>(P[nt][1]), fa), x1, acc[nt][1]);
            acc[nt][2] = __fmaf_rn(__fmul_rn(static_cast<float>(P[nt][2]), fb), x0, acc[nt][2]);
            acc[nt][3] = __fmaf_rn(__fmul_rn(static_cast<float>(P[nt][3]), fb), x1, acc[nt][3]);
            P[nt][0] = P[nt][1] = P[nt][2] = P[nt][3] = 0;
        }
    };

    // ---- consumer loop: one packed block (16 rows x 256 bytes of K, plus its scales) per step ----
    // Activation codes and scales are a few KB shared by the whole grid, but each warp touches a
    // given piece only once, so these reads mostly miss L1 and cost an L2 round trip. They are
    // requested one block ahead (registers xn / xsn) and never sit on the critical path.
    int si = 0;
    int ub = static_cast<int>(u0 % p.upt), rt = static_cast<int>(u0 / p.upt);
    bool ok = true;
    uint4 xc[4][MT], xn[4][MT];
    float xsc[GPU][MT][2], xsn[GPU][MT][2];
    auto load_x = [&](int kbase, uint4 (&dst)[4][MT]) {
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
#pragma unroll
            for (int nt = 0; nt < MT; ++nt) {
                if constexpr (FUSED) dst[ch][nt] = lds128(xq_s + kbase + ch * 64);
                else if (W8A8_ABLATED(1)) dst[ch][nt] = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
                else dst[ch][nt] = __ldg(reinterpret_cast<const uint4*>(xq[nt] + kbase + ch * 64));
            }
    };
    auto load_xs = [&](int unit_b, float (&dst)[GPU][MT][2]) {
#pragma unroll
        for (int q = 0; q < GPU; ++q)
#pragma unroll
            for (int nt = 0; nt < MT; ++nt) {
                if constexpr (FUSED) {
                    dst[q][nt][0] = xsp_s[0][unit_b * GPU + q];
                    dst[q][nt][1] = xsp_s[1][unit_b * GPU + q];
                } else if (W8A8_ABLATED(2)) {
                    dst[q][nt][0] = 1.0f;
                    dst[q][nt][1] = 1.0f;
                } else {
                    dst[q][nt][0] = __ldg(xsp[nt][0] + unit_b * GPU + q);
                    dst[q][nt][1] = __ldg(xsp[nt][1] + unit_b * GPU + q);
                }
            }
    };
    if (T > 0) {
        load_x(ub * p.bpu * 256, xc);
        load_xs(ub, xsc);
    }
    for (int t = 0; t < T; ++t) {
        const int slot = t % kStages;
        // position of the next block (the same row tile or the next one: K restarts at 0)
        int nsi = si + 1, nub = ub;
        if (nsi == p.bpu) { nsi = 0; if (++nub == p.upt) nub = 0; }
        if (t + 1 < T) {
            load_x((nub * p.bpu + nsi) * 256, xn);
            if (nsi == 0) load_xs(nub, xsn);
        }
        if (!ptx::mbar_wait_bounded(&bar[slot], (t / kStages) & 1)) {
            if (lane == 0) atomicExch(p.status, 600 + slot);
            ok = false;
            break;
        }
        const uint32_t st = ring + slot * kStagePitch;
        // this block's weight scales ride behind its weights: [16 rows][GPU] fp16
        __half sa[GPU], sb[GPU];
#pragma unroll
        for (int q = 0; q < GPU; ++q) {
            sa[q] = __ushort_as_half(static_cast<unsigned short>(lds16(st + kBlockW + (gq * GPU + q) * 2)));
            sb[q] = __ushort_as_half(static_cast<unsigned short>(lds16(st + kBlockW + ((gq + 8) * GPU + q) * 2)));
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {  // 64-byte K chunks
            const uint32_t fa = st + ch * 1024 + lane * 16;
            const uint4 wa = lds128(fa), wb = lds128(fa + 512);
#pragma unroll
            for (int nt = 0; nt < MT; ++nt) {
                mma_s8(P[nt], wa.x, wb.x, wa.y, wb.y, xc[ch][nt].x, xc[ch][nt].y);
                mma_s8(Q[nt], wa.z, wb.z, wa.w, wb.w, xc[ch][nt].z, xc[ch][nt].w);
            }
            if (GM == 64) promote(rt, ub * 4 + ch, sa[ch % GPU], sb[ch % GPU], xsc[ch % GPU]);
            if (GM == 128 && (ch & 1))
                promote(rt, ub * 2 + (ch >> 1), sa[(ch >> 1) % GPU], sb[(ch >> 1) % GPU], xsc[(ch >> 1) % GPU]);
        }
        // The block's bytes are in registers: the slot may be refilled.
        __syncwarp();
        // (No proxy fence: the shared-memory reads above have returned their data — the MMAs consumed it —
        // before the copy that overwrites the slot is even issued.)
        if (lane == 0 && pt < T) issue();
#ifdef W8A8_TAIL_TIMELINE
        if (t == 0) W8A8_STAMP(6);
#endif
        if (++si == p.bpu) {
            si = 0;
            if (GM == 256) promote(rt, ub, sa[0], sb[0], xsc[0]);
            // one call site for the tile end: the row tile is complete, or the range ends inside it
            ++ub;
            if (ub == p.upt || t + 1 == T) {
                finish_tile(rt);
                if (ub == p.upt) { ub = 0; ++rt; }
            }
#pragma unroll
            for (int q = 0; q < GPU; ++q)
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) { xsc[q][nt][0] = xsn[q][nt][0]; xsc[q][nt][1] = xsn[q][nt][1]; }
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
#pragma unroll
            for (int nt = 0; nt < MT; ++nt) xc[ch][nt] = xn[ch][nt];
    }
    if (!ok) {
        // Leave only once every requested block has landed (or a second bounded wait ran out): a TMA write
        // must not arrive in shared memory that already belongs to another CTA.
        pt = __shfl_sync(0xffffffffu, pt, 0);
        for (int s = 0; s < kStages; ++s)
            if (pt > s) ptx::mbar_wait_bounded(&bar[s], ((pt - 1 - s) / kStages) & 1, 1u << 16);
    }
#ifdef W8A8_TAIL_TIMELINE
    if (a.tail_kind == kTailNone && a.tail_counters) {
        W8A8_STAMP(7);
        W8A8_STAMP_FLUSH(a.tail_counters, blockIdx.x == gridDim.x - 1);
    }
#endif
    if constexpr (PRO == kProCodes && MT == 1) {
        if (a.tail_kind != kTailNone) {
            // every copy this CTA asked for has been consumed: the rings are free to serve as the tail's scratch
            W8A8_STAMP(7);  // this thread's own warp is done
            __syncthreads();
            W8A8_STAMP(2);
            unsigned char* scratch = smem_raw + (ring - warp * kRingBytes - ptx::smem_u32(smem_raw));
            if (a.tail_kind == kTailRowNorm) tail_row_norm(a, scratch, p.status, tl);
            else tail_group_quant(a, static_cast<int>(ct0), static_cast<int>(ct1), scratch, tl);
        }
    }
#ifdef W8A8_TRACE
    __syncthreads();  // diagnostic build: the record's end is the CTA's end, not warp 0's
    W8A8_TRACE_END(10u + PRO + 4u * a.tail_kind, static_cast<unsigned>(a.N));
#endif
}

struct Plan {
    int MT, GM, upt, bpu, block_bytes, tiles, ctas, pro, stages;
    long long U;
};

int num_sms() {  // of the current device (not cached: one process may drive several devices)
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
        v = 148;
    return v;
}

}  // namespace

// How many CTAs share the row tiles of a linear. Up to two per SM (their shared memory fits twice when M <= 8),
// as many as make the tiles per CTA equal: 160 row tiles on 148 SMs are 160 CTAs of one tile, not 136 of one
// and 12 of two. An SM that hosts two CTAs has twice the copies in flight and pulls twice the bytes in the same
// time, so what matters is that no CTA is the last one left streaming. Measured over the decode step: 1.92 ->
// 1.72 ms. The one-launch decode step deals its tiles by the same rule.
int gemv_packed_ctas(int tiles, int sms, bool two_per_sm) {
    if (tiles <= sms) return tiles;
    if (!two_per_sm) return sms;
    const int per_cta = (tiles + 2 * sms - 1) / (2 * sms);
    return (tiles + per_cta - 1) / per_cta;
}

namespace {

bool packable(int N, int K, int g) {
    return N > 0 && K > 0 && K % 256 == 0 && K % g == 0 && (g == 64 || g == 128 || g % 256 == 0);
}

size_t fused_smem_bytes(int K, int G) {  // norm weight + padded code rows + scales
    return static_cast<size_t>(K) * 2 + static_cast<size_t>(8) * (K + 64) + static_cast<size_t>(8) * G * 4;
}

bool make_plan(const LinearArgs& a, Plan& pl) {
    const bool fused = a.norm_weight != nullptr;
    if (a.M < 1 || a.M > 32 || !a.packed) return false;
    if (!packable(a.N, a.K, a.g)) return false;
    if (fused) {
        // one warp per row; the norm emulates the reference's 1024-thread block, which it launches for dim > 512
        if (a.M > 8 || !a.X || a.K <= 512 || a.K > 4096 || a.dump) return false;
        if (a.smooth_inv || a.act_scale) return false;
        if ((reinterpret_cast<uintptr_t>(a.X) | reinterpret_cast<uintptr_t>(a.norm_weight) |
             reinterpret_cast<uintptr_t>(a.norm_residual) | reinterpret_cast<uintptr_t>(a.norm_x_out) |
             reinterpret_cast<uintptr_t>(a.codes_out)) & 15u)
            return false;
        if (a.norm_residual && a.norm_x_out == a.X) return false;  // other CTAs still read X
    } else {
        if (!a.Xq || !a.Xs) return false;
        if (reinterpret_cast<uintptr_t>(a.Xq) & 15u) return false;
    }
    if (a.epilogue == W8A8_EPI_SWIGLU && a.N % 16 != 0) return false;
    if (a.tp.world > 0 && (a.epilogue != W8A8_EPI_NONE || a.M > a.tp.max_tokens || a.tail_kind != kTailNone)) return false;
    if (!a.Y && a.tp.world == 0) return false;
    if (a.tail_kind != kTailNone) {
        if (fused || a.M > 8 || !a.tail_counters) return false;
        const int tg = a.tail_g;
        if (a.tail_kind == kTailRowNorm) {
            // a CTA per row, two 16-byte pieces per thread; the norm emulates the reference's 1024-thread block
            if (a.epilogue != W8A8_EPI_NONE || a.N % 256 != 0 || a.N <= 512 || a.N > 4096) return false;
            if (!a.tail_x || !a.tail_norm_weight) return false;
            if (a.tail_Xq && (!a.tail_Xs || !(tg == 64 || tg == 128 || tg == 256))) return false;
            if ((reinterpret_cast<uintptr_t>(a.tail_x) | reinterpret_cast<uintptr_t>(a.tail_norm_weight) |
                 reinterpret_cast<uintptr_t>(a.Y) | reinterpret_cast<uintptr_t>(a.tail_normed_out) |
                 reinterpret_cast<uintptr_t>(a.tail_Xq)) & 15u)
                return false;
        } else {
            const int kout = a.epilogue == W8A8_EPI_SWIGLU ? a.N / 2 : a.N;
            const int cpt = a.epilogue == W8A8_EPI_SWIGLU ? 8 : 16;
            if (a.epilogue == W8A8_EPI_RESIDUAL || !a.tail_Xq || !a.tail_Xs) return false;
            if (tg <= 0 || tg % cpt != 0 || tg % 8 != 0 || kout % 8 != 0) return false;
            if ((kout + tg - 1) / tg > kTailCounterInts) return false;
            if ((reinterpret_cast<uintptr_t>(a.Y) | reinterpret_cast<uintptr_t>(a.tail_Xq)) & 15u) return false;
        }
    }
    pl.pro = fused ? kProNorm : kProCodes;
    pl.stages = fused ? 2 : 3;
    pl.MT = a.M <= 8 ? 1 : (a.M <= 16 ? 2 : 4);
    pl.GM = a.g == 64 ? 64 : a.g == 128 ? 128 : 256;
    pl.bpu = a.g > 256 ? a.g / 256 : 1;
    pl.upt = a.K / (256 * pl.bpu);
    pl.block_bytes = kBlockW + 32 * (a.g >= 256 ? 1 : 256 / a.g);
    pl.tiles = (a.N + 15) / 16;
    pl.U = static_cast<long long>(pl.tiles) * pl.upt;
    // Up to two CTAs per SM at M <= 8 (their registers and shared memory fit twice), never more CTAs than row tiles.
    pl.ctas = gemv_packed_ctas(pl.tiles, num_sms(), pl.MT == 1);
    if ((pl.U + 1) * static_cast<long long>(pl.ctas) * kWarps >= (1ll << 32)) return false;  // 32-bit range math
    if (pl.tiles / pl.ctas + 2 > kLocalTiles) return false;  // arrival counters of a CTA's tiles sit in shared memory
    return true;
}

template <int MT, int GM, int PRO, int ST, int KI>
int launch_variant(const LinearArgs& a, const Plan& pl, int* status, cudaStream_t stream) {
    GemvPackedParams p;
    p.a = a;
    p.packed = static_cast<const unsigned char*>(a.packed);
    p.block_bytes = pl.block_bytes;
    p.upt = pl.upt;
    p.bpu = pl.bpu;
    p.U = static_cast<unsigned>(pl.U);
    p.status = status;
#ifdef W8A8_TRACE
    {
        const char* v = std::getenv("W8A8_ABLATE");
        p.ablate = v ? std::atoi(v) : 0;
    }
#endif
    auto kern = gemv_packed_kernel<MT, GM, PRO, ST, KI>;
    const size_t ring = static_cast<size_t>(kWarps) * ST * kStagePitch + 128;
    const size_t smem = ring + (PRO == kProNorm ? fused_smem_bytes(a.K, a.G) : 0);
    {  // per device, so on every launch (a host-side table write)
        const size_t most = ring + (PRO == kProNorm ? fused_smem_bytes(256 * KI, 4 * KI) : 0);
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(most));
        if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.ctas, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled(kPdlLinear) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "gemv_packed launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}

template <int MT, int GM>
int launch_pro(const LinearArgs& a, const Plan& pl, int* status, cudaStream_t s) {
    if constexpr (MT == 1) {
        if (pl.pro == kProNorm) {
            if (a.K <= 2560) return launch_variant<1, GM, kProNorm, 2, 10>(a, pl, status, s);
            return launch_variant<1, GM, kProNorm, 2, 16>(a, pl, status, s);
        }
    }
    return launch_variant<MT, GM, kProCodes, 3, 1>(a, pl, status, s);
}

template <int MT>
int launch_gm(const LinearArgs& a, const Plan& pl, int* status, cudaStream_t s) {
    switch (pl.GM) {
        case 64: return launch_pro<MT, 64>(a, pl, status, s);
        case 128: return launch_pro<MT, 128>(a, pl, status, s);
        default: return launch_pro<MT, 256>(a, pl, status, s);
    }
}

// One thread per 16 bytes of the packed image.
__global__ void __launch_bounds__(256) pack_weight_kernel(const int8_t* __restrict__ W, const __half* __restrict__ S,
                                                          int N, int K, int g, int G, int block_bytes,
                                                          unsigned char* __restrict__ out, size_t total16) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total16) return;
    const int per_block = block_bytes / 16;
    const size_t blk = i / per_block;
    const int r = static_cast<int>(i % per_block);
    const int kblocks = K / 256;
    const int rt = static_cast<int>(blk / kblocks), kb = static_cast<int>(blk % kblocks);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < kBlockW / 16) {
        // [chunk][half][lane]: 16 bytes of row (lane/4) + 8*half at K offset chunk*64 + (lane%4)*16
        const int lane = r & 31, half = (r >> 5) & 1, ch = r >> 6;
        const int row = rt * 16 + (lane >> 2) + 8 * half;
        const int k = kb * 256 + ch * 64 + (lane & 3) * 16;
        if (row < N) v = *reinterpret_cast<const uint4*>(W + static_cast<size_t>(row) * K + k);
    } else {
        // scales: [16 rows][gpb] fp16, 8 halves per 16-byte piece
        const int gpb = g >= 256 ? 1 : 256 / g;
        __align__(16) __half h[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int idx = (r - kBlockW / 16) * 8 + e;  // row * gpb + q
            const int row = rt * 16 + idx / gpb, q = idx % gpb;
            const int j = g >= 256 ? (kb * 256) / g : kb * gpb + q;
            h[e] = row < N ? S[static_cast<size_t>(row) * G + j] : __float2half(0.0f);
        }
        v = *reinterpret_cast<const uint4*>(h);
    }
    reinterpret_cast<uint4*>(out)[i] = v;
}

}  // namespace

size_t packed_weight_bytes(int N, int K, int g) {
    g = norm_group(K, g);
    if (!packable(N, K, g)) return 0;
    const size_t block_bytes = kBlockW + 32 * (g >= 256 ? 1 : 256 / g);
    return static_cast<size_t>((N + 15) / 16) * (K / 256) * block_bytes;
}

int launch_pack_weight(const int8_t* W, const __half* S, int N, int K, int g, void* out, cudaStream_t s) {
    g = norm_group(K, g);
    const size_t bytes = packed_weight_bytes(N, K, g);
    if (bytes == 0) return fail(W8A8_ERR_UNSUPPORTED, "N=%d K=%d group=%d cannot be packed (K %% 256, group 64/128/k*256)", N, K, g);
    if ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(out)) & 15u)
        return fail(W8A8_ERR_INVALID_ARG, "pack_weight needs 16-byte aligned W and output");
    const int block_bytes = kBlockW + 32 * (g >= 256 ? 1 : 256 / g);
    const size_t total16 = bytes / 16;
    pack_weight_kernel<<<static_cast<unsigned>((total16 + 255) / 256), 256, 0, s>>>(
        W, S, N, K, g, num_groups(K, g), block_bytes, static_cast<unsigned char*>(out), total16);
    return check_launch("pack_weight_kernel");
}

bool gemv_packed_supports(const LinearArgs& a) {
    Plan pl;
    return make_plan(a, pl);
}

int launch_linear_gemv_packed(const LinearArgs& a, int* device_status, cudaStream_t s) {
    Plan pl;
    if (!make_plan(a, pl)) return fail(W8A8_ERR_UNSUPPORTED, "packed gemv kernel does not take this shape");
    switch (pl.MT) {
        case 1: return launch_gm<1>(a, pl, device_status, s);
        case 2: return launch_gm<2>(a, pl, device_status, s);
        default: return launch_gm<4>(a, pl, device_status, s);
    }
}

}  // namespace w8a8

W8A8_TRACE_READER(gemv_packed)
