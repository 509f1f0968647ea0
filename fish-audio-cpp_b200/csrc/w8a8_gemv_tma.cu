// Small-M (decode) W8A8 linear, TMA-fed persistent form: the HBM-roofline kernel.
//
// Same arithmetic as w8a8_gemv.cu (exact int32 sum per K-group from mma.sync.m16n8k32.s8 with the
// weights as the A operand, then acc = fma(float(P) * ws, xs, acc) over ascending groups); what
// differs is how the weight bytes reach the SM and how work is divided.
//
// * One CTA per SM, four warps, and every warp is its own pipeline: lane 0 keeps kStages TMA tile
//   loads (16 weight rows x 256 bytes of K = 4 KB per instruction, 128-byte swizzle) in flight into
//   a ring that belongs to the warp, all lanes wait on the tile's mbarrier, read their A fragments
//   with conflict-light 128-bit shared loads, and issue the MMAs. 4 warps x 4 stages x 4 KB = 64 KB
//   in flight per SM, independent of register count: that depth, not occupancy, is what fills HBM.
//   (Two such CTAs fit one SM, so the next launch's prologue can overlap this one's tail.)
// * Work is cut stream-K style. The matrix is a list of units (16 rows x one 256-byte K block, or
//   one whole K-group when groups are larger), ordered row tile by row tile; warp w of W takes the
//   contiguous range [w*U/W, (w+1)*U/W). All warps therefore stream the same number of bytes (+-1
//   unit), whatever N and K are. A row tile that lies wholly inside one warp's range is finished by
//   that warp; a tile cut by a range boundary is summed from per-warp fp32 partials in scratch by
//   whichever contributor arrives last, always in ascending-K order, so results do not depend on
//   timing.
// * Launched with programmatic dependent launch: the first kStages tiles of weights are requested
//   before griddepcontrol.wait, i.e. while the kernel producing the activations still runs.
//
// Every mbarrier wait is bounded; on expiry the warp records an error word and leaves.
#include "sm100_ptx.cuh"
#include "w8a8_internal.h"

namespace w8a8 {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 4;
constexpr int kStageBytes = 16 * 256;  // one TMA box: 16 rows x 2 K-blocks of 128 bytes
constexpr int kRingBytes = kStages * kStageBytes;
constexpr int kScaleQ = 8;  // units of weight scales kept in flight per warp

struct GemvTmaParams {
    LinearArgs a;
    int ublock;     // bytes of K per unit: max(g, 256)
    int upt;        // units per 16-row tile = K / ublock
    int spu;        // 256-byte steps (TMA boxes) per unit = ublock / 256
    int gpu;        // groups per unit = ublock / g
    unsigned U;     // units in all = ceil(N / 16) * upt   ((U + 1) * NW fits 32 bits, checked on the host)
    int NW;         // warps that take part: min(warps in the grid, U), so that none has an empty range
    float* partials;  // [NW][2][MT*4][32] fp32
    int* counters;    // [row tiles], zero between launches
    int* status;
};

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

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ float ld_cg(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];\n" : "=f"(v) : "l"(p));
    return v;
}

// GM: 64 or 128 = the group size itself; 256 = any group size that is a multiple of 256
// (then one unit is exactly one group).
template <int MT, int GM>
__global__ void __launch_bounds__(kThreads, 2)
gemv_tma_kernel(const __grid_constant__ CUtensorMap wmap, const GemvTmaParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bars[kWarps][kStages];
    __shared__ __align__(16) unsigned char scale_q[kWarps][kScaleQ][16 * 8];
    const LinearArgs& a = p.a;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gq = lane >> 2, c = lane & 3;
    constexpr int GPU = GM == 64 ? 4 : GM == 128 ? 2 : 1;  // groups per unit

    // ---- this warp's contiguous range of units; consecutive ranges sit on different SMs ----
    const unsigned gw = warp * gridDim.x + blockIdx.x;
    const unsigned NW = p.NW, U = p.U;
    const unsigned u0 = gw * U / NW, u1 = (gw + 1) * U / NW;
    const int T = gw < NW ? static_cast<int>(u1 - u0) * p.spu : 0;  // 256-byte steps

    const uint32_t ring = ((ptx::smem_u32(smem_raw) + 1023u) & ~1023u) + warp * kRingBytes;
    uint64_t* bar = bars[warp];
    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) ptx::mbar_init(&bar[s], 1);
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
    }
    __syncwarp();

    // producer cursor (lane 0): step index, position inside the unit, unit's K block and row tile
    int pt = 0, psi = 0;
    int pub = static_cast<int>(u0 % p.upt), prt = static_cast<int>(u0 / p.upt);
    auto issue = [&]() {  // lane 0 only
        const int slot = pt % kStages;
        ptx::mbar_arrive_expect_tx(&bar[slot], kStageBytes);
        // coordinates: byte inside the 128-byte K-block, K-block index, weight row
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(ring + slot * kStageBytes), "l"(&wmap), "r"(ptx::smem_u32(&bar[slot])), "r"(0),
              "r"((pub * p.ublock + psi * 256) >> 7), "r"(prt * 16)
            : "memory");
        ++pt;
        if (++psi == p.spu) {
            psi = 0;
            if (++pub == p.upt) { pub = 0; ++prt; }
        }
    };
    if (lane == 0) {
        const int pre = T < kStages ? T : kStages;
        for (int i = 0; i < pre; ++i) issue();
    }
    // Everything above touches only weights. Let the next launch begin its own prologue, then wait
    // for the kernel before this one: it produces the activations.
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();

    const int8_t* xq[MT];
    const float* xsp[MT][2];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        xq[nt] = a.Xq + static_cast<size_t>(min(nt * 8 + gq, a.M - 1)) * a.K + c * 16;
        xsp[nt][0] = a.Xs + static_cast<size_t>(min(nt * 8 + 2 * c, a.M - 1)) * a.G;
        xsp[nt][1] = a.Xs + static_cast<size_t>(min(nt * 8 + 2 * c + 1, a.M - 1)) * a.G;
    }

    int P[MT][4];
    float acc[MT][4];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int r = 0; r < 4; ++r) { P[nt][r] = 0; acc[nt][r] = 0.0f; }

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
                        __half y = __float2half(v[nt][2 * hrow + e]);
                        if (a.epilogue == W8A8_EPI_RESIDUAL)
                            y = __float2half(__half2float(y) + __half2float(a.residual[o]));
                        a.Y[o] = y;
                    }
                }
            }
        }
    };

    auto warp_of_unit = [&](unsigned u) -> unsigned {  // the warp whose range holds unit u
        return ((u + 1) * NW - 1) / U;
    };

    // Called when the warp has added its last unit of row tile rt into acc.
    auto finish_tile = [&](int rt) {
        const unsigned t_lo = static_cast<unsigned>(rt) * p.upt, t_hi = t_lo + p.upt;  // [t_lo, t_hi)
        if (u0 <= t_lo && t_hi <= u1) {
            store_tile(rt, acc);
        } else {
            // This warp holds only part of the tile's K range: park the partial, and if every other
            // contributor has parked too, add them up in ascending-K order and store.
            const unsigned first = warp_of_unit(t_lo), last = warp_of_unit(t_hi - 1);
            constexpr int kSlot = MT * 4 * 32;
            const int my_slot = (static_cast<int>(u0 / p.upt) == rt) ? 0 : 1;
            float* mine = p.partials + (static_cast<size_t>(gw) * 2 + my_slot) * kSlot;
#pragma unroll
            for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                for (int r = 0; r < 4; ++r) mine[(nt * 4 + r) * 32 + lane] = acc[nt][r];
            __threadfence();
            __syncwarp();
            unsigned old = 0;
            if (lane == 0) old = atomicAdd(reinterpret_cast<unsigned*>(&p.counters[rt]), 1u);
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old == last - first) {
                __threadfence();
                float sum[MT][4];
#pragma unroll
                for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                    for (int r = 0; r < 4; ++r) sum[nt][r] = 0.0f;
                // four contributors' loads are in flight at a time; the adds stay in ascending-K order
                for (unsigned w = first; w <= last; w += 4) {
                    float v[4][MT][4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const unsigned ww = w + q <= last ? w + q : last;
                        const int slot = (static_cast<int>((ww * U / NW) / p.upt) == rt) ? 0 : 1;
                        const float* src = p.partials + (static_cast<size_t>(ww) * 2 + slot) * kSlot;
#pragma unroll
                        for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                            for (int r = 0; r < 4; ++r) v[q][nt][r] = ld_cg(src + (nt * 4 + r) * 32 + lane);
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (w + q <= last) {
#pragma unroll
                            for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                                for (int r = 0; r < 4; ++r) sum[nt][r] += v[q][nt][r];
                        }
                }
                store_tile(rt, sum);
                if (lane == 0) p.counters[rt] = 0;  // ready for the next launch
            }
        }
#pragma unroll
        for (int nt = 0; nt < MT; ++nt)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[nt][r] = 0.0f;
    };

    auto promote = [&](int rt, int j, __half hsa, __half hsb) {
        const float fa = __half2float(hsa), fb = __half2float(hsb);
#pragma unroll
        for (int nt = 0; nt < MT; ++nt) {
            const float x0 = __ldg(xsp[nt][0] + j), x1 = __ldg(xsp[nt][1] + j);
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

    // ---- consumer loop: one 16 x 256-byte box per step ----
    int si = 0;
    int ub = static_cast<int>(u0 % p.upt), rt = static_cast<int>(u0 / p.upt);
    // Weight scales are 2-byte reads scattered over DRAM; a read issued when its unit starts would
    // stall every unit for a full memory latency. They are copied kScaleQ-1 units ahead instead, with
    // cp.async (no register is tied up while the copy is in flight), into a small per-warp queue in
    // shared memory: slot = unit sequence number % kScaleQ, 16 rows x 8 bytes per slot. One
    // commit group per unit (empty past the end of the range) keeps wait_group arithmetic exact.
    constexpr int kCopyBytes = GPU == 4 ? 8 : 4;  // GPU == 1: the aligned 4-byte word holding the scale
    const uint32_t sq = ptx::smem_u32(&scale_q[warp][0][0]);
    int sub = ub, srt = rt;  // cursor of the next unit whose scales get requested
    unsigned su = u0, sseq = 0;
    auto request_scales = [&]() {
        if (su < u1 && lane < 16) {
            const int row = min(srt * 16 + lane, a.N - 1);
            const size_t idx = static_cast<size_t>(row) * a.G + sub * GPU;
            const __half* src = a.w_scale + (GPU == 1 ? (idx & ~size_t(1)) : idx);
            const uint32_t dst = sq + ((sseq % kScaleQ) * 16 + lane) * 8;
            asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(dst), "l"(src), "n"(kCopyBytes) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (su < u1) {
            ++su;
            if (++sub == p.upt) { sub = 0; ++srt; }
        }
        ++sseq;
    };
    if (T > 0) {
#pragma unroll
        for (int d = 0; d + 1 < kScaleQ; ++d) request_scales();
    }
    __half sa[GPU], sb[GPU];
    unsigned useq = 0;  // sequence number of the unit being processed
    bool ok = true;
    for (int t = 0; t < T; ++t) {
        const int slot = t % kStages;
        const int kbase = ub * p.ublock + si * 256;
        if (si == 0) {  // a new unit: request the unit kScaleQ-1 ahead, then pick up this unit's scales
            request_scales();
            asm volatile("cp.async.wait_group %0;" ::"n"(kScaleQ - 1) : "memory");
            __syncwarp();
            const uint32_t base = sq + (useq % kScaleQ) * 16 * 8;
            if (GPU == 1) {
                // which half of the copied word: parity of the scale's element index
                const int rowA = min(rt * 16 + gq, a.N - 1), rowB = min(rt * 16 + gq + 8, a.N - 1);
                const uint32_t wa_ = lds32(base + gq * 8), wb_ = lds32(base + (gq + 8) * 8);
                const bool oa = ((static_cast<size_t>(rowA) * a.G + ub) & 1) != 0;
                const bool ob = ((static_cast<size_t>(rowB) * a.G + ub) & 1) != 0;
                sa[0] = __ushort_as_half(static_cast<unsigned short>(oa ? wa_ >> 16 : wa_ & 0xffffu));
                sb[0] = __ushort_as_half(static_cast<unsigned short>(ob ? wb_ >> 16 : wb_ & 0xffffu));
            } else {
#pragma unroll
                for (int q = 0; q < GPU; q += 2) {
                    const uint32_t wa_ = lds32(base + gq * 8 + q * 2), wb_ = lds32(base + (gq + 8) * 8 + q * 2);
                    sa[q] = __ushort_as_half(static_cast<unsigned short>(wa_ & 0xffffu));
                    sa[(q + 1) % GPU] = __ushort_as_half(static_cast<unsigned short>(wa_ >> 16));
                    sb[q] = __ushort_as_half(static_cast<unsigned short>(wb_ & 0xffffu));
                    sb[(q + 1) % GPU] = __ushort_as_half(static_cast<unsigned short>(wb_ >> 16));
                }
            }
            ++useq;
        }
        // Activation codes of the box's first K-block, from L1, before blocking on the weights.
        uint4 xv[2][MT];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int nt = 0; nt < MT; ++nt)
                xv[h][nt] = __ldg(reinterpret_cast<const uint4*>(xq[nt] + kbase + h * 64));

        if (!ptx::mbar_wait_bounded(&bar[slot], (t / kStages) & 1)) {
            if (lane == 0) atomicExch(p.status, 100 + slot);
            ok = false;
            break;
        }
        // Shared layout of a box: 128-byte lines ordered [row][K-block]; the 16-byte chunk index of a
        // line is XORed with (line & 7) by the 128-byte swizzle. Rows gq and gq+8 share that value.
        const uint32_t st = ring + slot * kStageBytes;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
            const uint32_t line = static_cast<uint32_t>(gq * 2 + kb);
            if (kb == 1) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int nt = 0; nt < MT; ++nt)
                        xv[h][nt] = __ldg(reinterpret_cast<const uint4*>(xq[nt] + kbase + 128 + h * 64));
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t phys = (static_cast<uint32_t>(h * 4 + c) ^ (line & 7u)) << 4;
                const uint4 wa = lds128(st + line * 128 + phys), wb = lds128(st + (line + 16) * 128 + phys);
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    mma_s8(P[nt], wa.x, wb.x, wa.y, wb.y, xv[h][nt].x, xv[h][nt].y);
                    mma_s8(P[nt], wa.z, wb.z, wa.w, wb.w, xv[h][nt].z, xv[h][nt].w);
                }
                if (GM == 64) promote(rt, ub * 4 + kb * 2 + h, sa[(kb * 2 + h) % GPU], sb[(kb * 2 + h) % GPU]);
            }
            if (GM == 128) promote(rt, ub * 2 + kb, sa[kb % GPU], sb[kb % GPU]);
        }
        // The box's bytes are in registers: the slot may be refilled.
        __syncwarp();
        if (lane == 0 && pt < T) {
            ptx::fence_proxy_async();
            issue();
        }
        if (++si == p.spu) {
            si = 0;
            if (GM == 256) promote(rt, ub, sa[0], sb[0]);
            if (++ub == p.upt) {
                finish_tile(rt);
                ub = 0;
                ++rt;
            }
        }
    }
    if (ok && T > 0 && ub != 0) finish_tile(rt);  // the range ended inside a tile
    if (!ok) {
        // Leave only once every requested box has landed (or a second bounded wait ran out): a TMA write
        // must not arrive in shared memory that already belongs to another CTA.
        pt = __shfl_sync(0xffffffffu, pt, 0);
        for (int s = 0; s < kStages; ++s)
            if (pt > s) ptx::mbar_wait_bounded(&bar[s], ((pt - 1 - s) / kStages) & 1, 1u << 16);
    }
}

struct Plan {
    int MT, GM, ublock, upt, spu;
    long long U;
    int ctas;
    size_t partial_bytes;
    int tiles;
};

int num_sms() {  // of the current device (not cached: one process may drive several devices)
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
        v = 148;
    return v;
}

bool make_plan(const LinearArgs& a, Plan& pl) {
    if (a.M < 1 || a.M > 32 || !a.Xq || !a.Xs) return false;
    if (a.K % 256 != 0 || a.K % a.g != 0) return false;
    if (!(a.g == 64 || a.g == 128 || a.g % 256 == 0)) return false;
    if ((reinterpret_cast<uintptr_t>(a.W) | reinterpret_cast<uintptr_t>(a.Xq)) & 15u) return false;
    if (a.epilogue == W8A8_EPI_SWIGLU && a.N % 16 != 0) return false;
    if (!a.splitk_partials || !a.splitk_counters) return false;
    pl.MT = a.M <= 8 ? 1 : (a.M <= 16 ? 2 : 4);
    pl.GM = a.g == 64 ? 64 : a.g == 128 ? 128 : 256;
    pl.ublock = a.g > 256 ? a.g : 256;
    if (a.K % pl.ublock != 0) return false;  // e.g. K = 128 with g = 64
    // scales are copied as aligned 4-byte words: the last element must not start a word of its own
    if (a.g >= 256 && ((static_cast<long long>(a.N) * a.G) & 1) != 0) return false;
    if ((reinterpret_cast<uintptr_t>(a.w_scale) & (a.g == 64 ? 7u : 3u)) != 0) return false;
    pl.upt = a.K / pl.ublock;
    pl.spu = pl.ublock / 256;
    pl.tiles = (a.N + 15) / 16;
    pl.U = static_cast<long long>(pl.tiles) * pl.upt;
    pl.ctas = num_sms();
    if ((pl.U + 1) * static_cast<long long>(pl.ctas) * kWarps >= (1ll << 32)) return false;  // 32-bit range math
    pl.partial_bytes = static_cast<size_t>(pl.ctas) * kWarps * 2 * pl.MT * 4 * 32 * sizeof(float);
    if (pl.partial_bytes > a.splitk_partial_bytes) return false;
    if (static_cast<size_t>(pl.tiles) > a.splitk_counter_count) return false;
    return true;
}

template <int MT, int GM>
int launch_variant(const LinearArgs& a, const Plan& pl, int* status, cudaStream_t stream) {
    CUtensorMap map;
    // W seen as [N rows][K/128 blocks][128 bytes]; one box = 16 rows x 2 blocks, 128-byte swizzle.
    int rc = make_tensor_map_3d_u8(&map, a.W, 128, static_cast<uint64_t>(a.K / 128), static_cast<uint64_t>(a.N),
                                   128, static_cast<uint64_t>(a.K), 128, 2, 16, 1);
    if (rc) return rc;
    GemvTmaParams p;
    p.a = a;
    p.ublock = pl.ublock;
    p.upt = pl.upt;
    p.spu = pl.spu;
    p.gpu = pl.ublock / a.g;
    p.U = static_cast<unsigned>(pl.U);
    p.NW = static_cast<int>(pl.U < static_cast<long long>(pl.ctas) * kWarps ? pl.U : pl.ctas * kWarps);
    p.partials = static_cast<float*>(a.splitk_partials);
    p.counters = a.splitk_counters;
    p.status = status;
    auto kern = gemv_tma_kernel<MT, GM>;
    const size_t smem = static_cast<size_t>(kWarps) * kRingBytes + 1024;
    {  // per device, so on every launch (a host-side table write)
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
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
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map, p);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "gemv_tma launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}

template <int MT>
int launch_gm(const LinearArgs& a, const Plan& pl, int* status, cudaStream_t s) {
    switch (pl.GM) {
        case 64: return launch_variant<MT, 64>(a, pl, status, s);
        case 128: return launch_variant<MT, 128>(a, pl, status, s);
        default: return launch_variant<MT, 256>(a, pl, status, s);
    }
}

}  // namespace

bool gemv_tma_supports(const LinearArgs& a) {
    Plan pl;
    return make_plan(a, pl);
}

int launch_linear_gemv_tma(const LinearArgs& a, int* device_status, cudaStream_t s) {
    Plan pl;
    if (!make_plan(a, pl)) return fail(W8A8_ERR_UNSUPPORTED, "TMA gemv kernel does not take this shape");
    switch (pl.MT) {
        case 1: return launch_gm<1>(a, pl, device_status, s);
        case 2: return launch_gm<2>(a, pl, device_status, s);
        default: return launch_gm<4>(a, pl, device_status, s);
    }
}

}  // namespace w8a8
