// Large-M (prefill) W8A8 linear on the 5th-generation tensor cores: TMA -> shared memory ->
// tcgen05.mma kind::i8 -> int32 accumulators in tensor memory -> fp32 promote per K-group.
//
// Replaces, for tokens > 32, the reference's loop of one cuBLAS int8 GEMM per K-group plus an
// accumulate pass over the whole [tokens, rows] matrix per group and a cast pass
// (int8_gemm.cu:423-505): here a K-group's exact int32 sums never leave the SM.
//
// One persistent CTA per SM walks over 128-token x 256-row output tiles; the shared-memory stage ring and the
// tensor-memory accumulator ring keep running across tiles, so the promote of a tile's last K-groups overlaps
// the MMAs of the next tile. A tile is 128 x 256 (the larger the tile, the fewer operand bytes per
// MAC have to come out of L2, which is what bounds this kernel) with three kinds of warps:
//   warp 0      producer: one lane issues TMA loads of 128 x 128-byte boxes of the activation codes
//               and of the weights (both are row-major with K contiguous, i.e. already the K-major
//               operand; the 128-byte swizzle is applied by TMA) into a ring of kStages stages;
//   warp 1      MMA issuer: one lane issues tcgen05.mma (M=128, N=256, K=32 per instruction), four per
//               128-byte stage. Each K-group accumulates into its own 256-column slice of tensor
//               memory (2 slices = all 512 columns), starting with "overwrite"; a tcgen05.commit
//               hands the slice to the epilogue and another frees the shared-memory stage;
//   warps 4..11 epilogue (two warpgroups; setmaxnreg moves registers from warpgroup 0 to them): thread <-> (token row = tensor-memory lane, 128 of the 256 columns). For every
//               K-group they read the int32 sums with tcgen05.ld and promote
//               acc = fma(float(P) * ws[n,j], xs[m,j], acc) in ascending group order into 128 fp32
//               registers per thread — the arithmetic and order of accumulate_group_kernel
//               (int8_gemm.cu:213-234) — while the MMA warp already fills the next slice. The promote is
//               the CUDA-core bottleneck of this kernel, so it uses packed fp32x2 add/mul/fma and, for
//               groups of at most 256 (|P| < 2^22), an exact integer-add + float-subtract conversion
//               instead of the quarter-rate I2F. Weight scales of the group are staged in shared memory
//               once per CTA; the final fp16 store applies the optional residual / SwiGLU epilogue.
// Every mbarrier wait is bounded; a wait that runs out records an error word, and the CTA still
// frees its tensor memory before it returns.
#include <cstdlib>

#include "sm100_ptx.cuh"
#include "w8a8_internal.h"

namespace w8a8 {
namespace {

#ifdef W8A8_TRACE
// Diagnostic build only: SM-clock stamps of CTA 0's producer lane (per K-block), MMA lane and first epilogue warp
// (per K-group), first kGemmEvents of each; read out and cleared by w8a8_trace_read_gemm.
constexpr int kGemmEvents = 512;
__device__ unsigned long long g_gemm_ev[3][kGemmEvents][4];
#define GEMM_EV(role, idx, slot, value)                                                   \
    do {                                                                                  \
        if (blockIdx.x == 0 && (idx) < kGemmEvents) g_gemm_ev[role][idx][slot] = (value); \
    } while (0)
#define GEMM_CLK() static_cast<unsigned long long>(clock64())
#define GEMM_ABLATE(bit) ((p.ablate & (bit)) != 0)
#else
#define GEMM_ABLATE(bit) false
#define GEMM_EV(role, idx, slot, value) do {} while (0)
#define GEMM_CLK() 0ull
#endif

constexpr int BM = 128, BN = 256, BK = 128;  // BK in bytes = int8 elements
constexpr int kStagesDirect = 4;   // operand stages when the epilogue stores straight to global memory
constexpr int kStagesStaged = 3;   // ... when the output tile is staged in shared memory for a TMA store (64 KB)
constexpr int kStagesPairDirect = 6, kStagesPairStaged = 4;  // a CTA of a pair holds 32 KB per stage, not 48
constexpr int kOutPanelBytes = BM * 128;              // 128 token rows x 64 fp16 columns, 128-byte swizzle
constexpr int kOutStageBytes = (BN / 64) * kOutPanelBytes;  // the whole 128 x 256 fp16 tile
constexpr int kAccStages = 2;  // 2 x 256 columns = the whole tensor memory
constexpr int kStageBytes = (BM + BN) * BK;
constexpr int kStageBytesPair = (BM + BN / 2) * BK;  // a CTA of a pair loads its 128 token rows and HALF of the weight rows
constexpr int kEpiWarps = 8;                // two per tensor-memory lane quadrant, 128 columns each
constexpr int kThreads = 128 + kEpiWarps * 32;  // warpgroup 0: producer, MMA issuer, two idle warps; 1-2: epilogue
// Registers per thread the 384-thread CTA is launched with (what ptxas reports for this kernel): warpgroup 0 gives up
// 128 x (168 - 40) = 16384, the two epilogue warpgroups take 2 x 128 x (232 - 168) = 16384.
constexpr int kLaunchRegs = 168;
static_assert(128 * (kLaunchRegs - 40) == (kEpiWarps / 4) * 128 * (232 - kLaunchRegs), "setmaxnreg sums must balance");
constexpr uint32_t kSpin = 1u << 21;
constexpr int kWsGroups = 4;

struct GemmParams {
    LinearArgs a;
    int* status;
    int mmas_per_group;  // g / 32
    int num_kblocks;     // K / 128
    int tiles_m, tiles_total;
    int ablate;  // diagnostic build only (W8A8_GEMM_ABLATE): 1 no sums read and no promote, 2 sums read but no promote,
                 // 4 no operand loads (the MMAs run on whatever shared memory holds). Results are wrong by design.
};

// ---- tcgen05 wrappers ----
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(smem_dst)),
                 "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// The same for a CTA pair (cta_group::2): one warp of EACH CTA of the pair, with the same warp index, issues them.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(smem_dst)),
                 "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// Completion of the pair's MMAs issued so far by this thread, signalled on the mbarrier at the same shared-memory
// offset in BOTH CTAs of the pair (an arrive, not a load: nothing is copied).
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     ptx::smem_u32(bar)), "h"(static_cast<uint16_t>(3))
                 : "memory");
}
__device__ __forceinline__ void mma_i8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address, in the cluster's shared-memory window, of `local` in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     ptx::smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- packed fp32x2 arithmetic (two IEEE round-to-nearest results per instruction) ----
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    return static_cast<uint64_t>(__float_as_uint(a)) | (static_cast<uint64_t>(__float_as_uint(b)) << 32);
}
__device__ __forceinline__ float lo2(uint64_t v) { return __uint_as_float(static_cast<uint32_t>(v)); }
__device__ __forceinline__ float hi2(uint64_t v) { return __uint_as_float(static_cast<uint32_t>(v >> 32)); }
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
// Four consecutive floats of shared memory as two packed pairs, in one 16-byte load.
__device__ __forceinline__ void lds_pairs(const float* p, uint64_t& lo, uint64_t& hi) {
    asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(lo), "=l"(hi) : "r"(ptx::smem_u32(p)));
}
// Exact int32 -> fp32 for |v| < 2^22: the integer lands in the mantissa of 1.5 * 2^23, which is then removed.
__device__ __forceinline__ uint64_t ints_to_floats_magic(uint32_t a, uint32_t b) {
    const uint64_t biased = static_cast<uint64_t>(a + 0x4B400000u) | (static_cast<uint64_t>(b + 0x4B400000u) << 32);
    return add2(biased, pack2(-12582912.0f, -12582912.0f));
}

// Shared-memory operand descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    return static_cast<uint64_t>((saddr & 0x3ffffu) >> 4) | (1ull << 16) /* leading offset (unused) */ |
           (static_cast<uint64_t>(1024 >> 4) << 32) /* stride between 8-row groups */ | (1ull << 46) /* version */ |
           (2ull << 61) /* SWIZZLE_128B */;
}
// Instruction descriptor: int8 x int8 -> int32, both operands K-major, M = 128, N = BN.
constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                            (static_cast<uint32_t>(BM >> 4) << 24);
// The pair's instruction: M = 256 (128 token rows from each CTA), N = BN (half of the weight rows from each CTA).
constexpr uint32_t kIdescPair = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                                (static_cast<uint32_t>((2 * BM) >> 4) << 24);

// MAGIC: groups of at most 256, whose sums convert to fp32 by integer add + float subtract. A template
// parameter, not a run-time flag: the flag cost a branch per four sums in the promote loop.
// STAGED: the finished fp16 tile goes to shared memory (64-column panels, 128-byte swizzle) and from there to global
// memory by TMA (cp.async.bulk.tensor store): the epilogue warps are back at the next tile's promote after about a
// microsecond instead of the 7-8 us their own 16-byte stores to 128 different rows took, during which the tensor
// pipe stood still (both accumulator stages full). The tile's store then overlaps the next tile. Costs one of the
// four operand stages. Needs an output row pitch that is a multiple of 16 bytes; other shapes store directly.
// PAIR: two CTAs on the two SMs of one cluster share a 256-token x 256-row tile: each loads its own 128 token rows and
// HALF of the 256 weight rows, the leader (cluster rank 0) issues tcgen05.mma.cta_group::2 (M = 256), which reads the
// operands out of both CTAs' shared memory and leaves each CTA's 128 x 256 sums in that CTA's own tensor memory.
// Operand bytes per MAC out of L2 drop by a third ((128 + 128) K instead of (128 + 256) K per 128 x 256 outputs),
// which is what bounds the kernel at g = 256. No load is multicast: each CTA issues plain TMA loads into its own
// shared memory, completing on the leader's mbarrier. Barriers: full[] lives in the leader (one arrive with the
// byte count of both CTAs); empty[] and acc_full[] exist in both CTAs and are signalled in both by the leader's
// commit; acc_empty[] lives in the leader and counts the epilogue warps of both CTAs. The epilogue is per CTA and
// does not know about the pair.
template <bool MAGIC, bool STAGED, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_y, const GemmParams p) {
    constexpr int kStages = PAIR ? (STAGED ? kStagesPairStaged : kStagesPairDirect) : (STAGED ? kStagesStaged : kStagesDirect);
    constexpr int kStageBytes = PAIR ? kStageBytesPair : w8a8::kStageBytes;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages];
    __shared__ __align__(8) uint64_t acc_full[kAccStages], acc_empty[kAccStages];
    __shared__ uint32_t tmem_base_s;
    __shared__ int failed_s;
    __shared__ __align__(16) float ws_s[2][kWsGroups][BN];  // weight scales of kWsGroups K-groups, double-buffered

    const LinearArgs& a = p.a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tiles = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t out_stage = tiles + kStages * kStageBytes;  // STAGED: the fp16 output tile (1024-byte aligned)
    const int G = a.G;
    // the unit that walks over tiles: a CTA, or a pair of CTAs
    const uint32_t crank = PAIR ? cluster_rank() : 0u;
    const int walker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int walkers = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    constexpr int kWalkM = PAIR ? 2 * BM : BM;  // token rows per tile of a walker
    auto tile_m0 = [&](int tile) { return (tile % p.tiles_m) * kWalkM + static_cast<int>(crank) * BM; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(&full_bar[s], 1); ptx::mbar_init(&empty_bar[s], 1); }
        for (int s = 0; s < kAccStages; ++s) {
            ptx::mbar_init(&acc_full[s], 1);
            ptx::mbar_init(&acc_empty[s], PAIR ? 2 * kEpiWarps : kEpiWarps);
        }
        failed_s = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            tmem_alloc_pair(&tmem_base_s, 512);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(&tmem_base_s, 512);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    // The activation codes come from the kernel before this one (the row quantiser).
    ptx::pdl_wait();

    if (warp < 4) {
      // warpgroup 0 gives registers away; the two epilogue warpgroups take them
      asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
      if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
          int kb = 0;  // running K-block counter over all the tiles of this CTA: the stage ring never restarts
          bool ok = true;
          // a pair's loads complete on the LEADER's barrier, which alone expects the bytes of both CTAs
          const uint32_t full0 = PAIR ? map_to_rank(ptx::smem_u32(&full_bar[0]), 0) : ptx::smem_u32(&full_bar[0]);
          for (int tile = walker; tile < p.tiles_total && ok; tile += walkers) {
            const int m0 = tile_m0(tile), n0 = (tile / p.tiles_m) * BN + (PAIR ? static_cast<int>(crank) * (BN / 2) : 0);
            for (int kbt = 0; kbt < p.num_kblocks; ++kbt, ++kb) {
                const int s = kb % kStages;
                GEMM_EV(0, kb, 0, GEMM_CLK());
                if (kb >= kStages && !ptx::mbar_wait_bounded(&empty_bar[s], ((kb / kStages) - 1) & 1, kSpin)) {
                    atomicExch(p.status, 200 + s);
                    atomicExch(&failed_s, 1);
                    ok = false;
                    break;
                }
                GEMM_EV(0, kb, 1, GEMM_CLK());
                if (GEMM_ABLATE(4)) {
                    if (crank == 0) ptx::mbar_arrive(&full_bar[s]);
                    continue;
                }
                const uint32_t dst = tiles + s * kStageBytes;
                const uint32_t bar = full0 + s * static_cast<uint32_t>(sizeof(uint64_t));
                if constexpr (PAIR) {
                    if (crank == 0) ptx::mbar_arrive_expect_tx(&full_bar[s], 2 * kStageBytes);
                    asm volatile(
                        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                        ::"r"(dst), "l"(&map_x), "r"(bar), "r"(kbt * BK), "r"(m0) : "memory");
                    asm volatile(
                        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                        ::"r"(dst + BM * BK), "l"(&map_w), "r"(bar), "r"(kbt * BK), "r"(n0) : "memory");
                } else {
                    ptx::mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                        ::"r"(dst), "l"(&map_x), "r"(bar), "r"(kbt * BK), "r"(m0) : "memory");
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                        ::"r"(dst + BM * BK), "l"(&map_w), "r"(bar), "r"(kbt * BK), "r"(n0) : "memory");
                }
            }
          }
        }
        __syncwarp();
      } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && crank == 0) {  // of a pair, the leader alone issues
            int my_tiles = 0;
            for (int tile = walker; tile < p.tiles_total; tile += walkers) ++my_tiles;
            // One iteration per K-block: wait for the stage, then its four MMAs back to back. The issuing thread's
            // own instruction latency bounds the tensor pipe (an MMA of this shape takes 128 clocks; a loop body of
            // fifty dependent scalar instructions per MMA took 415), so stage index, parities and operand
            // descriptors are carried incrementally and the K = 32 steps inside a stage are immediates.
            const int total_kb = my_tiles * p.num_kblocks;  // K-block and group counters run across tiles
            const uint64_t desc_stage0 = smem_desc(tiles);
            const int mpg = p.mmas_per_group;
            int st = 0, q_in_group = 0, group = 0;
            uint32_t full_parity = 0;
            bool ok = true;
            for (int kb = 0; kb < total_kb && ok; ++kb) {
                if (q_in_group == 0) GEMM_EV(1, group, 0, GEMM_CLK());
                if (!ptx::mbar_wait_bounded(&full_bar[st], full_parity, kSpin)) {
                    atomicExch(p.status, 300 + st); atomicExch(&failed_s, 1); ok = false; break;
                }
                tc_fence_after();
                if (q_in_group == 0) GEMM_EV(1, group, 1, GEMM_CLK());  // operands of the group's first K-block are there
                const uint64_t da = desc_stage0 + static_cast<uint64_t>((st * kStageBytes) >> 4);
                const uint64_t db = da + static_cast<uint64_t>((BM * BK) >> 4);
#pragma unroll
                for (int sub = 0; sub < 4; ++sub) {
                    const int as = group & (kAccStages - 1);
                    if (q_in_group == 0) {
                        if (group >= kAccStages) {
                            if (!ptx::mbar_wait_bounded(&acc_empty[as], ((group / kAccStages) - 1) & 1, kSpin)) {
                                atomicExch(p.status, 400 + as); atomicExch(&failed_s, 1); ok = false; break;
                            }
                            tc_fence_after();
                        }
                        GEMM_EV(1, group, 2, GEMM_CLK());  // the accumulator slice is free
                    }
                    // (a step of 32 bytes along K inside the 128-byte swizzled row: +2 in the descriptor's address field)
                    if constexpr (PAIR) mma_i8_pair(tmem_base + as * BN, da + 2 * sub, db + 2 * sub, kIdescPair, q_in_group != 0);
                    else mma_i8(tmem_base + as * BN, da + 2 * sub, db + 2 * sub, kIdesc, q_in_group != 0);
                    if (++q_in_group == mpg) {
                        if constexpr (PAIR) tc_commit_pair(&acc_full[as]); else
                        tc_commit(&acc_full[as]);                 // the K-group's sums are complete
                        GEMM_EV(1, group, 3, GEMM_CLK());  // the group's last MMA and its commit are issued
                        q_in_group = 0;
                        ++group;
                    }
                }
                if (!ok) break;
                // the stage may be refilled once these MMAs retire
                if constexpr (PAIR) tc_commit_pair(&empty_bar[st]); else tc_commit(&empty_bar[st]);
                if (++st == kStages) { st = 0; full_parity ^= 1u; }
            }
        }
        __syncwarp();
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;" ::: "memory");
        // ---------------- epilogue: 8 warps, thread <-> (token row, 128 columns) ----------------
        constexpr int HC = BN / (kEpiWarps / 4);  // columns per thread
        const int quad = warp & 3;               // the tensor-memory lane quadrant this warp may read
        const int half = (warp - 4) >> 2;        // which HC columns
        const int row = quad * 32 + lane;        // row inside the tile
        const int et = (warp - 4) * 32 + lane;   // 0..255: stages the weight scale of tile column et
        constexpr bool magic = MAGIC;            // |P| <= 128 * 128 * 256 = 2^22
        int jrun = 0;                            // running group counter over all the tiles of this CTA
        bool ok = true;
        // The first weight scales and the first activation scale of a tile are requested while the tile before it
        // is being stored (two L2 round trips that would otherwise sit between the tiles).
        float wpre[kWsGroups], xs_pre = 0.0f;
        const uint32_t acc_empty0 = PAIR ? map_to_rank(ptx::smem_u32(&acc_empty[0]), 0) : ptx::smem_u32(&acc_empty[0]);
        auto preload = [&](int tile) {
            const int pm = tile_m0(tile) + row, pn0 = (tile / p.tiles_m) * BN;
            const int pcol = min(pn0 + (et & (BN - 1)), a.N - 1);
#pragma unroll
            for (int q = 0; q < kWsGroups; ++q)
                wpre[q] = (et < BN && q < G) ? __half2float(a.w_scale[static_cast<size_t>(pcol) * G + q]) : 0.0f;
            xs_pre = a.Xs[static_cast<size_t>(pm < a.M ? pm : 0) * G];
        };
        if (walker < p.tiles_total) preload(walker);
        for (int tile = walker; tile < p.tiles_total && ok; tile += walkers) {
        const int m0 = tile_m0(tile), n0 = (tile / p.tiles_m) * BN;
        const int m = m0 + row;
        const bool m_ok = m < a.M;
        const float* xs_row = a.Xs + static_cast<size_t>(m_ok ? m : 0) * G;
        const int ncol = min(n0 + (et & (BN - 1)), a.N - 1);
        uint64_t acc2[HC / 2];
#pragma unroll
        for (int c = 0; c < HC / 2; ++c) acc2[c] = 0ull;
        // Weight scales are staged kWsGroups K-groups at a time (one block barrier per kWsGroups groups,
        // not per group); the activation scale of the next group is requested while this one is promoted.
        auto stage_ws = [&](int j0, int buf) {
#pragma unroll
            for (int q = 0; q < kWsGroups; ++q)
                if (et < BN && j0 + q < G) ws_s[buf][q][et] = __half2float(a.w_scale[static_cast<size_t>(ncol) * G + j0 + q]);
        };
#pragma unroll
        for (int q = 0; q < kWsGroups; ++q)
            if (et < BN && q < G) ws_s[0][q][et] = wpre[q];
        asm volatile("bar.sync 1, 256;" ::: "memory");
        float xs_next = xs_pre;
        for (int j = 0; j < G && ok; ++j, ++jrun) {
            const int as = jrun % kAccStages, buf = (j / kWsGroups) & 1, q = j % kWsGroups;
            const float xs = xs_next;
            if (j + 1 < G) xs_next = xs_row[j + 1];
            const uint64_t xs2 = pack2(xs, xs);
            if (q == 0 && j + kWsGroups < G) stage_ws(j + kWsGroups, buf ^ 1);  // lands long before it is read
            if (et == 0) GEMM_EV(2, jrun, 0, GEMM_CLK());
            if (!ptx::mbar_wait_bounded(&acc_full[as], (jrun / kAccStages) & 1, kSpin)) {
                atomicExch(p.status, 500 + as); atomicExch(&failed_s, 1); ok = false; break;
            }
            tc_fence_after();
            if (et == 0) GEMM_EV(2, jrun, 1, GEMM_CLK());
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + as * BN + half * HC;
            constexpr int CH = 32;  // columns per tensor-memory load
            uint32_t r[2][CH];
            if (GEMM_ABLATE(1)) {
                tc_fence_before();
                __syncwarp();
                if (et == 0) GEMM_EV(2, jrun, 2, GEMM_CLK());
                if (lane == 0) {
                    if (PAIR && crank != 0) mbar_arrive_cluster(acc_empty0 + as * static_cast<uint32_t>(sizeof(uint64_t)));
                    else ptx::mbar_arrive(&acc_empty[as]);
                }
            } else {
            tmem_ld32(taddr, r[0]);
#pragma unroll
            for (int ci = 0; ci < HC / CH; ++ci) {
                const int c0 = ci * CH;
                tmem_ld_wait();
                if (ci + 1 < HC / CH) {
                    tmem_ld32(taddr + c0 + CH, r[(ci + 1) & 1]);  // next chunk while this one is promoted
                } else {
                    // The group's last sums are in registers: this slice of tensor memory may be overwritten by group
                    // j + kAccStages while the last chunk is still being promoted.
                    tc_fence_before();
                    __syncwarp();
                    if (et == 0) GEMM_EV(2, jrun, 2, GEMM_CLK());
                    if (lane == 0) {
                        if constexpr (PAIR) {
                            if (crank == 0) ptx::mbar_arrive(&acc_empty[as]);
                            else mbar_arrive_cluster(acc_empty0 + as * static_cast<uint32_t>(sizeof(uint64_t)));
                        } else {
                            ptx::mbar_arrive(&acc_empty[as]);
                        }
                    }
                }
                const uint32_t (&rr)[CH] = r[ci & 1];
                if (GEMM_ABLATE(2)) {
                    uint32_t x = 0;
#pragma unroll
                    for (int c = 0; c < CH; ++c) x ^= rr[c];
                    acc2[c0 / 2] ^= x;
                    continue;
                }
#pragma unroll
                for (int c = 0; c < CH; c += 4) {
                    uint64_t w01, w23;
                    lds_pairs(&ws_s[buf][q][half * HC + c0 + c], w01, w23);
                    uint64_t f01, f23;
                    if constexpr (magic) {
                        f01 = ints_to_floats_magic(rr[c + 0], rr[c + 1]);
                        f23 = ints_to_floats_magic(rr[c + 2], rr[c + 3]);
                    } else {
                        f01 = pack2(static_cast<float>(static_cast<int>(rr[c + 0])), static_cast<float>(static_cast<int>(rr[c + 1])));
                        f23 = pack2(static_cast<float>(static_cast<int>(rr[c + 2])), static_cast<float>(static_cast<int>(rr[c + 3])));
                    }
                    acc2[(c0 + c) / 2] = fma2(mul2(f01, w01), xs2, acc2[(c0 + c) / 2]);
                    acc2[(c0 + c) / 2 + 1] = fma2(mul2(f23, w23), xs2, acc2[(c0 + c) / 2 + 1]);
                }
                if (a.dump && m_ok) {
#pragma unroll
                    for (int c = 0; c < CH; ++c)
                        if (n0 + half * HC + c0 + c < a.N)
                            a.dump[(static_cast<size_t>(m) * a.N + n0 + half * HC + c0 + c) * G + j] = static_cast<int>(rr[c]);
                }
            }
            }
            if (et == 0) GEMM_EV(2, jrun, 3, GEMM_CLK());
            if (q == kWsGroups - 1) asm volatile("bar.sync 1, 256;" ::: "memory");
        }
        if (tile + walkers < p.tiles_total) preload(tile + walkers);
        if constexpr (STAGED) {
            // ---- final store through shared memory and TMA ----
            auto accf = [&](int c) -> float { return (c & 1) ? hi2(acc2[c >> 1]) : lo2(acc2[c >> 1]); };
            // the TMA store of the tile before this one must have read the staging buffer
            if (et == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            asm volatile("bar.sync 1, 256;" ::: "memory");
            // chunk c16 (8 fp16 = 16 bytes) of row `row` inside a 64-column panel
            auto put = [&](int panel, int c16, const __half* o8) {
                const uint32_t addr = out_stage + panel * kOutPanelBytes + row * 128 + (((c16 ^ (row & 7)) & 7) << 4);
                const uint4 v = *reinterpret_cast<const uint4*>(o8);
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
            };
            if (a.epilogue == W8A8_EPI_SWIGLU) {
#pragma unroll
                for (int b = 0; b < HC / 32; ++b) {  // 32 columns -> 16 outputs = two chunks of panel `half`
                    __align__(16) __half o[16];
#pragma unroll
                    for (int hb = 0; hb < 2; ++hb)
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float g16 = __half2float(__float2half(accf(b * 32 + hb * 16 + i)));
                            const __half s16 = __float2half(g16 / (1.0f + expf(-g16)));
                            const float u16 = __half2float(__float2half(accf(b * 32 + hb * 16 + 8 + i)));
                            o[hb * 8 + i] = __float2half(__half2float(s16) * u16);
                        }
                    put(half, 2 * b, o);
                    put(half, 2 * b + 1, o + 8);
                }
            } else {
                const int nb = n0 + half * HC;
                const __half* rrow = (a.residual && m_ok) ? a.residual + static_cast<size_t>(m) * a.N + nb : nullptr;
#pragma unroll
                for (int b = 0; b < HC / 8; ++b) {  // 8 columns = one chunk
                    __align__(16) __half o[8];
                    __align__(16) __half rr[8];
                    if (a.epilogue == W8A8_EPI_RESIDUAL) {
                        if (rrow && nb + b * 8 + 8 <= a.N) {
                            *reinterpret_cast<uint4*>(rr) = *reinterpret_cast<const uint4*>(rrow + b * 8);
                        } else {
                            for (int i = 0; i < 8; ++i) rr[i] = (rrow && nb + b * 8 + i < a.N) ? rrow[b * 8 + i] : __float2half(0.f);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        __half y = __float2half(accf(b * 8 + i));
                        if (a.epilogue == W8A8_EPI_RESIDUAL) y = __float2half(__half2float(y) + __half2float(rr[i]));
                        o[i] = y;
                    }
                    put(half * (HC / 64) + b / 8, b & 7, o);
                }
            }
            // generic-proxy writes -> visible to the async proxy, then one thread hands the panels to TMA
            ptx::fence_proxy_async();
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (et == 0 && ok && m0 < a.M) {
                const int panels = a.epilogue == W8A8_EPI_SWIGLU ? BN / 128 : BN / 64;
                const int x0 = (a.epilogue == W8A8_EPI_SWIGLU ? n0 / 2 : n0) * 2;  // byte column of the tile in Y
                const int x_end = (a.epilogue == W8A8_EPI_SWIGLU ? a.N / 2 : a.N) * 2;
                for (int pnl = 0; pnl < panels; ++pnl)
                    if (x0 + pnl * 128 < x_end)  // (a box that starts inside the tensor is clipped at its edges by TMA)
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                 ::"l"(&map_y), "r"(out_stage + pnl * kOutPanelBytes), "r"(x0 + pnl * 128), "r"(m0) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        } else
        // ---- final store: fp16, optional residual add or SwiGLU, 16 bytes at a time ----
        if (ok && m_ok) {
            const int nb = n0 + half * HC;  // first column of this thread
            auto accf = [&](int c) -> float { return (c & 1) ? hi2(acc2[c >> 1]) : lo2(acc2[c >> 1]); };
            // A thread owns HC consecutive columns of one row, i.e. a contiguous run of the output: it is written
            // 32 bytes (one whole sector) per store where the row allows it, 16 bytes or element-wise otherwise.
            auto st32 = [](__half* dst, const __half* o16) {
                const uint4 lo = *reinterpret_cast<const uint4*>(o16), hi = *reinterpret_cast<const uint4*>(o16 + 8);
                asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(lo.x), "r"(lo.y), "r"(lo.z),
                             "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w) : "memory");
            };
            if (a.epilogue == W8A8_EPI_SWIGLU) {
                __half* yrow = a.Y + static_cast<size_t>(m) * (a.N / 2) + nb / 2;
                const bool wide = (a.N % 64) == 0 && (reinterpret_cast<uintptr_t>(a.Y) & 31u) == 0;
#pragma unroll
                for (int b = 0; b < HC / 32; ++b) {  // 32 columns -> 16 outputs
                    __align__(16) __half o[16];
#pragma unroll
                    for (int hb = 0; hb < 2; ++hb)
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float g16 = __half2float(__float2half(accf(b * 32 + hb * 16 + i)));
                            const __half s16 = __float2half(g16 / (1.0f + expf(-g16)));
                            const float u16 = __half2float(__float2half(accf(b * 32 + hb * 16 + 8 + i)));
                            o[hb * 8 + i] = __float2half(__half2float(s16) * u16);
                        }
                    if (wide && nb + b * 32 + 32 <= a.N) {
                        st32(yrow + b * 16, o);
                    } else {
                        if (nb + b * 32 + 16 <= a.N) *reinterpret_cast<uint4*>(yrow + b * 16) = *reinterpret_cast<const uint4*>(o);
                        if (nb + b * 32 + 32 <= a.N) *reinterpret_cast<uint4*>(yrow + b * 16 + 8) = *reinterpret_cast<const uint4*>(o + 8);
                    }
                }
            } else {
                __half* yrow = a.Y + static_cast<size_t>(m) * a.N + nb;
                const __half* rrow = a.residual ? a.residual + static_cast<size_t>(m) * a.N + nb : nullptr;
                const bool vec = (a.N % 8) == 0;
                const bool wide = (a.N % 16) == 0 && (reinterpret_cast<uintptr_t>(a.Y) & 31u) == 0;
#pragma unroll
                for (int b = 0; b < HC / 16; ++b) {  // 16 columns per step
                    if (nb + b * 16 >= a.N) break;
                    __align__(16) __half o[16];
                    __align__(16) __half rr[16];
                    const bool full = vec && nb + b * 16 + 16 <= a.N;
                    if (a.epilogue == W8A8_EPI_RESIDUAL) {
                        if (full) {
                            *reinterpret_cast<uint4*>(rr) = *reinterpret_cast<const uint4*>(rrow + b * 16);
                            *reinterpret_cast<uint4*>(rr + 8) = *reinterpret_cast<const uint4*>(rrow + b * 16 + 8);
                        } else {
                            for (int i = 0; i < 16; ++i) rr[i] = nb + b * 16 + i < a.N ? rrow[b * 16 + i] : __float2half(0.f);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        __half y = __float2half(accf(b * 16 + i));
                        if (a.epilogue == W8A8_EPI_RESIDUAL) y = __float2half(__half2float(y) + __half2float(rr[i]));
                        o[i] = y;
                    }
                    if (full && wide) {
                        st32(yrow + b * 16, o);
                    } else if (full) {
                        *reinterpret_cast<uint4*>(yrow + b * 16) = *reinterpret_cast<const uint4*>(o);
                        *reinterpret_cast<uint4*>(yrow + b * 16 + 8) = *reinterpret_cast<const uint4*>(o + 8);
                    } else {
                        for (int i = 0; i < 16; ++i)
                            if (nb + b * 16 + i < a.N) yrow[b * 16 + i] = o[i];
                    }
                }
            }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");  // nobody still reads this tile's weight scales
        }  // tiles
    }
    if constexpr (STAGED) {  // the last tile's store must have read shared memory before the CTA gives it up
        if (threadIdx.x == 128) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
    // ---- teardown: everyone meets, then the allocating warp frees the tensor memory ----
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // nothing of the peer still signals this CTA's barriers or uses its tensor memory
    if (warp == 1) {
        tc_fence_after();
        if constexpr (PAIR) tmem_dealloc_pair(tmem_base, 512); else
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace

bool gemm_supports(const LinearArgs& a) {
    if (a.M < 1 || !a.Xq || !a.Xs) return false;
    if (a.K % BK != 0 || a.g % 32 != 0 || a.K % a.g != 0) return false;
    if ((reinterpret_cast<uintptr_t>(a.W) | reinterpret_cast<uintptr_t>(a.Xq)) & 15u) return false;
    if (a.epilogue == W8A8_EPI_SWIGLU && (a.N % 16 != 0 || (reinterpret_cast<uintptr_t>(a.Y) & 15u))) return false;
    if (a.epilogue != W8A8_EPI_SWIGLU && a.N % 8 == 0 && (reinterpret_cast<uintptr_t>(a.Y) & 15u)) return false;
    if (a.residual && a.N % 8 == 0 && (reinterpret_cast<uintptr_t>(a.residual) & 15u)) return false;
    return true;
}

int launch_linear_gemm(const LinearArgs& a, int* device_status, cudaStream_t stream, int form) {
    if (!gemm_supports(a)) return fail(W8A8_ERR_UNSUPPORTED, "tcgen05 GEMM does not take this shape");
    CUtensorMap map_x, map_w;
    int rc = make_tensor_map_2d_u8(&map_x, a.Xq, static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.M),
                                   static_cast<uint64_t>(a.K), BK, BM, 1);
    if (rc) return rc;
    rc = make_tensor_map_2d_u8(&map_w, a.W, static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.N),
                               static_cast<uint64_t>(a.K), BK, BN, 1);
    if (rc) return rc;
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // CTA pairs (256-token tiles) once there are enough tokens to fill them and the groups are long enough for the
    // tensor pipe to matter: measured a few per cent faster at g = 256 and a few per cent slower at g = 64, where the
    // promote bounds the kernel and the pair only adds latency between the two CTAs' epilogues and the one issuer
    // (W8A8_GEMM_PAIR=0: never, =1: always).
    static const int pair_mode = [] {
        const char* v = std::getenv("W8A8_GEMM_PAIR");
        return v ? std::atoi(v) : -1;
    }();
    const bool pair = form >= 0 ? form != 0 : pair_mode >= 0 ? pair_mode != 0 : (a.M > BM && a.g >= 128);
    if (pair) {  // a CTA of a pair loads 128 of the tile's 256 weight rows per box
        rc = make_tensor_map_2d_u8(&map_w, a.W, static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.N),
                                   static_cast<uint64_t>(a.K), BK, BN / 2, 1);
        if (rc) return rc;
    }
    GemmParams p;
    p.a = a;
    p.status = device_status;
    p.mmas_per_group = a.g / 32;
    p.num_kblocks = a.K / BK;
    const int walk_m = pair ? 2 * BM : BM;
    p.tiles_m = (a.M + walk_m - 1) / walk_m;
    p.tiles_total = p.tiles_m * ((a.N + BN - 1) / BN);
    p.ablate = 0;
#ifdef W8A8_TRACE
    if (const char* v = std::getenv("W8A8_GEMM_ABLATE")) p.ablate = std::atoi(v);
#endif
    // The output through shared memory + TMA when its rows are 16-byte multiples (W8A8_GEMM_DIRECT_STORE=1: never).
    const int ycols = a.epilogue == W8A8_EPI_SWIGLU ? a.N / 2 : a.N;
    static const bool direct_only = [] {
        const char* v = std::getenv("W8A8_GEMM_DIRECT_STORE");
        return v && *v == '1';
    }();
    const bool staged = !direct_only && ycols % 8 == 0 && (reinterpret_cast<uintptr_t>(a.Y) & 15u) == 0;
    CUtensorMap map_y = map_x;  // (a valid map in either case; only the staged kernel reads it)
    if (staged) {
        // Y as rows of bytes; a box is 128 rows x 128 bytes (64 fp16 columns), 128-byte swizzle; stores clip at the
        // tensor's edges, so ragged last tiles need no care
        rc = make_tensor_map_2d_u8(&map_y, a.Y, static_cast<uint64_t>(ycols) * 2, static_cast<uint64_t>(a.M),
                                   static_cast<uint64_t>(ycols) * 2, 128, BM, 1);
        if (rc) return rc;
    }
    const int stages = pair ? (staged ? kStagesPairStaged : kStagesPairDirect) : (staged ? kStagesStaged : kStagesDirect);
    const size_t smem = static_cast<size_t>(stages) * (pair ? kStageBytesPair : kStageBytes) + (staged ? kOutStageBytes : 0) + 1024;
    const bool magic = a.g <= 256;
    using Kernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const GemmParams);
    static const Kernel table[8] = {
        gemm_i8_kernel<false, false, false>, gemm_i8_kernel<true, false, false>, gemm_i8_kernel<false, true, false>,
        gemm_i8_kernel<true, true, false>,   gemm_i8_kernel<false, false, true>, gemm_i8_kernel<true, false, true>,
        gemm_i8_kernel<false, true, true>,   gemm_i8_kernel<true, true, true>};
    Kernel kernel = table[(magic ? 1 : 0) | (staged ? 2 : 0) | (pair ? 4 : 0)];
    {
        // The attribute is per device and this library serves several devices of one process: set it on every
        // launch (a host-side table write) rather than remember it per process.
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        // setmaxnreg moves registers between the warpgroups; the sums balance only for the register count the
        // kernel was compiled to (kLaunchRegs per thread). An unbalanced sum blocks for ever in setmaxnreg.inc,
        // a wait nothing bounds, so a build that came out differently is refused here.
        cudaFuncAttributes fa;
        e = cudaFuncGetAttributes(&fa, kernel);
        if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "cudaFuncGetAttributes: %s", cudaGetErrorString(e));
        if (fa.numRegs != kLaunchRegs)
            return fail(W8A8_ERR_UNSUPPORTED,
                        "gemm_i8_kernel was compiled to %d registers per thread, its setmaxnreg balance needs %d",
                        fa.numRegs, kLaunchRegs);
    }
    cudaLaunchConfig_t cfg = {};
    // persistent: one CTA (or CTA pair) per SM (pair of SMs) walks its tiles (m fastest, so that concurrent CTAs
    // share weight tiles in L2)
    const int walkers_max = pair ? sms / 2 : sms;
    const int walkers = p.tiles_total < walkers_max ? p.tiles_total : walkers_max;
    cfg.gridDim = dim3(pair ? 2 * walkers : walkers, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pair) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 2;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (pdl_enabled(kPdlLinear)) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, map_x, map_w, map_y, p);
    if (e != cudaSuccess) return fail(W8A8_ERR_CUDA, "gemm launch: %s", cudaGetErrorString(e));
    return W8A8_OK;
}

}  // namespace w8a8

#ifdef W8A8_TRACE
extern "C" __attribute__((visibility("default"))) int w8a8_trace_read_gemm(void* out, int cap_bytes) {
    const int bytes = static_cast<int>(sizeof(unsigned long long)) * 3 * w8a8::kGemmEvents * 4;
    if (cap_bytes < bytes || cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(out, w8a8::g_gemm_ev, bytes) != cudaSuccess) return -1;
    void* dev = nullptr;
    if (cudaGetSymbolAddress(&dev, w8a8::g_gemm_ev) == cudaSuccess) cudaMemset(dev, 0, bytes);
    return bytes;
}
#endif
