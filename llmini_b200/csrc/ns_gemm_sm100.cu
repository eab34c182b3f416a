// Newton-Schulz GEMMs for sm_100a: D[M][N] = A * B^T on the 5th-generation tensor cores.
//
//   tcgen05.mma (kind::f16, BF16 or F16 operands, FP32 accumulators in TMEM), operands staged
//   in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), mbarrier pipeline,
//   warp-specialised persistent CTAs walking a tile list that spans every matrix of the plan.
//
// One kernel, three uses per iteration (crates/cuda-kernels/src/gpt/optimizer/muon/polar/
// fused.rs:64-92 in the reference):
//   Gram   G = X X^T                     (reference: tiles/symmetric.rs:28-40)
//   Poly   Q = c G G + b G + a I         (reference: tiles/symmetric.rs:42-65, store/plain.rs:175-178)
//   Apply  X' = Q X                      (reference: tiles.rs:14-38)
// Operands are read in their storage orientation: an operand whose reduction dimension is
// the slow one is described to the tensor core as MN-major, so no transpose is ever
// materialised.  16-bit results leave through a shared-memory slab and coalesced stores; the FP32 Gram
// tile that the polynomial epilogue needs is kept in a private fragment-ordered scratch so
// both sides access it fully coalesced.
//
// Two tile configurations:
//   PAIR  : a cluster of two CTAs computes a 256 x 256 tile with cta_group::2 MMAs.  Each
//           CTA stages its own 128 rows of A and half (128 rows) of B, so a k-block costs
//           32 KB of loads per SM instead of 48 KB: the kernel is bound by the L2-to-SM
//           path, and this raises FLOPs per loaded byte by 1.5x.  No multicast load is used.
//   single: one CTA computes 128 x BN (BN = 128 or 256).
//
// Three ways to launch the loop (the template parameter CHAINED separates the first from the other two):
//   per phase : one launch per GEMM flavour and iteration, tiles dealt round-robin, launches chained with
//               programmatic dependent launch.  The default.
//   chained   : one persistent grid over a work list of every tile of every iteration; CTAs draw tiles with an
//               atomic ticket and a per-matrix progress count orders a tile after the tiles it reads from.
//   fused     : a ticketed launch whose entries are a Gram tile AND the polynomial tile of the same position:
//               the FP32 Gram accumulator stays in tensor memory between the two.
//
// Every mbarrier wait, ring read and dependency wait is bounded: on expiry the CTA raises a status word, drains
// and frees its TMEM before returning.
#include <cuda.h>

#include "common.cuh"
#include "internal.h"

namespace b2 {

namespace {

constexpr int kBoxBytes = 64 * 128;          // 64 rows x 128 bytes
constexpr int kABytes = 2 * kBoxBytes;       // 128 x 64 16-bit operand tile
constexpr int kSlabBytes = 32 * 128;         // per-warp store staging: 32 rows x 128 bytes
constexpr int kSmemLimit = 227 * 1024;
constexpr uint32_t kSpinLimit = 1u << 24;    // hard cap on polls, whatever the timer says
constexpr uint64_t kWaitLimitNs = 2000000000ull;

template <int BN, bool PAIR>
struct Cfg {
    static constexpr int kBRows = PAIR ? 128 : BN;   // rows of B this CTA stages per k-block
    static constexpr int kBBytes = (kBRows / 64) * kBoxBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;
    // warp 0: TMA producer, warp 1: MMA issuer, then four epilogue warps (one per TMEM lane
    // quarter) for every 64 columns of the tile
    static constexpr int kEpiWarps = 4 * (BN / 64);
    static constexpr int kThreads = 32 * (2 + kEpiWarps);
    static constexpr int kStagingBytes = kEpiWarps * kSlabBytes;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kBarrierBytes = 512;   // mbarriers, flags, and the tile ring of the chained launch
    static constexpr int kStages = (kSmemLimit - kStagingBytes - kBarrierBytes - 1024) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
    static constexpr int kTileM = PAIR ? 256 : 128;  // rows of the (cluster) tile
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
// shared::cluster address of the same offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// arrive on a barrier given by its shared::cluster address (own or peer CTA)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Non-blocking probe of a barrier phase.  (mbarrier.try_wait may suspend the thread for a system-dependent time,
// measured here at about 5 us, before it reports that the phase is not complete; that is right for a wait, not
// for a probe.)
__device__ __forceinline__ uint32_t mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait (about two seconds of wall clock).  Returns false when the limit ran out or
// another role of this CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag) {
#pragma unroll 1
    for (int it = 0; it < 128; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = global_timer_ns();
#pragma unroll 1
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_timer_ns() - start > kWaitLimitNs) break;
        __nanosleep(it >= 1024 ? 256 : 32);
    }
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// orders this thread's generic-proxy accesses against its async-proxy ones (TMA loads and stores)
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Chained launch: words shared by every CTA.  All zero between launches; the last CTA to leave clears them.
struct ChainSync {
    uint32_t abort;      // a bounded wait ran out somewhere: everybody leaves
    uint32_t exited;
    uint32_t ticket;     // next unclaimed entry of the work list
    uint32_t reserved;
    uint32_t progress[1];  // per slot: epilogue warps that have finished a tile of the slot, over all phases
};
// Bounded wait until `*counter >= need`.  Returns false when the limit ran out or the launch is aborting.
//
// How a tile's outputs reach the CTA that reads them.  Every lane of the writer's epilogue warp orders its
// stores before what follows (__threadfence), the warp converges, and one lane raises the matrix's progress
// count with an atomic.
// The reader polls the count with relaxed loads that bypass L1; once it is high enough it reads it once more
// with acquire semantics and issues fence.proxy.async before its first TMA copy, which is what the PTX memory
// model asks for between a generic-proxy flag and async-proxy accesses.  Both fences were measured against a
// build without them: no difference beyond run-to-run noise.
__device__ __forceinline__ bool chain_wait(const uint32_t *counter, uint32_t need, uint32_t *launch_abort,
                                           volatile uint32_t *abort_flag) {
    if (ld_relaxed_gpu(counter) >= need) return true;
    const uint64_t start = global_timer_ns();
#pragma unroll 1
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        if (ld_relaxed_gpu(counter) >= need) return true;
        if (*abort_flag || ld_relaxed_gpu(launch_abort) != 0u) break;
        if (global_timer_ns() - start > kWaitLimitNs) break;
        __nanosleep(it >= 64 ? 128 : 20);
    }
    *abort_flag = 1;
    atomicExch(launch_abort, 1u);
    return false;
}

// Chained launch: which tile a CTA (pair) works on next is decided at run time (an atomic ticket over the work
// list, claimed by the leader's producer thread), so the roles of the CTA, and the peer CTA of a pair, learn it
// through a small ring in shared memory: entry k holds (k + 1) << 32 | tile for the k-th tile of this CTA.  No
// role is ever more than stages + 2 tiles behind the producer, far less than the ring's length.
constexpr uint32_t kTileRing = 16;
constexpr uint32_t kNoTile = 0xffffffffu;
__device__ __forceinline__ void ring_put_local(volatile uint64_t *ring, uint32_t seq, uint32_t tile) {
    ring[seq % kTileRing] = ((uint64_t)(seq + 1u) << 32) | tile;
}
__device__ __forceinline__ void ring_put_remote(uint32_t ring_cluster_addr, uint32_t seq, uint32_t tile) {
    const uint64_t v = ((uint64_t)(seq + 1u) << 32) | tile;
    asm volatile("st.volatile.shared::cluster.u64 [%0], %1;" ::"r"(ring_cluster_addr + 8u * (seq % kTileRing)), "l"(v)
                 : "memory");
}
// Bounded: gives kNoTile when the CTA is aborting or nothing arrives within the wait limit.
__device__ __forceinline__ uint32_t ring_get(volatile uint64_t *ring, uint32_t seq, volatile uint32_t *abort_flag) {
    const uint64_t want = (uint64_t)(seq + 1u);
    uint64_t v = ring[seq % kTileRing];
    if ((v >> 32) == want) return (uint32_t)v;
    const uint64_t start = global_timer_ns();
#pragma unroll 1
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        v = ring[seq % kTileRing];
        if ((v >> 32) == want) return (uint32_t)v;
        if (*abort_flag) return kNoTile;
        if (global_timer_ns() - start > kWaitLimitNs) break;
        __nanosleep(20);
    }
    *abort_flag = 1;
    return kNoTile;
}

template <bool PAIR>
__device__ __forceinline__ void tma_load_2d(uint32_t dst, uint64_t map, uint32_t bar, int x, int y) {
    if (PAIR)
        asm volatile(
            "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
            ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
            : "memory");
    else
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
            ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
            : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Arrive on `bar` once every MMA issued so far has retired.  PAIR: the arrival is delivered
// to the barrier at this offset in both CTAs of the pair.
template <bool PAIR>
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    if (PAIR)
        asm volatile(
            "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
            ::"r"(bar), "h"((uint16_t)3)
            : "memory");
    else
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                     : "memory");
}
template <bool PAIR>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
    if (PAIR)
        asm volatile(
            "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p; }"
            ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
            ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t *r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t *r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (sm_100).
//   K-major operand  (rows = M/N index, 128 bytes of K per row): 8-row groups are 1024 bytes
//   apart (stride byte offset); the leading byte offset is unused.
//   MN-major operand (rows = K index, 128 bytes = 64 M/N elements per row): 8-row groups of K
//   are 1024 bytes apart (stride), 64-element groups of M/N are one 64 x 64 box (8192 bytes)
//   apart (leading).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor for kind::f16: FP32 accumulate, A/B format F16 (0) or BF16 (1),
// per-operand major bit, N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ uint32_t instr_desc(int m, int n, int f16, uint32_t a_mn, uint32_t b_mn) {
    uint32_t fmt = f16 ? 0u : 1u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn << 15) | (b_mn << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// What one role needs to know about the tile it works on.  Plain launch: one GEMM flavour for the whole grid
// (epilogue, coefficients and scaling are launch arguments).  Chained launch: every entry of the list carries
// its own flavour, iteration and the progress count of its matrix that must be reached before its operands
// may be read.
struct TileWork {
    uint32_t problem, tile_m, tile_n, mirror, epilogue, slot, need, scale_pow, iter;
    uint32_t problem2, need2;   // second part of a kEpiGramPoly entry
};
// A work-list entry runs as one GEMM, or (kEpiGramPoly) as two on the same CTA (pair): part 0 the Gram tile,
// whose accumulator stays in tensor memory, part 1 the polynomial tile that consumes it.
struct TilePart {
    uint32_t problem, epilogue, need;
};
__device__ __forceinline__ uint32_t tile_parts(const TileWork &w) { return w.epilogue == kEpiGramPoly ? 2u : 1u; }
__device__ __forceinline__ TilePart tile_part(const TileWork &w, uint32_t part) {
    TilePart p;
    if (w.epilogue != kEpiGramPoly) {
        p.problem = w.problem; p.epilogue = w.epilogue; p.need = w.need;
    } else if (part == 0u) {
        p.problem = w.problem; p.epilogue = kEpiGramHold; p.need = w.need;
    } else {
        p.problem = w.problem2; p.epilogue = kEpiPolyFused; p.need = w.need2;
    }
    return p;
}
template <bool CHAINED>
__device__ __forceinline__ TileWork tile_work(const void *tiles, uint32_t t, uint32_t epilogue, uint32_t scale_pow) {
    TileWork w;
    w.problem2 = 0;
    w.need2 = 0;
    if (CHAINED) {
        const uint4 c = __ldg(reinterpret_cast<const uint4 *>(tiles) + 2 * (size_t)t);
        w.problem = c.x;
        w.tile_m = c.y & 0xffffu;
        w.tile_n = c.y >> 16;
        w.slot = c.z & 0xffffu;
        w.epilogue = (c.z >> 16) & 0xffu;
        w.mirror = (c.z >> 24) & 1u;
        w.scale_pow = (c.z >> 25) & 3u;
        w.iter = (c.z >> 27) & 31u;
        w.need = c.w;
        if (w.epilogue == kEpiGramPoly) {
            const uint4 d = __ldg(reinterpret_cast<const uint4 *>(tiles) + 2 * (size_t)t + 1);
            w.problem2 = d.x;
            w.need2 = d.y;
        }
    } else {
        const GemmTile tl = reinterpret_cast<const GemmTile *>(tiles)[t];
        w.problem = tl.problem;
        w.tile_m = tl.tile_m;
        w.tile_n = tl.tile_n;
        w.mirror = tl.reserved;
        w.epilogue = epilogue;
        w.slot = tl.problem;
        w.need = 0;
        w.scale_pow = scale_pow;
        w.iter = 0;
    }
    return w;
}

template <int BN, bool PAIR, bool CHAINED>
__global__ void __launch_bounds__((Cfg<BN, PAIR>::kThreads), 1)
k_ns_gemm(const GemmProblem *__restrict__ problems, const void *__restrict__ tiles,
          uint32_t tile_count, uint32_t epilogue_arg, int f16, GemmCoefficients coef,
          const float *__restrict__ slot_scale, uint32_t scale_pow_arg, uint32_t *status, ChainSync *sync,
          uint32_t slot_count, uint32_t debug_flags) {
    using C = Cfg<BN, PAIR>;
#ifdef B2_MEASURE
    const bool dbg_no_store = debug_flags & 1u;   // drop every epilogue store
    const bool dbg_no_global = debug_flags & 8u;  // stage in shared memory but issue no global store
#else
    constexpr bool dbg_no_store = false, dbg_no_global = false;
    (void)debug_flags;
#endif
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *stage_base = smem;
    uint8_t *staging = smem + C::kStages * C::kStageBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(staging + C::kStagingBytes);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * C::kStages + 4);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    // chained: one more than the index of the last tile whose dependency wait this CTA's producer has passed
    volatile uint32_t *passed_tile = tmem_slot + 2;
    volatile uint64_t *tile_ring = reinterpret_cast<volatile uint64_t *>(reinterpret_cast<uint8_t *>(bars) + 256);
    static_assert((2 * C::kStages + 4) * 8 + 16 <= 256 && 256 + kTileRing * 8 <= C::kBarrierBytes, "barrier region layout");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_cta_rank() : 0u;       // 0 = leader of the pair
    const uint32_t first_tile = PAIR ? blockIdx.x / 2 : blockIdx.x;
    const uint32_t tile_stride = PAIR ? gridDim.x / 2 : gridDim.x;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (C::kStages + s); };
    auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * C::kStages + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * C::kStages + 2 + a); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), PAIR ? 2 * C::kEpiWarps : C::kEpiWarps);
        }
        *abort_flag = 0;
        *passed_tile = 0;
        for (uint32_t k = 0; k < kTileRing; ++k) tile_ring[k] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                         "r"((uint32_t)C::kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                         "r"((uint32_t)C::kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch: the next launch of the stream may start its own prologue on
    // SMs this grid has left; nothing above reads what the previous launch wrote, everything
    // below may, so the wait for that launch (a no-op without the launch attribute) sits here.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            // Plain launch: tile first_tile + k * tile_stride.  Chained launch: the leader claims list entries in
            // order with an atomic ticket (a tile only ever waits for tiles with smaller tickets, which running
            // CTAs hold, so the launch makes progress however many CTAs are resident; the CTAs stay within one
            // wave of each other in the list, which keeps a matrix's operands in L2 while its tiles are worked
            // on; and a slower SM simply takes fewer tiles).  The ticket for the tile after next is claimed, and
            // the next tile's description and progress count fetched, while this tile's copies are issued.
            uint32_t seq = 0, t = first_tile, t_next = kNoTile;
            const bool claims = CHAINED && (!PAIR || rank == 0);
            // A list with fused Gram + polynomial entries: their second part waits for tiles with larger tickets, so
            // a CTA must not sit on a ticket it has not started.  The next ticket is then drawn only once the last
            // wait of the current tile has passed, and looked at after the tile's copies have been issued.
            const bool fused_list = CHAINED && epilogue_arg != 0u;
            const uint32_t peer_ring = (CHAINED && PAIR) ? map_to_cta(smem_u32(const_cast<uint64_t *>(tile_ring)), 1) : 0u;
            auto announce = [&](uint32_t tile) {   // leader: tell this CTA's roles (and the peer CTA) the seq-th tile
                ring_put_local(tile_ring, seq, tile);
                if (PAIR) ring_put_remote(peer_ring, seq, tile);
            };
            if (CHAINED) {
                if (claims) {
                    t = atomicAdd(&sync->ticket, 1u);
                    announce(t);
                    if (!fused_list && t < tile_count) t_next = atomicAdd(&sync->ticket, 1u);
                } else {
                    t = ring_get(tile_ring, seq, abort_flag);
                }
            }
            TileWork next = {};
            uint32_t next_seen = 0;
            auto describe_next = [&]() {
                if (t < tile_count) {
                    next = tile_work<CHAINED>(tiles, t, epilogue_arg, scale_pow_arg);
                    if (CHAINED && next.need != 0u) next_seen = ld_relaxed_gpu(&sync->progress[next.slot]);
                }
            };
            describe_next();
            while (ok && t < tile_count) {
                const TileWork tl = next;
                const uint32_t seen = next_seen;
                const uint32_t t_now = t;
                const uint32_t parts = CHAINED ? tile_parts(tl) : 1u;
                // the tile after this one
                if (!CHAINED) {
                    t += tile_stride;
                    describe_next();
                } else if (!fused_list) {
                    if (claims) {
                        t = t_next;
                        ++seq;
                        announce(t);
                        if (t < tile_count) t_next = atomicAdd(&sync->ticket, 1u);
                    } else {
                        ++seq;
                        t = ring_get(tile_ring, seq, abort_flag);
                    }
                    describe_next();
                }
                uint32_t drawn = kNoTile;
                for (uint32_t part = 0; ok && part < parts; ++part) {
                    TilePart tp;
                    if (CHAINED) {
                        tp = tile_part(tl, part);
                    } else {
                        tp.problem = tl.problem; tp.epilogue = tl.epilogue; tp.need = 0u;
                    }
                    const GemmProblem *p = problems + tp.problem;
                    const uint64_t map_a = p->map_a, map_b = p->map_b;
                    const uint32_t a_mn = p->a_mn_major, b_mn = p->b_mn_major, K = p->K;
                    const int m0 = tl.tile_m * C::kTileM + (int)rank * 128;
                    const int n0 = tl.tile_n * BN + (PAIR ? (int)rank * 128 : 0);
                    const int num_kb = (int)((K + kGemmBlockK - 1) / kGemmBlockK);
                    // A diagonal tile of X X^T or G G: this CTA's 128 rows of B are its 128 rows of A, in
                    // the same shared-memory layout.  They are loaded once and the MMA reads them twice.
                    const bool shared_operand = PAIR && tl.tile_m == tl.tile_n && map_a == map_b && a_mn == b_mn;
                    if (CHAINED && tp.need != 0u) {
                        // the operands are the outputs of the matrix's previous phase: every tile of that phase
                        // has been stored and published before the first copy is issued
                        if ((part != 0u || seen < tp.need) &&
                            !chain_wait(&sync->progress[tl.slot], tp.need, &sync->abort, abort_flag)) { ok = false; break; }
                        (void)ld_acquire_gpu(&sync->progress[tl.slot]);
                        fence_proxy_async_all();
                    }
                    if (CHAINED && part == 0u) *passed_tile = t_now + 1u;
                    if (fused_list && claims && part + 1u == parts) drawn = atomicAdd(&sync->ticket, 1u);
                    const uint32_t stage_tx = shared_operand ? 2u * (uint32_t)kABytes
                                                             : (uint32_t)C::kStageBytes * (PAIR ? 2u : 1u);
                    for (int kb = 0; kb < num_kb; ++kb) {
                        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                        // PAIR: both CTAs' copies complete on the leader's barrier, which expects
                        // the bytes of both
                        const uint32_t fb = PAIR ? map_to_cta(full_bar(stage), 0) : full_bar(stage);
                        if (!PAIR || rank == 0) mbar_expect_tx(full_bar(stage), stage_tx);
                        const uint32_t sa = smem_u32(stage_base + stage * C::kStageBytes);
                        const uint32_t sb = sa + kABytes;
                        const int k0 = kb * kGemmBlockK;
                        if (a_mn) {  // 64 x 64 boxes: x = M index, y = K index
                            tma_load_2d<PAIR>(sa, map_a, fb, m0, k0);
                            tma_load_2d<PAIR>(sa + kBoxBytes, map_a, fb, m0 + 64, k0);
                        } else {     // one 64 (K) x 128 (rows) box
                            tma_load_2d<PAIR>(sa, map_a, fb, k0, m0);
                        }
#pragma unroll
                        for (int j = 0; j < C::kBRows / 128; ++j) {
                            if (shared_operand) break;
                            if (b_mn) {
                                tma_load_2d<PAIR>(sb + (2 * j) * kBoxBytes, map_b, fb, n0 + 128 * j, k0);
                                tma_load_2d<PAIR>(sb + (2 * j + 1) * kBoxBytes, map_b, fb, n0 + 128 * j + 64, k0);
                            } else {
                                tma_load_2d<PAIR>(sb + (2 * j) * kBoxBytes, map_b, fb, k0, n0 + 128 * j);
                            }
                        }
                        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                    }
                }
                if (fused_list && ok) {
                    ++seq;
                    if (claims) {
                        t = drawn;
                        announce(t);
                    } else {
                        t = ring_get(tile_ring, seq, abort_flag);
                    }
                    describe_next();
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && rank == 0) {
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            uint32_t seq = 0;
            for (uint32_t t = CHAINED ? ring_get(tile_ring, 0u, abort_flag) : first_tile; ok && t < tile_count;
                 t = CHAINED ? ring_get(tile_ring, ++seq, abort_flag) : t + tile_stride) {
                const TileWork tl = tile_work<CHAINED>(tiles, t, epilogue_arg, scale_pow_arg);
                const uint32_t parts = CHAINED ? tile_parts(tl) : 1u;
                for (uint32_t part = 0; ok && part < parts; ++part) {
                    const GemmProblem *p = problems + (CHAINED ? tile_part(tl, part).problem : tl.problem);
                    const uint32_t a_mn = p->a_mn_major, b_mn = p->b_mn_major, K = p->K;
                    const int num_kb = (int)((K + kGemmBlockK - 1) / kGemmBlockK);
                    const uint32_t idesc = instr_desc(C::kTileM, BN, f16, a_mn, b_mn);
                    const bool shared_operand = PAIR && tl.tile_m == tl.tile_n && p->map_a == p->map_b && a_mn == b_mn;
                    if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + acc * BN;
                    for (int kb = 0; kb < num_kb; ++kb) {
                        if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t sa = smem_u32(stage_base + stage * C::kStageBytes);
                        const uint32_t sb = shared_operand ? sa : sa + kABytes;
#pragma unroll
                        for (int k = 0; k < kGemmBlockK / 16; ++k) {
                            const uint64_t ad = a_mn ? smem_desc(sa + k * 2048, kBoxBytes, 1024)
                                                     : smem_desc(sa + k * 32, 16, 1024);
                            const uint64_t bd = b_mn ? smem_desc(sb + k * 2048, kBoxBytes, 1024)
                                                     : smem_desc(sb + k * 32, 16, 1024);
                            tc_mma<PAIR>(d_tmem, ad, bd, idesc, (uint32_t)((kb | k) != 0));
                        }
                        tc_commit<PAIR>(empty_bar(stage));
                        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                    }
                    if (!ok) break;
                    tc_commit<PAIR>(tfull_bar(acc));
                    acc ^= 1u;
                    if (acc == 0) acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        // Warp w may read TMEM lanes 32 (w % 4) .. +31; the four warps of a lane quarter each take
        // one 64-column chunk of the tile, so an accumulator buffer is free again after ONE chunk
        // has been read and a tile's epilogue takes a quarter of the time it would on one warp.
        const int q = warp & 3;
        const int chunk = (warp - 2) >> 2;
        const int c0 = chunk * 64;
        // Results leave through a per-warp 4 KB slab in shared memory and plain 128-bit global stores: the warp
        // writes its 32 rows into the slab (one row per lane, 16-byte chunks XOR-swizzled by the row so that the
        // fill and the copy-out are both conflict-free), then copies it out with eight lanes per row, so every
        // store instruction writes whole 128-byte lines.  Plain stores need no bulk-group wait before the slab
        // is refilled or the launch ends, and a fence orders them before the progress count of a chained launch.
        uint8_t *slab = staging + (size_t)(warp - 2) * kSlabBytes;
        // 32 rows x 128 bytes, swizzled -> row-major tensor; rows >= row_limit and bytes >= byte_limit are dropped
        auto slab_to_global = [&](uint8_t *base, size_t pitch_bytes, int row0, int row_limit, int byte0, int byte_limit) {
#pragma unroll 2
            for (int i = 0; i < 8; ++i) {
                const int r = 4 * i + (lane >> 3), c = lane & 7;
                const uint4 w = *reinterpret_cast<const uint4 *>(slab + r * 128 + ((c ^ (r & 7)) << 4));
                const int gr = row0 + r, gb = byte0 + 16 * c;
                if (gr < row_limit && gb < byte_limit)
                    *reinterpret_cast<uint4 *>(base + (size_t)gr * pitch_bytes + gb) = w;
            }
        };
        // 64 rows x 64 bytes, plain row-major (the transposed block of a symmetric output)
        auto slab_t_to_global = [&](uint8_t *base, size_t pitch_bytes, int row0, int row_limit, int byte0, int byte_limit) {
#pragma unroll 2
            for (int i = 0; i < 8; ++i) {
                const int r = 8 * i + (lane >> 2), c = lane & 3;
                const uint4 w = *reinterpret_cast<const uint4 *>(slab + r * 64 + 16 * c);
                const int gr = row0 + r, gb = byte0 + 16 * c;
                if (gr < row_limit && gb < byte_limit)
                    *reinterpret_cast<uint4 *>(base + (size_t)gr * pitch_bytes + gb) = w;
            }
        };
        const uint32_t tempty_leader0 = PAIR ? map_to_cta(tempty_bar(0), 0) : tempty_bar(0);
        uint32_t acc = 0, acc_phase = 0;
        // Chained launch: a finished tile is published to the other CTAs by raising its matrix's progress count
        // once this warp's stores are ordered before it (every lane fences its own).  The fence is put off until
        // the next tile's accumulator has been read (the stores then had that long to land) unless the next
        // accumulator is not ready yet, in which case it is done first: a warp never blocks on other CTAs with a
        // count unpublished.
        constexpr uint32_t kNoSlot = 0xffffffffu;
        uint32_t unpublished = kNoSlot;
        auto publish = [&]() {
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(&sync->progress[unpublished], 1u);
            unpublished = kNoSlot;
        };
        uint32_t seq = 0;
        bool alive = true;
        for (uint32_t t = CHAINED ? ring_get(tile_ring, 0u, abort_flag) : first_tile; alive && t < tile_count;
             t = CHAINED ? ring_get(tile_ring, ++seq, abort_flag) : t + tile_stride) {
            const TileWork tl = tile_work<CHAINED>(tiles, t, epilogue_arg, scale_pow_arg);
            // the iteration's coefficient triple, picked without indexing the argument block by a register
            float ca = coef.v[0], cb = coef.v[1], cc = coef.v[2];
            if (CHAINED) {
#pragma unroll
                for (uint32_t i = 1; i < kMaxChainIterations; ++i)
                    if (tl.iter == i) { ca = coef.v[3 * i]; cb = coef.v[3 * i + 1]; cc = coef.v[3 * i + 2]; }
            }
            const uint32_t parts = CHAINED ? tile_parts(tl) : 1u;
#pragma unroll 1
            for (uint32_t part = 0; part < parts; ++part) {
            const uint32_t epilogue = CHAINED ? tile_part(tl, part).epilogue : tl.epilogue;
            const GemmProblem *p = problems + (CHAINED ? tile_part(tl, part).problem : tl.problem);
            const bool hold = CHAINED && epilogue == kEpiGramHold;    // the accumulator stays for the next part
            const bool fused = CHAINED && epilogue == kEpiPolyFused;  // combines with the held accumulator
            const uint32_t M = p->M, N = p->N;
            uint8_t *out16 = reinterpret_cast<uint8_t *>(p->out16), *out32 = reinterpret_cast<uint8_t *>(p->out32);
            const size_t pitch16 = (size_t)p->pitch16 * 2, pitch32 = (size_t)p->pitch32 * 4;
            // symmetric outputs (Gram, Poly): tiles below the diagonal are not computed; the tile
            // above writes them as its transpose (reference: tiles/symmetric.rs:76-92)
            const bool mirror = tl.mirror != 0;
            const float4 *frag = reinterpret_cast<const float4 *>(p->frag32);
            // fragment scratch is indexed by 128-row sub-tiles
            const uint32_t sub_m = PAIR ? (uint32_t)tl.tile_m * 2 + rank : tl.tile_m;
            const uint32_t tile_lin = sub_m * p->tiles_n + tl.tile_n;
            const int m0 = tl.tile_m * C::kTileM + (int)rank * 128, n0 = tl.tile_n * BN;
            const int row_in_tile = 32 * q + lane;
            const int grow = m0 + row_in_tile;
            const int slab_row0 = m0 + 32 * q;
            // fragment order: [128-row sub-tile][32-column unit][float4 index][row]
            const size_t unit0 = ((size_t)tile_lin * (BN / 32) + (size_t)(c0 / 32)) * 8;

            // The polynomial epilogue needs the FP32 Gram tile: fetch the first 32 columns before
            // the accumulator is ready so the latency hides behind the MMAs.
            float4 g[8];
            // chained: the Gram tile may be read early only if the matrix's Gram phase is already complete
            bool g_fetched = epilogue == kEpiPoly && !dbg_no_store;
            if (CHAINED && g_fetched) g_fetched = *passed_tile > t;   // this CTA's producer has seen the phase complete
            if (g_fetched) {
#pragma unroll
                for (int j = 0; j < 8; ++j) g[j] = __ldcg(frag + (unit0 + j) * kGemmBlockM + row_in_tile);
            }
            if (CHAINED && unpublished != kNoSlot && !mbar_test(tfull_bar(acc), acc_phase)) publish();

            bool ready = mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
            ready = __all_sync(0xffffffffu, ready);
            if (!ready) { alive = false; break; }
            tc_fence_after();
            if (CHAINED && epilogue == kEpiPoly && !dbg_no_store && !g_fetched) {
                // the accumulator is complete, so the producer has seen the Gram phase complete
#pragma unroll
                for (int j = 0; j < 8; ++j) g[j] = __ldcg(frag + (unit0 + j) * kGemmBlockM + row_in_tile);
            }
            const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + acc * BN + c0;
            // fused: the Gram accumulator of this tile sits in the other buffer
            const uint32_t held_taddr = tmem_base + ((uint32_t)(32 * q) << 16) + (acc ^ 1u) * BN + c0;
            const uint32_t tempty = tempty_leader0 + 8u * acc;
            const uint32_t held_tempty = tempty_leader0 + 8u * (acc ^ 1u);
            const bool in_range = n0 + c0 < (int)N && slab_row0 < (int)M && !dbg_no_store;   // warp-uniform
            // One-pass prepare: the operand of the first iteration is the un-normalised update, and
            // s = 1 / (1.01 |u| + 1e-7) of the tile's matrix enters here: G = (s s) X X^T, X1 = s (Q X).
            // (A fused polynomial part scales the held Gram accumulator, not its own.)
            float out_scale = 1.0f;
            if (slot_scale != nullptr && tl.scale_pow != 0u && epilogue != kEpiPoly) {
                const float sv = __ldcg(slot_scale + tl.slot);
                out_scale = tl.scale_pow == 2u ? sv * sv : sv;
            }
            const bool scaled = out_scale != 1.0f;   // warp-uniform

            if (epilogue == kEpiApplyLast) {
                // FP32 result in the storage layout: 32 columns (128 bytes) per staged slab
#pragma unroll 1
                for (int sub = 0; sub < 2; ++sub) {
                    uint32_t v[32];
                    tc_ld32(taddr + 32 * sub, v);
                    tc_ld_wait();
                    if (sub == 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(tempty);
                    }
                    if (!in_range || n0 + c0 + 32 * sub >= (int)N) continue;
                    if (CHAINED && sub == 1 && unpublished != kNoSlot) publish();
                    if (scaled) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * out_scale);
                    }
                    __syncwarp();   // the copy-out of the previous slab is done in every lane
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint4 w = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        *reinterpret_cast<uint4 *>(slab + lane * 128 + ((j ^ (lane & 7)) << 4)) = w;
                    }
                    __syncwarp();
                    if (!dbg_no_global)
                        slab_to_global(out32, pitch32, slab_row0, (int)M, (n0 + c0 + 32 * sub) * 4, (int)pitch32);
                }
            } else {
                // 16-bit result: the chunk's 64 columns are read in two halves of 32 and packed
                uint32_t packed[32];
                if (fused) {
                    // four quarters of 16 columns: this tile's accumulator and the held Gram accumulator, which
                    // enters as the unfused form would have read it back from memory
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        uint32_t v[16], h[16];
                        tc_ld16(taddr + 16 * k, v);
                        tc_ld16(held_taddr + 16 * k, h);
                        tc_ld_wait();
                        if (k == 3) {
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) { mbar_arrive_cluster(tempty); mbar_arrive_cluster(held_tempty); }
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int gcol = n0 + c0 + 16 * k + j;
                            const float ident = (gcol == grow) ? ca : 0.0f;
                            const float base = scaled ? __uint_as_float(h[j]) * out_scale : __uint_as_float(h[j]);
                            // store/plain.rs:175-178: fma(c, acc, fma(b, base, identity))
                            v[j] = __float_as_uint(fmaf(cc, __uint_as_float(v[j]), fmaf(cb, base, ident)));
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            packed[8 * k + j] = pack_operands(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]), f16);
                    }
                } else {
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) {
                    uint32_t v[32];
                    tc_ld32(taddr + 32 * sub, v);
                    tc_ld_wait();
                    if (sub == 1 && !hold) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(tempty);
                    }
                    if (scaled) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * out_scale);
                    }
                    if ((epilogue == kEpiGram || epilogue == kEpiPoly) && !dbg_no_store) {
                        const size_t unit = unit0 + 8 * sub;
                        if (epilogue == kEpiGram) {
                            if (!dbg_no_global) {
                                float4 *fw = const_cast<float4 *>(frag);
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    __stcg(fw + (unit + j) * kGemmBlockM + row_in_tile,
                                           make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                       __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3])));
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float gv[4] = {g[j].x, g[j].y, g[j].z, g[j].w};
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const int gcol = n0 + c0 + 32 * sub + 4 * j + e;
                                    const float ident = (gcol == grow) ? ca : 0.0f;
                                    // store/plain.rs:175-178: fma(c, acc, fma(b, base, identity))
                                    v[4 * j + e] = __float_as_uint(
                                        fmaf(cc, __uint_as_float(v[4 * j + e]), fmaf(cb, gv[e], ident)));
                                }
                            }
                            if (sub == 0) {   // the other 32 columns, while this half is packed
#pragma unroll
                                for (int j = 0; j < 8; ++j) g[j] = __ldcg(frag + (unit + 8 + j) * kGemmBlockM + row_in_tile);
                            }
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        packed[16 * sub + j] = pack_operands(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]), f16);
                }
                }
                if (CHAINED && unpublished != kNoSlot) publish();
                if (in_range) {
                    __syncwarp();   // the copy-out of the previous slab is done in every lane
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint4 w = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                        *reinterpret_cast<uint4 *>(slab + lane * 128 + ((j ^ (lane & 7)) << 4)) = w;
                    }
                    __syncwarp();
                    if (!dbg_no_global) slab_to_global(out16, pitch16, slab_row0, (int)M, (n0 + c0) * 2, (int)pitch16);
                    if (mirror) {
                        // transposed 64 x 32 block (rows = this chunk's columns), plain row-major
                        // 64-byte rows: lanes pair up so every lane stores two rows of one column
                        __syncwarp();
#pragma unroll
                        for (int c = 0; c < 64; c += 2) {
                            const uint32_t mine = packed[c >> 1];
                            const uint32_t other = __shfl_xor_sync(0xffffffffu, mine, 1);
                            const uint32_t out = (lane & 1) ? __byte_perm(other, mine, 0x7632) : __byte_perm(mine, other, 0x5410);
                            *reinterpret_cast<uint32_t *>(slab + (c + (lane & 1)) * 64 + (lane & ~1) * 2) = out;
                        }
                        __syncwarp();
                        if (!dbg_no_global)
                            slab_t_to_global(out16, pitch16, n0 + c0, (int)M, slab_row0 * 2, (int)pitch16);
                    }
                }
            }
            if (CHAINED) {
                if (unpublished != kNoSlot) publish();   // (a tile whose stores were all skipped)
                unpublished = tl.slot;
                // the other CTAs wait for a held Gram tile before they can go on: publish it at once
                if (hold) publish();
            }
            acc ^= 1u;
            if (acc == 0) acc_phase ^= 1u;
            }
        }
        if (CHAINED && unpublished != kNoSlot) publish();
    }

    __syncthreads();
    if (*abort_flag) {
        // A wait ran out: give copies and MMAs still in flight time to land before the shared
        // memory and TMEM are released, then report.
        for (int i = 0; i < 4096; ++i) __nanosleep(512);
        if (threadIdx.x == 0) atomicExch(status, 1u);
        __syncthreads();
    }
    if (PAIR) cluster_sync_all();  // neither CTA leaves while its peer may still touch it
    if (CHAINED && threadIdx.x == 0) {
        // leave the shared words as the next launch expects them
        if (*abort_flag) atomicExch(&sync->abort, 1u);
        __threadfence();
        if (atomicAdd(&sync->exited, 1u) == gridDim.x - 1) {
            for (uint32_t k = 0; k < slot_count; ++k) sync->progress[k] = 0;
            sync->abort = 0;
            sync->ticket = 0;
            sync->exited = 0;
        }
    }
    if (warp == 1) {
        if (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                         "r"((uint32_t)C::kTmemCols) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                         "r"((uint32_t)C::kTmemCols) : "memory");
    }
}

template <int BN, bool PAIR, bool CHAINED>
cudaError_t launch_impl(const GemmProblem *problems, const void *tiles, uint32_t tile_count, uint32_t epilogue,
                        int f16, const GemmCoefficients &coef, const float *slot_scale, uint32_t scale_pow,
                        uint32_t *status, void *sync, uint32_t slot_count, uint32_t debug_flags, int grid,
                        cudaStream_t s) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    unsigned n_attr = 0;
    bool chained = true;
#ifdef B2_MEASURE
    chained = !(debug_flags & 32u);   // plain stream order
#endif
    if (chained) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (PAIR) {
        int clusters = grid / 2;
        if ((uint32_t)clusters > tile_count) clusters = (int)tile_count;
        if (clusters < 1) clusters = 1;
        grid = 2 * clusters;
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 2;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    } else if ((uint32_t)grid > tile_count) {
        grid = (int)tile_count;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)Cfg<BN, PAIR>::kThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg<BN, PAIR>::kSmemBytes;
    cfg.stream = s;
    return cudaLaunchKernelEx(&cfg, k_ns_gemm<BN, PAIR, CHAINED>, problems, tiles, tile_count, epilogue, f16, coef,
                              slot_scale, scale_pow, status, static_cast<ChainSync *>(sync), slot_count, debug_flags);
}

template <bool CHAINED>
cudaError_t dispatch(int block_n, int pair, const GemmProblem *problems, const void *tiles, uint32_t tile_count,
                     uint32_t epilogue, int f16, const GemmCoefficients &coef, const float *slot_scale,
                     uint32_t scale_pow, uint32_t *status, void *sync, uint32_t slot_count, uint32_t debug_flags,
                     int grid, cudaStream_t s) {
    if (tile_count == 0) return cudaSuccess;
    if (pair && block_n == 256)
        return launch_impl<256, true, CHAINED>(problems, tiles, tile_count, epilogue, f16, coef, slot_scale, scale_pow,
                                                  status, sync, slot_count, debug_flags, grid, s);
    if (!pair && block_n == 256)
        return launch_impl<256, false, CHAINED>(problems, tiles, tile_count, epilogue, f16, coef, slot_scale, scale_pow,
                                                   status, sync, slot_count, debug_flags, grid, s);
    if (!pair && block_n == 128)
        return launch_impl<128, false, CHAINED>(problems, tiles, tile_count, epilogue, f16, coef, slot_scale, scale_pow,
                                                   status, sync, slot_count, debug_flags, grid, s);
    return cudaErrorInvalidValue;
}

template <int BN, bool PAIR>
cudaError_t configure_both() {
    cudaError_t e = cudaFuncSetAttribute(k_ns_gemm<BN, PAIR, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg<BN, PAIR>::kSmemBytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(k_ns_gemm<BN, PAIR, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                Cfg<BN, PAIR>::kSmemBytes);
}

}  // namespace

cudaError_t gemm_configure(int block_n, int pair) {
    if (pair && block_n == 256) return configure_both<256, true>();
    if (!pair && block_n == 256) return configure_both<256, false>();
    if (!pair && block_n == 128) return configure_both<128, false>();
    return cudaErrorInvalidValue;
}
namespace {
template <int BN, bool PAIR>
int resident_groups(int sm_count) {
    if (PAIR) {
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cfg.gridDim = dim3((unsigned)(sm_count & ~1), 1, 1);
        cfg.blockDim = dim3((unsigned)Cfg<BN, PAIR>::kThreads, 1, 1);
        cfg.dynamicSmemBytes = Cfg<BN, PAIR>::kSmemBytes;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, k_ns_gemm<BN, PAIR, true>, &cfg) != cudaSuccess) {
            (void)cudaGetLastError();
            return 0;
        }
        return clusters;
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_ns_gemm<BN, PAIR, true>, Cfg<BN, PAIR>::kThreads,
                                                      Cfg<BN, PAIR>::kSmemBytes) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return per_sm > 0 ? sm_count : 0;   // one CTA per SM is all a launch ever uses
}
}  // namespace
int gemm_resident_groups(int block_n, int pair, int sm_count) {
    if (pair && block_n == 256) return resident_groups<256, true>(sm_count);
    if (!pair && block_n == 256) return resident_groups<256, false>(sm_count);
    if (!pair && block_n == 128) return resident_groups<128, false>(sm_count);
    return 0;
}
cudaError_t launch_ns_gemm(int block_n, int pair, const GemmProblem *problems, const GemmTile *tiles,
                           uint32_t tile_count, uint32_t epilogue, int f16, float ca, float cb,
                           float cc, const float *slot_scale, uint32_t scale_pow, uint32_t *status,
                           uint32_t debug_flags, int grid, cudaStream_t s) {
    GemmCoefficients coef = {};
    coef.v[0] = ca; coef.v[1] = cb; coef.v[2] = cc;
    return dispatch<false>(block_n, pair, problems, tiles, tile_count, epilogue, f16, coef, slot_scale, scale_pow, status,
                           nullptr, 0u, debug_flags, grid, s);
}
size_t chain_sync_bytes(uint32_t slot_count) { return sizeof(ChainSync) + sizeof(uint32_t) * slot_count; }
uint32_t chain_epilogue_warps(int block_n, int pair) { return (uint32_t)(4 * (block_n / 64)) * (pair ? 2u : 1u); }
cudaError_t launch_ns_chain(int block_n, int pair, const GemmProblem *problems, const ChainTile *tiles,
                            uint32_t tile_count, int f16, const GemmCoefficients &coef, const float *slot_scale,
                            uint32_t *status, void *sync, uint32_t slot_count, uint32_t debug_flags, int grid,
                            cudaStream_t s, bool fused_list) {
    // the epilogue argument of the plain launch carries the list kind here
    return dispatch<true>(block_n, pair, problems, tiles, tile_count, fused_list ? 1u : 0u, f16, coef, slot_scale, 0u,
                          status, sync, slot_count, debug_flags, grid, s);
}

}  // namespace b2
