// Block-scaled NVFP4 GEMM for sm_100a:  D[M,N] = (A o SFA) * (B o SFB)^T, FP32 accumulation in TMEM,
// fused epilogue  y = cast(raw * alpha) (+ bias)  with crop.
//
//   A: e2m1 payload [M][K/2] (K-major), SFA: ue4m3, one per 16 elements, in 128-row x 4-scale blocks of
//      512 bytes ordered [M/128][K/64]; B, SFB likewise with N rows.  M, N, K are multiples of 128.
//
// One persistent CTA per SM, 320 threads, warp-specialised:
//   warp 0    TMA producer.  Per k-tile of 256 elements: A box 128 rows x 128 B and B box BN rows x 128 B (128-byte
//             swizzle) plus the scale blocks (boxes of four 512-byte blocks, unswizzled), all completing on the
//             stage's mbarrier.  Plain loads only: every CTA fetches its own tiles.
//   warp 1    allocates TMEM; one lane copies the stage's scale blocks from shared memory into the TMEM scale buffer
//             with tcgen05.cp (32x128b.warpx4: one 512-byte block fills four columns of all 128 lanes, which is the
//             four-fold replication the MMA expects), issues tcgen05.mma.kind::mxf4nvf4.block_scale (M128 x N x K64)
//             and commits to the stage / accumulator barriers.  Copies and MMAs execute in issue order, so the scale
//             buffers need no barriers.  The scale blocks are read from shared memory once per k-tile: shared-memory
//             bandwidth (operand reads by the tensor core + TMA writes) is what bounds this kernel, and moving the
//             scales through registers with one warp per TMEM sub-partition read them four times.
//   warps 2-9 epilogue, two per TMEM sub-partition, eight 16-column units of the tile each.  For BF16 output a warp
//             drains its units to registers: tcgen05.ld -> bf16(acc) -> x bf16(alpha), kept as packed BF16 pairs; with
//             256-column tiles the two accumulator stages share 32 columns, each warp reads its shared unit first and
//             arrives, which releases the next tile's MMAs, and only afterwards pushes the registers through a small
//             swizzled staging buffer into TMA stores (which also crop).  The next tile's MMAs therefore wait for one
//             16-column read, not for the drain or the stores.
//   The producer and MMA warps run their loops converged and elect one lane per instruction (elect.sync): a loop that
//   one lane entered alone makes every descriptor and coordinate a per-thread value that has to be moved into uniform
//   registers before each TMA / tcgen05 instruction, which costs far more than the instructions themselves.
// Every wait is bounded: on expiry the kernel raises the status word, all roles leave their loops, the producer
// waits (bounded) for loads still in flight, TMEM is freed and the kernel returns.
#include "common.cuh"

#include <cuda.h>

#include <algorithm>
#include <cstdlib>

namespace nvfp4 {

constexpr int GEMM_THREADS = 320;
constexpr int FIRST_EPI_WARP = 2;
constexpr int BM = 128;
constexpr int BK = 256;             // elements per k-tile = 128 payload bytes per row
constexpr int A_STAGE_BYTES = BM * 128;
constexpr int SF_BLOCK = 512;       // 128 rows x 4 scales
constexpr int EPI_SLAB_BYTES = 1024;  // 32 rows x 32 bytes per epilogue warp
constexpr int EPI_WARPS = 8;
constexpr long long WAIT_CYCLES = 4000000000LL;  // ~2 s at 2 GHz

// PAIR: two CTAs of a cluster work on one 256 x 256 tile with tcgen05.mma.cta_group::2 (256-row MMAs): each CTA loads
// its own 128 rows of A and its own 128 of the tile's 256 rows of B, holds the accumulator of its 128 rows, and the
// leader CTA (cluster rank 0) issues every MMA for both.
template <int BN, bool PAIR> struct GemmCfg {
    static_assert(!PAIR || BN == 256, "paired CTAs work on 256 x 256 tiles");
    static constexpr int B_ROWS = PAIR ? BN / 2 : BN;                 // rows of B this CTA loads per k-tile
    static constexpr int B_STAGE_BYTES = B_ROWS * 128;
    static constexpr int SFA_STAGE_BYTES = 4 * SF_BLOCK;
    static constexpr int SFB_STAGE_BYTES = (BN / 128) * 4 * SF_BLOCK;  // every CTA needs the scales of all BN columns
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES + SFA_STAGE_BYTES + SFB_STAGE_BYTES;
    static constexpr int STAGES = PAIR ? 5 : (BN == 256) ? 4 : 6;
    // Two accumulator stages.  Two 256-column accumulators and the scale buffers do not fit the 512 columns of tensor
    // memory, so with BN = 256 the stages OVERLAP by 32 columns: stage 0 = columns [0, 256), stage 1 = [224, 480), the
    // scale buffers behind them.  The epilogue reads the shared 32 columns first (the last 32 of a stage-0 tile, the
    // first 32 of a stage-1 tile), 16 per warp of a sub-partition, and only that read gates the next tile's MMAs; the
    // rest of the drain and all stores run under the next mainloop.
    // The scale buffers hold one k-block (one MMA) each and alternate: the copy for k-block i + 1 writes one buffer
    // while the MMA of k-block i reads the other (two buffers measured within 1 % of four).
    static constexpr bool OVERLAP = BN == 256;
    static constexpr int ACC_STAGES = 2;
    static constexpr int ACC_STRIDE = OVERLAP ? 224 : BN;
    static constexpr int SHARED_COLS = OVERLAP ? BN - ACC_STRIDE : 0;   // columns both stages use
    static constexpr int SFA_COLS = 4;              // one k-block: 128 rows x 4 scales
    static constexpr int SFB_COLS = BN / 32;
    static constexpr int SF_BUF_COLS = SFA_COLS + SFB_COLS;
    static constexpr int SF_BASE = ACC_STRIDE + BN;                     // 480 or 256
    static constexpr int SF_BUFS = 2;
    static constexpr int TMEM_COLS = 512;
    static constexpr int EPI_BYTES = EPI_WARPS * EPI_SLAB_BYTES;
    static constexpr int NUM_BARS = 2 * STAGES + 2 * ACC_STAGES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*alignment slack*/ + 512 /*barriers*/;
    static constexpr int CTAS = PAIR ? 2 : 1;
    static_assert(SF_BASE + SF_BUFS * SF_BUF_COLS <= TMEM_COLS, "TMEM budget");
    static_assert(NUM_BARS * 8 + 16 <= 512, "barrier area");
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct GemmArgs {
    const float* pts_a;  // null: no tensor scaling (raw accumulator output)
    const float* pts_b;
    const void* bias;    // null or N-vector
    void* out;
    int* status;         // null or device int, set non-zero when a bounded wait expired
    int64_t ldo;
    int bias_f32, out_f32, raw_bf16, tma_store;
    int M, N, K, rows, cols;
    int tiles_m, tiles_n, k_tiles;
};

// ---- PTX wrappers --------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// try_wait that lets the hardware park the thread until the phase completes or `ns` nanoseconds pass
__device__ __forceinline__ bool mbar_try_sleep(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the time limit passed or another role raised the abort flag.  Waiting threads
// are parked by the hardware (20 us per attempt) instead of spinning: fourteen warps polling shared memory cost power,
// and this kernel's speed is set by the clock the power cap allows.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_sleep(bar, parity, 20000u)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_CYCLES) { *abort_flag = 1; return false; }
    }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, const void* src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(src)) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// ---- forms used by paired CTAs (cluster of two) ----
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t leader_addr(const void* p) {   // the same shared-memory offset in cluster rank 0
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(r) : "r"(smem_u32(p)));
    return r;
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(leader_addr(bar)) : "memory");
}
// tile load into this CTA's shared memory whose bytes are counted on the leader CTA's barrier (no multicast)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(leader_addr(bar)) : "memory");
}
// arrive on the barrier at this offset in BOTH CTAs once every MMA issued so far has completed
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate,
                                            uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate,
                                       uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// one 512-byte scale block (32 rows x 16 bytes) into four TMEM columns of all 128 lanes
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
// paired form: each CTA's block at this shared-memory offset goes into its own tensor memory
__device__ __forceinline__ void tc_cp_sf_pair(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}

__device__ __forceinline__ bool elect_one() {   // true in exactly one lane of a converged warp
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
// Bounded wait by a whole converged warp; every lane returns the same answer.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}

// K-major, 128-byte swizzled operand tile (rows of 128 bytes, 8-row groups 1024 bytes apart).
__device__ __forceinline__ uint64_t operand_desc(uint32_t saddr) {
    return static_cast<uint64_t>((saddr & 0x3ffffu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// One 512-byte scale block seen as 32 rows x 16 bytes, unswizzled (8-row groups 128 bytes apart).
__device__ __forceinline__ uint64_t scale_desc(uint32_t saddr) {
    return static_cast<uint64_t>((saddr & 0x3ffffu) >> 4) | (8ull << 32) | (1ull << 46);
}
__device__ __forceinline__ uint32_t instr_desc(int n, int m = BM) {  // e2m1 x e2m1, ue4m3 scales, K-major A and B
    return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

template <int BN, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
            const __grid_constant__ CUtensorMap map_out, const GemmArgs g) {
    using Cfg = GemmCfg<BN, PAIR>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* epi_smem = smem + Cfg::STAGES * Cfg::STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + Cfg::EPI_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = full + Cfg::STAGES;
    uint64_t* acc_full = empty + Cfg::STAGES;
    uint64_t* acc_empty = acc_full + Cfg::ACC_STAGES;  // [ACC_STAGES]; OVERLAP uses [0] only: "shared columns drained"
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + Cfg::ACC_STAGES);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    // the warp index is made provably warp-uniform: the issuing roles below run converged and elect one lane per
    // instruction, which keeps descriptors and addresses in uniform registers
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    // PAIR: rank 0 of the cluster is the leader.  Barriers that gate the MMA issue (full, acc_empty) are the leader's
    // and count bytes / arrivals of both CTAs; barriers that release resources (empty, acc_full) exist in both CTAs
    // and are arrived on together by one committed tcgen05 operation.
    const int rank = PAIR ? static_cast<int>(cluster_rank()) : 0;
    const bool leader = rank == 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < Cfg::ACC_STAGES; ++a) mbar_init(&acc_full[a], 1);
        for (int a = 0; a < Cfg::ACC_STAGES; ++a) mbar_init(&acc_empty[a], EPI_WARPS * Cfg::CTAS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (PAIR) {   // the same warp of both CTAs allocates the same columns in both tensor memories
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(Cfg::TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(Cfg::TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync();   // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = g.tiles_m * g.tiles_n;     // PAIR: tiles_m counts 256-row tiles
    const int kb_total = g.K / 64;
    const int first_tile = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int tile_step = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        // the whole warp runs the loop converged and one elected lane issues: a loop entered by a single lane makes
        // every TMA / tcgen05 operand a per-thread value that has to be moved into uniform registers first, which
        // measurably slows the issue rate (2.8 -> 4.7 PFLOP/s on the MMA warp at 8192^3)
        {
            int stage = 0; uint32_t phase = 0;
            int issued = 0;
            bool ok = true;
            for (int t = first_tile; t < total_tiles && ok; t += tile_step) {
                const int tm = (t % g.tiles_m) * Cfg::CTAS + rank, tn = t / g.tiles_m;   // tm: this CTA's 128-row block
                for (int kt = 0; kt < g.k_tiles; ++kt) {
                    if (!mbar_wait_warp(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                    if (elect_one()) {
                        uint8_t* st = smem + stage * Cfg::STAGE_BYTES;
                        uint8_t* st_sfa = st + A_STAGE_BYTES + Cfg::B_STAGE_BYTES;
                        uint8_t* st_sfb = st_sfa + Cfg::SFA_STAGE_BYTES;
                        // scale boxes are always four blocks; past the last k-block they hold the next row block's scales
                        // (or the out-of-bounds fill), which no MMA reads
                        const int sfa_row = tm * kb_total + kt * 4;
                        if constexpr (PAIR) {
                            // the bytes of both CTAs are counted on the leader's barrier
                            if (leader) mbar_expect_tx(&full[stage], 2 * Cfg::STAGE_BYTES);
                            tma_load_2d_pair(st, &map_a, kt * 128, tm * BM, &full[stage]);
                            tma_load_2d_pair(st + A_STAGE_BYTES, &map_b, kt * 128, tn * BN + rank * Cfg::B_ROWS, &full[stage]);
                            tma_load_2d_pair(st_sfa, &map_sfa, 0, sfa_row, &full[stage]);
#pragma unroll
                            for (int nb = 0; nb < BN / 128; ++nb)
                                tma_load_2d_pair(st_sfb + nb * 4 * SF_BLOCK, &map_sfb, 0, (tn * (BN / 128) + nb) * kb_total + kt * 4, &full[stage]);
                        } else {
                            mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
                            tma_load_2d(st, &map_a, kt * 128, tm * BM, &full[stage]);
                            tma_load_2d(st + A_STAGE_BYTES, &map_b, kt * 128, tn * BN, &full[stage]);
                            tma_load_2d(st_sfa, &map_sfa, 0, sfa_row, &full[stage]);
#pragma unroll
                            for (int nb = 0; nb < BN / 128; ++nb)
                                tma_load_2d(st_sfb + nb * 4 * SF_BLOCK, &map_sfb, 0, (tn * (BN / 128) + nb) * kb_total + kt * 4, &full[stage]);
                        }
                    }
                    __syncwarp();
                    ++issued;
                    if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok && lane == 0) {
                // loads already issued still write into this CTA's shared memory: give them a bounded chance to land
                const int pending = min(issued, Cfg::STAGES);
                int s = stage; uint32_t ph = phase;
                for (int i = 0; i < pending; ++i) {
                    if (--s < 0) { s = Cfg::STAGES - 1; ph ^= 1; }
                    const long long t0 = clock64();
                    // PAIR: the byte counts live on the leader's barriers; the other CTA waits a fixed time instead
                    if (leader) while (!mbar_try(&full[s], ph) && clock64() - t0 < WAIT_CYCLES / 8) {}
                }
                if constexpr (PAIR) { const long long t0 = clock64(); while (clock64() - t0 < 400000) {} }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (leader) {
            const uint32_t idesc_full = instr_desc(BN, BM * Cfg::CTAS);
            int stage = 0; uint32_t phase = 0;
            int sfb = 0;
            int local = 0;
            bool ok = true;
            auto copy_sf = [](uint32_t taddr, uint64_t desc) { if constexpr (PAIR) tc_cp_sf_pair(taddr, desc); else tc_cp_sf(taddr, desc); };
            auto mma = [](uint32_t d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc, uint32_t tsfa, uint32_t tsfb) {
                if constexpr (PAIR) tc_mma_pair(d, da, db, idesc, acc, tsfa, tsfb); else tc_mma(d, da, db, idesc, acc, tsfa, tsfb);
            };
            auto commit = [](uint64_t* bar) { if constexpr (PAIR) tc_commit_pair(bar); else tc_commit(bar); };
            for (int t = first_tile; t < total_tiles && ok; t += tile_step, ++local) {
                const int acc = local & 1;
                const uint32_t tmem_acc = tmem_base + acc * Cfg::ACC_STRIDE;
                // the accumulator stage must be free.  OVERLAP: the previous tile's epilogue has read the shared columns
                // and every epilogue warp has finished reading the tile before it (the last user of this stage);
                // otherwise: the last user of this stage, two tiles ago, is fully drained
                if (Cfg::OVERLAP ? local > 0 : true) {
                    uint64_t* bar = Cfg::OVERLAP ? &acc_empty[0] : &acc_empty[acc];
                    const uint32_t parity = Cfg::OVERLAP ? ((local - 1) & 1) : (((local >> 1) & 1) ^ 1);
                    if (!mbar_wait_warp(bar, parity, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                }
                for (int kt = 0; kt < g.k_tiles; ++kt) {
                    if (!mbar_wait_warp(&full[stage], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
                    const uint32_t sb = sa + A_STAGE_BYTES;
                    const uint32_t ssfa = sb + Cfg::B_STAGE_BYTES;
                    const uint32_t ssfb = ssfa + Cfg::SFA_STAGE_BYTES;
                    const int kblocks = min(4, kb_total - kt * 4);
                    if (elect_one()) {
                        // each k-block's copies sit directly before its MMA (faster than all twelve up front, and than
                        // copying one k-tile ahead: 5.16 against 4.79 and 4.85 PFLOP/s at 8192^3); a copy queues behind
                        // the MMA that still reads its scale buffer (issued SF_BUFS k-blocks ago)
                        for (int kb = 0; kb < kblocks; ++kb) {
                            const uint32_t sfa_tmem = tmem_base + Cfg::SF_BASE + (sfb ^ (kb & 1)) * Cfg::SF_BUF_COLS;
                            const uint32_t sfb_tmem = sfa_tmem + Cfg::SFA_COLS;
                            copy_sf(sfa_tmem, scale_desc(ssfa + kb * SF_BLOCK));
#pragma unroll
                            for (int nb = 0; nb < BN / 128; ++nb)
                                copy_sf(sfb_tmem + nb * 4, scale_desc(ssfb + (nb * 4 + kb) * SF_BLOCK));
                            mma(tmem_acc, operand_desc(sa + kb * 32), operand_desc(sb + kb * 32), idesc_full, (kt | kb) ? 1u : 0u,
                                sfa_tmem, sfb_tmem);
                        }
                        commit(&empty[stage]);
                    }
                    __syncwarp();
                    sfb ^= kblocks & 1;   // every lane keeps the buffer parity: the elected lane need not stay the same
                    if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok && elect_one()) commit(&acc_full[acc]);
                __syncwarp();
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int sub = warp & 3;                    // TMEM sub-partition this warp may read
        const int half = (warp - FIRST_EPI_WARP) >> 2;   // the two warps of a sub-partition share the tile's columns
        constexpr int UNITS = BN / 32;               // 16-column units per warp
        const int row_in_tile = sub * 32 + lane;
        uint8_t* slab = epi_smem + (warp - FIRST_EPI_WARP) * EPI_SLAB_BYTES;
        float alpha = 1.f;
        const bool scaled = g.pts_a != nullptr;
        if (scaled) {
            alpha = __fmul_rn(__ldg(g.pts_a), __ldg(g.pts_b));
            if (g.raw_bf16) alpha = bf16_value(bf16_bits(alpha));
        }
        const __nv_bfloat162 alpha2 = __float2bfloat162_rn(alpha);
        const bool fast = !g.bias && !g.out_f32;   // BF16 output without bias: drain to packed registers first, store later
        int local = 0;
        bool ok = true;

        // writes 32 rows x 32 bytes held as two uint4 per lane: through the staging slab and a TMA store, or directly
        auto emit = [&](const uint4& q0, const uint4& q1, int64_t row, int64_t col0, int tile_row0, int cols_here) {
            if (g.tma_store) {
                if (lane == 0) bulk_wait_read<0>();      // the store that last read the slab has drained it
                __syncwarp();
                const int sw = (lane >> 2) & 1;            // 32-byte swizzle: 16-byte chunk index ^ bit 2 of the row
                *reinterpret_cast<uint4*>(slab + lane * 32 + ((0 ^ sw) << 4)) = q0;
                *reinterpret_cast<uint4*>(slab + lane * 32 + ((1 ^ sw) << 4)) = q1;
                fence_async_shared();
                __syncwarp();
                if (lane == 0) { tma_store_2d(&map_out, static_cast<int>(col0), tile_row0, slab); bulk_commit(); }
            } else if (row < g.rows) {
                const int esz = g.out_f32 ? 4 : 2;
                uint8_t* dst = static_cast<uint8_t*>(g.out) + (row * g.ldo + col0) * esz;
                if (col0 + cols_here <= g.cols && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                    reinterpret_cast<uint4*>(dst)[0] = q0; reinterpret_cast<uint4*>(dst)[1] = q1;
                } else {
                    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (j < cols_here && col0 + j < g.cols) {
                            if (g.out_f32) reinterpret_cast<uint32_t*>(dst)[j] = w[j & 7];
                            else reinterpret_cast<uint16_t*>(dst)[j] = static_cast<uint16_t>(w[j >> 1] >> ((j & 1) * 16));
                        }
                    }
                }
            }
        };

        auto release_acc = [&](uint64_t* bar) { if (PAIR && !leader) mbar_arrive_leader(bar); else mbar_arrive(bar); };
        for (int t = first_tile; t < total_tiles && ok; t += tile_step, ++local) {
            const int tm = (t % g.tiles_m) * Cfg::CTAS + rank, tn = t / g.tiles_m;
            const int acc = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int64_t row = static_cast<int64_t>(tm) * BM + row_in_tile;
            const int tile_row0 = tm * BM + sub * 32;
            const int64_t colbase = static_cast<int64_t>(tn) * BN;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(sub * 32) << 16) + acc * Cfg::ACC_STRIDE;
            const bool rows_live = tile_row0 < g.rows;
            // Which 16-column unit of the tile this warp handles i-th.  OVERLAP: the two units both stages use (the last
            // two of a stage-0 tile, the first two of a stage-1 tile) come first, one per warp of the sub-partition;
            // the next tile's MMAs are released as soon as every warp has read its shared unit.  The other fourteen
            // units are split seven / seven and drained (and stored) under the next mainloop.
            constexpr int SHARED_UNITS = Cfg::SHARED_COLS / 16;                      // 2 or 0
            constexpr int OWN_UNITS = (BN / 16 - SHARED_UNITS) / 2;                  // 7 or UNITS
            auto unit_of = [&](int i) -> int {
                if constexpr (!Cfg::OVERLAP) return half * UNITS + i;
                else if (i == 0) return acc == 0 ? BN / 16 - SHARED_UNITS + half : half;
                else return (acc == 0 ? 0 : SHARED_UNITS) + half * OWN_UNITS + (i - 1);
            };
            uint64_t* release_bar = Cfg::OVERLAP ? &acc_empty[0] : &acc_empty[acc];
            if (fast) {
                uint32_t packed[UNITS * 8];
#pragma unroll
                for (int i = 0; i < UNITS; ++i) {
                    uint32_t r[16];
                    tc_ld16(taddr + unit_of(i) * 16, r);
                    tc_wait_ld();
                    if (Cfg::OVERLAP && i == 0) {   // the shared unit is in registers
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) release_acc(release_bar);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        __nv_bfloat162 p;
                        if (g.raw_bf16) {
                            p = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                            if (scaled) p = __hmul2(p, alpha2);   // bf16 x bf16 is exact in FP32: one rounding, as in the FP32 chain
                        } else {   // FP32 chain: acc * alpha in FP32, one rounding to BF16
                            p = __floats2bfloat162_rn(__fmul_rn(__uint_as_float(r[2 * j]), alpha), __fmul_rn(__uint_as_float(r[2 * j + 1]), alpha));
                        }
                        packed[i * 8 + j] = *reinterpret_cast<uint32_t*>(&p);
                    }
                }
                if constexpr (!Cfg::OVERLAP) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) release_acc(release_bar);   // accumulator share is in registers
                }
                if (rows_live) {
#pragma unroll
                    for (int i = 0; i < UNITS; ++i) {
                        const int64_t col0 = colbase + unit_of(i) * 16;
                        if (col0 < g.cols)
                            emit(make_uint4(packed[i * 8], packed[i * 8 + 1], packed[i * 8 + 2], packed[i * 8 + 3]),
                                 make_uint4(packed[i * 8 + 4], packed[i * 8 + 5], packed[i * 8 + 6], packed[i * 8 + 7]), row, col0, tile_row0, 16);
                    }
                }
            } else {
                const int cols_per_slab = g.out_f32 ? 8 : 16;
#pragma unroll 1
                for (int i = 0; i < UNITS; ++i) {
                    const int64_t ucol = colbase + unit_of(i) * 16;
                    uint32_t r[16];
                    tc_ld16(taddr + unit_of(i) * 16, r);
                    tc_wait_ld();
                    if (Cfg::OVERLAP ? i == 0 : i + 1 == UNITS) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) release_acc(release_bar);
                    }
                    if (!rows_live) continue;
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int64_t col = ucol + j;
                        float x = __uint_as_float(r[j]);
                        if (g.raw_bf16) x = bf16_value(bf16_bits(x));
                        if (scaled) {
                            x = __fmul_rn(x, alpha);
                            if (g.raw_bf16) x = bf16_value(bf16_bits(x));
                        }
                        if (g.bias && col < g.cols) {
                            float b = g.bias_f32 ? __ldg(static_cast<const float*>(g.bias) + col)
                                                 : bf16_value(__ldg(static_cast<const uint16_t*>(g.bias) + col));
                            if (g.raw_bf16) b = bf16_value(bf16_bits(b));
                            x = __fadd_rn(x, b);
                            if (g.raw_bf16) x = bf16_value(bf16_bits(x));
                        }
                        v[j] = x;
                    }
#pragma unroll
                    for (int sl = 0; sl < 2; ++sl) {          // one 32-byte slab of BF16 or two of FP32 per unit
                        if (sl * cols_per_slab >= 16) break;
                        const int j0 = sl * cols_per_slab;
                        const int64_t col0 = ucol + j0;
                        if (col0 >= g.cols) continue;
                        uint4 q0, q1;
                        if (g.out_f32) {
                            q0 = make_uint4(__float_as_uint(v[j0]), __float_as_uint(v[j0 + 1]), __float_as_uint(v[j0 + 2]), __float_as_uint(v[j0 + 3]));
                            q1 = make_uint4(__float_as_uint(v[j0 + 4]), __float_as_uint(v[j0 + 5]), __float_as_uint(v[j0 + 6]), __float_as_uint(v[j0 + 7]));
                        } else {
                            uint32_t w[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) w[j] = bf16_bits(v[2 * j]) | (uint32_t(bf16_bits(v[2 * j + 1])) << 16);
                            q0 = make_uint4(w[0], w[1], w[2], w[3]); q1 = make_uint4(w[4], w[5], w[6], w[7]);
                        }
                        emit(q0, q1, row, col0, tile_row0, cols_per_slab);
                    }
                }
            }
        }
        if (lane == 0) bulk_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync();   // neither CTA leaves while the other may still touch its memory or barriers
    if (threadIdx.x == 0 && *abort_flag && g.status) atomicExch(g.status, NVFP4_ERR_TIMEOUT);
    if (warp == 1) {
        tc_fence_after();
        if constexpr (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(Cfg::TMEM_COLS) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(Cfg::TMEM_COLS) : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

static bool make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(k / 2), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(k / 2)};
    cuuint32_t box[2] = {128, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Scale blocks as rows of 512 bytes, [row blocks of 128][K / 64] in storage order; a box is the four blocks of a k-tile.
static bool make_scale_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {SF_BLOCK / 4, static_cast<cuuint64_t>((rows / 128) * (k / 64))};
    cuuint64_t strides[1] = {SF_BLOCK};
    cuuint32_t box[2] = {SF_BLOCK / 4, 4};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Output map for the epilogue's stores: boxes of 32 rows x 32 bytes, 32-byte swizzle; the bounds crop the tile.
static bool make_out_map(CUtensorMap* map, void* base, int64_t rows, int64_t cols, int64_t ldo, bool f32) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const int esz = f32 ? 4 : 2;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldo * esz)};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(32 / esz), 32};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, bool PAIR>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& msa, const CUtensorMap& msb,
                       const CUtensorMap& mo, GemmArgs& g, cudaStream_t st) {
    using Cfg = GemmCfg<BN, PAIR>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_kernel<BN, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        NVFP4_REQUIRE(e == cudaSuccess, NVFP4_ERR_LAUNCH, "nvfp4_gemm: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES, cudaGetErrorString(e));
        configured[dev] = true;
    }
    static int sm_count[64] = {};
    if (dev < 64 && !sm_count[dev]) cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
    // NVFP4_GEMM_RESERVE_SMS=n keeps n SMs out of the persistent grid, for kernels that run beside the GEMMs and cannot share
    // an SM with a CTA that holds all of its shared memory (the collectives of data-parallel training)
    static const int reserve = [] { const char* e = getenv("NVFP4_GEMM_RESERVE_SMS"); return e ? std::max(0, atoi(e)) : 0; }();
    const int sms = std::max(2, (dev < 64 && sm_count[dev] > 0 ? sm_count[dev] : 148) - reserve);
    g.tiles_n = g.N / BN;
    g.tiles_m = g.M / (BM * Cfg::CTAS);
    if constexpr (PAIR) {
        // persistent clusters of two CTAs (one per SM of a pair); an odd SM count leaves one SM idle
        const int clusters = std::min(g.tiles_m * g.tiles_n, sms / 2);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(clusters * 2));
        cfg.blockDim = dim3(GEMM_THREADS);
        cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_kernel<BN, PAIR>, ma, mb, msa, msb, mo, g);
        NVFP4_REQUIRE(e == cudaSuccess, NVFP4_ERR_LAUNCH, "nvfp4_gemm: cluster launch failed: %s", cudaGetErrorString(e));
    } else {
        const int grid = std::min(g.tiles_m * g.tiles_n, sms);
        gemm_kernel<BN, PAIR><<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(ma, mb, msa, msb, mo, g);
    }
    return launch_status("nvfp4_gemm");
}

}  // namespace nvfp4

using namespace nvfp4;

extern "C" int nvfp4_gemm(const uint8_t* a, const uint8_t* sfa, const float* pts_a, const uint8_t* b, const uint8_t* sfb,
                          const float* pts_b, int64_t M, int64_t N, int64_t K, const void* bias, int bias_dtype, void* out,
                          int out_dtype, int64_t ldo, int64_t rows, int64_t cols, int raw_bf16, int* status,
                          nvfp4_stream_t stream) {
    NVFP4_REQUIRE(a && sfa && b && sfb && out, NVFP4_ERR_ARG, "nvfp4_gemm: null pointer");
    NVFP4_REQUIRE((pts_a == nullptr) == (pts_b == nullptr), NVFP4_ERR_ARG, "nvfp4_gemm: give both tensor scales or neither");
    NVFP4_REQUIRE(M > 0 && N > 0 && K > 0 && M % 128 == 0 && N % 128 == 0 && K % 128 == 0, NVFP4_ERR_ARG,
                  "nvfp4_gemm: M, N, K must be positive multiples of 128 (got %lld %lld %lld)", (long long)M, (long long)N, (long long)K);
    NVFP4_REQUIRE(rows > 0 && cols > 0 && rows <= M && cols <= N && ldo >= cols, NVFP4_ERR_ARG, "nvfp4_gemm: invalid output crop");
    NVFP4_REQUIRE(M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31), NVFP4_ERR_ARG, "nvfp4_gemm: dimension exceeds 2^31");
    NVFP4_REQUIRE(out_dtype == NVFP4_F32 || out_dtype == NVFP4_BF16, NVFP4_ERR_DTYPE, "nvfp4_gemm: output must be FP32 or BF16");
    NVFP4_REQUIRE(!bias || bias_dtype == NVFP4_F32 || bias_dtype == NVFP4_BF16, NVFP4_ERR_DTYPE, "nvfp4_gemm: bias must be FP32 or BF16");
    for (const void* p : {static_cast<const void*>(a), static_cast<const void*>(b), static_cast<const void*>(sfa), static_cast<const void*>(sfb)})
        NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0, NVFP4_ERR_ALIGN, "nvfp4_gemm: operands and scales must be 16-byte aligned");
    GemmArgs g{};
    g.pts_a = pts_a; g.pts_b = pts_b; g.bias = bias; g.out = out; g.status = status;
    g.ldo = ldo; g.bias_f32 = bias_dtype == NVFP4_F32; g.out_f32 = out_dtype == NVFP4_F32; g.raw_bf16 = (raw_bf16 & 1) != 0;
    g.M = static_cast<int>(M); g.N = static_cast<int>(N); g.K = static_cast<int>(K);
    g.rows = static_cast<int>(rows); g.cols = static_cast<int>(cols);
    g.k_tiles = (g.K + BK - 1) / BK;
    const int bn = (N % 256 == 0) ? 256 : 128;
    const bool pair = bn == 256 && M % 256 == 0 && !(raw_bf16 & NVFP4_GEMM_SINGLE_CTA);
    const int esz = g.out_f32 ? 4 : 2;
    // the bulk-tensor store needs a 16-byte aligned base and row pitch; anything else takes the plain-store epilogue
    g.tma_store = (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (ldo * esz) % 16 == 0;
    CUtensorMap ma, mb, msa, msb, mo;
    NVFP4_REQUIRE(make_operand_map(&ma, a, M, K, BM) && make_operand_map(&mb, b, N, K, pair ? 128 : bn) &&
                      make_scale_map(&msa, sfa, M, K) && make_scale_map(&msb, sfb, N, K), NVFP4_ERR_LAUNCH,
                  "nvfp4_gemm: cuTensorMapEncodeTiled failed or is unavailable");
    if (g.tma_store && !make_out_map(&mo, out, rows, cols, ldo, g.out_f32)) g.tma_store = 0;
    if (!g.tma_store) mo = ma;  // unused by the kernel in this mode, but the parameter must hold a valid map
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (pair) return launch_gemm<256, true>(ma, mb, msa, msb, mo, g, st);
    return bn == 256 ? launch_gemm<256, false>(ma, mb, msa, msb, mo, g, st) : launch_gemm<128, false>(ma, mb, msa, msb, mo, g, st);
}
