// Tensor-core matmuls on CTA pairs (tcgen05.mma.cta_group::2), two operand kinds from one kernel template:
//
//   Bfp8 kind   C[M,N] (bfloat16) = A[M,K] (bfloat16) @ W[K,N], W stored as Bfp8_b tiles.
//               Reference semantics: torch.matmul on the decoded operands
//               (pybuda/pybuda/op/eval/pybuda/matmul.py:20-33; weight format rule pybuda/csrc/passes/dataformat.cpp:409-418).
//   Int8 kind   acc[M,N] (int32) = A[M,K] (int8) @ W[K,N] (int8 tiles of an Int8 queue), then in the epilogue
//               nothing / requantisation to int8 / dequantisation to float32.  Reference semantics: an int8 matmul
//               yields int32 (pybuda/pybuda/op/eval/common.py:50-65) and a matmul carrying the "requant" attribute is
//               followed by requantization of its result (pybuda/csrc/graph_lib/python_bindings.cpp:655-676):
//               round(float(acc) * scale + zero_point) clamped to int8 (pybuda/pybuda/op/eval/buda/quantize.py:42-53);
//               dequantization is (float(acc) - zero_point) * scale (quantize.py:35-40).
//
// Why pairs.  The single-CTA Bfp8 kernel is bound by the integer work of turning Bfp8_b blocks into bfloat16
// operands: every CTA decodes a 256-column slab of W for 256 rows of A.  Here two CTAs on neighbouring SMs
// issue one MMA that covers M = 256 (128 rows in each CTA's tensor memory) x N = 256, and the hardware reads
// the weight operand half from each CTA's shared memory.  So each CTA prepares only 128 columns per k-block
// while its tensor core still sees all 256: half the decode work per flop, and (for int8, whose tensor
// throughput is twice that of bfloat16) half the weight bytes pulled from L2 per flop.
//
// Pair tile: 512 rows x 256 columns (two M = 256 accumulators, all 512 tensor-memory columns of both
// SMs); k-block = 128 bytes of K (64 bfloat16 / 128 int8).  In each CTA (rank r = 0 leader, 1 peer):
//   warp 8        producer: TMA-loads this CTA's two 128-row activation boxes per k-block; the loads of both CTAs
//                 are counted on ONE barrier in the leader (the load's .cta_group::2 form; each CTA fetches its own boxes)
//   warps 10..17  weights: this CTA's 128 columns of the k-block, global -> registers -> N-major swizzled
//                 operand stage (Bfp8: decoded to bfloat16; Int8: the 16-byte face rows are copied as they are),
//                 then arrive on the LEADER's full_b barrier
//   warp 9        leader: one thread issues the MMAs for the pair and commits completion to both
//                 CTAs' barriers (multicast commit).  peer: idle
//   warps 0-7     epilogue for this CTA's 2 x 128 rows (two warps per tensor-memory lane quadrant, half
//                 of the columns each); both CTAs' epilogues release the accumulators on the leader's
//                 acc_empty barrier.  A one-device launch writes each 32-row x 64-column piece (bfloat16, or
//                 requantised int8) into one of the warp's two staging buffers in shared memory and hands it to the
//                 copy engine as one bulk tensor store; 4-byte outputs and launches that feed peers store from
//                 registers.  In a launch that also feeds peer devices the same warps then forward
//                 the piece they wrote to the peers' copies while the next tile's MMAs run: one plain store per
//                 peer, or ONE multimem store to the multicast address of the matrix, which the NVSwitch
//                 replicates to every device of the group
// Every mbarrier wait is bounded; a wait that gives up raises the device status word, the CTA winds
// down, its partner runs into its own limit, and both meet at the closing cluster barrier (tensor
// memory is freed on every path).
#include <atomic>
#include <cstdio>
#include <cstdlib>

#include "gemm_common.cuh"

namespace buda {

namespace gemm_pair {

using namespace gemm;

constexpr int kPairM = 512;        // rows of C per pair tile
constexpr int kBN = 256;           // columns of C per pair tile
constexpr int kHalfN = 128;        // weight columns decoded by one CTA
constexpr int kBKBytes = 128;      // k-block: one 128-byte swizzled row of K (64 bfloat16 / 128 int8)
constexpr int kBStages = 4;   // decoded-weight ring (per CTA: 128 columns x 64 deep)
constexpr int kABytes = 2 * 128 * kBKBytes;  // 32768
constexpr int kBBytes = kHalfN * kBKBytes;   // 16384
constexpr int kDecodeWarps = 8;
constexpr int kEpiWarps = 8;        // two per tensor-memory lane quadrant: each takes half of the columns
constexpr int kProducerWarp = kEpiWarps, kMmaWarp = kEpiWarps + 1, kFirstDecodeWarp = kEpiWarps + 2;
constexpr int kThreads = 32 * (kEpiWarps + 1 + 1 + kDecodeWarps);
constexpr int kTmemCols = 512;
constexpr int kEpiStageBytes = 2 * 32 * 128;   // per epilogue warp: two buffers of what it hands to one bulk tensor store


// Shared-memory plan (the same for a launch that also writes peers' memory, kScatter): 3 x 32 KB of activations,
// 4 x 16 KB of weight operand, 8 x 8 KB of epilogue staging, barriers.
template <bool kScatter>
struct Layout {
    static constexpr int kAStages = 3;                  // activation ring (per CTA: two 128-row boxes per stage); the fourth
                                                        // stage's 32 KB serve the epilogue's second staging buffers better (+1.1 %)
    static constexpr int kSmemA = 0;
    static constexpr int kSmemB = kSmemA + kAStages * kABytes;
    static constexpr int kSmemEpi = kSmemB + kBStages * kBBytes;      // per epilogue warp: two pieces of 32 rows x 64 bfloat16 columns, 128-byte swizzle
    static constexpr int kSmemBar = kSmemEpi + kEpiWarps * kEpiStageBytes;
    static constexpr int kNumBars = 2 * kAStages + 2 * kBStages + 2;
    static constexpr int kSmemBytes = kSmemBar + kNumBars * 8 + 16 + 1024;
};

enum : int { kKindBfp8 = 0, kKindI8 = 1 };

template <int Kind>
struct KindTraits;
template <>
struct KindTraits<kKindBfp8> {
    static constexpr int kBK = 64;          // elements of K per k-block
    static constexpr int kKTiles = 2;       // 32-deep tile rows per k-block
    static constexpr int kRecordBytes = 1088;
    static constexpr int kPrefetch = 3;     // k-blocks of raw weight records in flight per decode thread
    // instruction descriptor: D = F32, A = B = BF16, A K-major, B MN-major, N = 256, M = 256 (pair)
    static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(kBN >> 3) << 17) |
                                       ((uint32_t)(256 >> 4) << 24);
    // weight operand stage, N-major: 64-column atoms 1024 B apart, 8-deep k groups 2048 B apart
    static constexpr uint32_t kBLbo = 1024, kBSbo = 2048;
};
template <>
struct KindTraits<kKindI8> {
    static constexpr int kBK = 128;
    static constexpr int kKTiles = 4;
    static constexpr int kRecordBytes = 1024;   // Int8 tile: four 16x16 faces, 16 bytes per face row, no exponents
    static constexpr int kPrefetch = 2;     // four units per warp and k-block: a third k-block in flight costs registers (spills), 0.436 -> 0.430 ms with two
    // instruction descriptor: D = S32, A = B = S8, A K-major, B MN-major, N = 256, M = 256 (pair)
    static constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(kBN >> 3) << 17) |
                                       ((uint32_t)(256 >> 4) << 24);
    // weight operand stage, N-major: one 128-column atom per 8-deep k group, groups 1024 B apart
    static constexpr uint32_t kBLbo = 1024, kBSbo = 1024;
};

// TMA tile load whose completion is counted on a barrier of the pair's leader CTA (given as a shared::cluster address):
// both CTAs' activation boxes land on ONE barrier, so the issuing thread waits for one thing and nobody relays.
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *tmap, int x, int y, uint32_t leader_bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(leader_bar)
        : "memory");
}

template <int Kind>
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    if constexpr (Kind == kKindBfp8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// arrive on the barrier at this shared-memory offset in BOTH CTAs of the pair once every MMA issued so far is complete
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     smem_u32(bar)),
                 "h"((uint16_t)3)
                 : "memory");
}

// one 16-byte store that the switch delivers to every device bound to the multicast address
__device__ __forceinline__ void multimem_st_16(void *mc_addr, const uint4 v)
{
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}

template <int Kind, bool kScatter>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ Params p, const __grid_constant__ OutMaps out_maps)
{
    using KT = KindTraits<Kind>;
    using L = Layout<kScatter>;
    constexpr int kBK = KT::kBK;
    constexpr int kPrefetch = KT::kPrefetch;
    constexpr int kAStages = L::kAStages, kSmemA = L::kSmemA, kSmemB = L::kSmemB, kSmemBar = L::kSmemBar,
                  kNumBars = L::kNumBars;
    extern __shared__ uint8_t smem_raw[];
    // identical carve-up in both CTAs: the MMA addresses the peer's operands by the leader's offsets
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sA = smem + kSmemA;
    uint8_t *sB = smem + kSmemB;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kSmemBar);
    uint64_t *full_a = bars;                    // [kAStages] leader only: both CTAs' activations landed (TMA bytes of both)
    uint64_t *empty_a = full_a + kAStages;      // [kAStages] MMAs reading the activations are done (both CTAs)
    uint64_t *full_b = empty_a + kAStages;      // [kBStages] leader only: both CTAs' decoded weights written
    uint64_t *empty_b = full_b + kBStages;      // [kBStages] MMAs reading the decoded weights are done (both CTAs)
    uint64_t *acc_full = empty_b + kBStages;    // accumulators complete (both CTAs)
    uint64_t *acc_empty = acc_full + 1;         // leader only: both CTAs' epilogues drained the accumulators
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + kNumBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const uint32_t total_tiles = p.m_tiles * p.n_tiles;

    if (tid == 0) {
        for (int s = 0; s < kAStages; s++) {
            mbar_init(&full_a[s], 1);
            mbar_init(&empty_a[s], 1);
        }
        for (int t = 0; t < kBStages; t++) {
            mbar_init(&full_b[t], 2 * kDecodeWarps);
            mbar_init(&empty_b[t], 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 2 * kEpiWarps);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == kProducerWarp) {
        // one warp of each CTA of the pair allocates all 512 tensor-memory columns of its SM
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();  // both CTAs' barriers are initialised before anything arrives on them remotely
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == kProducerWarp) {
        // ------------------------------------------------------------------ producer (both CTAs)
        if (lane == 0) {
            uint32_t i = 0;
            bool ok = true;
            for (uint32_t tile = pair; tile < total_tiles && ok; tile += num_pairs) {
                uint32_t m_blk, n_blk_unused;
                tile_coords(p, tile, m_blk, n_blk_unused);
                const int row0 = (int)(m_blk * kPairM + rank * 128);
                for (uint32_t kb = 0; kb < p.k_blocks; kb++, i++) {
                    const int s = i % kAStages;
                    const uint32_t ph = ((i / kAStages) & 1u) ^ 1u;
                    if (!mbar_wait_bounded(&empty_a[s], ph, abort_flag, p.status, BUDA_DEVSTAT_GEMM_WAIT)) {
                        ok = false;
                        break;
                    }
                    const uint32_t leader_bar = map_to_cta(smem_u32(&full_a[s]), 0);
                    if (rank == 0) mbar_arrive_expect_tx(&full_a[s], 2 * kABytes);   // this CTA's boxes and the partner's
                    tma_load_2d_pair(sA + s * kABytes, &tmap_a, (int)(kb * kBK), row0, leader_bar);
                    tma_load_2d_pair(sA + s * kABytes + kABytes / 2, &tmap_a, (int)(kb * kBK), row0 + 256, leader_bar);
                }
            }
            const uint32_t back = i < (uint32_t)kAStages ? i : (uint32_t)kAStages;
            if ((!ok || *abort_flag) && rank == 0) {
                // let the copies already issued land before shared memory is released (the partner's are counted on this
                // CTA's barriers too, and the partner stays until the closing cluster barrier)
                for (uint32_t k = 1; k <= back; k++) {
                    const uint32_t j = i - k;
                    uint64_t t0 = global_timer_ns();
                    while (!mbar_try_wait(&full_a[j % kAStages], (j / kAStages) & 1u) && global_timer_ns() - t0 < 100000000ull) {
                    }
                }
            } else if (ok && !*abort_flag) {
                // the leader's last commits arrive on this CTA's barriers asynchronously: see them land before leaving
                for (uint32_t k = 1; k <= back; k++) {
                    const uint32_t j = i - k;
                    if (!mbar_wait_bounded(&empty_a[j % kAStages], (j / kAStages) & 1u, abort_flag, p.status, BUDA_DEVSTAT_GEMM_WAIT)) break;
                }
            }
        }
        __syncwarp();
    } else if (warp == kMmaWarp) {
        if (lane == 0 && rank == 0) {
            // -------------------------------------------------------------- MMA issue (leader)
            uint32_t i = 0, tile_iter = 0;
            bool ok = true;
            for (uint32_t tile = pair; tile < total_tiles && ok; tile += num_pairs, tile_iter++) {
                if (tile_iter > 0) {  // both epilogues must have drained the previous tile's accumulators
                    if (!mbar_wait_bounded_cluster(acc_empty, (tile_iter - 1) & 1u, abort_flag, p.status, BUDA_DEVSTAT_GEMM_WAIT)) break;
                    tc_fence_after();
                }
                for (uint32_t kb = 0; kb < p.k_blocks; kb++, i++) {
                    const int s = i % kAStages, t = i % kBStages;
                    // The two barriers of this k-block are probed back to back, so the probes' latencies overlap, and
                    // only a barrier that is not complete yet is waited for.  This thread is the pair's only source of
                    // MMAs: with one probe after the other (then three: the partner's activations had a barrier
                    // of their own) it spent a fifth of its time in their round trips even when everything was ready
                    // (0.810 -> 0.767 ms on 8192 x 4096 x 16384).
                    const bool r0 = mbar_test_wait(&full_a[s], (i / kAStages) & 1u);
                    const bool r2 = mbar_test_wait(&full_b[t], (i / kBStages) & 1u);
                    if (!(r0 && r2) &&
                        (!mbar_wait_bounded_cluster(&full_a[s], (i / kAStages) & 1u, abort_flag, p.status, BUDA_DEVSTAT_GEMM_WAIT) ||
                         !mbar_wait_bounded_cluster(&full_b[t], (i / kBStages) & 1u, abort_flag, p.status, BUDA_DEVSTAT_GEMM_WAIT))) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(sA + s * kABytes), b_addr = smem_u32(sB + t * kBBytes);
#pragma unroll
                    for (int h = 0; h < 2; h++) {
#pragma unroll
                        for (int j = 0; j < kBKBytes / 32; j++) {
                            // A: K-major, 8-row groups 1024 B apart, 32 B per 16-deep k-step inside the swizzled row
                            const uint64_t adesc = smem_desc(a_addr + h * (kABytes / 2) + j * 32, 16, 1024);
                            // B (this CTA's 128 columns, N-major): 32 bytes of K = 4096 B of the stage per step
                            const uint64_t bdesc = smem_desc(b_addr + j * 4096, KT::kBLbo, KT::kBSbo);
                            umma_pair<Kind>(tmem_base + h * kBN, adesc, bdesc, KT::kIdesc, (kb > 0 || j > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit_pair(&empty_a[s]);
                    umma_commit_pair(&empty_b[t]);
                }
                if (ok) umma_commit_pair(acc_full);
            }
        }
        __syncwarp();
    } else if (warp >= kFirstDecodeWarp) {
        // ------------------------------------------------------------------ weight warps (both CTAs)
        // Units of 32 face rows (16 values at fixed k): kKTiles x 4 tile records per k-block, two units per record.
        constexpr int kUnits = KT::kKTiles * 4 * 2 / kDecodeWarps;
        const int dw = warp - kFirstDecodeWarp;
        // Raw records go global -> registers kPrefetch k-blocks ahead of their decode (a fetch cursor walks the
        // same (tile, k-block) sequence as the loop below), so the loop never waits for a load it just issued.
        uint4 mq[kPrefetch][kUnits];
        uint32_t eq[kPrefetch][kUnits];
        uint32_t f_tile = pair, f_kb = 0;
        auto fetch_into = [&](uint4 (&m)[kUnits], uint32_t (&e)[kUnits]) {
            if (f_tile < total_tiles) {
                uint32_t m_blk_unused, n_blk;
                tile_coords(p, f_tile, m_blk_unused, n_blk);
#pragma unroll
                for (int it = 0; it < kUnits; it++) {
                    const int u = it * kDecodeWarps + dw;
                    const int r = u >> 1;                           // record: k-tile r / 4, n-tile r % 4
                    const int blk = (u & 1) * 32 + lane;            // block = face * 16 + face row
                    const uint8_t *rec = p.W + ((uint64_t)(f_kb * KT::kKTiles + (r >> 2)) * p.Nt + (uint64_t)n_blk * 8 + rank * 4 +
                                                (r & 3)) * KT::kRecordBytes;
                    if constexpr (Kind == kKindBfp8) {
                        m[it] = __ldg(reinterpret_cast<const uint4 *>(rec + 64 + blk * 16));
                        e[it] = __ldg(rec + blk);
                    } else {
                        m[it] = __ldg(reinterpret_cast<const uint4 *>(rec + blk * 16));
                        e[it] = 0u;
                    }
                }
                if (++f_kb == p.k_blocks) {
                    f_kb = 0;
                    f_tile += num_pairs;
                }
            } else {
#pragma unroll
                for (int it = 0; it < kUnits; it++) {
                    m[it] = make_uint4(0u, 0u, 0u, 0u);
                    e[it] = 0u;
                }
            }
        };
#pragma unroll
        for (int d = 0; d < kPrefetch; d++) fetch_into(mq[d], eq[d]);
        uint32_t i = 0;
        bool ok = true;
        for (uint32_t tile = pair; tile < total_tiles && ok; tile += num_pairs) {
            for (uint32_t kb = 0; kb < p.k_blocks; kb++, i++) {
                const int t = i % kBStages;
                uint4 mant_cur[kUnits];
                uint32_t exp_cur[kUnits];
#pragma unroll
                for (int it = 0; it < kUnits; it++) {
                    mant_cur[it] = mq[0][it];
                    exp_cur[it] = eq[0][it];
                }
#pragma unroll
                for (int d = 0; d + 1 < kPrefetch; d++) {
#pragma unroll
                    for (int it = 0; it < kUnits; it++) {
                        mq[d][it] = mq[d + 1][it];
                        eq[d][it] = eq[d + 1][it];
                    }
                }
                fetch_into(mq[kPrefetch - 1], eq[kPrefetch - 1]);
                const bool got = mbar_wait_bounded(&empty_b[t], ((i / kBStages) & 1u) ^ 1u, abort_flag, p.status, BUDA_DEVSTAT_GEMM_WAIT);
                if (!__all_sync(0xffffffffu, got)) {  // the whole warp leaves together
                    ok = false;
                    break;
                }
                uint8_t *bst = sB + t * kBBytes;
#pragma unroll
                for (int it = 0; it < kUnits; it++) {
                    const int u = it * kDecodeWarps + dw;
                    const int r = u >> 1;
                    const int blk = (u & 1) * 32 + lane;
                    const int k_local = (r >> 2) * 32 + (blk >> 5) * 16 + (blk & 15);
                    const int n_local = (r & 3) * 32 + ((blk >> 4) & 1) * 16;
                    if constexpr (Kind == kKindBfp8) {
                        decode_block_to_operand<kHalfN / 64>(mant_cur[it], exp_cur[it], bst, k_local, n_local);
                    } else {
                        // 16 int8 values of one k: one 16-byte chunk of the 128-byte row k of its 8-deep group
                        const int kr = k_local & 7;
                        *reinterpret_cast<uint4 *>(bst + (k_local >> 3) * 1024 + kr * 128 + (((n_local >> 4) ^ kr) << 4)) = mant_cur[it];
                    }
                }
                fence_async_smem();  // the tensor cores read shared memory through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&full_b[t]), 0));
            }
        }
        if (ok && dw == 0 && lane == 0) {
            // as in the producer: the last stage releases must have landed on this CTA's barriers
            const uint32_t back = i < (uint32_t)kBStages ? i : (uint32_t)kBStages;
            for (uint32_t k = 1; k <= back; k++) {
                const uint32_t j = i - k;
                if (!mbar_wait_bounded(&empty_b[j % kBStages], (j / kBStages) & 1u, abort_flag, p.status, BUDA_DEVSTAT_GEMM_WAIT)) break;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue warps (both CTAs)
        // A warp reads the tensor-memory lanes of its quadrant (warp % 4); the two warps of a quadrant split the
        // 256 columns of each accumulator.  Two 32-column loads are in flight before the first is waited for.
        const int quad = warp & 3, col_half = warp >> 2;
        uint32_t tile_iter = 0;
        uint32_t piece = 0;   // pieces this warp has handed to the copy engine (picks the staging buffer when there are two)
        for (uint32_t tile = pair; tile < total_tiles; tile += num_pairs, tile_iter++) {
            uint32_t m_blk, n_blk;
            tile_coords(p, tile, m_blk, n_blk);
            const bool got = mbar_wait_bounded(acc_full, tile_iter & 1u, abort_flag, p.status, BUDA_DEVSTAT_GEMM_WAIT);
            if (!__all_sync(0xffffffffu, got)) break;  // the whole warp leaves together
            tc_fence_after();
            if (Kind == kKindBfp8 && p.tma_epilogue) {
                // The warp's 32 rows x 64 columns go to shared memory as bfloat16 (lane = row; the 16-byte chunks of a row
                // are permuted by the row number so that the lanes' stores do not meet in a bank -- the 128-byte swizzle
                // of the tensor map undoes it), and one elected lane hands the piece to the copy engine: one bulk tensor
                // store per destination, this device's matrix and every peer's alike.  The warp neither issues 32
                // separate lines per store instruction nor waits for NVLink; rows past M are clipped by the tensor map.
                uint8_t *stage = smem + L::kSmemEpi + warp * kEpiStageBytes;
#pragma unroll 1
                for (int h = 0; h < 2; h++) {
                    const int y = (int)(m_blk * kPairM) + h * 256 + (int)rank * 128 + quad * 32;
                    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(h * kBN + col_half * (kBN / 2));
#pragma unroll 1
                    for (int c = 0; c < kBN / 2 / 64; c++) {
                        uint32_t v0[32], v1[32];
                        tmem_ld32_issue(taddr + c * 64, v0);
                        tmem_ld32_issue(taddr + c * 64 + 32, v1);
                        tmem_ld_wait();
                        uint4 o[8];
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            o[q].x = pack_bf16x2(__uint_as_float(v0[8 * q]), __uint_as_float(v0[8 * q + 1]));
                            o[q].y = pack_bf16x2(__uint_as_float(v0[8 * q + 2]), __uint_as_float(v0[8 * q + 3]));
                            o[q].z = pack_bf16x2(__uint_as_float(v0[8 * q + 4]), __uint_as_float(v0[8 * q + 5]));
                            o[q].w = pack_bf16x2(__uint_as_float(v0[8 * q + 6]), __uint_as_float(v0[8 * q + 7]));
                            o[q + 4].x = pack_bf16x2(__uint_as_float(v1[8 * q]), __uint_as_float(v1[8 * q + 1]));
                            o[q + 4].y = pack_bf16x2(__uint_as_float(v1[8 * q + 2]), __uint_as_float(v1[8 * q + 3]));
                            o[q + 4].z = pack_bf16x2(__uint_as_float(v1[8 * q + 4]), __uint_as_float(v1[8 * q + 5]));
                            o[q + 4].w = pack_bf16x2(__uint_as_float(v1[8 * q + 6]), __uint_as_float(v1[8 * q + 7]));
                        }
                        // the piece that used this buffer last has been read out of it (with two buffers: the piece before
                        // the previous one, whose read-out has had a whole piece's work to finish)
                        constexpr int kBufs = kEpiStageBytes / 4096;
                        uint8_t *buf = stage + (kBufs > 1 ? (piece & 1u) * 4096u : 0u);
                        piece++;
                        if (lane == 0) {
                            if (kBufs > 1) bulk_wait_read_but_one();
                            else bulk_wait_read_all();
                        }
                        __syncwarp();
                        uint8_t *rowp = buf + lane * 128;
#pragma unroll
                        for (int q = 0; q < 8; q++) *reinterpret_cast<uint4 *>(rowp + ((q ^ (lane & 7)) << 4)) = o[q];
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            const int x = (int)(n_blk * kBN) + col_half * (kBN / 2) + c * 64;
                            for (int d = 0; d < p.n_dst; d++) tma_store_2d(&out_maps.m[d], buf, x, y);
                            bulk_commit();
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(acc_empty), 0));
                continue;
            }
            if (Kind == kKindI8 && p.tma_epilogue) {
                // The same for the requantised int8 output: 32 rows x 64 bytes per piece, 64-byte swizzle.
                uint8_t *stage = smem + L::kSmemEpi + warp * kEpiStageBytes;
#pragma unroll 1
                for (int h = 0; h < 2; h++) {
                    const int y = (int)(m_blk * kPairM) + h * 256 + (int)rank * 128 + quad * 32;
                    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(h * kBN + col_half * (kBN / 2));
#pragma unroll 1
                    for (int c = 0; c < kBN / 2 / 64; c++) {
                        uint32_t v0[32], v1[32];
                        tmem_ld32_issue(taddr + c * 64, v0);
                        tmem_ld32_issue(taddr + c * 64 + 32, v1);
                        tmem_ld_wait();
                        const int x = (int)(n_blk * kBN) + col_half * (kBN / 2) + c * 64;
                        uint32_t w0[8], w1[8];
                        requant_row32(v0, p, x, w0);
                        requant_row32(v1, p, x + 32, w1);
                        // two 2 KB buffers: the piece before the previous one has been read out of this one
                        uint8_t *buf = stage + (piece & 1u) * 2048u;
                        piece++;
                        if (lane == 0) bulk_wait_read_but_one();
                        __syncwarp();
                        uint8_t *rowp = buf + lane * 64;
                        const int sw = (lane >> 1) & 3;
                        *reinterpret_cast<uint4 *>(rowp + ((0 ^ sw) << 4)) = make_uint4(w0[0], w0[1], w0[2], w0[3]);
                        *reinterpret_cast<uint4 *>(rowp + ((1 ^ sw) << 4)) = make_uint4(w0[4], w0[5], w0[6], w0[7]);
                        *reinterpret_cast<uint4 *>(rowp + ((2 ^ sw) << 4)) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
                        *reinterpret_cast<uint4 *>(rowp + ((3 ^ sw) << 4)) = make_uint4(w1[4], w1[5], w1[6], w1[7]);
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_2d(&out_maps.m[0], buf, x, y);
                            bulk_commit();
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(acc_empty), 0));
                continue;
            }
#pragma unroll 1
            for (int h = 0; h < 2; h++) {
                const int64_t row = (int64_t)m_blk * kPairM + h * 256 + rank * 128 + quad * 32 + lane;
                const int64_t off = row * p.ldc + (int64_t)n_blk * kBN + col_half * (kBN / 2);
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(h * kBN + col_half * (kBN / 2));
#pragma unroll 1
                for (int c = 0; c < kBN / 2 / 64; c++) {
                    uint32_t v0[32], v1[32];
                    tmem_ld32_issue(taddr + c * 64, v0);
                    tmem_ld32_issue(taddr + c * 64 + 32, v1);
                    tmem_ld_wait();
                    if (row < p.M)
                    {
                        if constexpr (Kind == kKindBfp8) {
                            // this device's copy: straight from registers
                            store_row32(v0, p.C, 1, off + c * 64);
                            store_row32(v1, p.C, 1, off + c * 64 + 32);
                        } else {
                            const int col = (int)n_blk * kBN + col_half * (kBN / 2) + c * 64;
                            store_row32_i8(v0, p, off + c * 64, col);
                            store_row32_i8(v1, p, off + c * 64 + 32, col + 32);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(acc_empty), 0));
            if constexpr (Kind == kKindBfp8 && kScatter) {
                // The accumulators are released: the next tile's MMAs run while this warp forwards the piece of the
                // output it has just written (its own 32 rows x 128 columns of both halves) to the peers.  It
                // re-reads the piece from this device's memory (L2) with lanes running along the row, so every
                // store instruction carries two whole 256-byte row segments over NVLink instead of 32 fragments
                // of 16 bytes; nothing is read from a peer.  __syncwarp orders the lanes' own stores before the
                // re-read; ld.global.cg does not look in L1.
                __syncwarp();
                const int ch = lane & 15;
#pragma unroll 1
                for (int h = 0; h < 2; h++) {
                    const int64_t row_base = (int64_t)m_blk * kPairM + h * 256 + rank * 128 + quad * 32;
                    const int64_t col_base = (int64_t)n_blk * kBN + col_half * (kBN / 2) + ch * 8;
#pragma unroll 4
                    for (int it = 0; it < 16; it++) {
                        const int64_t grow = row_base + it * 2 + (lane >> 4);
                        if (grow < p.M) {
                            const int64_t eo = grow * p.ldc + col_base;
                            const uint4 val = __ldcg(reinterpret_cast<const uint4 *>(p.C[0] + eo));
                            if (p.C_mc) multimem_st_16(p.C_mc + eo, val);   // every device of the group, this one included
                            else
                                for (int d = 1; d < p.n_dst; d++) *reinterpret_cast<uint4 *>(p.C[d] + eo) = val;
                        }
                    }
                }
            }
        }
    }

    // the bulk tensor stores of the epilogue are complete before the kernel is (only the lanes that issued any hold a group)
    if (warp < kEpiWarps && lane == 0) bulk_wait_all();
    // every path ends here: neither CTA leaves while its partner may still touch its shared memory or barriers
    tc_fence_before();
    cluster_sync_all();
    if (warp == kProducerWarp) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

}  // namespace gemm_pair

int gemm_kernel_choice(int which);

namespace {

template <int Kind, bool kScatter>
cudaError_t launch_pair(const CUtensorMap &tmap, const gemm::Params &p_in, const gemm::OutMaps &out_maps, int sm_count, cudaStream_t stream)
{
    using namespace gemm_pair;
    constexpr int kSmemBytes = Layout<kScatter>::kSmemBytes;
    static std::atomic<int> max_pairs[64];   // 0 = this device has not been set up for this instantiation yet
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    int resident = max_pairs[dev].load(std::memory_order_acquire);
    if (resident == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<Kind, kScatter>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        // how many pairs the device can hold at once (SMs that cannot be paired inside their GPC stay idle)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(sm_count & ~1), 1, 1);
        cfg.blockDim = dim3(kThreads, 1, 1);
        cfg.dynamicSmemBytes = kSmemBytes;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<Kind, kScatter>, &cfg);
        if (e != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = sm_count / 2;
        }
        resident = n;
        max_pairs[dev].store(n, std::memory_order_release);
    }
    gemm::Params p = p_in;
    p.m_tiles = (uint32_t)((p.M + kPairM - 1) / kPairM);
    // groups of 8 tile rows (32 MB of bfloat16 activations at K = 4096): 1342 TFLOP/s on 8192 x 4096 x 16384 against
    // 1289 walking all 16 tile rows per column (groups of 1 / 2 / 4: 1309 / 1319 / 1331)
    // (the int8 kind, whose operands come out of L2 at twice the rate, loses 4 % that way and keeps whole columns)
    p.raster_m = (Kind == gemm_pair::kKindBfp8 && p.m_tiles > 8u) ? 8u : p.m_tiles;
    p.n_tiles = (uint32_t)(p.N / kBN);
    p.k_blocks = (uint32_t)(p.K / KindTraits<Kind>::kBK);
    p.Nt = (uint32_t)(p.N / 32);
    const uint32_t tiles = p.m_tiles * p.n_tiles;
    uint32_t pairs = tiles;
    if (pairs > (uint32_t)resident) pairs = (uint32_t)resident;
    if constexpr (kScatter) {
        // A launch that also feeds the peers is bound by what each pair sends after each of its tiles, so every pair
        // should send the same amount: the fewest pairs that still finish in the same number of rounds (256 tiles on
        // 74 pairs are 4 rounds with 34 pairs sending in the last one; on 64 pairs they are 4 rounds of 64).
        const uint32_t rounds = (tiles + pairs - 1u) / pairs;
        pairs = (tiles + rounds - 1u) / rounds;
    }
    gemm_pair_kernel<Kind, kScatter><<<2 * pairs, kThreads, kSmemBytes, stream>>>(tmap, p, out_maps);
    return cudaGetLastError();
}

}  // namespace

// Launch of the CTA-pair Bfp8 kernel.  Same contract as the single-CTA launch; the caller has validated the shapes.
cudaError_t launch_bfp8b_gemm_pair(const CUtensorMap &tmap, const gemm::Params &p, const gemm::OutMaps &out_maps, int sm_count,
                                   cudaStream_t stream)
{
    if (p.n_dst > 1 || p.C_mc) return launch_pair<gemm_pair::kKindBfp8, true>(tmap, p, out_maps, sm_count, stream);
    return launch_pair<gemm_pair::kKindBfp8, false>(tmap, p, out_maps, sm_count, stream);
}

// int8 x int8 -> int32 matmul with the requantise / dequantise epilogue (see the header of this file).
cudaError_t launch_i8_gemm(const void *A, int64_t M, int64_t K, int64_t lda, const void *W, int64_t N, const float *scale,
                           int64_t scale_len, float zero_point, int out_mode, void *C, int64_t ldc, int sm_count, cudaStream_t stream,
                           unsigned int *status, char *err, size_t err_len)
{
    using namespace gemm;
    if (M <= 0 || N <= 0 || K <= 0 || (N % 256) || (K % 128)) {
        snprintf(err, err_len, "int8 gemm needs N %% 256 == 0 and K %% 128 == 0 (got M=%lld N=%lld K=%lld)", (long long)M, (long long)N,
                 (long long)K);
        return cudaErrorInvalidValue;
    }
    if (out_mode < BUDA_I8_OUT_INT32 || out_mode > BUDA_I8_OUT_DEQUANT_F32) {
        snprintf(err, err_len, "int8 gemm: unknown output mode %d", out_mode);
        return cudaErrorInvalidValue;
    }
    if (out_mode != BUDA_I8_OUT_INT32 && (!scale || (scale_len != 1 && scale_len != N))) {
        snprintf(err, err_len, "int8 gemm: scale must hold 1 or N = %lld values (got %lld)", (long long)N, (long long)scale_len);
        return cudaErrorInvalidValue;
    }
    const int out_elem = out_mode == BUDA_I8_OUT_REQUANT_I8 ? 1 : 4;
    if (lda < K || ldc < N || (lda % 16) || ((ldc * out_elem) % 16) || (reinterpret_cast<uintptr_t>(A) & 15) ||
        (reinterpret_cast<uintptr_t>(C) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) ||
        (scale_len > 1 && (reinterpret_cast<uintptr_t>(scale) & 15))) {
        snprintf(err, err_len, "int8 gemm needs 16-byte aligned A, W, C, scale and row strides that are multiples of 16 bytes");
        return cudaErrorInvalidValue;
    }
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) {
        snprintf(err, err_len, "cuTensorMapEncodeTiled is not available from this driver");
        return cudaErrorNotSupported;
    }
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)lda};
    const cuuint32_t box[2] = {128, 128};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(A), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        snprintf(err, err_len, "cuTensorMapEncodeTiled failed with code %d", (int)cr);
        return cudaErrorInvalidValue;
    }
    Params p = {};
    p.W = static_cast<const uint8_t *>(W);
    p.C[0] = static_cast<uint16_t *>(C);
    p.n_dst = 1;
    p.C_mc = nullptr;
    p.M = M; p.N = N; p.K = K; p.ldc = ldc;
    p.status = status;
    p.out_mode = out_mode;
    p.scale = scale;
    p.scale_len = scale_len;
    p.zero_point = zero_point;
    p.lo = -128.0f;
    p.hi = 127.0f;
    // the requantised int8 output leaves as bulk tensor stores (see the Bfp8 kind); 4-byte outputs store from registers
    OutMaps out_maps = {};
    p.tma_epilogue = (out_mode == BUDA_I8_OUT_REQUANT_I8 && gemm_kernel_choice(-1) != 3) ? 1 : 0;
    if (p.tma_epilogue) {
        const cuuint64_t cdims[2] = {(cuuint64_t)N, (cuuint64_t)M};
        const cuuint64_t cstrides[1] = {(cuuint64_t)ldc};
        const cuuint32_t cbox[2] = {64, 32};
        cr = encode(&out_maps.m[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, C, cdims, cstrides, cbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) {
            snprintf(err, err_len, "cuTensorMapEncodeTiled failed for the output with code %d", (int)cr);
            return cudaErrorInvalidValue;
        }
    }
    return launch_pair<gemm_pair::kKindI8, false>(tmap, p, out_maps, sm_count, stream);
}

}  // namespace buda
