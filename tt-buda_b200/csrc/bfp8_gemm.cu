// K7: C[M,N] (bfloat16) = A[M,K] (bfloat16) @ W[K,N], W stored as Bfp8_b tiles, binary32
// accumulation on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// The device counterpart of a matmul whose weight queue has data format Bfp8_b (the reference
// evaluates it as torch.matmul on the decoded operands, pybuda/pybuda/op/eval/pybuda/matmul.py:20-33;
// the weight format rule is pybuda/csrc/passes/dataformat.cpp:409-418).
//
// One persistent CTA per SM computes 256x256 output tiles as two 128x256 accumulators (all 512
// tensor-memory columns), so every decoded weight element feeds 256 rows of activations:
//   warp 4        producer: per 64-deep k-block, TMA-loads two 128x64 activation boxes (128B swizzle,
//                 K-major)
//   warps 6..     decode: each thread loads one 16-value block (one face row: fixed k, 16 consecutive
//                 n, one shared exponent) of the raw Bfp8_b records straight from global memory into
//                 registers, one k-block ahead; turns sign + 7-bit magnitude into bfloat16 pairs with
//                 one packed fma per pair ((128+m)*s - 128*s, exact) and writes them into the N-major
//                 ("MN-major") 128B-swizzled operand tile.  Shared memory only ever holds operands the
//                 tensor core reads: its bandwidth is what bounds this kernel.
//   warp 5        one thread issues tcgen05.mma (M=128, N=256, K=16; 2 halves x 4 k-steps per
//                 k-block) and commits completion to the mbarriers that free the stages
//   warps 0-3     epilogue: tcgen05.ld the accumulators, round to bfloat16, store C
// Every mbarrier wait is bounded; a wait that gives up raises the device status word and the CTA
// winds down (tensor memory is freed on every path).
#include <atomic>
#include <cstdio>
#include <cstdlib>

#include "gemm_common.cuh"

namespace buda {

namespace gemm {

constexpr int kBM = 256;           // rows of C per tile (two UMMA M=128 halves)
constexpr int kBN = 256;           // columns of C per tile
constexpr int kBK = 64;            // k-block
#ifndef GEMM_A_STAGES
#define GEMM_A_STAGES 3
#endif
#ifndef GEMM_B_STAGES
#define GEMM_B_STAGES 3
#endif
constexpr int kLoadStages = GEMM_A_STAGES;  // activation ring
constexpr int kBStages = GEMM_B_STAGES;     // decoded-weight ring
constexpr int kABytes = kBM * kBK * 2;           // 32768
constexpr int kBBytes = kBN * kBK * 2;           // 32768
template <int DW>
constexpr int threads_for() { return 32 * (4 + 1 + 1 + DW); }  // epilogue + producer + MMA + decode warps
constexpr int kTmemCols = 512;
#ifndef GEMM_PREFETCH
#define GEMM_PREFETCH 2
#endif
constexpr int kPrefetch = GEMM_PREFETCH;   // k-blocks of raw weight records in flight per decode thread

constexpr int kSmemA = 0;
constexpr int kSmemB = kSmemA + kLoadStages * kABytes;
constexpr int kSmemBar = kSmemB + kBStages * kBBytes;
constexpr int kNumBars = 2 * kLoadStages + 2 * kBStages + 2;
constexpr int kSmemBytes = kSmemBar + kNumBars * 8 + 16 + 1024;  // + tmem holder / abort flag, + alignment slack

// instruction descriptor: D = F32, A = B = BF16, A K-major, B MN-major, N = 256, M = 128
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (1u << 16) | ((uint32_t)(kBN >> 3) << 17) |
                            ((uint32_t)(128 >> 4) << 24);


template <int kDecodeWarps>
__global__ void __launch_bounds__(threads_for<kDecodeWarps>(), 1)
bfp8b_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ Params p)
{
    static_assert(32 % kDecodeWarps == 0, "32 decode units per k-block");
    extern __shared__ uint8_t smem_raw[];
    // 128B-swizzled operand tiles repeat every 1024 bytes: align the carve-up to that
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sA = smem + kSmemA;
    uint8_t *sB = smem + kSmemB;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kSmemBar);
    uint64_t *full_a = bars;                       // [kLoadStages] activations landed (TMA bytes)
    uint64_t *empty_a = full_a + kLoadStages;      // [kLoadStages] MMAs reading the activations are done
    uint64_t *full_b = empty_a + kLoadStages;      // [kBStages] decoded weights written
    uint64_t *empty_b = full_b + kBStages;         // [kBStages] MMAs reading the decoded weights are done
    uint64_t *acc_full = empty_b + kBStages;       // accumulators complete
    uint64_t *acc_empty = acc_full + 1;            // accumulators drained by the epilogue
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + kNumBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t total_tiles = p.m_tiles * p.n_tiles;

    if (tid == 0) {
        for (int s = 0; s < kLoadStages; s++) {
            mbar_init(&full_a[s], 1);
            mbar_init(&empty_a[s], 1);
        }
        for (int t = 0; t < kBStages; t++) {
            mbar_init(&full_b[t], kDecodeWarps);
            mbar_init(&empty_b[t], 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 4);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 4) {
        // the whole warp allocates all 512 tensor-memory columns and gives up the right to allocate more
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 4) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            uint32_t i = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const uint32_t m_blk = tile % p.m_tiles;
                for (uint32_t kb = 0; kb < p.k_blocks; kb++, i++) {
                    const int s = i % kLoadStages;
                    const uint32_t ph = ((i / kLoadStages) & 1u) ^ 1u;
                    if (!mbar_wait_bounded(&empty_a[s], ph, abort_flag, p.status, BUDA_DEVSTAT_GEMM_WAIT)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&full_a[s], kABytes);
                    tma_load_2d(sA + s * kABytes, &tmap_a, (int)(kb * kBK), (int)(m_blk * kBM), &full_a[s]);
                    tma_load_2d(sA + s * kABytes + kABytes / 2, &tmap_a, (int)(kb * kBK), (int)(m_blk * kBM + 128), &full_a[s]);
                }
            }
            if (!ok || *abort_flag) {
                // let the copies already issued land before shared memory is released
                const uint32_t back = i < (uint32_t)kLoadStages ? i : (uint32_t)kLoadStages;
                for (uint32_t k = 1; k <= back; k++) {
                    const uint32_t j = i - k;
                    uint64_t t0 = global_timer_ns();
                    while (!mbar_try_wait(&full_a[j % kLoadStages], (j / kLoadStages) & 1u) &&
                           global_timer_ns() - t0 < 100000000ull) {
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            uint32_t i = 0, tile_iter = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, tile_iter++) {
                if (tile_iter > 0) {  // the epilogue must have drained the previous tile's accumulators
                    if (!mbar_wait_bounded(acc_empty, (tile_iter - 1) & 1u, abort_flag, p.status, BUDA_DEVSTAT_GEMM_WAIT)) break;
                    tc_fence_after();
                }
                for (uint32_t kb = 0; kb < p.k_blocks; kb++, i++) {
                    const int s = i % kLoadStages, t = i % kBStages;
                    if (!mbar_wait_bounded(&full_a[s], (i / kLoadStages) & 1u, abort_flag, p.status, BUDA_DEVSTAT_GEMM_WAIT) ||
                        !mbar_wait_bounded(&full_b[t], (i / kBStages) & 1u, abort_flag, p.status, BUDA_DEVSTAT_GEMM_WAIT)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(sA + s * kABytes), b_addr = smem_u32(sB + t * kBBytes);
#pragma unroll
                    for (int h = 0; h < 2; h++) {
#pragma unroll
                        for (int j = 0; j < kBK / 16; j++) {
                            // A: K-major, 8-row groups 1024 B apart, 32 B per 16-deep k-step inside the swizzled row
                            const uint64_t adesc = smem_desc(a_addr + h * (kABytes / 2) + j * 32, 16, 1024);
                            // B: N-major, 64-column atoms 1024 B apart, 8-deep k groups 4096 B apart
                            const uint64_t bdesc = smem_desc(b_addr + j * 8192, 1024, 4096);
                            umma_bf16(tmem_base + h * kBN, adesc, bdesc, kIdesc, (kb > 0 || j > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(&empty_a[s]);
                    umma_commit(&empty_b[t]);
                }
                if (ok) umma_commit(acc_full);
            }
        }
        __syncwarp();
    } else if (warp >= 6) {
        // ------------------------------------------------------------------ decode warps
        // Raw records go global -> registers (coalesced 16-byte loads, one block per thread per unit),
        // kPrefetch k-blocks ahead of the decode, so they never cost shared-memory bandwidth and the
        // loop never waits for a load it just issued.
        constexpr int kUnits = 32 / kDecodeWarps;  // units of 32 blocks per warp per k-block
        const int dw = warp - 6;
        uint4 mq[kPrefetch][kUnits];
        uint32_t eq[kPrefetch][kUnits];
        uint32_t f_tile = blockIdx.x, f_kb = 0;   // fetch cursor: walks the same (tile, k-block) sequence, kPrefetch ahead
        auto fetch_into = [&](uint4 (&m)[kUnits], uint32_t (&e)[kUnits]) {
            if (f_tile < total_tiles) {
                const uint32_t n_blk = f_tile / p.m_tiles;
#pragma unroll
                for (int it = 0; it < kUnits; it++) {
                    const int u = it * kDecodeWarps + dw;          // 32 units: (record, half of its 64 blocks)
                    const int r = u >> 1;                           // record: k-tile r / 8, n-tile r % 8
                    const int blk = (u & 1) * 32 + lane;            // block = face * 16 + face row
                    const uint8_t *rec = p.W + ((uint64_t)(f_kb * 2 + (r >> 3)) * p.Nt + (uint64_t)n_blk * 8 + (r & 7)) * kRecord;
                    m[it] = __ldg(reinterpret_cast<const uint4 *>(rec + 64 + blk * 16));
                    e[it] = __ldg(rec + blk);
                }
                if (++f_kb == p.k_blocks) {
                    f_kb = 0;
                    f_tile += gridDim.x;
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
        for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
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
                    const int k_local = (r >> 3) * 32 + (blk >> 5) * 16 + (blk & 15);
                    const int n_local = (r & 7) * 32 + ((blk >> 4) & 1) * 16;
                    decode_block_to_operand<kBN / 64>(mant_cur[it], exp_cur[it], bst, k_local, n_local);
                }
                fence_async_smem();  // the tensor core reads shared memory through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_b[t]);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps 0-3
        uint32_t tile_iter = 0;
        for (uint32_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, tile_iter++) {
            const uint32_t m_blk = tile % p.m_tiles, n_blk = tile / p.m_tiles;
            const bool got = mbar_wait_bounded(acc_full, tile_iter & 1u, abort_flag, p.status, BUDA_DEVSTAT_GEMM_WAIT);
            if (!__all_sync(0xffffffffu, got)) break;  // the whole warp leaves together
            tc_fence_after();
#pragma unroll 1
            for (int h = 0; h < 2; h++) {
                const int64_t row = (int64_t)m_blk * kBM + h * 128 + warp * 32 + lane;
                const int64_t off = row * p.ldc + (int64_t)n_blk * kBN;
#pragma unroll 1
                for (int c = 0; c < kBN / 32; c++) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(h * kBN + c * 32), v);
                    if (row < p.M)
                        store_row32(v, p.C, p.n_dst, off + c * 32);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
        }
    }

    // every path ends here; the allocating warp frees tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

}  // namespace gemm

// Process-wide choice of matmul kernel: 0 auto, 1 single-CTA, 2 CTA pair, 3 CTA pair with the epilogue that stores
// from registers (the one the multicast route uses).  which < 0 only reads.
// Returns the previous value.
int gemm_kernel_choice(int which)
{
    static std::atomic<int> choice{0};
    const int cur = choice.load();
    if (which >= 0 && which <= 3) choice.store(which);
    return cur;
}

cudaError_t launch_bfp8b_gemm_pair(const CUtensorMap &tmap, const gemm::Params &p, const gemm::OutMaps &out_maps, int sm_count,
                                   cudaStream_t stream);

// C[d] (d < n_dst) all receive the product: C[0] on this device, the rest may be peers' memory mapped into
// this process (plain stores from the epilogue; nothing is read from a peer).
// C_mc (may be null): the multicast address of the same matrix on every device of an NVSwitch group; the pair
// kernel's epilogue then issues one multimem store per 16 bytes instead of one store per peer.
cudaError_t launch_bfp8b_gemm(const void *A, int64_t M, int64_t K, int64_t lda, const void *W, int64_t N, void *const *C, int n_dst,
                              void *C_mc, int64_t ldc, int sm_count, cudaStream_t stream, unsigned int *status, char *err,
                              size_t err_len)
{
    using namespace gemm;
    if (M <= 0 || N <= 0 || K <= 0 || (N % kBN) || (K % kBK)) {
        snprintf(err, err_len, "bfp8b gemm needs N %% %d == 0 and K %% %d == 0 (got M=%lld N=%lld K=%lld)", kBN, kBK, (long long)M,
                 (long long)N, (long long)K);
        return cudaErrorInvalidValue;
    }
    if (n_dst < 1 || n_dst > kMaxDst) {
        snprintf(err, err_len, "bfp8b gemm writes 1..%d destinations (got %d)", kMaxDst, n_dst);
        return cudaErrorInvalidValue;
    }
    bool aligned = !(reinterpret_cast<uintptr_t>(A) & 15) && !(reinterpret_cast<uintptr_t>(W) & 15);
    for (int d = 0; d < n_dst; d++) aligned = aligned && C[d] && !(reinterpret_cast<uintptr_t>(C[d]) & 15);
    if (lda < K || ldc < N || (lda % 8) || (ldc % 8) || !aligned) {
        snprintf(err, err_len, "bfp8b gemm needs 16-byte aligned A, W, C and row strides that are multiples of 8 elements");
        return cudaErrorInvalidValue;
    }
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) {
        snprintf(err, err_len, "cuTensorMapEncodeTiled is not available from this driver");
        return cudaErrorNotSupported;
    }
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)lda * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, 128};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(A), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        snprintf(err, err_len, "cuTensorMapEncodeTiled failed with code %d", (int)cr);
        return cudaErrorInvalidValue;
    }
    // Kernel choice: gemm_kernel_choice() (0 auto, 1 single-CTA, 2 CTA pair).  Auto gives the pair kernel every
    // problem with more than 256 rows (below that its 512-row tile would be mostly padding).
    const int forced = gemm_kernel_choice(-1);
    Params p;
    p.W = static_cast<const uint8_t *>(W);
    for (int d = 0; d < kMaxDst; d++) p.C[d] = d < n_dst ? static_cast<uint16_t *>(C[d]) : nullptr;
    p.n_dst = n_dst;
    p.C_mc = static_cast<uint16_t *>(C_mc);
    if (C_mc && (reinterpret_cast<uintptr_t>(C_mc) & 15)) {
        snprintf(err, err_len, "bfp8b gemm needs a 16-byte aligned multicast address");
        return cudaErrorInvalidValue;
    }
    p.M = M; p.N = N; p.K = K; p.ldc = ldc;
    p.m_tiles = (uint32_t)((M + kBM - 1) / kBM);
    p.n_tiles = (uint32_t)(N / kBN);
    p.k_blocks = (uint32_t)(K / kBK);
    p.Nt = (uint32_t)(N / 32);
    p.status = status;
    const bool use_pair = forced >= 2 || (forced == 0 && M > 256) || C_mc != nullptr;   // only the pair kernel forwards
    if (use_pair) {
        // Output tiles of a one-device launch leave the pair kernel as bulk tensor stores: 0.801 ms against 0.830 ms with
        // stores from registers on 8192 x 4096 x 16384 (alternating runs, same device).  A launch that also feeds
        // peers stores from registers and forwards with plain stores: bulk tensor stores into the peers' matrices
        // measured 0.428 ms against 0.405 ms at 4 GPUs.
        OutMaps out_maps = {};
        p.tma_epilogue = (C_mc == nullptr && forced != 3 && n_dst == 1) ? 1 : 0;
        if (p.tma_epilogue) {
            const cuuint64_t cdims[2] = {(cuuint64_t)N, (cuuint64_t)M};
            const cuuint64_t cstrides[1] = {(cuuint64_t)ldc * 2};
            const cuuint32_t cbox[2] = {64, 32};
            for (int d = 0; d < n_dst; d++) {
                cr = encode(&out_maps.m[d], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C[d], cdims, cstrides, cbox, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                if (cr != CUDA_SUCCESS) {
                    snprintf(err, err_len, "cuTensorMapEncodeTiled failed for output %d with code %d", d, (int)cr);
                    return cudaErrorInvalidValue;
                }
            }
        }
        return launch_bfp8b_gemm_pair(tmap, p, out_maps, sm_count, stream);
    }
    p.tma_epilogue = 0;

    static std::atomic<bool> attr_done[64];
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    if (!attr_done[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(bfp8b_gemm_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev].store(true, std::memory_order_release);
    }
    uint32_t grid = p.m_tiles * p.n_tiles;
    if (grid > (uint32_t)sm_count) grid = (uint32_t)sm_count;
    bfp8b_gemm_kernel<8><<<grid, threads_for<8>(), kSmemBytes, stream>>>(tmap, p);   // 8 decode warps measured faster than 16
    return cudaGetLastError();
}

}  // namespace buda
