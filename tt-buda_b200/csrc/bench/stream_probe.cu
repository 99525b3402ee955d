// Bare streaming kernels with the access shapes of the conversion kernels and none of their arithmetic: what the
// memory system gives for a read : write mix, against which the real kernels are judged (the measured "copy" peak is
// a 1 : 1 stream; a tilize + pack reads 4 bytes for each one it writes, an unpack + untilize the other way round).
//
// A band is 32 rows x 1 KiB inside rows of 16 KiB (what a staged work item touches on the row-major side); the other
// side of a band is contiguous.  A block of 256 threads moves one band at a time: 8 warps x 4 rows, a warp
// instruction covers 512 contiguous bytes of a row.
//
// Built into its own small library (libbuda_probe.so) that only bench.py loads: a measurement aid, not part of the
// conversion library or its interface.
#include <cuda_runtime.h>
#include <stdint.h>

namespace buda {

constexpr int kProbeRow = 16384;     // bytes between two rows of the banded side
constexpr int kProbePiece = 1024;    // bytes of a row inside one band
constexpr int kProbePieces = kProbeRow / kProbePiece;

// which band a block takes next: 0 = its own only (one short-lived block per band), 1 = fixed stride over the grid,
// 2 = next value of a device counter
struct ProbeSched {
    unsigned long long *counter;
    int mode;
};

__device__ __forceinline__ size_t probe_first_band(const ProbeSched &s, unsigned long long *slot)
{
    if (s.mode != 2) return blockIdx.x;
    if (threadIdx.x == 0) *slot = atomicAdd(s.counter, 1ull);
    __syncthreads();
    return (size_t)*slot;
}

__device__ __forceinline__ size_t probe_next_band(const ProbeSched &s, size_t b, size_t nbands, unsigned long long *slot)
{
    if (s.mode == 0) return nbands;
    if (s.mode == 1) return b + gridDim.x;
    __syncthreads();
    if (threadIdx.x == 0) *slot = atomicAdd(s.counter, 1ull);
    __syncthreads();
    return (size_t)*slot;
}

// MIX 0: 4 bytes read (banded) : 1 byte written (contiguous).  MIX 1: 1 byte read (contiguous) : 4 bytes written
// (banded).  MIX 2: banded reads only.  MIX 3: banded writes only.
template <int MIX>
__global__ void __launch_bounds__(256)
stream_probe_kernel(const uint8_t *__restrict__ narrow_in, uint8_t *__restrict__ narrow_out, const float *__restrict__ wide_in,
                    float *__restrict__ wide_out, size_t nbands, ProbeSched sched, float *sink)
{
    __shared__ unsigned long long slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float acc = 0.0f;
    for (size_t b = probe_first_band(sched, &slot); b < nbands; b = probe_next_band(sched, b, nbands, &slot)) {
        const size_t wide_off = (b / kProbePieces) * 32 * (size_t)kProbeRow + (b % kProbePieces) * kProbePiece;   // bytes
        const size_t narrow_off = b * (size_t)(32 * kProbePiece / 4);                                             // bytes
        if (MIX == 0 || MIX == 2) {
            float4 v[8];
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < 2; c++)
                    v[r * 2 + c] = *reinterpret_cast<const float4 *>(reinterpret_cast<const char *>(wide_in) + wide_off +
                                                                     (size_t)(warp * 4 + r) * kProbeRow + c * 512 + lane * 16);
#pragma unroll
            for (int k = 0; k < 8; k++) {
                if (MIX == 0) {
                    const uint32_t w = ((uint32_t)(int)v[k].x & 0xffu) | (((uint32_t)(int)v[k].y & 0xffu) << 8) |
                                       (((uint32_t)(int)v[k].z & 0xffu) << 16) | ((uint32_t)(int)v[k].w << 24);
                    reinterpret_cast<uint32_t *>(narrow_out + narrow_off)[(warp * 8 + k) * 32 + lane] = w;
                } else {
                    acc += v[k].x + v[k].y + v[k].z + v[k].w;
                }
            }
        } else {
#pragma unroll
            for (int r = 0; r < 4; r++) {
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t w = 0x01020304u;
                    if (MIX == 1)
                        w = reinterpret_cast<const uint32_t *>(narrow_in + narrow_off)[((warp * 4 + r) * 2 + c) * 32 + lane];
                    const float4 v = make_float4((float)(int8_t)w, (float)(int8_t)(w >> 8), (float)(int8_t)(w >> 16),
                                                 (float)(int8_t)(w >> 24));
                    *reinterpret_cast<float4 *>(reinterpret_cast<char *>(wide_out) + wide_off +
                                                (size_t)(warp * 4 + r) * kProbeRow + c * 512 + lane * 16) = v;
                }
            }
        }
    }
    if (MIX == 2 && acc == 123.456f) *sink = acc;   // keeps the loads alive
}

template <int MIX>
static cudaError_t probe_launch(const uint8_t *narrow, uint8_t *narrow_w, const float *wide, float *wide_w, size_t nbands,
                                int schedule, int sm_count, unsigned long long *counter, float *sink, cudaStream_t stream)
{
    ProbeSched sched{counter, schedule};
    if (schedule == 2) {
        cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(unsigned long long), stream);
        if (e != cudaSuccess) return e;
    }
    const size_t resident = (size_t)sm_count * 8;
    const unsigned grid = (unsigned)(schedule == 0 ? nbands : (nbands < resident ? nbands : resident));
    stream_probe_kernel<MIX><<<grid, 256, 0, stream>>>(narrow, narrow_w, wide, wide_w, nbands, sched, sink);
    return cudaGetLastError();
}

// elements: a multiple of 131072 (32 rows of 4096 four-byte elements).  Allocates elements * 5 bytes for the run.
cudaError_t run_stream_probe(int mix, int schedule, uint64_t elements, int reps, int sm_count, cudaStream_t stream, float *ms_out)
{
    uint8_t *narrow = nullptr;
    float *wide = nullptr;
    unsigned long long *counter = nullptr;
    cudaEvent_t a = nullptr, b = nullptr;
    cudaError_t e = cudaMalloc(&narrow, elements);
    if (e == cudaSuccess) e = cudaMalloc(&wide, elements * 4);
    if (e == cudaSuccess) e = cudaMalloc(&counter, 16);
    if (e == cudaSuccess) e = cudaMemsetAsync(narrow, 1, elements, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(wide, 0, elements * 4, stream);
    if (e == cudaSuccess) e = cudaEventCreate(&a);
    if (e == cudaSuccess) e = cudaEventCreate(&b);
    const size_t nbands = (size_t)(elements * 4 / (32 * kProbePiece));
    float *sink = reinterpret_cast<float *>(counter + 1);
    for (int i = 0; i < 2 + reps && e == cudaSuccess; i++) {
        if (i == 2) e = cudaEventRecord(a, stream);
        if (e != cudaSuccess) break;
        switch (mix) {
            case 0: e = probe_launch<0>(narrow, narrow, wide, wide, nbands, schedule, sm_count, counter, sink, stream); break;
            case 1: e = probe_launch<1>(narrow, narrow, wide, wide, nbands, schedule, sm_count, counter, sink, stream); break;
            case 2: e = probe_launch<2>(narrow, narrow, wide, wide, nbands, schedule, sm_count, counter, sink, stream); break;
            default: e = probe_launch<3>(narrow, narrow, wide, wide, nbands, schedule, sm_count, counter, sink, stream); break;
        }
    }
    if (e == cudaSuccess) e = cudaEventRecord(b, stream);
    if (e == cudaSuccess) e = cudaEventSynchronize(b);
    float ms = 0.0f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, a, b);
    if (e == cudaSuccess) *ms_out = ms / (float)reps;
    if (a) cudaEventDestroy(a);
    if (b) cudaEventDestroy(b);
    cudaFree(counter);
    cudaFree(wide);
    cudaFree(narrow);
    return e;
}

// A block of `rows` rows x row_bytes (a multiple of 512) read from src and stored to the same place in up to 7 other
// matrices of the same pitch (peers' memory mapped into this process): the traffic of the column-parallel matmul's
// exchange with none of its arithmetic.  A warp instruction covers 512 contiguous bytes of a row; nothing is read from a peer.
struct PeerDsts {
    uint8_t *p[7];
    int n;
};

__global__ void __launch_bounds__(256)
peer_store_probe_kernel(const uint8_t *__restrict__ src, PeerDsts dsts, uint32_t rows, uint32_t row_bytes, uint64_t pitch)
{
    const uint32_t pieces_per_row = row_bytes / 512u;
    const uint64_t pieces = (uint64_t)rows * pieces_per_row;
    const int lane = threadIdx.x & 31;
    const uint64_t warps = (uint64_t)gridDim.x * 8u;
    for (uint64_t w = (uint64_t)blockIdx.x * 8u + (threadIdx.x >> 5); w < pieces; w += warps) {
        const uint64_t off = (w / pieces_per_row) * pitch + (w % pieces_per_row) * 512u + (uint64_t)lane * 16u;
        const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(src + off));
        for (int d = 0; d < dsts.n; d++) *reinterpret_cast<uint4 *>(dsts.p[d] + off) = v;
    }
}

}  // namespace buda

// One launch of the peer-store probe on `stream` (no synchronisation: the caller times a series of launches with its own
// events, on every rank at once).  src and every dsts[i] are 16-byte aligned device addresses valid in this process;
// row_bytes is a multiple of 512, pitch_bytes of 16.  Returns 0, or 1 for bad arguments / a launch error.
extern "C" int buda_probe_peer_stores(const void *src, void *const *dsts, int n_dsts, uint32_t rows, uint32_t row_bytes,
                                      uint64_t pitch_bytes, void *stream)
{
    if (!src || !dsts || n_dsts < 1 || n_dsts > 7 || rows == 0 || row_bytes == 0 || row_bytes % 512u || pitch_bytes % 16u ||
        pitch_bytes < row_bytes || ((uintptr_t)src & 15u))
        return 1;
    buda::PeerDsts d = {};
    d.n = n_dsts;
    for (int i = 0; i < n_dsts; i++) {
        if (!dsts[i] || ((uintptr_t)dsts[i] & 15u)) return 1;
        d.p[i] = static_cast<uint8_t *>(dsts[i]);
    }
    int dev = 0, sm_count = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 1;
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 1;
    buda::peer_store_probe_kernel<<<(unsigned)(sm_count * 8), 256, 0, (cudaStream_t)stream>>>(static_cast<const uint8_t *>(src), d, rows,
                                                                                              row_bytes, pitch_bytes);
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// mix: 0 = 4 bytes read per byte written (tilize + pack, quantise), 1 = 1 byte read per 4 written (unpack + untilize,
// dequantise), 2 = reads only, 3 = writes only.  schedule: 0 = one short-lived block per band, 1 = resident blocks on
// a fixed stride, 2 = resident blocks that take bands in address order from a device counter.  elements: a multiple
// of 131072, at most 2^30; 5 bytes per element are allocated on the current device for the run and freed.  Runs 2
// untimed and `reps` (1..1000) timed launches on `stream`, synchronises, and stores the mean milliseconds per launch
// in *ms_out.  Returns 0, or 1 for bad arguments / a CUDA error.
extern "C" int buda_probe_stream(int mix, int schedule, uint64_t elements, int reps, float *ms_out, void *stream)
{
    if (!ms_out || mix < 0 || mix > 3 || schedule < 0 || schedule > 2 || reps < 1 || reps > 1000) return 1;
    if (elements == 0 || elements % 131072u || elements > (1ull << 30)) return 1;
    int dev = 0, sm_count = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 1;
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 1;
    return buda::run_stream_probe(mix, schedule, elements, reps, sm_count, (cudaStream_t)stream, ms_out) == cudaSuccess ? 0 : 1;
}
