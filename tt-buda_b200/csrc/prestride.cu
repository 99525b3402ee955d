// Prestride transform of a convolution activation, applied while it is pushed to a queue whose descriptor
// carries a StrideDescriptor (pybuda/pybuda/tensor.py:1415-1422 sets it; golden semantics
// pybuda/pybuda/op/eval/pybuda/tm.py:316-335, "no transpose in Prestride transform in BE tilize",
// tm.py:616): the [w, z, H, W] activation, H and W zero-padded up to multiples of the stride s, is cut
// into the s*s phase images act[:, :, y::s, x::s] (one per (x, y) offset of the descriptor, in its order),
// the phases are stacked along z, and each [H/s, W/s] image is flattened into one row:
//     out[w, 0, k*z + zc, hr*(W/s) + wc] = act[w, zc, hr*s + y_k, wc*s + x_k]
// The output is written dense and zero-padded to the queue's tile-aligned [rows, cols], ready for the
// tilize + pack kernels.  One thread per output element; a gather, bound by its strided reads.
#include "buda_common.cuh"

namespace buda {

constexpr int kMaxStrideOffsets = 64;

struct PrestrideJob {
    uint32_t W, Z, H, Wd;              // source dims
    uint64_t sw, sz, sh;               // source byte strides (innermost = element size)
    uint32_t s, n_off, Hs, Ws;         // stride, offsets, output image dims
    uint32_t rows, cols;               // destination rows / columns (>= n_off*Z, >= Hs*Ws)
    int16_t off_x[kMaxStrideOffsets], off_y[kMaxStrideOffsets];
};

template <typename T>
__global__ void __launch_bounds__(256) prestride_kernel(const __grid_constant__ PrestrideJob j, const uint8_t *__restrict__ src,
                                                        T *__restrict__ dst)
{
    const uint64_t per_entry = (uint64_t)j.rows * j.cols;
    const uint64_t total = per_entry * j.W;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t w = (uint32_t)(i / per_entry);
        const uint64_t rem = i - (uint64_t)w * per_entry;
        const uint32_t r = (uint32_t)(rem / j.cols), c = (uint32_t)(rem - (uint64_t)r * j.cols);
        T v = 0;
        if (r < j.n_off * j.Z && c < j.Hs * j.Ws) {
            const uint32_t k = r / j.Z, zc = r - k * j.Z;
            const uint32_t hr = c / j.Ws, wc = c - hr * j.Ws;
            const uint32_t y = hr * j.s + (uint32_t)j.off_y[k], x = wc * j.s + (uint32_t)j.off_x[k];
            if (y < j.H && x < j.Wd)
                v = *reinterpret_cast<const T *>(src + (uint64_t)w * j.sw + (uint64_t)zc * j.sz + (uint64_t)y * j.sh + (uint64_t)x * sizeof(T));
        }
        dst[i] = v;
    }
}

cudaError_t launch_prestride(const void *src, int elem_bytes, const uint32_t shape[4], const uint64_t strides[4], int stride,
                             const int *xy_offsets, int n_offsets, void *dst, uint32_t dst_rows, uint32_t dst_cols, int sm_count,
                             cudaStream_t stream)
{
    PrestrideJob j;
    j.W = shape[0]; j.Z = shape[1]; j.H = shape[2]; j.Wd = shape[3];
    j.sw = strides[0]; j.sz = strides[1]; j.sh = strides[2];
    j.s = (uint32_t)stride;
    j.n_off = (uint32_t)n_offsets;
    j.Hs = (j.H + j.s - 1) / j.s;
    j.Ws = (j.Wd + j.s - 1) / j.s;
    j.rows = dst_rows; j.cols = dst_cols;
    for (int k = 0; k < kMaxStrideOffsets; k++) {
        j.off_x[k] = k < n_offsets ? (int16_t)xy_offsets[2 * k] : 0;
        j.off_y[k] = k < n_offsets ? (int16_t)xy_offsets[2 * k + 1] : 0;
    }
    const uint64_t total = (uint64_t)j.W * dst_rows * dst_cols;
    uint64_t blocks = (total + 255) / 256;
    const uint64_t cap = (uint64_t)sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) return cudaSuccess;
    const uint8_t *s8 = static_cast<const uint8_t *>(src);
    if (elem_bytes == 4) prestride_kernel<uint32_t><<<(unsigned)blocks, 256, 0, stream>>>(j, s8, static_cast<uint32_t *>(dst));
    else if (elem_bytes == 2) prestride_kernel<uint16_t><<<(unsigned)blocks, 256, 0, stream>>>(j, s8, static_cast<uint16_t *>(dst));
    else if (elem_bytes == 1) prestride_kernel<uint8_t><<<(unsigned)blocks, 256, 0, stream>>>(j, s8, static_cast<uint8_t *>(dst));
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace buda
