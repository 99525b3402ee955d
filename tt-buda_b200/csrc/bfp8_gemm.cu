// placeholder until the tcgen05 kernel lands
#include <cstdio>
#include "buda_common.cuh"
namespace buda {
cudaError_t launch_bfp8b_gemm(const void *, int64_t, int64_t, int64_t, const void *, int64_t, void *, int64_t, int,
                              cudaStream_t, unsigned int *, char *err, size_t err_len)
{
    snprintf(err, err_len, "bfp8b gemm kernel not built");
    return cudaErrorNotSupported;
}
}  // namespace buda
