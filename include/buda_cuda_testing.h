/*
 * buda_cuda_testing.h -- hooks of libbuda_cuda.so that exist for its tests and measurements.  They are NOT part of
 * the drop-in interface (include/buda_cuda.h): nothing in the reference corresponds to them and a host layer never
 * needs them.  Same conventions as buda_cuda.h.
 */
#ifndef BUDA_CUDA_TESTING_H
#define BUDA_CUDA_TESTING_H

#include "buda_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* buda_tilize_pack_batch / buda_unpack_untilize_batch with the kernel chosen by the caller: path 0 = staged
 * (shared-memory staging by bulk async copies; needs 16-byte aligned rows), 1 = direct (4 lanes per block, warp
 * shuffle exponent reduction; any alignment).  The library picks by alignment; the tests run both on the same input
 * and the bench times one against the other. */
int buda_tilize_pack_batch_path(int n, const void *const *srcs_host, int src_df, const uint32_t shape[4],
                                const uint64_t strides_bytes[4], const buda_queue_geom *geom, int dst_df,
                                int with_header, void *const *dsts_host, uint64_t dst_bytes_each, void *stream,
                                int path);
int buda_unpack_untilize_batch_path(int n, const void *const *srcs_host, int src_df, int with_header,
                                    const buda_queue_geom *geom, void *const *dsts_host, int dst_df,
                                    const uint32_t shape[4], const uint64_t strides_bytes[4], void *stream,
                                    int path);

/* Which tensor-core kernel buda_bfp8b_gemm* launches: 0 = automatic (CTA-pair kernel for M > 256, single-CTA
 * kernel otherwise), 1 = single-CTA, 2 = CTA pair, 3 = CTA pair with the epilogue that stores from registers
 * instead of through bulk tensor stores (also honoured by buda_i8_gemm).  Process-wide; a negative value only
 * reads.  Returns the previous setting.  All of them give identical bits; the tests check that. */
int buda_gemm_select_kernel(int which);

/* Self-test of the failure path every kernel of the library shares: launches one CTA that waits, with the
 * library's bounded mbarrier wait, for a barrier phase that nothing completes, for at most limit_ms
 * (1..1000) milliseconds; the wait then gives up, records BUDA_DEVSTAT_SELFTEST_WAIT in the device status word
 * and the kernel returns normally.  Nothing faults, traps or spins without a limit; the context stays usable.
 * buda_device_status() afterwards returns BUDA_TIMEOUT_ERROR with that code, once. */
int buda_selftest_bounded_wait(uint32_t limit_ms, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* BUDA_CUDA_TESTING_H */
