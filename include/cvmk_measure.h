/*
 * Measurement and self-test helpers (libcvm_measure.so).  None of them has a counterpart in the
 * reference and none is part of the runtime library: benchmarks and tests load this library beside
 * libcvm_runtime.so.  Status codes are those of cvmk_kernels.h (CVMK_OK = 0).
 */
#ifndef CVMK_MEASURE_H_
#define CVMK_MEASURE_H_

#include "cvmk_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

/* The int8 tensor-core rate of the current GPU in TOP/s (2 * MACs), measured by issuing `reps`
 * tcgen05.mma kind::i8 instructions of shape M = 128, N = n, K = 32 per SM on operands resident in
 * shared memory and timing the launch with CUDA events.  bench.py uses n = 256 as the denominator of
 * the tensor roofline. */
CVMK_API int cvmk_measure_i8_mma_rate(int n, int reps, double* tops);

/* The same with the A operand read the way the 3 x 3 halo mode of the convolution kernel reads it:
 * rows of `row_bytes` bytes (32, 64 or 128, with the matching swizzle), the first row
 * `a_offset_rows` rows after the tile's 1024-byte aligned start, 8-row groups `group_stride_rows`
 * rows apart (8 = a dense tile).  Shows what a window that straddles swizzle atoms costs. */
CVMK_API int cvmk_measure_i8_mma_rate_window(int n, int reps, int row_bytes, int a_offset_rows, int group_stride_rows,
                                             double* tops);

/* Lets a bounded device-side wait run out on purpose: one thread waits, with the wait the
 * tensor-core kernels use, on an mbarrier that nothing arrives at, for `limit` polls of about 2 us
 * (1..65536).  The wait gives up, the kernel returns normally and *status_word receives what a
 * convolution kernel would have ORed into its status word (0x100 | role code); *waited_clocks the
 * SM clocks the wait lasted. */
CVMK_API int cvmk_measure_wait_timeout(unsigned limit, int* status_word, long long* waited_clocks);

/* Text of the last error of this library on this thread. */
CVMK_API const char* cvmk_measure_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* CVMK_MEASURE_H_ */
