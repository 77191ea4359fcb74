// Measurement and self-test helpers, built into libcvm_measure.so (NOT into the runtime library):
//   - the int8 tensor-core rate of this GPU, measured the way the convolution kernel uses the
//     tensor cores: one CTA per SM issues `reps` tcgen05.mma.cta_group::1.kind::i8 instructions
//     (M = 128, N = n, K = 32, operands resident in shared memory, one accumulator) from one
//     thread and waits for their completion; the time is taken with CUDA events around the launch;
//   - a kernel whose only job is to let one of the bounded waits the tensor-core kernels are built
//     from run out, so that a test can see the wait give up and report instead of hanging.
#include <stdio.h>
#include <string.h>
#include "cvmk_measure.h"
#include "tc_common.cuh"

namespace cvmk {
namespace {

using namespace tc;

thread_local char g_measure_err[256] = {0};
int fail(int code, const char* what, cudaError_t e = cudaSuccess) {
  snprintf(g_measure_err, sizeof(g_measure_err), "%s%s%s", what, e != cudaSuccess ? ": " : "",
           e != cudaSuccess ? cudaGetErrorString(e) : "");
  return code;
}

// row_bytes: row length of the A tile (128, 64 or 32: its swizzle); a_offset: bytes from the tile's
// (1024-byte aligned) start to the first row the instruction reads; group_stride: bytes from one
// 8-row group of A to the next.  (128, 0, 1024) is a dense K-major tile; a window of a staged input
// halo, as the 3 x 3 halo mode of the convolution kernel reads it, starts some rows in and steps
// one halo row (10 pixels) per group.
__global__ void __launch_bounds__(128) mma_rate_kernel(int n, int reps, int* status, int row_bytes, int a_offset,
                                                       int group_stride) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  __shared__ volatile int abort_flag;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  for (int i = threadIdx.x; i < (BLOCK_M + 256) * 128 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x01010101u;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  fence_async_smem();
  if (threadIdx.x < 32) tmem_alloc(&slot, 256u);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = umma_idesc_i8(n);
    uint64_t da = umma_desc(smem_u32(smem) + (uint32_t)a_offset, row_bytes);
    da = (da & ~((uint64_t)0x3FFF << 32)) | ((uint64_t)((uint32_t)group_stride >> 4) << 32);
    const uint64_t db = umma_desc(smem_u32(smem + BLOCK_M * 128), row_bytes);
    const int kmask = row_bytes / 32 - 1;
    for (int i = 0; i < reps; ++i) {
      const uint64_t koff = (uint64_t)(2 * (i & kmask));
      mma_i8(tmem, da + koff, db + koff, idesc, 1u);
    }
    mma_commit(&bar);
    if (!mbar_wait(&bar, 0u, &abort_flag, 1)) atomicOr(status, 0x400);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tmem_dealloc(tmem, 256u);
  }
}


// One thread waits on an mbarrier that nothing ever arrives at, with the same bounded wait the
// convolution kernels use but `limit` polls (about 2 us each) instead of about a second.  The wait
// gives up, raises the CTA's abort flag and the kernel ORs 0x100 | code into *status -- exactly what
// a starved role of conv_tc_kernel does -- and returns normally: no trap, no hang.
__global__ void wait_timeout_kernel(uint32_t limit, int* status, long long* waited_clocks) {
  __shared__ uint64_t bar;
  __shared__ volatile int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const long long t0 = clock64();
    const bool ok = mbar_wait(&bar, 0u, &abort_flag, 5, limit);
    *waited_clocks = clock64() - t0;
    if (!ok && abort_flag) atomicOr(status, 0x100 | abort_flag);
  }
}

}  // namespace
}  // namespace cvmk

using namespace cvmk;

extern "C" const char* cvmk_measure_last_error(void) { return g_measure_err; }

// tops: 2 * multiply-accumulates per second / 1e12 over all SMs.  n: 32..256 (multiple of 16).
extern "C" int cvmk_measure_i8_mma_rate(int n, int reps, double* tops) {
  return cvmk_measure_i8_mma_rate_window(n, reps, 128, 0, 8, tops);
}

extern "C" int cvmk_measure_i8_mma_rate_window(int n, int reps, int row_bytes, int a_offset_rows, int group_stride_rows,
                                               double* tops) {
  if (!tops || n < 32 || n > 256 || n % 16 || reps < 1) return fail(CVMK_ERR_ARG, "measure_i8_mma_rate: bad argument");
  if ((row_bytes != 128 && row_bytes != 64 && row_bytes != 32) || a_offset_rows < 0 || a_offset_rows > 32 ||
      group_stride_rows < 8 || group_stride_rows > 16)
    return fail(CVMK_ERR_ARG, "measure_i8_mma_rate_window: row_bytes 32/64/128, offset 0..32 rows, group stride 8..16 rows");
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int* status = nullptr;
  cudaError_t e = cudaMalloc(&status, 4);
  if (e != cudaSuccess) return fail(CVMK_ERR_CUDA, "cudaMalloc", e);
  cudaMemset(status, 0, 4);
  const int smem = (BLOCK_M + 256) * 128 + 1024;
  e = cudaFuncSetAttribute(mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) { cudaFree(status); return fail(CVMK_ERR_CUDA, "cudaFuncSetAttribute", e); }
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  // (the window stays inside the (128 + 256) x 128 bytes the kernel fills: 32 + 15 * 16 + 8 rows at most)
  const int a_off = a_offset_rows * row_bytes, gstride = group_stride_rows * row_bytes;
  mma_rate_kernel<<<sms, 128, smem>>>(n, reps / 10 + 1, status, row_bytes, a_off, gstride);  // warm-up
  cudaEventRecord(e0);
  mma_rate_kernel<<<sms, 128, smem>>>(n, reps, status, row_bytes, a_off, gstride);
  cudaEventRecord(e1);
  cudaError_t err = cudaEventSynchronize(e1);
  float ms = 0;
  cudaEventElapsedTime(&ms, e0, e1);
  int hs = 0;
  cudaMemcpy(&hs, status, 4, cudaMemcpyDeviceToHost);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(status);
  if (err != cudaSuccess || hs != 0) return fail(CVMK_ERR_CUDA, "measure_i8_mma_rate: kernel did not complete", err);
  *tops = 2.0 * (double)sms * reps * BLOCK_M * n * 32.0 / (ms * 1e-3) / 1e12;
  return CVMK_OK;
}

extern "C" int cvmk_measure_wait_timeout(unsigned limit, int* status_word, long long* waited_clocks) {
  if (!status_word || !waited_clocks || limit == 0 || limit > (1u << 16))
    return fail(CVMK_ERR_ARG, "measure_wait_timeout: bad argument (limit 1..65536 polls)");
  int* dstatus = nullptr;
  long long* dclk = nullptr;
  cudaError_t e = cudaMalloc(&dstatus, 4);
  if (e == cudaSuccess) e = cudaMalloc(&dclk, 8);
  if (e != cudaSuccess) { cudaFree(dstatus); return fail(CVMK_ERR_CUDA, "cudaMalloc", e); }
  cudaMemset(dstatus, 0, 4);
  cudaMemset(dclk, 0, 8);
  wait_timeout_kernel<<<1, 32>>>(limit, dstatus, dclk);
  e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(status_word, dstatus, 4, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemcpy(waited_clocks, dclk, 8, cudaMemcpyDeviceToHost);
  cudaFree(dstatus);
  cudaFree(dclk);
  return e == cudaSuccess ? CVMK_OK : fail(CVMK_ERR_CUDA, "measure_wait_timeout", e);
}
