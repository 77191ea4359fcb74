// Measurement helper: the int8 tensor-core rate of this GPU, measured the way the convolution
// kernel uses it.  One CTA per SM issues `reps` tcgen05.mma.cta_group::1.kind::i8 instructions
// (M = 128, N = n, K = 32, operands resident in shared memory, one accumulator) from one thread and
// waits for their completion; the time is taken with CUDA events around the launch.
#include <string.h>
#include "tc_common.cuh"

namespace cvmk {
namespace {

using namespace tc;

__global__ void __launch_bounds__(128) mma_rate_kernel(int n, int reps, int* status) {
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
    const uint64_t da = umma_desc(smem_u32(smem), 128), db = umma_desc(smem_u32(smem + BLOCK_M * 128), 128);
    for (int i = 0; i < reps; ++i) {
      const uint64_t koff = (uint64_t)(2 * (i & 3));
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

}  // namespace
}  // namespace cvmk

using namespace cvmk;

// tops: 2 * multiply-accumulates per second / 1e12 over all SMs.  n: 32..256 (multiple of 16).
extern "C" int cvmk_measure_i8_mma_rate(int n, int reps, double* tops) {
  if (!tops || n < 32 || n > 256 || n % 16 || reps < 1) { set_error("measure_i8_mma_rate: bad argument"); return CVMK_ERR_ARG; }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int* status = nullptr;
  if (check_cuda(cudaMalloc(&status, 4), "cudaMalloc")) return CVMK_ERR_CUDA;
  cudaMemset(status, 0, 4);
  const int smem = (BLOCK_M + 256) * 128 + 1024;
  if (check_cuda(cudaFuncSetAttribute(mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "cudaFuncSetAttribute")) {
    cudaFree(status);
    return CVMK_ERR_CUDA;
  }
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  mma_rate_kernel<<<sms, 128, smem>>>(n, reps / 10 + 1, status);  // warm-up
  cudaEventRecord(e0);
  mma_rate_kernel<<<sms, 128, smem>>>(n, reps, status);
  cudaEventRecord(e1);
  cudaError_t err = cudaEventSynchronize(e1);
  float ms = 0;
  cudaEventElapsedTime(&ms, e0, e1);
  int hs = 0;
  cudaMemcpy(&hs, status, 4, cudaMemcpyDeviceToHost);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(status);
  if (err != cudaSuccess || hs != 0) { set_error("measure_i8_mma_rate: kernel did not complete (%s, status 0x%x)", cudaGetErrorString(err), hs); return CVMK_ERR_CUDA; }
  *tops = 2.0 * (double)sms * reps * BLOCK_M * n * 32.0 / (ms * 1e-3) / 1e12;
  return CVMK_OK;
}
