// Measures what the tensor pipe sustains for the MMA shape the contraction issues: every SM runs
// one block whose single issuing lane streams tcgen05.mma.kind::tf32 (M = 128, N = n_cols, K = 8)
// over operand tiles that sit in shared memory, exactly as cgemm_tma.cu issues them, with no
// loads, no split and no epilogue.  The rate is the tensor-peak denominator the convolution
// roofline is quoted against (no counterpart in the reference, which has no tensor-core code).
#include <cuda_runtime.h>

#include "fft2d_small.cuh"  // mbarrier helpers, the bounded wait, the device status word
#include "kernels.h"

namespace fbfft_b200 {

namespace {

constexpr int kErrPeakWait = 902;
constexpr int kPeakSmem = 200 * 1024;  // one block per SM

__device__ __forceinline__ unsigned long long peak_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
  return (unsigned long long)((addr >> 4) & 0x3FFF) | ((unsigned long long)((lbo_bytes >> 4) & 0x3FFF) << 16) |
         ((unsigned long long)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ULL << 46);
}

__global__ void __launch_bounds__(128, 1) tf32_peak_kernel(int n_cols, int batches, int per_batch) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bar_mem;
  __shared__ unsigned tmem_slot;
  // operand tiles: A 128 x 8 and B n_cols x 8 tf32 values, K-major core matrices, all zero
  for (int i = threadIdx.x; i < (128 * 8 + 256 * 8); i += blockDim.x) reinterpret_cast<float*>(smem)[i] = 0.0f;
  const unsigned bar = smem_u32(&bar_mem);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    fence_async_smem();
  }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = tmem_slot;
  if (threadIdx.x == 0) {
    const unsigned a_addr = smem_u32(smem), b_addr = a_addr + 128 * 8 * 4;
    const unsigned long long da = peak_desc(a_addr, (128 / 8) * 128, 128);
    const unsigned long long db = peak_desc(b_addr, (unsigned)(n_cols / 8) * 128, 128);
    // D fp32, A and B tf32, both K-major, M = 128, N = n_cols
    const unsigned idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(n_cols >> 3) << 17) | ((128u >> 4) << 24);
    unsigned phase = 0;
    for (int b = 0; b < batches; ++b) {
      for (int i = 0; i < per_batch; ++i) {
        // two accumulators in turn, so that consecutive products do not serialise on one
        const unsigned d = tmem_base + ((i & 1) ? 256u : 0u);
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(d),
            "l"(da), "l"(db), "r"(idesc), "r"(1u), "r"(0), "r"(0), "r"(0), "r"(0)
            : "memory");
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
      if (!mbar_wait(bar, phase, kErrPeakWait)) break;
      phase ^= 1;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
  }
}

}  // namespace

int measure_tf32_peak(int n_cols, double* tflops) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(tf32_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem);
    configured[dev] = true;
  }
  const int grid = sm_count(), batches = 64, per_batch = 256;
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return kCudaError;
  float best_ms = 0.0f;
  bool ok = true;
  for (int rep = 0; rep < 4 && ok; ++rep) {  // the first launch warms up
    cudaEventRecord(e0, 0);
    tf32_peak_kernel<<<grid, 128, kPeakSmem, 0>>>(n_cols, batches, per_batch);
    cudaEventRecord(e1, 0);
    ok = cudaPeekAtLastError() == cudaSuccess && cudaEventSynchronize(e1) == cudaSuccess;
    float ms = 0.0f;
    if (ok) cudaEventElapsedTime(&ms, e0, e1);
    if (rep > 0 && (best_ms == 0.0f || ms < best_ms)) best_ms = ms;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (!ok || best_ms <= 0.0f) return kCudaError;
  const double flops = 2.0 * 128.0 * n_cols * 8.0 * (double)batches * per_batch * grid;
  *tflops = flops / (best_ms * 1e-3) / 1e12;
  return kSuccess;
}

int read_device_error_peak() { return device_error_word_read(); }
int clear_device_error_peak() { return device_error_word_clear(); }

}  // namespace fbfft_b200
