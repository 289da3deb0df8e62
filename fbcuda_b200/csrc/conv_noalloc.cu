// updateOutput for callers that cannot allocate device memory.
//
// fbfft_b200_conv_update_output() needs a workspace for its spectra, and its
// callers normally get one from cudaMalloc or a framework allocator.  Some
// callers cannot: code running where the allocator must not be entered (a plugin
// called while its host framework holds the allocator lock, a real-time loop with
// a no-allocation rule after start-up, a process whose memory pool is already
// handed out in full to another library).  For them this file keeps one fixed
// scratch area inside the library image itself and runs the same pass on it.
//
// Has no counterpart in the reference.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/fbfft_b200.h"
#include "common.cuh"

namespace {

// Lives in every GPU context that loads the library, from load until exit.
static __device__ __align__(256) unsigned char g_noalloc_scratch[FBFFT_B200_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_addr[kMaxDevices];  // device address of g_noalloc_scratch, per device
bool g_have_addr[kMaxDevices];

// The array's name is only a host-side handle; kernels need its device address,
// which differs per device.  Looked up once per device, with that device current.
int scratch_for_current_device(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fbfft_b200::set_last_error("conv_update_output_noalloc: cannot identify the current device");
    return FBFFT_CUDA_ERROR;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_have_addr[dev]) {
    void* p = nullptr;
    const cudaError_t rc = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (rc != cudaSuccess || p == nullptr) {
      fbfft_b200::set_last_error("conv_update_output_noalloc: cudaGetSymbolAddress failed for the scratch area");
      return FBFFT_CUDA_ERROR;
    }
    g_scratch_addr[dev] = p;
    g_have_addr[dev] = true;
  }
  *out = g_scratch_addr[dev];
  return FBFFT_SUCCESS;
}

}  // namespace

extern "C" int fbfft_b200_conv_update_output_noalloc(int fft_size, const float* in, const int* in_size,
                                                     const int* in_stride, int in_padL, int in_padU,
                                                     const float* weight, const int* w_size, const int* w_stride,
                                                     float* out, const int* out_size, const int* out_stride,
                                                     int out_padL, int out_padU, void* stream) {
  if (!in_size || !w_size || !out_size || !in_stride || !w_stride || !out_stride) {
    fbfft_b200::set_last_error("null argument");
    return FBFFT_UNSUPPORTED_DIMENSION;
  }
  if (!(fft_size == 8 || fft_size == 16 || fft_size == 32 || fft_size == 64 || fft_size == 128)) {
    fbfft_b200::set_last_error("conv_update_output_noalloc: transform size must be 8, 16, 32, 64 or 128");
    return FBFFT_UNSUPPORTED_SIZE;
  }
  const size_t need = fbfft_b200_conv_workspace_bytes(fft_size, in_size[0], in_size[1], w_size[0]);
  if (need > (size_t)FBFFT_B200_NOALLOC_SCRATCH_BYTES) {
    fbfft_b200::set_last_error(
        "conv_update_output_noalloc: this layer needs more spectrum scratch than the built-in "
        "FBFFT_B200_NOALLOC_SCRATCH_BYTES; use fbfft_b200_conv_update_output with a caller-owned workspace");
    return FBFFT_UNSUPPORTED_SIZE;
  }
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != FBFFT_SUCCESS) return rc;
  // Every region of the scratch that the pass reads is written earlier in the same
  // call (the two forward transforms, then the non-accumulating contraction), so
  // nothing left behind by the previous call needs clearing.
  return fbfft_b200_conv_update_output(fft_size, in, in_size, in_stride, in_padL, in_padU, weight, w_size, w_stride,
                                       out, out_size, out_stride, out_padL, out_padU, scratch,
                                       (size_t)FBFFT_B200_NOALLOC_SCRATCH_BYTES, 0, stream);
}
