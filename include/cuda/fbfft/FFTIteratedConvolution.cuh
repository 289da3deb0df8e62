// The reference's tile-list convolution entry point (fbfft/FFTIteratedConvolution.cuh:70-95,
// 616-632), forwarding to libfbfft_b200.so.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

#include "cuda/DeviceTensor.cuh"
#include "fbfft_b200.h"

namespace facebook { namespace cuda { namespace fbfft { namespace detail {

// padL, padU, then the tensor: the reference's field order, equal to fbfft_tiled_tensor4 for <float, 4>
template <typename T, int Dims>
struct TiledDeviceTensor {
  TiledDeviceTensor() : padL(-1), padU(-1), tensor() {}
  TiledDeviceTensor(DeviceTensor<T, Dims>& t, int leftPadding, int upPadding)
      : padL(leftPadding), padU(upPadding), tensor(t) {}
  int padL;
  int padU;
  DeviceTensor<T, Dims> tensor;
};
static_assert(sizeof(TiledDeviceTensor<float, 4>) == sizeof(fbfft_tiled_tensor4), "layouts must agree");

struct FFTConvolutionPassFFI {
  static const int FFT_UpdateOutput = 0;
  static const int FFT_UpdateGradInput = 1;
  static const int FFT_AccGradParameters = 2;
  int pass;
};

// ins / outs: DEVICE arrays of numTiles descriptors, as in the reference
template <int FFTSize>
bool FFTIteratedConvolution(TiledDeviceTensor<float, 4>* ins, TiledDeviceTensor<float, 4>* outs,
                            const DeviceTensor<float, 4> weight, FFTConvolutionPassFFI pass, float scale,
                            int batchSize, size_t numTiles, cudaStream_t s) {
  return fbfft_b200_iterated_convolution(FFTSize, reinterpret_cast<const fbfft_tiled_tensor4*>(ins),
                                         reinterpret_cast<const fbfft_tiled_tensor4*>(outs), weight.data(),
                                         weight.sizes(), weight.strides(), pass.pass, scale, batchSize, numTiles,
                                         s) != 0;
}

}}}}  // namespace facebook::cuda::fbfft::detail
