// The reference's fbfft templates (fbfft/FBFFT.cuh:11-56), forwarding to libfbfft_b200.so.
// Include path and names are the reference's, so existing call sites compile unchanged.
#pragma once
#include <cuda_runtime.h>

#include "cuda/Complex.cuh"
#include "cuda/DeviceTensor.cuh"
#include "cuda/fbfft/FBFFTParameters.h"
#include "fbfft_b200.h"

namespace facebook { namespace cuda { namespace fbfft {

template <int BatchDims>
FBFFTParameters::ErrorCode fbfft1D(DeviceTensor<float, BatchDims + 1>& real,
                                   DeviceTensor<float, BatchDims + 2>& complex, const int padL = 0,
                                   cudaStream_t s = 0) {
  static_assert(BatchDims == 1, "one batch dimension, as in the reference (fbfft/FBFFT-inl.cuh:33)");
  return (FBFFTParameters::ErrorCode)fbfft_b200_fbfft1d(real.data(), real.sizes(), real.strides(), complex.data(),
                                                        complex.sizes(), complex.strides(), padL, s);
}

template <int BatchDims>
FBFFTParameters::ErrorCode fbifft1D(DeviceTensor<float, BatchDims + 1>& real,
                                    DeviceTensor<float, BatchDims + 2>& complex, const int padL = 0,
                                    cudaStream_t s = 0) {
  static_assert(BatchDims == 1, "one batch dimension, as in the reference");
  return (FBFFTParameters::ErrorCode)fbfft_b200_fbifft1d(real.data(), real.sizes(), real.strides(), complex.data(),
                                                         complex.sizes(), complex.strides(), padL, s);
}

template <int BatchDims>
FBFFTParameters::ErrorCode fbfft2D(DeviceTensor<float, BatchDims + 2>& real,
                                   DeviceTensor<float, BatchDims + 3>& complexAsFloat, const int padL = 0,
                                   const int padU = 0, cudaStream_t s = 0) {
  static_assert(BatchDims == 1, "one batch dimension, as in the reference (fbfft/FBFFT2D-inl.cuh:480)");
  return (FBFFTParameters::ErrorCode)fbfft_b200_fbfft2d(real.data(), real.sizes(), real.strides(),
                                                        complexAsFloat.data(), complexAsFloat.sizes(),
                                                        complexAsFloat.strides(), padL, padU, s);
}

template <int BatchDims>
FBFFTParameters::ErrorCode fbfft2D(DeviceTensor<Complex, BatchDims + 2>& src, DeviceTensor<Complex, BatchDims + 2>& dst,
                                   cudaStream_t s = 0) {
  static_assert(BatchDims == 1, "one batch dimension, as in the reference");
  return (FBFFTParameters::ErrorCode)fbfft_b200_fbfft2d_c2c((const float*)src.data(), src.sizes(), src.strides(),
                                                            (float*)dst.data(), dst.sizes(), dst.strides(), s);
}

template <int BatchDims>
FBFFTParameters::ErrorCode fbifft2D(DeviceTensor<float, BatchDims + 3>& src, DeviceTensor<float, BatchDims + 3>& dst,
                                    cudaStream_t s = 0) {
  static_assert(BatchDims == 1, "one batch dimension, as in the reference");
  return (FBFFTParameters::ErrorCode)fbfft_b200_fbifft2d_c2c(src.data(), src.sizes(), src.strides(), dst.data(),
                                                             dst.sizes(), dst.strides(), s);
}

template <int BatchDims>
FBFFTParameters::ErrorCode fbifft2D(DeviceTensor<Complex, BatchDims + 2>& complexSrc,
                                    DeviceTensor<float, BatchDims + 2>& realDst, const int padL = 0,
                                    const int padU = 0, cudaStream_t s = 0) {
  static_assert(BatchDims == 1, "one batch dimension, as in the reference");
  return (FBFFTParameters::ErrorCode)fbfft_b200_fbifft2d((const float*)complexSrc.data(), complexSrc.sizes(),
                                                         complexSrc.strides(), realDst.data(), realDst.sizes(),
                                                         realDst.strides(), padL, padU, s);
}

}}}  // namespace facebook::cuda::fbfft
