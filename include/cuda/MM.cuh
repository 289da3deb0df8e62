// The reference's transposeMM (MM.cuh:11-17), forwarding to libfbfft_b200.so.
#pragma once
#include <cuda_runtime.h>

#include "cuda/DeviceTensor.cuh"
#include "fbfft_b200.h"

namespace facebook { namespace cuda {

template <int Dim, bool ConjugateTransposeA, bool ConjugateTransposeB, bool Accumulate>
void transposeMM(DeviceTensor<float, Dim>& A, DeviceTensor<float, Dim>& B, DeviceTensor<float, Dim>& C, float invNorm,
                 cudaStream_t s = 0) {
  fbfft_b200_transpose_mm(Dim, ConjugateTransposeA, ConjugateTransposeB, Accumulate, A.data(), A.sizes(), A.strides(),
                          B.data(), B.sizes(), B.strides(), C.data(), C.sizes(), C.strides(), invNorm, s);
}

}}  // namespace facebook::cuda
