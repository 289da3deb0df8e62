// Host-side stand-in for the reference's DeviceTensor<T, Dim> (DeviceTensor.cuh:53-246), for
// code that keeps calling the fbfft templates while linking libfbfft_b200.so.  Only what the
// fbfft entry points read is provided -- pointer, sizes and strides -- in the reference's own
// field order (pointer, strides, sizes; DeviceTensor.cuh:237-245), so a pointer to one of these
// can be handed to code compiled against the reference and vice versa.
#pragma once
#include <cstddef>

namespace facebook { namespace cuda {

template <typename T, int Dim>
class DeviceTensor {
 public:
  DeviceTensor() : data_(nullptr) {
    for (int i = 0; i < Dim; ++i) stride_[i] = 0, size_[i] = 0;
  }
  // contiguous tensor of the given sizes
  DeviceTensor(T* data, const int (&sizes)[Dim]) : data_(data) {
    int s = 1;
    for (int i = Dim - 1; i >= 0; --i) {
      size_[i] = sizes[i];
      stride_[i] = s;
      s *= sizes[i];
    }
  }
  DeviceTensor(T* data, const int (&sizes)[Dim], const int (&strides)[Dim]) : data_(data) {
    for (int i = 0; i < Dim; ++i) size_[i] = sizes[i], stride_[i] = strides[i];
  }
  T* data() const { return data_; }
  const int* sizes() const { return size_; }
  const int* strides() const { return stride_; }
  int getSize(int i) const { return size_[i]; }
  int getStride(int i) const { return stride_[i]; }
  size_t numElements() const {
    size_t n = 1;
    for (int i = 0; i < Dim; ++i) n *= (size_t)size_[i];
    return n;
  }

 private:
  T* data_;
  int stride_[Dim];
  int size_[Dim];
};

}}  // namespace facebook::cuda
