// The reference's Complex is a cuComplex wrapper: two floats, real part first (Complex.cuh:16-140).
#pragma once
namespace facebook { namespace cuda {
struct Complex {
  float re_, im_;
  Complex() : re_(0.f), im_(0.f) {}
  Complex(float r, float i = 0.f) : re_(r), im_(i) {}
  float re() const { return re_; }
  float im() const { return im_; }
};
static_assert(sizeof(Complex) == 8, "Complex is two packed floats");
}}  // namespace facebook::cuda
