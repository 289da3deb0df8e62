// In-register complex FFTs of length 2..32 with compile-time twiddles.
//
// Every index is a template constant, so after inlining the arrays live in
// registers, the bit reversal is a renaming and the twiddles are immediates.
// This replaces the reference's shuffle butterflies and twiddle tables
// (fbfft/FBFFTCommon.cuh:432-474, fbfft/FFT2D32.cuh:132-219,
// fbfft/Twiddles.cuh:13-305): there a warp lane owns one element and each
// radix-2 stage costs four shuffles; here a thread owns a whole line and lines
// are moved between threads through shared memory once per pass.
#pragma once
#include <cuda_runtime.h>

#include <utility>

namespace fbfft_b200 {

// ---------------------------------------------------------------- static_for
template <int... Is, typename F>
__device__ __forceinline__ void static_for_impl(std::integer_sequence<int, Is...>, F&& f) {
  (f(std::integral_constant<int, Is>{}), ...);
}
// calls f(integral_constant<int, 0>) ... f(integral_constant<int, N-1>)
template <int N, typename F>
__device__ __forceinline__ void static_for(F&& f) {
  static_for_impl(std::make_integer_sequence<int, N>{}, static_cast<F&&>(f));
}

// ---------------------------------------------------------------- constexpr trig
// cos/sin(2*pi*k/n) evaluated in double at compile time, exact at multiples of
// a quarter turn, rounded once to fp32.
constexpr double kPi = 3.141592653589793238462643383279502884;

constexpr double cx_sin_series(double x) {  // |x| <= pi/2
  double term = x, sum = x;
  for (int i = 1; i < 16; ++i) {
    term *= -x * x / (double)((2 * i) * (2 * i + 1));
    sum += term;
  }
  return sum;
}
constexpr double cx_cos_series(double x) {  // |x| <= pi/2
  double term = 1.0, sum = 1.0;
  for (int i = 1; i < 16; ++i) {
    term *= -x * x / (double)((2 * i - 1) * (2 * i));
    sum += term;
  }
  return sum;
}
constexpr double cx_cos2pi(long k, long n) {
  k = ((k % n) + n) % n;
  if (k == 0) return 1.0;
  if (4 * k == n || 4 * k == 3 * n) return 0.0;
  if (2 * k == n) return -1.0;
  if (2 * k > n) k = n - k;               // cos is even about half a turn
  if (4 * k > n) return -cx_cos_series(2.0 * kPi * (double)(n - 2 * k) / (double)(2 * n));
  return cx_cos_series(2.0 * kPi * (double)k / (double)n);
}
constexpr double cx_sin2pi(long k, long n) {
  k = ((k % n) + n) % n;
  if (k == 0 || 2 * k == n) return 0.0;
  if (4 * k == n) return 1.0;
  if (4 * k == 3 * n) return -1.0;
  if (2 * k > n) return -cx_sin2pi(n - k, n);
  if (4 * k > n) return cx_sin_series(2.0 * kPi * (double)(n - 2 * k) / (double)(2 * n));
  return cx_sin_series(2.0 * kPi * (double)k / (double)n);
}

// exp(-2*pi*i*K/N) (forward) or exp(+2*pi*i*K/N) (inverse)
template <int K, int N, bool INV>
struct Tw {
  static constexpr float c = (float)cx_cos2pi(K, N);
  static constexpr float s = (float)(INV ? cx_sin2pi(K, N) : -cx_sin2pi(K, N));
};

__device__ __forceinline__ float2 cadd(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ float2 csub(float2 a, float2 b) { return make_float2(a.x - b.x, a.y - b.y); }
// Complex add / subtract as ONE packed fp32x2 instruction each (Blackwell's FADD2 / FFMA2).
// The butterflies are issue-bound and two thirds of their instructions are these; whether
// the packed form wins depends on how the kernel's operands reach register pairs, so each
// kernel chooses (template parameter PK of the transforms below).
template <bool PK>
__device__ __forceinline__ float2 cadd_t(float2 a, float2 b) {
  if constexpr (PK) return __fadd2_rn(a, b);
  return make_float2(a.x + b.x, a.y + b.y);
}
template <bool PK>
__device__ __forceinline__ float2 csub_t(float2 a, float2 b) {
  if constexpr (PK) return __ffma2_rn(b, make_float2(-1.f, -1.f), a);
  return make_float2(a.x - b.x, a.y - b.y);
}
__device__ __forceinline__ float2 cmul(float2 a, float2 b) {
  return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}
__device__ __forceinline__ float2 cconj(float2 a) { return make_float2(a.x, -a.y); }

// a * exp(-+ 2*pi*i*K/N) with the trivial rotations spelled out
template <int K, int N, bool INV>
__device__ __forceinline__ float2 mul_tw(float2 a) {
  constexpr int k = ((K % N) + N) % N;
  if constexpr (k == 0) {
    return a;
  } else if constexpr (2 * k == N) {
    return make_float2(-a.x, -a.y);
  } else if constexpr (4 * k == N) {  // forward: -i, inverse: +i
    return INV ? make_float2(-a.y, a.x) : make_float2(a.y, -a.x);
  } else if constexpr (4 * k == 3 * N) {
    return INV ? make_float2(a.y, -a.x) : make_float2(-a.y, a.x);
  } else if constexpr ((8 * k) % N == 0) {  // odd multiples of an eighth turn
    constexpr float r = 0.70710678118654752440f;
    constexpr float c = Tw<k, N, INV>::c, s = Tw<k, N, INV>::s;
    constexpr float sc = c > 0 ? 1.f : -1.f, ss = s > 0 ? 1.f : -1.f;
    // (x + iy)(sc + i ss) r
    return make_float2(r * (sc * a.x - ss * a.y), r * (ss * a.x + sc * a.y));
  } else {
    constexpr float c = Tw<k, N, INV>::c, s = Tw<k, N, INV>::s;
    return make_float2(a.x * c - a.y * s, a.x * s + a.y * c);
  }
}

__host__ __device__ constexpr int ilog2c(int n) { return n <= 1 ? 0 : 1 + ilog2c(n / 2); }
__host__ __device__ constexpr int brev(int v, int n) {  // reverse the log2(n) low bits of v
  int r = 0;
  for (int b = 1; b < n; b <<= 1) {
    r = (r << 1) | (v & 1);
    v >>= 1;
  }
  return r;
}

// Radix-2 decimation in frequency on a[OFF + j*ST], j in [0, N): afterwards
// output k sits at a[OFF + brev(k, N)*ST].
template <int N, int OFF, int ST, bool INV, int TOTAL, bool PK = false>
struct Dif {
  static __device__ __forceinline__ void run(float2 (&a)[TOTAL]) {
    if constexpr (N >= 2) {
      static_for<N / 2>([&](auto jc) {
        constexpr int j = decltype(jc)::value;
        float2 u = a[OFF + j * ST], v = a[OFF + (j + N / 2) * ST];
        a[OFF + j * ST] = cadd_t<PK>(u, v);
        a[OFF + (j + N / 2) * ST] = mul_tw<j, N, INV>(csub_t<PK>(u, v));
      });
      Dif<N / 2, OFF, ST, INV, TOTAL, PK>::run(a);
      Dif<N / 2, OFF + (N / 2) * ST, ST, INV, TOTAL, PK>::run(a);
    }
  }
};

// In-place FFT of a[0..N); output k is left at a[brev(k, N)].  PK: packed fp32x2 butterflies.
template <int N, bool INV, bool PK = false>
__device__ __forceinline__ void fft_bitrev(float2 (&a)[N]) {
  Dif<N, 0, 1, INV, N, PK>::run(a);
}

}  // namespace fbfft_b200
