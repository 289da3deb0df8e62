// Block-cooperative FFT of lines that sit in shared memory: M = R1 * R2 points per
// line, two register passes (radix R1, then radix R2) with one twiddle multiply
// in between.  Used by the 1-D transforms, the N >= 64 two-call protocol and the
// single-call N >= 64 kernels.
#pragma once
#include "fft_regs.cuh"

namespace fbfft_b200 {

template <int M>
struct Split;  // M = R1 * R2
template <>
struct Split<8> {
  static constexpr int R1 = 4, R2 = 2;
};
template <>
struct Split<16> {
  static constexpr int R1 = 4, R2 = 4;
};
template <>
struct Split<32> {
  static constexpr int R1 = 8, R2 = 4;
};
template <>
struct Split<64> {
  static constexpr int R1 = 8, R2 = 8;
};
template <>
struct Split<128> {
  static constexpr int R1 = 16, R2 = 8;
};
template <>
struct Split<256> {
  static constexpr int R1 = 16, R2 = 16;
};

// Where output k of a line is found after smem_fft_lines: the transform leaves
// X[k1 + R1*k2] at slot k1*R2 + (k2 ^ (k1 & (R2-1))).
template <int M>
__device__ __forceinline__ int fft_slot(int k) {
  constexpr int R1 = Split<M>::R1, R2 = Split<M>::R2;
  const int k1 = k % R1, k2 = k / R1;
  return k1 * R2 + (k2 ^ (k1 & (R2 - 1)));
}

// exp(-2*pi*i*k/M), k in [0, M), computed once per block in double precision
template <int M>
__device__ __forceinline__ void fill_twiddles(float2* tw) {
  for (int k = threadIdx.x; k < M; k += blockDim.x) {
    double s, c;
    sincospi(-2.0 * (double)k / (double)M, &s, &c);
    tw[k] = make_float2((float)c, (float)s);
  }
}

// In-place transform of `lines` lines of M complex values, line l at
// tile[l * pitch ...], natural order in, fft_slot order out.  Needs
// blockDim.x >= lines * max(R1, R2); ends with a __syncthreads().  `tw` holds
// the forward roots; the inverse conjugates them.  Every thread of the block must
// call it.
template <int M, bool INV>
__device__ __forceinline__ void smem_fft_lines(float2* tile, int pitch, int lines, const float2* tw) {
  constexpr int R1 = Split<M>::R1, R2 = Split<M>::R2;
  const int tid = threadIdx.x;
  {
    // pass 1: radix R1 over n1 for fixed n2 (elements n1*R2 + n2)
    const int line = tid / R2, n2 = tid % R2;
    const bool active = line < lines;
    float2 a[R1];
    if (active) {
#pragma unroll
      for (int n1 = 0; n1 < R1; ++n1) a[n1] = tile[line * pitch + n1 * R2 + n2];
      fft_bitrev<R1, INV>(a);
    }
    __syncthreads();
    if (active) {
      static_for<R1>([&](auto kc) {
        constexpr int k1 = decltype(kc)::value;
        float2 v = a[brev(k1, R1)];
        if (k1 > 0) {
          float2 w = tw[n2 * k1];
          if (INV) w.y = -w.y;
          v = cmul(v, w);
        }
        tile[line * pitch + k1 * R2 + (n2 ^ (k1 & (R2 - 1)))] = v;
      });
    }
  }
  __syncthreads();
  {
    // pass 2: radix R2 over n2 for fixed k1; result k2 goes back to the slot n2 = k2
    const int line = tid / R1, k1 = tid % R1;
    if (line < lines) {
      float2 b[R2];
      float2* row = tile + line * pitch + k1 * R2;
      const int sw = k1 & (R2 - 1);
#pragma unroll
      for (int n2 = 0; n2 < R2; ++n2) b[n2] = row[n2 ^ sw];
      fft_bitrev<R2, INV>(b);
      static_for<R2>([&](auto kc) {
        constexpr int k2 = decltype(kc)::value;
        row[k2 ^ sw] = b[brev(k2, R2)];
      });
    }
  }
  __syncthreads();
}

}  // namespace fbfft_b200
