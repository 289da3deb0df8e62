// Per-frequency-bin complex contraction: the reference's transposeMM
// (MM.cuh:11-17, MM-inl.cuh:515-814).
//
//   C[i][j][x] (+)= invNorm * sum_k op(A)[i][k][x] * op(B)[k][j][x],   x = frequency bin
//
// with op(A)[i][k] = conj(A[k][i]) when A is "conjugate transposed"
// (MM-inl.cuh:121-131,150-163).  The three convolution passes use
// (conjA, conjB) = (0,1) updateOutput, (1,0) accGradParameters, (0,0)
// updateGradInput (MM-inl.cuh:194-196).
//
// FP32 CUDA-core version.  Bins are the contiguous index of all three tensors, so
// a warp takes 32 consecutive bins (256-byte coalesced complex loads, no
// shared-memory staging needed because lanes share nothing) and each thread keeps
// an 8 x 4 tile of C for its bin in registers: 12 complex loads feed 32 complex
// multiply-adds per k.  A block of 8 warps covers 16 x 16 of (i, j) so the L1
// absorbs the 3x reuse between its warps.  The reference's generic fallback, the
// only path it has for 64 x 64 and 128 x 128 transforms, is a 16-thread block with
// a 4 x 2 tile (MM-inl.cuh:787-813).
#include "common.cuh"
#include "kernels.h"

namespace fbfft_b200 {

namespace {

constexpr int TI = 8, TJ = 4;          // per-thread tile of C
constexpr int WI = 2, WJ = 4;          // warps per block along i and j
constexpr int kMmThreads = 32 * WI * WJ;

template <bool CA, bool CB, bool ACC>
__global__ void __launch_bounds__(kMmThreads, 2)
cgemm_bins_kernel(const float2* __restrict__ A, long long a_s0, long long a_s1, const float2* __restrict__ B,
                  long long b_s0, long long b_s1, float2* __restrict__ C, long long c_s0, long long c_s1, int I, int J,
                  int K, int X, float inv_norm) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int x = blockIdx.x * 32 + lane;
  const int xc = x < X ? x : X - 1;
  const int i0 = (blockIdx.y * WI + (warp % WI)) * TI;
  const int j0 = (blockIdx.z * WJ + (warp / WI)) * TJ;
  if (i0 >= I || j0 >= J) return;

  // clamp so that the inner loop needs no predicates; out-of-range rows are not stored
  long long a_off[TI], b_off[TJ];
#pragma unroll
  for (int ii = 0; ii < TI; ++ii) {
    const int i = i0 + ii < I ? i0 + ii : I - 1;
    a_off[ii] = (CA ? (long long)i * a_s1 : (long long)i * a_s0) + xc;
  }
#pragma unroll
  for (int jj = 0; jj < TJ; ++jj) {
    const int j = j0 + jj < J ? j0 + jj : J - 1;
    b_off[jj] = (CB ? (long long)j * b_s0 : (long long)j * b_s1) + xc;
  }
  const long long a_sk = CA ? a_s0 : a_s1, b_sk = CB ? b_s1 : b_s0;

  float2 acc[TI][TJ];
#pragma unroll
  for (int ii = 0; ii < TI; ++ii)
#pragma unroll
    for (int jj = 0; jj < TJ; ++jj) acc[ii][jj] = make_float2(0.f, 0.f);

  for (int k = 0; k < K; ++k) {
    float2 a[TI], b[TJ];
#pragma unroll
    for (int ii = 0; ii < TI; ++ii) a[ii] = __ldg(A + a_off[ii] + (long long)k * a_sk);
#pragma unroll
    for (int jj = 0; jj < TJ; ++jj) b[jj] = __ldg(B + b_off[jj] + (long long)k * b_sk);
#pragma unroll
    for (int ii = 0; ii < TI; ++ii) {
      // conj(a) * b and a * conj(b) differ from a * b only in two signs
      const float ax = a[ii].x, ay = CA ? -a[ii].y : a[ii].y;
#pragma unroll
      for (int jj = 0; jj < TJ; ++jj) {
        const float bx = b[jj].x, by = CB ? -b[jj].y : b[jj].y;
        acc[ii][jj].x = fmaf(ax, bx, acc[ii][jj].x);
        acc[ii][jj].x = fmaf(-ay, by, acc[ii][jj].x);
        acc[ii][jj].y = fmaf(ax, by, acc[ii][jj].y);
        acc[ii][jj].y = fmaf(ay, bx, acc[ii][jj].y);
      }
    }
  }

  if (x < X) {
#pragma unroll
    for (int ii = 0; ii < TI; ++ii) {
      if (i0 + ii < I) {
#pragma unroll
        for (int jj = 0; jj < TJ; ++jj) {
          if (j0 + jj < J) {
            float2* dst = C + (long long)(i0 + ii) * c_s0 + (long long)(j0 + jj) * c_s1 + x;
            float2 v = make_float2(acc[ii][jj].x * inv_norm, acc[ii][jj].y * inv_norm);
            if (ACC) {
              const float2 old = *dst;
              v.x += old.x;
              v.y += old.y;
            }
            *dst = v;
          }
        }
      }
    }
  }
}

// A float tensor [d0][d1][bins...][2] seen as complex [d0][d1][X]: returns false
// when the bin dimensions are not densely packed.
bool collapse(int dim, const int* size, const int* stride, long long* s0, long long* s1, int* X) {
  if (size[dim - 1] != 2 || stride[dim - 1] != 1) return false;
  long long expect = 2;
  long long bins = 1;
  for (int d = dim - 2; d >= 2; --d) {
    if (size[d] != 1 && stride[d] != expect) return false;
    expect *= size[d];
    bins *= size[d];
  }
  if ((stride[0] & 1) || (stride[1] & 1)) return false;
  *s0 = stride[0] / 2;
  *s1 = stride[1] / 2;
  *X = (int)bins;
  return true;
}

}  // namespace

int transpose_mm(int dim, bool conjA, bool conjB, bool accumulate, const float* a, const int* a_size,
                 const int* a_stride, const float* b, const int* b_size, const int* b_stride, float* c,
                 const int* c_size, const int* c_stride, float inv_norm, cudaStream_t s) {
  long long as0, as1, bs0, bs1, cs0, cs1;
  int xa, xb, xc;
  if (!collapse(dim, a_size, a_stride, &as0, &as1, &xa) || !collapse(dim, b_size, b_stride, &bs0, &bs1, &xb) ||
      !collapse(dim, c_size, c_stride, &cs0, &cs1, &xc)) {
    set_last_error("transpose_mm: the frequency dimensions must be densely packed with interleaved re/im");
    return kUnsupportedDimension;
  }
  const int I = conjA ? a_size[1] : a_size[0], K = conjA ? a_size[0] : a_size[1];
  const int Kb = conjB ? b_size[1] : b_size[0], J = conjB ? b_size[0] : b_size[1];
  if (K != Kb || c_size[0] != I || c_size[1] != J || xa != xb || xa != xc) {
    set_last_error("transpose_mm: operand shapes do not agree");
    return kUnsupportedDimension;
  }
  return cgemm_bins(conjA, conjB, accumulate, a, as0, as1, b, bs0, bs1, c, cs0, cs1, I, J, K, xa, inv_norm, s);
}

int cgemm_bins(bool conjA, bool conjB, bool accumulate, const float* a, long long as0, long long as1, const float* b,
               long long bs0, long long bs1, float* c, long long cs0, long long cs1, int I, int J, int K, int X,
               float inv_norm, cudaStream_t s) {
  if (I == 0 || J == 0 || X == 0) return kSuccess;
  if (conjA && conjB) {
    set_last_error("transpose_mm: both operands conjugate-transposed is not a convolution pass");
    return kUnsupportedDimension;
  }
  if (K > 0) {
    // tensor-core path: the larger of I and J becomes the 128-row MMA dimension
    // (complex multiplication commutes, so C = op(A) op(B) = (op(B)^T op(A)^T)^T)
    const long long a_rs = conjA ? as1 : as0, a_ks = conjA ? as0 : as1;   // op(A)[i][k]
    const long long b_rs = conjB ? bs0 : bs1, b_ks = conjB ? bs1 : bs0;   // op(B)[k][j] seen as rows j
    if (J >= I) {
      if (cgemm_tc_supported(b, b_rs, b_ks, a, a_rs, a_ks, c, cs1, cs0, J, I, K, X))
        return cgemm_tc(b, b_rs, b_ks, conjB, a, a_rs, a_ks, conjA, c, cs1, cs0, J, I, K, X, inv_norm, accumulate, s);
    } else {
      if (cgemm_tc_supported(a, a_rs, a_ks, b, b_rs, b_ks, c, cs0, cs1, I, J, K, X))
        return cgemm_tc(a, a_rs, a_ks, conjA, b, b_rs, b_ks, conjB, c, cs0, cs1, I, J, K, X, inv_norm, accumulate, s);
    }
  }
  const float2* A = reinterpret_cast<const float2*>(a);
  const float2* B = reinterpret_cast<const float2*>(b);
  float2* C = reinterpret_cast<float2*>(c);
  dim3 grid((X + 31) / 32, (I + WI * TI - 1) / (WI * TI), (J + WJ * TJ - 1) / (WJ * TJ));
  if (grid.y > 65535 || grid.z > 65535) {
    set_last_error("transpose_mm: operand too large");
    return kUnsupportedSize;
  }
#define LAUNCH(CA, CB, AC) \
  cgemm_bins_kernel<CA, CB, AC><<<grid, kMmThreads, 0, s>>>(A, as0, as1, B, bs0, bs1, C, cs0, cs1, I, J, K, X, inv_norm)
  if (conjA && conjB) {
    set_last_error("transpose_mm: both operands conjugate-transposed is not a convolution pass");
    return kUnsupportedDimension;
  }
  if (!conjA && conjB) {
    if (accumulate) LAUNCH(false, true, true); else LAUNCH(false, true, false);
  } else if (conjA && !conjB) {
    if (accumulate) LAUNCH(true, false, true); else LAUNCH(true, false, false);
  } else {
    if (accumulate) LAUNCH(false, false, true); else LAUNCH(false, false, false);
  }
#undef LAUNCH
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

}  // namespace fbfft_b200
