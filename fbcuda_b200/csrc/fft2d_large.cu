// Single-call batched 2-D real-to-complex / complex-to-real FFTs for N in
// {64, 128, 256}, in the reference's layout for this size class: the spectrum is
// stored transposed, [B][kx in 0..N/2][ky in 0..N) (what its two calls
// fbfft/FBFFT2D-inl.cuh:597-617 and :627-669 leave behind), the inverse is
// unnormalised and crops at (padU, padL) (fbfft/FBIFFT2D-inl.cuh:529-742).
//
// N = 64, 128: one block owns one image, which never leaves shared memory between
// the row pass and the column pass -- the reference's HBM round trip through a
// caller-owned [B][N][N/2+1] buffer is gone.  Rows are transformed two at a time
// as one complex line; the bins kx = 0 and kx = N/2 of a real row are real, so
// their two columns travel as one complex column through the column pass.
// N = 256 (no reference counterpart; it rejects N > 128): an image no longer fits
// in shared memory, so the forward transform writes its row pass transposed into
// the output tensor and transforms the lines of that tensor in place.
#include "common.cuh"
#include "kernels.h"
#include "smem_fft.cuh"

namespace fbfft_b200 {

namespace {

template <int N>
struct LargeCfg {
  static constexpr int R = Split<N>::R1 > Split<N>::R2 ? Split<N>::R1 : Split<N>::R2;
  static constexpr int LINES = N / 2;            // row pairs, and packed columns
  static constexpr int THREADS = LINES * R;      // 256 for N = 64, 1024 for N = 128
  static constexpr int P = N + 1;                // line pitch in float2
  static constexpr int SMEM = (2 * LINES * P + N) * (int)sizeof(float2);
};

// ------------------------------------------------------------------ forward
template <int N>
__global__ void __launch_bounds__(LargeCfg<N>::THREADS) fft2d_large_fwd_kernel(RealView in, CplxView out, int B,
                                                                              int padL, int padU) {
  using C = LargeCfg<N>;
  constexpr int L = C::LINES, P = C::P, T = C::THREADS;
  extern __shared__ __align__(16) float2 smem[];
  float2* ta = smem;              // row pairs:      ta[l][x]  = P[2l][x] + i P[2l+1][x]
  float2* tb = smem + L * P;      // packed columns: tb[kx][y], tb[0] = (X[0], X[N/2])
  float2* tw = smem + 2 * L * P;
  fill_twiddles<N>(tw);
  for (int b = blockIdx.x; b < B; b += gridDim.x) {
    const float* src = in.p + (long long)b * in.sb;
    for (int e = threadIdx.x; e < L * N; e += T) {
      const int line = e / N, x = e % N;
      const unsigned xx = (unsigned)(x - padL);
      const unsigned y0 = (unsigned)(2 * line - padU), y1 = y0 + 1u;
      float2 v = make_float2(0.f, 0.f);
      if (xx < (unsigned)in.w) {
        if (y0 < (unsigned)in.h) v.x = __ldg(src + (long long)y0 * in.sy + (long long)xx * in.sx);
        if (y1 < (unsigned)in.h) v.y = __ldg(src + (long long)y1 * in.sy + (long long)xx * in.sx);
      }
      ta[line * P + x] = v;
    }
    __syncthreads();
    smem_fft_lines<N, false>(ta, P, L, tw);
    // separate the two rows of every pair and transpose: tb[kx][y]
    for (int e = threadIdx.x; e < L * (N / 2); e += T) {
      const int k = e / L, line = e % L;  // consecutive threads -> consecutive y
      const float2 z = ta[line * P + fft_slot<N>(k)];
      if (k == 0) {
        const float2 h = ta[line * P + fft_slot<N>(N / 2)];
        tb[2 * line] = make_float2(z.x, h.x);
        tb[2 * line + 1] = make_float2(z.y, h.y);
      } else {
        const float2 m = ta[line * P + fft_slot<N>(N - k)];
        tb[k * P + 2 * line] = make_float2(0.5f * (z.x + m.x), 0.5f * (z.y - m.y));
        tb[k * P + 2 * line + 1] = make_float2(0.5f * (z.y + m.y), 0.5f * (m.x - z.x));
      }
    }
    __syncthreads();
    smem_fft_lines<N, false>(tb, P, L, tw);
    // store out[kx][ky]; line 0 unpacks into kx = 0 and kx = N/2
    float* dst = out.p + (long long)b * out.sb;
    for (int e = threadIdx.x; e < (L + 1) * N; e += T) {
      const int kx = e / N, ky = e % N;
      float2 r;
      if (kx == 0 || kx == N / 2) {
        const float2 v = tb[fft_slot<N>(ky)], m = tb[fft_slot<N>((N - ky) % N)];
        r = (kx == 0) ? make_float2(0.5f * (v.x + m.x), 0.5f * (v.y - m.y))
                      : make_float2(0.5f * (v.y + m.y), 0.5f * (m.x - v.x));
      } else {
        r = tb[kx * P + fft_slot<N>(ky)];
      }
      float* q = dst + (long long)kx * out.sr + (long long)ky * out.sc;
      q[0] = r.x;
      q[out.sz] = r.y;
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------ inverse
template <int N>
__global__ void __launch_bounds__(LargeCfg<N>::THREADS) fft2d_large_inv_kernel(CplxView in, RealView out, int B,
                                                                              int padL, int padU) {
  using C = LargeCfg<N>;
  constexpr int L = C::LINES, P = C::P, T = C::THREADS;
  extern __shared__ __align__(16) float2 smem[];
  float2* ta = smem;
  float2* tb = smem + L * P;
  float2* tw = smem + 2 * L * P;
  fill_twiddles<N>(tw);
  for (int b = blockIdx.x; b < B; b += gridDim.x) {
    const float* src = in.p + (long long)b * in.sb;
    // tb[kx][ky] for kx in 1..N/2-1; tb[0] = X[0] + i X[N/2] (both are transforms of real sequences)
    for (int e = threadIdx.x; e < L * N; e += T) {
      const int kx = e / N, ky = e % N;
      const float* q = src + (long long)kx * in.sr + (long long)ky * in.sc;
      float2 v = make_float2(__ldg(q), __ldg(q + in.sz));
      if (kx == 0) {
        const float* qh = src + (long long)(N / 2) * in.sr + (long long)ky * in.sc;
        const float2 h = make_float2(__ldg(qh), __ldg(qh + in.sz));
        v = make_float2(v.x - h.y, v.y + h.x);
      }
      tb[kx * P + ky] = v;
    }
    __syncthreads();
    smem_fft_lines<N, true>(tb, P, L, tw);
    // row pairs: ta[l][kx] = G_{2l}[kx] + i G_{2l+1}[kx], Hermitian-extended in kx
    for (int e = threadIdx.x; e < L * (N / 2); e += T) {
      const int k = e / L, line = e % L;
      const float2 g0 = tb[k * P + fft_slot<N>(2 * line)], g1 = tb[k * P + fft_slot<N>(2 * line + 1)];
      if (k == 0) {
        ta[line * P] = make_float2(g0.x, g1.x);
        ta[line * P + N / 2] = make_float2(g0.y, g1.y);
      } else {
        ta[line * P + k] = make_float2(g0.x - g1.y, g0.y + g1.x);
        ta[line * P + N - k] = make_float2(g0.x + g1.y, g1.x - g0.y);
      }
    }
    __syncthreads();
    smem_fft_lines<N, true>(ta, P, L, tw);
    float* dst = out.p + (long long)b * out.sb;
    for (int e = threadIdx.x; e < L * N; e += T) {
      const int line = e / N, x = e % N;
      const unsigned xx = (unsigned)(x - padL);
      if (xx < (unsigned)out.w) {
        const float2 z = ta[line * P + fft_slot<N>(x)];
        const unsigned y0 = (unsigned)(2 * line - padU), y1 = y0 + 1u;
        if (y0 < (unsigned)out.h) dst[(long long)y0 * out.sy + (long long)xx * out.sx] = z.x;
        if (y1 < (unsigned)out.h) dst[(long long)y1 * out.sy + (long long)xx * out.sx] = z.y;
      }
    }
    __syncthreads();
  }
}

template <int N>
int launch_fwd(const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s) {
  using C = LargeCfg<N>;
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(fft2d_large_fwd_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    cudaFuncSetAttribute(fft2d_large_inv_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    configured[dev] = true;
  }
  const int per_sm = (N == 64) ? 6 : 1;
  const int cap = sm_count() * per_sm;
  fft2d_large_fwd_kernel<N><<<B < cap ? B : cap, C::THREADS, C::SMEM, s>>>(in, out, B, padL, padU);
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

template <int N>
int launch_inv(const CplxView& in, const RealView& out, int B, int padL, int padU, cudaStream_t s) {
  using C = LargeCfg<N>;
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(fft2d_large_fwd_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    cudaFuncSetAttribute(fft2d_large_inv_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    configured[dev] = true;
  }
  const int per_sm = (N == 64) ? 6 : 1;
  const int cap = sm_count() * per_sm;
  fft2d_large_inv_kernel<N><<<B < cap ? B : cap, C::THREADS, C::SMEM, s>>>(in, out, B, padL, padU);
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

}  // namespace

int fft2d_large_forward(int n, const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s) {
  if (fft2d_coop_supported(n, out)) return fft2d_coop_forward(n, in, out, B, padL, padU, s);
  if (n == 64) return launch_fwd<64>(in, out, B, padL, padU, s);
  if (n == 128) return launch_fwd<128>(in, out, B, padL, padU, s);
  if (n == 256 && fft2d_256_supported(in, out, B)) return fft2d_256_forward(in, out, B, padL, padU, s);
  if (n == 256) {
    // (strided or unaligned output) row pass straight into the output tensor, transposed: out[b][kx][y]; then
    // every line out[b][kx][*] is transformed in place
    CplxView t = out;
    t.sr = out.sc;
    t.sc = out.sr;
    int rc = fft2d_large_rows_forward(256, in, t, B, padL, padU, s);
    if (rc != kSuccess) return rc;
    return fft_lines_inplace(256, out, B, 129, false, s);
  }
  return kUnsupportedSize;
}

int fft2d_large_inverse(int n, const CplxView& in, const RealView& out, int B, int padL, int padU, cudaStream_t s) {
  if (fft2d_coop_supported(n, in)) return fft2d_coop_inverse(n, in, out, B, padL, padU, s);
  if (n == 64) return launch_inv<64>(in, out, B, padL, padU, s);
  if (n == 128) return launch_inv<128>(in, out, B, padL, padU, s);
  if (n == 256 && fft2d_256_inverse_supported(in, out, B, padL, padU)) return fft2d_256_inverse(in, out, B, s);
  set_last_error(
      "single-call inverse for N = 256 needs contiguous, 16-byte aligned tensors and full 256 x 256 output images "
      "without crop (the output doubles as the intermediate buffer); otherwise use the two-call protocol");
  return kUnsupportedSize;
}

}  // namespace fbfft_b200
