// Drop-in check in the reference's own vocabulary: the fbfft templates over DeviceTensor, the
// way the reference's test bindings exercise a kernel (allocate, copy, call, copy back, compare
// with a host computation; e.g. TopKTestBindings.cu:46-68).  Host oracle: a direct O(N^2) DFT in
// double precision.  Exit code 0 and a final "PASS" line on success.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "cuda/MM.cuh"
#include "cuda/fbfft/FBFFT.cuh"
#include "cuda/fbfft/FFTIteratedConvolution.cuh"

using namespace facebook::cuda;
using namespace facebook::cuda::fbfft;

#define CK(x)                                                                  \
  do {                                                                         \
    cudaError_t e = (x);                                                       \
    if (e != cudaSuccess) {                                                    \
      printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__); \
      return 1;                                                                \
    }                                                                          \
  } while (0)

static double rel_l2(const std::vector<double>& got, const std::vector<double>& want) {
  double num = 0, den = 0;
  for (size_t i = 0; i < got.size(); ++i) num += (got[i] - want[i]) * (got[i] - want[i]), den += want[i] * want[i];
  return std::sqrt(num / den);
}

// F[ky][kx] of an h x w image placed at (padU, padL) of an N x N canvas
static void dft2(const float* img, int h, int w, int n, int padL, int padU, std::vector<double>& re,
                 std::vector<double>& im) {
  re.assign((size_t)n * n, 0.0), im.assign((size_t)n * n, 0.0);
  const double two_pi = 6.283185307179586476925286766559;
  std::vector<double> rr((size_t)n * n, 0.0), ri((size_t)n * n, 0.0);  // row transforms
  for (int y = 0; y < n; ++y)
    for (int kx = 0; kx < n; ++kx) {
      double sr = 0, si = 0;
      for (int x = 0; x < n; ++x) {
        int yy = y - padU, xx = x - padL;
        if (yy < 0 || yy >= h || xx < 0 || xx >= w) continue;
        double v = img[yy * w + xx], a = -two_pi * kx * x / n;
        sr += v * std::cos(a), si += v * std::sin(a);
      }
      rr[y * n + kx] = sr, ri[y * n + kx] = si;
    }
  for (int ky = 0; ky < n; ++ky)
    for (int kx = 0; kx < n; ++kx) {
      double sr = 0, si = 0;
      for (int y = 0; y < n; ++y) {
        double a = -two_pi * ky * y / n, c = std::cos(a), s = std::sin(a);
        sr += rr[y * n + kx] * c - ri[y * n + kx] * s, si += rr[y * n + kx] * s + ri[y * n + kx] * c;
      }
      re[ky * n + kx] = sr, im[ky * n + kx] = si;
    }
}

static int check_2d(int n, int B, int h, int w, int padL, int padU) {
  const int half = n / 2 + 1;
  std::vector<float> x((size_t)B * h * w);
  srand(n + B);
  for (auto& v : x) v = 2.f * rand() / RAND_MAX - 1.f;
  float *dx, *dspec, *dback;
  CK(cudaMalloc(&dx, x.size() * 4));
  CK(cudaMalloc(&dspec, (size_t)B * half * n * 2 * 4));
  CK(cudaMalloc(&dback, x.size() * 4));
  CK(cudaMemcpy(dx, x.data(), x.size() * 4, cudaMemcpyHostToDevice));
  int rs[3] = {B, h, w}, cs[4] = {B, half, n, 2}, zs[3] = {B, half, n};
  DeviceTensor<float, 3> real(dx, rs), back(dback, rs);
  DeviceTensor<float, 4> spec(dspec, cs);
  if (fbfft2D<1>(real, spec, padL, padU) != FBFFTParameters::Success) return printf("fbfft2D failed: %s\n", fbfft_b200_last_error()), 1;
  DeviceTensor<Complex, 3> cspec((Complex*)dspec, zs);
  if (fbifft2D<1>(cspec, back, padL, padU) != FBFFTParameters::Success) return printf("fbifft2D failed\n"), 1;
  std::vector<float> got((size_t)B * half * n * 2), gback(x.size());
  CK(cudaMemcpy(got.data(), dspec, got.size() * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(gback.data(), dback, gback.size() * 4, cudaMemcpyDeviceToHost));
  std::vector<double> g, wv, re, im;
  for (int b = 0; b < B; ++b) {
    dft2(&x[(size_t)b * h * w], h, w, n, padL, padU, re, im);
    for (int ky = 0; ky < half; ++ky)
      for (int kx = 0; kx < n; ++kx) {
        size_t o = (((size_t)b * half + ky) * n + kx) * 2;
        g.push_back(got[o]), g.push_back(got[o + 1]);
        wv.push_back(re[ky * n + kx]), wv.push_back(im[ky * n + kx]);
      }
  }
  double e1 = rel_l2(g, wv);
  std::vector<double> gb(gback.begin(), gback.end()), wb;
  for (auto v : x) wb.push_back((double)v * n * n);
  double e2 = rel_l2(gb, wb);
  printf("fbfft2D<1> N=%d B=%d %dx%d pad(%d,%d): spectrum rel-L2 %.2e, round trip %.2e\n", n, B, h, w, padL, padU, e1, e2);
  cudaFree(dx), cudaFree(dspec), cudaFree(dback);
  return (e1 < 1e-5 && e2 < 1e-5) ? 0 : 1;
}

static int check_1d(int n, int B) {
  std::vector<float> x((size_t)B * n);
  srand(n);
  for (auto& v : x) v = 2.f * rand() / RAND_MAX - 1.f;
  float *dx, *dc;
  CK(cudaMalloc(&dx, x.size() * 4));
  CK(cudaMalloc(&dc, (size_t)B * (n / 2 + 1) * 2 * 4));
  CK(cudaMemcpy(dx, x.data(), x.size() * 4, cudaMemcpyHostToDevice));
  int rs[2] = {B, n}, cs[3] = {B, n / 2 + 1, 2};
  DeviceTensor<float, 2> real(dx, rs);
  DeviceTensor<float, 3> cplx(dc, cs);
  if (fbfft1D<1>(real, cplx) != FBFFTParameters::Success) return printf("fbfft1D failed\n"), 1;
  std::vector<float> got((size_t)B * (n / 2 + 1) * 2);
  CK(cudaMemcpy(got.data(), dc, got.size() * 4, cudaMemcpyDeviceToHost));
  std::vector<double> g(got.begin(), got.end()), wv;
  for (int b = 0; b < B; ++b)
    for (int k = 0; k <= n / 2; ++k) {
      double sr = 0, si = 0;
      for (int j = 0; j < n; ++j) {
        double a = -6.283185307179586476925286766559 * k * j / n;
        sr += x[(size_t)b * n + j] * std::cos(a), si += x[(size_t)b * n + j] * std::sin(a);
      }
      wv.push_back(sr), wv.push_back(si);
    }
  double e = rel_l2(g, wv);
  printf("fbfft1D<1> N=%d B=%d: rel-L2 %.2e\n", n, B, e);
  cudaFree(dx), cudaFree(dc);
  return e < 1e-5 ? 0 : 1;
}

// transposeMM<5, false, true, false>: C[b][f] = sum_p A[b][p] conj(B[f][p]) per bin
static int check_mm() {
  const int Bn = 3, P = 4, F = 5, R = 5, Cc = 8, X = R * Cc;
  std::vector<float> a((size_t)Bn * P * X * 2), b((size_t)F * P * X * 2);
  srand(7);
  for (auto& v : a) v = 2.f * rand() / RAND_MAX - 1.f;
  for (auto& v : b) v = 2.f * rand() / RAND_MAX - 1.f;
  float *da, *db, *dc;
  CK(cudaMalloc(&da, a.size() * 4));
  CK(cudaMalloc(&db, b.size() * 4));
  CK(cudaMalloc(&dc, (size_t)Bn * F * X * 2 * 4));
  CK(cudaMemcpy(da, a.data(), a.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(db, b.data(), b.size() * 4, cudaMemcpyHostToDevice));
  int sa[5] = {Bn, P, R, Cc, 2}, sb[5] = {F, P, R, Cc, 2}, sc[5] = {Bn, F, R, Cc, 2};
  DeviceTensor<float, 5> A(da, sa), B(db, sb), C(dc, sc);
  transposeMM<5, false, true, false>(A, B, C, 0.5f);
  std::vector<float> got((size_t)Bn * F * X * 2);
  CK(cudaMemcpy(got.data(), dc, got.size() * 4, cudaMemcpyDeviceToHost));
  std::vector<double> g(got.begin(), got.end()), wv;
  for (int i = 0; i < Bn; ++i)
    for (int j = 0; j < F; ++j)
      for (int x = 0; x < X; ++x) {
        double sr = 0, si = 0;
        for (int k = 0; k < P; ++k) {
          double ar = a[(((size_t)i * P + k) * X + x) * 2], ai = a[(((size_t)i * P + k) * X + x) * 2 + 1];
          double br = b[(((size_t)j * P + k) * X + x) * 2], bi = -b[(((size_t)j * P + k) * X + x) * 2 + 1];
          sr += ar * br - ai * bi, si += ar * bi + ai * br;
        }
        wv.push_back(0.5 * sr), wv.push_back(0.5 * si);
      }
  double e = rel_l2(g, wv);
  printf("transposeMM<5,false,true,false>: rel-L2 %.2e\n", e);
  return e < 1e-5 ? 0 : 1;
}

// FFTIteratedConvolution<16>, updateOutput on one tile: out[b][o] = sum_c in[b][c] (x) w[o][c]
// (valid cross-correlation), descriptors in device memory as the reference expects.
static int check_iterated() {
  const int B = 2, C = 3, O = 4, hw = 14, k = 3, oh = hw - k + 1;
  std::vector<float> x((size_t)B * C * hw * hw), w((size_t)O * C * k * k);
  srand(11);
  for (auto& v : x) v = 2.f * rand() / RAND_MAX - 1.f;
  for (auto& v : w) v = 2.f * rand() / RAND_MAX - 1.f;
  float *dx, *dw, *dout;
  CK(cudaMalloc(&dx, x.size() * 4));
  CK(cudaMalloc(&dw, w.size() * 4));
  CK(cudaMalloc(&dout, (size_t)B * O * oh * oh * 4));
  CK(cudaMemcpy(dx, x.data(), x.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(dw, w.data(), w.size() * 4, cudaMemcpyHostToDevice));
  int xs[4] = {B, C, hw, hw}, ws[4] = {O, C, k, k}, os[4] = {B, O, oh, oh};
  DeviceTensor<float, 4> tx(dx, xs), tw(dw, ws), to(dout, os);
  detail::TiledDeviceTensor<float, 4> hin(tx, 0, 0), hout(to, 0, 0), *din, *dtout;
  CK(cudaMalloc(&din, sizeof(hin)));
  CK(cudaMalloc(&dtout, sizeof(hout)));
  CK(cudaMemcpy(din, &hin, sizeof(hin), cudaMemcpyHostToDevice));
  CK(cudaMemcpy(dtout, &hout, sizeof(hout), cudaMemcpyHostToDevice));
  detail::FFTConvolutionPassFFI pass;
  pass.pass = detail::FFTConvolutionPassFFI::FFT_UpdateOutput;
  if (!detail::FFTIteratedConvolution<16>(din, dtout, tw, pass, 1.0f, B, 1, 0)) return printf("iterated conv refused\n"), 1;
  std::vector<float> got((size_t)B * O * oh * oh);
  CK(cudaMemcpy(got.data(), dout, got.size() * 4, cudaMemcpyDeviceToHost));
  std::vector<double> g(got.begin(), got.end()), wv;
  for (int b = 0; b < B; ++b)
    for (int o = 0; o < O; ++o)
      for (int y = 0; y < oh; ++y)
        for (int xx = 0; xx < oh; ++xx) {
          double acc = 0;
          for (int c = 0; c < C; ++c)
            for (int ky = 0; ky < k; ++ky)
              for (int kx = 0; kx < k; ++kx)
                acc += (double)x[(((size_t)b * C + c) * hw + y + ky) * hw + xx + kx] *
                       w[(((size_t)o * C + c) * k + ky) * k + kx];
          wv.push_back(acc);
        }
  double e = rel_l2(g, wv);
  printf("FFTIteratedConvolution<16> updateOutput: rel-L2 %.2e\n", e);
  return e < 1e-4 ? 0 : 1;
}

int main() {
  int bad = 0;
  bad += check_1d(32, 5);
  bad += check_1d(128, 4);
  bad += check_2d(8, 9, 8, 8, 0, 0);
  bad += check_2d(16, 5, 13, 12, 1, 2);
  bad += check_2d(32, 7, 27, 27, 0, 0);
  bad += check_mm();
  bad += check_iterated();
  CK(cudaDeviceSynchronize());
  if (fbfft_b200_device_status() != 0) bad += 1;
  printf(bad ? "FAIL\n" : "PASS\n");
  return bad ? 1 : 0;
}
