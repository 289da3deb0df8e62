// Scalar fp32 CPU restatement of the reference's fbfft algorithm.
//
// TEST INFRASTRUCTURE / CPU BASELINE -- not product code.  Only tests/,
// __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may load
// this library.  The reference has no CPU implementation of this path (every
// function is __device__ or __global__), so this file restates its arithmetic
// step by step in plain C++: the same radix-2 decimation in frequency, the same
// rounded-to-fp32 twiddle values, the same two-reals-in-one-complex packings and
// the same per-bin multiply-accumulate.  Parity is UNPINNED by the reference's
// own tests (it ships none for this path); this port is itself checked against
// the float64 definitions in fbfft_oracle.py.
//
// What each part follows (paths are relative to the reference tree):
//   twiddle values               fbfft/Twiddles.cuh:15-47,322-453
//   radix-2 DIF + bit reversal   fbfft/FBFFTCommon.cuh:432-474,179-222,616-708
//   1-D packing of two signals   fbfft/FBFFTCommon.cuh:307-351,387-430
//   2-D, N <= 32                 fbfft/FFT2D32.cuh:132-219,257-358,361-470
//   2-D, N >= 64 (two passes)    fbfft/FBFFT2D-inl.cuh:230-418,
//                                fbfft/FBIFFT2D-inl.cuh:61-138,252-474
//   per-bin contraction          MM-inl.cuh:188-196,301-326
//   convolution passes           fbfft/FFTIteratedConvolution.cuh:97-207,254-363,409-524
//
// Work is spread over the batch with one std::thread per requested thread.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

namespace {

struct cf {
  float re, im;
};
inline cf mk(float r, float i) { return cf{r, i}; }
inline cf operator+(cf a, cf b) { return mk(a.re + b.re, a.im + b.im); }
inline cf operator-(cf a, cf b) { return mk(a.re - b.re, a.im - b.im); }
inline cf operator*(cf a, cf b) { return mk(a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re); }
inline cf conj(cf a) { return mk(a.re, -a.im); }
inline cf swapri(cf a) { return mk(a.im, a.re); }  // the reference's Complex::transpose()
inline cf scale(cf a, float s) { return mk(a.re * s, a.im * s); }

// kTable[k] = exp(+i * pi * k / 128) rounded to fp32: the reference's 128-entry
// half-circle table.  The per-size constants cexp<N>(k) = exp(i*pi*k/N) it uses
// for N <= 32 are the same values at the same angles.
constexpr int kTableSize = 128;
cf kTable[kTableSize];
struct TableInit {
  TableInit() {
    for (int k = 0; k < kTableSize; ++k) {
      double a = M_PI * (double)k / (double)kTableSize;
      kTable[k] = mk((float)std::cos(a), (float)std::sin(a));
    }
  }
} g_table_init;

// exp(+i*pi*k/n) for n a power of two <= 128, 0 <= k < n
inline cf cexp_pi(int k, int n) { return kTable[k * (kTableSize / n)]; }

inline int bitrev(int v, int bits) {
  int r = 0;
  for (int i = 0; i < bits; ++i) {
    r = (r << 1) | ((v >> i) & 1);
  }
  return r;
}
inline int ilog2(int n) {
  int l = 0;
  while ((1 << l) < n) ++l;
  return l;
}

// In-place radix-2 decimation in frequency over n points with element stride
// `st`, followed by the bit-reversal permutation (natural order in and out).
// forward: exp(-2*pi*i*k*j/n); inverse: exp(+...), unnormalised.  n <= 256.
void fft_dif(cf* a, int n, int st, bool forward) {
  for (int span = n; span >= 2; span >>= 1) {
    int half = span >> 1;
    for (int base = 0; base < n; base += span) {
      for (int j = 0; j < half; ++j) {
        cf& u = a[(base + j) * st];
        cf& v = a[(base + j + half) * st];
        cf s = u + v;
        cf d = u - v;
        // exp(-+ 2*pi*i*j/span) = exp(-+ i*pi*j/half); half <= 128 because n <= 256
        cf w = (j > 0) ? cexp_pi(j, half) : mk(1.f, 0.f);
        if (forward) w = conj(w);
        u = s;
        v = (j == 0) ? d : d * w;
      }
    }
  }
  int bits = ilog2(n);
  for (int i = 0; i < n; ++i) {
    int r = bitrev(i, bits);
    if (i < r) {
      cf t = a[i * st];
      a[i * st] = a[r * st];
      a[r * st] = t;
    }
  }
}

void parallel_for(int count, int nthreads, const std::function<void(int, int)>& body) {
  if (nthreads <= 1 || count <= 1) {
    body(0, count);
    return;
  }
  if (nthreads > count) nthreads = count;
  std::vector<std::thread> pool;
  int per = (count + nthreads - 1) / nthreads;
  for (int t = 0; t < nthreads; ++t) {
    int lo = t * per, hi = std::min(count, lo + per);
    if (lo >= hi) break;
    pool.emplace_back(body, lo, hi);
  }
  for (auto& th : pool) th.join();
}

inline float canvas_at(const float* img, int h, int w, int y, int x, int padU, int padL) {
  unsigned yy = (unsigned)(y - padU), xx = (unsigned)(x - padL);
  return (yy < (unsigned)h && xx < (unsigned)w) ? img[(size_t)yy * w + xx] : 0.f;
}

// ---------------------------------------------------------------- 2-D, N <= 32
// Column pass: N reals of a column as N/2 complex values, half-size transform,
// then the real-transform post-processing that also leaves X[0] and X[N/2]
// packed in a[0] as (X0, XN2).
void vertical_forward(cf* a, int n) {
  int h = n / 2;
  fft_dif(a, h, 1, true);
  a[0] = conj(a[0]) + swapri(a[0]);
  for (int i = 1; i < h / 2; ++i) {
    cf si = scale(a[i] + conj(a[h - i]), 0.5f);
    cf di = scale(a[i] - conj(a[h - i]), 0.5f);
    a[i] = si - di * swapri(cexp_pi(i, h));
    a[h - i] = conj(si) - (scale(conj(di), -1.f)) * swapri(cexp_pi(h - i, h));
  }
  a[h / 2] = conj(a[h / 2]);
}

void vertical_inverse(cf* a, int n) {
  int h = n / 2;
  a[0] = conj(a[0]) + swapri(a[0]);
  for (int i = 1; i < h / 2; ++i) {
    cf si = a[i] + conj(a[h - i]);
    cf di = a[i] - conj(a[h - i]);
    a[i] = si - di * conj(swapri(cexp_pi(i, h)));
    a[h - i] = conj(si) - (scale(conj(di), -1.f) * conj(swapri(cexp_pi(h - i, h))));
  }
  {
    cf si = a[h / 2] + conj(a[h / 2]);
    cf di = a[h / 2] - conj(a[h / 2]);
    a[h / 2] = si - (scale(conj(di), -1.f) * conj(swapri(cexp_pi(h / 2, h))));
  }
  fft_dif(a, h, 1, false);
}

// work[r][t]: r in [0, n/2) packed rows, t in [0, n) columns
void small_forward_packed(const float* img, int h, int w, int n, int padL, int padU, cf* work) {
  int hn = n / 2;
  cf col[16];
  for (int t = 0; t < n; ++t) {
    for (int i = 0; i < n; i += 2) {
      col[i / 2] = mk(canvas_at(img, h, w, i, t, padU, padL), canvas_at(img, h, w, i + 1, t, padU, padL));
    }
    vertical_forward(col, n);
    for (int r = 0; r < hn; ++r) work[r * n + t] = col[r];
  }
  for (int r = 0; r < hn; ++r) fft_dif(work + r * n, n, 1, true);
}

void small_forward(const float* img, int h, int w, int n, int padL, int padU, cf* out /*[n/2+1][n]*/) {
  int hn = n / 2;
  cf work[16 * 32];
  small_forward_packed(img, h, w, n, padL, padU, work);
  for (int r = 1; r < hn; ++r)
    for (int t = 0; t < n; ++t) out[r * n + t] = work[r * n + t];
  out[0] = mk(work[0].re, 0.f);
  out[hn * n] = mk(work[0].im, 0.f);
  for (int t = 1; t < n; ++t) {
    cf me = work[t], other = work[n - t];
    out[t] = scale(conj(other) + me, 0.5f);
    out[hn * n + t] = swapri(conj(scale(conj(other) - me, 0.5f)));
  }
}

// packed rows -> n*n times the canvas
void small_inverse_packed(cf* work, int n, float* canvas /*[n][n]*/) {
  int hn = n / 2;
  for (int r = 0; r < hn; ++r) fft_dif(work + r * n, n, 1, false);
  cf col[16];
  for (int t = 0; t < n; ++t) {
    for (int r = 0; r < hn; ++r) col[r] = work[r * n + t];
    vertical_inverse(col, n);
    for (int i = 0; i < n; i += 2) {
      canvas[i * n + t] = col[i / 2].re;
      canvas[(i + 1) * n + t] = col[i / 2].im;
    }
  }
}

void small_inverse(const cf* in /*[n/2+1][n]*/, int n, float* canvas) {
  int hn = n / 2;
  cf work[16 * 32];
  for (int r = 1; r < hn; ++r)
    for (int t = 0; t < n; ++t) work[r * n + t] = in[r * n + t];
  work[0] = mk(in[0].re, in[hn * n].re);
  for (int t = 1; t < n; ++t) work[t] = in[t] - conj(swapri(in[hn * n + t]));
  small_inverse_packed(work, n, canvas);
}

void crop_store(const float* canvas, int n, float* img, int h, int w, int padL, int padU, float mul) {
  for (int y = 0; y < n; ++y)
    for (int x = 0; x < n; ++x) {
      unsigned yy = (unsigned)(y - padU), xx = (unsigned)(x - padL);
      if (yy < (unsigned)h && xx < (unsigned)w) img[(size_t)yy * w + xx] = canvas[y * n + x] * mul;
    }
}

// ---------------------------------------------------------------- 2-D, N >= 64
// pass 1: rows as complex transforms with a zero imaginary part, first n/2+1 kept
void large_forward_rows(const float* img, int h, int w, int n, int padL, int padU, cf* buf /*[n][n/2+1]*/) {
  int hc = n / 2 + 1;
  std::vector<cf> row(n);
  for (int y = 0; y < n; ++y) {
    for (int x = 0; x < n; ++x) row[x] = mk(canvas_at(img, h, w, y, x, padU, padL), 0.f);
    fft_dif(row.data(), n, 1, true);
    for (int k = 0; k < hc; ++k) buf[y * hc + k] = row[k];
  }
}
// pass 2: transposed read, column transform, dst[kx][ky]
void large_forward_cols(const cf* buf, int n, cf* dst /*[n/2+1][n]*/) {
  int hc = n / 2 + 1;
  for (int kx = 0; kx < hc; ++kx) {
    cf* line = dst + (size_t)kx * n;
    for (int y = 0; y < n; ++y) line[y] = buf[y * hc + kx];
    fft_dif(line, n, 1, true);
  }
}

inline cf hermitian_fetch(const cf* src /*[n/2+1][n]*/, int n, int r, int c) {
  if (r < n / 2 + 1) return src[(size_t)r * n + c];
  return conj(src[(size_t)(n - r) * n + ((n - c) % n)]);
}

// inverse pass 1 on a pair of images: dst[kx][y] = IFFT_ky (Xa + i Xb)[kx][ky]
void large_inverse_rows(const cf* a, const cf* b /*may be null*/, int n, cf* dst /*[n][n]*/) {
  for (int r = 0; r < n; ++r) {
    cf* line = dst + (size_t)r * n;
    for (int c = 0; c < n; ++c) {
      cf v = hermitian_fetch(a, n, r, c);
      if (b) {
        cf t = hermitian_fetch(b, n, r, c);
        v = v + mk(-t.im, t.re);
      }
      line[c] = v;
    }
    fft_dif(line, n, 1, false);
  }
}
// inverse pass 2: IFFT along kx of dst[kx][y]; real -> image a, imag -> image b
void large_inverse_cols(const cf* buf /*[n][n]*/, int n, float* canvas_a, float* canvas_b) {
  std::vector<cf> line(n);
  for (int y = 0; y < n; ++y) {
    for (int kx = 0; kx < n; ++kx) line[kx] = buf[(size_t)kx * n + y];
    fft_dif(line.data(), n, 1, false);
    for (int x = 0; x < n; ++x) {
      canvas_a[y * n + x] = line[x].re;
      if (canvas_b) canvas_b[y * n + x] = line[x].im;
    }
  }
}

void forward_image(const float* img, int h, int w, int n, int padL, int padU, cf* out) {
  if (n <= 32) {
    small_forward(img, h, w, n, padL, padU, out);
  } else {
    std::vector<cf> buf((size_t)n * (n / 2 + 1));
    large_forward_rows(img, h, w, n, padL, padU, buf.data());
    large_forward_cols(buf.data(), n, out);
  }
}

}  // namespace

extern "C" {

int cpuref_hardware_threads() { return (int)std::thread::hardware_concurrency(); }

// real [B][N] -> cplx [B][N/2+1][2]; signals (b, b+1), b even, share one complex transform
void cpuref_fbfft1d(const float* real, float* cplx, int B, int N, int padL, int nthreads) {
  int hc = N / 2 + 1;
  cf* out = reinterpret_cast<cf*>(cplx);
  parallel_for((B + 1) / 2, nthreads, [=](int lo, int hi) {
    std::vector<cf> z(N);
    for (int p = lo; p < hi; ++p) {
      int b0 = 2 * p, b1 = 2 * p + 1;
      for (int x = 0; x < N; ++x) {
        bool in = (x - padL >= 0);
        float r0 = in ? real[(size_t)b0 * N + x - padL] : 0.f;
        float r1 = (in && b1 < B) ? real[(size_t)b1 * N + x - padL] : 0.f;
        z[x] = mk(r0, r1);
      }
      fft_dif(z.data(), N, 1, true);
      for (int m = 0; m < hc; ++m) {
        cf me = z[m], other = z[(N - m) % N];
        out[(size_t)b0 * hc + m] = mk(0.5f * (me.re + other.re), 0.5f * (me.im - other.im));
        if (b1 < B) out[(size_t)b1 * hc + m] = mk(0.5f * (me.im + other.im), 0.5f * (-me.re + other.re));
      }
    }
  });
}

// cplx [B][N/2+1][2] -> real [B][N] = N * x, stored at real[b][x - padL]
void cpuref_fbifft1d(const float* cplx, float* real, int B, int N, int padL, int nthreads) {
  int hc = N / 2 + 1;
  const cf* in = reinterpret_cast<const cf*>(cplx);
  parallel_for((B + 1) / 2, nthreads, [=](int lo, int hi) {
    std::vector<cf> z(N);
    for (int p = lo; p < hi; ++p) {
      int b0 = 2 * p, b1 = 2 * p + 1;
      for (int x = 0; x < N; ++x) {
        cf t1 = (x < hc) ? in[(size_t)b0 * hc + x] : conj(in[(size_t)b0 * hc + (N - x)]);
        cf t2 = mk(0.f, 0.f);
        if (b1 < B) t2 = (x < hc) ? in[(size_t)b1 * hc + x] : conj(in[(size_t)b1 * hc + (N - x)]);
        z[x] = mk(t1.re - t2.im, t1.im + t2.re);
      }
      fft_dif(z.data(), N, 1, false);
      for (int x = padL; x < N; ++x) {
        real[(size_t)b0 * N + x - padL] = z[x].re;
        if (b1 < B) real[(size_t)b1 * N + x - padL] = z[x].im;
      }
    }
  });
}

// real [B][h][w] -> cplx [B][N/2+1][N][2] (layout of the size class)
void cpuref_fbfft2d(const float* real, float* cplx, int B, int h, int w, int N, int padL, int padU, int nthreads) {
  size_t per = (size_t)(N / 2 + 1) * N;
  cf* out = reinterpret_cast<cf*>(cplx);
  parallel_for(B, nthreads, [=](int lo, int hi) {
    for (int b = lo; b < hi; ++b) forward_image(real + (size_t)b * h * w, h, w, N, padL, padU, out + b * per);
  });
}

// N >= 64 first call: real [B][h][w] -> buffer [B][N][N/2+1][2]
void cpuref_fbfft2d_rows(const float* real, float* buffer, int B, int h, int w, int N, int padL, int padU,
                         int nthreads) {
  size_t per = (size_t)(N / 2 + 1) * N;
  cf* out = reinterpret_cast<cf*>(buffer);
  parallel_for(B, nthreads, [=](int lo, int hi) {
    for (int b = lo; b < hi; ++b) large_forward_rows(real + (size_t)b * h * w, h, w, N, padL, padU, out + b * per);
  });
}

// N >= 64 second call: buffer [B][N][N/2+1] -> dst [B][N/2+1][N]
void cpuref_fbfft2d_cols(const float* buffer, float* dst, int B, int N, int nthreads) {
  size_t per = (size_t)(N / 2 + 1) * N;
  const cf* in = reinterpret_cast<const cf*>(buffer);
  cf* out = reinterpret_cast<cf*>(dst);
  parallel_for(B, nthreads, [=](int lo, int hi) {
    for (int b = lo; b < hi; ++b) large_forward_cols(in + b * per, N, out + b * per);
  });
}

// cplx [B][N/2+1][N][2] -> real [B][h][w] = N*N * canvas cropped at (padU, padL)
void cpuref_fbifft2d(const float* cplx, float* real, int B, int h, int w, int N, int padL, int padU, int nthreads) {
  size_t per = (size_t)(N / 2 + 1) * N;
  const cf* in = reinterpret_cast<const cf*>(cplx);
  if (N <= 32) {
    parallel_for(B, nthreads, [=](int lo, int hi) {
      std::vector<float> canvas((size_t)N * N);
      for (int b = lo; b < hi; ++b) {
        small_inverse(in + b * per, N, canvas.data());
        crop_store(canvas.data(), N, real + (size_t)b * h * w, h, w, padL, padU, 1.f);
      }
    });
  } else {
    int G = (B + 1) / 2;
    parallel_for(G, nthreads, [=](int lo, int hi) {
      std::vector<cf> buf((size_t)N * N);
      std::vector<float> ca((size_t)N * N), cb((size_t)N * N);
      for (int p = lo; p < hi; ++p) {
        bool two = p + G < B;
        large_inverse_rows(in + p * per, two ? in + (p + G) * per : nullptr, N, buf.data());
        large_inverse_cols(buf.data(), N, ca.data(), two ? cb.data() : nullptr);
        crop_store(ca.data(), N, real + (size_t)p * h * w, h, w, padL, padU, 1.f);
        if (two) crop_store(cb.data(), N, real + (size_t)(p + G) * h * w, h, w, padL, padU, 1.f);
      }
    });
  }
}

// inverse first call for N >= 64: src [B][N/2+1][N][2] -> dst [B][N][N][2] (first ceil(B/2) slices)
void cpuref_fbifft2d_rows(const float* src, float* dst, int B, int N, int nthreads) {
  size_t per = (size_t)(N / 2 + 1) * N;
  const cf* in = reinterpret_cast<const cf*>(src);
  cf* out = reinterpret_cast<cf*>(dst);
  int G = (B + 1) / 2;
  parallel_for(G, nthreads, [=](int lo, int hi) {
    for (int p = lo; p < hi; ++p)
      large_inverse_rows(in + p * per, (p + G < B) ? in + (p + G) * per : nullptr, N, out + (size_t)p * N * N);
  });
}

// inverse second call for N >= 64
void cpuref_fbifft2d_cols(const float* buffer, float* real, int B, int h, int w, int N, int padL, int padU,
                          int nthreads) {
  const cf* in = reinterpret_cast<const cf*>(buffer);
  int G = (B + 1) / 2;
  parallel_for(G, nthreads, [=](int lo, int hi) {
    std::vector<float> ca((size_t)N * N), cb((size_t)N * N);
    for (int p = lo; p < hi; ++p) {
      bool two = p + G < B;
      large_inverse_cols(in + (size_t)p * N * N, N, ca.data(), two ? cb.data() : nullptr);
      crop_store(ca.data(), N, real + (size_t)p * h * w, h, w, padL, padU, 1.f);
      if (two) crop_store(cb.data(), N, real + (size_t)(p + G) * h * w, h, w, padL, padU, 1.f);
    }
  });
}

// C[i][j][bins] (+)= invNorm * sum_k op(A)[i][k][bins] op(B)[k][j][bins]; op = swap leading indices + conj.
// A is [a0][a1][bins], B is [b0][b1][bins], C is [I][J][bins], all complex, contiguous.
void cpuref_transpose_mm(const float* A, const float* Bm, float* C, int a0, int a1, int b0, int b1, int bins,
                         int conjA, int conjB, int accumulate, float invNorm, int nthreads) {
  const cf* a = reinterpret_cast<const cf*>(A);
  const cf* b = reinterpret_cast<const cf*>(Bm);
  cf* c = reinterpret_cast<cf*>(C);
  int I = conjA ? a1 : a0, K = conjA ? a0 : a1, J = conjB ? b0 : b1;
  parallel_for(I, nthreads, [=](int lo, int hi) {
    std::vector<cf> acc(bins);
    for (int i = lo; i < hi; ++i)
      for (int j = 0; j < J; ++j) {
        for (int x = 0; x < bins; ++x) acc[x] = mk(0.f, 0.f);
        for (int k = 0; k < K; ++k) {
          const cf* pa = conjA ? a + ((size_t)k * a1 + i) * bins : a + ((size_t)i * a1 + k) * bins;
          const cf* pb = conjB ? b + ((size_t)j * b1 + k) * bins : b + ((size_t)k * b1 + j) * bins;
          for (int x = 0; x < bins; ++x) {
            cf va = conjA ? conj(pa[x]) : pa[x];
            cf vb = conjB ? conj(pb[x]) : pb[x];
            acc[x] = acc[x] + va * vb;
          }
        }
        cf* pc = c + ((size_t)i * J + j) * bins;
        for (int x = 0; x < bins; ++x) {
          cf v = scale(acc[x], invNorm);
          pc[x] = accumulate ? pc[x] + v : v;
        }
      }
  });
}

// The three convolution passes on one tile, as forward transforms, per-bin
// multiply-accumulate over planes, inverse transform, crop and scale by 1/N^2.
//   pass 0: out[b][o] = sum_c in[b][c] (x) conj(w[o][c])    -> writes out
//   pass 1: in [b][c] = sum_o out[b][o] (x) w[o][c]         -> writes in
//   pass 2: w  [o][c] = scale * sum_b in[b][c] (x) conj(out[b][o]) -> writes w
// in  [B][C][ih][iw] placed at (inPadU, inPadL); out [B][O][oh][ow] placed at
// (outPadU, outPadL); w [O][C][kh][kw] placed at (0, 0).
void cpuref_conv_pass(int pass, float* in, float* out, float* w, int B, int C, int O, int ih, int iw, int oh, int ow,
                      int kh, int kw, int N, int inPadL, int inPadU, int outPadL, int outPadU, float scale_,
                      int nthreads) {
  size_t per = (size_t)(N / 2 + 1) * N;
  std::vector<cf> fin, fout, fw;
  auto fwd = [&](const float* src, int planes, int h, int ww, int pl, int pu, std::vector<cf>& dst) {
    dst.resize((size_t)planes * per);
    cf* d = dst.data();
    parallel_for(planes, nthreads, [=](int lo, int hi) {
      for (int p = lo; p < hi; ++p) forward_image(src + (size_t)p * h * ww, h, ww, N, pl, pu, d + p * per);
    });
  };
  auto inv = [&](const std::vector<cf>& src, int planes, float* dst, int h, int ww, int pl, int pu, float mul) {
    const cf* s = src.data();
    parallel_for(planes, nthreads, [=](int lo, int hi) {
      std::vector<float> canvas((size_t)N * N);
      std::vector<cf> buf((size_t)N * N);
      for (int p = lo; p < hi; ++p) {
        if (N <= 32) {
          small_inverse(s + p * per, N, canvas.data());
        } else {
          large_inverse_rows(s + p * per, nullptr, N, buf.data());
          large_inverse_cols(buf.data(), N, canvas.data(), nullptr);
        }
        crop_store(canvas.data(), N, dst + (size_t)p * h * ww, h, ww, pl, pu, mul);
      }
    });
  };
  float invn = 1.0f / (float)(N * N);
  int bins = (int)per;
  if (pass == 0) {
    fwd(in, B * C, ih, iw, inPadL, inPadU, fin);
    fwd(w, O * C, kh, kw, 0, 0, fw);
    fout.resize((size_t)B * O * per);
    cpuref_transpose_mm((float*)fin.data(), (float*)fw.data(), (float*)fout.data(), B, C, O, C, bins, 0, 1, 0, 1.f,
                        nthreads);
    inv(fout, B * O, out, oh, ow, outPadL, outPadU, invn);
  } else if (pass == 1) {
    fwd(out, B * O, oh, ow, outPadL, outPadU, fout);
    fwd(w, O * C, kh, kw, 0, 0, fw);
    fin.resize((size_t)B * C * per);
    cpuref_transpose_mm((float*)fout.data(), (float*)fw.data(), (float*)fin.data(), B, O, O, C, bins, 0, 0, 0, 1.f,
                        nthreads);
    inv(fin, B * C, in, ih, iw, inPadL, inPadU, invn);
  } else {
    fwd(in, B * C, ih, iw, inPadL, inPadU, fin);
    fwd(out, B * O, oh, ow, outPadL, outPadU, fout);
    fw.resize((size_t)O * C * per);
    // w[o][c] = sum_b conj(out[b][o]) in[b][c]  (conj-transposed A = out)
    cpuref_transpose_mm((float*)fout.data(), (float*)fin.data(), (float*)fw.data(), B, O, B, C, bins, 1, 0, 0, 1.f,
                        nthreads);
    inv(fw, O * C, w, kh, kw, 0, 0, invn * scale_);
  }
}

}  // extern "C"
