// Transforms built on the block-cooperative shared-memory line FFT:
//   * fbfft1D / fbifft1D for N in {8..256}          (fbfft/FBFFT-inl.cuh:19-150,
//                                                    fbfft/FBFFTCommon.cuh:307-430,797-833)
//   * the reference's two-call protocol for N >= 64 (fbfft/FBFFT2D-inl.cuh:230-444,
//                                                    fbfft/FBIFFT2D-inl.cuh:252-521)
// Real lines are always transformed two at a time as the real and imaginary part
// of one complex line and separated afterwards, as the reference does for its
// 1-D batches (fbfft/FBFFTCommon.cuh:323-350,397-429).
#include "common.cuh"
#include "kernels.h"
#include "smem_fft.cuh"

namespace fbfft_b200 {

namespace {

constexpr int kLineThreads = 256;

template <int M>
constexpr int lines_per_block() {
  return kLineThreads / (Split<M>::R1 > Split<M>::R2 ? Split<M>::R1 : Split<M>::R2);
}
template <int M>
constexpr int line_pitch() {
  return M + 1;
}
template <int M>
constexpr int line_smem_bytes() {
  return (lines_per_block<M>() * line_pitch<M>() + M) * (int)sizeof(float2);
}

// ------------------------------------------------------------------ 1-D forward
template <int N>
__global__ void __launch_bounds__(kLineThreads) fft1d_fwd_kernel(const float* __restrict__ real, long long rs0, int rs1,
                                                                float* __restrict__ cplx, long long cs0, int cs1,
                                                                int cs2, int B, int padL) {
  constexpr int L = lines_per_block<N>(), P = line_pitch<N>();
  extern __shared__ __align__(16) float2 smem[];
  float2* tile = smem;
  float2* tw = smem + L * P;
  fill_twiddles<N>(tw);
  const int pairs = (B + 1) / 2;
  for (int base = blockIdx.x * L; base < pairs; base += gridDim.x * L) {
    const int lines = min(L, pairs - base);
    for (int e = threadIdx.x; e < L * N; e += kLineThreads) {
      const int line = e / N, x = e % N;
      float2 v = make_float2(0.f, 0.f);
      if (line < lines && x >= padL) {
        const int b0 = 2 * (base + line);
        v.x = __ldg(real + b0 * rs0 + (long long)(x - padL) * rs1);
        if (b0 + 1 < B) v.y = __ldg(real + (b0 + 1) * rs0 + (long long)(x - padL) * rs1);
      }
      tile[line * P + x] = v;
    }
    __syncthreads();
    smem_fft_lines<N, false>(tile, P, lines, tw);
    constexpr int H = N / 2 + 1;
    for (int e = threadIdx.x; e < lines * H; e += kLineThreads) {
      const int line = e / H, k = e % H;
      const float2 z = tile[line * P + fft_slot<N>(k)], m = tile[line * P + fft_slot<N>((N - k) % N)];
      const int b0 = 2 * (base + line);
      float* o0 = cplx + b0 * cs0 + (long long)k * cs1;
      o0[0] = 0.5f * (z.x + m.x);
      o0[cs2] = 0.5f * (z.y - m.y);
      if (b0 + 1 < B) {
        float* o1 = o0 + cs0;
        o1[0] = 0.5f * (z.y + m.y);
        o1[cs2] = 0.5f * (m.x - z.x);
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------ 1-D inverse
template <int N>
__global__ void __launch_bounds__(kLineThreads) fft1d_inv_kernel(const float* __restrict__ cplx, long long cs0, int cs1,
                                                                int cs2, float* __restrict__ real, long long rs0,
                                                                int rs1, int B, int padL) {
  constexpr int L = lines_per_block<N>(), P = line_pitch<N>();
  extern __shared__ __align__(16) float2 smem[];
  float2* tile = smem;
  float2* tw = smem + L * P;
  fill_twiddles<N>(tw);
  const int pairs = (B + 1) / 2;
  for (int base = blockIdx.x * L; base < pairs; base += gridDim.x * L) {
    const int lines = min(L, pairs - base);
    for (int e = threadIdx.x; e < L * N; e += kLineThreads) {
      const int line = e / N, x = e % N;
      float2 v = make_float2(0.f, 0.f);
      if (line < lines) {
        const int b0 = 2 * (base + line);
        const bool upper = x > N / 2;
        const int k = upper ? N - x : x;
        const float* s0 = cplx + b0 * cs0 + (long long)k * cs1;
        float2 t1 = make_float2(__ldg(s0), __ldg(s0 + cs2)), t2 = make_float2(0.f, 0.f);
        if (b0 + 1 < B) t2 = make_float2(__ldg(s0 + cs0), __ldg(s0 + cs0 + cs2));
        if (upper) {
          t1.y = -t1.y;
          t2.y = -t2.y;
        }
        v = make_float2(t1.x - t2.y, t1.y + t2.x);
      }
      tile[line * P + x] = v;
    }
    __syncthreads();
    smem_fft_lines<N, true>(tile, P, lines, tw);
    for (int e = threadIdx.x; e < lines * N; e += kLineThreads) {
      const int line = e / N, x = e % N;
      if (x >= padL) {
        const float2 z = tile[line * P + fft_slot<N>(x)];
        const int b0 = 2 * (base + line);
        real[b0 * rs0 + (long long)(x - padL) * rs1] = z.x;
        if (b0 + 1 < B) real[(b0 + 1) * rs0 + (long long)(x - padL) * rs1] = z.y;
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------ 2-D rows, forward (first call, N >= 64)
// grid (row blocks, B).  out[b][y][kx], element at out.p[b*sb + y*sr + kx*sc + z*sz].
template <int N>
__global__ void __launch_bounds__(kLineThreads) rows_fwd_kernel(RealView in, CplxView out, int padL, int padU) {
  constexpr int L = lines_per_block<N>(), P = line_pitch<N>(), H = N / 2 + 1;
  extern __shared__ __align__(16) float2 smem[];
  float2* tile = smem;
  float2* tw = smem + L * P;
  fill_twiddles<N>(tw);
  const int b = blockIdx.y;
  const int y_base = blockIdx.x * 2 * L;  // first canvas row of this block
  const float* src = in.p + (long long)b * in.sb;
  for (int e = threadIdx.x; e < L * N; e += kLineThreads) {
    const int line = e / N, x = e % N;
    const unsigned xx = (unsigned)(x - padL);
    const unsigned y0 = (unsigned)(y_base + 2 * line - padU), y1 = y0 + 1u;
    float2 v = make_float2(0.f, 0.f);
    if (xx < (unsigned)in.w) {
      if (y0 < (unsigned)in.h) v.x = __ldg(src + (long long)y0 * in.sy + (long long)xx * in.sx);
      if (y1 < (unsigned)in.h) v.y = __ldg(src + (long long)y1 * in.sy + (long long)xx * in.sx);
    }
    tile[line * P + x] = v;
  }
  __syncthreads();
  smem_fft_lines<N, false>(tile, P, L, tw);
  float* dst = out.p + (long long)b * out.sb;
  const bool k_fast = out.sc <= out.sr;  // iterate the memory-contiguous index fastest
  for (int e = threadIdx.x; e < L * H; e += kLineThreads) {
    const int line = k_fast ? e / H : e % L, k = k_fast ? e % H : e / L;
    const float2 z = tile[line * P + fft_slot<N>(k)], m = tile[line * P + fft_slot<N>((N - k) % N)];
    const int y = y_base + 2 * line;
    float* o0 = dst + (long long)y * out.sr + (long long)k * out.sc;
    o0[0] = 0.5f * (z.x + m.x);
    o0[out.sz] = 0.5f * (z.y - m.y);
    float* o1 = o0 + out.sr;
    o1[0] = 0.5f * (z.y + m.y);
    o1[out.sz] = 0.5f * (m.x - z.x);
  }
}

// ------------------------------------------------------------------ complex lines (second call, N >= 64)
// Line l of batch b: element i at p[b*sb + l*sl + i*se (+1 for im)].  grid (line blocks, B).
struct LineView {
  float* p;
  long long sb;
  int sl, se;
};

template <int N, bool INV>
__global__ void __launch_bounds__(kLineThreads) lines_c2c_kernel(LineView src, LineView dst, int lines_per_batch) {
  constexpr int L = lines_per_block<N>(), P = line_pitch<N>();
  extern __shared__ __align__(16) float2 smem[];
  float2* tile = smem;
  float2* tw = smem + L * P;
  fill_twiddles<N>(tw);
  const int b = blockIdx.y;
  const int l0 = blockIdx.x * L;
  const int lines = min(L, lines_per_batch - l0);
  const float* s = src.p + (long long)b * src.sb;
  // iterate the memory-contiguous index fastest
  const bool src_elem_fast = src.se <= src.sl;
  for (int e = threadIdx.x; e < L * N; e += kLineThreads) {
    const int line = src_elem_fast ? e / N : e % L, i = src_elem_fast ? e % N : e / L;
    if (line < lines) {
      const float* q = s + (long long)(l0 + line) * src.sl + (long long)i * src.se;
      tile[line * P + i] = make_float2(__ldg(q), __ldg(q + 1));
    }
  }
  __syncthreads();
  smem_fft_lines<N, INV>(tile, P, lines, tw);
  float* d = dst.p + (long long)b * dst.sb;
  const bool dst_elem_fast = dst.se <= dst.sl;
  for (int e = threadIdx.x; e < L * N; e += kLineThreads) {
    const int line = dst_elem_fast ? e / N : e % L, k = dst_elem_fast ? e % N : e / L;
    if (line < lines) {
      const float2 z = tile[line * P + fft_slot<N>(k)];
      float* q = d + (long long)(l0 + line) * dst.sl + (long long)k * dst.se;
      *reinterpret_cast<float2*>(q) = z;
    }
  }
}

// ------------------------------------------------------------------ inverse, first call (N >= 64)
// src [B][N/2+1 (kx)][N (ky)] -> dst[p][kx in 0..N)[y]; p pairs image p with image p+G.
// grid (line blocks over kx, G).
template <int N>
__global__ void __launch_bounds__(kLineThreads) inv_rows_kernel(CplxView src, CplxView dst, int B, int G) {
  constexpr int L = lines_per_block<N>(), P = line_pitch<N>();
  extern __shared__ __align__(16) float2 smem[];
  float2* tile = smem;
  float2* tw = smem + L * P;
  fill_twiddles<N>(tw);
  const int p = blockIdx.y, r0 = blockIdx.x * L;
  const bool two = p + G < B;
  const float* sa = src.p + (long long)p * src.sb;
  const float* sb = src.p + (long long)(p + G) * src.sb;
  for (int e = threadIdx.x; e < L * N; e += kLineThreads) {
    const int line = e / N, c = e % N, r = r0 + line;
    const bool mirror = r > N / 2;
    const int rr = mirror ? N - r : r, cc = mirror ? (N - c) % N : c;
    const long long off = (long long)rr * src.sr + (long long)cc * src.sc;
    float2 a = make_float2(__ldg(sa + off), __ldg(sa + off + src.sz));
    if (mirror) a.y = -a.y;
    if (two) {
      float2 t = make_float2(__ldg(sb + off), __ldg(sb + off + src.sz));
      if (mirror) t.y = -t.y;
      a.x -= t.y;
      a.y += t.x;
    }
    tile[line * P + c] = a;
  }
  __syncthreads();
  smem_fft_lines<N, true>(tile, P, L, tw);
  float* d = dst.p + (long long)p * dst.sb;
  for (int e = threadIdx.x; e < L * N; e += kLineThreads) {
    const int line = e / N, y = e % N;
    const float2 z = tile[line * P + fft_slot<N>(y)];
    float* q = d + (long long)(r0 + line) * dst.sr + (long long)y * dst.sc;
    q[0] = z.x;
    q[dst.sz] = z.y;
  }
}

// ------------------------------------------------------------------ inverse, second call (N >= 64)
// buffer[p][kx][y] -> inverse along kx; real part -> image p, imaginary part -> image p+G.
// grid (line blocks over y, G).
template <int N>
__global__ void __launch_bounds__(kLineThreads) inv_cols_kernel(CplxView buf, RealView out, int B, int G, int padL,
                                                               int padU) {
  constexpr int L = lines_per_block<N>(), P = line_pitch<N>();
  extern __shared__ __align__(16) float2 smem[];
  float2* tile = smem;
  float2* tw = smem + L * P;
  fill_twiddles<N>(tw);
  const int p = blockIdx.y, y0 = blockIdx.x * L;
  const float* s = buf.p + (long long)p * buf.sb;
  for (int e = threadIdx.x; e < L * N; e += kLineThreads) {
    const int line = e % L, kx = e / L;  // y is the contiguous index of the buffer
    const float* q = s + (long long)kx * buf.sr + (long long)(y0 + line) * buf.sc;
    tile[line * P + kx] = make_float2(__ldg(q), __ldg(q + buf.sz));
  }
  __syncthreads();
  smem_fft_lines<N, true>(tile, P, L, tw);
  const bool two = p + G < B;
  float* da = out.p + (long long)p * out.sb;
  float* db = out.p + (long long)(p + G) * out.sb;
  for (int e = threadIdx.x; e < L * N; e += kLineThreads) {
    const int line = e / N, x = e % N;
    const unsigned yy = (unsigned)(y0 + line - padU), xx = (unsigned)(x - padL);
    if (yy < (unsigned)out.h && xx < (unsigned)out.w) {
      const float2 z = tile[line * P + fft_slot<N>(x)];
      const long long off = (long long)yy * out.sy + (long long)xx * out.sx;
      da[off] = z.x;
      if (two) db[off] = z.y;
    }
  }
}

template <typename K>
int finish(K) {
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

template <typename F>
int dispatch_size(int n, F&& f) {
  switch (n) {
    case 8:
      return f(std::integral_constant<int, 8>{});
    case 16:
      return f(std::integral_constant<int, 16>{});
    case 32:
      return f(std::integral_constant<int, 32>{});
    case 64:
      return f(std::integral_constant<int, 64>{});
    case 128:
      return f(std::integral_constant<int, 128>{});
    case 256:
      return f(std::integral_constant<int, 256>{});
    default:
      set_last_error("unsupported transform size");
      return kUnsupportedSize;
  }
}

}  // namespace

int fft1d_forward(int n, const float* real, int rs0, int rs1, float* cplx, int cs0, int cs1, int cs2, int B, int padL,
                  cudaStream_t s) {
  if (B >= 64 && fft1d_fast_supported(n, real, rs0, rs1, cplx, cs0, cs1, cs2, padL)) {
    // whole groups of signals through the register kernels, the rest below
    const int g = fft1d_fast_group(n), done = (B / g) * g;
    if (int rc = fft1d_fast(n, false, real, cplx, B / g, s)) return rc;
    if (done == B) return kSuccess;
    real += (long long)done * rs0, cplx += (long long)done * cs0, B -= done;
  } else if (B >= 64 && rs1 == 1 && cs2 == 1 && cs1 == 2 && cs0 == n + 2 &&
             fft1d_fast_ragged_supported(n, real, rs0, 0, 1, n - padL, padL, 0, 1, cplx)) {
    // a stride between the signals or a left pad (in 16-byte units): same kernels, one bulk copy per signal
    const int g = fft1d_fast_group(n), done = (B / g) * g;
    if (int rc = fft1d_fast_ragged(n, real, rs0, 0, 1, n - padL, padL, 0, 1, cplx, B / g, s)) return rc;
    if (done == B) return kSuccess;
    real += (long long)done * rs0, cplx += (long long)done * cs0, B -= done;
  }
  return dispatch_size(n, [&](auto nc) {
    constexpr int N = decltype(nc)::value;
    const int pairs = (B + 1) / 2, L = lines_per_block<N>();
    const int want = (pairs + L - 1) / L, cap = sm_count() * 8;
    fft1d_fwd_kernel<N><<<want < cap ? want : cap, kLineThreads, line_smem_bytes<N>(), s>>>(real, rs0, rs1, cplx, cs0,
                                                                                          cs1, cs2, B, padL);
    return finish(0);
  });
}

int fft1d_inverse(int n, const float* cplx, int cs0, int cs1, int cs2, float* real, int rs0, int rs1, int B, int padL,
                  cudaStream_t s) {
  if (B >= 64 && fft1d_fast_supported(n, real, rs0, rs1, cplx, cs0, cs1, cs2, padL)) {
    const int g = fft1d_fast_group(n), done = (B / g) * g;
    if (int rc = fft1d_fast(n, true, cplx, real, B / g, s)) return rc;
    if (done == B) return kSuccess;
    real += (long long)done * rs0, cplx += (long long)done * cs0, B -= done;
  } else if (B >= 64 && rs1 == 1 && cs2 == 1 && cs1 == 2 && cs0 == n + 2 &&
             fft1d_fast_ragged_supported(n, real, rs0, 0, 1, n - padL, padL, 0, 1, cplx)) {
    // a stride between the signals or a left pad (in 16-byte units): x = padL .. N - 1 of every result goes to
    // the start of its row
    const int g = fft1d_fast_group(n), done = (B / g) * g;
    if (int rc = fft1d_fast_ragged_inverse(n, cplx, real, rs0, 0, 1, n - padL, padL, 0, 1, B / g, s)) return rc;
    if (done == B) return kSuccess;
    real += (long long)done * rs0, cplx += (long long)done * cs0, B -= done;
  }
  return dispatch_size(n, [&](auto nc) {
    constexpr int N = decltype(nc)::value;
    const int pairs = (B + 1) / 2, L = lines_per_block<N>();
    const int want = (pairs + L - 1) / L, cap = sm_count() * 8;
    fft1d_inv_kernel<N><<<want < cap ? want : cap, kLineThreads, line_smem_bytes<N>(), s>>>(cplx, cs0, cs1, cs2, real,
                                                                                          rs0, rs1, B, padL);
    return finish(0);
  });
}

int fft2d_large_rows_forward(int n, const RealView& in, const CplxView& buffer, int B, int padL, int padU,
                             cudaStream_t s) {
  if (n < 64) return kUnsupportedSize;
  // contiguous N x N images into a contiguous [B][N][N/2+1] buffer: the row pass is a batch of
  // B * N 1-D transforms (whole groups of rows; N is a multiple of the group)
  if (n <= 256 && padL == 0 && padU == 0 && in.h == n && in.w == n && in.sx == 1 && in.sy == n && !buffer.blk_planes &&
      buffer.sz == 1 && buffer.sc == 2 && buffer.sr == n + 2 && (B <= 1 || (in.sb == (long long)n * n && buffer.sb == (long long)n * (n + 2))) &&
      fft1d_fast_supported(n, in.p, n, 1, buffer.p, n + 2, 2, 1, 0)) {
    return fft1d_fast(n, false, in.p, buffer.p, (long long)B * n / fft1d_fast_group(n), s);
  }
  // zero-padded images (rows of whole 16-byte units) into the same contiguous buffer: the row pass is still a
  // batch of B * N 1-D transforms, every canvas row fetched by one bulk copy of its w floats
  if (n <= 256 && in.sx == 1 && !buffer.blk_planes && buffer.sz == 1 && buffer.sc == 2 && buffer.sr == n + 2 &&
      (B <= 1 || buffer.sb == (long long)n * (n + 2)) && in.h <= n - padU && padU >= 0 &&
      fft1d_fast_ragged_supported(n, in.p, in.sb, in.sy, in.h, in.w, padL, padU, n, buffer.p)) {
    return fft1d_fast_ragged(n, in.p, in.sb, in.sy, in.h, in.w, padL, padU, n, buffer.p,
                             (long long)B * n / fft1d_fast_group(n), s);
  }
  return dispatch_size(n, [&](auto nc) {
    constexpr int N = decltype(nc)::value;
    if constexpr (N >= 64) {
      constexpr int L = lines_per_block<N>();
      for (int b0 = 0; b0 < B; b0 += 65535) {
        const int nb = B - b0 < 65535 ? B - b0 : 65535;
        RealView i2 = in;
        i2.p += (long long)b0 * in.sb;
        CplxView o2 = buffer;
        o2.p += (long long)b0 * buffer.sb;
        rows_fwd_kernel<N><<<dim3(N / (2 * L), nb), kLineThreads, line_smem_bytes<N>(), s>>>(i2, o2, padL, padU);
      }
      return finish(0);
    }
    return (int)kUnsupportedSize;
  });
}

int fft2d_large_cols_forward(int n, const CplxView& buffer, const CplxView& dst, int B, cudaStream_t s) {
  if (n < 64) return kUnsupportedSize;
  if (buffer.sz != 1 || dst.sz != 1) {
    set_last_error("complex tensors must interleave re/im");
    return kUnsupportedDimension;
  }
  if (fft2d_cols_fast_supported(n, buffer, dst, B)) return fft2d_cols_fast(n, buffer, dst, B, s);
  return dispatch_size(n, [&](auto nc) {
    constexpr int N = decltype(nc)::value;
    if constexpr (N >= 64) {
      constexpr int L = lines_per_block<N>(), H = N / 2 + 1;
      for (int b0 = 0; b0 < B; b0 += 65535) {
        const int nb = B - b0 < 65535 ? B - b0 : 65535;
        // source line = column kx of buffer[y][kx]; destination line = row kx of dst[kx][ky]
        LineView sv{buffer.p + (long long)b0 * buffer.sb, buffer.sb, buffer.sc, buffer.sr};
        LineView dv{dst.p + (long long)b0 * dst.sb, dst.sb, dst.sr, dst.sc};
        lines_c2c_kernel<N, false><<<dim3((H + L - 1) / L, nb), kLineThreads, line_smem_bytes<N>(), s>>>(sv, dv, H);
      }
      return finish(0);
    }
    return (int)kUnsupportedSize;
  });
}

int fft_lines_inplace(int n, const CplxView& t, int B, int lines, bool inverse, cudaStream_t s) {
  if (t.sz != 1) {
    set_last_error("complex tensors must interleave re/im");
    return kUnsupportedDimension;
  }
  return dispatch_size(n, [&](auto nc) {
    constexpr int N = decltype(nc)::value;
    constexpr int L = lines_per_block<N>();
    for (int b0 = 0; b0 < B; b0 += 65535) {
      const int nb = B - b0 < 65535 ? B - b0 : 65535;
      LineView v{t.p + (long long)b0 * t.sb, t.sb, t.sr, t.sc};
      if (inverse) {
        lines_c2c_kernel<N, true><<<dim3((lines + L - 1) / L, nb), kLineThreads, line_smem_bytes<N>(), s>>>(v, v, lines);
      } else {
        lines_c2c_kernel<N, false><<<dim3((lines + L - 1) / L, nb), kLineThreads, line_smem_bytes<N>(), s>>>(v, v, lines);
      }
    }
    return finish(0);
  });
}

int fft2d_large_rows_inverse(int n, const CplxView& src, const CplxView& buffer, int B, cudaStream_t s) {
  if (n < 64) return kUnsupportedSize;
  if (fft2d_rows_inv_fast_supported(n, src, buffer, B)) return fft2d_rows_inv_fast(n, src, buffer, B, s);
  return dispatch_size(n, [&](auto nc) {
    constexpr int N = decltype(nc)::value;
    if constexpr (N >= 64) {
      constexpr int L = lines_per_block<N>();
      const int G = (B + 1) / 2;
      for (int p0 = 0; p0 < G; p0 += 65535) {
        // pairs are (p, p + G): shifting both views by p0 keeps the pairing
        const int np = G - p0 < 65535 ? G - p0 : 65535;
        CplxView s2 = src, d2 = buffer;
        s2.p += (long long)p0 * src.sb;
        d2.p += (long long)p0 * buffer.sb;
        inv_rows_kernel<N><<<dim3(N / L, np), kLineThreads, line_smem_bytes<N>(), s>>>(s2, d2, B - p0, G);
      }
      return finish(0);
    }
    return (int)kUnsupportedSize;
  });
}

int fft2d_large_cols_inverse(int n, const CplxView& buffer, const RealView& out, int B, int padL, int padU,
                             cudaStream_t s) {
  if (n < 64) return kUnsupportedSize;
  if (fft2d_cols_inv_fast_supported(n, buffer, out, B, padL, padU)) return fft2d_cols_inv_fast(n, buffer, out, B, padL, padU, s);
  return dispatch_size(n, [&](auto nc) {
    constexpr int N = decltype(nc)::value;
    if constexpr (N >= 64) {
      constexpr int L = lines_per_block<N>();
      const int G = (B + 1) / 2;
      for (int p0 = 0; p0 < G; p0 += 65535) {
        const int np = G - p0 < 65535 ? G - p0 : 65535;
        CplxView b2 = buffer;
        b2.p += (long long)p0 * buffer.sb;
        RealView o2 = out;
        o2.p += (long long)p0 * out.sb;
        inv_cols_kernel<N><<<dim3(N / L, np), kLineThreads, line_smem_bytes<N>(), s>>>(b2, o2, B - p0, G, padL, padU);
      }
      return finish(0);
    }
    return (int)kUnsupportedSize;
  });
}

}  // namespace fbfft_b200
