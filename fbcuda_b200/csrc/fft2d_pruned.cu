// 2-D transforms of images with a small support (convolution weights: 3x3, 5x5, 7x7 inside an
// N x N canvas) evaluated directly instead of through N-point butterflies.  Same results and
// layouts as the general kernels: stored spectrum S[r][c], r in 0..N/2, c in 0..N-1, with
// (r, c) = (ky, kx) for N <= 32 and (kx, ky) for N >= 64 (the reference's two size classes,
// fbfft/FBFFT2D-inl.cuh:480-617); unnormalised inverse (fbfft/FBIFFT2D-inl.cuh:535-669).
//
//   forward   S[r][c] = sum_b w^(c (b + pb)) * G[r][b],   G[r][b] = sum_a w^(r (a + pa)) * img[a][b]
//             (a, b = the image coordinates that pair with r and c; w = exp(-2 pi i / N)).
//             G is (N/2+1) x support values per plane in shared memory; thread c keeps its
//             `support` twiddles in registers and walks r: `support` complex multiply-adds per
//             bin instead of a share of two N-point FFTs, so the kernel is bound by its stores.
//   inverse   img[a][b] = Re sum_c w^-(c (b + pb)) T[a][c],  T[a][c] = sum_r g_r w^-(r (a + pa)) S[r][c]
//             with g_r = 1 for r = 0 and N/2, else 2 (Hermitian symmetry of a real image's
//             spectrum); thread c accumulates T[.][c] over r from coalesced loads, then the
//             support x support real sums are reduced over c with shuffles.
// One block handles 128 / N planes at a time (N = 128: one).
#include "fft2d_small.cuh"
#include "kernels.h"

namespace fbfft_b200 {

namespace {

constexpr int kThreadsP = 128;
constexpr int kMaxSupport = 8;

__device__ __forceinline__ float2 cmulf(float2 a, float2 b) { return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x); }

// address (in floats) of stored bin (r, c) of plane P
template <int N>
__device__ __forceinline__ long long bin_offset(const CplxView& v, long long P, int r, int c) {
  if (v.blk_planes) {
    const int x = r * N + c, sh = v.blk_bins == 4 ? 2 : 4;  // blocks of 4 or 16 bins
    return ((((long long)(x >> sh) * v.blk_planes + P) << sh) + (x & ((1 << sh) - 1))) * 2;
  }
  return P * v.sb + (long long)r * v.sr + (long long)c * v.sc;
}

template <int N>
__global__ void __launch_bounds__(kThreadsP) pruned_fwd_kernel(RealView in, CplxView out, int planes, int padL, int padU) {
  constexpr int G = kThreadsP / N, HR = N / 2 + 1;
  constexpr bool TR = N >= 64;  // stored rows are kx: the roles of x and y swap
  __shared__ float2 tw[N];
  __shared__ float img[G][kMaxSupport * kMaxSupport];
  __shared__ float2 gs[G][HR][kMaxSupport];
  const int tid = threadIdx.x, g = tid / N, c = tid % N;
  // extents along a (pairs with r) and b (pairs with c), and their offsets inside the canvas
  const int na = TR ? in.w : in.h, nb = TR ? in.h : in.w, pa = TR ? padL : padU, pb = TR ? padU : padL;
  for (int i = tid; i < N; i += kThreadsP) {
    float sn, cs;
    sincospif(-2.0f * (float)i / (float)N, &sn, &cs);
    tw[i] = make_float2(cs, sn);
  }
  float2 twc[kMaxSupport];
  for (int p0 = blockIdx.x * G; p0 < planes; p0 += gridDim.x * G) {
    __syncthreads();  // the previous planes' G and image are consumed (and the table is written)
    for (int i = tid; i < G * na * nb; i += kThreadsP) {
      const int gg = i / (na * nb), rem = i % (na * nb), a = rem / nb, b = rem % nb;
      const int y = TR ? b : a, x = TR ? a : b;
      const long long P = p0 + gg;
      // canvas semantics: what falls outside the N x N canvas is dropped
      const bool ok = P < planes && a + pa < N && b + pb < N;
      img[gg][a * kMaxSupport + b] = ok ? in.p[P * in.sb + (long long)y * in.sy + (long long)x * in.sx] : 0.f;
    }
    __syncthreads();
    for (int i = tid; i < G * HR * nb; i += kThreadsP) {
      const int gg = i / (HR * nb), rem = i % (HR * nb), r = rem / nb, b = rem % nb;
      float2 acc = make_float2(0.f, 0.f);
      for (int a = 0; a < na; ++a) {
        const float2 t = tw[(r * (a + pa)) & (N - 1)];
        const float v = img[gg][a * kMaxSupport + b];
        acc.x += v * t.x, acc.y += v * t.y;
      }
      gs[gg][r][b] = acc;
    }
#pragma unroll
    for (int b = 0; b < kMaxSupport; ++b) twc[b] = (b < nb) ? tw[(c * (b + pb)) & (N - 1)] : make_float2(0.f, 0.f);
    __syncthreads();
    const long long P = p0 + g;
    if (P < planes) {
      // stored row r of column c: the offset is linear in r in both layouts
      float* dst = out.p + bin_offset<N>(out, P, 0, c);
      const long long rstride = bin_offset<N>(out, P, 1, c) - bin_offset<N>(out, P, 0, c);
      for (int r = 0; r < HR; ++r, dst += rstride) {
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int b = 0; b < kMaxSupport; ++b) {
          if (b < nb) {
            const float2 v = gs[g][r][b];
            acc.x += v.x * twc[b].x - v.y * twc[b].y;
            acc.y += v.x * twc[b].y + v.y * twc[b].x;
          }
        }
        *reinterpret_cast<float2*>(dst) = acc;
      }
    }
  }
}

template <int N>
__global__ void __launch_bounds__(kThreadsP) pruned_inv_kernel(CplxView in, RealView out, int planes, int padL, int padU) {
  constexpr int G = kThreadsP / N, HR = N / 2 + 1;
  constexpr bool TR = N >= 64;
  constexpr int WPG = (N + 31) / 32;  // warps per plane (N = 16: two planes share a warp)
  __shared__ float2 tw[N];  // exp(+2 pi i n / N)
  __shared__ float red[G][WPG][kMaxSupport * kMaxSupport];
  const int tid = threadIdx.x, g = tid / N, c = tid % N, lane = tid & 31;
  const int na = TR ? out.w : out.h, nb = TR ? out.h : out.w, pa = TR ? padL : padU, pb = TR ? padU : padL;
  for (int i = tid; i < N; i += kThreadsP) {
    float sn, cs;
    sincospif(2.0f * (float)i / (float)N, &sn, &cs);
    tw[i] = make_float2(cs, sn);
  }
  __syncthreads();
  for (int p0 = blockIdx.x * G; p0 < planes; p0 += gridDim.x * G) {
    const long long P = p0 + g;
    const bool live = P < planes;
    float2 T[kMaxSupport];
#pragma unroll
    for (int a = 0; a < kMaxSupport; ++a) T[a] = make_float2(0.f, 0.f);
    // rows in batches of RB: all loads of a batch are in flight before the first is used.  Every
    // row is accumulated with weight 2; rows 0 and N/2 (weight 1) are corrected afterwards.
    constexpr int RB = 11;
    const float* src = in.p + bin_offset<N>(in, live ? P : 0, 0, c);
    const long long rstride = bin_offset<N>(in, 0, 1, c) - bin_offset<N>(in, 0, 0, c);
    int idx[kMaxSupport];  // (r * (a + pa)) mod N, advanced by a + pa per row
#pragma unroll
    for (int a = 0; a < kMaxSupport; ++a) idx[a] = 0;
    float2 f_first = make_float2(0.f, 0.f), f_last = make_float2(0.f, 0.f);
    for (int r0 = 0; r0 < HR; r0 += RB) {
      float2 f[RB];
#pragma unroll
      for (int i = 0; i < RB; ++i) {
        f[i] = make_float2(0.f, 0.f);
        if (live && r0 + i < HR) f[i] = __ldg(reinterpret_cast<const float2*>(src + (long long)(r0 + i) * rstride));
      }
#pragma unroll
      for (int i = 0; i < RB; ++i) {
        const int r = r0 + i;
        if (r < HR) {
          if (r == 0) f_first = f[i];
          if (r == N / 2) f_last = f[i];
#pragma unroll
          for (int a = 0; a < kMaxSupport; ++a) {
            if (a < na) {
              const float2 t = tw[idx[a]];
              idx[a] = (idx[a] + a + pa) & (N - 1);
              T[a].x += f[i].x * t.x - f[i].y * t.y;
              T[a].y += f[i].x * t.y + f[i].y * t.x;
            }
          }
        }
      }
    }
#pragma unroll
    for (int a = 0; a < kMaxSupport; ++a) {
      // 2 * sum - f[0] - f[N/2] * w^-(N/2 (a + pa)),  w^-(N/2 j) = (-1)^j
      const float sg = ((a + pa) & 1) ? -1.f : 1.f;
      T[a].x = 2.f * T[a].x - f_first.x - sg * f_last.x;
      T[a].y = 2.f * T[a].y - f_first.y - sg * f_last.y;
    }
    // out[a][b] = sum_c Re(T[a][c] * w^-(c (b + pb))): reduce over the lanes that share a plane
#pragma unroll
    for (int a = 0; a < kMaxSupport; ++a) {
      if (a < na) {
        for (int b = 0; b < nb; ++b) {
          const float2 t = tw[(c * (b + pb)) & (N - 1)];
          float v = T[a].x * t.x - T[a].y * t.y;
          constexpr int SPAN = N < 32 ? N : 32;
#pragma unroll
          for (int o = SPAN / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if ((lane & (SPAN - 1)) == 0) red[g][(c / 32) % WPG][a * kMaxSupport + b] = v;
        }
      }
    }
    __syncthreads();
    for (int i = tid; i < G * na * nb; i += kThreadsP) {
      const int gg = i / (na * nb), rem = i % (na * nb), a = rem / nb, b = rem % nb;
      const long long Pp = p0 + gg;
      if (Pp < planes) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WPG; ++w) v += red[gg][w][a * kMaxSupport + b];
        const int y = TR ? b : a, x = TR ? a : b;
        out.p[Pp * out.sb + (long long)y * out.sy + (long long)x * out.sx] = v;
      }
    }
    __syncthreads();
  }
}

bool view_ok(const CplxView& v) {
  if (v.blk_planes) return aligned16(v.p);
  return v.sz == 1 && v.sc == 2 && (v.sr % 2) == 0 && (v.sb % 2) == 0 && (reinterpret_cast<uintptr_t>(v.p) & 7u) == 0;
}

}  // namespace

// images with a support of at most 8 x 8 that lies inside the canvas, complex side contiguous
// in (re, im) pairs
bool fft2d_pruned_supported(int n, const RealView& real, const CplxView& cplx, int padL, int padU) {
  if (n != 16 && n != 32 && n != 64 && n != 128) return false;
  if (real.h < 1 || real.w < 1 || real.h > kMaxSupport || real.w > kMaxSupport) return false;
  if (padL < 0 || padU < 0 || real.h + padU > n || real.w + padL > n) return false;
  return view_ok(cplx);
}

int fft2d_pruned_forward(int n, const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s) {
  const int per = kThreadsP / n;
  const int want = (B + per - 1) / per, cap = sm_count() * 8;
  const int grid = want < cap ? want : cap;
  switch (n) {
    case 16: pruned_fwd_kernel<16><<<grid, kThreadsP, 0, s>>>(in, out, B, padL, padU); break;
    case 32: pruned_fwd_kernel<32><<<grid, kThreadsP, 0, s>>>(in, out, B, padL, padU); break;
    case 64: pruned_fwd_kernel<64><<<grid, kThreadsP, 0, s>>>(in, out, B, padL, padU); break;
    case 128: pruned_fwd_kernel<128><<<grid, kThreadsP, 0, s>>>(in, out, B, padL, padU); break;
    default: return kUnsupportedSize;
  }
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

int fft2d_pruned_inverse(int n, const CplxView& in, const RealView& out, int B, int padL, int padU, cudaStream_t s) {
  const int per = kThreadsP / n;
  const int want = (B + per - 1) / per, cap = sm_count() * 8;
  const int grid = want < cap ? want : cap;
  switch (n) {
    case 16: pruned_inv_kernel<16><<<grid, kThreadsP, 0, s>>>(in, out, B, padL, padU); break;
    case 32: pruned_inv_kernel<32><<<grid, kThreadsP, 0, s>>>(in, out, B, padL, padU); break;
    case 64: pruned_inv_kernel<64><<<grid, kThreadsP, 0, s>>>(in, out, B, padL, padU); break;
    case 128: pruned_inv_kernel<128><<<grid, kThreadsP, 0, s>>>(in, out, B, padL, padU); break;
    default: return kUnsupportedSize;
  }
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

}  // namespace fbfft_b200
