// Forward 2-D transforms of images with a small support (convolution weights: 3x3 ... 8x8 inside
// an N x N canvas) evaluated directly instead of through N-point butterflies.  Same results and
// layouts as the general kernels: stored spectrum S[r][c], r in 0..N/2, c in 0..N-1, with
// (r, c) = (ky, kx) for N <= 32 and (kx, ky) for N >= 64 (the reference's two size classes,
// fbfft/FBFFT2D-inl.cuh:480-617).
//
//   forward   S[r][c] = sum_b w^(c (b + pb)) * G[r][b],   G[r][b] = sum_a w^(r (a + pa)) * img[a][b]
//             (a, b = the image coordinates that pair with r and c; w = exp(-2 pi i / N)).
//             G is (N/2+1) x support values per plane in shared memory; a thread keeps the
//             `support` twiddles of two adjacent columns in registers and walks r: `support` complex multiply-adds per
//             bin instead of a share of two N-point FFTs, so the kernel is bound by its stores.
// One block handles 256 / N planes at a time.
#include "fft2d_small.cuh"
#include "kernels.h"

namespace fbfft_b200 {

namespace {

constexpr int kThreadsP = 128;
constexpr int kMaxSupport = 8;

// address (in floats) of stored bin (r, c) of plane P
template <int N>
__device__ __forceinline__ long long bin_offset(const CplxView& v, long long P, int r, int c) {
  if (v.blk_planes) {
    const int x = r * N + c, sh = 31 - __clz(v.blk_bins);  // blocks of 4 or N bins (powers of two)
    return ((((long long)(x >> sh) * v.blk_planes + P) << sh) + (x & ((1 << sh) - 1))) * 2;
  }
  return P * v.sb + (long long)r * v.sr + (long long)c * v.sc;
}

// MB: compile-time bound of the support along b (4 or 8)
template <int N, int MB>
__global__ void __launch_bounds__(kThreadsP) pruned_fwd_kernel(RealView in, CplxView out, int planes, int padL, int padU) {
  constexpr int TPP = N / 2;  // threads per plane: each takes two adjacent columns (16-byte stores)
  constexpr int G = kThreadsP / TPP, HR = N / 2 + 1;
  constexpr bool TR = N >= 64;  // stored rows are kx: the roles of x and y swap
  __shared__ float2 tw[N];
  __shared__ float img[G][kMaxSupport * kMaxSupport];
  __shared__ float2 gs[G][HR][MB];
  const int tid = threadIdx.x, g = tid / TPP, c = 2 * (tid % TPP);
  // extents along a (pairs with r) and b (pairs with c), and their offsets inside the canvas
  const int na = TR ? in.w : in.h, nb = TR ? in.h : in.w, pa = TR ? padL : padU, pb = TR ? padU : padL;
  for (int i = tid; i < N; i += kThreadsP) {
    float sn, cs;
    sincospif(-2.0f * (float)i / (float)N, &sn, &cs);
    tw[i] = make_float2(cs, sn);
  }
  float2 twc[MB], twd[MB];  // twiddles of columns c and c + 1
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
    for (int b = 0; b < MB; ++b) {
      twc[b] = (b < nb) ? tw[(c * (b + pb)) & (N - 1)] : make_float2(0.f, 0.f);
      twd[b] = (b < nb) ? tw[((c + 1) * (b + pb)) & (N - 1)] : make_float2(0.f, 0.f);
    }
    __syncthreads();
    const long long P = p0 + g;
    if (P < planes) {
      // stored row r of column c: the offset is linear in r in both layouts
      float* dst = out.p + bin_offset<N>(out, P, 0, c);
      const long long rstride = bin_offset<N>(out, P, 1, c) - bin_offset<N>(out, P, 0, c);
      for (int r = 0; r < HR; ++r, dst += rstride) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int b = 0; b < MB; ++b) {
          if (b < nb) {
            const float2 v = gs[g][r][b];
            acc.x += v.x * twc[b].x - v.y * twc[b].y;
            acc.y += v.x * twc[b].y + v.y * twc[b].x;
            acc.z += v.x * twd[b].x - v.y * twd[b].y;
            acc.w += v.x * twd[b].y + v.y * twd[b].x;
          }
        }
        *reinterpret_cast<float4*>(dst) = acc;
      }
    }
  }
}

bool view_ok(const CplxView& v) {
  if (v.blk_planes) return aligned16(v.p);
  return v.sz == 1 && v.sc == 2 && (v.sr % 4) == 0 && (v.sb % 4) == 0 && aligned16(v.p);
}

}  // namespace

// images with a support of at most 8 x 8 that lies inside the canvas (measured: at 13 x 13 the
// butterflies win again), complex side contiguous
// in (re, im) pairs
bool fft2d_pruned_supported(int n, const RealView& real, const CplxView& cplx, int padL, int padU) {
  if (n != 16 && n != 32 && n != 64 && n != 128) return false;
  if (real.h < 1 || real.w < 1 || real.h > kMaxSupport || real.w > kMaxSupport) return false;
  if (padL < 0 || padU < 0 || real.h + padU > n || real.w + padL > n) return false;
  return view_ok(cplx);
}

template <int N>
static void launch_pruned(const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s) {
  const int per = kThreadsP / (N / 2);
  const int want = (B + per - 1) / per, cap = sm_count() * 8;
  const int grid = want < cap ? want : cap;
  const int nb = N >= 64 ? in.h : in.w;
  if (nb <= 4) {
    pruned_fwd_kernel<N, 4><<<grid, kThreadsP, 0, s>>>(in, out, B, padL, padU);
  } else {
    pruned_fwd_kernel<N, 8><<<grid, kThreadsP, 0, s>>>(in, out, B, padL, padU);
  }
}

int fft2d_pruned_forward(int n, const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s) {
  switch (n) {
    case 16: launch_pruned<16>(in, out, B, padL, padU, s); break;
    case 32: launch_pruned<32>(in, out, B, padL, padU, s); break;
    case 64: launch_pruned<64>(in, out, B, padL, padU, s); break;
    case 128: launch_pruned<128>(in, out, B, padL, padU, s); break;
    default: return kUnsupportedSize;
  }
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

}  // namespace fbfft_b200
