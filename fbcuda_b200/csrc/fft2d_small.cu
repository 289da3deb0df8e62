// Batched 2-D real-to-complex / complex-to-real FFTs for N in {8, 16, 32}.
//
// Replaces the reference's fbfft2DVertical_{8,16,32} / fbifft2DVertical_{8,16,32}
// kernels (fbfft/FFT2D32.cuh:361-533, dispatched from fbfft/FBFFT2D-inl.cuh:476-570
// and fbfft/FBIFFT2D-inl.cuh:591-682).  Output layout is the reference's for this
// size class: [B][ky in 0..N/2][kx in 0..N) complex, Hermitian half along the ROW
// frequency; inverse is unnormalised (returns N*N*x) and crops at (padU, padL).
//
// Design: a warp owns 32/(N/2) images at a time and never synchronises with any
// other warp.  Both passes are length-N complex FFTs held entirely in one
// thread's registers:
//   pass A  thread (image, l) loads columns l and l+N/2 as re/im of one complex
//           line (coalesced 4-byte loads, zero padding by predicate), transforms
//           it and separates the two real-input spectra; rows 0 and N/2 are real
//           and travel packed as one complex row;
//   pass B  after a transpose through padded shared memory, thread (image, r)
//           transforms packed row r; row 0 is then unpacked into rows 0 and N/2;
//   store   the finished (N/2+1) x N block is copied out with 16-byte stores.
// The inverse runs the same passes backwards.  No twiddle is ever shuffled or
// read from memory.
#include "common.cuh"
#include "fft_regs.cuh"

namespace fbfft_b200 {

namespace {

// Shared-memory pitches in float2 units: RS between rows of an image, IS between
// images of a warp.  Chosen by exhaustive search so that the 8-byte column writes
// of pass A, the 16-byte row reads of pass B and the 16-byte copy-out are free of
// bank conflicts (N = 8 keeps a 2-way conflict on the row reads).
template <int N>
struct SmallCfg;
template <>
struct SmallCfg<8> {
  static constexpr int RS = 8, IS = 44;
};
template <>
struct SmallCfg<16> {
  static constexpr int RS = 18, IS = 168;
};
template <>
struct SmallCfg<32> {
  static constexpr int RS = 34, IS = 578;
};

constexpr int kSmallThreads = 128;

template <int N>
__device__ __forceinline__ void load_row(const float2* row, float2 (&v)[N]) {
#pragma unroll
  for (int c = 0; c < N; c += 2) {
    float4 t = *reinterpret_cast<const float4*>(row + c);
    v[c] = make_float2(t.x, t.y);
    v[c + 1] = make_float2(t.z, t.w);
  }
}

// ------------------------------------------------------------------ forward
template <int N, bool VEC>
__global__ void __launch_bounds__(kSmallThreads, 4) fft2d_small_fwd_kernel(RealView in, CplxView out, int B, int padL,
                                                                       int padU, int ntasks) {
  constexpr int T = N / 2, IPW = 32 / T, ROWS = T + 1;
  constexpr int RS = SmallCfg<N>::RS, IS = SmallCfg<N>::IS;
  extern __shared__ __align__(16) float2 smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wpc = blockDim.x >> 5;
  float2* buf = smem + warp * (IPW * IS);
  const int li = lane / T, l = lane % T;
  float2* ib = buf + li * IS;

  for (int task = blockIdx.x * wpc + warp; task < ntasks; task += gridDim.x * wpc) {
    const int b = task * IPW + li;
    const bool valid = b < B;
    {
      // ---- pass A: columns l and l+T of image b as one complex line
      float2 a[N];
      const float* src = in.p + (long long)(valid ? b : 0) * in.sb;
      const unsigned x0 = (unsigned)(l - padL), x1 = (unsigned)(l + T - padL);
      const bool ok0 = valid && x0 < (unsigned)in.w, ok1 = valid && x1 < (unsigned)in.w;
#pragma unroll
      for (int y = 0; y < N; ++y) {
        const unsigned yy = (unsigned)(y - padU);
        const bool oky = yy < (unsigned)in.h;
        a[y].x = (oky && ok0) ? __ldg(src + (long long)yy * in.sy + (long long)x0 * in.sx) : 0.f;
        a[y].y = (oky && ok1) ? __ldg(src + (long long)yy * in.sy + (long long)x1 * in.sx) : 0.f;
      }
      fft_bitrev<N, false>(a);
      // separate: A = (Z[r] + conj Z[N-r]) / 2 (column l), Bc = (Z[r] - conj Z[N-r]) / 2i (column l+T)
      {
        const float2 z0 = a[0], zh = a[brev(N / 2, N)];
        ib[l] = make_float2(z0.x, zh.x);
        ib[l + T] = make_float2(z0.y, zh.y);
      }
      static_for<T - 1>([&](auto rc) {
        constexpr int r = decltype(rc)::value + 1;
        const float2 zr = a[brev(r, N)], zm = a[brev(N - r, N)];
        ib[r * RS + l] = make_float2(0.5f * (zr.x + zm.x), 0.5f * (zr.y - zm.y));
        ib[r * RS + l + T] = make_float2(0.5f * (zr.y + zm.y), 0.5f * (zm.x - zr.x));
      });
    }
    __syncwarp();
    {
      // ---- pass B: packed row l of image li
      float2 v[N];
      load_row<N>(ib + l * RS, v);
      fft_bitrev<N, false>(v);
      static_for<N / 2>([&](auto cc) {
        constexpr int c = decltype(cc)::value * 2;
        const float2 p = v[brev(c, N)], q = v[brev(c + 1, N)];
        *reinterpret_cast<float4*>(ib + l * RS + c) = make_float4(p.x, p.y, q.x, q.y);
      });
    }
    __syncwarp();
    {
      // ---- unpack row 0 = F[0] + i F[N/2]: lane l owns the pair (kx, N-kx), kx = l
      // (lane 0 owns the self-paired kx = 0 and kx = N/2)
      const int k0 = (l == 0) ? 0 : l, k1 = (l == 0) ? T : N - l;
      const float2 va = ib[k0], vb = ib[k1];
      const float2 ma = (l == 0) ? va : vb;  // V[(N-k0)%N]
      const float2 mb = (l == 0) ? vb : va;  // V[(N-k1)%N]
      ib[k0] = make_float2(0.5f * (va.x + ma.x), 0.5f * (va.y - ma.y));
      ib[T * RS + k0] = make_float2(0.5f * (va.y + ma.y), 0.5f * (ma.x - va.x));
      ib[k1] = make_float2(0.5f * (vb.x + mb.x), 0.5f * (vb.y - mb.y));
      ib[T * RS + k1] = make_float2(0.5f * (vb.y + mb.y), 0.5f * (mb.x - vb.x));
    }
    __syncwarp();
    // ---- copy out IPW images x ROWS x N complex
    if (VEC) {
      constexpr int PER = ROWS * (N / 2);  // float4 per image
      for (int e = lane; e < IPW * PER; e += 32) {
        const int img = e / PER, rem = e % PER, row = rem / (N / 2), c4 = rem % (N / 2);
        const int bb = task * IPW + img;
        if (bb < B) {
          const float4 t = *reinterpret_cast<const float4*>(buf + img * IS + row * RS + c4 * 2);
          *reinterpret_cast<float4*>(out.p + (long long)bb * out.sb + (long long)rem * 4) = t;
        }
      }
    } else {
      constexpr int PER = ROWS * N;
      for (int e = lane; e < IPW * PER; e += 32) {
        const int img = e / PER, rem = e % PER, row = rem / N, c = rem % N;
        const int bb = task * IPW + img;
        if (bb < B) {
          const float2 t = buf[img * IS + row * RS + c];
          float* dst = out.p + (long long)bb * out.sb + (long long)row * out.sr + (long long)c * out.sc;
          dst[0] = t.x;
          dst[out.sz] = t.y;
        }
      }
    }
    __syncwarp();
  }
}

// ------------------------------------------------------------------ inverse
template <int N, bool VEC>
__global__ void __launch_bounds__(kSmallThreads, 4) fft2d_small_inv_kernel(CplxView in, RealView out, int B, int padL,
                                                                       int padU, int ntasks) {
  constexpr int T = N / 2, IPW = 32 / T, ROWS = T + 1;
  constexpr int RS = SmallCfg<N>::RS, IS = SmallCfg<N>::IS;
  extern __shared__ __align__(16) float2 smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wpc = blockDim.x >> 5;
  float2* buf = smem + warp * (IPW * IS);
  const int li = lane / T, l = lane % T;
  float2* ib = buf + li * IS;

  for (int task = blockIdx.x * wpc + warp; task < ntasks; task += gridDim.x * wpc) {
    // ---- copy in
    if (VEC) {
      constexpr int PER = ROWS * (N / 2);
      for (int e = lane; e < IPW * PER; e += 32) {
        const int img = e / PER, rem = e % PER, row = rem / (N / 2), c4 = rem % (N / 2);
        const int bb = task * IPW + img;
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (bb < B) t = __ldg(reinterpret_cast<const float4*>(in.p + (long long)bb * in.sb + (long long)rem * 4));
        *reinterpret_cast<float4*>(buf + img * IS + row * RS + c4 * 2) = t;
      }
    } else {
      constexpr int PER = ROWS * N;
      for (int e = lane; e < IPW * PER; e += 32) {
        const int img = e / PER, rem = e % PER, row = rem / N, c = rem % N;
        const int bb = task * IPW + img;
        float2 t = make_float2(0.f, 0.f);
        if (bb < B) {
          const float* s = in.p + (long long)bb * in.sb + (long long)row * in.sr + (long long)c * in.sc;
          t = make_float2(__ldg(s), __ldg(s + in.sz));
        }
        buf[img * IS + row * RS + c] = t;
      }
    }
    __syncwarp();
    {
      // ---- pack rows 0 and N/2 into row 0: P = F[0] + i F[N/2]; the imaginary
      // parts of F[0][0] and F[N/2][0] carry no information and are dropped
      // (fbfft/FFT2D32.cuh:313-315)
      const int k0 = l, k1 = l + T;
      const float2 a0 = ib[k0], h0 = ib[T * RS + k0], a1 = ib[k1], h1 = ib[T * RS + k1];
      ib[k0] = (l == 0) ? make_float2(a0.x, h0.x) : make_float2(a0.x - h0.y, a0.y + h0.x);
      ib[k1] = make_float2(a1.x - h1.y, a1.y + h1.x);
    }
    __syncwarp();
    {
      // ---- pass B^-1: inverse transform of packed row l along kx
      float2 v[N];
      load_row<N>(ib + l * RS, v);
      fft_bitrev<N, true>(v);
      static_for<N / 2>([&](auto cc) {
        constexpr int c = decltype(cc)::value * 2;
        const float2 p = v[brev(c, N)], q = v[brev(c + 1, N)];
        *reinterpret_cast<float4*>(ib + l * RS + c) = make_float4(p.x, p.y, q.x, q.y);
      });
    }
    __syncwarp();
    {
      // ---- pass A^-1: columns l and l+T; Z[r] = G_l[r] + i G_{l+T}[r] with the
      // Hermitian extension G[N-r] = conj G[r]
      float2 z[N];
      {
        const float2 g0 = ib[l], g1 = ib[l + T];
        z[0] = make_float2(g0.x, g1.x);
        z[N / 2] = make_float2(g0.y, g1.y);
      }
      static_for<T - 1>([&](auto rc) {
        constexpr int r = decltype(rc)::value + 1;
        const float2 g0 = ib[r * RS + l], g1 = ib[r * RS + l + T];
        z[r] = make_float2(g0.x - g1.y, g0.y + g1.x);
        z[N - r] = make_float2(g0.x + g1.y, g1.x - g0.y);
      });
      fft_bitrev<N, true>(z);
      const int b = task * IPW + li;
      if (b < B) {
        float* dst = out.p + (long long)b * out.sb;
        const unsigned x0 = (unsigned)(l - padL), x1 = (unsigned)(l + T - padL);
        const bool ok0 = x0 < (unsigned)out.w, ok1 = x1 < (unsigned)out.w;
        static_for<N>([&](auto yc) {
          constexpr int y = decltype(yc)::value;
          const unsigned yy = (unsigned)(y - padU);
          if (yy < (unsigned)out.h) {
            const float2 t = z[brev(y, N)];
            if (ok0) dst[(long long)yy * out.sy + (long long)x0 * out.sx] = t.x;
            if (ok1) dst[(long long)yy * out.sy + (long long)x1 * out.sx] = t.y;
          }
        });
      }
    }
    __syncwarp();
  }
}

template <int N>
constexpr int small_smem_bytes() {
  return (kSmallThreads / 32) * (32 / (N / 2)) * SmallCfg<N>::IS * (int)sizeof(float2);
}

bool cplx_is_vectorizable(const CplxView& c, int rows, int cols) {
  return c.sz == 1 && c.sc == 2 && c.sr == 2 * cols && (c.sb % 4) == 0 && aligned16(c.p);
}

template <int N>
int launch_fwd(const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s) {
  constexpr int IPW = 32 / (N / 2);
  const int ntasks = (B + IPW - 1) / IPW;
  const int wpc = kSmallThreads / 32;
  const int want = (ntasks + wpc - 1) / wpc;
  const int grid = want < sm_count() * 8 ? want : sm_count() * 8;
  const int smem = small_smem_bytes<N>();
  if (cplx_is_vectorizable(out, N / 2 + 1, N)) {
    fft2d_small_fwd_kernel<N, true><<<grid, kSmallThreads, smem, s>>>(in, out, B, padL, padU, ntasks);
  } else {
    fft2d_small_fwd_kernel<N, false><<<grid, kSmallThreads, smem, s>>>(in, out, B, padL, padU, ntasks);
  }
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

template <int N>
int launch_inv(const CplxView& in, const RealView& out, int B, int padL, int padU, cudaStream_t s) {
  constexpr int IPW = 32 / (N / 2);
  const int ntasks = (B + IPW - 1) / IPW;
  const int wpc = kSmallThreads / 32;
  const int want = (ntasks + wpc - 1) / wpc;
  const int grid = want < sm_count() * 8 ? want : sm_count() * 8;
  const int smem = small_smem_bytes<N>();
  if (cplx_is_vectorizable(in, N / 2 + 1, N)) {
    fft2d_small_inv_kernel<N, true><<<grid, kSmallThreads, smem, s>>>(in, out, B, padL, padU, ntasks);
  } else {
    fft2d_small_inv_kernel<N, false><<<grid, kSmallThreads, smem, s>>>(in, out, B, padL, padU, ntasks);
  }
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

}  // namespace

int fft2d_small_forward(int n, const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s) {
  if (B <= 0) return kSuccess;
  switch (n) {
    case 8:
      return launch_fwd<8>(in, out, B, padL, padU, s);
    case 16:
      return launch_fwd<16>(in, out, B, padL, padU, s);
    case 32:
      return launch_fwd<32>(in, out, B, padL, padU, s);
    default:
      return kUnsupportedSize;
  }
}

int fft2d_small_inverse(int n, const CplxView& in, const RealView& out, int B, int padL, int padU, cudaStream_t s) {
  if (B <= 0) return kSuccess;
  switch (n) {
    case 8:
      return launch_inv<8>(in, out, B, padL, padU, s);
    case 16:
      return launch_inv<16>(in, out, B, padL, padU, s);
    case 32:
      return launch_inv<32>(in, out, B, padL, padU, s);
    default:
      return kUnsupportedSize;
  }
}

}  // namespace fbfft_b200
