// Second call of the reference's two-call forward protocol for N = 64 and 128
// (fbfft/FBFFT2D-inl.cuh:627-669): buffer[b][y][kx] (kx in 0..N/2) -> dst[b][kx][ky], a complex
// transform along y written transposed, on contiguous tensors.
//
// One block owns one image.  The image (N x (N/2+1) complex values, contiguous) arrives by one
// cp.async.bulk (completion on an mbarrier, bounded wait).  Column kx < N/2 belongs to Q = N/64
// neighbouring lanes, which read it from shared memory (lanes run over kx: no bank conflicts) and
// transform it in registers (coop_fft.cuh); the last column kx = N/2 has no lanes of its own.  It is
// set aside and transformed in a second round by lanes of warp 0 -- at N = 128, where that round
// would otherwise idle the other three warps once per image, the set-aside columns of four
// consecutive images of the block wait for ONE such round and their rows kx = N/2 leave by bulk
// stores of their own (234 -> 193 us for 8192 images: 0.71 -> 0.86 of the copy bandwidth).  The other results overwrite the image as a [N/2+1][N] tile whose rows leave
// through bulk stores.
#include "coop_fft.cuh"
#include "fft2d_small.cuh"  // bulk-copy / mbarrier helpers
#include "kernels.h"

namespace fbfft_b200 {

namespace {

enum : int { kErrColsFwdWait = 108 };

template <int N>
struct ColsCfg {
  static constexpr int R = 64, Q = N / 64, H = N / 2, HC = N / 2 + 1, T = H * Q, PO = N + 2;
  static constexpr int REGION = HC * PO;                  // complex values: tile [HC][PO] >= image [N][HC]
  // images whose last columns share one extra round (measured at N = 64, where a block is one warp:
  // sharing the round among 8 images at 10 blocks per SM changed nothing, 201 -> 205 us for 32 768
  // images; the pass is not bound by its arithmetic there)
  static constexpr int G = N == 128 ? 4 : 1;
  static constexpr int SMEM = (REGION + G * N) * 8 + 16;  // + the set-aside columns + the mbarrier
  static constexpr int BLOCKS = N == 64 ? 12 : 3;
};

template <int N>
__global__ void __launch_bounds__(ColsCfg<N>::T, ColsCfg<N>::BLOCKS) cols_fwd_kernel(const float* __restrict__ buf,
                                                                                    float* __restrict__ dst, int B) {
  using C = ColsCfg<N>;
  constexpr int R = C::R, Q = C::Q, P = R / Q, LP = 32 / Q, H = C::H, HC = C::HC, T = C::T, PO = C::PO, G = C::G;
  extern __shared__ __align__(16) float2 sm[];
  float2* img = sm;            // [N][HC]
  float2* tile = sm;           // [HC][PO]
  float2* last = sm + C::REGION;  // column N/2 of up to G images: [G][N]
  const unsigned bar = smem_u32(sm + C::REGION + G * N);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = lane / LP, kx = warp * LP + (lane % LP);
  float2 lf[Q];
  lane_factors<Q, false>(q, lf);
  constexpr unsigned kImageBytes = N * HC * 8;
  auto fetch = [&](int b) {
    if (threadIdx.x == 0) {
      fence_async_smem();
      mbar_expect_tx(bar, kImageBytes);
      bulk_g2s(smem_u32(img), buf + (long long)b * (2 * N * HC), kImageBytes, bar);
    }
  };
  // transform of the `count` set-aside columns (images first_b, first_b + gridDim.x, ...) by warp 0,
  // line j in the lanes of column j; the rows kx = N/2 go back into `last` and leave from there
  auto flush_last = [&](int first_b, int count) {
    if (warp == 0) {
      float2 a[R];
      const int j = lane % LP;  // line slot; slots >= count transform stale values that are never stored
      const float2* src = last + (j < G ? j : 0) * N;
#pragma unroll
      for (int m = 0; m < Q; ++m) {
#pragma unroll
        for (int jl = 0; jl < P; ++jl) a[m * P + jl] = src[jl + P * q + R * m];
      }
      coop_fft<N, R, Q, false>(a, q, lf);
      __syncwarp();  // every lane has read its line before any lane overwrites it
      if (j < count) {
        static_for<R>([&](auto kc) {
          constexpr int k = decltype(kc)::value;
          last[j * N + Q * k + q] = a[brev(k, R)];
        });
      }
      fence_async_smem();
      __syncwarp();
      if (lane < count)
        bulk_s2g(dst + (long long)(first_b + lane * (int)gridDim.x) * (2 * N * HC) + (long long)H * (2 * N), smem_u32(last + lane * N),
                 N * 8);
      bulk_commit();
      bulk_wait_read();  // the lines are free again
    }
  };
  if (threadIdx.x == 0) mbar_init(bar, 1);
  fence_async_smem();
  __syncthreads();
  unsigned phase = 0;
  int pending = 0, first_pending = 0;
  if (blockIdx.x < B) fetch(blockIdx.x);
  for (int b = blockIdx.x; b < B; b += gridDim.x) {
    if (!mbar_wait(bar, phase, kErrColsFwdWait)) return;
    phase ^= 1;
    float2 a[R];
#pragma unroll
    for (int m = 0; m < Q; ++m) {
#pragma unroll
      for (int jl = 0; jl < P; ++jl) a[m * P + jl] = img[(jl + P * q + R * m) * HC + kx];
    }
    if (pending == 0) first_pending = b;
    for (int y = threadIdx.x; y < N; y += T) last[pending * N + y] = img[y * HC + H];
    ++pending;
    __syncthreads();  // the image is in registers (and its last column set aside): the tile may overwrite it
    coop_fft<N, R, Q, false>(a, q, lf);
    static_for<R>([&](auto kc) {
      constexpr int k = decltype(kc)::value;
      tile[kx * PO + Q * k + q] = a[brev(k, R)];
    });
    if (pending == G || b + (int)gridDim.x >= B) {
      flush_last(first_pending, pending);
      pending = 0;
    }
    fence_async_smem();
    __syncthreads();
    float* out = dst + (long long)b * (2 * N * HC);
    for (int r = threadIdx.x; r < H; r += T) bulk_s2g(out + (long long)r * (2 * N), smem_u32(tile + r * PO), N * 8);
    bulk_commit();
    bulk_wait_read();
    __syncthreads();
    if (b + gridDim.x < B) fetch(b + gridDim.x);
  }
}

template <int N>
int launch_cols(const float* buf, float* dst, int B, cudaStream_t s) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(cols_fwd_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, ColsCfg<N>::SMEM);
    configured[dev] = true;
  }
  const int cap = sm_count() * ColsCfg<N>::BLOCKS;
  cols_fwd_kernel<N><<<B < cap ? B : cap, ColsCfg<N>::T, ColsCfg<N>::SMEM, s>>>(buf, dst, B);
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

// ---- second call of the inverse protocol (fbfft/FBIFFT2D-inl.cuh:529-742): buffer[p][kx][y] complex,
// p < G = ceil(B/2) -> unnormalised inverse along kx; the real part is image p, the imaginary part
// image p + G (when it exists); contiguous N x N outputs.  A block takes 64 consecutive y of one p:
// N bulk copies of 512 bytes (one per kx) into shared memory, lanes run over y, transform in
// registers, the two real tiles overwrite the input at a pitch of N + 4 floats and leave by one
// bulk store per image row.
template <int N>
struct ColsInvCfg {
  static constexpr int R = 64, Q = N / 64, YB = 64, T = YB * Q, PT = N + 4;
  static constexpr int TILE = YB * PT;                               // floats per real tile
  static constexpr int REGION = 2 * TILE > 2 * N * YB ? 2 * TILE : 2 * N * YB;  // floats
  static constexpr int SMEM = REGION * 4 + 16;
  static constexpr int BLOCKS = N == 64 ? 6 : 3;
};

// where the N x N result of an image goes: rows padU .. padU + h - 1, columns padL .. padL + w - 1 of it
// are stored as the h x w image at out + b * sb + y * sy (all in 16-byte units); full images: h = w = N
struct CropOut {
  long long sb, sy;
  int h, w, padL, padU;
};

template <int N>
__global__ void __launch_bounds__(ColsInvCfg<N>::T, ColsInvCfg<N>::BLOCKS) cols_inv_kernel(const float* __restrict__ buf,
                                                                                          float* __restrict__ out,
                                                                                          int B, int G, CropOut crop) {
  using C = ColsInvCfg<N>;
  constexpr int R = C::R, Q = C::Q, P = R / Q, LP = 32 / Q, YB = C::YB, T = C::T, PT = C::PT;
  extern __shared__ __align__(16) float smf[];
  const float2* in = reinterpret_cast<const float2*>(smf);  // [N][YB]
  float* tile_a = smf;                                      // [YB][PT]
  float* tile_b = smf + C::TILE;
  const unsigned bar = smem_u32(smf + C::REGION);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = lane / LP, yi = warp * LP + (lane % LP);
  float2 lf[Q];
  lane_factors<Q, true>(q, lf);
  constexpr int YBLOCKS = N / YB;
  const long long work_total = (long long)G * YBLOCKS;
  static_assert(T >= N || T * 2 >= N, "row copies are spread over the block's threads");
  auto fetch = [&](long long work) {
    const long long p = work / YBLOCKS;
    const int y0 = (int)(work % YBLOCKS) * YB;
    if (threadIdx.x == 0) {
      fence_async_smem();
      mbar_expect_tx(bar, N * YB * 8);
    }
    __syncthreads();
    for (int kx = threadIdx.x; kx < N; kx += T)
      bulk_g2s(smem_u32(smf + kx * YB * 2), buf + (p * N + kx) * (2LL * N) + 2 * y0, YB * 8, bar);
  };
  if (threadIdx.x == 0) mbar_init(bar, 1);
  fence_async_smem();
  __syncthreads();
  unsigned phase = 0;
  if (blockIdx.x < work_total) fetch(blockIdx.x);
  for (long long work = blockIdx.x; work < work_total; work += gridDim.x) {
    const long long p = work / YBLOCKS;
    const int y0 = (int)(work % YBLOCKS) * YB;
    if (!mbar_wait(bar, phase, kErrColsFwdWait)) return;
    phase ^= 1;
    float2 a[R];
#pragma unroll
    for (int m = 0; m < Q; ++m) {
#pragma unroll
      for (int jl = 0; jl < P; ++jl) a[m * P + jl] = in[(jl + P * q + R * m) * YB + yi];
    }
    __syncthreads();  // the input is in registers: the tiles may overwrite it
    coop_fft<N, R, Q, true>(a, q, lf);
    static_for<R>([&](auto kc) {
      constexpr int k = decltype(kc)::value;
      tile_a[yi * PT + Q * k + q] = a[brev(k, R)].x;
      tile_b[yi * PT + Q * k + q] = a[brev(k, R)].y;
    });
    fence_async_smem();
    __syncthreads();
    const bool two = p + G < B;
    for (int r = threadIdx.x; r < YB; r += T) {
      const int y = y0 + r - crop.padU;  // row of the cropped image
      if ((unsigned)y < (unsigned)crop.h) {
        bulk_s2g(out + p * crop.sb + (long long)y * crop.sy, smem_u32(tile_a + r * PT + crop.padL), crop.w * 4);
        if (two) bulk_s2g(out + (p + G) * crop.sb + (long long)y * crop.sy, smem_u32(tile_b + r * PT + crop.padL), crop.w * 4);
      }
    }
    bulk_commit();
    bulk_wait_read();
    if (work + gridDim.x < work_total) fetch(work + gridDim.x);
  }
}

template <int N>
int launch_cols_inv(const float* buf, float* out, int B, const CropOut& crop, cudaStream_t s) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(cols_inv_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, ColsInvCfg<N>::SMEM);
    configured[dev] = true;
  }
  const int G = (B + 1) / 2;
  const long long work = (long long)G * (N / ColsInvCfg<N>::YB), cap = (long long)sm_count() * ColsInvCfg<N>::BLOCKS;
  cols_inv_kernel<N><<<(int)(work < cap ? work : cap), ColsInvCfg<N>::T, ColsInvCfg<N>::SMEM, s>>>(buf, out, B, G, crop);
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

// ---- first call of the inverse protocol (fbfft/FBIFFT2D-inl.cuh:252-521): spectra src[b][kx][ky],
// kx in 0..N/2 -> buffer[p][r][y], r in 0..N-1, p < G = ceil(B/2): the unnormalised inverse along ky of
//   A[r] + i B[r]                               for r <= N/2   (A, B = spectra of images p and p + G)
//   conj A[N-r][-ky] + i conj B[N-r][-ky]       for r >  N/2   (Hermitian half), which equals
//   conj(inverse of (A[N-r] - i B[N-r])).
// A block takes 32 stored rows kx of one pair (and row N/2 with the first 32): bulk copies of the
// rows of both spectra into shared memory at a pitch of N + 2 complex values, 64 lines -- side 0:
// r = kx, side 1: r = N - kx (r = N/2 in place of kx = 0) -- each transformed in registers by Q lanes,
// parked as a [64][N + 2] tile over the input and stored row by row with bulk copies.
template <int N>
struct RowsInvCfg {
  static constexpr int R = 64, Q = N / 64, KB = 32, T = 2 * KB * Q, PT = N + 2;   // PT: complex values
  static constexpr int IN = 2 * (KB + 1) * PT, OUT = 2 * KB * PT;
  static constexpr int REGION = IN > OUT ? IN : OUT;                               // complex values
  static constexpr int SMEM = REGION * 8 + 16;
  static constexpr int BLOCKS = N == 64 ? 6 : 3;
};

template <int N>
__global__ void __launch_bounds__(RowsInvCfg<N>::T, RowsInvCfg<N>::BLOCKS) rows_inv_kernel(const float* __restrict__ src,
                                                                                          float* __restrict__ buf,
                                                                                          int B, int G) {
  using C = RowsInvCfg<N>;
  constexpr int R = C::R, Q = C::Q, P = R / Q, LP = 32 / Q, KB = C::KB, T = C::T, PT = C::PT, HC = N / 2 + 1;
  extern __shared__ __align__(16) float2 smr[];
  const float2* sa = smr;                     // rows of A: [KB + 1][PT]
  const float2* sb = smr + (KB + 1) * PT;     // rows of B
  float2* tile = smr;                         // [2 KB][PT]
  const unsigned bar = smem_u32(smr + C::REGION);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = lane / LP, li = warp * LP + (lane % LP);  // line 0..63
  const int side = li / KB, kl = li % KB;
  float2 lf[Q];
  lane_factors<Q, true>(q, lf);
  constexpr int KBLOCKS = (N / 2) / KB;
  const long long work_total = (long long)G * KBLOCKS;
  auto fetch = [&](long long work) {
    const long long p = work / KBLOCKS;
    const int kb = (int)(work % KBLOCKS);
    const bool two = p + G < B;
    const int rows = KB + (kb == 0 ? 1 : 0);
    if (threadIdx.x == 0) {
      fence_async_smem();
      mbar_expect_tx(bar, (two ? 2 : 1) * rows * N * 8);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * rows; i += T) {
      const int which = i / rows, slot = i % rows;
      if (which == 1 && !two) continue;
      const int kx = slot < KB ? kb * KB + slot : N / 2;
      const long long img = which ? p + G : p;
      bulk_g2s(smem_u32(smr + (which * (KB + 1) + slot) * PT), src + (img * HC + kx) * (2LL * N), N * 8, bar);
    }
  };
  if (threadIdx.x == 0) mbar_init(bar, 1);
  fence_async_smem();
  __syncthreads();
  unsigned phase = 0;
  if (blockIdx.x < work_total) fetch(blockIdx.x);
  for (long long work = blockIdx.x; work < work_total; work += gridDim.x) {
    const long long p = work / KBLOCKS;
    const int kb = (int)(work % KBLOCKS);
    const bool two = p + G < B;
    if (!mbar_wait(bar, phase, kErrColsFwdWait)) return;
    phase ^= 1;
    const int kx = kb * KB + kl;
    // stored row 0 has no mirror: its side-1 line transforms r = N/2 instead
    const bool nyq = side == 1 && kx == 0;
    const int slot = nyq ? KB : kl;
    const float sign = (side == 1 && !nyq) ? -1.f : 1.f;
    const int r = side == 0 ? kx : (nyq ? N / 2 : N - kx);
    float2 a[R];
    const float2* ra = sa + slot * PT;
    const float2* rb = sb + slot * PT;
#pragma unroll
    for (int m = 0; m < Q; ++m) {
#pragma unroll
      for (int jl = 0; jl < P; ++jl) {
        const int c = jl + P * q + R * m;
        const float2 A = ra[c];
        const float2 Bv = two ? rb[c] : make_float2(0.f, 0.f);
        a[m * P + jl] = make_float2(A.x - sign * Bv.y, A.y + sign * Bv.x);
      }
    }
    __syncthreads();  // the rows are in registers: the tile may overwrite them
    coop_fft<N, R, Q, true>(a, q, lf);
    static_for<R>([&](auto kc) {
      constexpr int k = decltype(kc)::value;
      const float2 z = a[brev(k, R)];
      tile[li * PT + Q * k + q] = make_float2(z.x, sign * z.y);
    });
    fence_async_smem();
    __syncthreads();
    if (q == 0) {
      bulk_s2g(buf + (p * N + r) * (2LL * N), smem_u32(tile + li * PT), N * 8);
      bulk_commit();
    }
    bulk_wait_read();
    if (work + gridDim.x < work_total) fetch(work + gridDim.x);
  }
}

template <int N>
int launch_rows_inv(const float* src, float* buf, int B, cudaStream_t s) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(rows_inv_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, RowsInvCfg<N>::SMEM);
    configured[dev] = true;
  }
  const int G = (B + 1) / 2;
  const long long work = (long long)G * ((N / 2) / RowsInvCfg<N>::KB), cap = (long long)sm_count() * RowsInvCfg<N>::BLOCKS;
  rows_inv_kernel<N><<<(int)(work < cap ? work : cap), RowsInvCfg<N>::T, RowsInvCfg<N>::SMEM, s>>>(src, buf, B, G);
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

}  // namespace

// contiguous [B][N][N/2+1][2] buffer and [B][N/2+1][N][2] destination, 16-byte aligned
bool fft2d_cols_fast_supported(int n, const CplxView& buffer, const CplxView& dst, int B) {
  if (n != 64 && n != 128) return false;
  if (buffer.blk_planes || dst.blk_planes || buffer.sz != 1 || dst.sz != 1) return false;
  const long long image = (long long)n * (n + 2);
  return buffer.sc == 2 && buffer.sr == n + 2 && dst.sc == 2 && dst.sr == 2 * n &&
         (B <= 1 || (buffer.sb == image && dst.sb == image)) && aligned16(buffer.p) && aligned16(dst.p);
}

int fft2d_cols_fast(int n, const CplxView& buffer, const CplxView& dst, int B, cudaStream_t s) {
  if (n == 64) return launch_cols<64>(buffer.p, dst.p, B, s);
  return launch_cols<128>(buffer.p, dst.p, B, s);
}

// contiguous [G][N][N][2] buffer and contiguous [B][N][N] images, 16-byte aligned, no crop
// contiguous buffer; output images (full or cropped) with rows, strides and pads in 16-byte units
bool fft2d_cols_inv_fast_supported(int n, const CplxView& buffer, const RealView& out, int B, int padL, int padU) {
  if (n != 64 && n != 128) return false;
  if (buffer.blk_planes || buffer.sz != 1 || padL < 0 || padU < 0) return false;
  if (!(buffer.sc == 2 && buffer.sr == 2 * n && (B <= 2 || buffer.sb == 2LL * n * n) && aligned16(buffer.p))) return false;
  return out.sx == 1 && out.w >= 4 && out.w % 4 == 0 && padL % 4 == 0 && padL + out.w <= n && out.h >= 1 &&
         padU + out.h <= n && out.sy % 4 == 0 && (B <= 1 || out.sb % 4 == 0) && aligned16(out.p);
}

int fft2d_cols_inv_fast(int n, const CplxView& buffer, const RealView& out, int B, int padL, int padU, cudaStream_t s) {
  CropOut crop;
  crop.sb = out.sb, crop.sy = out.sy, crop.h = out.h, crop.w = out.w, crop.padL = padL, crop.padU = padU;
  if (n == 64) return launch_cols_inv<64>(buffer.p, out.p, B, crop, s);
  return launch_cols_inv<128>(buffer.p, out.p, B, crop, s);
}

// contiguous [B][N/2+1][N][2] spectra and contiguous [.][N][N][2] buffer, 16-byte aligned
bool fft2d_rows_inv_fast_supported(int n, const CplxView& src, const CplxView& buffer, int B) {
  if (n != 64 && n != 128) return false;
  if (src.blk_planes || buffer.blk_planes || src.sz != 1 || buffer.sz != 1) return false;
  return src.sc == 2 && src.sr == 2 * n && (B <= 1 || src.sb == (long long)(n + 2) * n) && buffer.sc == 2 &&
         buffer.sr == 2 * n && (B <= 2 || buffer.sb == 2LL * n * n) && aligned16(src.p) && aligned16(buffer.p);
}

int fft2d_rows_inv_fast(int n, const CplxView& src, const CplxView& buffer, int B, cudaStream_t s) {
  if (n == 64) return launch_rows_inv<64>(src.p, buffer.p, B, s);
  return launch_rows_inv<128>(src.p, buffer.p, B, s);
}

int read_device_error_cols() { return device_error_word_read(); }
int clear_device_error_cols() { return device_error_word_clear(); }

}  // namespace fbfft_b200
