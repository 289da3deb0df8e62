// Forward 2-D real-to-complex FFT for N = 256 on contiguous tensors, in the reference's layout
// for this size class: transposed spectrum [B][kx in 0..128][ky in 0..255] (what its two calls,
// fbfft/FBFFT2D-inl.cuh:597-617 then :627-669, leave behind).
//
// A 256 x 256 image and its spectrum (264 KB) do not fit one SM's shared memory, so the transform
// keeps the reference's two passes, but without its separate [B][N][N/2+1] buffer: the row pass
// writes its result transposed straight into the output tensor, the column pass transforms the
// output's lines in place.  Both passes hold every line in registers, shared by 4 neighbouring lane
// groups of a warp (radix-4 step, one all-to-all by __shfl_xor_sync, 64-point FFT per lane with
// compile-time twiddles: coop_fft.cuh).
//   rows     a block takes 64 consecutive rows of one image (contiguous images: 32 bulk copies of one
//            row pair each into shared memory, completion on an mbarrier with a bounded wait);
//            rows 2l and 2l+1 travel as re/im of one complex line (a warp holds 8 lines); the lines' transforms Z are parked in shared
//            memory, then thread (kx, l) separates the two real spectra, A = (Z[kx] + conj Z[N-kx])/2
//            and B = (Z[kx] - conj Z[N-kx])/2i, and stores both as 16 bytes at out[kx][2l..2l+1]:
//            a warp writes 512 contiguous bytes.
//   columns  a warp takes 8 lines out[kx][*] (2 KB each, contiguous) through its shared-memory slot:
//            bulk copies in, transform in registers, bulk copies out.
// HBM traffic is twice the algorithmic bytes (the spectrum is written, read and written again).
// Measured and dropped, 1024 images (forward / inverse, this design: 206 / 230 us):
//   * both passes launched per chunk of 32..256 images so that the half-transformed chunk stays in L2:
//     593..250 / 657..288 us (launch gaps and tails of the short kernels cost more than the traffic saves);
//   * one pass by a cluster of 4 blocks per image (each block transforms 64 rows, parks them in its
//     shared memory, gathers its 32 columns from all four through distributed shared memory): correct,
//     HBM traffic halved (22 % of the DRAM peak), 243 / 282 us.  With 160 registers a thread and 66 KB a
//     block only 12 warps fit an SM and either design issues 0.35 instructions per cycle and scheduler
//     (stalls spread over remote loads, the shared-memory queue, barriers and fences): the two 64-point
//     register transforms per thread bound the time, not the bytes.
#include "coop_fft.cuh"
#include "fft2d_small.cuh"  // bulk-copy / mbarrier helpers
#include "kernels.h"

namespace fbfft_b200 {

namespace {

constexpr int N256 = 256, R256 = 64, Q256 = 4, P256 = R256 / Q256, LP256 = 32 / Q256;
constexpr int kRowsThreads = 128;                       // 4 warps x 8 lines = 32 lines = 64 rows
constexpr int kLinesPerBlock = (kRowsThreads / 32) * LP256;
constexpr int PZ = N256 + 2;                            // line pitch in shared memory (complex values)
enum : int { kErrColsWait = 106, kErrRowsWait = 107 };

// FULL: the images are contiguous 256 x 256 without padding (16-byte loads, no predicates)
template <bool FULL>
__global__ void __launch_bounds__(kRowsThreads, 3) fft256_rows_kernel(RealView in, float* __restrict__ out, long long out_sb,
                                                                       int B, int padL, int padU) {
  extern __shared__ __align__(16) float2 zs[];  // [32 lines][PZ], then the mbarrier (FULL)
  const unsigned bar = smem_u32(zs + kLinesPerBlock * PZ);
  unsigned phase = 0;
  if (FULL) {
    if (threadIdx.x == 0) mbar_init(bar, 1);
    fence_async_smem();
    __syncthreads();
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = lane / LP256, line = warp * LP256 + (lane % LP256);
  float2 lf[Q256];
  lane_factors<Q256, false>(q, lf);
  const int bands = N256 / (2 * kLinesPerBlock);  // 4
  for (long long work = blockIdx.x; work < (long long)B * bands; work += gridDim.x) {
    const long long b = work / bands;
    const int band = (int)(work % bands);
    const int y0 = band * 2 * kLinesPerBlock + 2 * line;  // canvas rows y0 (re) and y0 + 1 (im)
    float2 a[R256];
    const float* src = in.p + b * in.sb;
    if constexpr (FULL) {
      // the band's 64 rows arrive as 32 bulk copies of one row pair (2 KB) each into the lines'
      // own regions (pitch 258 complex values: the 16-byte reads below are free of bank conflicts)
      fence_async_smem();  // this thread's accesses to the lines precede the copies that overwrite them
      if (threadIdx.x == 0) mbar_expect_tx(bar, kLinesPerBlock * 2 * N256 * 4);
      __syncthreads();  // (also: the previous band's lines have been read)
      if (q == 0) bulk_g2s(smem_u32(zs + line * PZ), src + (long long)y0 * N256, 2 * N256 * 4, bar);
      if (!mbar_wait(bar, phase, kErrRowsWait)) return;
      phase ^= 1;
      const float* r0 = reinterpret_cast<const float*>(zs + line * PZ) + P256 * q;
#pragma unroll
      for (int m = 0; m < Q256; ++m) {
#pragma unroll
        for (int j4 = 0; j4 < P256 / 4; ++j4) {
          const float4 u = *reinterpret_cast<const float4*>(r0 + m * R256 + 4 * j4);
          const float4 v = *reinterpret_cast<const float4*>(r0 + N256 + m * R256 + 4 * j4);
          a[m * P256 + j4 * 4 + 0] = make_float2(u.x, v.x);
          a[m * P256 + j4 * 4 + 1] = make_float2(u.y, v.y);
          a[m * P256 + j4 * 4 + 2] = make_float2(u.z, v.z);
          a[m * P256 + j4 * 4 + 3] = make_float2(u.w, v.w);
        }
      }
    } else {
      const unsigned ya = (unsigned)(y0 - padU), yb = (unsigned)(y0 + 1 - padU);
      const bool oka = ya < (unsigned)in.h, okb = yb < (unsigned)in.h;
      const float* r0 = src + (long long)ya * in.sy;
      const float* r1 = src + (long long)yb * in.sy;
#pragma unroll
      for (int m = 0; m < Q256; ++m) {
#pragma unroll
        for (int jl = 0; jl < P256; ++jl) {
          const unsigned x = (unsigned)(jl + P256 * q + R256 * m - padL);
          const bool okx = x < (unsigned)in.w;
          a[m * P256 + jl].x = (oka && okx) ? __ldg(r0 + (long long)x * in.sx) : 0.f;
          a[m * P256 + jl].y = (okb && okx) ? __ldg(r1 + (long long)x * in.sx) : 0.f;
        }
      }
    }
    coop_fft<N256, R256, Q256, false>(a, q, lf);
    if constexpr (FULL) {
      __syncwarp();  // the lanes of a line have read its staged rows
    } else {
      __syncthreads();  // the previous band's lines have been read
    }
    static_for<R256>([&](auto kc) {
      constexpr int k = decltype(kc)::value;
      zs[line * PZ + Q256 * k + q] = a[brev(k, R256)];
    });
    __syncthreads();
    // out[b][kx][y0 .. y0+1] for the block's 32 lines: line fastest, 16 bytes per thread
    float* dst = out + b * out_sb + (long long)band * 4 * kLinesPerBlock;  // 2 rows x 2 floats per line
    for (int e = threadIdx.x; e < (N256 / 2 + 1) * kLinesPerBlock; e += kRowsThreads) {
      const int kx = e / kLinesPerBlock, l = e % kLinesPerBlock;
      const float2 z = zs[l * PZ + kx], m = zs[l * PZ + ((N256 - kx) & (N256 - 1))];
      const float4 v = make_float4(0.5f * (z.x + m.x), 0.5f * (z.y - m.y), 0.5f * (z.y + m.y), 0.5f * (m.x - z.x));
      *reinterpret_cast<float4*>(dst + (long long)kx * (2 * N256) + 4 * l) = v;
    }
  }
}

// in-place transform of `lines` contiguous lines of 256 complex values.  A warp takes 8 lines at a
// time: one cp.async.bulk per line into the warp's slot (pitch 258 complex values, so that the
// 16-byte reads of the 8 lines fall on different banks; completion on the warp's mbarrier, bounded
// wait), transform in registers, lines parked back in natural order, one bulk store per line.
constexpr int kColsWarps = 4;
constexpr int kColsSlot = LP256 * PZ;  // complex values per warp
constexpr int kColsSmem = kColsWarps * (kColsSlot * (int)sizeof(float2) + 16);


__global__ void __launch_bounds__(kColsWarps * 32, 3) fft256_cols_kernel(float* __restrict__ data, long long lines) {
  extern __shared__ __align__(16) float2 cs[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, q = lane / LP256, l = lane % LP256;
  float2* region = cs + warp * kColsSlot + l * PZ;
  const unsigned bar = smem_u32(cs + kColsWarps * kColsSlot) + warp * 16;
  if (lane == 0) mbar_init(bar, 1);
  fence_async_smem();
  __syncwarp();
  float2 lf[Q256];
  lane_factors<Q256, false>(q, lf);
  const long long tasks = (lines + LP256 - 1) / LP256;
  const long long gw = (long long)blockIdx.x * kColsWarps + warp, nw = (long long)gridDim.x * kColsWarps;
  auto issue = [&](long long task) {
    const long long first = task * LP256;
    const int valid = lines - first < LP256 ? (int)(lines - first) : LP256;
    if (lane < LP256) bulk_wait_read();  // this lane's line has left the slot
    __syncwarp();
    if (lane == 0) {
      fence_async_smem();
      mbar_expect_tx(bar, valid * N256 * 8);
    }
    __syncwarp();
    if (lane < valid) bulk_g2s(smem_u32(region), data + (first + l) * (2 * N256), N256 * 8, bar);
  };
  unsigned phase = 0;
  long long t = gw;
  if (t < tasks) issue(t);
  for (; t < tasks; t += nw) {
    if (!mbar_wait(bar, phase, kErrColsWait)) return;
    phase ^= 1;
    float2 a[R256];
#pragma unroll
    for (int m = 0; m < Q256; ++m) {
#pragma unroll
      for (int j2 = 0; j2 < P256 / 2; ++j2) {
        const float4 u = *reinterpret_cast<const float4*>(region + P256 * q + R256 * m + 2 * j2);
        a[m * P256 + 2 * j2] = make_float2(u.x, u.y);
        a[m * P256 + 2 * j2 + 1] = make_float2(u.z, u.w);
      }
    }
    coop_fft<N256, R256, Q256, false>(a, q, lf);
    __syncwarp();
    static_for<R256>([&](auto kc) {
      constexpr int k = decltype(kc)::value;
      region[Q256 * k + q] = a[brev(k, R256)];
    });
    fence_async_smem();
    __syncwarp();
    const long long line = t * LP256 + l;
    if (lane < LP256 && line < lines) {
      bulk_s2g(data + line * (2 * N256), smem_u32(region), N256 * 8);
      bulk_commit();
    }
    if (t + nw < tasks) issue(t + nw);
  }
  bulk_wait_read();
}

// ------------------------------------------------------------------ inverse
// Complex-to-real for N = 256, also in two passes and also without a buffer of its own: the real
// output image (256 KB) is exactly as large as the 128 packed complex values per row that the first
// pass leaves behind, so it doubles as the intermediate.
//   columns  a block takes 32 lines in[kx][*] (kx = 32 g ...; 2 KB each, one bulk copy per line),
//            inverse transforms them along ky in registers and writes T[kx][y] transposed into the
//            output image: out[y][2 kx], out[y][2 kx + 1] = T[kx][y] for kx = 1..127, 256 contiguous
//            bytes per row and block.  The lines kx = 0 and kx = 128 only contribute their real
//            parts to a real image (the imaginary parts belong to the Hermitian half that is not
//            stored) and share slot 0 of the row as (Re T[0][y], Re T[128][y]); the block of kx = 0
//            transforms line 128 in an extra round.
//   rows     a warp takes 8 row pairs (2 KB each: bulk copy in, bulk copy out): rows y and y + 1 become
//            one complex line C[kx] = G_y[kx] + i G_{y+1}[kx], extended to all 256 bins by
//            C[256 - kx] = conj(G_y[kx]) + i conj(G_{y+1}[kx]); its inverse transform holds row y in
//            the real and row y + 1 in the imaginary parts, which overwrite the pair in place.
// HBM traffic is again twice the algorithmic bytes.
constexpr int kInvLines = kLinesPerBlock + 1;  // the block's 32 lines and the slot of line 128
enum : int { kErrInvColsWait = 108, kErrInvRowsWait = 109 };

__global__ void __launch_bounds__(kRowsThreads, 3) ifft256_cols_kernel(const float* __restrict__ in, long long in_sb,
                                                                       float* __restrict__ out, int B) {
  extern __shared__ __align__(16) float2 zs[];  // [33 lines][PZ], then the mbarrier
  const unsigned bar = smem_u32(zs + kInvLines * PZ);
  unsigned phase = 0;
  if (threadIdx.x == 0) mbar_init(bar, 1);
  fence_async_smem();
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = lane / LP256, line = warp * LP256 + (lane % LP256);
  float2 lf[Q256];
  lane_factors<Q256, true>(q, lf);
  const int bands = N256 / 2 / kLinesPerBlock;  // 4 blocks of 32 lines (and line 128 with the first)
  // transform of the line staged at zs[slot], parked back in natural order
  auto transform = [&](int slot) {
    float2 a[R256];
    const float2* src = zs + slot * PZ + P256 * q;
#pragma unroll
    for (int m = 0; m < Q256; ++m) {
#pragma unroll
      for (int j2 = 0; j2 < P256 / 2; ++j2) {
        const float4 u = *reinterpret_cast<const float4*>(src + R256 * m + 2 * j2);
        a[m * P256 + 2 * j2] = make_float2(u.x, u.y);
        a[m * P256 + 2 * j2 + 1] = make_float2(u.z, u.w);
      }
    }
    coop_fft<N256, R256, Q256, true>(a, q, lf);
    __syncwarp();  // the lanes of a line have read it
    static_for<R256>([&](auto kc) {
      constexpr int k = decltype(kc)::value;
      zs[slot * PZ + Q256 * k + q] = a[brev(k, R256)];
    });
  };
  for (long long work = blockIdx.x; work < (long long)B * bands; work += gridDim.x) {
    const long long b = work / bands;
    const int g = (int)(work % bands), kx0 = g * kLinesPerBlock;
    const float* src = in + b * in_sb;
    fence_async_smem();  // this thread's accesses to the lines precede the copies that overwrite them
    if (threadIdx.x == 0) mbar_expect_tx(bar, (kLinesPerBlock + (g == 0 ? 1 : 0)) * N256 * 8);
    __syncthreads();     // (also: the previous work item's lines have been written out)
    if (q == 0) bulk_g2s(smem_u32(zs + line * PZ), src + (long long)(kx0 + line) * (2 * N256), N256 * 8, bar);
    if (g == 0 && threadIdx.x == 1) bulk_g2s(smem_u32(zs + kLinesPerBlock * PZ), src + (long long)(N256 / 2) * (2 * N256), N256 * 8, bar);
    if (!mbar_wait(bar, phase, kErrInvColsWait)) return;
    phase ^= 1;
    transform(line);
    if (g == 0) {
      __syncthreads();
      if (warp == 0) transform(kLinesPerBlock);  // every lane group of the warp works on line 128
      __syncthreads();
      // slot 0 of every row: (Re T[0][y], Re T[128][y])
      for (int y = threadIdx.x; y < N256; y += kRowsThreads) zs[y].y = zs[kLinesPerBlock * PZ + y].x;
    }
    __syncthreads();
    // out[b][y][2 (kx0 + l) ..]: two lines (16 bytes) per thread, line pair fastest
    float* dst = out + b * ((long long)N256 * N256) + 2 * kx0;
    for (int e = threadIdx.x; e < N256 * (kLinesPerBlock / 2); e += kRowsThreads) {
      const int y = e / (kLinesPerBlock / 2), l2 = e % (kLinesPerBlock / 2);
      const float2 u = zs[(2 * l2) * PZ + y], v = zs[(2 * l2 + 1) * PZ + y];
      *reinterpret_cast<float4*>(dst + (long long)y * N256 + 4 * l2) = make_float4(u.x, u.y, v.x, v.y);
    }
  }
}

__global__ void __launch_bounds__(kColsWarps * 32, 3) ifft256_rows_kernel(float* __restrict__ data, long long pairs) {
  extern __shared__ __align__(16) float2 cs[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, q = lane / LP256, l = lane % LP256;
  float2* region = cs + warp * kColsSlot + l * PZ;
  const unsigned bar = smem_u32(cs + kColsWarps * kColsSlot) + warp * 16;
  if (lane == 0) mbar_init(bar, 1);
  fence_async_smem();
  __syncwarp();
  float2 lf[Q256];
  lane_factors<Q256, true>(q, lf);
  const long long tasks = (pairs + LP256 - 1) / LP256;
  const long long gw = (long long)blockIdx.x * kColsWarps + warp, nw = (long long)gridDim.x * kColsWarps;
  auto issue = [&](long long task) {
    const long long first = task * LP256;
    const int valid = pairs - first < LP256 ? (int)(pairs - first) : LP256;
    if (lane < LP256) bulk_wait_read();  // this lane's pair has left the slot
    __syncwarp();
    if (lane == 0) {
      fence_async_smem();
      mbar_expect_tx(bar, valid * N256 * 8);
    }
    __syncwarp();
    if (lane < valid) bulk_g2s(smem_u32(region), data + (first + l) * (2 * N256), N256 * 8, bar);
  };
  unsigned phase = 0;
  long long t = gw;
  if (t < tasks) issue(t);
  for (; t < tasks; t += nw) {
    if (!mbar_wait(bar, phase, kErrInvRowsWait)) return;
    phase ^= 1;
    // rows y and y + 1 of the pair: slot 0 holds (G[0], G[128]), slot kx holds G[kx] for kx = 1..127
    const float2* ry = region;
    const float2* r1 = region + N256 / 2;
    float2 a[R256];
#pragma unroll
    for (int m = 0; m < Q256; ++m) {
#pragma unroll
      for (int jl = 0; jl < P256; ++jl) {
        const int j = jl + P256 * q + R256 * m;  // bin of the complex line
        if (m < Q256 / 2) {
          const float2 u = ry[j], v = r1[j];     // G_y[j], G_{y+1}[j]
          a[m * P256 + jl] = make_float2(u.x - v.y, u.y + v.x);
        } else {
          const int jj = (N256 - j) & (N256 / 2 - 1);  // mirror bin; j = 128 maps to slot 0
          const float2 u = ry[jj], v = r1[jj];
          a[m * P256 + jl] = make_float2(u.x + v.y, v.x - u.y);
        }
      }
    }
    if (q == 0) {
      // bins 0 and 128 are real for both rows and share slot 0 as (G[0], G[128])
      const float2 u = ry[0], v = r1[0];
      a[0] = make_float2(u.x, v.x);
      a[(Q256 / 2) * P256] = make_float2(u.y, v.y);
    }
    coop_fft<N256, R256, Q256, true>(a, q, lf);
    __syncwarp();
    float* oy = reinterpret_cast<float*>(region);
    static_for<R256>([&](auto kc) {
      constexpr int k = decltype(kc)::value;
      const float2 v = a[brev(k, R256)];
      oy[Q256 * k + q] = v.x;
      oy[N256 + Q256 * k + q] = v.y;
    });
    fence_async_smem();
    __syncwarp();
    const long long pair = t * LP256 + l;
    if (lane < LP256 && pair < pairs) {
      bulk_s2g(data + pair * (2 * N256), smem_u32(region), N256 * 8);
      bulk_commit();
    }
    if (t + nw < tasks) issue(t + nw);
  }
  bulk_wait_read();
}

}  // namespace

bool fft2d_256_inverse_supported(const CplxView& in, const RealView& out, int B, int padL, int padU) {
  if (in.blk_planes) return false;
  const bool in_ok = in.sz == 1 && in.sc == 2 && in.sr == 2 * N256 && (in.sb % 4) == 0 && aligned16(in.p);
  const bool out_ok = out.sx == 1 && out.sy == N256 && out.h == N256 && out.w == N256 && padL == 0 && padU == 0 &&
                      (B <= 1 || out.sb == (long long)N256 * N256) && aligned16(out.p);
  return in_ok && out_ok && B >= 1;
}

int fft2d_256_inverse(const CplxView& in, const RealView& out, int B, cudaStream_t s) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  const int smem = kInvLines * PZ * (int)sizeof(float2) + 16;
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(ifft256_cols_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    cudaFuncSetAttribute(ifft256_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kColsSmem);
    configured[dev] = true;
  }
  const long long work = (long long)B * 4;
  const int cap = sm_count() * 3;
  ifft256_cols_kernel<<<work < cap ? (int)work : cap, kRowsThreads, smem, s>>>(in.p, in.sb, out.p, B);
  if (cudaPeekAtLastError() != cudaSuccess) return kCudaError;
  const long long pairs = (long long)B * (N256 / 2);
  const long long wblocks = (pairs + kColsWarps * LP256 - 1) / (kColsWarps * LP256);
  ifft256_rows_kernel<<<wblocks < cap ? (int)wblocks : cap, kColsWarps * 32, kColsSmem, s>>>(out.p, pairs);
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

bool fft2d_256_supported(const RealView& in, const CplxView& out, int B) {
  if (out.blk_planes) return false;
  const bool out_ok = out.sz == 1 && out.sc == 2 && out.sr == 2 * N256 && out.sb == (long long)(N256 / 2 + 1) * 2 * N256 &&
                      aligned16(out.p);
  return out_ok && B >= 1 && in.h <= N256 && in.w <= N256;
}

int fft2d_256_forward(const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  const int smem = kLinesPerBlock * PZ * (int)sizeof(float2) + 16;
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(fft256_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    cudaFuncSetAttribute(fft256_rows_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    cudaFuncSetAttribute(fft256_cols_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kColsSmem);
    configured[dev] = true;
  }
  const long long work = (long long)B * 4;
  const int cap = sm_count() * 3;
  const int grid = work < cap ? (int)work : cap;
  const bool full = in.sx == 1 && in.sy == N256 && in.h == N256 && in.w == N256 && padL == 0 && padU == 0 &&
                    (in.sb % 4) == 0 && aligned16(in.p);
  if (full) {
    fft256_rows_kernel<true><<<grid, kRowsThreads, smem, s>>>(in, out.p, out.sb, B, padL, padU);
  } else {
    fft256_rows_kernel<false><<<grid, kRowsThreads, smem, s>>>(in, out.p, out.sb, B, padL, padU);
  }
  if (cudaPeekAtLastError() != cudaSuccess) return kCudaError;
  const long long lines = (long long)B * (N256 / 2 + 1);
  const long long wblocks = (lines + kColsWarps * LP256 - 1) / (kColsWarps * LP256);
  const int grid2 = wblocks < cap ? (int)wblocks : cap;
  fft256_cols_kernel<<<grid2, kColsWarps * 32, kColsSmem, s>>>(out.p, lines);
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

int read_device_error_256() { return device_error_word_read(); }
int clear_device_error_256() { return device_error_word_clear(); }

}  // namespace fbfft_b200
