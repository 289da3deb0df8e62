// fbfft2D / fbifft2D for N = 8 on contiguous full 8 x 8 images: one thread per image.
//
// The general N <= 32 kernel (fft2d_small.cu) gives an image to N/2 lanes and moves lines between
// them through shared memory once per pass; at N = 8 that is 4 lanes for 64 values, and the kernel
// runs at 0.80 of the copy bandwidth on issue slots, not bytes.  Here a thread holds the whole
// image in registers -- both passes are fully unrolled 8-point FFTs with compile-time twiddles
// (fft_regs.cuh), no shuffle, no barrier -- and shared memory is only the staging area of the
// copies:
//   task     32 consecutive images, one per lane of a warp
//   forward  every lane brings its 256 bytes in with one cp.async.bulk into its own region (pitch
//            336 bytes: the 16-byte reads and writes of 8 lanes fall on different banks; completion
//            on the warp's mbarrier, bounded wait); columns x and x + 4 travel as re/im of one complex
//            line through the transform along y and are separated (fbfft/FBFFTCommon.cuh:323-350), the
//            5 stored rows ky = 0..4 are transformed along x, written back into the lane's region
//            (320 bytes) and leave by one bulk store per lane.  Two slots per warp: the next task's
//            images arrive while this one is transformed.
//   inverse  the mirror image: 320 bytes in, rows ky = 0..4 along kx, Hermitian extension of the column
//            pairs (the imaginary parts of ky = 0 and ky = 4 carry nothing for a real image), unnormalised
//            inverse along ky, 256 bytes out.
// Layout as for every N <= 32: stored spectrum S[ky][kx], ky = 0..4, kx = 0..7 (fbfft/FBFFT2D-inl.cuh:480-617).
// Images beyond the last whole group of 32, padded, cropped or strided tensors and the blocked
// workspace layouts stay with the general kernel.
#include "fft2d_small.cuh"  // bulk-copy / mbarrier helpers
#include "fft_regs.cuh"
#include "kernels.h"

namespace fbfft_b200 {

namespace {

constexpr int kN8Warps = 4, kN8Pitch = 84;  // floats per lane region (336 bytes)
constexpr int kN8Slot = 32 * kN8Pitch;      // floats per slot
constexpr int kN8Smem = kN8Warps * (2 * kN8Slot * 4 + 16);
enum : int { kErrN8Wait = 121 };

template <bool INV>
__global__ void __launch_bounds__(kN8Warps * 32, 2) fft2d_n8_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                                   long long tasks) {
  constexpr int IN_F = INV ? 80 : 64, OUT_F = INV ? 64 : 80;  // floats per image
  extern __shared__ __align__(16) float sm8[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* slots = sm8 + warp * 2 * kN8Slot;
  const unsigned bars = smem_u32(sm8 + kN8Warps * 2 * kN8Slot) + warp * 16;
  if (lane == 0) {
    mbar_init(bars, 1);
    mbar_init(bars + 8, 1);
  }
  fence_async_smem();
  __syncwarp();
  const long long gw = (long long)blockIdx.x * kN8Warps + warp, nw = (long long)gridDim.x * kN8Warps;
  auto issue = [&](long long task, int slot) {
    bulk_wait_read();  // this lane's previous result has left the slot
    __syncwarp();
    if (lane == 0) {
      fence_async_smem();
      mbar_expect_tx(bars + 8 * slot, 32 * IN_F * 4);
    }
    __syncwarp();
    bulk_g2s(smem_u32(slots + slot * kN8Slot + lane * kN8Pitch), src + (task * 32 + lane) * IN_F, IN_F * 4, bars + 8 * slot);
  };
  unsigned phases = 0;
  long long t = gw;
  if (t < tasks) issue(t, 0);
  for (int i = 0; t < tasks; t += nw, ++i) {
    const int slot = i & 1;
    if (t + nw < tasks) issue(t + nw, slot ^ 1);
    if (!mbar_wait(bars + 8 * slot, (phases >> slot) & 1, kErrN8Wait)) return;
    phases ^= 1u << slot;
    float* reg = slots + slot * kN8Slot + lane * kN8Pitch;
    if constexpr (!INV) {
      float img[8][8];
#pragma unroll
      for (int y = 0; y < 8; ++y) {
        const float4 u = *reinterpret_cast<const float4*>(reg + 8 * y), v = *reinterpret_cast<const float4*>(reg + 8 * y + 4);
        img[y][0] = u.x, img[y][1] = u.y, img[y][2] = u.z, img[y][3] = u.w;
        img[y][4] = v.x, img[y][5] = v.y, img[y][6] = v.z, img[y][7] = v.w;
      }
      __syncwarp();  // (the region is rewritten below at the same pitch by the same lane; nothing to wait for)
      // along y: columns x and x + 4 as one complex line; G[ky][x] for ky = 0..4
      float2 g[5][8];
      static_for<4>([&](auto xc) {
        constexpr int x = decltype(xc)::value;
        float2 z[8];
#pragma unroll
        for (int y = 0; y < 8; ++y) z[y] = make_float2(img[y][x], img[y][x + 4]);
        fft_bitrev<8, false>(z);
        static_for<5>([&](auto kc) {
          constexpr int k = decltype(kc)::value;
          const float2 a = z[brev(k, 8)], m = z[brev((8 - k) % 8, 8)];
          g[k][x] = make_float2(0.5f * (a.x + m.x), 0.5f * (a.y - m.y));
          g[k][x + 4] = make_float2(0.5f * (a.y + m.y), 0.5f * (m.x - a.x));
        });
      });
      // along x for the 5 stored rows; S[ky][kx] at reg[(ky * 8 + kx) * 2]
      static_for<5>([&](auto kc) {
        constexpr int k = decltype(kc)::value;
        fft_bitrev<8, false>(g[k]);
        static_for<4>([&](auto jc) {
          constexpr int j = 2 * decltype(jc)::value;
          const float2 p = g[k][brev(j, 8)], q = g[k][brev(j + 1, 8)];
          *reinterpret_cast<float4*>(reg + (k * 8 + j) * 2) = make_float4(p.x, p.y, q.x, q.y);
        });
      });
    } else {
      // along kx for the 5 stored rows: G[ky][x]
      float2 g[5][8];
      static_for<5>([&](auto kc) {
        constexpr int k = decltype(kc)::value;
        static_for<4>([&](auto jc) {
          constexpr int j = 2 * decltype(jc)::value;
          const float4 u = *reinterpret_cast<const float4*>(reg + (k * 8 + j) * 2);
          g[k][j] = make_float2(u.x, u.y), g[k][j + 1] = make_float2(u.z, u.w);
        });
        fft_bitrev<8, true>(g[k]);
      });
      __syncwarp();
      // along ky: Z[ky] = G_x[ky] + i G_{x+4}[ky], Z[8 - ky] = conj(G_x[ky]) + i conj(G_{x+4}[ky])
      float out[8][8];
      static_for<4>([&](auto xc) {
        constexpr int x = decltype(xc)::value;
        float2 z[8];
        static_for<5>([&](auto kc) {
          constexpr int k = decltype(kc)::value;
          const float2 a = g[k][brev(x, 8)], b = g[k][brev(x + 4, 8)];
          if constexpr (k == 0 || k == 4) {
            z[k] = make_float2(a.x, b.x);  // real for a real image
          } else {
            z[k] = make_float2(a.x - b.y, a.y + b.x);
            z[8 - k] = make_float2(a.x + b.y, b.x - a.y);
          }
        });
        fft_bitrev<8, true>(z);
#pragma unroll
        for (int y = 0; y < 8; ++y) {
          out[y][x] = z[brev(y, 8)].x;
          out[y][x + 4] = z[brev(y, 8)].y;
        }
      });
#pragma unroll
      for (int y = 0; y < 8; ++y) {
        *reinterpret_cast<float4*>(reg + 8 * y) = make_float4(out[y][0], out[y][1], out[y][2], out[y][3]);
        *reinterpret_cast<float4*>(reg + 8 * y + 4) = make_float4(out[y][4], out[y][5], out[y][6], out[y][7]);
      }
    }
    fence_async_smem();
    bulk_s2g(dst + (t * 32 + lane) * OUT_F, smem_u32(reg), OUT_F * 4);
    bulk_commit();
  }
  bulk_wait_read();
}

template <bool INV>
int launch_n8(const float* src, float* dst, long long tasks, cudaStream_t s) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(fft2d_n8_kernel<INV>, cudaFuncAttributeMaxDynamicSharedMemorySize, kN8Smem);
    configured[dev] = true;
  }
  const long long want = (tasks + kN8Warps - 1) / kN8Warps, cap = (long long)sm_count() * 2;
  fft2d_n8_kernel<INV><<<(int)(want < cap ? want : cap), kN8Warps * 32, kN8Smem, s>>>(src, dst, tasks);
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

}  // namespace

// contiguous [B][8][8] real and [B][5][8][2] complex tensors, 16-byte aligned, no padding or crop
bool fft2d_n8_supported(const RealView& real, const CplxView& cplx, int B, int padL, int padU) {
  if (cplx.blk_planes || padL != 0 || padU != 0 || B < 32) return false;
  const bool r_ok = real.h == 8 && real.w == 8 && real.sx == 1 && real.sy == 8 && real.sb == 64 && aligned16(real.p);
  const bool c_ok = cplx.sz == 1 && cplx.sc == 2 && cplx.sr == 16 && cplx.sb == 80 && aligned16(cplx.p);
  return r_ok && c_ok;
}

// transforms the first `tasks` * 32 images
int fft2d_n8(bool inverse, const float* src, float* dst, long long tasks, cudaStream_t s) {
  if (tasks <= 0) return kSuccess;
  return inverse ? launch_n8<true>(src, dst, tasks, s) : launch_n8<false>(src, dst, tasks, s);
}

int read_device_error_n8() { return device_error_word_read(); }
int clear_device_error_n8() { return device_error_word_clear(); }

}  // namespace fbfft_b200
