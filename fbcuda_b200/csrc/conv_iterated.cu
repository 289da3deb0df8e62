// FFTIteratedConvolution<8|16|32>: the reference's tile-list convolution entry
// point (fbfft/FFTIteratedConvolution.cuh:624-755).  Like the reference's kernels
// (:97-207, :254-363, :409-524) it needs no device memory besides its operands:
// every spectrum is recomputed where it is used.  Two kernels: a block of 8 warps
// produces a group of 4 x 4 output planes and shares the operand spectra inside the
// group (iterated_grouped_kernel, further down; layers with at least 3 planes on
// both sides of the group), or one warp produces one output plane:
//   pass 0  out[tile][b][o] = sum_c  in[tile][b][c]  (x) conj(w[o][c])
//   pass 1  in [tile][b][c] = sum_o  out[tile][b][o] (x) w[o][c]
//   pass 2  w[o][c]         = scale * sum_tile,b in[tile][b][c] (x) conj(out[tile][b][o])
// all scaled by 1/N^2.  The two operands of a product are transformed side by side
// by the same warp (they are the "images" of one pass of the batched 2-D kernel,
// fft2d_small.cuh), multiplied bin by bin out of shared memory and accumulated in
// registers; one inverse transform per output plane follows.  Tile descriptors are
// read on the device, as in the reference (:113-114).
//
// This entry point keeps the reference's contract (no workspace).  Layers where a
// workspace is available run much faster through fbfft_b200_conv_* (conv.cu), which
// transforms every plane once.
#include "../../include/fbfft_b200.h"
#include "fft2d_small.cuh"
#include "kernels.h"

namespace fbfft_b200 {

namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;

struct Weight4 {
  float* p;
  int size[4];
  int stride[4];
};

template <int N, int PASS>
__global__ void __launch_bounds__(kThreads, 3) iterated_kernel(const fbfft_tiled_tensor4* __restrict__ ins,
                                                              const fbfft_tiled_tensor4* __restrict__ outs, Weight4 w,
                                                              float scale, int batch, int num_tiles, int num_items) {
  constexpr int T = N / 2, IPW = 32 / T, ROWS = T + 1, PP = IPW / 2;
  constexpr int RS = SmallCfg<N>::RS, IS = SmallCfg<N>::IS;
  constexpr int BINS = ROWS * N, ACC = (BINS + 31) / 32;
  extern __shared__ __align__(16) float2 smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float2* buf = smem + warp * (IPW * IS);
  const int li = lane / T, l = lane % T;
  float2* ib = buf + li * IS;
  const int pair = li >> 1, second = li & 1;
  const int O = w.size[0], C = w.size[1];

  for (int item = blockIdx.x * kWarps + warp; item < num_items; item += gridDim.x * kWarps) {
    // item -> (tile, b, plane) for passes 0/1, (o, c) for pass 2
    int tile = 0, b = 0, plane = 0, o = 0, c = 0;
    if (PASS == 2) {
      o = item / C;
      c = item % C;
    } else {
      const int planes = PASS == 0 ? O : C;
      plane = item % planes;
      b = (item / planes) % batch;
      tile = item / (planes * batch);
    }
    float2 acc[ACC];
#pragma unroll
    for (int j = 0; j < ACC; ++j) acc[j] = make_float2(0.f, 0.f);

    const int outer = PASS == 2 ? num_tiles : 1;
    for (int t = 0; t < outer; ++t) {
      const fbfft_tiled_tensor4& ti = ins[PASS == 2 ? t : tile];
      const fbfft_tiled_tensor4& to = outs[PASS == 2 ? t : tile];
      const int K = PASS == 0 ? C : (PASS == 1 ? O : ti.size[0]);
      if (PASS != 2 && b >= ti.size[0]) continue;
      for (int k0 = 0; k0 < K; k0 += PP) {
        const int k = k0 + pair;
        const bool valid = k < K;
        const float* src = nullptr;
        long long sy = 0, sx = 0;
        int h = 0, wd = 0, pl = 0, pu = 0;
        if (valid) {
          // first operand (second == 0) and second operand (second == 1) of the product
          if (PASS == 0) {
            if (!second) {
              src = ti.data + (long long)b * ti.stride[0] + (long long)k * ti.stride[1];
              sy = ti.stride[2], sx = ti.stride[3], h = ti.size[2], wd = ti.size[3], pl = ti.padL, pu = ti.padU;
            } else {
              src = w.p + (long long)plane * w.stride[0] + (long long)k * w.stride[1];
              sy = w.stride[2], sx = w.stride[3], h = w.size[2], wd = w.size[3];
            }
          } else if (PASS == 1) {
            if (!second) {
              src = to.data + (long long)b * to.stride[0] + (long long)k * to.stride[1];
              sy = to.stride[2], sx = to.stride[3], h = to.size[2], wd = to.size[3], pl = to.padL, pu = to.padU;
            } else {
              src = w.p + (long long)k * w.stride[0] + (long long)plane * w.stride[1];
              sy = w.stride[2], sx = w.stride[3], h = w.size[2], wd = w.size[3];
            }
          } else {
            if (!second) {
              src = ti.data + (long long)k * ti.stride[0] + (long long)c * ti.stride[1];
              sy = ti.stride[2], sx = ti.stride[3], h = ti.size[2], wd = ti.size[3], pl = ti.padL, pu = ti.padU;
            } else {
              src = to.data + (long long)k * to.stride[0] + (long long)o * to.stride[1];
              sy = to.stride[2], sx = to.stride[3], h = to.size[2], wd = to.size[3], pl = to.padL, pu = to.padU;
            }
          }
        }
        {
          float2 a[N];
          load_columns<N>(src, sy, sx, h, wd, pl, pu, valid, l, a);
          fft_bitrev<N, false>(a);
          fwd_separate_store<N>(a, ib, l);
        }
        __syncwarp();
        fwd_rows_unpack<N>(ib, l);
        // multiply-accumulate bin by bin; lane owns bins lane, lane+32, ...
#pragma unroll
        for (int j = 0; j < ACC; ++j) {
          const int e = lane + 32 * j;
          if (e < BINS) {
            const int off = (e / N) * RS + (e % N);
#pragma unroll
            for (int p = 0; p < PP; ++p) {
              if (k0 + p < K) {
                const float2 x = buf[(2 * p) * IS + off], y = buf[(2 * p + 1) * IS + off];
                if (PASS == 1) {  // x * y
                  acc[j].x += x.x * y.x - x.y * y.y;
                  acc[j].y += x.x * y.y + x.y * y.x;
                } else {          // x * conj(y)
                  acc[j].x += x.x * y.x + x.y * y.y;
                  acc[j].y += x.y * y.x - x.x * y.y;
                }
              }
            }
          }
        }
        __syncwarp();
      }
    }
    // inverse transform of the accumulated spectrum (image slot 0 of the warp)
#pragma unroll
    for (int j = 0; j < ACC; ++j) {
      const int e = lane + 32 * j;
      if (e < BINS) buf[(e / N) * RS + (e % N)] = acc[j];
    }
    __syncwarp();
    inv_pack_rows<N>(ib, l);
    {
      float2 z[N];
      inv_columns<N>(ib, l, z);
      if (li == 0) {
        const float inv = 1.0f / (float)(N * N);
        if (PASS == 0) {
          const fbfft_tiled_tensor4& to = outs[tile];
          if (b < to.size[0])
            store_columns<N>(to.data + (long long)b * to.stride[0] + (long long)plane * to.stride[1], to.stride[2],
                             to.stride[3], to.size[2], to.size[3], to.padL, to.padU, l, z, inv);
        } else if (PASS == 1) {
          const fbfft_tiled_tensor4& ti = ins[tile];
          if (b < ti.size[0])
            store_columns<N>(ti.data + (long long)b * ti.stride[0] + (long long)plane * ti.stride[1], ti.stride[2],
                             ti.stride[3], ti.size[2], ti.size[3], ti.padL, ti.padU, l, z, inv);
        } else {
          store_columns<N>(w.p + (long long)o * w.stride[0] + (long long)c * w.stride[1], w.stride[2], w.stride[3],
                           w.size[2], w.size[3], 0, 0, l, z, inv * scale);
        }
      }
    }
    __syncwarp();
  }
}

// Grouped version: a block of 8 warps produces a group of 4 x 4 output planes,
//   P[i][j] = sum_k X[i][k] (x) op(Y[j][k]),   i, j in 0..3,
//   pass 0  X = in[tile][b0+i][c=k],   Y = w[o0+j][c=k]      -> out[tile][b0+i][o0+j]
//   pass 1  X = out[tile][b0+i][o=k],  Y = w[o=k][c0+j]      -> in[tile][b0+i][c0+j]
//   pass 2  X = in[tile][b=k][c0+i],   Y = out[tile][b=k][o0+j] (summed over the tiles too) -> w[o0+j][c0+i]
// so the 8 spectra of a value of k are computed once and multiplied 16 times: a quarter of the
// transforms of the one-plane-per-warp kernel above, still without any device memory besides the
// operands.  The 8 warps transform 8 * IPW images side by side (the 4 + 4 members of IPW / 2 values
// of k), meet at a barrier, and warp w accumulates the products (w / 2, 2 (w % 2)) and
// (w / 2, 2 (w % 2) + 1) of every k of the round in registers (three shared-memory reads per two
// complex multiply-adds); at the end it inverse transforms its two sums side by side.
// Members beyond the tensors (group tails) are transformed as zero images and never stored.
constexpr int kGThreads = 256, kGWarps = 8, kGroup = 4;

template <int N, int PASS>
__global__ void __launch_bounds__(kGThreads, 1) iterated_grouped_kernel(const fbfft_tiled_tensor4* __restrict__ ins,
                                                                       const fbfft_tiled_tensor4* __restrict__ outs, Weight4 w,
                                                                       float scale, int num_tiles, int gi_count, int gj_count,
                                                                       int num_items) {
  constexpr int T = N / 2, IPW = 32 / T, ROWS = T + 1;
  constexpr int RS = SmallCfg<N>::RS, IS = SmallCfg<N>::IS;
  constexpr int BINS = ROWS * N, ACC = (BINS + 31) / 32;
  constexpr int KPI = kGWarps * IPW / (2 * kGroup);  // values of k per round
  extern __shared__ __align__(16) float2 smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int li = lane / T, l = lane % T;
  const int gslot = warp * IPW + li;              // image slot of this lane group: (k of the round, member)
  const int kl = gslot / (2 * kGroup), member = gslot % (2 * kGroup);
  float2* ib = smem + gslot * IS;
  const int mi = warp >> 1, mj = (warp & 1) * 2;  // this warp's products (mi, mj) and (mi, mj + 1)
  const int O = w.size[0], C = w.size[1];

  for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
    const int jg = item % gj_count, ig = (item / gj_count) % gi_count, tile = item / (gj_count * gi_count);
    const int i0 = ig * kGroup, j0 = jg * kGroup;
    float2 acc[2][ACC];
#pragma unroll
    for (int j = 0; j < ACC; ++j) acc[0][j] = acc[1][j] = make_float2(0.f, 0.f);

    const int outer = PASS == 2 ? num_tiles : 1;
    for (int t = 0; t < outer; ++t) {
      const fbfft_tiled_tensor4& ti = ins[PASS == 2 ? t : tile];
      const fbfft_tiled_tensor4& to = outs[PASS == 2 ? t : tile];
      const int K = PASS == 0 ? C : (PASS == 1 ? O : ti.size[0]);
      for (int k0 = 0; k0 < K; k0 += KPI) {
        const int k = k0 + kl;
        bool valid = k < K;
        const float* src = nullptr;
        long long sy = 0, sx = 0;
        int h = 0, wd = 0, pl = 0, pu = 0;
        const bool is_x = member < kGroup;
        const int idx = (is_x ? i0 : j0 - kGroup) + member;  // b, c or o of this member
        if (PASS == 0) {
          if (is_x) {
            valid = valid && idx < ti.size[0];
            src = ti.data + (long long)idx * ti.stride[0] + (long long)k * ti.stride[1];
            sy = ti.stride[2], sx = ti.stride[3], h = ti.size[2], wd = ti.size[3], pl = ti.padL, pu = ti.padU;
          } else {
            valid = valid && idx < O;
            src = w.p + (long long)idx * w.stride[0] + (long long)k * w.stride[1];
            sy = w.stride[2], sx = w.stride[3], h = w.size[2], wd = w.size[3];
          }
        } else if (PASS == 1) {
          if (is_x) {
            valid = valid && idx < to.size[0];
            src = to.data + (long long)idx * to.stride[0] + (long long)k * to.stride[1];
            sy = to.stride[2], sx = to.stride[3], h = to.size[2], wd = to.size[3], pl = to.padL, pu = to.padU;
          } else {
            valid = valid && idx < C;
            src = w.p + (long long)k * w.stride[0] + (long long)idx * w.stride[1];
            sy = w.stride[2], sx = w.stride[3], h = w.size[2], wd = w.size[3];
          }
        } else {
          if (is_x) {
            valid = valid && idx < C;
            src = ti.data + (long long)k * ti.stride[0] + (long long)idx * ti.stride[1];
            sy = ti.stride[2], sx = ti.stride[3], h = ti.size[2], wd = ti.size[3], pl = ti.padL, pu = ti.padU;
          } else {
            valid = valid && idx < O;
            src = to.data + (long long)k * to.stride[0] + (long long)idx * to.stride[1];
            sy = to.stride[2], sx = to.stride[3], h = to.size[2], wd = to.size[3], pl = to.padL, pu = to.padU;
          }
        }
        if (!valid) src = w.p;  // (never dereferenced: every element is predicated off)
        {
          float2 a[N];
          load_columns<N>(src, sy, sx, h, wd, pl, pu, valid, l, a);
          fft_bitrev<N, false>(a);
          fwd_separate_store<N>(a, ib, l);
        }
        __syncwarp();
        fwd_rows_unpack<N>(ib, l);
        __syncthreads();
#pragma unroll
        for (int r = 0; r < KPI; ++r) {
          if (k0 + r < K) {
            const float2* X = smem + (r * 2 * kGroup + mi) * IS;
            const float2* Ya = smem + (r * 2 * kGroup + kGroup + mj) * IS;
            const float2* Yb = Ya + IS;
#pragma unroll
            for (int j = 0; j < ACC; ++j) {
              const int e = lane + 32 * j;
              if (e < BINS) {
                const int off = (e / N) * RS + (e % N);
                const float2 x = X[off], ya = Ya[off], yb = Yb[off];
                if (PASS == 1) {  // x * y
                  acc[0][j].x += x.x * ya.x - x.y * ya.y;
                  acc[0][j].y += x.x * ya.y + x.y * ya.x;
                  acc[1][j].x += x.x * yb.x - x.y * yb.y;
                  acc[1][j].y += x.x * yb.y + x.y * yb.x;
                } else {          // x * conj(y)
                  acc[0][j].x += x.x * ya.x + x.y * ya.y;
                  acc[0][j].y += x.y * ya.x - x.x * ya.y;
                  acc[1][j].x += x.x * yb.x + x.y * yb.y;
                  acc[1][j].y += x.y * yb.x - x.x * yb.y;
                }
              }
            }
          }
        }
        __syncthreads();
      }
    }
    // the warp's two sums go to its first two image slots and are inverse transformed side by side
    float2* buf = smem + warp * IPW * IS;
#pragma unroll
    for (int j = 0; j < ACC; ++j) {
      const int e = lane + 32 * j;
      if (e < BINS) {
        const int off = (e / N) * RS + (e % N);
        buf[off] = acc[0][j];
        buf[IS + off] = acc[1][j];
      }
    }
    __syncwarp();
    inv_pack_rows<N>(ib, l);
    {
      float2 z[N];
      inv_columns<N>(ib, l, z);
      if (li < 2) {
        const float inv = 1.0f / (float)(N * N);
        const int i = i0 + mi, j = j0 + mj + li;
        if (PASS == 0) {
          const fbfft_tiled_tensor4& to = outs[tile];
          if (i < to.size[0] && j < O)
            store_columns<N>(to.data + (long long)i * to.stride[0] + (long long)j * to.stride[1], to.stride[2], to.stride[3],
                             to.size[2], to.size[3], to.padL, to.padU, l, z, inv);
        } else if (PASS == 1) {
          const fbfft_tiled_tensor4& ti = ins[tile];
          if (i < ti.size[0] && j < C)
            store_columns<N>(ti.data + (long long)i * ti.stride[0] + (long long)j * ti.stride[1], ti.stride[2], ti.stride[3],
                             ti.size[2], ti.size[3], ti.padL, ti.padU, l, z, inv);
        } else {
          if (i < C && j < O)
            store_columns<N>(w.p + (long long)j * w.stride[0] + (long long)i * w.stride[1], w.stride[2], w.stride[3], w.size[2],
                             w.size[3], 0, 0, l, z, inv * scale);
        }
      }
    }
    __syncthreads();  // the slots are rewritten by the next item's transforms
  }
}

template <int N, int PASS>
bool launch_grouped(const fbfft_tiled_tensor4* ins, const fbfft_tiled_tensor4* outs, const Weight4& w, float scale, int num_tiles,
                    int ni, int nj, int tiles_outer, cudaStream_t s) {
  constexpr int IPW = 32 / (N / 2);
  const int smem = kGWarps * IPW * SmallCfg<N>::IS * (int)sizeof(float2);
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(iterated_grouped_kernel<N, PASS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    configured[dev] = true;
  }
  const int gi = (ni + kGroup - 1) / kGroup, gj = (nj + kGroup - 1) / kGroup;
  const long long items = (long long)tiles_outer * gi * gj;
  if (items <= 0 || items > 0x7fffffffLL) return false;
  const int cap = sm_count() * 2;
  const int grid = items < cap ? (int)items : cap;
  iterated_grouped_kernel<N, PASS><<<grid, kGThreads, smem, s>>>(ins, outs, w, scale, num_tiles, gi, gj, (int)items);
  return cudaPeekAtLastError() == cudaSuccess;
}

template <int N>
int launch(const fbfft_tiled_tensor4* ins, const fbfft_tiled_tensor4* outs, const Weight4& w, int pass, float scale,
           int batch, int num_tiles, cudaStream_t s) {
  constexpr int IPW = 32 / (N / 2);
  const int smem = kWarps * IPW * SmallCfg<N>::IS * (int)sizeof(float2);
  const long long items = pass == 0 ? (long long)num_tiles * batch * w.size[0]
                                    : (pass == 1 ? (long long)num_tiles * batch * w.size[1]
                                                 : (long long)w.size[0] * w.size[1]);
  if (items <= 0) return 1;
  if (items > 0x7fffffffLL) return 0;
  // groups of 4 x 4 output planes share their spectra whenever both sides of the group have at least 3 members
  {
    const int O = w.size[0], C = w.size[1];
    if (pass == 0 && batch >= 3 && O >= 3) return launch_grouped<N, 0>(ins, outs, w, scale, num_tiles, batch, O, num_tiles, s) ? 1 : 0;
    if (pass == 1 && batch >= 3 && C >= 3) return launch_grouped<N, 1>(ins, outs, w, scale, num_tiles, batch, C, num_tiles, s) ? 1 : 0;
    if (pass == 2 && C >= 3 && O >= 3) return launch_grouped<N, 2>(ins, outs, w, scale, num_tiles, C, O, 1, s) ? 1 : 0;
  }
  const int want = (int)((items + kWarps - 1) / kWarps), cap = sm_count() * 16;
  const int grid = want < cap ? want : cap;
  if (pass == 0) iterated_kernel<N, 0><<<grid, kThreads, smem, s>>>(ins, outs, w, scale, batch, num_tiles, (int)items);
  if (pass == 1) iterated_kernel<N, 1><<<grid, kThreads, smem, s>>>(ins, outs, w, scale, batch, num_tiles, (int)items);
  if (pass == 2) iterated_kernel<N, 2><<<grid, kThreads, smem, s>>>(ins, outs, w, scale, batch, num_tiles, (int)items);
  return cudaPeekAtLastError() == cudaSuccess ? 1 : 0;
}

}  // namespace

int iterated_convolution(int fft_size, const fbfft_tiled_tensor4* ins, const fbfft_tiled_tensor4* outs, float* weight,
                         const int* weight_size, const int* weight_stride, int pass, float scale, int batch_size,
                         size_t num_tiles, cudaStream_t s) {
  Weight4 w;
  w.p = weight;
  for (int d = 0; d < 4; ++d) {
    w.size[d] = weight_size[d];
    w.stride[d] = weight_stride[d];
  }
  if (num_tiles == 0 || num_tiles > 0x7fffffffu || batch_size < 0) return 0;
  if (pass != 2 && batch_size == 0) return 1;
  switch (fft_size) {
    case 8:
      return launch<8>(ins, outs, w, pass, scale, batch_size, (int)num_tiles, s);
    case 16:
      return launch<16>(ins, outs, w, pass, scale, batch_size, (int)num_tiles, s);
    case 32:
      return launch<32>(ins, outs, w, pass, scale, batch_size, (int)num_tiles, s);
    default:
      return 0;
  }
}

}  // namespace fbfft_b200
