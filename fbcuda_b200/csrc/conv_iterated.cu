// FFTIteratedConvolution<8|16|32>: the reference's tile-list convolution entry
// point (fbfft/FFTIteratedConvolution.cuh:624-755).  Like the reference's kernels
// (:97-207, :254-363, :409-524) it needs no device memory besides its operands:
// every spectrum is recomputed where it is used.  One warp produces one output
// plane:
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
