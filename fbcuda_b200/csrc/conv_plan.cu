// The step above the convolution passes: which transform size to use for a layer, and the loop
// over overlap-save tiles when the image is larger than the transform.
//
// In the reference both lived in the caller: it picked the instantiation
// FFTIteratedConvolution<8|16|32> (fbfft/FFTIteratedConvolution.cuh:624-755) or chained
// fbfft2D / transposeMM / fbifft2D for larger sizes, and it built the tile lists the kernels walk
// (fbfft/FFTIteratedConvolution.cuh:70-95, 105-114, 431-442).  Host code only.
#include <vector>

#include "../../include/fbfft_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace fbfft_b200 {
namespace {

int fail(int code, const char* msg) {
  set_last_error(msg);
  return code;
}

long long cdiv(long long a, long long b) { return (a + b - 1) / b; }

// Cost model of one pass of a layer at transform size n, in microseconds.  A pass writes and reads
// the spectra of its two batch-sized tensors once per tile, streams the weight spectrum once per
// tile (and writes it once), and multiplies 3 x 8 B C O flops per bin and tile on the tensor cores;
// every tile costs a handful of launches that small grids do not hide.  The constants are fitted to
// measurements of the passes on a B200 (2 TB/s-class effective spectrum traffic, 600 TFLOP/s of split
// products, 25 us per tile) and only have to rank the candidates.
double pass_cost_us(int n, long long B, long long C, long long O, int OH, int OW, int kh, int kw, long long* tiles_out) {
  const int th = n - kh + 1, tw = n - kw + 1;
  if (th < 1 || tw < 1) return -1.0;
  const long long tiles = cdiv(OH, th) * cdiv(OW, tw);
  const double bins = (double)(n / 2 + 1) * n;
  const double bytes = 8.0 * bins * ((double)tiles * (2.0 * B * C + 2.0 * B * O + (double)O * C) + (double)O * C);
  const double flops = 3.0 * 8.0 * (double)B * C * O * bins * (double)tiles;
  if (tiles_out) *tiles_out = tiles;
  return bytes / 3.5e6 + flops / 6.0e8 + 25.0 * (double)tiles;
}

struct Tile {
  fbfft_tiled_tensor4 in, out;
};

// the tile windows of a layer (style 0 or 1 of fbfft_b200_plan_tiles) as host descriptors
int tiles_of(int n, int kh, int kw, int pad_h, int pad_w, int style, const float* in, const int* in_size,
             const int* in_stride, const float* out, const int* out_size, const int* out_stride, std::vector<Tile>* tiles) {
  const int count = fbfft_b200_plan_tiles(n, kh, kw, pad_h, pad_w, style, const_cast<float*>(in), in_size, in_stride,
                                          const_cast<float*>(out), out_size, out_stride, nullptr, nullptr, 0);
  if (count < 0) return kUnsupportedDimension;
  std::vector<fbfft_tiled_tensor4> ins(count), outs(count);
  fbfft_b200_plan_tiles(n, kh, kw, pad_h, pad_w, style, const_cast<float*>(in), in_size, in_stride,
                        const_cast<float*>(out), out_size, out_stride, ins.data(), outs.data(), (size_t)count);
  tiles->resize(count);
  for (int i = 0; i < count; ++i) (*tiles)[i] = Tile{ins[i], outs[i]};
  return kSuccess;
}

bool null_any(const void* a, const void* b, const void* c, const void* d, const void* e, const void* f) {
  return !a || !b || !c || !d || !e || !f;
}

}  // namespace
}  // namespace fbfft_b200

using namespace fbfft_b200;

extern "C" {

int fbfft_b200_conv_plan(int batch, int in_planes, int out_planes, int in_h, int in_w, int kernel_h, int kernel_w,
                         int pad_h, int pad_w, int world, fbfft_b200_conv_plan_t* plan) {
  if (!plan) return fail(kUnsupportedDimension, "conv_plan: null output");
  if (batch < 1 || in_planes < 1 || out_planes < 1 || kernel_h < 1 || kernel_w < 1 || pad_h < 0 || pad_w < 0 || world < 1)
    return fail(kUnsupportedDimension, "conv_plan: sizes must be positive, pads non-negative");
  const int OH = in_h + 2 * pad_h - kernel_h + 1, OW = in_w + 2 * pad_w - kernel_w + 1;
  if (OH < 1 || OW < 1) return fail(kUnsupportedDimension, "conv_plan: the kernel is larger than the padded image");
  if (kernel_h > 128 || kernel_w > 128) return fail(kUnsupportedSize, "conv_plan: kernels above 128 do not fit the largest transform");
  const long long shard = (batch + world - 1) / world;  // images per GPU
  const int sizes[5] = {8, 16, 32, 64, 128};
  double best = -1.0;
  int best_n = 0;
  long long best_tiles = 0;
  for (int i = 0; i < 5; ++i) {
    long long tiles = 0;
    const double us = pass_cost_us(sizes[i], shard, in_planes, out_planes, OH, OW, kernel_h, kernel_w, &tiles);
    plan->est_us[i] = us < 0 ? 0.0f : (float)us;
    // a transform no larger than the kernel yields tiles of a single output: never worth it
    if (us < 0 || sizes[i] < 2 * kernel_h - 1 || sizes[i] < 2 * kernel_w - 1) continue;
    if (best < 0 || us < best) best = us, best_n = sizes[i], best_tiles = tiles;
  }
  if (best_n == 0) {
    // kernels above 64: only the largest transform holds them
    long long tiles = 0;
    best = pass_cost_us(128, shard, in_planes, out_planes, OH, OW, kernel_h, kernel_w, &tiles);
    best_n = 128, best_tiles = tiles;
  }
  plan->fft_size = best_n;
  plan->tile_out_h = best_n - kernel_h + 1;
  plan->tile_out_w = best_n - kernel_w + 1;
  plan->tiles = (int)best_tiles;
  // tensor cores whenever the passes lay their spectra out for them (same rule as the passes)
  plan->contraction = (best_n >= 16 && (long long)in_planes * out_planes >= 256) ? 0 : 1;
  const long long planes = (long long)in_planes * out_planes;
  plan->dw_mode = world > 1 && planes % world == 0 ? FBFFT_DP_FREQUENCY_REDUCE_SCATTER : FBFFT_DP_FREQUENCY_ALLREDUCE;
  plan->workspace_bytes = fbfft_b200_conv_workspace_bytes(best_n, (int)shard, in_planes, out_planes);
  return kSuccess;
}

int fbfft_b200_conv_tiled_update_output(int fft_size, const float* in, const int* in_size, const int* in_stride,
                                        const float* weight, const int* w_size, const int* w_stride, float* out,
                                        const int* out_size, const int* out_stride, int pad_h, int pad_w,
                                        void* workspace, size_t workspace_bytes, int flags, void* stream) {
  if (null_any(in_size, in_stride, w_size, w_stride, out_size, out_stride)) return fail(kUnsupportedDimension, "null argument");
  std::vector<Tile> tiles;
  int rc = tiles_of(fft_size, w_size[2], w_size[3], pad_h, pad_w, 0, in, in_size, in_stride, out, out_size, out_stride, &tiles);
  if (rc) return rc;
  int f = flags & FBFFT_CONV_REUSE_WEIGHT_SPECTRUM;
  for (const Tile& t : tiles) {
    rc = fbfft_b200_conv_update_output(fft_size, t.in.data, t.in.size, t.in.stride, t.in.padL, t.in.padU, weight, w_size,
                                       w_stride, t.out.data, t.out.size, t.out.stride, t.out.padL, t.out.padU, workspace,
                                       workspace_bytes, f, stream);
    if (rc) return rc;
    f = FBFFT_CONV_REUSE_WEIGHT_SPECTRUM;  // the weight spectrum is the same for every tile
  }
  return kSuccess;
}

int fbfft_b200_conv_tiled_update_grad_input(int fft_size, float* grad_in, const int* in_size, const int* in_stride,
                                            const float* weight, const int* w_size, const int* w_stride,
                                            const float* grad_out, const int* out_size, const int* out_stride, int pad_h,
                                            int pad_w, void* workspace, size_t workspace_bytes, int flags, void* stream) {
  if (null_any(in_size, in_stride, w_size, w_stride, out_size, out_stride)) return fail(kUnsupportedDimension, "null argument");
  std::vector<Tile> tiles;
  int rc = tiles_of(fft_size, w_size[2], w_size[3], pad_h, pad_w, 1, grad_in, in_size, in_stride, grad_out, out_size,
                    out_stride, &tiles);
  if (rc) return rc;
  int f = flags & FBFFT_CONV_REUSE_WEIGHT_SPECTRUM;
  for (const Tile& t : tiles) {
    rc = fbfft_b200_conv_update_grad_input(fft_size, t.in.data, t.in.size, t.in.stride, t.in.padL, t.in.padU, weight,
                                           w_size, w_stride, t.out.data, t.out.size, t.out.stride, t.out.padL, t.out.padU,
                                           workspace, workspace_bytes, f, stream);
    if (rc) return rc;
    f = FBFFT_CONV_REUSE_WEIGHT_SPECTRUM;
  }
  return kSuccess;
}

int fbfft_b200_conv_tiled_acc_grad_parameters(int fft_size, const float* in, const int* in_size, const int* in_stride,
                                              float* grad_weight, const int* w_size, const int* w_stride,
                                              const float* grad_out, const int* out_size, const int* out_stride,
                                              int pad_h, int pad_w, float scale, void* workspace, size_t workspace_bytes,
                                              int flags, void* stream) {
  if (null_any(in_size, in_stride, w_size, w_stride, out_size, out_stride)) return fail(kUnsupportedDimension, "null argument");
  std::vector<Tile> tiles;
  int rc = tiles_of(fft_size, w_size[2], w_size[3], pad_h, pad_w, 0, in, in_size, in_stride, grad_out, out_size,
                    out_stride, &tiles);
  if (rc) return rc;
  if (tiles.empty()) return fail(kUnsupportedDimension, "conv_tiled_acc_grad_parameters: empty output");
  // the contractions of all tiles add up in the result region; one inverse transform at the end
  int f = FBFFT_CONV_STOP_AFTER_CONTRACTION;
  for (const Tile& t : tiles) {
    rc = fbfft_b200_conv_acc_grad_parameters(fft_size, t.in.data, t.in.size, t.in.stride, t.in.padL, t.in.padU,
                                             grad_weight, w_size, w_stride, t.out.data, t.out.size, t.out.stride,
                                             t.out.padL, t.out.padU, scale, workspace, workspace_bytes, f, stream);
    if (rc) return rc;
    f = FBFFT_CONV_STOP_AFTER_CONTRACTION | FBFFT_CONV_ACCUMULATE_RESULT;
  }
  if (flags & FBFFT_CONV_STOP_AFTER_CONTRACTION) return kSuccess;
  const Tile& t = tiles[0];
  return fbfft_b200_conv_acc_grad_parameters(fft_size, t.in.data, t.in.size, t.in.stride, t.in.padL, t.in.padU,
                                             grad_weight, w_size, w_stride, t.out.data, t.out.size, t.out.stride,
                                             t.out.padL, t.out.padU, scale, workspace, workspace_bytes,
                                             FBFFT_CONV_START_FROM_SPECTRUM, stream);
}

}  // extern "C"
