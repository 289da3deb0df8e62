// Fourier-domain convolution passes (updateOutput / updateGradInput /
// accGradParameters) for every supported transform size, as transform ->
// per-bin contraction -> inverse transform over a caller-owned workspace.
//
// The reference ships this chain only as building blocks (fbfft2D, transposeMM,
// fbifft2D; the host code that chained them lived in its caller) plus a fused
// prototype for N <= 32 (fbfft/FFTIteratedConvolution.cuh).  The math of each
// pass is that prototype's (:161-186, :316-341, :482-523) with the contraction
// roles of MM-inl.cuh:194-196:
//   updateOutput       outF[b][o] = sum_c inF[b][c] * conj(wF[o][c])
//   updateGradInput    inF [b][c] = sum_o outF[b][o] * wF[o][c]
//   accGradParameters  wF  [o][c] = sum_b conj(outF[b][o]) * inF[b][c]
// every result scaled by 1/N^2 (accGradParameters also by `scale`) and cropped at
// the tensor's (padU, padL) offset inside the N x N canvas; weights sit at (0, 0).
#include "../../include/fbfft_b200.h"
#include "common.cuh"
#include "dp_comm.h"
#include "kernels.h"

namespace fbfft_b200 {

namespace {

struct Tensor4 {
  float* p;
  int size[4];
  int stride[4];
};

long long bins_of(int n) { return (long long)(n / 2 + 1) * n; }

struct Regions {
  long long in_off, out_off, w_off, res_off, total;  // in floats
};

Regions regions(int n, long long B, long long C, long long O) {
  const long long per = bins_of(n) * 2;
  Regions r;
  r.in_off = 0;
  r.out_off = r.in_off + B * C * per;
  r.w_off = r.out_off + B * O * per;
  r.res_off = r.w_off + O * C * per;
  long long m = B * C;
  if (B * O > m) m = B * O;
  if (O * C > m) m = O * C;
  r.total = r.res_off + m * per;
  return r;
}

bool fail(const char* msg) {
  set_last_error(msg);
  return false;
}

// [d0][d1][h][w] -> batch of d0*d1 images; the two leading dimensions must collapse
bool as_images(const Tensor4& t, RealView* v, int* count) {
  if (t.size[0] > 1 && t.stride[0] != t.size[1] * t.stride[1]) return fail("leading dimensions must be collapsible");
  v->p = t.p;
  v->sb = t.stride[1];
  v->sy = t.stride[2];
  v->sx = t.stride[3];
  v->h = t.size[2];
  v->w = t.size[3];
  *count = t.size[0] * t.size[1];
  return true;
}

// planes > 0: bin-blocked layout over that many planes, in blocks of blk_bins bins (see CplxView)
CplxView spectrum_view(float* p, int n, long long planes, int blk_bins) {
  CplxView v;
  v.p = p;
  v.sb = bins_of(n) * 2;
  v.sr = 2 * n;
  v.sc = 2;
  v.sz = 1;
  v.blk_planes = planes;
  v.blk_bins = blk_bins;
  return v;
}

int forward(int n, const Tensor4& t, int padL, int padU, float* spec, bool blocked, cudaStream_t s) {
  RealView v;
  int count;
  if (!as_images(t, &v, &count)) return kUnsupportedDimension;
  // forward spectra are contraction operands: 4-bin blocks
  const CplxView sv = spectrum_view(spec, n, blocked ? count : 0, 4);
  // weights (3x3, 5x5, 7x7): direct evaluation, bound by the spectrum's bytes instead of butterflies
  if (n >= 64 && v.h * 4 <= n && v.w * 4 <= n && fft2d_pruned_supported(n, v, sv, padL, padU))
    return fft2d_pruned_forward(n, v, sv, count, padL, padU, s);
  if (n <= 32) return fft2d_small_forward(n, v, sv, count, padL, padU, s);
  return fft2d_large_forward(n, v, sv, count, padL, padU, s);
}

int inverse(int n, float* spec, const Tensor4& t, int padL, int padU, bool blocked, cudaStream_t s) {
  RealView v;
  int count;
  if (!as_images(t, &v, &count)) return kUnsupportedDimension;
  // the contraction's result: one stored row per block (one bulk copy per row in the inverse transform)
  const CplxView sv = spectrum_view(spec, n, blocked ? count : 0, n);
  if (n <= 32) return fft2d_small_inverse(n, sv, v, count, padL, padU, s);
  return fft2d_large_inverse(n, sv, v, count, padL, padU, s);
}

// The workspace spectra use the bin-blocked layout whenever the tensor-core contraction will
// run (its operand rows are then contiguous runs instead of isolated 32-byte sectors).  The
// decision depends on the transform size, the plane counts and the process-wide contraction mode
// only -- never on the batch -- so spectra reused across passes agree, and so do the result regions
// of ranks that hold batch shards of different sizes (an empty shard included) and sum them
// between STOP_AFTER_CONTRACTION and START_FROM_SPECTRUM.
bool use_blocked(int n, long long C, long long O) {
  return n >= 16 && contraction_mode() != 1 && C * O >= 16 * 16;
}

// D[m][n] (+)= inv_norm * sum_k opA(A[m][k]) opB(B[n][k]) per bin, where element (m, k) of A is
// plane a_pm*m + a_pk*k of a spectrum region of a_planes planes (same for B and D)
int contract(int n, bool blocked, const float* a, long long a_pm, long long a_pk, long long a_planes, bool conjA,
             const float* b, long long b_pn, long long b_pk, long long b_planes, bool conjB, float* d, long long d_pm,
             long long d_pn, long long d_planes, int M, int N, int K, float inv_norm, cudaStream_t s,
             bool accumulate = false, bool d_plane_major = false) {
  const long long X = bins_of(n);
  if (blocked) {
    // result: row blocks of n bins with the planes adjacent inside a block, or (d_plane_major) plane by plane
    const long long dm = d_plane_major ? d_pm * X : d_pm * n, dn = d_plane_major ? d_pn * X : d_pn * n;
    const long long dbs = d_plane_major ? 16 : d_planes * n;
    const int dqb = d_plane_major ? 16 : n;
    // operands in 4-bin blocks (plane stride 4 complex), result in blocks of one stored row (n bins).
    // The MMA tile is 128 rows of m by 16 / 32 / 64 columns of n: the two operands swap roles
    // (complex products commute) when that pads less, e.g. 64 planes against a batch of 128.
    auto padded = [](long long rows, long long cols) {
      const long long p48 = (cols + 47) / 48 * 48, p64 = (cols + 63) / 64 * 64;
      const long long pc = cols <= 16 ? 16 : (cols <= 32 ? 32 : (p48 < p64 ? p48 : p64));
      return ((rows + 127) / 128 * 128) * pc;
    };
    // a shard of at most 8 images leaves a contraction with 8 columns or 8 terms: no tile of the
    // tensor-core kernel fits that, the FP32 kernels stream the large operand (or the result) once
    if (contraction_mode() == 0 &&
        cgemm_small_supported(a, b, d, dm, dn, dbs, dqb, 4, 4, M, N, K, (int)X, accumulate)) {
      const int rc = cgemm_small(a, a_pm * 4, a_pk * 4, conjA, b, b_pn * 4, b_pk * 4, conjB, d, dm, dn, M, N, K,
                                 (int)X, inv_norm, s, a_planes * 4, b_planes * 4, dbs, dqb);
      if (rc != -1) return rc;  // -1: a tensor map could not be encoded, the general kernel takes over
    }
    if (padded(N, M) < padded(M, N)) {
      return cgemm_tc(b, b_pn * 4, b_pk * 4, conjB, a, a_pm * 4, a_pk * 4, conjA, d, dn, dm, N, M, K, (int)X,
                      inv_norm, accumulate, s, b_planes * 4, a_planes * 4, dbs, 4, 4, dqb);
    }
    return cgemm_tc(a, a_pm * 4, a_pk * 4, conjA, b, b_pn * 4, b_pk * 4, conjB, d, dm, dn, M, N, K, (int)X,
                    inv_norm, accumulate, s, a_planes * 4, b_planes * 4, dbs, 4, 4, dqb);
  }
  // natural layout: D[m][n] = sum_k opA(A[m][k]) opB(B[n][k]) = cgemm_bins with A' = A (rows m),
  // B' = B^T: C[i=m][j=n] = sum_k opA(A[i][k]) * opB'(B'[k][j]), B'[k][j] = B[j][k] -> "conj-transposed" flag
  // carries the transposition, so express through strides instead: use the generic entry with
  // as0 = a_pm*X, as1 = a_pk*X; B given as [k][j] with bs0 = b_pk*X, bs1 = b_pn*X
  if (conjA && !conjB) {
    // cgemm_bins conjugates only together with a transposition: op(A)[i][k] = conj(A[k][i]) with
    // strides (as0 for k, as1 for i)
    return cgemm_bins(true, false, accumulate, a, a_pk * X, a_pm * X, b, b_pk * X, b_pn * X, d, d_pm * X, d_pn * X, M, N, K,
                      (int)X, inv_norm, s);
  }
  if (!conjA && conjB) {
    return cgemm_bins(false, true, accumulate, a, a_pm * X, a_pk * X, b, b_pn * X, b_pk * X, d, d_pm * X, d_pn * X, M, N, K,
                      (int)X, inv_norm, s);
  }
  return cgemm_bins(false, false, accumulate, a, a_pm * X, a_pk * X, b, b_pk * X, b_pn * X, d, d_pm * X, d_pn * X, M, N, K,
                    (int)X, inv_norm, s);
}

Tensor4 make_tensor(const float* p, const int* size, const int* stride) {
  Tensor4 t;
  t.p = const_cast<float*>(p);
  for (int d = 0; d < 4; ++d) {
    t.size[d] = size[d];
    t.stride[d] = stride[d];
  }
  return t;
}

// the transforms reject negative offsets into the canvas; so do the passes
int check_pads(int in_padL, int in_padU, int out_padL, int out_padU) {
  if (in_padL < 0 || in_padU < 0 || out_padL < 0 || out_padU < 0) {
    set_last_error("convolution: negative padding");
    return kUnsupportedDimension;
  }
  return kSuccess;
}

int check_common(int n, const Tensor4& in, const Tensor4& w, const Tensor4& out, void* ws, size_t ws_bytes) {
  if (!(n == 8 || n == 16 || n == 32 || n == 64 || n == 128)) {
    set_last_error("convolution: transform size must be 8, 16, 32, 64 or 128");
    return kUnsupportedSize;
  }
  if (in.size[0] != out.size[0] || in.size[1] != w.size[1] || out.size[1] != w.size[0]) {
    set_last_error("convolution: batch / plane counts of input, weight and output do not agree");
    return kUnsupportedDimension;
  }
  const Regions r = regions(n, in.size[0], in.size[1], out.size[1]);
  if (!ws || ws_bytes < (size_t)r.total * sizeof(float)) {
    set_last_error("convolution: workspace too small (see fbfft_b200_conv_workspace_bytes)");
    return kUnsupportedDimension;
  }
  if (reinterpret_cast<uintptr_t>(ws) & 15u) {
    set_last_error("convolution: workspace must be 16-byte aligned");
    return kUnsupportedDimension;
  }
  return kSuccess;
}

}  // namespace
}  // namespace fbfft_b200

using namespace fbfft_b200;

extern "C" {

size_t fbfft_b200_conv_workspace_bytes(int fft_size, int batch, int in_planes, int out_planes) {
  return (size_t)regions(fft_size, batch, in_planes, out_planes).total * sizeof(float);
}

int fbfft_b200_conv_workspace_region(int fft_size, int batch, int in_planes, int out_planes, int which,
                                     size_t* offset_bytes, size_t* size_bytes) {
  const Regions r = regions(fft_size, batch, in_planes, out_planes);
  const long long per = bins_of(fft_size) * 2;
  long long off, sz;
  switch (which) {
    case FBFFT_CONV_REGION_INPUT:
      off = r.in_off, sz = (long long)batch * in_planes * per;
      break;
    case FBFFT_CONV_REGION_OUTPUT:
      off = r.out_off, sz = (long long)batch * out_planes * per;
      break;
    case FBFFT_CONV_REGION_WEIGHT:
      off = r.w_off, sz = (long long)out_planes * in_planes * per;
      break;
    case FBFFT_CONV_REGION_RESULT:
      off = r.res_off, sz = r.total - r.res_off;
      break;
    default:
      set_last_error("conv_workspace_region: unknown region");
      return kUnsupportedDimension;
  }
  if (offset_bytes) *offset_bytes = (size_t)off * sizeof(float);
  if (size_bytes) *size_bytes = (size_t)sz * sizeof(float);
  return kSuccess;
}

int fbfft_b200_conv_update_output(int fft_size, const float* in, const int* in_size, const int* in_stride, int in_padL,
                                  int in_padU, const float* weight, const int* w_size, const int* w_stride, float* out,
                                  const int* out_size, const int* out_stride, int out_padL, int out_padU,
                                  void* workspace, size_t workspace_bytes, int flags, void* stream) {
  if (!in || !weight || !out || !in_size || !w_size || !out_size || !in_stride || !w_stride || !out_stride) {
    set_last_error("null argument");
    return kUnsupportedDimension;
  }
  if (int prc = check_pads(in_padL, in_padU, out_padL, out_padU)) return prc;
  const Tensor4 ti = make_tensor(in, in_size, in_stride), tw = make_tensor(weight, w_size, w_stride),
                to = make_tensor(out, out_size, out_stride);
  int rc = check_common(fft_size, ti, tw, to, workspace, workspace_bytes);
  if (rc) return rc;
  const int n = fft_size, B = ti.size[0], C = ti.size[1], O = to.size[1];
  if (B == 0) return kSuccess;
  const Regions r = regions(n, B, C, O);
  float* ws = static_cast<float*>(workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool blk = use_blocked(n, C, O) && (reinterpret_cast<uintptr_t>(ws) & 31u) == 0;
  if (!(flags & FBFFT_CONV_START_FROM_SPECTRUM)) {
    if (!(flags & FBFFT_CONV_REUSE_INPUT_SPECTRUM) && (rc = forward(n, ti, in_padL, in_padU, ws + r.in_off, blk, s)))
      return rc;
    if (!(flags & FBFFT_CONV_REUSE_WEIGHT_SPECTRUM) && (rc = forward(n, tw, 0, 0, ws + r.w_off, blk, s))) return rc;
    if (flags & FBFFT_CONV_STOP_AFTER_TRANSFORMS) return kSuccess;
    // res[b][o] = sum_c conj(w[o][c]) in[b][c] / N^2      (m = o, n = b, k = c)
    rc = contract(n, blk, ws + r.w_off, C, 1, (long long)O * C, true, ws + r.in_off, C, 1, (long long)B * C, false,
                  ws + r.res_off, 1, O, (long long)B * O, O, B, C, 1.0f / ((float)n * (float)n), s);
    if (rc) return rc;
  }
  if (flags & FBFFT_CONV_STOP_AFTER_CONTRACTION) return kSuccess;
  return inverse(n, ws + r.res_off, to, out_padL, out_padU, blk, s);
}

int fbfft_b200_conv_update_grad_input(int fft_size, float* grad_in, const int* in_size, const int* in_stride,
                                      int in_padL, int in_padU, const float* weight, const int* w_size,
                                      const int* w_stride, const float* grad_out, const int* out_size,
                                      const int* out_stride, int out_padL, int out_padU, void* workspace,
                                      size_t workspace_bytes, int flags, void* stream) {
  if (!grad_in || !weight || !grad_out || !in_size || !w_size || !out_size || !in_stride || !w_stride || !out_stride) {
    set_last_error("null argument");
    return kUnsupportedDimension;
  }
  if (int prc = check_pads(in_padL, in_padU, out_padL, out_padU)) return prc;
  const Tensor4 ti = make_tensor(grad_in, in_size, in_stride), tw = make_tensor(weight, w_size, w_stride),
                to = make_tensor(grad_out, out_size, out_stride);
  int rc = check_common(fft_size, ti, tw, to, workspace, workspace_bytes);
  if (rc) return rc;
  const int n = fft_size, B = ti.size[0], C = ti.size[1], O = to.size[1];
  if (B == 0) return kSuccess;
  const Regions r = regions(n, B, C, O);
  float* ws = static_cast<float*>(workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool blk = use_blocked(n, C, O) && (reinterpret_cast<uintptr_t>(ws) & 31u) == 0;
  if (!(flags & FBFFT_CONV_START_FROM_SPECTRUM)) {
    if (!(flags & FBFFT_CONV_REUSE_OUTPUT_SPECTRUM) &&
        (rc = forward(n, to, out_padL, out_padU, ws + r.out_off, blk, s)))
      return rc;
    if (!(flags & FBFFT_CONV_REUSE_WEIGHT_SPECTRUM) && (rc = forward(n, tw, 0, 0, ws + r.w_off, blk, s))) return rc;
    if (flags & FBFFT_CONV_STOP_AFTER_TRANSFORMS) return kSuccess;
    // res[b][c] = sum_o w[o][c] out[b][o] / N^2           (m = c, n = b, k = o)
    rc = contract(n, blk, ws + r.w_off, 1, C, (long long)O * C, false, ws + r.out_off, O, 1, (long long)B * O, false,
                  ws + r.res_off, 1, C, (long long)B * C, C, B, O, 1.0f / ((float)n * (float)n), s);
    if (rc) return rc;
  }
  if (flags & FBFFT_CONV_STOP_AFTER_CONTRACTION) return kSuccess;
  return inverse(n, ws + r.res_off, ti, in_padL, in_padU, blk, s);
}

int fbfft_b200_conv_acc_grad_parameters(int fft_size, const float* in, const int* in_size, const int* in_stride,
                                        int in_padL, int in_padU, float* grad_weight, const int* w_size,
                                        const int* w_stride, const float* grad_out, const int* out_size,
                                        const int* out_stride, int out_padL, int out_padU, float scale,
                                        void* workspace, size_t workspace_bytes, int flags, void* stream) {
  // an empty batch shard may come with null data pointers
  if (!grad_weight || !in_size || !w_size || !out_size || !in_stride || !w_stride || !out_stride ||
      (in_size[0] > 0 && (!in || !grad_out))) {
    set_last_error("null argument");
    return kUnsupportedDimension;
  }
  if (int prc = check_pads(in_padL, in_padU, out_padL, out_padU)) return prc;
  const Tensor4 ti = make_tensor(in, in_size, in_stride), tw = make_tensor(grad_weight, w_size, w_stride),
                to = make_tensor(grad_out, out_size, out_stride);
  int rc = check_common(fft_size, ti, tw, to, workspace, workspace_bytes);
  if (rc) return rc;
  const int n = fft_size, B = ti.size[0], C = ti.size[1], O = to.size[1];
  const Regions r = regions(n, B, C, O);
  float* ws = static_cast<float*>(workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long X = bins_of(n);
  const bool blk = use_blocked(n, C, O) && (reinterpret_cast<uintptr_t>(ws) & 31u) == 0;
  if (!(flags & FBFFT_CONV_START_FROM_SPECTRUM)) {
    if (B == 0) {
      if (!(flags & FBFFT_CONV_ACCUMULATE_RESULT) && cudaMemsetAsync(ws + r.res_off, 0, (size_t)O * C * X * 2 * sizeof(float), s) != cudaSuccess) return kCudaError;
    } else {
      if (!(flags & FBFFT_CONV_REUSE_INPUT_SPECTRUM) && (rc = forward(n, ti, in_padL, in_padU, ws + r.in_off, blk, s)))
        return rc;
      if (!(flags & FBFFT_CONV_REUSE_OUTPUT_SPECTRUM) &&
          (rc = forward(n, to, out_padL, out_padU, ws + r.out_off, blk, s)))
        return rc;
      if (flags & FBFFT_CONV_STOP_AFTER_TRANSFORMS) return kSuccess;
      // res[o][c] = scale / N^2 * sum_b conj(out[b][o]) in[b][c]      (m = o, n = c, k = b)
      rc = contract(n, blk, ws + r.out_off, 1, O, (long long)B * O, true, ws + r.in_off, 1, C, (long long)B * C, false,
                    ws + r.res_off, C, 1, (long long)O * C, O, C, B, scale / ((float)n * (float)n), s,
                    (flags & FBFFT_CONV_ACCUMULATE_RESULT) != 0, (flags & FBFFT_CONV_RESULT_PLANE_MAJOR) != 0);
      if (rc) return rc;
    }
  }
  if (flags & FBFFT_CONV_STOP_AFTER_CONTRACTION) return kSuccess;
  return inverse(n, ws + r.res_off, tw, 0, 0, blk && !(flags & FBFFT_CONV_RESULT_PLANE_MAJOR), s);
}

// accGradParameters over batch shards on several GPUs: every rank contracts its own shard, the
// weight gradient is summed over the communicator, every rank ends with the full gradient.
int fbfft_b200_conv_acc_grad_parameters_dp(fbfft_b200_comm* comm, int mode, int fft_size, const float* in,
                                           const int* in_size, const int* in_stride, int in_padL, int in_padU,
                                           float* grad_weight, const int* w_size, const int* w_stride,
                                           const float* grad_out, const int* out_size, const int* out_stride,
                                           int out_padL, int out_padU, float scale, void* workspace,
                                           size_t workspace_bytes, int flags, void* stream) {
  if (!comm) {
    set_last_error("conv_acc_grad_parameters_dp: null communicator");
    return kUnsupportedDimension;
  }
  if (mode < FBFFT_DP_FREQUENCY_ALLREDUCE || mode > FBFFT_DP_SPATIAL_ALLREDUCE) {
    set_last_error("conv_acc_grad_parameters_dp: unknown reduction mode");
    return kUnsupportedDimension;
  }
  if (flags & FBFFT_CONV_ACCUMULATE_RESULT) {
    set_last_error("conv_acc_grad_parameters_dp: ACCUMULATE_RESULT cannot be combined with the cross-GPU sum");
    return kUnsupportedDimension;
  }
  Comm* c = reinterpret_cast<Comm*>(comm);
  const int world = comm_world(c), rank = comm_rank(c);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // this rank's contraction (argument checks included); an empty shard zeroes the result region
  int rc = kSuccess;
  if (!(flags & FBFFT_CONV_START_FROM_SPECTRUM)) {
    rc = fbfft_b200_conv_acc_grad_parameters(fft_size, in, in_size, in_stride, in_padL, in_padU, grad_weight, w_size,
                                             w_stride, grad_out, out_size, out_stride, out_padL, out_padU, scale,
                                             workspace, workspace_bytes, flags | FBFFT_CONV_STOP_AFTER_CONTRACTION, stream);
    if (rc) return rc;
    if (flags & (FBFFT_CONV_STOP_AFTER_CONTRACTION | FBFFT_CONV_STOP_AFTER_TRANSFORMS)) return kSuccess;
  } else {
    if (!in_size || !w_size || !out_size || !in_stride || !w_stride || !out_stride || !grad_weight) {
      set_last_error("null argument");
      return kUnsupportedDimension;
    }
    const Tensor4 ti = make_tensor(in, in_size, in_stride), tw = make_tensor(grad_weight, w_size, w_stride),
                  to = make_tensor(grad_out, out_size, out_stride);
    if ((rc = check_common(fft_size, ti, tw, to, workspace, workspace_bytes))) return rc;
  }
  const int n = fft_size, B = in_size[0], C = in_size[1], O = out_size[1];
  const long long planes = (long long)O * C, X = bins_of(n);
  const Tensor4 tw = make_tensor(grad_weight, w_size, w_stride);
  const bool gw_dense = tw.stride[3] == 1 && tw.stride[2] == tw.size[3] && tw.stride[1] == tw.size[2] * tw.size[3] &&
                        tw.stride[0] == tw.size[1] * tw.stride[1];
  const size_t gw_count = (size_t)planes * tw.size[2] * tw.size[3];
  const Regions r = regions(n, B, C, O);
  float* res = static_cast<float*>(workspace) + r.res_off;
  // the result region: row blocks, or plane by plane when the caller asked for that (or the layer has no blocks)
  const bool blk = use_blocked(n, C, O) && (reinterpret_cast<uintptr_t>(workspace) & 31u) == 0 &&
                   !(flags & FBFFT_CONV_RESULT_PLANE_MAJOR);
  if (mode == FBFFT_DP_SPATIAL_ALLREDUCE) {
    if (!gw_dense) {
      set_last_error("conv_acc_grad_parameters_dp: the spatial all-reduce needs a contiguous grad_weight");
      return kUnsupportedDimension;
    }
    if ((rc = inverse(n, res, tw, 0, 0, blk, s))) return rc;
    return world > 1 ? comm_all_reduce(c, grad_weight, gw_count, s) : kSuccess;
  }
  if (world == 1) return inverse(n, res, tw, 0, 0, blk, s);
  if (mode == FBFFT_DP_FREQUENCY_REDUCE_SCATTER && planes % world == 0 && gw_dense) {
    // Every rank receives the sum of 1/world of the planes, inverse-transforms and crops only those,
    // and the spatial gradients are gathered.  In the row-blocked layout a plane's bins are spread
    // over N/2+1 row blocks of [planes][N] complex values: one reduce-scatter per row block, as a group.
    const long long mine = planes / world, lo = mine * rank;
    if (blk) {
      rc = comm_reduce_scatter_rows(c, res, n / 2 + 1, (size_t)planes * n * 2, (size_t)mine * n * 2, s);
    } else {
      rc = comm_reduce_scatter_rows(c, res, 1, 0, (size_t)mine * X * 2, s);
    }
    if (rc) return rc;
    RealView v;
    int count;
    if (!as_images(tw, &v, &count)) return kUnsupportedDimension;
    v.p += lo * v.sb;
    CplxView sv = spectrum_view(res + lo * (blk ? (long long)n * 2 : X * 2), n, blk ? planes : 0, n);
    rc = n <= 32 ? fft2d_small_inverse(n, sv, v, (int)mine, 0, 0, s) : fft2d_large_inverse(n, sv, v, (int)mine, 0, 0, s);
    if (rc) return rc;
    return comm_all_gather(c, grad_weight, (size_t)mine * tw.size[2] * tw.size[3], s);
  }
  // the sum of the whole frequency-domain gradient on every rank, then the full inverse everywhere
  if ((rc = comm_all_reduce(c, res, (size_t)planes * X * 2, s))) return rc;
  return inverse(n, res, tw, 0, 0, blk, s);
}

}  // extern "C"
