// C ABI: argument validation and dispatch to the kernels.  Mirrors the host
// dispatch of the reference (fbfft/FBFFT-inl.cuh:19-150, fbfft/FBFFT2D-inl.cuh:450-669,
// fbfft/FBIFFT2D-inl.cuh:529-742, MM-inl.cuh:515-814,
// fbfft/FFTIteratedConvolution.cuh:624-755) but reports violated preconditions as
// error codes instead of aborting.
#include "../../include/fbfft_b200.h"

#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace fbfft_b200 {

namespace {
thread_local char g_last_error[256] = "";
}

void set_last_error(const char* msg) {
  std::strncpy(g_last_error, msg, sizeof(g_last_error) - 1);
  g_last_error[sizeof(g_last_error) - 1] = 0;
}

int sm_count() {
  static std::mutex mu;
  static int cached[64];
  static bool have[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
    have[dev] = true;
  }
  return cached[dev];
}

namespace {

int fail(int code, const char* msg) {
  set_last_error(msg);
  return code;
}

bool is_pow2(int n) { return n > 0 && (n & (n - 1)) == 0; }
bool small_size(int n) { return n == 8 || n == 16 || n == 32; }
bool large_size(int n) { return n == 64 || n == 128 || n == 256; }

RealView real_view(const float* p, const int* size, const int* stride) {
  RealView v;
  v.p = const_cast<float*>(p);
  v.sb = stride[0];
  v.sy = stride[1];
  v.sx = stride[2];
  v.h = size[1];
  v.w = size[2];
  return v;
}

// float tensor [B][rows][cols][2]
CplxView cplx_view_f4(const float* p, const int* stride) {
  CplxView v;
  v.p = const_cast<float*>(p);
  v.sb = stride[0];
  v.sr = stride[1];
  v.sc = stride[2];
  v.sz = stride[3];
  return v;
}

// Complex tensor [B][rows][cols], strides in complex elements
CplxView cplx_view_c3(const float* p, const int* stride) {
  CplxView v;
  v.p = const_cast<float*>(p);
  v.sb = 2LL * stride[0];
  v.sr = 2 * stride[1];
  v.sc = 2 * stride[2];
  v.sz = 1;
  return v;
}

int check_ptrs(const void* a, const void* b) {
  if (!a || !b) return fail(kUnsupportedDimension, "null tensor pointer");
  return kSuccess;
}

}  // namespace
}  // namespace fbfft_b200

using namespace fbfft_b200;

extern "C" {

int fbfft_b200_version(void) { return 100; }

const char* fbfft_b200_last_error(void) { return g_last_error; }

int fbfft_b200_device_status(void) {
  const int a = read_device_error(), b = read_device_error_coop(), c = read_device_error_tc(), d = read_device_error_tma(),
            e = read_device_error_fft1d(), f = read_device_error_256(), g = read_device_error_cols(),
            h = read_device_error_peak(), i = read_device_error_small(), j = read_device_error_n8();
  return a != 0 ? a : (b != 0 ? b : (c != 0 ? c : (d != 0 ? d : (e != 0 ? e : (f != 0 ? f : (g != 0 ? g : (h != 0 ? h : (i != 0 ? i : j))))))));
}

int fbfft_b200_clear_device_status(void) {
  const int r = clear_device_error() | clear_device_error_coop() | clear_device_error_tc() | clear_device_error_tma() |
                clear_device_error_fft1d() | clear_device_error_256() | clear_device_error_cols() |
                clear_device_error_peak() | clear_device_error_small() | clear_device_error_n8();
  if (cudaDeviceSynchronize() != cudaSuccess || r != 0) return fail(kCudaError, "clear_device_status: cannot reset the status words");
  return kSuccess;
}

int fbfft_b200_selftest_bounded_wait(int max_tries, unsigned long long* elapsed_ns) {
  if (max_tries < 1 || max_tries > (1 << 20)) return fail(kUnsupportedDimension, "selftest_bounded_wait: max_tries must be in 1..2^20");
  if (selftest_bounded_wait(max_tries, elapsed_ns) != kSuccess) return fail(kCudaError, "selftest_bounded_wait: launch or read-back failed");
  return kSuccess;
}

int fbfft_b200_measure_tf32_peak(int n_cols, double* tflops) {
  if (!tflops || !(n_cols == 64 || n_cols == 128 || n_cols == 256))
    return fail(kUnsupportedDimension, "measure_tf32_peak: n_cols must be 64, 128 or 256 and the output non-null");
  if (measure_tf32_peak(n_cols, tflops) != kSuccess) return fail(kCudaError, "measure_tf32_peak: launch or timing failed");
  return kSuccess;
}

int fbfft_b200_set_contraction_reserved_sms(int sms) {
  if (sms < 0 || sms > 128) return fail(kUnsupportedDimension, "set_contraction_reserved_sms: 0..128");
  set_contraction_reserved_sms(sms);
  return kSuccess;
}

int fbfft_b200_set_contraction_mode(int mode) {
  if (mode < 0 || mode > 2)
    return fail(kUnsupportedDimension, "set_contraction_mode: 0 (tensor cores), 1 (FP32 cores) or 2 (tensor cores, gather kernel)");
  set_contraction_mode(mode);
  return kSuccess;
}

int fbfft_b200_fft2d_r2c(int n, const float* real, const int* real_size, const int* real_stride, float* cplx,
                         const int* cplx_size, const int* cplx_stride, int padL, int padU, void* stream) {
  if (!real_size || !real_stride || !cplx_size || !cplx_stride) return fail(kUnsupportedDimension, "null size/stride");
  const int B = real_size[0];
  if (B == 0) return kSuccess;
  if (check_ptrs(real, cplx)) return kUnsupportedDimension;
  if (!small_size(n) && !large_size(n)) return fail(kUnsupportedSize, "fft2d_r2c: N must be 8, 16, 32, 64, 128 or 256");
  if (cplx_size[0] != B || cplx_size[1] != n / 2 + 1 || cplx_size[2] != n || cplx_size[3] != 2)
    return fail(kUnsupportedDimension, "fft2d_r2c: complex tensor must be [B][N/2+1][N][2]");
  if (padL < 0 || padU < 0) return fail(kUnsupportedDimension, "fft2d_r2c: negative padding");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  RealView in = real_view(real, real_size, real_stride);
  CplxView out = cplx_view_f4(cplx, cplx_stride);
  if (small_size(n)) return fft2d_small_forward(n, in, out, B, padL, padU, s);
  return fft2d_large_forward(n, in, out, B, padL, padU, s);
}

int fbfft_b200_fft2d_c2r(int n, const float* cplx, const int* cplx_size, const int* cplx_stride, float* real,
                         const int* real_size, const int* real_stride, int padL, int padU, void* stream) {
  if (!real_size || !real_stride || !cplx_size || !cplx_stride) return fail(kUnsupportedDimension, "null size/stride");
  const int B = real_size[0];
  if (B == 0) return kSuccess;
  if (check_ptrs(real, cplx)) return kUnsupportedDimension;
  if (!small_size(n) && !large_size(n)) return fail(kUnsupportedSize, "fft2d_c2r: N must be 8, 16, 32, 64, 128 or 256");
  if (cplx_size[0] != B || cplx_size[1] != n / 2 + 1 || cplx_size[2] != n || cplx_size[3] != 2)
    return fail(kUnsupportedDimension, "fft2d_c2r: complex tensor must be [B][N/2+1][N][2]");
  if (padL < 0 || padU < 0) return fail(kUnsupportedDimension, "fft2d_c2r: negative padding");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CplxView in = cplx_view_f4(cplx, cplx_stride);
  RealView out = real_view(real, real_size, real_stride);
  if (small_size(n)) return fft2d_small_inverse(n, in, out, B, padL, padU, s);
  return fft2d_large_inverse(n, in, out, B, padL, padU, s);
}

namespace {
int check_storage(const char* who, int n, int real_type, int cplx_type, const void* real, const int* real_size,
                  const int* real_stride, const void* cplx, const int* cplx_size, const int* cplx_stride, int padL,
                  int padU) {
  static thread_local char msg[160];
  auto bad = [&](int code, const char* what) {
    std::snprintf(msg, sizeof(msg), "%s: %s", who, what);
    return fail(code, msg);
  };
  if (!real_size || !real_stride || !cplx_size || !cplx_stride) return bad(kUnsupportedDimension, "null size/stride");
  if (!small_size(n)) return bad(kUnsupportedSize, "16-bit storage covers N = 8, 16 and 32");
  if (real_type < FBFFT_STORAGE_F32 || real_type > FBFFT_STORAGE_BF16 || cplx_type < FBFFT_STORAGE_F32 ||
      cplx_type > FBFFT_STORAGE_BF16)
    return bad(kUnsupportedDimension, "storage types are FBFFT_STORAGE_F32, _F16 or _BF16");
  const int B = real_size[0], h = real_size[1], w = real_size[2];
  if (B == 0) return kSuccess;
  if (!real || !cplx) return bad(kUnsupportedDimension, "null tensor pointer");
  if (cplx_size[0] != B || cplx_size[1] != n / 2 + 1 || cplx_size[2] != n || cplx_size[3] != 2)
    return bad(kUnsupportedDimension, "complex tensor must be [B][N/2+1][N][2]");
  if (h < 1 || w < 1 || h > n || w > n || padL < 0 || padU < 0)
    return bad(kUnsupportedDimension, "the image must fit the transform and the padding be non-negative");
  if (real_stride[2] != 1 || real_stride[1] != w || (B > 1 && real_stride[0] != h * w) || cplx_stride[3] != 1 ||
      cplx_stride[2] != 2 || cplx_stride[1] != 2 * n || (B > 1 && cplx_stride[0] != (n / 2 + 1) * n * 2))
    return bad(kUnsupportedDimension, "tensors must be contiguous");
  if ((reinterpret_cast<uintptr_t>(real) & 3u) || (reinterpret_cast<uintptr_t>(cplx) & 15u))
    return bad(kUnsupportedDimension, "the real tensor must be 4-byte aligned, the complex tensor 16-byte aligned");
  return kSuccess;
}
}  // namespace

int fbfft_b200_fft2d_r2c_storage(int n, int real_type, int cplx_type, const void* real, const int* real_size,
                                 const int* real_stride, void* cplx, const int* cplx_size, const int* cplx_stride, int padL,
                                 int padU, void* stream) {
  const int rc = check_storage("fft2d_r2c_storage", n, real_type, cplx_type, real, real_size, real_stride, cplx, cplx_size,
                               cplx_stride, padL, padU);
  if (rc != kSuccess || real_size[0] == 0) return rc;
  return fft2d_small_storage(n, false, real_type, cplx_type, real, cplx, real_size[0], real_size[1], real_size[2], padL, padU,
                             static_cast<cudaStream_t>(stream));
}

int fbfft_b200_fft2d_c2r_storage(int n, int cplx_type, int real_type, const void* cplx, const int* cplx_size,
                                 const int* cplx_stride, void* real, const int* real_size, const int* real_stride, int padL,
                                 int padU, void* stream) {
  const int rc = check_storage("fft2d_c2r_storage", n, real_type, cplx_type, real, real_size, real_stride, cplx, cplx_size,
                               cplx_stride, padL, padU);
  if (rc != kSuccess || real_size[0] == 0) return rc;
  return fft2d_small_storage(n, true, cplx_type, real_type, cplx, real, real_size[0], real_size[1], real_size[2], padL, padU,
                             static_cast<cudaStream_t>(stream));
}

int fbfft_b200_fbfft2d(const float* real, const int* real_size, const int* real_stride, float* cplx,
                       const int* cplx_size, const int* cplx_stride, int padL, int padU, void* stream) {
  if (!real_size || !real_stride || !cplx_size || !cplx_stride) return fail(kUnsupportedDimension, "null size/stride");
  // Size class by the shape of the complex tensor, as the reference does
  // (fbfft/FBFFT2D-inl.cuh:479,511,543 test dimension 2; :599-616 dimension 1).
  const int d1 = cplx_size[1], d2 = cplx_size[2];
  if (d1 > 256 || d2 > 256) return fail(kUnsupportedSize, "fbfft2d: transform size above 256");
  if (small_size(d2) && d1 == d2 / 2 + 1) {
    return fbfft_b200_fft2d_r2c(d2, real, real_size, real_stride, cplx, cplx_size, cplx_stride, padL, padU, stream);
  }
  if (large_size(d1) && d2 == d1 / 2 + 1) {
    const int B = real_size[0];
    if (B == 0) return kSuccess;
    if (check_ptrs(real, cplx)) return kUnsupportedDimension;
    if (cplx_size[0] != B || cplx_size[3] != 2) return fail(kUnsupportedDimension, "fbfft2d: buffer must be [B][N][N/2+1][2]");
    if (padL < 0 || padU < 0) return fail(kUnsupportedDimension, "fbfft2d: negative padding");
    return fft2d_large_rows_forward(d1, real_view(real, real_size, real_stride), cplx_view_f4(cplx, cplx_stride), B,
                                    padL, padU, static_cast<cudaStream_t>(stream));
  }
  return fail(kUnsupportedSize, "fbfft2d: complex tensor is neither [B][N/2+1][N][2] (N<=32) nor [B][N][N/2+1][2] (N>=64)");
}

int fbfft_b200_fbfft2d_c2c(const float* src, const int* src_size, const int* src_stride, float* dst,
                           const int* dst_size, const int* dst_stride, void* stream) {
  if (!src_size || !src_stride || !dst_size || !dst_stride) return fail(kUnsupportedDimension, "null size/stride");
  const int B = src_size[0], n = src_size[1];
  if (B == 0) return kSuccess;
  if (check_ptrs(src, dst)) return kUnsupportedDimension;
  if (!large_size(n)) return fail(kUnsupportedSize, "fbfft2d_c2c: N must be 64, 128 or 256");
  if (src_size[2] != n / 2 + 1) return fail(kUnsupportedDimension, "fbfft2d_c2c: src must be [B][N][N/2+1]");
  if (dst_size[0] != B || dst_size[1] != n / 2 + 1 || dst_size[2] != n)
    return fail(kUnsupportedDimension, "fbfft2d_c2c: dst must be [B][N/2+1][N]");
  if (src == dst) return fail(kUnsupportedDimension, "fbfft2d_c2c: src and dst must differ");
  return fft2d_large_cols_forward(n, cplx_view_c3(src, src_stride), cplx_view_c3(dst, dst_stride), B,
                                  static_cast<cudaStream_t>(stream));
}

int fbfft_b200_fbifft2d_c2c(const float* src, const int* src_size, const int* src_stride, float* dst,
                            const int* dst_size, const int* dst_stride, void* stream) {
  if (!src_size || !src_stride || !dst_size || !dst_stride) return fail(kUnsupportedDimension, "null size/stride");
  const int B = src_size[0], n = src_size[2];
  if (B == 0) return kSuccess;
  if (check_ptrs(src, dst)) return kUnsupportedDimension;
  if (!large_size(n)) return fail(kUnsupportedSize, "fbifft2d_c2c: N must be 64, 128 or 256");
  if (src_size[1] != n / 2 + 1 || src_size[3] != 2) return fail(kUnsupportedDimension, "fbifft2d_c2c: src must be [B][N/2+1][N][2]");
  if (dst_size[0] != B || dst_size[1] != n || dst_size[2] != n || dst_size[3] != 2)
    return fail(kUnsupportedDimension, "fbifft2d_c2c: dst must be [B][N][N][2]");
  if (src == dst) return fail(kUnsupportedDimension, "fbifft2d_c2c: src and dst must differ");
  return fft2d_large_rows_inverse(n, cplx_view_f4(src, src_stride), cplx_view_f4(dst, dst_stride), B,
                                  static_cast<cudaStream_t>(stream));
}

int fbfft_b200_fbifft2d(const float* src, const int* src_size, const int* src_stride, float* real,
                        const int* real_size, const int* real_stride, int padL, int padU, void* stream) {
  if (!src_size || !src_stride || !real_size || !real_stride) return fail(kUnsupportedDimension, "null size/stride");
  const int d1 = src_size[1], d2 = src_size[2];
  if (d1 > 256 || d2 > 256) return fail(kUnsupportedSize, "fbifft2d: transform size above 256");
  const int B = real_size[0];
  if (small_size(d2) && d1 == d2 / 2 + 1) {
    if (B == 0) return kSuccess;
    if (check_ptrs(src, real)) return kUnsupportedDimension;
    if (src_size[0] != B) return fail(kUnsupportedDimension, "fbifft2d: batch sizes differ");
    if (padL < 0 || padU < 0) return fail(kUnsupportedDimension, "fbifft2d: negative padding");
    return fft2d_small_inverse(d2, cplx_view_c3(src, src_stride), real_view(real, real_size, real_stride), B, padL,
                               padU, static_cast<cudaStream_t>(stream));
  }
  if (large_size(d1) && d2 == d1) {
    if (B == 0) return kSuccess;
    if (check_ptrs(src, real)) return kUnsupportedDimension;
    if (src_size[0] != B) return fail(kUnsupportedDimension, "fbifft2d: batch sizes differ");
    if (padL < 0 || padU < 0) return fail(kUnsupportedDimension, "fbifft2d: negative padding");
    return fft2d_large_cols_inverse(d1, cplx_view_c3(src, src_stride), real_view(real, real_size, real_stride), B,
                                    padL, padU, static_cast<cudaStream_t>(stream));
  }
  return fail(kUnsupportedSize, "fbifft2d: src is neither [B][N/2+1][N] (N<=32) nor [B][N][N] (N>=64)");
}

int fbfft_b200_fbfft1d(const float* real, const int* real_size, const int* real_stride, float* cplx,
                       const int* cplx_size, const int* cplx_stride, int padL, void* stream) {
  if (!real_size || !real_stride || !cplx_size || !cplx_stride) return fail(kUnsupportedDimension, "null size/stride");
  const int B = real_size[0], n = real_size[1];
  if (B == 0) return kSuccess;
  if (check_ptrs(real, cplx)) return kUnsupportedDimension;
  if (!is_pow2(n) || n < 8 || n > 256) return fail(kUnsupportedSize, "fbfft1d: N must be a power of two in [8, 256]");
  if (cplx_size[0] != B || cplx_size[1] != n / 2 + 1 || cplx_size[2] != 2)
    return fail(kUnsupportedDimension, "fbfft1d: complex tensor must be [B][N/2+1][2]");
  if (padL < 0) return fail(kUnsupportedDimension, "fbfft1d: negative padding");
  return fft1d_forward(n, real, real_stride[0], real_stride[1], cplx, cplx_stride[0], cplx_stride[1], cplx_stride[2],
                       B, padL, static_cast<cudaStream_t>(stream));
}

int fbfft_b200_fbifft1d(float* real, const int* real_size, const int* real_stride, const float* cplx,
                        const int* cplx_size, const int* cplx_stride, int padL, void* stream) {
  if (!real_size || !real_stride || !cplx_size || !cplx_stride) return fail(kUnsupportedDimension, "null size/stride");
  const int B = real_size[0], n = real_size[1];
  if (B == 0) return kSuccess;
  if (check_ptrs(real, cplx)) return kUnsupportedDimension;
  if (!is_pow2(n) || n < 8 || n > 256) return fail(kUnsupportedSize, "fbifft1d: N must be a power of two in [8, 256]");
  if (cplx_size[0] != B || cplx_size[1] != n / 2 + 1 || cplx_size[2] != 2)
    return fail(kUnsupportedDimension, "fbifft1d: complex tensor must be [B][N/2+1][2]");
  if (padL < 0) return fail(kUnsupportedDimension, "fbifft1d: negative padding");
  return fft1d_inverse(n, cplx, cplx_stride[0], cplx_stride[1], cplx_stride[2], real, real_stride[0], real_stride[1],
                       B, padL, static_cast<cudaStream_t>(stream));
}

int fbfft_b200_transpose_mm(int dim, int conj_transpose_a, int conj_transpose_b, int accumulate, const float* a,
                            const int* a_size, const int* a_stride, const float* b, const int* b_size,
                            const int* b_stride, float* c, const int* c_size, const int* c_stride, float inv_norm,
                            void* stream) {
  if (!a_size || !a_stride || !b_size || !b_stride || !c_size || !c_stride)
    return fail(kUnsupportedDimension, "null size/stride");
  if (dim < 4 || dim > 6) return fail(kUnsupportedDimension, "transpose_mm: dim must be 4, 5 or 6");
  if (!a || !b || !c) return fail(kUnsupportedDimension, "null tensor pointer");
  return transpose_mm(dim, conj_transpose_a != 0, conj_transpose_b != 0, accumulate != 0, a, a_size, a_stride, b,
                      b_size, b_stride, c, c_size, c_stride, inv_norm, static_cast<cudaStream_t>(stream));
}

int fbfft_b200_iterated_convolution(int fft_size, const fbfft_tiled_tensor4* ins, const fbfft_tiled_tensor4* outs,
                                    float* weight, const int* weight_size, const int* weight_stride, int pass,
                                    float scale, int batch_size, size_t num_tiles, void* stream) {
  if (!small_size(fft_size)) {
    set_last_error("iterated_convolution: FFT size must be 8, 16 or 32");
    return 0;
  }
  if (pass < 0 || pass > 2 || !ins || !outs || !weight || !weight_size || !weight_stride) {
    set_last_error("iterated_convolution: unknown pass or null argument");
    return 0;
  }
  return iterated_convolution(fft_size, ins, outs, weight, weight_size, weight_stride, pass, scale, batch_size,
                              num_tiles, static_cast<cudaStream_t>(stream));
}

int fbfft_b200_plan_tiles(int fft_size, int kernel_h, int kernel_w, int pad_h, int pad_w, int style, float* input,
                          const int* in_size, const int* in_stride, float* output, const int* out_size,
                          const int* out_stride, fbfft_tiled_tensor4* ins_host, fbfft_tiled_tensor4* outs_host,
                          size_t capacity) {
  if (!in_size || !in_stride || !out_size || !out_stride || (style != 0 && style != 1)) {
    set_last_error("plan_tiles: null argument or unknown style");
    return -1;
  }
  const int n = fft_size, H = in_size[2], W = in_size[3], OH = out_size[2], OW = out_size[3];
  if (n < 2 || kernel_h < 1 || kernel_w < 1 || kernel_h > n || kernel_w > n || pad_h < 0 || pad_w < 0 ||
      OH != H + 2 * pad_h - kernel_h + 1 || OW != W + 2 * pad_w - kernel_w + 1 || OH < 1 || OW < 1 ||
      in_size[0] != out_size[0]) {
    set_last_error("plan_tiles: sizes do not describe a stride-1 convolution that fits the transform");
    return -1;
  }
  // a window [lo, lo + len) of an axis of extent `extent`: the part inside, and the pad that puts
  // the window's first element at canvas position 0
  struct Span { int begin, count, pad; };
  auto clip = [](int lo, int len, int extent) {
    Span s;
    s.begin = lo < 0 ? 0 : lo;
    const int end = lo + len < extent ? lo + len : extent;
    s.count = end > s.begin ? end - s.begin : 0;
    s.pad = lo < 0 ? -lo : 0;
    return s;
  };
  auto emit = [&](fbfft_tiled_tensor4* dst, float* base, const int* size, const int* stride, Span y, Span x, int padU,
                  int padL) {
    dst->padL = padL;
    dst->padU = padU;
    dst->data = base ? base + (long long)y.begin * stride[2] + (long long)x.begin * stride[3] : nullptr;
    for (int d = 0; d < 4; ++d) dst->stride[d] = stride[d];
    dst->size[0] = size[0], dst->size[1] = size[1], dst->size[2] = y.count, dst->size[3] = x.count;
  };
  const int th = n - kernel_h + 1, tw = n - kernel_w + 1;  // outputs (style 0) / gradInput rows (style 1) per tile
  const int ext_y = style == 0 ? OH : H, ext_x = style == 0 ? OW : W;
  int count = 0;
  for (int y0 = 0; y0 < ext_y; y0 += th) {
    for (int x0 = 0; x0 < ext_x; x0 += tw) {
      const int hh = ext_y - y0 < th ? ext_y - y0 : th, ww = ext_x - x0 < tw ? ext_x - x0 : tw;
      if ((size_t)count < capacity && ins_host && outs_host) {
        if (style == 0) {
          // outputs [y0, y0 + hh) need input rows [y0 - pad, y0 - pad + hh + k - 1)
          const Span iy = clip(y0 - pad_h, hh + kernel_h - 1, H), ix = clip(x0 - pad_w, ww + kernel_w - 1, W);
          emit(ins_host + count, input, in_size, in_stride, iy, ix, iy.pad, ix.pad);
          emit(outs_host + count, output, out_size, out_stride, Span{y0, hh, 0}, Span{x0, ww, 0}, 0, 0);
        } else {
          // gradInput rows [y0, y0 + hh) need gradOutput rows [y0 + pad - (k - 1), y0 + pad + hh) and
          // sit at canvas rows k - 1 ... of the full convolution
          const Span gy = clip(y0 + pad_h - (kernel_h - 1), hh + kernel_h - 1, OH),
                     gx = clip(x0 + pad_w - (kernel_w - 1), ww + kernel_w - 1, OW);
          emit(ins_host + count, input, in_size, in_stride, Span{y0, hh, 0}, Span{x0, ww, 0}, kernel_h - 1, kernel_w - 1);
          emit(outs_host + count, output, out_size, out_stride, gy, gx, gy.pad, gx.pad);
        }
      }
      ++count;
    }
  }
  return count;
}

}  // extern "C"
