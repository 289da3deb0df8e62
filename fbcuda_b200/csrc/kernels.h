// Internal entry points behind the C ABI (one per kernel family).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

#include "../../include/fbfft_b200.h"
#include "common.cuh"

namespace fbfft_b200 {

// N in {8, 16, 32}: [B][N/2+1][N] layout (fft2d_small.cu)
int fft2d_small_forward(int n, const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s);
int fft2d_small_inverse(int n, const CplxView& in, const RealView& out, int B, int padL, int padU, cudaStream_t s);

// the same transforms with fp16 / bf16 storage of either tensor (FBFFT_STORAGE_*), contiguous tensors (fft2d_small16.cu)
int fft2d_small_storage(int n, bool inverse, int src_type, int dst_type, const void* src, void* dst, int B, int h, int w,
                        int padL, int padU, cudaStream_t s);

// N in {64, 128, 256}: transposed [B][N/2+1 (kx)][N (ky)] layout (fft2d_large.cu)
int fft2d_large_forward(int n, const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s);
int fft2d_large_inverse(int n, const CplxView& in, const RealView& out, int B, int padL, int padU, cudaStream_t s);
// contiguous fast path for N in {64, 128} (fft2d_coop.cu)
bool fft2d_coop_supported(int n, const CplxView& c);
int fft2d_coop_forward(int n, const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s);
int fft2d_coop_inverse(int n, const CplxView& in, const RealView& out, int B, int padL, int padU, cudaStream_t s);
int read_device_error_coop();
int clear_device_error_coop();
// N = 256 forward on a contiguous spectrum: two register passes, no intermediate buffer (fft2d_256.cu)
bool fft2d_256_supported(const RealView& in, const CplxView& out, int B);
int fft2d_256_forward(const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s);
// N = 256 inverse into contiguous, uncropped 256 x 256 images, which double as the intermediate buffer (fft2d_256.cu)
bool fft2d_256_inverse_supported(const CplxView& in, const RealView& out, int B, int padL, int padU);
int fft2d_256_inverse(const CplxView& in, const RealView& out, int B, cudaStream_t s);
// forward transform by direct evaluation for images with a support of at most 8 x 8, N in {16, 32, 64, 128} (fft2d_pruned.cu)
bool fft2d_pruned_supported(int n, const RealView& real, const CplxView& cplx, int padL, int padU);
int fft2d_pruned_forward(int n, const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s);
// the reference's two-call protocol for N >= 64 (fft_lines.cu)
int fft2d_large_rows_forward(int n, const RealView& in, const CplxView& buffer, int B, int padL, int padU,
                             cudaStream_t s);
// block-per-image column pass for contiguous tensors, N = 64 / 128 (fft2d_cols.cu)
bool fft2d_cols_fast_supported(int n, const CplxView& buffer, const CplxView& dst, int B);
int fft2d_cols_fast(int n, const CplxView& buffer, const CplxView& dst, int B, cudaStream_t s);
bool fft2d_cols_inv_fast_supported(int n, const CplxView& buffer, const RealView& out, int B, int padL, int padU);
int fft2d_cols_inv_fast(int n, const CplxView& buffer, const RealView& out, int B, int padL, int padU, cudaStream_t s);
bool fft2d_rows_inv_fast_supported(int n, const CplxView& src, const CplxView& buffer, int B);
int fft2d_rows_inv_fast(int n, const CplxView& src, const CplxView& buffer, int B, cudaStream_t s);
int read_device_error_cols();
int clear_device_error_cols();
int fft2d_large_cols_forward(int n, const CplxView& buffer, const CplxView& dst, int B, cudaStream_t s);
int fft2d_large_rows_inverse(int n, const CplxView& src, const CplxView& buffer, int B, cudaStream_t s);
int fft2d_large_cols_inverse(int n, const CplxView& buffer, const RealView& out, int B, int padL, int padU,
                             cudaStream_t s);

// in-place transform of `lines` contiguous-or-strided lines per batch of a [B][lines][N] complex tensor
int fft_lines_inplace(int n, const CplxView& t, int B, int lines, bool inverse, cudaStream_t s);

// 1-D (fft_lines.cu)
// register-resident fast path for contiguous tensors, N <= 64 (fft1d_fast.cu)
bool fft1d_fast_supported(int n, const float* real, long long rs0, int rs1, const float* cplx, long long cs0, int cs1,
                          int cs2, int padL);
int fft1d_fast_group(int n);
int fft1d_fast(int n, bool inverse, const float* src, float* dst, long long tasks, cudaStream_t s);
// forward transform of rows of w floats inside a zero canvas (padded images of the two-call protocol, strided or
// left-padded 1-D signals): see fft1d_fast.cu
bool fft1d_fast_ragged_supported(int n, const float* p, long long sb, long long sy, int h, int w, int padL, int padU,
                                 int rpi, const float* cplx);
int fft1d_fast_ragged(int n, const float* p, long long sb, long long sy, int h, int w, int padL, int padU, int rpi,
                      float* dst, long long tasks, cudaStream_t s);
int fft1d_fast_ragged_inverse(int n, const float* src, float* p, long long sb, long long sy, int h, int w, int padL,
                              int padU, int rpi, long long tasks, cudaStream_t s);
// N = 8 on contiguous full images, one thread per image (fft2d_n8.cu): whole groups of 32 images
bool fft2d_n8_supported(const RealView& real, const CplxView& cplx, int B, int padL, int padU);
int fft2d_n8(bool inverse, const float* src, float* dst, long long tasks, cudaStream_t s);
int read_device_error_n8();
int clear_device_error_n8();
int read_device_error_fft1d();
int clear_device_error_fft1d();
int read_device_error_256();
int clear_device_error_256();
int fft1d_forward(int n, const float* real, int rs0, int rs1, float* cplx, int cs0, int cs1, int cs2, int B, int padL,
                  cudaStream_t s);
int fft1d_inverse(int n, const float* cplx, int cs0, int cs1, int cs2, float* real, int rs0, int rs1, int B, int padL,
                  cudaStream_t s);

// per-bin complex contraction (cgemm_bins.cu)
int transpose_mm(int dim, bool conjA, bool conjB, bool accumulate, const float* a, const int* a_size,
                 const int* a_stride, const float* b, const int* b_size, const int* b_stride, float* c,
                 const int* c_size, const int* c_stride, float inv_norm, cudaStream_t s);

// the same contraction on complex views [d0][d1][X] with strides in complex elements
int cgemm_bins(bool conjA, bool conjB, bool accumulate, const float* a, long long as0, long long as1, const float* b,
               long long bs0, long long bs1, float* c, long long cs0, long long cs1, int I, int J, int K, int X,
               float inv_norm, cudaStream_t s);

// tensor-core (tcgen05, 3xTF32) version of the contraction (cgemm_tc.cu):
// D[m][n][x] (+)= inv_norm * sum_k opA(A[m][k][x]) opB(B[n][k][x]), strides in complex elements
bool cgemm_tc_supported(const float* a, long long a_rs, long long a_ks, const float* b, long long b_rs, long long b_ks,
                        const float* d, long long d_ms, long long d_ns, int M, int N, int K, int X);
int cgemm_tc(const float* a, long long a_rs, long long a_ks, bool conjA, const float* b, long long b_rs, long long b_ks,
             bool conjB, float* d, long long d_ms, long long d_ns, int M, int N, int K, int X, float inv_norm,
             bool accumulate, cudaStream_t s, long long a_bs = 16, long long b_bs = 16, long long d_bs = 16, int a_qb = 16,
             int b_qb = 16, int d_qb = 16);
// persistent TMA-fed version (cgemm_tma.cu); returns -1 when a tensor map cannot be encoded
bool cgemm_tma_supported(const float* a, long long a_rs, long long a_ks, long long a_bs, const float* b, long long b_rs,
                         long long b_ks, long long b_bs, const float* d, long long d_ms, long long d_ns, long long d_bs,
                         int d_qb, int M, int N, int K, int X);
int cgemm_tma(const float* a, long long a_rs, long long a_ks, bool conjA, const float* b, long long b_rs, long long b_ks,
              bool conjB, float* d, long long d_ms, long long d_ns, int M, int N, int K, int X, float inv_norm,
              bool accumulate, cudaStream_t s, long long a_bs, long long b_bs, long long d_bs, int a_qb, int b_qb, int d_qb);
// fp32 tensor map (zero fill outside the tensor; swizzle 0, 32 or 128 bytes) into a 128-byte, 64-byte aligned buffer
// (cgemm_tma.cu)
bool encode_tensor_map_f32(void* map, const float* base, int rank, const unsigned long long* dims,
                           const unsigned long long* strides_bytes, const unsigned* box, int swizzle_bytes = 0);
int read_device_error_tma();
int clear_device_error_tma();
// FP32 CUDA-core version for n <= 8 columns or k <= 8 terms, operands in 4-bin blocks, overwriting result (cgemm_small.cu)
bool cgemm_small_supported(const float* a, const float* b, const float* d, long long d_ms, long long d_ns, long long d_bs,
                           int d_qb, int a_qb, int b_qb, int M, int N, int K, int X, bool accumulate);
int cgemm_small(const float* a, long long a_rs, long long a_ks, bool conjA, const float* b, long long b_rs, long long b_ks,
                bool conjB, float* d, long long d_ms, long long d_ns, int M, int N, int K, int X, float inv_norm,
                cudaStream_t s, long long a_bs, long long b_bs, long long d_bs, int d_qb);
int read_device_error_small();
int clear_device_error_small();
// 0: tensor cores when the operands qualify, 1: FP32 CUDA cores only, 2: tensor cores, gather kernel only
void set_contraction_mode(int mode);
int contraction_mode();
// SMs the persistent contraction leaves free (for collectives that run beside it)
void set_contraction_reserved_sms(int n);
int contraction_reserved_sms();
int read_device_error_tc();
int clear_device_error_tc();

// tiled convolution passes (conv_iterated.cu)
int iterated_convolution(int fft_size, const fbfft_tiled_tensor4* ins, const fbfft_tiled_tensor4* outs, float* weight,
                         const int* weight_size, const int* weight_stride, int pass, float scale, int batch_size,
                         size_t num_tiles, cudaStream_t s);

// value of the device-side error word (0 = none; set when a bounded wait inside a kernel ran out)
int read_device_error();
int clear_device_error();
// tensor-pipe rate of tcgen05.mma.kind::tf32 (M = 128, N = n_cols, K = 8) from shared-memory operands (tf32_peak.cu)
int measure_tf32_peak(int n_cols, double* tflops);
int read_device_error_peak();
int clear_device_error_peak();
// one block waits `max_tries` attempts on a barrier that nothing completes, gives up, records
// code 901 and returns; *elapsed_ns (host pointer) receives the time the wait took (fft2d_small.cu)
int selftest_bounded_wait(int max_tries, unsigned long long* elapsed_ns);

}  // namespace fbfft_b200
