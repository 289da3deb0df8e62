/* C ABI of the B200 fbfft library (libfbfft_b200.so).
 *
 * Every function is a drop-in for one host entry point of the reference's fbfft
 * path; the comment above each declaration names the reference interface it
 * replaces (paths relative to the reference tree).  Tensors cross the boundary
 * as the three fields of the reference's DeviceTensor<T, Dim> POD
 * (DeviceTensor.cuh:237-245): a device pointer, `Dim` sizes and `Dim` strides,
 * both in elements of T.  All pointers are device pointers unless stated; work
 * is enqueued on `stream` (a cudaStream_t) and nothing synchronises.  The caller
 * owns every buffer; the library allocates no device memory.
 *
 * Return values are those of FBFFTParameters::ErrorCode
 * (fbfft/FBFFTParameters.h:9-14).  Conditions the reference checks with
 * assert()/CHECK_*() and aborts on are reported as FBFFT_UNSUPPORTED_DIMENSION
 * instead; fbfft_b200_last_error() returns a description.
 */
#ifndef FBFFT_B200_H_
#define FBFFT_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  FBFFT_SUCCESS = 0,
  FBFFT_UNSUPPORTED_SIZE = 1,
  FBFFT_UNSUPPORTED_DIMENSION = 2,
  FBFFT_CUDA_ERROR = 3
};

/* Layout of the reference's TiledDeviceTensor<float, 4>
 * (fbfft/FFTIteratedConvolution.cuh:70-88): two pads, then the DeviceTensor POD. */
typedef struct fbfft_tiled_tensor4 {
  int padL;
  int padU;
  float* data;
  int stride[4];
  int size[4];
} fbfft_tiled_tensor4;

/* Library version (major * 100 + minor). */
int fbfft_b200_version(void);

/* Text describing the last non-success return on the calling thread. */
const char* fbfft_b200_last_error(void);

/* Synchronising health check (no counterpart in the reference): returns 0 when no
 * kernel of this library has recorded a device-side error on the current device,
 * else the code it recorded (a bounded wait on an asynchronous copy that ran out:
 * 101 / 102 forward / inverse transform for N <= 32, 103 inverse transform for N = 64, 128, 201 / 202 and 211-216 tensor-core contraction,
 * 901 the self-test below, 902 the tensor-peak measurement), or -1 if the status cannot be read. */
int fbfft_b200_device_status(void);

/* Resets the device-side error code of the current device to 0 (synchronises).  The code is
 * sticky until cleared; no counterpart in the reference. */
int fbfft_b200_clear_device_status(void);

/* Test hook (no counterpart in the reference): launches one block whose single waiting thread
 * waits, with the transforms' own bounded wait, on a barrier that nothing ever completes, with a
 * limit of `max_tries` (1 .. 2^20, the limit the kernels use) suspended attempts.  The wait runs
 * out, the kernel returns by itself, fbfft_b200_device_status() then reports 901 until cleared,
 * and *elapsed_ns (a host pointer, may be NULL) receives the time the wait took on the device, so
 * that a caller can convert the kernels' limit into seconds.  Synchronises. */
int fbfft_b200_selftest_bounded_wait(int max_tries, unsigned long long* elapsed_ns);

/* Measurement hook (no counterpart in the reference): the rate, in TFLOP/s, at which this GPU's
 * tensor cores run the MMA the contraction issues (tcgen05.mma kind::tf32, M = 128, N = n_cols in
 * {64, 128, 256}, K = 8, operands in shared memory) when nothing else competes -- the tensor-peak
 * denominator of the convolution roofline.  Creates two events, launches a few short kernels on
 * the default stream and synchronises; *tflops is a host pointer. */
int fbfft_b200_measure_tf32_peak(int n_cols, double* tflops);

/* How fbfft_b200_transpose_mm and the convolution passes contract (process-wide; no
 * counterpart in the reference, whose transposeMM is FP32 CUDA-core code only):
 * 0 (default) tensor cores -- tcgen05 MMAs on a 3xTF32 split of the fp32 operands,
 * accumulating in fp32 -- whenever the operands qualify (bin count a multiple of 4,
 * 16-byte aligned bases, even strides), FP32 CUDA cores otherwise; 1 FP32 CUDA cores
 * always; 2 tensor cores through the earlier gather kernel only (comparison point;
 * needs 32-byte aligned operands and strides that are multiples of 4). */
int fbfft_b200_set_contraction_mode(int mode);

/* Number of SMs the tensor-core contraction leaves free (process-wide, default 0; no counterpart in
 * the reference).  The contraction runs one persistent block per SM that fills the SM's shared
 * memory, so no other kernel starts on an SM it occupies; a data-parallel caller that wants the
 * weight-gradient collective (NCCL kernels on a second stream) to run BESIDE the contractions of the
 * other passes, not after them, reserves a few SMs for it. */
int fbfft_b200_set_contraction_reserved_sms(int sms);

/* fbfft1D<1>(DeviceTensor<float,2>& real, DeviceTensor<float,3>& complex, padL, s)
 * -- fbfft/FBFFT.cuh:11-16, fbfft/FBFFT-inl.cuh:19-87.
 * real [B][N], N = real_size[1] in {8..256}; complex [B][N/2+1][2].
 * complex[b][k] = sum_n p[n] exp(-2 pi i k n / N), p[n] = real[b][n - padL] for
 * padL <= n < N, else 0. */
int fbfft_b200_fbfft1d(const float* real, const int* real_size, const int* real_stride, float* cplx,
                       const int* cplx_size, const int* cplx_stride, int padL, void* stream);

/* fbifft1D<1>(real, complex, padL, s) -- fbfft/FBFFT.cuh:18-23,
 * fbfft/FBFFT-inl.cuh:89-150.  Unnormalised: real[b][x - padL] = N * p[x]. */
int fbfft_b200_fbifft1d(float* real, const int* real_size, const int* real_stride, const float* cplx,
                        const int* cplx_size, const int* cplx_stride, int padL, void* stream);

/* fbfft2D<1>(DeviceTensor<float,3>& real, DeviceTensor<float,4>& complexAsFloat,
 * padL, padU, s) -- fbfft/FBFFT.cuh:30-36, fbfft/FBFFT2D-inl.cuh:450-623.
 * real [B][h][w] is placed at (padU, padL) of an N x N canvas of zeros.
 *  - cplx_size = {B, N/2+1, N, 2}, N in {8,16,32}: the finished transform,
 *    cplx[b][ky][kx] = F[ky][kx].
 *  - cplx_size = {B, N, N/2+1, 2}, N in {64,128,256}: the first half of the
 *    reference's two-call protocol, row transforms only:
 *    cplx[b][y][kx] = sum_x P[y][x] exp(-2 pi i kx x / N). */
int fbfft_b200_fbfft2d(const float* real, const int* real_size, const int* real_stride, float* cplx,
                       const int* cplx_size, const int* cplx_stride, int padL, int padU, void* stream);

/* fbfft2D<1>(DeviceTensor<Complex,3>& src, DeviceTensor<Complex,3>& dst, s)
 * -- fbfft/FBFFT.cuh:38-43, fbfft/FBFFT2D-inl.cuh:627-669.  Second half for
 * N >= 64: src [B][N][N/2+1] -> dst [B][N/2+1][N],
 * dst[b][kx][ky] = sum_y src[b][y][kx] exp(-2 pi i ky y / N).  Sizes and strides
 * count complex elements; src and dst must not overlap. */
int fbfft_b200_fbfft2d_c2c(const float* src, const int* src_size, const int* src_stride, float* dst,
                           const int* dst_size, const int* dst_stride, void* stream);

/* fbifft2D<1>(DeviceTensor<float,4>& src, DeviceTensor<float,4>& dst, s)
 * -- fbfft/FBFFT.cuh:45-49, fbfft/FBIFFT2D-inl.cuh:529-563.  First half of the
 * inverse for N >= 64: src [B][N/2+1][N][2] -> dst [B][N][N][2]; images b and
 * b + ceil(B/2) are combined as X_b + i X_{b+ceil(B/2)}, the spectrum is extended
 * to all N values of kx by Hermitian symmetry and inverse transformed along ky;
 * only the first ceil(B/2) slices of dst are written. */
int fbfft_b200_fbifft2d_c2c(const float* src, const int* src_size, const int* src_stride, float* dst,
                            const int* dst_size, const int* dst_stride, void* stream);

/* fbifft2D<1>(DeviceTensor<Complex,3>& src, DeviceTensor<float,3>& real, padL,
 * padU, s) -- fbfft/FBFFT.cuh:50-56, fbfft/FBIFFT2D-inl.cuh:567-742.
 *  - src_size = {B, N/2+1, N}, N in {8,16,32}: full inverse of the [ky][kx]
 *    layout, real[b][y-padU][x-padL] = N*N * P[y][x] for in-bounds (y, x).
 *  - src_size = {B, N, N}, N in {64,128,256}: second half of the two-call
 *    inverse; src is the buffer written by fbfft_b200_fbifft2d_c2c.
 * Sizes and strides of src count complex elements. */
int fbfft_b200_fbifft2d(const float* src, const int* src_size, const int* src_stride, float* real,
                        const int* real_size, const int* real_stride, int padL, int padU, void* stream);

/* Single-call 2-D transforms for every N in {8,...,256}; no counterpart in the
 * reference for N >= 64, where it needs two calls and a caller-owned buffer
 * (fbfft/FBFFT2D-inl.cuh:597-617 then :627-669).  cplx is [B][N/2+1][N][2] in the
 * reference's final layout for the size class: [ky][kx] for N <= 32, transposed
 * [kx][ky] for N >= 64.  n is the transform size.
 * N = 256: an image and its spectrum do not fit one SM, so both directions run two passes
 * without a buffer of their own -- the forward transform works inside the spectrum tensor, the
 * inverse inside the real tensor, which must therefore be the full, contiguous, 16-byte aligned
 * [B][256][256] image with padL = padU = 0 (FBFFT_UNSUPPORTED_SIZE otherwise: crops and strides
 * go through the two-call protocol with its caller-owned [B][N][N][2] buffer). */
int fbfft_b200_fft2d_r2c(int n, const float* real, const int* real_size, const int* real_stride, float* cplx,
                         const int* cplx_size, const int* cplx_stride, int padL, int padU, void* stream);
int fbfft_b200_fft2d_c2r(int n, const float* cplx, const int* cplx_size, const int* cplx_stride, float* real,
                         const int* real_size, const int* real_stride, int padL, int padU, void* stream);

/* fbfft2D / fbifft2D for N in {8, 16, 32} with the images, the spectra, or both stored as fp16 or
 * bf16; the arithmetic stays fp32.  The reference leaves this open ("TODO: f16 implementation",
 * fbfft/FFT2D32.cuh:385 and :451); layouts, padding rule and normalisation are those of the fp32
 * transforms (fbfft/FFT2D32.cuh:361-470).  real_type / cplx_type are FBFFT_STORAGE_*; sizes and
 * strides count elements of the storage type; tensors must be contiguous, the real tensor 4-byte
 * and the complex tensor 16-byte aligned, the image no larger than the transform.
 * Accuracy: a 16-bit result carries the rounding of its storage type on top of the fp32 error --
 * against the float64 transform of the stored (already rounded) input the relative L2 error stays
 * below 2^-11 + 1e-5 with fp16 results and 2^-8 + 1e-5 with bf16 results (half a unit in the last
 * place of an 11- / 8-bit significand per element; about 1/sqrt(3) of that on average), and below
 * 1e-5, as for fbfft_b200_fft2d_r2c, with fp32 results.  fp16 holds magnitudes up to 65504: the
 * unnormalised spectrum of an N x N image of values in [-1, 1] is bounded by N*N <= 1024. */
enum { FBFFT_STORAGE_F32 = 0, FBFFT_STORAGE_F16 = 1, FBFFT_STORAGE_BF16 = 2 };
int fbfft_b200_fft2d_r2c_storage(int n, int real_type, int cplx_type, const void* real, const int* real_size,
                                 const int* real_stride, void* cplx, const int* cplx_size, const int* cplx_stride, int padL,
                                 int padU, void* stream);
int fbfft_b200_fft2d_c2r_storage(int n, int cplx_type, int real_type, const void* cplx, const int* cplx_size,
                                 const int* cplx_stride, void* real, const int* real_size, const int* real_stride, int padL,
                                 int padU, void* stream);

/* transposeMM<Dim, ConjugateTransposeA, ConjugateTransposeB, Accumulate>(A, B, C,
 * invNorm, s) -- MM.cuh:11-17, MM-inl.cuh:515-814.  A, B, C are float tensors of
 * `dim` dimensions whose last dimension is 2 (re, im) and whose dimensions
 * 2..dim-2 are the frequency bins:
 *   C[i][j][bin] (+)= invNorm * sum_k op(A)[i][k][bin] * op(B)[k][j][bin],
 * where a conjugate-transposed operand has its two leading indices swapped and
 * its value conjugated (MM-inl.cuh:121-131,150-163). */
int fbfft_b200_transpose_mm(int dim, int conj_transpose_a, int conj_transpose_b, int accumulate, const float* a,
                            const int* a_size, const int* a_stride, const float* b, const int* b_size,
                            const int* b_stride, float* c, const int* c_size, const int* c_stride, float inv_norm,
                            void* stream);

/* FFTIteratedConvolution<FFTSize>(ins, outs, weight, pass, scale, batchSize,
 * numTiles, s) -- fbfft/FFTIteratedConvolution.cuh:624-755.  ins / outs are
 * DEVICE arrays of numTiles descriptors (the reference dereferences them on the
 * device, :113-114).  pass: 0 updateOutput (writes outs), 1 updateGradInput
 * (writes ins), 2 accGradParameters (overwrites weight with scale * gradient).
 * Returns 1 (true) when the pass was launched, 0 (false) otherwise, as the
 * reference does.  fft_size in {8, 16, 32}. */
int fbfft_b200_iterated_convolution(int fft_size, const fbfft_tiled_tensor4* ins, const fbfft_tiled_tensor4* outs,
                                    float* weight, const int* weight_size, const int* weight_stride, int pass,
                                    float scale, int batch_size, size_t num_tiles, void* stream);

/* Tile lists for FFTIteratedConvolution when the image exceeds the transform: overlap-save
 * tiles of (fft_size - kernel + 1) outputs.  The reference's caller built these lists
 * (the descriptors and their pads: fbfft/FFTIteratedConvolution.cuh:70-95, 105-114); this
 * is that host-side step.  Host code only: nothing is launched or copied.
 *
 * input  [B][C][H][W], output [B][O][OH][OW] with OH = H + 2*pad_h - kernel_h + 1 (same for W);
 * both given as pointer, sizes and strides in elements (device pointers are only offset).
 * style 0 (updateOutput, accGradParameters): input tiles overlap by kernel - 1 and carry the
 *   image padding as (padU, padL); output tiles are disjoint.
 * style 1 (updateGradInput): input (gradInput) tiles are disjoint and are cropped at
 *   (kernel_h - 1, kernel_w - 1) of the canvas; output (gradOutput) tiles overlap.
 * ins_host / outs_host receive `capacity` descriptors at most (may be NULL to count only).
 * Returns the number of tiles, or -1 for bad arguments (kernel larger than the transform,
 * mismatching sizes).  Copy the descriptors to device memory before the convolution call. */
int fbfft_b200_plan_tiles(int fft_size, int kernel_h, int kernel_w, int pad_h, int pad_w, int style, float* input,
                          const int* in_size, const int* in_stride, float* output, const int* out_size,
                          const int* out_stride, fbfft_tiled_tensor4* ins_host, fbfft_tiled_tensor4* outs_host,
                          size_t capacity);

/* ---- Convolution passes over a caller-owned workspace ------------------------
 * The transform -> per-bin contraction -> inverse transform chain for one tile of
 * any transform size in {8, 16, 32, 64, 128}.  The reference ships the chain only
 * as its building blocks (fbfft2D, transposeMM, fbifft2D: MM-inl.cuh:188-196; the
 * code chaining them lived in its caller) and, for N <= 32, as the fused
 * FFTIteratedConvolution prototype whose math these follow
 * (fbfft/FFTIteratedConvolution.cuh:161-186,316-341,482-523).
 *
 * in / grad_in   [B][C][ih][iw] placed at (in_padU, in_padL) of the N x N canvas
 * out / grad_out [B][O][oh][ow] placed at (out_padU, out_padL)
 * weight         [O][C][kh][kw] placed at (0, 0)
 * The two leading dimensions of each tensor must be collapsible
 * (stride[0] == size[1] * stride[1]).
 *
 * The workspace holds four spectrum regions (input, output, weight, result); a
 * pass can skip a forward transform whose spectrum an earlier pass left in the
 * workspace (REUSE flags), and every pass can stop after the contraction
 * (STOP_AFTER_CONTRACTION) and resume from the result region (START_FROM_SPECTRUM),
 * so that a caller can sum the frequency-domain weight gradient across GPUs in
 * between (fbfft_b200_conv_acc_grad_parameters_dp does exactly that).  The layout of
 * the spectra inside the workspace depends on the transform size, the two plane
 * counts and the contraction mode, never on the batch: ranks holding batch shards of
 * different sizes (an empty one included) may add their result regions element by
 * element. */
enum {
  FBFFT_CONV_REUSE_INPUT_SPECTRUM = 1,
  FBFFT_CONV_REUSE_OUTPUT_SPECTRUM = 2,
  FBFFT_CONV_REUSE_WEIGHT_SPECTRUM = 4,
  FBFFT_CONV_STOP_AFTER_CONTRACTION = 8,
  FBFFT_CONV_START_FROM_SPECTRUM = 16,
  /* accGradParameters: add this call's contraction to the result region instead of overwriting it
   * (the weight gradient summed over the tiles of an image larger than the transform) */
  FBFFT_CONV_ACCUMULATE_RESULT = 32,
  /* run the forward transforms that are not marked REUSE, then return: a caller that holds the
   * weights fixed over several calls transforms them once this way */
  FBFFT_CONV_STOP_AFTER_TRANSFORMS = 64,
  /* accGradParameters (and its data-parallel form; no counterpart in the reference): the result region holds
   * the frequency-domain weight gradient plane by plane, [O*C][N/2+1][N] complex values, instead of in the
   * row blocks the contraction otherwise writes.  Both halves of a STOP_AFTER_CONTRACTION /
   * START_FROM_SPECTRUM pair, and every rank of a data-parallel sum, must agree on it.  Data-parallel callers
   * set it when every rank's batch shard is small (at most 8 images: the contraction then writes whole lines
   * in either layout): each rank's share of the planes is one contiguous piece, and the reduce-scatter of
   * FBFFT_DP_FREQUENCY_REDUCE_SCATTER is a single collective instead of one per stored row. */
  FBFFT_CONV_RESULT_PLANE_MAJOR = 128
};
enum {
  FBFFT_CONV_REGION_INPUT = 0,
  FBFFT_CONV_REGION_OUTPUT = 1,
  FBFFT_CONV_REGION_WEIGHT = 2,
  FBFFT_CONV_REGION_RESULT = 3
};

size_t fbfft_b200_conv_workspace_bytes(int fft_size, int batch, int in_planes, int out_planes);

/* Byte offset and size of one spectrum region inside the workspace.  Spectra are
 * [planes...][N/2+1][N][2] floats in the layout of the size class. */
int fbfft_b200_conv_workspace_region(int fft_size, int batch, int in_planes, int out_planes, int which,
                                     size_t* offset_bytes, size_t* size_bytes);

/* out[b][o][y][x] = sum_c sum_ij in_canvas[b][c][y+i][x+j] w[o][c][i][j]
 * (updateOutputIteratedKernel, fbfft/FFTIteratedConvolution.cuh:97-207). */
int fbfft_b200_conv_update_output(int fft_size, const float* in, const int* in_size, const int* in_stride, int in_padL,
                                  int in_padU, const float* weight, const int* w_size, const int* w_stride, float* out,
                                  const int* out_size, const int* out_stride, int out_padL, int out_padU,
                                  void* workspace, size_t workspace_bytes, int flags, void* stream);

/* grad_in[b][c] = sum_o (grad_out_canvas[b][o] circularly convolved with w[o][c])
 * (updateGradInputIteratedKernel, fbfft/FFTIteratedConvolution.cuh:254-363). */
int fbfft_b200_conv_update_grad_input(int fft_size, float* grad_in, const int* in_size, const int* in_stride,
                                      int in_padL, int in_padU, const float* weight, const int* w_size,
                                      const int* w_stride, const float* grad_out, const int* out_size,
                                      const int* out_stride, int out_padL, int out_padU, void* workspace,
                                      size_t workspace_bytes, int flags, void* stream);

/* grad_weight[o][c][i][j] = scale * sum_b sum_yx in_canvas[b][c][y+i][x+j] grad_out_canvas[b][o][y][x];
 * overwrites grad_weight (accGradParametersIteratedKernel,
 * fbfft/FFTIteratedConvolution.cuh:409-524). */
int fbfft_b200_conv_acc_grad_parameters(int fft_size, const float* in, const int* in_size, const int* in_stride,
                                        int in_padL, int in_padU, float* grad_weight, const int* w_size,
                                        const int* w_stride, const float* grad_out, const int* out_size,
                                        const int* out_stride, int out_padL, int out_padU, float scale,
                                        void* workspace, size_t workspace_bytes, int flags, void* stream);

/* ---- Whole layers: choice of the transform size and the loop over tiles ---------------------
 * In the reference both were the caller's job: it chose the instantiation
 * FFTIteratedConvolution<8|16|32> (fbfft/FFTIteratedConvolution.cuh:624-755) or chained the
 * building blocks for larger transforms, and it built the tile lists (:70-95, 105-114, 431-442).
 *
 * fbfft_b200_conv_plan: for a stride-1 convolution of [batch][in_planes][in_h][in_w] with
 * [out_planes][in_planes][kernel_h][kernel_w] and implicit zero padding (pad_h, pad_w), with the
 * batch sharded over `world` GPUs, picks the transform size (the cheapest of 8..128 under a
 * bytes + flops + per-tile cost model fitted to B200 measurements; est_us[i] is the estimate for
 * size 8 << i, 0 where the kernel does not fit), and reports the number of overlap-save tiles,
 * the outputs per tile, the contraction mode the passes will use (0 tensor cores, 1 FP32), the
 * reduction mode for fbfft_b200_conv_acc_grad_parameters_dp and the workspace one GPU needs.
 * Host arithmetic only. */
typedef struct fbfft_b200_conv_plan_t {
  int fft_size;
  int tiles;
  int tile_out_h, tile_out_w;
  int contraction;
  int dw_mode;
  size_t workspace_bytes;
  float est_us[5];
} fbfft_b200_conv_plan_t;
int fbfft_b200_conv_plan(int batch, int in_planes, int out_planes, int in_h, int in_w, int kernel_h, int kernel_w,
                         int pad_h, int pad_w, int world, fbfft_b200_conv_plan_t* plan);

/* The three passes on whole images of any size: the library walks the overlap-save tiles of
 * fbfft_b200_plan_tiles itself (the tile loops of fbfft/FFTIteratedConvolution.cuh:105-114 and
 * :431-442), the weight spectrum is computed once per call (never, with
 * FBFFT_CONV_REUSE_WEIGHT_SPECTRUM in `flags`), and the weight gradient is summed over the tiles in
 * the frequency domain with a single inverse transform at the end.  in [B][C][H][W],
 * out [B][O][H + 2 pad_h - kh + 1][W + 2 pad_w - kw + 1]; the workspace is the one of a single tile
 * (fbfft_b200_conv_workspace_bytes).  Nothing synchronises and nothing is allocated on the device,
 * so a call can be captured into a CUDA graph like the single-tile passes. */
int fbfft_b200_conv_tiled_update_output(int fft_size, const float* in, const int* in_size, const int* in_stride,
                                        const float* weight, const int* w_size, const int* w_stride, float* out,
                                        const int* out_size, const int* out_stride, int pad_h, int pad_w,
                                        void* workspace, size_t workspace_bytes, int flags, void* stream);
int fbfft_b200_conv_tiled_update_grad_input(int fft_size, float* grad_in, const int* in_size, const int* in_stride,
                                            const float* weight, const int* w_size, const int* w_stride,
                                            const float* grad_out, const int* out_size, const int* out_stride, int pad_h,
                                            int pad_w, void* workspace, size_t workspace_bytes, int flags, void* stream);
int fbfft_b200_conv_tiled_acc_grad_parameters(int fft_size, const float* in, const int* in_size, const int* in_stride,
                                              float* grad_weight, const int* w_size, const int* w_stride,
                                              const float* grad_out, const int* out_size, const int* out_stride,
                                              int pad_h, int pad_w, float scale, void* workspace, size_t workspace_bytes,
                                              int flags, void* stream);

/* ---- Data-parallel accGradParameters (no counterpart in the reference, which has no
 * multi-GPU code; what is summed is its accGradParameters,
 * fbfft/FFTIteratedConvolution.cuh:409-524, over batch shards) -------------------------
 * One process per GPU; the batch is sharded, weights are replicated; updateOutput and
 * updateGradInput need no communication.  The communicator wraps NCCL, which is loaded
 * on first use (libnccl.so.2; inside a process that already loaded one, that copy).
 *
 * fbfft_b200_comm_unique_id: rank 0 fills FBFFT_B200_UNIQUE_ID_BYTES bytes (host memory) and
 *   hands them to the other ranks by any means.
 * fbfft_b200_comm_init: every rank, with its device current.  Bounded: when the ranks have not
 *   all joined within timeout_ms the half-built communicator is aborted and FBFFT_CUDA_ERROR
 *   returned.  The same limit bounds every later wait of the host on this communicator.  The
 *   environment variable FBFFT_B200_NCCL_MAX_CTAS (1..64), read here, caps the blocks NCCL's kernels
 *   use (see fbfft_b200_set_contraction_reserved_sms).
 * fbfft_b200_comm_destroy: after the last call's work has finished on the stream.
 * fbfft_b200_dp_shard: the contiguous shard [lo, lo + count) of `total` units for `rank`
 *   (the first total % world ranks hold one more); host arithmetic only. */
#define FBFFT_B200_UNIQUE_ID_BYTES 128
typedef struct fbfft_b200_comm fbfft_b200_comm;
int fbfft_b200_comm_unique_id(void* id_out);
int fbfft_b200_comm_init(const void* unique_id, int rank, int world, int timeout_ms, fbfft_b200_comm** out);
int fbfft_b200_comm_info(const fbfft_b200_comm* comm, int* rank, int* world);
int fbfft_b200_comm_destroy(fbfft_b200_comm* comm);
int fbfft_b200_dp_shard(long long total, int world, int rank, long long* lo, long long* count);

/* How the weight gradient is summed over the ranks:
 *  FREQUENCY_ALLREDUCE       one all-reduce of the frequency-domain gradient
 *                            ([O][C][N/2+1][N] complex) between the contraction and its inverse
 *                            transform, which every rank then runs in full;
 *  FREQUENCY_REDUCE_SCATTER  the same sum taken as a reduce-scatter over the O*C planes: every rank
 *                            receives 1/world of the planes, inverse-transforms and crops only those,
 *                            and an all-gather distributes the (small) spatial gradient -- half the
 *                            bytes on the links and 1/world of the inverse work.  Needs O*C divisible
 *                            by world and a contiguous grad_weight, else it runs as the all-reduce;
 *  SPATIAL_ALLREDUCE         inverse transform first, all-reduce of the spatial gradient (equal up to
 *                            rounding, by linearity).
 * All ranks must pass the same mode, transform size, plane counts and flags; batch sizes may
 * differ (0 included).  Arguments as fbfft_b200_conv_acc_grad_parameters; in, grad_out and the
 * batch are this rank's shard.  STOP_AFTER_CONTRACTION returns before the collective and
 * START_FROM_SPECTRUM runs only the collective and what follows it, so that the sum can run on
 * a second stream under the other passes.  Work is enqueued on `stream`; the host may wait, within
 * the communicator's time limit, for NCCL to accept the calls. */
enum {
  FBFFT_DP_FREQUENCY_ALLREDUCE = 0,
  FBFFT_DP_FREQUENCY_REDUCE_SCATTER = 1,
  FBFFT_DP_SPATIAL_ALLREDUCE = 2
};
int fbfft_b200_conv_acc_grad_parameters_dp(fbfft_b200_comm* comm, int mode, int fft_size, const float* in,
                                           const int* in_size, const int* in_stride, int in_padL, int in_padU,
                                           float* grad_weight, const int* w_size, const int* w_stride,
                                           const float* grad_out, const int* out_size, const int* out_stride,
                                           int out_padL, int out_padU, float scale, void* workspace,
                                           size_t workspace_bytes, int flags, void* stream);

/* updateOutput without any device allocation, for callers that must not allocate:
 * a plugin invoked while its host holds the allocator, a loop with a
 * no-allocation rule after start-up, a process whose device memory is already
 * fully handed out.  Has no counterpart in the reference.
 *
 * Same arguments and result as fbfft_b200_conv_update_output without workspace and
 * flags: the spectra live in a fixed scratch area of
 * FBFFT_B200_NOALLOC_SCRATCH_BYTES that is part of the library image, so every GPU
 * that loads the library carries that much extra memory until the process exits.
 * Layers whose fbfft_b200_conv_workspace_bytes() exceeds it are refused with
 * FBFFT_UNSUPPORTED_SIZE.  The function calls no cudaMalloc / cudaFree and no
 * allocating library routine.
 *
 * The first call on each device looks up the device address of the scratch area
 * (with that device current); make that first call outside any stream capture.
 * All calls on a device share the one scratch area and it keeps whatever the last
 * call left in it: nothing in it needs clearing between calls, but two calls that
 * overlap on the GPU (different streams, or graphs replayed concurrently) race on
 * it -- serialise them. */
#define FBFFT_B200_NOALLOC_SCRATCH_BYTES (32u << 20)
int fbfft_b200_conv_update_output_noalloc(int fft_size, const float* in, const int* in_size, const int* in_stride,
                                          int in_padL, int in_padU, const float* weight, const int* w_size,
                                          const int* w_stride, float* out, const int* out_size,
                                          const int* out_stride, int out_padL, int out_padU, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FBFFT_B200_H_ */
