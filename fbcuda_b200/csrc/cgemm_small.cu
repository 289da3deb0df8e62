// Per-frequency-bin complex contraction for the two shapes a small batch shard leaves behind (the
// data-parallel passes on 4 or 8 GPUs): same math as cgemm_tma.cu / the reference's transposeMM
// (MM-inl.cuh:188-196),
//
//   D[m][n][x] = inv_norm * sum_k opA(A[m][k][x]) * opB(B[n][k][x]),  x = frequency bin,
//
// on FP32 CUDA cores, for operands in the convolution workspace's 4-bin blocks.
//   few columns (n <= 8: updateOutput / updateGradInput of a shard of at most 8 images): the big
//       operand A (the weight spectrum) streams through shared memory exactly once, every thread
//       owns one row of m and half of the 4 bins and keeps n accumulators.  The tensor-core kernel
//       spends a whole 128-row split and six padded MMAs on the same bytes.  Measured, FFT-64 layer
//       (128 x 128 planes, 277 MB of weights) at 8 images: 69 us against 104 us; FFT-128 layer (96 x 96,
//       613 MB) at 4 images: 106-115 us against 272 us (the bytes alone take 94 us at the copy rate).
//       How A is described to the copy engine matters as much as the math: as 32-byte runs (one 4-bin
//       element) the stream stops at 4.0-4.4 TB/s; described as 1 KB runs of 32 adjacent rows, or as
//       128-byte runs of 4 adjacent k with the 128-byte swizzle, whichever the operand's strides allow,
//       the same bytes arrive at 5.0-5.9 TB/s.
//   short sum (k <= 8: accGradParameters of such a shard): a rank-k update whose only real traffic is
//       the result; a thread keeps its row of A in registers and walks the columns; the 8 lanes of a
//       row write 16 consecutive bins, a whole 128-byte line (FFT-128 layer at 4 images: 118 us against
//       179 us, 613 MB of result; with 32-byte pieces of lines the same kernel took 254 us).
// Operands arrive by tensor copies (cp.async.bulk.tensor, zero fill outside the tensors, completion
// on mbarriers with bounded waits); a lane pair holds the two 16-byte halves of an element, so every
// store is a whole 32-byte sector.
#include <cuda.h>  // CUtensorMap

#include <cstring>

#include "fft2d_small.cuh"  // mbarrier helpers, bounded wait, device status word
#include "kernels.h"

namespace fbfft_b200 {

namespace {

constexpr int SM_ROWS = 128;  // rows of m per tile
constexpr int SK = 4;         // values of k per stage
constexpr int KB = 8;         // longest short sum
enum : int { kErrSmallFull = 221, kErrSmallFree = 222, kErrSmallKWait = 223 };

struct SmallArgs {
  float* D;
  long long d_ms, d_ns, d_bs;  // bin x of (m, n) at D + 2 * ((x/d_qb)*d_bs + x%d_qb + m*d_ms + n*d_ns) floats
  int d_qb;
  int M, N, K, X;
  int m_tiles, n_tiles, total_tiles;
  float inv_norm;
  float sa;     // sign of A's imaginary part after folding both conjugations into A
  int conj_out; // conjugate the sum at the end (B was conjugated)
  int a_mode;   // few columns, how A arrives: 0 = 32-byte runs, 1 = 1 KB runs of 32 rows, 2 = 128-byte runs of 4 k (swizzled)
};

__device__ __forceinline__ void tma_load4s(unsigned dst, const CUtensorMap* tm, int c0, int c1, int c2, int c3, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tma_load3s(unsigned dst, const CUtensorMap* tm, int c0, int c1, int c2, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}

__device__ __forceinline__ float* d_addr(const SmallArgs& g, int x0, int m, int n) {
  return g.D + 2 * ((long long)(x0 / g.d_qb) * g.d_bs + (x0 % g.d_qb) + (long long)m * g.d_ms + (long long)n * g.d_ns);
}

// Complex multiply-add on the packed FP32 pipe (fma.rn.f32x2): with the element of the streamed
// operand duplicated, (ar, ar) and (ai, ai), and the shared operand as it lies in memory, (br, bi),
//   P += (ar, ar) * (br, bi),   Q += (ai, ai) * (br, bi),   sum = (P.x - Q.y, P.y + Q.x):
// two instructions per complex product instead of four.
struct Dup {
  float2 re0, im0, re1, im1;  // bins 0 and 1 of a thread's 16 bytes
};
__device__ __forceinline__ Dup dup_of(const float4 a, float sa) {
  Dup d;
  d.re0 = make_float2(a.x, a.x), d.im0 = make_float2(a.y * sa, a.y * sa);
  d.re1 = make_float2(a.z, a.z), d.im1 = make_float2(a.w * sa, a.w * sa);
  return d;
}
struct Acc {
  float2 p0, q0, p1, q1;
};
__device__ __forceinline__ void acc_zero(Acc& c) { c.p0 = c.q0 = c.p1 = c.q1 = make_float2(0.f, 0.f); }
__device__ __forceinline__ void acc_mad(Acc& c, const Dup& a, const float4 b) {
#ifndef FBFFT_SMALL_NOMATH
  const float2 b0 = make_float2(b.x, b.y), b1 = make_float2(b.z, b.w);
  c.p0 = __ffma2_rn(a.re0, b0, c.p0);
  c.q0 = __ffma2_rn(a.im0, b0, c.q0);
  c.p1 = __ffma2_rn(a.re1, b1, c.p1);
  c.q1 = __ffma2_rn(a.im1, b1, c.q1);
#endif
}
__device__ __forceinline__ float4 acc_value(const Acc& c, float inv_norm, float sgn) {
  return make_float4((c.p0.x - c.q0.y) * inv_norm, (c.p0.y + c.q0.x) * sgn, (c.p1.x - c.q1.y) * inv_norm,
                     (c.p1.y + c.q1.x) * sgn);
}

// ------------------------------------------------------------------ few columns
// 8 consumer warps (thread = row t/2, half t%2) and one producer warp; stages of SK values of k:
// A [SK][128 rows][32 B], B [SK][NB columns][32 B].
template <int NB>
struct FewCfg {
  // 8 columns need 152 registers: one block of 10 stages per SM; 4 columns: two blocks of 5 stages
  static constexpr int MINB = NB == 8 ? 1 : 2;
  static constexpr int NS = MINB == 2 ? 5 : 10;
  static constexpr int A_BYTES = SK * SM_ROWS * 32, B_BYTES = SK * NB * 32, STAGE = A_BYTES + ((B_BYTES + 1023) / 1024) * 1024;
  static constexpr int SMEM = NS * STAGE + 256;
  static constexpr int THREADS = 9 * 32;
};

template <int NB>
__global__ void __launch_bounds__(FewCfg<NB>::THREADS, FewCfg<NB>::MINB) cgemm_fewcols_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                               const __grid_constant__ CUtensorMap map_b,
                                                                               SmallArgs g) {
  using C = FewCfg<NB>;
  extern __shared__ __align__(1024) unsigned char sm[];
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(sm + C::NS * C::STAGE);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto full = [&](int i) { return smem_u32(bars + i); };
  auto empty = [&](int i) { return smem_u32(bars + C::NS + i); };
  if (tid == 0) {
    for (int i = 0; i < C::NS; ++i) {
      mbar_init(full(i), 1);
      mbar_init(empty(i), 8);
    }
    fence_async_smem();
  }
  __syncthreads();
  const int nsteps = (g.K + SK - 1) / SK;
  if (warp == 8) {
    if (lane == 0) {
      unsigned it = 0;
      for (int t = blockIdx.x; t < g.total_tiles; t += gridDim.x) {
        const int x0 = (t / g.m_tiles) * 4, m0 = (t % g.m_tiles) * SM_ROWS;
        for (int s = 0; s < nsteps; ++s, ++it) {
          const int st = it % C::NS;
          if (it >= (unsigned)C::NS && !mbar_wait(empty(st), ((it / C::NS) - 1) & 1, kErrSmallFree)) return;
          const unsigned dst = smem_u32(sm + st * C::STAGE);
          mbar_expect_tx(full(st), (unsigned)(C::A_BYTES + C::B_BYTES));
          if (g.a_mode == 2) {
            tma_load3s(dst, &map_a, s * SK * 8, m0, x0 / 4, full(st));
          } else {
            tma_load4s(dst, &map_a, 0, g.a_mode == 1 ? m0 / 32 : m0, s * SK, x0 / 4, full(st));
          }
          tma_load4s(dst + C::A_BYTES, &map_b, 0, 0, s * SK, x0 / 4, full(st));
        }
      }
    }
    return;
  }
  // modes 0 and 1: [k][row][32 B], a lane pair shares a row; mode 2: [row][4 k x 32 B] with the 16-byte
  // pieces of a row XORed with (row % 8) (128-byte swizzle), 8 consecutive lanes take 8 consecutive rows
  const bool kruns = g.a_mode == 2;
  const int row = kruns ? ((tid & 7) | ((tid >> 4) << 3)) : tid >> 1, half = kruns ? (tid >> 3) & 1 : tid & 1;
  const int a_base = kruns ? row * 128 : row * 32 + half * 16, a_step = kruns ? 0 : SM_ROWS * 32;
  unsigned it = 0;
  for (int t = blockIdx.x; t < g.total_tiles; t += gridDim.x) {
    const int x0 = (t / g.m_tiles) * 4, m0 = (t % g.m_tiles) * SM_ROWS;
    Acc acc[NB];
#pragma unroll
    for (int n = 0; n < NB; ++n) acc_zero(acc[n]);
    for (int s = 0; s < nsteps; ++s, ++it) {
      const int st = it % C::NS;
      if (!mbar_wait(full(st), (it / C::NS) & 1, kErrSmallFull)) return;
      const unsigned char* pa = sm + st * C::STAGE + a_base;
      const unsigned char* pb = sm + st * C::STAGE + C::A_BYTES + half * 16;
#pragma unroll
      for (int j = 0; j < SK; ++j) {
        const int piece = kruns ? ((2 * j + half) ^ (row & 7)) << 4 : 0;
        const Dup a = dup_of(*reinterpret_cast<const float4*>(pa + j * a_step + piece), g.sa);
#pragma unroll
        for (int n = 0; n < NB; ++n) acc_mad(acc[n], a, *reinterpret_cast<const float4*>(pb + (j * NB + n) * 32));
      }
      __syncwarp();
      if (lane == 0) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty(st)) : "memory");
      }
    }
    const int m = m0 + row;
    if (m < g.M) {
      const float sgn = g.conj_out ? -g.inv_norm : g.inv_norm;
#pragma unroll
      for (int n = 0; n < NB; ++n) {
        if (n < g.N) *reinterpret_cast<float4*>(d_addr(g, x0, m, n) + 4 * half) = acc_value(acc[n], g.inv_norm, sgn);
      }
    }
  }
}

// ------------------------------------------------------------------ short sum
// One tile: 32 rows of m x 32 columns of n x 16 bins (4 blocks of 4), all k (<= KT) at once.  The
// tensor copies order the dimensions (8 floats, 4-bin blocks, rows, k), so that shared memory holds
// [k][row][4 blocks][32 B]: the 8 lanes (block, half) of a row read 128 contiguous bytes and write a
// whole 128-byte line of the result (16 consecutive bins of one plane).
constexpr int SR = 32, SC = 32;
template <int KT>
struct ShortCfg {
  static constexpr int A_BYTES = KT * SR * 128, B_BYTES = KT * SC * 128, SMEM = A_BYTES + B_BYTES + 64;
};

template <int KT>
__global__ void __launch_bounds__(256, 2) cgemm_shortsum_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                const __grid_constant__ CUtensorMap map_b, SmallArgs g) {
  using C = ShortCfg<KT>;
  extern __shared__ __align__(1024) unsigned char sm[];
  const unsigned bar = smem_u32(sm + C::A_BYTES + C::B_BYTES);
  const int tid = threadIdx.x;
  if (tid == 0) {
    mbar_init(bar, 1);
    fence_async_smem();
  }
  __syncthreads();
  const int t = blockIdx.x;
  const int nt = t % g.n_tiles, mt = (t / g.n_tiles) % g.m_tiles, x0 = (t / (g.n_tiles * g.m_tiles)) * 16;
  const int m0 = mt * SR, n0 = nt * SC;
  if (tid == 0) {
    mbar_expect_tx(bar, (unsigned)(C::A_BYTES + C::B_BYTES));
    tma_load4s(smem_u32(sm), &map_a, 0, x0 / 4, m0, 0, bar);
    tma_load4s(smem_u32(sm + C::A_BYTES), &map_b, 0, x0 / 4, n0, 0, bar);
  }
  if (!mbar_wait(bar, 0, kErrSmallKWait)) return;
  const int row = tid >> 3, sub = tid & 7;  // sub = 2 * (block of 4 bins) + half
  Dup a[KT];
#pragma unroll
  for (int k = 0; k < KT; ++k) a[k] = dup_of(*reinterpret_cast<const float4*>(sm + (k * SR + row) * 128 + sub * 16), g.sa);
  const int m = m0 + row;
  const float sgn = g.conj_out ? -g.inv_norm : g.inv_norm;
  const unsigned char* pb = sm + C::A_BYTES + sub * 16;
  int ncols = g.N - n0;
  if (ncols > SC) ncols = SC;
  if (m >= g.M) return;
  float* dst = d_addr(g, x0, m, n0) + 4 * sub;  // 2 floats per bin, 2 bins per 16 bytes
#pragma unroll 2
  for (int n = 0; n < ncols; ++n) {
    Acc acc;
    acc_zero(acc);
#pragma unroll
    for (int k = 0; k < KT; ++k) acc_mad(acc, a[k], *reinterpret_cast<const float4*>(pb + (k * SC + n) * 128));
    *reinterpret_cast<float4*>(dst + 2 * (long long)n * g.d_ns) = acc_value(acc, g.inv_norm, sgn);
  }
}

// 4-D map of an operand in 4-bin blocks: (8 floats, rows, k, blocks), box {8, box_rows, box_k, 1}
bool small_map(CUtensorMap* m, const float* p, long long rs, long long ks, long long bs, int rows, int kcount, int X,
               int box_rows, int box_k) {
  const unsigned long long dims[4] = {8ULL, (unsigned long long)rows, (unsigned long long)kcount, (unsigned long long)(X / 4)};
  const unsigned long long strides[3] = {(unsigned long long)rs * 8, (unsigned long long)ks * 8, (unsigned long long)bs * 8};
  const unsigned box[4] = {8u, (unsigned)box_rows, (unsigned)box_k, 1u};
  return encode_tensor_map_f32(m, p, 4, dims, strides, box);
}

// the same tensor when its rows are adjacent planes (row stride 4 complex values) and a multiple of
// 32: (256 floats = 32 rows, groups of 32 rows, k, blocks), box {256, box_rows / 32, box_k, 1} -- the
// same bytes land in the same places, but the copy engine moves 1 KB runs instead of 32-byte ones
bool small_map_row_runs(CUtensorMap* m, const float* p, long long ks, long long bs, int rows, int kcount, int X,
                        int box_rows, int box_k) {
  const unsigned long long dims[4] = {256ULL, (unsigned long long)(rows / 32), (unsigned long long)kcount,
                                      (unsigned long long)(X / 4)};
  const unsigned long long strides[3] = {1024ULL, (unsigned long long)ks * 8, (unsigned long long)bs * 8};
  const unsigned box[4] = {256u, (unsigned)(box_rows / 32), (unsigned)box_k, 1u};
  return encode_tensor_map_f32(m, p, 4, dims, strides, box);
}

// the same tensor when consecutive k are adjacent planes (k stride 4 complex values): (8 K floats, rows,
// blocks), box {32 floats = 4 k, box_rows, 1}, 128-byte swizzle
bool small_map_k_runs(CUtensorMap* m, const float* p, long long rs, long long bs, int rows, int kcount, int X, int box_rows) {
  const unsigned long long dims[3] = {8ULL * (unsigned long long)kcount, (unsigned long long)rows, (unsigned long long)(X / 4)};
  const unsigned long long strides[2] = {(unsigned long long)rs * 8, (unsigned long long)bs * 8};
  const unsigned box[3] = {8u * SK, (unsigned)box_rows, 1u};
  return encode_tensor_map_f32(m, p, 3, dims, strides, box, 128);
}

// the same tensor with the blocks second: (8 floats, blocks, rows, k), box {8, 4, box_rows, box_k}
bool small_map_blocks_inner(CUtensorMap* m, const float* p, long long rs, long long ks, long long bs, int rows, int kcount,
                            int X, int box_rows, int box_k) {
  const unsigned long long dims[4] = {8ULL, (unsigned long long)(X / 4), (unsigned long long)rows, (unsigned long long)kcount};
  const unsigned long long strides[3] = {(unsigned long long)bs * 8, (unsigned long long)rs * 8, (unsigned long long)ks * 8};
  const unsigned box[4] = {8u, 4u, (unsigned)box_rows, (unsigned)box_k};
  return encode_tensor_map_f32(m, p, 4, dims, strides, box);
}

template <int KT>
int launch_shortsum(const CUtensorMap& ma, const CUtensorMap& mb, const SmallArgs& g, int blocks, cudaStream_t s) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(cgemm_shortsum_kernel<KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, ShortCfg<KT>::SMEM);
    configured[dev] = true;
  }
  cgemm_shortsum_kernel<KT><<<blocks, 256, ShortCfg<KT>::SMEM, s>>>(ma, mb, g);
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

}  // namespace

// Operands in 4-bin blocks (a_qb = b_qb = 4), overwriting result, n <= 8 or k <= 8, 32-byte aligned D elements
bool cgemm_small_supported(const float* a, const float* b, const float* d, long long d_ms, long long d_ns, long long d_bs,
                           int d_qb, int a_qb, int b_qb, int M, int N, int K, int X, bool accumulate) {
  if (accumulate || a_qb != 4 || b_qb != 4 || X % 4 != 0 || M < 1 || N < 1 || K < 1) return false;
  if (!(N <= 8 || (K <= KB && X % 16 == 0 && d_qb % 16 == 0))) return false;
  if (d_qb < 4 || d_qb % 4 != 0 || d_ms % 2 != 0 || d_ns % 2 != 0 || d_bs % 2 != 0) return false;
  if (!aligned16(a) || !aligned16(b) || (reinterpret_cast<uintptr_t>(d) & 31u) != 0) return false;
  return true;
}

int cgemm_small(const float* a, long long a_rs, long long a_ks, bool conjA, const float* b, long long b_rs, long long b_ks,
                bool conjB, float* d, long long d_ms, long long d_ns, int M, int N, int K, int X, float inv_norm,
                cudaStream_t s, long long a_bs, long long b_bs, long long d_bs, int d_qb) {
  SmallArgs g;
  g.D = d, g.d_ms = d_ms, g.d_ns = d_ns, g.d_bs = d_bs, g.d_qb = d_qb;
  g.M = M, g.N = N, g.K = K, g.X = X, g.inv_norm = inv_norm;
  // opA(a) opB(b): with B conjugated, sum_k opA(a) conj(b) = conj(sum_k conj(opA(a)) b)
  g.conj_out = conjB ? 1 : 0;
  g.sa = (conjA != conjB) ? -1.f : 1.f;
  g.a_mode = 0;
  alignas(64) CUtensorMap ma, mb;
  if (N <= 8) {
    static bool configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      cudaFuncSetAttribute(cgemm_fewcols_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, FewCfg<4>::SMEM);
      cudaFuncSetAttribute(cgemm_fewcols_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, FewCfg<8>::SMEM);
      configured[dev] = true;
    }
    const int NB = N <= 4 ? 4 : 8;
    g.a_mode = (a_rs == 4 && M % 32 == 0) ? 1 : (a_ks == 4 ? 2 : 0);
    if (!(g.a_mode == 1   ? small_map_row_runs(&ma, a, a_ks, a_bs, M, K, X, SM_ROWS, SK)
          : g.a_mode == 2 ? small_map_k_runs(&ma, a, a_rs, a_bs, M, K, X, SM_ROWS)
                          : small_map(&ma, a, a_rs, a_ks, a_bs, M, K, X, SM_ROWS, SK)) ||
        !small_map(&mb, b, b_rs, b_ks, b_bs, N, K, X, NB, SK))
      return -1;
    g.m_tiles = (M + SM_ROWS - 1) / SM_ROWS;
    g.n_tiles = 1;
    const long long total = (long long)g.m_tiles * (X / 4);
    if (total > 0x7fffffffLL) return -1;
    g.total_tiles = (int)total;
    // persistent blocks fill their SMs' shared memory: a caller that runs collectives beside the contraction
    // keeps some SMs free for them (set_contraction_reserved_sms), as the tensor-core kernel does
    const int sms = sm_count() - contraction_reserved_sms();
    const long long cap = (long long)(NB == 8 ? FewCfg<8>::MINB : FewCfg<4>::MINB) * (sms > 1 ? sms : 1);
    const int grid = (int)(total < cap ? total : cap);
    if (NB == 4) {
      cgemm_fewcols_kernel<4><<<grid, FewCfg<4>::THREADS, FewCfg<4>::SMEM, s>>>(ma, mb, g);
    } else {
      cgemm_fewcols_kernel<8><<<grid, FewCfg<8>::THREADS, FewCfg<8>::SMEM, s>>>(ma, mb, g);
    }
    return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
  }
  const int KT = K <= 4 ? 4 : KB;
  if (!small_map_blocks_inner(&ma, a, a_rs, a_ks, a_bs, M, K, X, SR, KT) ||
      !small_map_blocks_inner(&mb, b, b_rs, b_ks, b_bs, N, K, X, SC, KT))
    return -1;
  g.m_tiles = (M + SR - 1) / SR;
  g.n_tiles = (N + SC - 1) / SC;
  const long long total = (long long)g.m_tiles * g.n_tiles * (X / 16);
  if (total > 0x7fffffffLL) return -1;
  g.total_tiles = (int)total;
  return KT == 4 ? launch_shortsum<4>(ma, mb, g, (int)total, s) : launch_shortsum<KB>(ma, mb, g, (int)total, s);
}

int read_device_error_small() { return device_error_word_read(); }
int clear_device_error_small() { return device_error_word_clear(); }

}  // namespace fbfft_b200
