// Per-frequency-bin complex contraction for the two shapes a small batch shard leaves behind (the
// data-parallel passes on 4 or 8 GPUs): same math as cgemm_tma.cu / the reference's transposeMM
// (MM-inl.cuh:188-196),
//
//   D[m][n][x] = inv_norm * sum_k opA(A[m][k][x]) * opB(B[n][k][x]),  x = frequency bin,
//
// on FP32 CUDA cores, for operands in the convolution workspace's 4-bin blocks.
//   few columns (n <= 8: updateOutput / updateGradInput of a shard of at most 8 images): the big
//       operand A (the weight spectrum) streams through shared memory exactly once, every thread
//       owns one row of m and half of the 4 bins and keeps n accumulators; 8 complex multiply-adds
//       per 16 bytes of weights is below what the FP32 pipes sustain per byte of HBM, so the pass
//       runs at the rate the weights arrive.  The tensor-core kernel spends a whole 128-row split
//       and six padded MMAs on the same bytes (104 us against the 48 us the bytes take, FFT-64
//       layer at 8 images).
//   short sum (k <= 8: accGradParameters of such a shard): a rank-k update whose only real traffic is
//       the result; a thread keeps its row of A in registers and walks the columns.
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
};

__device__ __forceinline__ void tma_load4s(unsigned dst, const CUtensorMap* tm, int c0, int c1, int c2, int c3, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

__device__ __forceinline__ float* d_addr(const SmallArgs& g, int x0, int m, int n) {
  return g.D + 2 * ((long long)(x0 / g.d_qb) * g.d_bs + (x0 % g.d_qb) + (long long)m * g.d_ms + (long long)n * g.d_ns);
}

// ------------------------------------------------------------------ few columns
// 8 consumer warps (thread = row t/2, half t%2) and one producer warp; stages of SK values of k:
// A [SK][128 rows][32 B], B [SK][NB columns][32 B].
template <int NB>
struct FewCfg {
  static constexpr int NS = 5;
  static constexpr int A_BYTES = SK * SM_ROWS * 32, B_BYTES = SK * NB * 32, STAGE = A_BYTES + ((B_BYTES + 127) / 128) * 128;
  static constexpr int SMEM = NS * STAGE + 256;
  static constexpr int THREADS = 9 * 32;
};

template <int NB>
__global__ void __launch_bounds__(FewCfg<NB>::THREADS, 2) cgemm_fewcols_kernel(const __grid_constant__ CUtensorMap map_a,
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
          tma_load4s(dst, &map_a, 0, m0, s * SK, x0 / 4, full(st));
          tma_load4s(dst + C::A_BYTES, &map_b, 0, 0, s * SK, x0 / 4, full(st));
        }
      }
    }
    return;
  }
  const int row = tid >> 1, half = tid & 1;
  unsigned it = 0;
  for (int t = blockIdx.x; t < g.total_tiles; t += gridDim.x) {
    const int x0 = (t / g.m_tiles) * 4, m0 = (t % g.m_tiles) * SM_ROWS;
    float4 acc[NB];  // (bin0.re, bin0.im, bin1.re, bin1.im) of this thread's two bins, per column
#pragma unroll
    for (int n = 0; n < NB; ++n) acc[n] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < nsteps; ++s, ++it) {
      const int st = it % C::NS;
      if (!mbar_wait(full(st), (it / C::NS) & 1, kErrSmallFull)) return;
      const unsigned char* sa = sm + st * C::STAGE + row * 32 + half * 16;
      const unsigned char* sb = sm + st * C::STAGE + C::A_BYTES + half * 16;
#pragma unroll
      for (int j = 0; j < SK; ++j) {
        float4 a = *reinterpret_cast<const float4*>(sa + j * (SM_ROWS * 32));
        a.y *= g.sa, a.w *= g.sa;
#pragma unroll
        for (int n = 0; n < NB; ++n) {
          const float4 b = *reinterpret_cast<const float4*>(sb + (j * NB + n) * 32);
          acc[n].x += a.x * b.x - a.y * b.y;
          acc[n].y += a.x * b.y + a.y * b.x;
          acc[n].z += a.z * b.z - a.w * b.w;
          acc[n].w += a.z * b.w + a.w * b.z;
        }
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
        if (n < g.N)
          *reinterpret_cast<float4*>(d_addr(g, x0, m, n) + 4 * half) =
              make_float4(acc[n].x * g.inv_norm, acc[n].y * sgn, acc[n].z * g.inv_norm, acc[n].w * sgn);
      }
    }
  }
}

// ------------------------------------------------------------------ short sum
// One tile: 128 rows of m x NC columns of n x 4 bins, all k (<= KB) at once.
constexpr int KB = 8, NC = 64;
constexpr int SHORT_A = KB * SM_ROWS * 32, SHORT_B = KB * NC * 32, SHORT_SMEM = SHORT_A + SHORT_B + 64;

__global__ void __launch_bounds__(256, 4) cgemm_shortsum_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                const __grid_constant__ CUtensorMap map_b, SmallArgs g) {
  extern __shared__ __align__(1024) unsigned char sm[];
  const unsigned bar = smem_u32(sm + SHORT_A + SHORT_B);
  const int tid = threadIdx.x;
  if (tid == 0) {
    mbar_init(bar, 1);
    fence_async_smem();
  }
  __syncthreads();
  const int t = blockIdx.x;
  const int nt = t % g.n_tiles, mt = (t / g.n_tiles) % g.m_tiles, x0 = (t / (g.n_tiles * g.m_tiles)) * 4;
  const int m0 = mt * SM_ROWS, n0 = nt * NC;
  if (tid == 0) {
    mbar_expect_tx(bar, (unsigned)(SHORT_A + SHORT_B));
    tma_load4s(smem_u32(sm), &map_a, 0, m0, 0, x0 / 4, bar);
    tma_load4s(smem_u32(sm + SHORT_A), &map_b, 0, n0, 0, x0 / 4, bar);
  }
  if (!mbar_wait(bar, 0, kErrSmallKWait)) return;
  const int row = tid >> 1, half = tid & 1;
  float4 a[KB];
#pragma unroll
  for (int k = 0; k < KB; ++k) {
    a[k] = *reinterpret_cast<const float4*>(sm + (k * SM_ROWS + row) * 32 + half * 16);
    a[k].y *= g.sa, a[k].w *= g.sa;
  }
  const int m = m0 + row;
  const float sgn = g.conj_out ? -g.inv_norm : g.inv_norm;
  const unsigned char* sb = sm + SHORT_A + half * 16;
  int ncols = g.N - n0;
  if (ncols > NC) ncols = NC;
#pragma unroll 2
  for (int n = 0; n < ncols; ++n) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < KB; ++k) {
      const float4 b = *reinterpret_cast<const float4*>(sb + (k * NC + n) * 32);
      acc.x += a[k].x * b.x - a[k].y * b.y;
      acc.y += a[k].x * b.y + a[k].y * b.x;
      acc.z += a[k].z * b.z - a[k].w * b.w;
      acc.w += a[k].z * b.w + a[k].w * b.z;
    }
    if (m < g.M)
      *reinterpret_cast<float4*>(d_addr(g, x0, m, n0 + n) + 4 * half) =
          make_float4(acc.x * g.inv_norm, acc.y * sgn, acc.z * g.inv_norm, acc.w * sgn);
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

}  // namespace

// Operands in 4-bin blocks (a_qb = b_qb = 4), overwriting result, n <= 8 or k <= 8, 32-byte aligned D elements
bool cgemm_small_supported(const float* a, const float* b, const float* d, long long d_ms, long long d_ns, long long d_bs,
                           int d_qb, int a_qb, int b_qb, int M, int N, int K, int X, bool accumulate) {
  if (accumulate || a_qb != 4 || b_qb != 4 || X % 4 != 0 || M < 1 || N < 1 || K < 1) return false;
  if (!(N <= 8 || K <= KB)) return false;
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
  g.m_tiles = (M + SM_ROWS - 1) / SM_ROWS;
  alignas(64) CUtensorMap ma, mb;
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(cgemm_fewcols_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, FewCfg<4>::SMEM);
    cudaFuncSetAttribute(cgemm_fewcols_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, FewCfg<8>::SMEM);
    cudaFuncSetAttribute(cgemm_shortsum_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SHORT_SMEM);
    configured[dev] = true;
  }
  if (N <= 8) {
    const int NB = N <= 4 ? 4 : 8;
    if (!small_map(&ma, a, a_rs, a_ks, a_bs, M, K, X, SM_ROWS, SK) || !small_map(&mb, b, b_rs, b_ks, b_bs, N, K, X, NB, SK)) return -1;
    g.n_tiles = 1;
    const long long total = (long long)g.m_tiles * (X / 4);
    g.total_tiles = (int)total;
    const long long cap = 2LL * sm_count();
    const int grid = (int)(total < cap ? total : cap);
    if (NB == 4) {
      cgemm_fewcols_kernel<4><<<grid, FewCfg<4>::THREADS, FewCfg<4>::SMEM, s>>>(ma, mb, g);
    } else {
      cgemm_fewcols_kernel<8><<<grid, FewCfg<8>::THREADS, FewCfg<8>::SMEM, s>>>(ma, mb, g);
    }
  } else {
    if (!small_map(&ma, a, a_rs, a_ks, a_bs, M, K, X, SM_ROWS, KB) || !small_map(&mb, b, b_rs, b_ks, b_bs, N, K, X, NC, KB)) return -1;
    g.n_tiles = (N + NC - 1) / NC;
    const long long total = (long long)g.m_tiles * g.n_tiles * (X / 4);
    if (total > 0x7fffffffLL) return -1;
    g.total_tiles = (int)total;
    cgemm_shortsum_kernel<<<(int)total, 256, SHORT_SMEM, s>>>(ma, mb, g);
  }
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

int read_device_error_small() { return device_error_word_read(); }
int clear_device_error_small() { return device_error_word_clear(); }

}  // namespace fbfft_b200
