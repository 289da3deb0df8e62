// Per-frequency-bin complex contraction, persistent warp-specialised version: operands arrive by
// asynchronous copies into shared memory, the 3xTF32 split runs from there, the products run on
// the 5th-generation tensor cores (tcgen05.mma kind::tf32, accumulators in tensor memory) and the
// result leaves by TMA tensor stores.  Same math as cgemm_bins.cu / the reference's transposeMM
// (MM-inl.cuh:188-196):
//
//   D[m][n][x] (+)= inv_norm * sum_k opA(A[m][k][x]) * opB(B[n][k][x]),  x = frequency bin.
//
// A tile is 128 rows of m, BN columns of n and 4 consecutive bins (32 contiguous bytes of every
// operand element: one DRAM sector).  Each block walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...
// Roles (17 warps):
//   warps 8-11    bring the raw fp32 operands of 4 values of k into a ring of NR stages ([k][row][32 B]
//                 per operand).  Operands in 4-bin blocks (the convolution workspace) arrive by two
//                 tensor copies per stage, issued by one thread (cp.async.bulk.tensor with the 32-byte
//                 swizzle, zero fill outside the tensor, completion bytes on the stage's mbarrier).
//                 Other layouts take 16-byte cp.async copies issued by all four warps, lanes following
//                 the direction in which the operand is contiguous; that path levels off near 32 KB in
//                 flight per SM (FFT-64 layer: 170 us per contraction against 136 us with tensor copies).
//   warps 0-7     read the raw stages into registers, hand them back at once, split every fp32 into
//                 hi = tf32(x) and lo = x - hi, and write K-major operand tiles in the tensor core's
//                 no-swizzle layout (8 x 16-byte core matrices) per bin: Ar, Ai (hi and lo) and the
//                 stack [-s Bi | Br | s Bi] (hi and lo; s = -1 when B is conjugated), into a ring of two
//                 half stages of two bins each;
//   warp 12       one lane issues, per bin and k-step of 8, six MMAs of 128 x 2BN x 8 into the bin's
//                 [Re | Im] accumulator:  Ar_h x S_h, Ai_h x S'_h, Ar_h x S_l, Ai_h x S'_l, Ar_l x S_h,
//                 Ai_l x S'_h with S = rows BN..3BN of the stack = [Br | s Bi] and S' = rows 0..2BN =
//                 [-s Bi | Br] (the Ai products negated when A is conjugated); tcgen05.commit frees
//                 the half stage and, after the last k-step, hands the accumulators to the epilogue;
//   warps 13-16   read the accumulators (tcgen05.ld, each warp its own 32 lanes = rows), scale,
//                 interleave the 4 bins' re/im into 32 bytes per (m, n) in a 4 KB staging buffer and
//                 issue one tensor store (or reduce-add when accumulating) per 4 columns of n.
// What bounds it, measured with roles switched off one at a time (FFT-64 layer, B = 64, before the
// tensor copies: 171 us): everything but the copies 119 us, the copies alone 115 us, the barrier
// skeleton with the accumulator reads 44 us, MMAs and stores under 10 us each.  The split and the
// MMAs' operand reads share the shared-memory bandwidth (per half stage the MMAs read 96 KB of
// operand tiles, the split writes 56 KB and reads 24 KB, the copies write 24 KB), and the two half
// stages serialise split and MMAs of a bin pair through two barrier hand-overs.  Tried and measured
// slower: stores of the result straight from registers (32-byte st.global.v8: 184 us; two 16-byte
// halves: 209 us), the 128-row operand loaded straight into registers one k-step ahead (same time
// for row-contiguous operands, 205 us for k-contiguous ones), L2 prefetches ahead of the copies
// (290 us), busy polling instead of suspending waits (182 us), MMAs issued by the last converter
// warp to arrive (201 us), a third half stage or six raw stages for column tiles <= 32 (no change),
// the epilogue's staging buffer as two halves stored separately (145 us against 138 us).  Second
// ablation, on this kernel (138 us): without the epilogue 109, without the split 125, without the
// copies 122, without the MMAs 126; barrier skeleton alone 27, with the accumulator reads 44.
// Every mbarrier wait is bounded; a wait that runs out records an error, the roles drain, and the
// block still releases its tensor memory before returning.
#include <cuda.h>  // CUtensorMap and its enums; the encoder itself is looked up through the runtime

#include <cstring>

#include "fft2d_small.cuh"  // mbarrier helpers, fence_async_smem
#include "kernels.h"

namespace fbfft_b200 {

namespace {

constexpr int kConvThreads = 256;  // warps 0-7
constexpr int kProdThreads = 128;  // warps 8-11
constexpr int kWarpProd = 8, kWarpMma = 12, kWarpEpi = 13;
constexpr int kThreads = 17 * 32;
constexpr int BM = 128, XB = 4, KQ = 4, KS = 8;
enum : int { kErrRawFull = 211, kErrRawFree = 212, kErrCvFull = 213, kErrCvFree = 214, kErrAccFull = 215, kErrAccFree = 216 };

template <int BN>
struct Cfg {
  static constexpr int NR = 4;                       // raw stages (4 values of k each; a k-step of 8 needs two)
  static constexpr int NH = 2;                       // converted half stages (2 bins x 8 k each)
  static constexpr int NACC = (BN >= 48) ? 1 : 2;    // accumulator sets in tensor memory
  static constexpr int ACC_COLS = XB * 2 * BN;
  static constexpr int TMEM_COLS = (NACC * ACC_COLS > 256) ? 512 : 256;  // a power of two >= the accumulators
  // raw stage: [k][row][32 bytes] per operand, the k slices 32 bytes further apart than their size so that
  // copies issued k-fastest do not all land in the same banks
  static constexpr int A_KSTRIDE = BM * 32 + 32, B_KSTRIDE = BN * 32 + 32;
  static constexpr int A_RAW = KQ * A_KSTRIDE, B_RAW = KQ * B_KSTRIDE, RAW = A_RAW + B_RAW;
  // tensor copies write dense boxes: k slices BM*32 / BN*32 bytes apart, B behind the 16 KB of A
  static constexpr int A_RAW_T = KQ * BM * 32;
  static constexpr int A_TILE = BM * KS * 4;         // one (bin, part, split) tile of A
  static constexpr int B_TILE = 3 * BN * KS * 4;     // one (bin, split) stack of B
  static constexpr int HALF_A = 2 * 2 * 2 * A_TILE, HALF_B = 2 * 2 * B_TILE, HSTAGE = HALF_A + HALF_B;
  static constexpr int EPI_WARP = 32 * 4 * 32;       // staging per epilogue warp: 32 rows x 4 columns x 32 bytes
  static constexpr int A_LBO = (BM / 8) * 128, B_LBO = (3 * BN / 8) * 128, SBO = 128;
  static constexpr int OFF_CONV = NR * RAW, OFF_EPI = OFF_CONV + NH * HSTAGE, OFF_BAR = OFF_EPI + 4 * EPI_WARP;
  static constexpr int SMEM = OFF_BAR + 256;
};

__device__ __forceinline__ unsigned long long smem_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
  // K-major, no swizzle: 8-row x 16-byte core matrices; LBO between the two 16-byte k-chunks of
  // an 8-wide k-step, SBO between 8-row groups; descriptor version 1 (bits 46-47)
  return (unsigned long long)((addr >> 4) & 0x3FFF) | ((unsigned long long)((lbo_bytes >> 4) & 0x3FFF) << 16) |
         ((unsigned long long)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ULL << 46);
}
__device__ __forceinline__ unsigned instr_desc(int n, bool neg_a) {
  // D fp32, A and B tf32, both K-major, M = 128
  return (1u << 4) | (2u << 7) | (2u << 10) | ((neg_a ? 1u : 0u) << 13) | ((unsigned)(n >> 3) << 17) |
         ((unsigned)(BM >> 4) << 24);
}
__device__ __forceinline__ void mma_tf32(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc,
                                         unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
__device__ __forceinline__ void mma_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld4(unsigned taddr, float (&v)[4]) {
  unsigned r0, r1, r2, r3;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(taddr));
  v[0] = __uint_as_float(r0), v[1] = __uint_as_float(r1), v[2] = __uint_as_float(r2), v[3] = __uint_as_float(r3);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src, unsigned src_bytes) {
  asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void tma_load4(unsigned dst, const CUtensorMap* tm, int c0, int c1, int c2, int c3, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store4(const CUtensorMap* tm, int c0, int c1, int c2, int c3, unsigned src) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(tm), "r"(c0),
               "r"(c1), "r"(c2), "r"(c3), "r"(src)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add4(const CUtensorMap* tm, int c0, int c1, int c2, int c3, unsigned src) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(tm),
               "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(src)
               : "memory");
}
// Bounded wait: gives up after two seconds, or as soon as another role of the block has given up
// (abort word in shared memory), recording `code`
__device__ __forceinline__ bool wait_bar(unsigned bar, unsigned parity, int code, volatile int* abort_word) {
  if (mbar_try(bar, parity)) return true;
  unsigned long long t0, t1;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    if (mbar_try(bar, parity)) return true;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (*abort_word != 0 || t1 - t0 > 2000000000ULL) break;
  }
  *abort_word = 1;
  atomicExch(&g_device_error, code);
  return false;
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// hi = the operand rounded to tf32 (exactly what the tensor core then reads); lo = the remainder,
// of which the tensor core keeps the top 10 bits
__device__ __forceinline__ void split4(const float (&v)[4], float4* hi, float4* lo) {
  float h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    unsigned r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v[i]));
    h[i] = __uint_as_float(r);
  }
  *hi = make_float4(h[0], h[1], h[2], h[3]);
  *lo = make_float4(v[0] - h[0], v[1] - h[1], v[2] - h[2], v[3] - h[3]);
}
__device__ __forceinline__ float4 flip4(float4 v, unsigned mask) {
  return make_float4(__uint_as_float(__float_as_uint(v.x) ^ mask), __uint_as_float(__float_as_uint(v.y) ^ mask),
                     __uint_as_float(__float_as_uint(v.z) ^ mask), __uint_as_float(__float_as_uint(v.w) ^ mask));
}

struct TmaArgs {
  // bin x of element (m, k) of A sits at A + (x/a_qb)*a_bs + x%a_qb + m*a_rs + k*a_ks (complex
  // elements): bins in blocks of a_qb (16 or 4); a_qb = a_bs = 16 is the natural bins-innermost layout
  const float2* A;
  long long a_rs, a_ks, a_bs;
  const float2* B;
  long long b_rs, b_ks, b_bs;  // B[n][k][x]
  int a_qb, b_qb;
  int M, N, K, X;
  int d_qb;  // bins per block of D; 0 = bins innermost (store coordinates (2x, m, n, 0) instead of (2*(x % d_qb), m, n, x / d_qb))
  float inv_norm;
  int conjA, conjB, accumulate;
  int n_tiles, m_tiles, total_tiles;
  int use_tma;  // operands arrive by tensor copies (the convolution workspace) instead of 16-byte cp.async copies
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1) cgemm_tma_kernel(const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_a,
                                                                const __grid_constant__ CUtensorMap map_b, TmaArgs g) {
  using C = Cfg<BN>;
  constexpr int NR = C::NR, NH = C::NH, NACC = C::NACC;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* raw_mem = smem_raw;
  unsigned char* conv_mem = smem_raw + C::OFF_CONV;
  unsigned char* epi_mem = smem_raw + C::OFF_EPI;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem_raw + C::OFF_BAR);
  // barrier indices
  constexpr int RAW_FULL = 0, RAW_FREE = NR, CV_FULL = 2 * NR, CV_FREE = 2 * NR + NH, ACC_FULL = 2 * NR + 2 * NH,
                ACC_FREE = ACC_FULL + 2, NBARS = ACC_FREE + 2;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + NBARS);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto bar = [&](int i) { return smem_u32(bars + i); };

  if (tid == 0) {
    *abort_word = 0;
    for (int i = 0; i < NR; ++i) {
      mbar_init(bar(RAW_FULL + i), g.use_tma ? 1 : kProdThreads);
      mbar_init(bar(RAW_FREE + i), kConvThreads / 32);
    }
    for (int i = 0; i < NH; ++i) {
      mbar_init(bar(CV_FULL + i), kConvThreads / 32);
      mbar_init(bar(CV_FREE + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(ACC_FULL + i), 1);
      mbar_init(bar(ACC_FREE + i), 4);
    }
    fence_async_smem();
  }
  if (warp == kWarpMma) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(C::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;

  const int nsteps = (g.K + KS - 1) / KS;
  // tile t -> (n tile, m tile, bin quad); the loop bounds are the same in every role
  // (the 4 bin quads of a 128-byte line of the operands are the fastest index when the bin count
  // allows it, then n tiles: blocks that run at the same time share operand lines in L2)
  const bool quad_fast = (g.X & 15) == 0;
  auto tile_coords = [&](int t, int* n0, int* m0, int* x0) {
    const int qf = quad_fast ? (t & 3) : 0, u = quad_fast ? (t >> 2) : t;
    *n0 = (u % g.n_tiles) * BN;
    *m0 = ((u / g.n_tiles) % g.m_tiles) * BM;
    const int xr = u / (g.n_tiles * g.m_tiles);
    *x0 = (quad_fast ? xr * 4 + qf : xr) * XB;
  };

  if (warp >= kWarpProd && warp < kWarpMma) {
    // ------------------------------------------------------------------ operand loads
    // Two lanes per 32-byte segment (one row, one k, the tile's 4 bins); every thread issues its
    // share of a raw stage as 16-byte asynchronous copies (zero-filled outside the tensor) and lets
    // the stage's barrier count their completion.  Consecutive segments of a warp follow the
    // direction in which the operand is contiguous (rows or k), so that a warp's copies coalesce
    // into whole 128-byte lines when the layout allows it.
    if (g.use_tma) {
      // One thread, two tensor copies per raw stage: box {32 bytes, rows, 4 values of k} of each operand,
      // zero-filled outside the tensor, written as [k][row][32 B] with the 32-byte swizzle (the two
      // 16-byte halves of a row swap places every 4 rows: the split's reads stay free of bank conflicts).
      // Tensor copies have no per-SM cap on requests in flight; the 16-byte cp.async path below levels
      // off near 32 KB in flight per SM, which is about half of what the HBM latency needs.
      if (tid == kWarpProd * 32) {
        unsigned rs = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < g.total_tiles && ok; t += gridDim.x) {
          int n0, m0, x0;
          tile_coords(t, &n0, &m0, &x0);
          for (int q = 0; q < 2 * nsteps; ++q, ++rs) {
            const unsigned st = rs % NR;
            if (rs >= NR && !wait_bar(bar(RAW_FREE + st), ((rs / NR) - 1) & 1, kErrRawFree, abort_word)) {
              ok = false;
              break;
            }
            const unsigned dst = smem_u32(raw_mem + st * C::RAW);
            mbar_expect_tx(bar(RAW_FULL + st), (unsigned)((BM + BN) * KQ * 32));
            tma_load4(dst, &map_a, 2 * (x0 % g.a_qb), m0, q * KQ, x0 / g.a_qb, bar(RAW_FULL + st));
            tma_load4(dst + C::A_RAW_T, &map_b, 2 * (x0 % g.b_qb), n0, q * KQ, x0 / g.b_qb, bar(RAW_FULL + st));
          }
        }
      }
    } else {
    const int p = tid - kWarpProd * 32, half = p & 1, sp = p >> 1;  // sp in 0..63
    // unit u = i*64 + sp of an operand with R rows: k-fastest (row = u / 4, j = u % 4) or row-fastest
    const bool a_kfast = g.a_ks < g.a_rs, b_kfast = g.b_ks < g.b_rs;
    unsigned rs = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < g.total_tiles && ok; t += gridDim.x) {
      int n0, m0, x0;
      tile_coords(t, &n0, &m0, &x0);
      const float2* pa = g.A + (long long)(x0 / g.a_qb) * g.a_bs + (x0 % g.a_qb) + 2 * half;
      const float2* pb = g.B + (long long)(x0 / g.b_qb) * g.b_bs + (x0 % g.b_qb) + 2 * half;
      for (int q = 0; q < 2 * nsteps; ++q, ++rs) {
        const unsigned st = rs % NR;
        if (rs >= NR && !wait_bar(bar(RAW_FREE + st), ((rs / NR) - 1) & 1, kErrRawFree, abort_word)) {
          ok = false;
          break;
        }
        // the two 16-byte halves of a row's 32 bytes swap places every 4 rows: the split's 16-byte
        // reads of consecutive rows then fall into different banks
        const unsigned dst = smem_u32(raw_mem + st * C::RAW);
#pragma unroll
        for (int i = 0; i < (KQ * BM) / 64; ++i) {
          const int u = i * 64 + sp;
          const int row = a_kfast ? (u >> 2) : (u % BM), j = a_kfast ? (u & 3) : (u / BM);
          const int k = q * KQ + j;
          const bool v = k < g.K && m0 + row < g.M;
          cp_async16(dst + j * C::A_KSTRIDE + row * 32 + ((half ^ ((row >> 2) & 1)) << 4), v ? pa + (long long)(m0 + row) * g.a_rs + (long long)k * g.a_ks : g.A,
                     v ? 16u : 0u);
        }
#pragma unroll
        for (int i = 0; i < (KQ * BN) / 64; ++i) {
          const int u = i * 64 + sp;
          const int row = b_kfast ? (u >> 2) : (u % BN), j = b_kfast ? (u & 3) : (u / BN);
          const int k = q * KQ + j;
          const bool v = k < g.K && n0 + row < g.N;
          cp_async16(dst + C::A_RAW + j * C::B_KSTRIDE + row * 32 + ((half ^ ((row >> 2) & 1)) << 4),
                     v ? pb + (long long)(n0 + row) * g.b_rs + (long long)k * g.b_ks : g.B, v ? 16u : 0u);
        }
        // the barrier receives this thread's arrival once all its copies above have landed
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar(RAW_FULL + st)) : "memory");
      }
    }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const unsigned id_r = instr_desc(2 * BN, false);
      const unsigned id_i = instr_desc(2 * BN, g.conjA != 0);  // conj(A): the Ai products change sign
      unsigned h = 0, it = 0;  // half stages consumed, tiles done
      bool ok = true;
      for (int t = blockIdx.x; t < g.total_tiles && ok; t += gridDim.x, ++it) {
        const unsigned acc = it % NACC;
        if (it >= NACC && !wait_bar(bar(ACC_FREE + acc), ((it / NACC) - 1) & 1, kErrAccFree, abort_word)) {
          ok = false;
          break;
        }
        tc_fence_after();
        for (int s = 0; s < nsteps && ok; ++s) {
          for (int pair = 0; pair < 2; ++pair, ++h) {
            const unsigned buf = h % NH;
            if (!wait_bar(bar(CV_FULL + buf), (h / NH) & 1, kErrCvFull, abort_word)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const unsigned base = smem_u32(conv_mem + buf * C::HSTAGE);
            const unsigned long long da0 = smem_desc(base, C::A_LBO, C::SBO);
            const unsigned long long db0 = smem_desc(base + C::HALF_A, C::B_LBO, C::SBO);
            const unsigned first = (s > 0) ? 1u : 0u;  // the first product into an accumulator overwrites it
#pragma unroll
            for (int binl = 0; binl < 2; ++binl) {
              const unsigned d = tmem_base + acc * C::ACC_COLS + (pair * 2 + binl) * (2 * BN);
              const unsigned long long a_rh = da0 + (unsigned long long)((((binl * 2 + 0) * 2 + 0) * C::A_TILE) >> 4);
              const unsigned long long a_rl = da0 + (unsigned long long)((((binl * 2 + 0) * 2 + 1) * C::A_TILE) >> 4);
              const unsigned long long a_ih = da0 + (unsigned long long)((((binl * 2 + 1) * 2 + 0) * C::A_TILE) >> 4);
              const unsigned long long a_il = da0 + (unsigned long long)((((binl * 2 + 1) * 2 + 1) * C::A_TILE) >> 4);
              const unsigned long long t_h = db0 + (unsigned long long)(((binl * 2 + 0) * C::B_TILE) >> 4);  // S'_hi
              const unsigned long long t_l = db0 + (unsigned long long)(((binl * 2 + 1) * C::B_TILE) >> 4);  // S'_lo
              const unsigned long long s_h = t_h + (unsigned long long)(((BN / 8) * 128) >> 4);              // S_hi
              const unsigned long long s_l = t_l + (unsigned long long)(((BN / 8) * 128) >> 4);              // S_lo
              mma_tf32(d, a_rh, s_h, id_r, first);
              mma_tf32(d, a_ih, t_h, id_i, 1u);
              mma_tf32(d, a_rh, s_l, id_r, 1u);
              mma_tf32(d, a_ih, t_l, id_i, 1u);
              mma_tf32(d, a_rl, s_h, id_r, 1u);
              mma_tf32(d, a_il, t_h, id_i, 1u);
            }
            mma_commit(bar(CV_FREE + buf));  // frees the half stage when these MMAs retire
          }
        }
        if (ok) mma_commit(bar(ACC_FULL + acc));  // all products of the tile retired: epilogue may read
      }
    }
    __syncwarp();
  } else if (warp >= kWarpEpi) {
    // ------------------------------------------------------------------ epilogue
    const int lq = warp & 3;  // the quarter of the tensor-memory lanes this warp may read
    unsigned char* stag = epi_mem + (warp - kWarpEpi) * C::EPI_WARP;
    const unsigned stag_u32 = smem_u32(stag);
    unsigned it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < g.total_tiles && ok; t += gridDim.x, ++it) {
      int n0, m0, x0;
      tile_coords(t, &n0, &m0, &x0);
      const unsigned acc = it % NACC;
      if (!wait_bar(bar(ACC_FULL + acc), (it / NACC) & 1, kErrAccFull, abort_word)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int dx = g.d_qb ? 2 * (x0 % g.d_qb) : 2 * x0, db = g.d_qb ? x0 / g.d_qb : 0;
      const int mrow = m0 + lq * 32;
      const int ncols = (g.N - n0 < BN) ? g.N - n0 : BN;
      const int nch = (mrow < g.M) ? (ncols + 3) / 4 : 0;  // chunks of 4 columns this warp stores
      const unsigned tacc = tmem_base + ((unsigned)(lq * 32) << 16) + acc * C::ACC_COLS;
      auto load_chunk = [&](int c, float (&v)[XB][2][4]) {
#pragma unroll
        for (int bin = 0; bin < XB; ++bin) {
#pragma unroll
          for (int part = 0; part < 2; ++part) tmem_ld4(tacc + bin * (2 * BN) + part * BN + c * 4, v[bin][part]);
        }
      };
      // this warp's reads of the accumulators are complete: the next tile may overwrite them
      auto release = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(ACC_FREE + acc));
      };
      auto emit = [&](const float (&v)[XB][2][4], int c) {
        // the previous store of this warp must have finished reading the staging buffer
        if (lane == 0) bulk_wait_read();
        __syncwarp();
        unsigned char* buf = stag;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float4* dst = reinterpret_cast<float4*>(buf + (j * 32 + lane) * 32);
          dst[0] = make_float4(v[0][0][j] * g.inv_norm, v[0][1][j] * g.inv_norm, v[1][0][j] * g.inv_norm,
                               v[1][1][j] * g.inv_norm);
          dst[1] = make_float4(v[2][0][j] * g.inv_norm, v[2][1][j] * g.inv_norm, v[3][0][j] * g.inv_norm,
                               v[3][1][j] * g.inv_norm);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (g.accumulate) {
            tma_reduce_add4(&map_d, dx, mrow, n0 + c * 4, db, stag_u32);
          } else {
            tma_store4(&map_d, dx, mrow, n0 + c * 4, db, stag_u32);
          }
          bulk_commit();
        }
      };
      if (nch == 0) {
        release();
      } else {
        // two register sets: the accumulator reads of the next chunk fly while this one is stored
        float va[XB][2][4], vb[XB][2][4];
        load_chunk(0, va);
#pragma unroll 1
        for (int c = 0; c < nch; c += 2) {
          tmem_ld_wait();
          if (c + 1 < nch) load_chunk(c + 1, vb); else release();
          emit(va, c);
          if (c + 1 < nch) {
            tmem_ld_wait();
            if (c + 2 < nch) load_chunk(c + 2, va); else release();
            emit(vb, c + 1);
          }
        }
      }
    }
    if (lane == 0) bulk_wait_all();
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ converters (warps 0-7)
    const int a_row = tid % BM, a_kq = tid / BM;            // A: 128 rows x 2 k-quads
    const int bt = tid % 128, b_sel = tid / 128;            // B: (row, k-quad) units, one bin of the pair each
    const bool has_b = bt < 2 * BN;
    const int b_row = bt % BN, b_kq = (bt / BN) & 1;
    const unsigned a_dst = (unsigned)(a_kq * C::A_LBO + (a_row / 8) * 128 + (a_row % 8) * 16);
    const unsigned b_dst = (unsigned)(b_kq * C::B_LBO + (b_row / 8) * 128 + (b_row % 8) * 16);
    const unsigned s_mask = g.conjB ? 0x80000000u : 0u;  // sign of the imaginary part of B
    constexpr int G = (BN / 8) * 128;                    // bytes between the blocks of a B stack
    unsigned rs = 0, h = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < g.total_tiles && ok; t += gridDim.x) {
      for (int s = 0; s < nsteps && ok; ++s, rs += 2) {
        const unsigned st0 = rs % NR, st1 = (rs + 1) % NR;
        if (!wait_bar(bar(RAW_FULL + st0), (rs / NR) & 1, kErrRawFull, abort_word) ||
            !wait_bar(bar(RAW_FULL + st1), ((rs + 1) / NR) & 1, kErrRawFull, abort_word)) {
          ok = false;
          break;
        }
        const unsigned char* ra = raw_mem + (a_kq ? st1 : st0) * C::RAW;
        const unsigned char* rb = raw_mem + (b_kq ? st1 : st0) * C::RAW + (g.use_tma ? C::A_RAW_T : C::A_RAW);
        const int a_kst = g.use_tma ? BM * 32 : C::A_KSTRIDE, b_kst = g.use_tma ? BN * 32 : C::B_KSTRIDE;
        // Everything this thread needs of the two raw stages goes to registers first and the stages are
        // handed back at once: the copies of the k-step after next start while this one is still being
        // split, instead of after it (FFT-128 layer: 335 -> 308 us per contraction).
        float4 va[2][4];  // [pair][j]: k = 4*a_kq + j, (bin0.re, bin0.im, bin1.re, bin1.im) of the pair
        float2 vb[2][4];  // [pair][j]: (re, im) of bin 2*pair + b_sel
#pragma unroll
        for (int pair = 0; pair < 2; ++pair) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            va[pair][j] = *reinterpret_cast<const float4*>(ra + j * a_kst + a_row * 32 + ((pair ^ ((a_row >> 2) & 1)) << 4));
            vb[pair][j] = has_b ? *reinterpret_cast<const float2*>(rb + j * b_kst + b_row * 32 + ((pair ^ ((b_row >> 2) & 1)) << 4) + b_sel * 8)
                                : make_float2(0.f, 0.f);
          }
        }
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bar(RAW_FREE + st0));
          mbar_arrive(bar(RAW_FREE + st1));
        }
#pragma unroll
        for (int pair = 0; pair < 2; ++pair, ++h) {
          const unsigned buf = h % NH;
          // the MMAs that read this half stage NH half steps ago must have retired
          if (h >= NH && !wait_bar(bar(CV_FREE + buf), ((h / NH) - 1) & 1, kErrCvFree, abort_word)) {
            ok = false;
            break;
          }
          unsigned char* cst = conv_mem + buf * C::HSTAGE;
          {
            const float4(&v)[4] = va[pair];
#pragma unroll
            for (int c = 0; c < 4; ++c) {  // c = binl*2 + part
              const float w[4] = {c == 0 ? v[0].x : c == 1 ? v[0].y : c == 2 ? v[0].z : v[0].w,
                                  c == 0 ? v[1].x : c == 1 ? v[1].y : c == 2 ? v[1].z : v[1].w,
                                  c == 0 ? v[2].x : c == 1 ? v[2].y : c == 2 ? v[2].z : v[2].w,
                                  c == 0 ? v[3].x : c == 1 ? v[3].y : c == 2 ? v[3].z : v[3].w};
              float4 hi, lo;
              split4(w, &hi, &lo);
              unsigned char* tdst = cst + (c * 2) * C::A_TILE + a_dst;
              *reinterpret_cast<float4*>(tdst) = hi;
              *reinterpret_cast<float4*>(tdst + C::A_TILE) = lo;
            }
          }
          if (has_b) {
            const float2(&v)[4] = vb[pair];
            const float wr[4] = {v[0].x, v[1].x, v[2].x, v[3].x}, wi[4] = {v[0].y, v[1].y, v[2].y, v[3].y};
            float4 brh, brl, bih, bil;
            split4(wr, &brh, &brl);
            split4(wi, &bih, &bil);
            bih = flip4(bih, s_mask);  // s Bi
            bil = flip4(bil, s_mask);
            unsigned char* tdst = cst + C::HALF_A + (b_sel * 2) * C::B_TILE + b_dst;
            *reinterpret_cast<float4*>(tdst) = flip4(bih, 0x80000000u);  // hi stack: [-s Bi | Br | s Bi]
            *reinterpret_cast<float4*>(tdst + G) = brh;
            *reinterpret_cast<float4*>(tdst + 2 * G) = bih;
            *reinterpret_cast<float4*>(tdst + C::B_TILE) = flip4(bil, 0x80000000u);  // lo stack
            *reinterpret_cast<float4*>(tdst + C::B_TILE + G) = brl;
            *reinterpret_cast<float4*>(tdst + C::B_TILE + 2 * G) = bil;
          }
          fence_async_smem();  // generic-proxy writes -> visible to the tensor core
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(CV_FULL + buf));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kWarpMma) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS));
  }
}

// ---------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encoder() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 4-D view of a tensor whose bin x of element (row, k) sits at p + (x/qb)*bs + x%qb + row*rs + k*ks
// complex elements: (floats of a block's bins, rows, k, blocks).  bs == qb is the natural
// bins-innermost layout, seen as one "block" holding all X bins.
bool make_map(CUtensorMap* m, const float* p, long long rs, long long ks, long long bs, int qb, int rows, int kcount,
              int X, int box_rows, int box_k, bool swizzle32 = false) {
  EncodeTiledFn enc = encoder();
  if (!enc) return false;
  const bool blocked = bs != qb;
  const cuuint64_t dims[4] = {(cuuint64_t)(blocked ? 2 * qb : 2 * X), (cuuint64_t)rows, (cuuint64_t)kcount,
                              (cuuint64_t)(blocked ? X / qb : 1)};
  const cuuint64_t strides[3] = {(cuuint64_t)rs * 8, (cuuint64_t)ks * 8, (cuuint64_t)(blocked ? bs * 8 : (long long)X * 8)};
  const cuuint32_t box[4] = {8, (cuuint32_t)box_rows, (cuuint32_t)box_k, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(p), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN>
int launch_tma(const CUtensorMap& md, const CUtensorMap& ma, const CUtensorMap& mb, TmaArgs a, cudaStream_t s) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(cgemm_tma_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::SMEM);
    configured[dev] = true;
  }
  a.n_tiles = (a.N + BN - 1) / BN;
  a.m_tiles = (a.M + BM - 1) / BM;
  const long long total = (long long)a.n_tiles * a.m_tiles * (a.X / XB);
  a.total_tiles = (int)total;
  // one persistent block per SM; a caller that runs collectives beside the contraction can keep some
  // SMs free for them (a block fills an SM's shared memory, so nothing else starts there before it ends)
  const int sms = sm_count() - contraction_reserved_sms();
  const int cap = sms > 1 ? sms : 1;
  const int grid = total < cap ? (int)total : cap;
  cgemm_tma_kernel<BN><<<grid, kThreads, Cfg<BN>::SMEM, s>>>(md, ma, mb, a);
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

}  // namespace

// fp32 tensor map without swizzle or interleave, zero fill outside the tensor (shared with the
// transforms that stage zero-padded images by tensor copies); false when the driver lacks the encoder
bool encode_tensor_map_f32(void* map, const float* base, int rank, const unsigned long long* dims,
                           const unsigned long long* strides_bytes, const unsigned* box, int swizzle_bytes) {
  EncodeTiledFn enc = encoder();
  if (!enc || rank < 1 || rank > 5) return false;
  cuuint64_t d[5], st[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) d[i] = dims[i], bx[i] = box[i], es[i] = 1;
  for (int i = 0; i + 1 < rank; ++i) st[i] = strides_bytes[i];
  return enc(static_cast<CUtensorMap*>(map), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<float*>(base), d, st,
             bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
             swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : (swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE),
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool cgemm_tma_supported(const float* a, long long a_rs, long long a_ks, long long a_bs, const float* b, long long b_rs,
                         long long b_ks, long long b_bs, const float* d, long long d_ms, long long d_ns, long long d_bs,
                         int d_qb, int M, int N, int K, int X) {
  if (X % 4 != 0 || M < 1 || N < 1 || K < 1) return false;
  if (d_qb < 4 || d_qb % 4 != 0 || (d_bs != d_qb && X % d_qb != 0)) return false;
  // tensor copies: 16-byte aligned bases and strides (an even number of complex elements)
  const long long st[9] = {a_rs, a_ks, a_bs, b_rs, b_ks, b_bs, d_ms, d_ns, d_bs};
  for (long long v : st)
    if (v <= 0 || v % 2 != 0 || v * 8 >= (1LL << 40)) return false;
  if (!aligned16(a) || !aligned16(b) || !aligned16(d)) return false;
  if ((long long)((N + 15) / 16) * ((M + BM - 1) / BM) * (X / 4) > 0x7fffffffLL) return false;
  return encoder() != nullptr;
}

int cgemm_tma(const float* a, long long a_rs, long long a_ks, bool conjA, const float* b, long long b_rs, long long b_ks,
              bool conjB, float* d, long long d_ms, long long d_ns, int M, int N, int K, int X, float inv_norm,
              bool accumulate, cudaStream_t s, long long a_bs, long long b_bs, long long d_bs, int a_qb, int b_qb, int d_qb) {
  // column tile: 16 / 32 for small n; otherwise 48 when that pads less than 64 (e.g. n = 96)
  const int BN = N <= 16 ? 16 : (N <= 32 ? 32 : (((N + 47) / 48) * 48 < ((N + 63) / 64) * 64 ? 48 : 64));
  alignas(64) CUtensorMap md;
  if (!make_map(&md, d, d_ms, d_ns, d_bs, d_qb, M, N, X, 32, 4)) {
    return -1;  // the caller falls back to the gather kernel
  }
  TmaArgs t;
  t.A = reinterpret_cast<const float2*>(a), t.a_rs = a_rs, t.a_ks = a_ks, t.a_bs = a_bs;
  t.B = reinterpret_cast<const float2*>(b), t.b_rs = b_rs, t.b_ks = b_ks, t.b_bs = b_bs;
  t.M = M, t.N = N, t.K = K, t.X = X, t.inv_norm = inv_norm;
  t.a_qb = a_qb, t.b_qb = b_qb;
  t.d_qb = (d_bs != d_qb) ? d_qb : 0;
  t.conjA = conjA, t.conjB = conjB, t.accumulate = accumulate;
  t.n_tiles = t.m_tiles = t.total_tiles = 0;
  // operands in 4-bin blocks (the convolution workspace) arrive by tensor copies
  alignas(64) CUtensorMap ma, mb;
  std::memset(&ma, 0, sizeof(ma));
  std::memset(&mb, 0, sizeof(mb));
#ifndef FBFFT_OPERAND_TMA
#define FBFFT_OPERAND_TMA 1
#endif
  t.use_tma = FBFFT_OPERAND_TMA && a_qb == XB && b_qb == XB && a_bs != a_qb && b_bs != b_qb &&
              make_map(&ma, a, a_rs, a_ks, a_bs, a_qb, M, K, X, BM, KQ, true) &&
              make_map(&mb, b, b_rs, b_ks, b_bs, b_qb, N, K, X, BN, KQ, true);
  if (BN == 16) return launch_tma<16>(md, ma, mb, t, s);
  if (BN == 32) return launch_tma<32>(md, ma, mb, t, s);
  if (BN == 48) return launch_tma<48>(md, ma, mb, t, s);
  return launch_tma<64>(md, ma, mb, t, s);
}

int read_device_error_tma() { return device_error_word_read(); }
int clear_device_error_tma() { return device_error_word_clear(); }

}  // namespace fbfft_b200
