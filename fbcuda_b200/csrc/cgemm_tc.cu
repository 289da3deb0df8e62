// Per-frequency-bin complex contraction on the 5th-generation tensor cores
// (tcgen05.mma, kind::tf32, accumulators in tensor memory) with a 3xTF32 split that
// keeps fp32 accuracy.  Same math as cgemm_bins.cu / the reference's transposeMM
// (MM-inl.cuh:188-196):
//
//   D[m][n][x] (+)= inv_norm * sum_k opA(A[m][k][x]) * opB(B[n][k][x]),  x = frequency bin,
//
// op = identity or complex conjugate.  Callers map the three convolution passes onto it
// with the plane dimension as m and the batch as n, so that m fills the 128 rows of the
// MMA even when the batch per GPU is small.
//
// A block owns 4 consecutive bins (32 contiguous bytes of every operand element -- one
// DRAM sector -- so loads stay sector-efficient although bins are the innermost index of
// the tensors), one 128-row tile of m and one tile of BN columns of n.  Per k-step of 8:
//   * every thread gathers 4 consecutive k of one operand row for the 4 bins (two 16-byte
//     loads per element), splits each fp32 into hi = top 19 bits and lo = x - hi, and
//     writes real and imaginary parts of every bin as separate K-major operand tiles in
//     the tensor core's canonical no-swizzle shared-memory layout (8 x 16-byte core
//     matrices);
//   * one thread issues, per bin, 4 real products (re*re, im*im -> Re D; re*im, im*re ->
//     Im D; signs and conjugations through the instruction descriptor's negate bits)
//     times 3 split terms (hi*hi, hi*lo, lo*hi) = 12 MMAs of 128 x BN x 8 into the bin's
//     two accumulators in tensor memory, then commits to an mbarrier that frees the
//     shared-memory stage; two stages alternate so gathering overlaps the MMAs.
// The epilogue reads the accumulators with tcgen05.ld, interleaves re/im of the 4 bins
// into 32 contiguous bytes per (m, n) and stores them scaled by inv_norm.
// Every mbarrier wait is bounded; a wait that runs out records an error, and the block
// still releases its tensor memory before returning.
#include "fft2d_small.cuh"  // mbarrier helpers, fence_async_smem
#include "kernels.h"

namespace fbfft_b200 {

namespace {

constexpr int kProducers = 256;           // gather / split / epilogue threads (8 warps)
constexpr int kTcThreads = kProducers + 32;  // plus one warp that only issues MMAs
constexpr int BM = 128;   // rows of m per block
constexpr int XB = 4;     // bins per block
constexpr int KS = 8;     // k per stage (one tf32 MMA)
enum : int { kErrTcStageWait = 201, kErrTcFinalWait = 202 };

__device__ __forceinline__ unsigned long long smem_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
  // K-major, no swizzle: 8-row x 16-byte core matrices; LBO between the two 16-byte k-chunks
  // of an 8-wide k-step, SBO between 8-row groups; version 1 (bits 46-47)
  return (unsigned long long)((addr >> 4) & 0x3FFF) | ((unsigned long long)((lbo_bytes >> 4) & 0x3FFF) << 16) |
         ((unsigned long long)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ULL << 46);
}

__device__ __forceinline__ unsigned instr_desc(int n, bool neg_a, bool neg_b) {
  // D fp32, A and B tf32, both K-major, M = 128
  return (1u << 4) | (2u << 7) | (2u << 10) | ((neg_a ? 1u : 0u) << 13) | ((neg_b ? 1u : 0u) << 14) |
         ((unsigned)(n >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
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
__device__ __forceinline__ void tmem_ld8(unsigned taddr, float (&v)[8]) {
  unsigned r0, r1, r2, r3, r4, r5, r6, r7;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3), "=r"(r4), "=r"(r5), "=r"(r6), "=r"(r7)
               : "r"(taddr));
  v[0] = __uint_as_float(r0), v[1] = __uint_as_float(r1), v[2] = __uint_as_float(r2), v[3] = __uint_as_float(r3);
  v[4] = __uint_as_float(r4), v[5] = __uint_as_float(r5), v[6] = __uint_as_float(r6), v[7] = __uint_as_float(r7);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

struct TcArgs {
  const float2* A;
  long long a_rs, a_ks;  // A[m][k][x] at A + m*a_rs + k*a_ks + x   (complex elements)
  const float2* B;
  long long b_rs, b_ks;  // B[n][k][x]
  float2* D;
  long long d_ms, d_ns;  // D[m][n][x]
  int M, N, K, X;
  float inv_norm;
  int conjA, conjB, accumulate;
};

// hi = the operand rounded to tf32 (10-bit mantissa, low 13 bits zero: exactly what the
// tensor core then reads); lo = the remainder, of which the tensor core keeps the top 10 bits
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

template <int BN>
__global__ void __launch_bounds__(kTcThreads, 1) cgemm_tc_kernel(TcArgs g) {
  constexpr int A_TILE = BM * KS * 4;            // bytes of one (bin, part, split) tile of A
  constexpr int B_TILE = BN * KS * 4;
  constexpr int A_STAGE = XB * 2 * 2 * A_TILE;   // 4 bins x (re, im) x (hi, lo)
  constexpr int B_STAGE = XB * 2 * 2 * B_TILE;
  constexpr int STAGE = A_STAGE + B_STAGE;
  constexpr int A_LBO = (BM / 8) * 128, B_LBO = (BN / 8) * 128, SBO = 128;
  constexpr int TMEM_COLS = 512;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* stage_mem = smem_raw;
  // [0],[1] stage filled (256 producer arrivals), [2],[3] stage free (MMA commit), [4] all MMAs done
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem_raw + 2 * STAGE);
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 5);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int x0 = blockIdx.x * XB, m0 = blockIdx.y * BM, n0 = blockIdx.z * BN;

  if (tid == 0) {
    mbar_init(smem_u32(bars + 0), kProducers);
    mbar_init(smem_u32(bars + 1), kProducers);
    mbar_init(smem_u32(bars + 2), 1);
    mbar_init(smem_u32(bars + 3), 1);
    mbar_init(smem_u32(bars + 4), 1);
    fence_async_smem();
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;

  // ---- gather roles: every thread owns one (row, k-quad) unit of A; threads < 2*BN also one of B
  const int a_row = tid % BM, a_kq = (tid / BM) & 1;     // kq in {0, 1}
  const bool has_b = tid < 2 * BN;
  const int b_row = tid % BN, b_kq = tid / BN;
  const bool a_row_ok = m0 + a_row < g.M, b_row_ok = has_b && (n0 + b_row < g.N);
  const float2* a_src = g.A + (long long)(m0 + a_row) * g.a_rs + x0;
  const float2* b_src = g.B + (long long)(n0 + b_row) * g.b_rs + x0;
  const unsigned a_dst = (unsigned)(a_kq * A_LBO + (a_row / 8) * 128 + (a_row % 8) * 16);
  const unsigned b_dst = (unsigned)(b_kq * B_LBO + (b_row / 8) * 128 + (b_row % 8) * 16);

  float4 ra[4][2], rb[4][2];  // [k in quad][bins 0-1 | bins 2-3] = (re, im, re, im)
  auto gather = [&](int k0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int ka = k0 + a_kq * 4 + j, kb = k0 + b_kq * 4 + j;
      if (a_row_ok && ka < g.K) {
        const float4* p = reinterpret_cast<const float4*>(a_src + (long long)ka * g.a_ks);
        ra[j][0] = __ldg(p);
        ra[j][1] = __ldg(p + 1);
      } else {
        ra[j][0] = ra[j][1] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      if (b_row_ok && kb < g.K) {
        const float4* p = reinterpret_cast<const float4*>(b_src + (long long)kb * g.b_ks);
        rb[j][0] = __ldg(p);
        rb[j][1] = __ldg(p + 1);
      } else {
        rb[j][0] = rb[j][1] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  };
  // component c of a float4 (compile-time c)
  auto comp = [](const float4& v, int c) { return c == 0 ? v.x : (c == 1 ? v.y : (c == 2 ? v.z : v.w)); };
  auto scatter = [&](unsigned char* st) {
#pragma unroll
    for (int bin = 0; bin < XB; ++bin) {
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        const int c = (bin & 1) * 2 + part, h = bin >> 1;
        float4 hi, lo;
        {
          const float v[4] = {comp(ra[0][h], c), comp(ra[1][h], c), comp(ra[2][h], c), comp(ra[3][h], c)};
          split4(v, &hi, &lo);
          unsigned char* t = st + ((bin * 2 + part) * 2) * A_TILE + a_dst;
          *reinterpret_cast<float4*>(t) = hi;
          *reinterpret_cast<float4*>(t + A_TILE) = lo;
        }
        if (has_b) {
          const float v[4] = {comp(rb[0][h], c), comp(rb[1][h], c), comp(rb[2][h], c), comp(rb[3][h], c)};
          split4(v, &hi, &lo);
          unsigned char* t = st + A_STAGE + ((bin * 2 + part) * 2) * B_TILE + b_dst;
          *reinterpret_cast<float4*>(t) = hi;
          *reinterpret_cast<float4*>(t + B_TILE) = lo;
        }
      }
    }
  };

  const int nsteps = (g.K + KS - 1) / KS;
  bool ok = true;
  if (warp == kProducers / 32) {
    // ---- MMA warp: one lane issues; it never touches operands, only descriptors
    if (lane == 0) {
      const unsigned long long a_desc0 = smem_desc(smem_u32(stage_mem), A_LBO, SBO);
      const unsigned long long b_desc0 = smem_desc(smem_u32(stage_mem) + A_STAGE, B_LBO, SBO);
      const unsigned idesc_pos = instr_desc(BN, false, false), idesc_neg = instr_desc(BN, true, false);
      // (A part, B part, target): Re D = Ar*Br -/+ Ai*Bi, Im D = +/- Ar*Bi +/- Ai*Br;
      // conj(A) flips the sign of Ai, conj(B) of Bi
      const unsigned id1 = !(g.conjA ^ g.conjB) ? idesc_neg : idesc_pos;  // Ai*Bi
      const unsigned id2 = g.conjB ? idesc_neg : idesc_pos;               // Ar*Bi
      const unsigned id3 = g.conjA ? idesc_neg : idesc_pos;               // Ai*Br
      unsigned full_phase[2] = {0, 0};
      for (int s = 0; s < nsteps && ok; ++s) {
        const int buf = s & 1;
        if (!mbar_wait(smem_u32(bars + buf), full_phase[buf], kErrTcStageWait)) {
          ok = false;
          break;
        }
        full_phase[buf] ^= 1;
        tc_fence_after();
        const unsigned long long da0 = a_desc0 + (unsigned long long)((buf * STAGE) >> 4);
        const unsigned long long db0 = b_desc0 + (unsigned long long)((buf * STAGE) >> 4);
#pragma unroll
        for (int bin = 0; bin < XB; ++bin) {
          const unsigned d_re = tmem_base + bin * (2 * BN), d_im = d_re + BN;
#pragma unroll
          for (int term = 0; term < 4; ++term) {
            const int pa = (term == 1 || term == 3) ? 1 : 0;   // 0 = re, 1 = im
            const int pb = (term == 1 || term == 2) ? 1 : 0;
            const unsigned d = (term < 2) ? d_re : d_im;
            const unsigned idesc = term == 0 ? idesc_pos : (term == 1 ? id1 : (term == 2 ? id2 : id3));
#pragma unroll
            for (int sp = 0; sp < 3; ++sp) {
              const int sa_split = (sp == 2) ? 1 : 0, sb_split = (sp == 1) ? 1 : 0;  // hi*hi, hi*lo, lo*hi
              const unsigned long long da = da0 + (unsigned long long)((((bin * 2 + pa) * 2 + sa_split) * A_TILE) >> 4);
              const unsigned long long db = db0 + (unsigned long long)((((bin * 2 + pb) * 2 + sb_split) * B_TILE) >> 4);
              // the first product into each accumulator overwrites it
              const unsigned acc = (s > 0 || (term & 1) || sp > 0) ? 1u : 0u;
              mma_tf32(d, da, db, idesc, acc);
            }
          }
        }
        mma_commit(smem_u32(bars + 2 + buf));                 // frees the stage when these MMAs retire
        if (s == nsteps - 1) mma_commit(smem_u32(bars + 4));  // and, after the last step, releases the epilogue
      }
    }
    __syncwarp();
  } else {
    // ---- producers
    unsigned free_phase[2] = {0, 0};
    gather(0);
    for (int s = 0; s < nsteps; ++s) {
      const int buf = s & 1;
      unsigned char* st = stage_mem + buf * STAGE;
      if (s >= 2 && ok) {
        // the MMAs that read this stage two steps ago must have retired
        if (!mbar_wait(smem_u32(bars + 2 + buf), free_phase[buf], kErrTcStageWait)) ok = false;
        free_phase[buf] ^= 1;
      }
      scatter(st);
      if (s + 1 < nsteps) gather((s + 1) * KS);  // next step's loads fly while this step's MMAs run
      fence_async_smem();                        // generic-proxy writes -> visible to the tensor core
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bars + buf)) : "memory");
    }
    // ---- epilogue: all MMAs done -> tensor memory -> global
    if (ok && !mbar_wait(smem_u32(bars + 4), 0, kErrTcFinalWait)) ok = false;
    tc_fence_after();
    if (ok) {
      const int lq = warp & 3, ch = warp >> 2;            // lane quarter of tensor memory, column half
      const int m = m0 + lq * 32 + lane;
      constexpr int CHUNKS = BN / 16;                     // 8-column chunks per column half
#pragma unroll 1
      for (int cc = 0; cc < CHUNKS; ++cc) {
        const int col = ch * (BN / 2) + cc * 8;
        float v[XB][2][8];
#pragma unroll
        for (int bin = 0; bin < XB; ++bin) {
#pragma unroll
          for (int part = 0; part < 2; ++part) {
            tmem_ld8(tmem_base + ((unsigned)(lq * 32) << 16) + bin * (2 * BN) + part * BN + col, v[bin][part]);
          }
        }
        tmem_ld_wait();
        if (m < g.M) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int n = n0 + col + j;
            if (n < g.N) {
              float4* dst = reinterpret_cast<float4*>(g.D + (long long)m * g.d_ms + (long long)n * g.d_ns + x0);
              float4 o0 = make_float4(v[0][0][j] * g.inv_norm, v[0][1][j] * g.inv_norm, v[1][0][j] * g.inv_norm,
                                      v[1][1][j] * g.inv_norm);
              float4 o1 = make_float4(v[2][0][j] * g.inv_norm, v[2][1][j] * g.inv_norm, v[3][0][j] * g.inv_norm,
                                      v[3][1][j] * g.inv_norm);
              if (g.accumulate) {
                const float4 p0 = dst[0], p1 = dst[1];
                o0.x += p0.x, o0.y += p0.y, o0.z += p0.z, o0.w += p0.w;
                o1.x += p1.x, o1.y += p1.y, o1.z += p1.z, o1.w += p1.w;
              }
              dst[0] = o0;
              dst[1] = o1;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
}

template <int BN>
constexpr int tc_smem_bytes() {
  return 2 * (XB * 2 * 2 * (BM * KS * 4) + XB * 2 * 2 * (BN * KS * 4)) + 64;
}

template <int BN>
int launch_tc(const TcArgs& a, cudaStream_t s) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(cgemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc_smem_bytes<BN>());
    configured[dev] = true;
  }
  dim3 grid(a.X / XB, (a.M + BM - 1) / BM, (a.N + BN - 1) / BN);
  cgemm_tc_kernel<BN><<<grid, kTcThreads, tc_smem_bytes<BN>(), s>>>(a);
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

int g_mode = 0;  // 0 auto (tensor cores when the operands qualify), 1 FP32 CUDA cores only

}  // namespace

void set_contraction_mode(int mode) { g_mode = mode; }
int contraction_mode() { return g_mode; }

bool cgemm_tc_supported(const float* a, long long a_rs, long long a_ks, const float* b, long long b_rs, long long b_ks,
                        const float* d, long long d_ms, long long d_ns, int M, int N, int K, int X) {
  if (g_mode != 0) return false;
  if (X % XB != 0 || M < 1 || N < 1 || K < 1) return false;
  // 32-byte aligned bin quads: bases 16-byte aligned, every stride a multiple of 2 complex
  const long long st[6] = {a_rs, a_ks, b_rs, b_ks, d_ms, d_ns};
  for (long long v : st)
    if (v % 2 != 0) return false;
  if (!aligned16(a) || !aligned16(b) || !aligned16(d)) return false;
  const long long grid_y = (M + BM - 1) / BM, grid_z = (N + 15) / 16;
  if (grid_y > 65535 || grid_z > 65535) return false;
  // small problems are not worth a 128-row tile
  return (long long)M * N * K >= 16 * 16 * 8;
}

// D[m][n][x] (+)= inv_norm * sum_k opA(A[m][k][x]) opB(B[n][k][x]); strides in complex elements
int cgemm_tc(const float* a, long long a_rs, long long a_ks, bool conjA, const float* b, long long b_rs, long long b_ks,
             bool conjB, float* d, long long d_ms, long long d_ns, int M, int N, int K, int X, float inv_norm,
             bool accumulate, cudaStream_t s) {
  TcArgs t;
  t.A = reinterpret_cast<const float2*>(a), t.a_rs = a_rs, t.a_ks = a_ks;
  t.B = reinterpret_cast<const float2*>(b), t.b_rs = b_rs, t.b_ks = b_ks;
  t.D = reinterpret_cast<float2*>(d), t.d_ms = d_ms, t.d_ns = d_ns;
  t.M = M, t.N = N, t.K = K, t.X = X, t.inv_norm = inv_norm;
  t.conjA = conjA, t.conjB = conjB, t.accumulate = accumulate;
  if (N <= 16) return launch_tc<16>(t, s);
  if (N <= 32) return launch_tc<32>(t, s);
  return launch_tc<64>(t, s);
}

int read_device_error_tc() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_device_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace fbfft_b200
