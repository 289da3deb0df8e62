// Batched 1-D real-to-complex / complex-to-real FFTs for N = 8 ... 64 on contiguous tensors
// (fbfft1D / fbifft1D, fbfft/FBFFT.cuh:11-23; the reference's warp-level kernels are
// fbfft/FBFFT-inl.cuh:19-150 over fbfft/FBFFTCommon.cuh:307-430).
//
// As in the reference two real signals travel as the real and imaginary part of one complex
// line and are separated afterwards (fbfft/FBFFTCommon.cuh:323-350,397-429).  Here a thread holds
// the whole line in registers (fully unrolled length-N FFT with compile-time twiddles,
// fft_regs.cuh) and a warp never synchronises with other warps:
//   task     32 consecutive signal pairs = 64 signals, owned by one warp
//   forward  one cp.async.bulk brings the task's 64*N floats into the warp's slot (completion on
//            the warp's mbarrier, bounded wait; at N = 64 one copy per lane, to a conflict-free
//            pitch); lane t reads pair t with 16-byte loads, transforms,
//            separates the two spectra and writes them back into the slot at the pitch of the
//            output tensor, 2*(N+2) floats per pair, which is free of bank conflicts; the slot
//            leaves through one bulk store.
//   inverse  the mirror image: one bulk load of 32 * 2*(N+2) floats, Z = A + iB rebuilt with its
//            Hermitian half in registers, unnormalised inverse FFT, one bulk store of 64*N floats.
// Rows that are narrower than N or not adjacent in memory (zero-padded images of the two-call row
// pass, signals with a stride between them, a left pad; all in 16-byte units) take the RAGGED
// variants of the same kernels: one bulk copy per row, the zeros around it written by the lane
// (forward); one bulk store per row of the columns that are kept (inverse).
// Leftover signals (B mod 64) and every other shape go through the shared-memory line kernels.
#include "fft2d_small.cuh"  // bulk-copy / mbarrier helpers
#include "coop_fft.cuh"
#include "fft_regs.cuh"
#include "kernels.h"

namespace fbfft_b200 {

namespace {

enum : int { kErrFft1dWait = 105 };

template <int N>
struct Fast1dCfg {  // slots per warp, warps per block, resident blocks per SM, per-lane input copies
  static constexpr int NSLOT = 2, WARPS = 4, BLOCKS = 3;
  static constexpr bool PADIN = false;
};
template <>
struct Fast1dCfg<8> {
  static constexpr int NSLOT = 2, WARPS = 8, BLOCKS = 4;
  static constexpr bool PADIN = false;
};
template <>
struct Fast1dCfg<16> {
  static constexpr int NSLOT = 2, WARPS = 8, BLOCKS = 3;
  static constexpr bool PADIN = false;
};
template <>
struct Fast1dCfg<64> {
  static constexpr int NSLOT = 1, WARPS = 4, BLOCKS = 3;
  static constexpr bool PADIN = true  /* measured: 0.80 -> 0.88; no gain at N = 32 */;
};

template <int N>
constexpr int slot_floats() {
  return 32 * (2 * N + 4);
}
template <int N>
constexpr int fast1d_smem() {
  return Fast1dCfg<N>::WARPS * (Fast1dCfg<N>::NSLOT * slot_floats<N>() * 4 + 16);
}

// RAGGED (forward): the rows are not one dense [rows][N] array but rows of w <= N floats inside a zero
// canvas -- zero-padded images of the two-call protocol (row g is canvas row g % rpi of image g / rpi,
// image row (g % rpi) - padU), signals with a stride between them, or a left pad.  Every lane brings in
// its pair's two rows with one bulk copy each (w * 4 bytes, to column padL of its region) and writes the
// zeros around them itself; rows outside the image are all zeros and cost no copy.
struct RaggedIn {
  const float* p;
  long long sb, sy;  // floats between images and between image rows
  int h, w, padL, padU, rpi;
};

// the two rows (2 * pair, 2 * pair + 1) of a pair: source pointers or nullptr for rows outside the image
__device__ __forceinline__ void ragged_rows(const RaggedIn& rg, long long pair, const float* (&src)[2]) {
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const long long g = 2 * pair + r;
    const long long b = g / rg.rpi;
    const int y = (int)(g % rg.rpi) - rg.padU;
    src[r] = ((unsigned)y < (unsigned)rg.h) ? rg.p + b * rg.sb + (long long)y * rg.sy : nullptr;
  }
}
// zeros of a pair's region (two rows of N floats) that the copies leave untouched
template <int N>
__device__ __forceinline__ void ragged_zero(const RaggedIn& rg, float* region, const float* const (&src)[2]) {
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float4* row = reinterpret_cast<float4*>(region + r * N);
    const int lo = src[r] ? rg.padL / 4 : N / 4, hi = src[r] ? (rg.padL + rg.w) / 4 : N / 4;
    for (int i = 0; i < lo; ++i) row[i] = z;
    for (int i = hi; i < N / 4; ++i) row[i] = z;
  }
}

// INV = false: src real [tasks*64][N], dst complex [tasks*64][N/2+1][2];  INV = true: the reverse
template <int N, bool INV, bool RAGGED = false>
__global__ void __launch_bounds__(Fast1dCfg<N>::WARPS * 32, Fast1dCfg<N>::BLOCKS)
    fft1d_fast_kernel(const float* __restrict__ src, float* __restrict__ dst, long long tasks, RaggedIn rg) {
  constexpr int NSLOT = Fast1dCfg<N>::NSLOT, WARPS = Fast1dCfg<N>::WARPS;
  constexpr int PC = 2 * N + 4, PR = 2 * N;          // floats per pair: complex side, real side
  constexpr int PIN = INV ? PC : PR, POUT = INV ? PR : PC;
  constexpr int SLOT = slot_floats<N>();
  extern __shared__ __align__(16) float smem1d[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* slots = smem1d + warp * NSLOT * SLOT;
  const unsigned bars = smem_u32(smem1d + WARPS * NSLOT * SLOT) + warp * 16;
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < NSLOT; ++i) mbar_init(bars + 8 * i, 1);
  }
  fence_async_smem();
  __syncwarp();
  const long long gw = (long long)blockIdx.x * WARPS + warp, nw = (long long)gridDim.x * WARPS;
  // PADIN (forward): every lane copies its own pair to the output pitch, so that the 16-byte reads
  // below are free of bank conflicts (the dense layout puts all lanes on the same four banks)
  constexpr bool PADIN = !INV && (Fast1dCfg<N>::PADIN || RAGGED);
  auto issue = [&](long long task, int slot) {
    if constexpr (RAGGED && INV) {
      bulk_wait_read();  // this lane's rows of the slot's previous result have left
      __syncwarp();
    }
    if constexpr (RAGGED && !INV) {
      const float* rows[2];
      ragged_rows(rg, task * 32 + lane, rows);
      float* region = slots + slot * SLOT + lane * PC;
      if (lane == 0) bulk_wait_read();  // the slot's previous result has left
      __syncwarp();
      ragged_zero<N>(rg, region, rows);
      const unsigned mine = ((rows[0] ? 1u : 0u) + (rows[1] ? 1u : 0u)) * (unsigned)rg.w * 4u;
      const unsigned total = __reduce_add_sync(0xffffffffu, mine);
      if (lane == 0) {
        fence_async_smem();
        mbar_expect_tx(bars + 8 * slot, total);
      }
      __syncwarp();
#pragma unroll
      for (int r = 0; r < 2; ++r)
        if (rows[r]) bulk_g2s(smem_u32(region + r * N + rg.padL), rows[r], (unsigned)rg.w * 4u, bars + 8 * slot);
      return;
    }
    if (lane == 0) {
      bulk_wait_read();  // the slot's previous result has left
      fence_async_smem();
      mbar_expect_tx(bars + 8 * slot, 32 * PIN * 4);
      if (!PADIN) bulk_g2s(smem_u32(slots + slot * SLOT), src + task * (32 * PIN), 32 * PIN * 4, bars + 8 * slot);
    }
    if (PADIN) {
      __syncwarp();
      bulk_g2s(smem_u32(slots + slot * SLOT + lane * PC), src + task * (32 * PR) + lane * PR, PR * 4, bars + 8 * slot);
    }
  };
  unsigned phases = 0;
  long long t = gw;
  if (t < tasks) issue(t, 0);
  for (int i = 0; t < tasks; t += nw, ++i) {
    const int slot = (NSLOT == 2) ? (i & 1) : 0;
    if (NSLOT == 2 && t + nw < tasks) issue(t + nw, slot ^ 1);
    if (!mbar_wait(bars + 8 * slot, (phases >> slot) & 1, kErrFft1dWait)) return;
    phases ^= 1u << slot;
    float* base = slots + slot * SLOT;
    float2 a[N];
    if constexpr (!INV) {
      const float4* s0 = reinterpret_cast<const float4*>(base + lane * (PADIN ? PC : PR));
#pragma unroll
      for (int j = 0; j < N / 4; ++j) {
        const float4 u = s0[j], v = s0[N / 4 + j];
        a[4 * j + 0] = make_float2(u.x, v.x);
        a[4 * j + 1] = make_float2(u.y, v.y);
        a[4 * j + 2] = make_float2(u.z, v.z);
        a[4 * j + 3] = make_float2(u.w, v.w);
      }
      __syncwarp();  // the output pitch differs: lanes overwrite one another's input
      fft_bitrev<N, false>(a);
      float* o = base + lane * PC;
      // A[k] = (Z[k] + conj Z[N-k]) / 2 at o[2k], B[k] = (Z[k] - conj Z[N-k]) / 2i at o[N+2+2k]
      auto sepA = [&](int zk, int mk) {
        return make_float2(0.5f * (a[zk].x + a[mk].x), 0.5f * (a[zk].y - a[mk].y));
      };
      auto sepB = [&](int zk, int mk) {
        return make_float2(0.5f * (a[zk].y + a[mk].y), 0.5f * (a[mk].x - a[zk].x));
      };
      static_for<N / 4>([&](auto kc) {
        constexpr int k = 2 * decltype(kc)::value;
        const float2 p = sepA(brev(k, N), brev((N - k) % N, N)), q = sepA(brev(k + 1, N), brev(N - k - 1, N));
        *reinterpret_cast<float4*>(o + 2 * k) = make_float4(p.x, p.y, q.x, q.y);
      });
      *reinterpret_cast<float2*>(o + N) = sepA(brev(N / 2, N), brev(N / 2, N));
      *reinterpret_cast<float2*>(o + N + 2) = sepB(brev(0, N), brev(0, N));
      static_for<N / 4>([&](auto kc) {
        constexpr int k = 2 * decltype(kc)::value + 1;
        const float2 p = sepB(brev(k, N), brev(N - k, N)), q = sepB(brev(k + 1, N), brev(N - k - 1, N));
        *reinterpret_cast<float4*>(o + N + 2 + 2 * k) = make_float4(p.x, p.y, q.x, q.y);
      });
    } else {
      const float* o = base + lane * PC;
      // Z[k] = A[k] + i B[k] for k <= N/2, Z[N-k] = conj A[k] + i conj B[k] for 0 < k < N/2
      auto put = [&](int k, float2 A, float2 Bv) {
        a[k] = make_float2(A.x - Bv.y, A.y + Bv.x);
        if (k > 0 && k < N / 2) a[(N - k) % N] = make_float2(A.x + Bv.y, Bv.x - A.y);
      };
      float2 A[N / 2 + 1], Bv[N / 2 + 1];
      static_for<N / 4>([&](auto kc) {
        constexpr int k = 2 * decltype(kc)::value;
        const float4 u = *reinterpret_cast<const float4*>(o + 2 * k);
        A[k] = make_float2(u.x, u.y), A[k + 1] = make_float2(u.z, u.w);
      });
      A[N / 2] = *reinterpret_cast<const float2*>(o + N);
      Bv[0] = *reinterpret_cast<const float2*>(o + N + 2);
      static_for<N / 4>([&](auto kc) {
        constexpr int k = 2 * decltype(kc)::value + 1;
        const float4 u = *reinterpret_cast<const float4*>(o + N + 2 + 2 * k);
        Bv[k] = make_float2(u.x, u.y), Bv[k + 1] = make_float2(u.z, u.w);
      });
      static_for<N / 2 + 1>([&](auto kc) {
        constexpr int k = decltype(kc)::value;
        put(k, A[k], Bv[k]);
      });
      __syncwarp();
      fft_bitrev<N, true>(a);
      float4* s0 = reinterpret_cast<float4*>(base + lane * PR);
      static_for<N / 4>([&](auto jc) {
        constexpr int j = decltype(jc)::value;
        const float2 z0 = a[brev(4 * j, N)], z1 = a[brev(4 * j + 1, N)], z2 = a[brev(4 * j + 2, N)], z3 = a[brev(4 * j + 3, N)];
        s0[j] = make_float4(z0.x, z1.x, z2.x, z3.x);
        s0[N / 4 + j] = make_float4(z0.y, z1.y, z2.y, z3.y);
      });
    }
    fence_async_smem();
    __syncwarp();
    if constexpr (RAGGED && INV) {
      // every lane stores columns padL .. padL + w - 1 of its pair's two rows where the rows live
      const float* rows[2];
      ragged_rows(rg, t * 32 + lane, rows);
#pragma unroll
      for (int r = 0; r < 2; ++r)
        if (rows[r]) bulk_s2g(const_cast<float*>(rows[r]), smem_u32(base + lane * PR + r * N + rg.padL), (unsigned)rg.w * 4u);
      bulk_commit();
    } else if (lane == 0) {
      bulk_s2g(dst + t * (32 * POUT), smem_u32(base), 32 * POUT * 4);
      bulk_commit();
    }
    if (NSLOT == 1 && t + nw < tasks) issue(t + nw, 0);
  }
  bulk_wait_read();
}

// ---- N = 128, 256: a line shared by Q = N/64 lanes (coop_fft.cuh), 32/Q pairs per warp ------------
// Same slot protocol with one slot per warp.  Forward: one bulk copy per pair to the output pitch;
// lane (q, l) loads its quarter-runs of pair l, the transform leaves Z[Q*k + q] in lane q, the line is
// parked in the pair's own region, every lane separates the bins k = q, q + Q, ... <= N/2 into
// registers and (after the warp has read everything) writes A and B in the output layout; one bulk
// store per task.  Inverse: one bulk load per task, Z[x] rebuilt while loading (mirrored for
// x > N/2), one bulk store per pair.
template <int N>
constexpr int coop1d_smem() {
  return 4 * ((32 / (N / 64)) * (2 * N + 4) * 4 + 16);
}

template <int N, bool INV, bool RAGGED = false>
__global__ void __launch_bounds__(128, 3) fft1d_coop_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                            long long tasks, RaggedIn rg) {
  constexpr int R = 64, Q = N / R, P = R / Q, LP = 32 / Q, WARPS = 4;
  constexpr int PC = 2 * N + 4, PR = 2 * N, SLOT = LP * PC;
  extern __shared__ __align__(16) float smem1d[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, q = lane / LP, l = lane % LP;
  float* slot = smem1d + warp * SLOT;
  float* region = slot + l * PC;
  const unsigned bar = smem_u32(smem1d + WARPS * SLOT) + warp * 16;
  if (lane == 0) mbar_init(bar, 1);
  fence_async_smem();
  __syncwarp();
  float2 lf[Q];
  lane_factors<Q, INV>(q, lf);
  const long long gw = (long long)blockIdx.x * WARPS + warp, nw = (long long)gridDim.x * WARPS;
  auto issue = [&](long long task) {
    if constexpr (RAGGED && !INV) {
      const float* rows[2] = {nullptr, nullptr};
      if (lane == 0) bulk_wait_read();  // the slot's previous result has left
      __syncwarp();
      if (lane < LP) {
        ragged_rows(rg, task * LP + l, rows);
        ragged_zero<N>(rg, region, rows);
      }
      const unsigned mine = lane < LP ? ((rows[0] ? 1u : 0u) + (rows[1] ? 1u : 0u)) * (unsigned)rg.w * 4u : 0u;
      const unsigned total = __reduce_add_sync(0xffffffffu, mine);
      if (lane == 0) {
        fence_async_smem();
        mbar_expect_tx(bar, total);
      }
      __syncwarp();
#pragma unroll
      for (int r = 0; r < 2; ++r)
        if (rows[r]) bulk_g2s(smem_u32(region + r * N + rg.padL), rows[r], (unsigned)rg.w * 4u, bar);
      return;
    }
    if (INV && lane < LP) bulk_wait_read();  // this lane's pair has left the slot
    __syncwarp();
    if (lane == 0) {
      if (!INV) bulk_wait_read();
      fence_async_smem();
      mbar_expect_tx(bar, LP * (INV ? PC : PR) * 4);
      if (INV) bulk_g2s(smem_u32(slot), src + task * SLOT, SLOT * 4, bar);
    }
    if (!INV) {
      __syncwarp();
      if (lane < LP) bulk_g2s(smem_u32(region), src + (task * LP + l) * PR, PR * 4, bar);
    }
  };
  unsigned phase = 0;
  long long t = gw;
  if (t < tasks) issue(t);
  for (; t < tasks; t += nw) {
    if (!mbar_wait(bar, phase, kErrFft1dWait)) return;
    phase ^= 1;
    float2 a[R];
    if constexpr (!INV) {
#pragma unroll
      for (int m = 0; m < Q; ++m) {
#pragma unroll
        for (int j4 = 0; j4 < P / 4; ++j4) {
          const float4 u = *reinterpret_cast<const float4*>(region + P * q + R * m + 4 * j4);
          const float4 v = *reinterpret_cast<const float4*>(region + N + P * q + R * m + 4 * j4);
          a[m * P + 4 * j4 + 0] = make_float2(u.x, v.x);
          a[m * P + 4 * j4 + 1] = make_float2(u.y, v.y);
          a[m * P + 4 * j4 + 2] = make_float2(u.z, v.z);
          a[m * P + 4 * j4 + 3] = make_float2(u.w, v.w);
        }
      }
      coop_fft<N, R, Q, false>(a, q, lf);
      __syncwarp();
      float2* zl = reinterpret_cast<float2*>(region);
      static_for<R>([&](auto kc) {
        constexpr int k = decltype(kc)::value;
        zl[Q * k + q] = a[brev(k, R)];
      });
      __syncwarp();
      // bins k = q + Q*i <= N/2 (a[] is dead from here on)
      constexpr int NB = N / 2 / Q + 1;
      float2 sa[NB], sb[NB];
#pragma unroll
      for (int i = 0; i < NB; ++i) {
        const int k = q + Q * i;
        if (k <= N / 2) {
          const float2 z = zl[k], m = zl[(N - k) & (N - 1)];
          sa[i] = make_float2(0.5f * (z.x + m.x), 0.5f * (z.y - m.y));
          sb[i] = make_float2(0.5f * (z.y + m.y), 0.5f * (m.x - z.x));
        }
      }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < NB; ++i) {
        const int k = q + Q * i;
        if (k <= N / 2) {
          zl[k] = sa[i];
          zl[N / 2 + 1 + k] = sb[i];
        }
      }
    } else {
      const float2* zl = reinterpret_cast<const float2*>(region);
#pragma unroll
      for (int m = 0; m < Q; ++m) {
#pragma unroll
        for (int jl = 0; jl < P; ++jl) {
          const int x = jl + P * q + R * m;
          const bool low = x <= N / 2;
          const int k = low ? x : N - x;
          const float2 A = zl[k], Bv = zl[N / 2 + 1 + k];
          a[m * P + jl] = low ? make_float2(A.x - Bv.y, A.y + Bv.x) : make_float2(A.x + Bv.y, Bv.x - A.y);
        }
      }
      coop_fft<N, R, Q, true>(a, q, lf);
      __syncwarp();
      static_for<R>([&](auto kc) {
        constexpr int k = decltype(kc)::value;
        region[Q * k + q] = a[brev(k, R)].x;
        region[N + Q * k + q] = a[brev(k, R)].y;
      });
    }
    fence_async_smem();
    __syncwarp();
    if (INV) {
      if (lane < LP) {
        if constexpr (RAGGED) {
          const float* rows[2];
          ragged_rows(rg, t * LP + l, rows);
#pragma unroll
          for (int r = 0; r < 2; ++r)
            if (rows[r]) bulk_s2g(const_cast<float*>(rows[r]), smem_u32(region + r * N + rg.padL), (unsigned)rg.w * 4u);
        } else {
          bulk_s2g(dst + (t * LP + l) * PR, smem_u32(region), PR * 4);
        }
        bulk_commit();
      }
    } else if (lane == 0) {
      bulk_s2g(dst + t * SLOT, smem_u32(slot), SLOT * 4);
      bulk_commit();
    }
    if (t + nw < tasks) issue(t + nw);
  }
  bulk_wait_read();
}

template <int N, bool INV, bool RAGGED = false>
int launch_coop1d(const float* src, float* dst, long long tasks, cudaStream_t s, const RaggedIn& rg = RaggedIn{}) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(fft1d_coop_kernel<N, INV, RAGGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, coop1d_smem<N>());
    configured[dev] = true;
  }
  const long long want = (tasks + 3) / 4, cap = (long long)sm_count() * 3;
  fft1d_coop_kernel<N, INV, RAGGED><<<(int)(want < cap ? want : cap), 128, coop1d_smem<N>(), s>>>(src, dst, tasks, rg);
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

template <int N, bool INV, bool RAGGED = false>
int launch_fast(const float* src, float* dst, long long tasks, cudaStream_t s, const RaggedIn& rg = RaggedIn{}) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(fft1d_fast_kernel<N, INV, RAGGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, fast1d_smem<N>());
    configured[dev] = true;
  }
  constexpr int W = Fast1dCfg<N>::WARPS;
  const long long want = (tasks + W - 1) / W, cap = (long long)sm_count() * Fast1dCfg<N>::BLOCKS;
  fft1d_fast_kernel<N, INV, RAGGED><<<(int)(want < cap ? want : cap), W * 32, fast1d_smem<N>(), s>>>(src, dst, tasks, rg);
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

}  // namespace

// contiguous [B][N] real and [B][N/2+1][2] complex tensors, 16-byte aligned, no padding
bool fft1d_fast_supported(int n, const float* real, long long rs0, int rs1, const float* cplx, long long cs0, int cs1,
                          int cs2, int padL) {
  if (n != 8 && n != 16 && n != 32 && n != 64 && n != 128 && n != 256) return false;
  return padL == 0 && rs1 == 1 && rs0 == n && cs2 == 1 && cs1 == 2 && cs0 == n + 2 && aligned16(real) && aligned16(cplx);
}

// signals per task (a warp's unit of work)
int fft1d_fast_group(int n) { return n <= 64 ? 64 : 64 / (n / 64); }

// transforms the first `tasks` * fft1d_fast_group(n) signals
int fft1d_fast(int n, bool inverse, const float* src, float* dst, long long tasks, cudaStream_t s) {
  if (tasks <= 0) return kSuccess;
  switch (n) {
    case 8: return inverse ? launch_fast<8, true>(src, dst, tasks, s) : launch_fast<8, false>(src, dst, tasks, s);
    case 16: return inverse ? launch_fast<16, true>(src, dst, tasks, s) : launch_fast<16, false>(src, dst, tasks, s);
    case 32: return inverse ? launch_fast<32, true>(src, dst, tasks, s) : launch_fast<32, false>(src, dst, tasks, s);
    case 64: return inverse ? launch_fast<64, true>(src, dst, tasks, s) : launch_fast<64, false>(src, dst, tasks, s);
    case 128: return inverse ? launch_coop1d<128, true>(src, dst, tasks, s) : launch_coop1d<128, false>(src, dst, tasks, s);
    case 256: return inverse ? launch_coop1d<256, true>(src, dst, tasks, s) : launch_coop1d<256, false>(src, dst, tasks, s);
    default: return kUnsupportedSize;
  }
}

// Rows of w floats (element stride 1) inside a zero canvas of N columns: image row y of image b at
// p + b*sb + y*sy, placed at canvas row y + padU, column padL; rpi canvas rows per image (N for the 2-D
// row pass, 1 for 1-D signals with h = 1).  Bulk copies need 16-byte units: w, padL, sb, sy multiples of 4
// floats and p aligned.
bool fft1d_fast_ragged_supported(int n, const float* p, long long sb, long long sy, int h, int w, int padL, int padU,
                                 int rpi, const float* cplx) {
  if (n != 8 && n != 16 && n != 32 && n != 64 && n != 128 && n != 256) return false;
  if (w < 4 || w % 4 != 0 || padL < 0 || padL % 4 != 0 || padL + w > n || padU < 0 || h < 1 || rpi < 1) return false;
  if (sb % 4 != 0 || (h > 1 && sy % 4 != 0)) return false;
  return aligned16(p) && aligned16(cplx);
}

// transforms the first `tasks` * fft1d_fast_group(n) canvas rows into dst [rows][N/2+1][2] (contiguous)
int fft1d_fast_ragged(int n, const float* p, long long sb, long long sy, int h, int w, int padL, int padU, int rpi,
                      float* dst, long long tasks, cudaStream_t s) {
  if (tasks <= 0) return kSuccess;
  RaggedIn rg;
  rg.p = p, rg.sb = sb, rg.sy = sy, rg.h = h, rg.w = w, rg.padL = padL, rg.padU = padU, rg.rpi = rpi;
  switch (n) {
    case 8: return launch_fast<8, false, true>(nullptr, dst, tasks, s, rg);
    case 16: return launch_fast<16, false, true>(nullptr, dst, tasks, s, rg);
    case 32: return launch_fast<32, false, true>(nullptr, dst, tasks, s, rg);
    case 64: return launch_fast<64, false, true>(nullptr, dst, tasks, s, rg);
    case 128: return launch_coop1d<128, false, true>(nullptr, dst, tasks, s, rg);
    case 256: return launch_coop1d<256, false, true>(nullptr, dst, tasks, s, rg);
    default: return kUnsupportedSize;
  }
}

// the inverse: src complex [rows][N/2+1][2] (contiguous); columns padL .. padL + w - 1 of every transformed
// row go to the row's place in the real tensor described as above
int fft1d_fast_ragged_inverse(int n, const float* src, float* p, long long sb, long long sy, int h, int w, int padL,
                              int padU, int rpi, long long tasks, cudaStream_t s) {
  if (tasks <= 0) return kSuccess;
  RaggedIn rg;
  rg.p = p, rg.sb = sb, rg.sy = sy, rg.h = h, rg.w = w, rg.padL = padL, rg.padU = padU, rg.rpi = rpi;
  switch (n) {
    case 8: return launch_fast<8, true, true>(src, nullptr, tasks, s, rg);
    case 16: return launch_fast<16, true, true>(src, nullptr, tasks, s, rg);
    case 32: return launch_fast<32, true, true>(src, nullptr, tasks, s, rg);
    case 64: return launch_fast<64, true, true>(src, nullptr, tasks, s, rg);
    case 128: return launch_coop1d<128, true, true>(src, nullptr, tasks, s, rg);
    case 256: return launch_coop1d<256, true, true>(src, nullptr, tasks, s, rg);
    default: return kUnsupportedSize;
  }
}

int read_device_error_fft1d() { return device_error_word_read(); }
int clear_device_error_fft1d() { return device_error_word_clear(); }

}  // namespace fbfft_b200
