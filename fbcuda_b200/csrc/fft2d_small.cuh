// Warp-level building blocks of the N in {8, 16, 32} 2-D transforms, shared by the
// batched FFT kernels (fft2d_small.cu) and the tile-list convolution kernel
// (conv_iterated.cu).  A warp handles IPW = 32/(N/2) images at a time; lane
// (li, l) = (lane / (N/2), lane % (N/2)) works on image li.  Between the passes an
// image lives in shared memory as (N/2+1) rows of N complex values, row pitch RS,
// image pitch IS (float2 units).
#pragma once
#include "common.cuh"
#include "fft_regs.cuh"

namespace fbfft_b200 {

// Pitches chosen by exhaustive search so that the 8-byte column accesses of pass A,
// the 16-byte row accesses of pass B and 16-byte row copies are free of bank
// conflicts (N = 8 keeps a 2-way conflict on the row accesses).
template <int N>
struct SmallCfg;
template <>
struct SmallCfg<8> {
  static constexpr int RS = 8, IS = 44;
};
template <>
struct SmallCfg<16> {
  static constexpr int RS = 18, IS = 168;
};
template <>
struct SmallCfg<32> {
  static constexpr int RS = 34, IS = 578;
};

template <int N>
__device__ __forceinline__ void load_row16(const float2* row, float2 (&v)[N]) {
#pragma unroll
  for (int c = 0; c < N; c += 2) {
    const float4 t = *reinterpret_cast<const float4*>(row + c);
    v[c] = make_float2(t.x, t.y);
    v[c + 1] = make_float2(t.z, t.w);
  }
}

// Columns l and l+N/2 of the N x N canvas of one image, read from `src` (global or
// shared, generic address) with row stride sy and element stride sx; rows/columns
// outside the h x w image read as zero (MemoryAccess.cuh:19-25).
template <int N>
__device__ __forceinline__ void load_columns(const float* src, long long sy, long long sx, int h, int w, int padL,
                                             int padU, bool valid, int l, float2 (&a)[N]) {
  constexpr int T = N / 2;
  const unsigned x0 = (unsigned)(l - padL), x1 = (unsigned)(l + T - padL);
  const bool ok0 = valid && x0 < (unsigned)w, ok1 = valid && x1 < (unsigned)w;
  const float* p0 = src + (long long)x0 * sx - (long long)padU * sy;
  const float* p1 = src + (long long)x1 * sx - (long long)padU * sy;
#pragma unroll
  for (int y = 0; y < N; ++y) {
    const bool oky = (unsigned)(y - padU) < (unsigned)h;
    a[y].x = (oky && ok0) ? p0[(long long)y * sy] : 0.f;
    a[y].y = (oky && ok1) ? p1[(long long)y * sy] : 0.f;
  }
}

// The same for an image staged in shared memory with row pitch w (32-bit offsets): one uniform
// bounds test per row, and lanes whose column lies outside the image read a zero word through a
// zero stride instead of carrying a predicate.  `zero` points at a float that holds 0.
template <int N>
__device__ __forceinline__ void load_columns_staged(const float* src, const float* zero, int h, int w, int padL, int padU,
                                                    int l, float2 (&a)[N]) {
  constexpr int T = N / 2;
  const unsigned x0 = (unsigned)(l - padL), x1 = (unsigned)(l + T - padL);
  const bool ok0 = x0 < (unsigned)w, ok1 = x1 < (unsigned)w;
  const int s0 = ok0 ? w : 0, s1 = ok1 ? w : 0;
  const float* p0 = ok0 ? src + (int)x0 - padU * w : zero;
  const float* p1 = ok1 ? src + (int)x1 - padU * w : zero;
#pragma unroll
  for (int y = 0; y < N; ++y) {
    a[y] = make_float2(0.f, 0.f);
    if ((unsigned)(y - padU) < (unsigned)h) {
      a[y].x = p0[y * s0];
      a[y].y = p1[y * s1];
    }
  }
}

// The same for a contiguous N x N image without padding: compile-time offsets, no predicates.
template <int N>
__device__ __forceinline__ void load_columns_full(const float* src, int l, float2 (&a)[N]) {
  constexpr int T = N / 2;
#pragma unroll
  for (int y = 0; y < N; ++y) {
    a[y].x = src[y * N + l];
    a[y].y = src[y * N + l + T];
  }
}

// Pass A tail: a[] holds the bit-reversed transform Z of (column l) + i (column
// l+T).  Separates A = (Z[r] + conj Z[N-r])/2 and B = (Z[r] - conj Z[N-r])/2i and
// writes rows 0..T-1 of both columns; rows 0 and N/2 are real and share row 0 as
// (re, im).
template <int N>
__device__ __forceinline__ void fwd_separate_store(float2 (&a)[N], float2* ib, int l) {
  constexpr int T = N / 2, RS = SmallCfg<N>::RS;
  {
    const float2 z0 = a[0], zh = a[brev(N / 2, N)];
    ib[l] = make_float2(z0.x, zh.x);
    ib[l + T] = make_float2(z0.y, zh.y);
  }
  static_for<T - 1>([&](auto rc) {
    constexpr int r = decltype(rc)::value + 1;
    const float2 zr = a[brev(r, N)], zm = a[brev(N - r, N)];
    ib[r * RS + l] = make_float2(0.5f * (zr.x + zm.x), 0.5f * (zr.y - zm.y));
    ib[r * RS + l + T] = make_float2(0.5f * (zr.y + zm.y), 0.5f * (zm.x - zr.x));
  });
}

// Pass B (in place): transform of packed row l along x, then row 0 is unpacked into
// rows 0 and N/2.  Leaves the finished [N/2+1][N] block in ib.  Warp-synchronous:
// every lane of the warp must call it.
template <int N>
__device__ __forceinline__ void fwd_rows_unpack(float2* ib, int l) {
  constexpr int T = N / 2, RS = SmallCfg<N>::RS;
  {
    float2 v[N];
    load_row16<N>(ib + l * RS, v);
    fft_bitrev<N, false>(v);
    static_for<N / 2>([&](auto cc) {
      constexpr int c = decltype(cc)::value * 2;
      const float2 p = v[brev(c, N)], q = v[brev(c + 1, N)];
      *reinterpret_cast<float4*>(ib + l * RS + c) = make_float4(p.x, p.y, q.x, q.y);
    });
  }
  __syncwarp();
  {
    // lane l owns the pair (kx, N-kx), kx = l; lane 0 owns the self-paired 0 and N/2
    const int k0 = (l == 0) ? 0 : l, k1 = (l == 0) ? T : N - l;
    const float2 va = ib[k0], vb = ib[k1];
    const float2 ma = (l == 0) ? va : vb;  // V[(N-k0)%N]
    const float2 mb = (l == 0) ? vb : va;  // V[(N-k1)%N]
    ib[k0] = make_float2(0.5f * (va.x + ma.x), 0.5f * (va.y - ma.y));
    ib[T * RS + k0] = make_float2(0.5f * (va.y + ma.y), 0.5f * (ma.x - va.x));
    ib[k1] = make_float2(0.5f * (vb.x + mb.x), 0.5f * (vb.y - mb.y));
    ib[T * RS + k1] = make_float2(0.5f * (vb.y + mb.y), 0.5f * (mb.x - vb.x));
  }
  __syncwarp();
}

// Inverse, first half (in place): rows 0 and N/2 are packed into row 0 as
// F[0] + i F[N/2] (the imaginary parts of F[0][0] and F[N/2][0] carry nothing and
// are dropped, fbfft/FFT2D32.cuh:313-315), then packed row l is inverse transformed
// along kx.  Warp-synchronous.
template <int N>
__device__ __forceinline__ void inv_pack_rows(float2* ib, int l) {
  constexpr int T = N / 2, RS = SmallCfg<N>::RS;
  {
    const int k0 = l, k1 = l + T;
    const float2 a0 = ib[k0], h0 = ib[T * RS + k0], a1 = ib[k1], h1 = ib[T * RS + k1];
    ib[k0] = (l == 0) ? make_float2(a0.x, h0.x) : make_float2(a0.x - h0.y, a0.y + h0.x);
    ib[k1] = make_float2(a1.x - h1.y, a1.y + h1.x);
  }
  __syncwarp();
  {
    float2 v[N];
    load_row16<N>(ib + l * RS, v);
    fft_bitrev<N, true, true>(v);
    static_for<N / 2>([&](auto cc) {
      constexpr int c = decltype(cc)::value * 2;
      const float2 p = v[brev(c, N)], q = v[brev(c + 1, N)];
      *reinterpret_cast<float4*>(ib + l * RS + c) = make_float4(p.x, p.y, q.x, q.y);
    });
  }
  __syncwarp();
}

// Inverse, second half: columns l and l+T.  Z[r] = G_l[r] + i G_{l+T}[r] with the
// Hermitian extension G[N-r] = conj G[r]; afterwards z[brev(y, N)] = N*N * (P[y][l],
// P[y][l+T]).
template <int N>
__device__ __forceinline__ void inv_columns_load(const float2* ib, int l, float2 (&z)[N]) {
  constexpr int T = N / 2, RS = SmallCfg<N>::RS;
  {
    const float2 g0 = ib[l], g1 = ib[l + T];
    z[0] = make_float2(g0.x, g1.x);
    z[N / 2] = make_float2(g0.y, g1.y);
  }
  static_for<T - 1>([&](auto rc) {
    constexpr int r = decltype(rc)::value + 1;
    const float2 g0 = ib[r * RS + l], g1 = ib[r * RS + l + T];
    z[r] = make_float2(g0.x - g1.y, g0.y + g1.x);
    z[N - r] = make_float2(g0.x + g1.y, g1.x - g0.y);
  });
}
template <int N>
__device__ __forceinline__ void inv_columns(const float2* ib, int l, float2 (&z)[N]) {
  inv_columns_load<N>(ib, l, z);
  fft_bitrev<N, true, true>(z);
}

// Cropped store of the two columns held in z (see inv_columns), scaled by `mul`.
template <int N>
__device__ __forceinline__ void store_columns(float* dst, long long sy, long long sx, int h, int w, int padL, int padU,
                                              int l, const float2 (&z)[N], float mul) {
  constexpr int T = N / 2;
  const unsigned x0 = (unsigned)(l - padL), x1 = (unsigned)(l + T - padL);
  const bool ok0 = x0 < (unsigned)w, ok1 = x1 < (unsigned)w;
  float* p0 = dst + (long long)x0 * sx - (long long)padU * sy;
  float* p1 = dst + (long long)x1 * sx - (long long)padU * sy;
  static_for<N>([&](auto yc) {
    constexpr int y = decltype(yc)::value;
    if ((unsigned)(y - padU) < (unsigned)h) {
      const float2 t = z[brev(y, N)];
      if (ok0) p0[(long long)y * sy] = t.x * mul;
      if (ok1) p1[(long long)y * sy] = t.y * mul;
    }
  });
}

// The same for a contiguous N x N output without crop offset.
template <int N>
__device__ __forceinline__ void store_columns_full(float* dst, int l, const float2 (&z)[N]) {
  constexpr int T = N / 2;
  static_for<N>([&](auto yc) {
    constexpr int y = decltype(yc)::value;
    const float2 t = z[brev(y, N)];
    dst[y * N + l] = t.x;
    dst[y * N + l + T] = t.y;
  });
}

// ---------------------------------------------------------------- async bulk copies
// cp.async.bulk (the untiled TMA path) with mbarrier completion.  Addresses must be
// 16-byte aligned and sizes multiples of 16 bytes.  Waits are bounded: a wait that
// runs out records an error code in g_device_error and the caller abandons its work.
// one copy per translation unit (no relocatable device code); the unit that waits exports a reader
// and a clearer built from the two helpers below
static __device__ int g_device_error = 0;

static inline int device_error_word_read() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_device_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}
static inline int device_error_word_clear() {
  const int zero = 0;
  return cudaMemcpyToSymbol(g_device_error, &zero, sizeof(int)) == cudaSuccess ? 0 : -1;
}

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try(unsigned bar, unsigned parity) {
  // try_wait suspends the thread in hardware until the phase completes or a time limit expires
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// true when the phase completed; false (after recording `code`) when `max_tries` suspended
// attempts went by without it (each try_wait parks the thread for a hardware-defined slice of
// time, so the bound is a time bound; fbfft_b200_selftest_bounded_wait measures the slice).
// Every wait of the library goes through here or through the contraction's wait_bar, which is
// bounded by the nanosecond timer and an abort word shared by the block's roles.
constexpr int kWaitMaxTries = 1 << 20;
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int code, int max_tries = kWaitMaxTries) {
  for (int i = 0; i < max_tries; ++i) {
    if (mbar_try(bar, parity)) return true;
  }
  atomicExch(&g_device_error, code);
  return false;
}
__device__ __forceinline__ void bulk_g2s(unsigned dst_smem, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, unsigned src_smem, unsigned bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until this thread's bulk stores have finished READING shared memory
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}  // namespace fbfft_b200
