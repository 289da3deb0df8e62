// Single-call batched 2-D real-to-complex / complex-to-real FFTs for N = 64 and
// N = 128 on contiguous tensors, in the reference's layout for this size class:
// transposed spectrum [B][kx in 0..N/2][ky in 0..N) (what its two calls,
// fbfft/FBFFT2D-inl.cuh:597-617 then :627-669, leave behind), unnormalised inverse
// with crop at (padU, padL) (fbfft/FBIFFT2D-inl.cuh:529-742).
//
// One block owns one image, which never leaves the SM between the two passes (the
// reference round-trips a [B][N][N/2+1] buffer through HBM).  Every 1-D transform
// is a length-N complex FFT shared by Q = N/32 neighbouring lanes: a radix-Q
// decimation-in-frequency step on each lane's own data, one exchange between the Q
// lanes with __shfl_xor_sync, then an independent 32-point FFT held in each lane's
// registers with compile-time twiddles (fft_regs.cuh).
//   forward  pass A: lanes (q, p) take columns p and p+N/2 as re/im of one complex
//            line (coalesced global loads, zero padding by predicate) and transform
//            along y; all N bins of the line go to shared memory, mid[ky][p];
//            pass B: lanes (q, ky) rebuild row ky of the two real-input spectra from
//            mid[ky][*] and mid[N-ky][*] while loading, transform along x and scatter
//            the result (and its Hermitian mirror) into the transposed output tile;
//            rows ky = 0 and N/2 are real and travel as one complex row.
//            The finished tile leaves through cp.async.bulk row stores.
//   inverse  the same two passes backwards; the spectrum rows arrive through
//            cp.async.bulk copies completing on an mbarrier (bounded wait).
#include <cuda.h>  // CUtensorMap

#include <cstring>

#include "coop_fft.cuh"
#include "fft2d_small.cuh"  // bulk-copy / mbarrier helpers
#include "kernels.h"

namespace fbfft_b200 {

namespace {

enum : int { kErrCoopInvWait = 103, kErrCoopFwdWait = 104 };

template <int N>
struct CoopCfg;
// R: length of the FFT one lane holds in registers; Q = N/R lanes share a line.
template <>
struct CoopCfg<64> {
  static constexpr int R = 64, Q = 1, PM = 34, PO = 66, BLOCKS_PER_SM = 12, MIN_BLOCKS = 10;
};
template <>
struct CoopCfg<128> {
  static constexpr int R = 64, Q = 2, PM = 66, PO = 130, BLOCKS_PER_SM = 3, MIN_BLOCKS = 3;
};

// block-wide barrier; a one-warp block only needs the warp to reconverge
template <int THREADS>
__device__ __forceinline__ void block_sync() {
  if constexpr (THREADS <= 32) {
    __syncwarp();
  } else {
    __syncthreads();
  }
}

// ------------------------------------------------------------------ forward
// IN_BULK: the real input is contiguous with a 16-byte aligned base; each image is staged in
// shared memory by one cp.async.bulk (into the region the image's own mid/tile reuse afterwards).
// FULL (with IN_BULK): the images are N x N with no padding, so pass A reads the staged image
// with compile-time strides and no bounds predicates.
// SMALLW (N = 128, without IN_BULK): images of at most 16 x 16 that sit in the first 16 canvas
// columns (convolution weights).  The column pass is evaluated directly -- thread ky sums the image's
// rows against its 16 twiddles, 16 columns at a time -- instead of transforming 64 column pairs of
// zeros, and the row pass reads only those 16 columns.
// CANVAS (with IN_BULK): zero-padded images whose rows are whole 16-byte units.  One tensor copy
// (cp.async.bulk.tensor, zero fill outside the image) brings the whole N x N canvas of an image
// into shared memory at a compile-time pitch of N + 4 floats: the copy starts at column
// -4 ceil(padL / 4) of the image (a tensor copy's innermost coordinate must sit on a 16-byte
// boundary) and row -padU, so the padding never costs a predicate and pass A reads with
// compile-time strides like FULL.
template <int N, bool IN_BULK, bool FULL = false, bool SMALLW = false, bool CANVAS = false>
__global__ void __launch_bounds__((N / 2) * CoopCfg<N>::Q, CoopCfg<N>::MIN_BLOCKS) fft2d_coop_fwd_kernel(RealView in, float* __restrict__ out,
                                                                                long long out_sb, int B, int padL,
                                                                                int padU, long long blk_planes,
                                                                                const __grid_constant__ CUtensorMap cmap) {
  constexpr int R = CoopCfg<N>::R, Q = CoopCfg<N>::Q, P = R / Q, LP = 32 / Q;
  constexpr int PM = CoopCfg<N>::PM, PO = CoopCfg<N>::PO;
  constexpr int H = N / 2, T = H * Q;
  extern __shared__ __align__(128) float2 smem[];
  float2* mid = smem;   // [N][PM]        pass A -> pass B
  float2* tile = smem;  // [H+1][PO]      pass B -> bulk stores (aliases mid)
  // the packed row's two halves live in the tile's padding columns N (direct) and N + 1 (mirrored),
  // so that every row scatters with the same compile-time stride
  float2* vsd = smem + N;
  float2* vsm = smem + N + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = lane / LP, item = warp * LP + (lane % LP);  // item: column pair p (pass A), row r (pass B)
  float2 lf[Q];
  lane_factors<Q, false>(q, lf);
  // staging (IN_BULK): raw image bytes at the start of the region, mbarrier behind the region
  constexpr int REGION = (N * PM > (H + 1) * PO) ? N * PM : (H + 1) * PO;
  const unsigned bar = smem_u32(smem + REGION);
  const long long img_bytes = (long long)in.h * in.w * 4, total_bytes = img_bytes * B;
  unsigned phase = 0;
  // 16-byte aligned window around image b; false when it would reach past the tensor's end
  auto window = [&](int b, long long* lo, unsigned* bytes) {
    const long long g0 = (long long)b * img_bytes, g1 = g0 + img_bytes;
    *lo = g0 & ~15LL;
    const long long hi = (g1 + 15) & ~15LL;
    *bytes = (unsigned)(hi - *lo);
    return hi <= total_bytes || (total_bytes & 15) == 0;
  };
  bool staged = false;
  constexpr int CP = N + 4;  // canvas pitch (floats)
  auto fetch = [&](int b) {
    if constexpr (CANVAS) {
      staged = true;
      if (threadIdx.x == 0) {
        fence_async_smem();
        mbar_expect_tx(bar, CP * N * 4);
        const int cx = -4 * ((padL + 3) / 4), cy = -padU;
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
                smem_u32(smem)),
            "l"(&cmap), "r"(cx), "r"(cy), "r"(b), "r"(bar)
            : "memory");
      }
      return;
    }
    long long lo;
    unsigned bytes;
    staged = window(b, &lo, &bytes);
    if (staged && threadIdx.x == 0) {
      fence_async_smem();
      mbar_expect_tx(bar, bytes);
      bulk_g2s(smem_u32(smem), reinterpret_cast<const char*>(in.p) + lo, bytes, bar);
    }
  };
  if (IN_BULK) {
    if (threadIdx.x == 0) {
      mbar_init(bar, 1);
      smem[REGION + 1] = make_float2(0.f, 0.f);  // the zero word out-of-image lanes read
    }
    fence_async_smem();
    block_sync<T>();
    if (blockIdx.x < B) fetch(blockIdx.x);
  }

  // SMALLW: behind the region (and its barrier / zero word): the image as [16][16] floats, then N roots
  float* simg = reinterpret_cast<float*>(smem + REGION + 2);
  float2* stw = reinterpret_cast<float2*>(simg + 256);
  if constexpr (SMALLW) {
    static_assert(!SMALLW || (N == 128 && T == N && !IN_BULK && !FULL), "one thread per ky");
    for (int i = threadIdx.x; i < N; i += T) {
      float sn, cs;
      sincospif(-2.0f * (float)i / (float)N, &sn, &cs);
      stw[i] = make_float2(cs, sn);
    }
  }

  for (int b = blockIdx.x; b < B; b += gridDim.x) {
    float2 a[R];
    if constexpr (SMALLW) {
      // ---- pass A by direct evaluation: mid[ky][x] = sum_y img[y][x - padL] w^(ky (y + padU)), x < 16
      const float* src = in.p + (long long)b * in.sb;
      for (int i = threadIdx.x; i < 256; i += T) {
        const int y = i >> 4, xx = (i & 15) - padL;
        simg[i] = (y < in.h && (unsigned)xx < (unsigned)in.w) ? src[(long long)y * in.sy + (long long)xx * in.sx] : 0.f;
      }
      // the previous image's rows may still be leaving the tile that mid aliases
      bulk_wait_read();
      block_sync<T>();
      const int ky = threadIdx.x;
      float2 acc[16];
#pragma unroll
      for (int x = 0; x < 16; ++x) acc[x] = make_float2(0.f, 0.f);
#pragma unroll 4
      for (int y = 0; y < 16; ++y) {
        const float2 w = stw[(ky * (y + padU)) & (N - 1)];
        const float4* row = reinterpret_cast<const float4*>(simg + y * 16);
#pragma unroll
        for (int x4 = 0; x4 < 4; ++x4) {
          const float4 v = row[x4];
          acc[4 * x4 + 0].x += v.x * w.x, acc[4 * x4 + 0].y += v.x * w.y;
          acc[4 * x4 + 1].x += v.y * w.x, acc[4 * x4 + 1].y += v.y * w.y;
          acc[4 * x4 + 2].x += v.z * w.x, acc[4 * x4 + 2].y += v.z * w.y;
          acc[4 * x4 + 3].x += v.w * w.x, acc[4 * x4 + 3].y += v.w * w.y;
        }
      }
#pragma unroll
      for (int x = 0; x < 16; x += 2)
        *reinterpret_cast<float4*>(mid + ky * PM + x) = make_float4(acc[x].x, acc[x].y, acc[x + 1].x, acc[x + 1].y);
      block_sync<T>();
      if (threadIdx.x < 16) {
        // rows 0 and H travel packed: the same combination the butterfly path stores (see below)
        const float2 u = mid[threadIdx.x], v = mid[H * PM + threadIdx.x];
        mid[threadIdx.x] = make_float2(u.x - v.y, u.y + v.x);
        mid[H * PM + threadIdx.x] = make_float2(u.x + v.y, u.y - v.x);
      }
    } else {
      // ---- pass A: columns item and item+H, rows y = jl + P*q + R*m
      const float* src = in.p + (long long)b * in.sb;
      long long sy = in.sy, sx = in.sx;
      int soff = 0;  // float offset of the image inside the staging region
      if (IN_BULK) {
        if (staged) {
          if (!mbar_wait(bar, phase, kErrCoopFwdWait)) return;
          phase ^= 1;
          soff = (int)((((long long)b * img_bytes) & 15) >> 2);
        } else {
          // (the last images of a tensor whose size is not a multiple of 16 bytes) plain copy
          float* st = reinterpret_cast<float*>(smem);
          for (int i = threadIdx.x; i < in.h * in.w; i += T) st[i] = src[i];
          block_sync<T>();
        }
      }
      if constexpr (CANVAS) {
        // canvas column X sits at float X + 4 ceil(padL / 4) - padL of a canvas row
        const float* p0 = reinterpret_cast<const float*>(smem) + item + (4 * ((padL + 3) / 4) - padL) + P * q * CP;
#pragma unroll
        for (int m = 0; m < Q; ++m) {
#pragma unroll
          for (int jl = 0; jl < P; ++jl) {
            a[m * P + jl].x = p0[(jl + R * m) * CP];
            a[m * P + jl].y = p0[(jl + R * m) * CP + H];
          }
        }
      } else if constexpr (FULL) {
        const float* p0 = reinterpret_cast<const float*>(smem) + item + P * q * N;
#pragma unroll
        for (int m = 0; m < Q; ++m) {
#pragma unroll
          for (int jl = 0; jl < P; ++jl) {
            a[m * P + jl].x = p0[(jl + R * m) * N];
            a[m * P + jl].y = p0[(jl + R * m) * N + H];
          }
        }
      } else if constexpr (IN_BULK) {
        // staged image, row pitch in.w, 32-bit offsets: one uniform bounds test per row; lanes whose
        // column lies outside the image read the zero word behind the region through a zero stride
        const float* st = reinterpret_cast<const float*>(smem) + soff;
        const float* zero = reinterpret_cast<const float*>(smem + REGION + 1);  // the float2 behind the mbarrier
        const unsigned x0 = (unsigned)(item - padL), x1 = (unsigned)(item + H - padL);
        const bool ok0 = x0 < (unsigned)in.w, ok1 = x1 < (unsigned)in.w;
        const int s0 = ok0 ? in.w : 0, s1 = ok1 ? in.w : 0;
        const int ybase = P * q - padU;
        const float* p0 = ok0 ? st + (int)x0 + ybase * in.w : zero;
        const float* p1 = ok1 ? st + (int)x1 + ybase * in.w : zero;
#pragma unroll
        for (int m = 0; m < Q; ++m) {
#pragma unroll
          for (int jl = 0; jl < P; ++jl) {
            const int yo = jl + R * m;
            a[m * P + jl] = make_float2(0.f, 0.f);
            if ((unsigned)(ybase + yo) < (unsigned)in.h) {
              a[m * P + jl].x = p0[yo * s0];
              a[m * P + jl].y = p1[yo * s1];
            }
          }
        }
      } else {
        const unsigned x0 = (unsigned)(item - padL), x1 = (unsigned)(item + H - padL);
        const bool ok0 = x0 < (unsigned)in.w, ok1 = x1 < (unsigned)in.w;
        const float* p0 = src + (long long)x0 * sx + (long long)(P * q - padU) * sy;
        const float* p1 = src + (long long)x1 * sx + (long long)(P * q - padU) * sy;
        const int ybase = P * q - padU;
#pragma unroll
        for (int m = 0; m < Q; ++m) {
#pragma unroll
          for (int jl = 0; jl < P; ++jl) {
            const int yo = jl + R * m;
            const bool oky = (unsigned)(ybase + yo) < (unsigned)in.h;
            a[m * P + jl].x = (oky && ok0) ? p0[(long long)yo * sy] : 0.f;
            a[m * P + jl].y = (oky && ok1) ? p1[(long long)yo * sy] : 0.f;
          }
        }
      }
      if (IN_BULK) block_sync<T>();  // the staged image is in registers: mid may overwrite it
      coop_fft<N, R, Q, false>(a, q, lf);
      if (!IN_BULK) {
        // the previous image's rows may still be leaving the tile that mid aliases
        bulk_wait_read();
        block_sync<T>();
      }
      if (q == 0) {
        // Rows ky = 0 and ky = H of a column pair hold four real numbers (sums and
        // alternating sums of two real columns).  Pass B wants them packed as one complex
        // row; store u' = u + i v, v' = u - i v (componentwise as below) so that its general
        // "separate two real spectra" formula yields exactly that packing for row 0.
        const float2 u = a[brev(0, R)], v = a[brev(R / 2, R)];
        a[brev(0, R)] = make_float2(u.x - v.y, u.y + v.x);
        a[brev(R / 2, R)] = make_float2(u.x + v.y, u.y - v.x);
      }
      static_for<R>([&](auto kc) {
        constexpr int k = decltype(kc)::value;
        mid[(Q * k + q) * PM + item] = a[brev(k, R)];
      });
    }
    block_sync<T>();
    {
      // ---- pass B: row item (0 = packed rows 0 and N/2).  The lane needs x = jl + P*q + R*m;
      // x < H comes from the first column of pair p = x, x >= H from the second of p = x - H
      const int r = item;
      const float2* row1 = mid + r * PM;
      const float2* row2 = mid + ((r == 0) ? H : N - r) * PM;
      auto take = [&](float4 u, float4 v, float2& a0, float2& a1, float2& b0, float2& b1) {
        a0 = make_float2(0.5f * (u.x + v.x), 0.5f * (u.y - v.y)), b0 = make_float2(0.5f * (u.y + v.y), 0.5f * (v.x - u.x));
        a1 = make_float2(0.5f * (u.z + v.z), 0.5f * (u.w - v.w)), b1 = make_float2(0.5f * (u.w + v.w), 0.5f * (v.z - u.z));
      };
      if constexpr (SMALLW) {
        // Only canvas columns 0..15 are non-zero (and no column has a partner in the second half): a
        // 128-point transform with 16 inputs is 8 independent 16-point transforms,
        //   X[8 m + s] = sum_n (x[n] w128^(n s)) w16^(n m),  s = 0..7,
        // four per lane of the line's pair (s = 4 q + i), no exchange between the lanes: half the
        // instructions of the 64-point transform per lane plus the radix-2 step and its shuffles.
        static_assert(!SMALLW || (N == 128 && Q == 2), "pruned rows: N = 128");
        float2 x[16];
#pragma unroll
        for (int p = 0; p < 16; p += 2) {
          const float4 u = *reinterpret_cast<const float4*>(row1 + p), v = *reinterpret_cast<const float4*>(row2 + p);
          float2 b0, b1;
          take(u, v, x[p], x[p + 1], b0, b1);
        }
        if (q == 1) {  // s = 4 + i: the factor w128^(4 n) = w32^n of the lane
          static_for<16>([&](auto nc) {
            constexpr int n = decltype(nc)::value;
            x[n] = mul_tw<n, 32, false>(x[n]);
          });
        }
        block_sync<T>();  // every lane has read its part of mid: the tile may overwrite it
        float2* direct = (r == 0) ? vsd : tile + r;
        float2* mirror = (r == 0) ? vsm : tile + (N - r);
        static_for<4>([&](auto ic) {
          constexpr int i = decltype(ic)::value;
          float2 t[16];
          static_for<16>([&](auto nc) {
            constexpr int n = decltype(nc)::value;
            t[n] = mul_tw<n * i, N, false>(x[n]);
          });
          fft_bitrev<16, false, true>(t);
          static_for<16>([&](auto mc) {
            constexpr int m = decltype(mc)::value;
            const int kx = 8 * m + 4 * q + i;
            const float2 v = t[brev(m, 16)];
            if (kx <= H) direct[kx * PO] = v;
            if (kx >= H || kx == 0) mirror[((N - kx) & (N - 1)) * PO] = make_float2(v.x, -v.y);
          });
        });
      } else if constexpr (Q == 1) {
#pragma unroll
        for (int p = 0; p < H; p += 2) {
          const float4 u = *reinterpret_cast<const float4*>(row1 + p), v = *reinterpret_cast<const float4*>(row2 + p);
          take(u, v, a[p], a[p + 1], a[p + H], a[p + H + 1]);
        }
      } else {
#pragma unroll
        for (int m = 0; m < Q / 2; ++m) {
#pragma unroll
          for (int jl = 0; jl < P; jl += 2) {
            const int p = jl + P * q + R * m;
            const float4 u = *reinterpret_cast<const float4*>(row1 + p), v = *reinterpret_cast<const float4*>(row2 + p);
            take(u, v, a[m * P + jl], a[m * P + jl + 1], a[(m + Q / 2) * P + jl], a[(m + Q / 2) * P + jl + 1]);
          }
        }
      }
      // Row r > 0 scatters F[r][kx] to tile[kx][r] (kx <= H) and its Hermitian mirror
      // conj(F[r][kx]) to tile[(N-kx)%N][N-r] (kx >= H or kx == 0).  The packed row 0 does
      // the same into the two halves of the scratch row: vsd[kx] = V[kx], vsm[j] = conj(V[(N-j)%N]).
      if constexpr (!SMALLW) {
        coop_fft<N, R, Q, false, true>(a, q, lf);
        block_sync<T>();  // every lane has read its part of mid: the tile may overwrite it
        float2* direct = (r == 0) ? vsd : tile + r;
        float2* mirror = (r == 0) ? vsm : tile + (N - r);
        static_for<R>([&](auto kc) {
          constexpr int k = decltype(kc)::value;
          const int kx = Q * k + q;
          const float2 v = a[brev(k, R)];
          if (Q * k + Q - 1 <= H || kx <= H) {
            if (kx <= H) direct[kx * PO] = v;
          }
          if (Q * k >= H - (Q - 1) || k == 0) {
            if (kx >= H || kx == 0) mirror[((N - kx) & (N - 1)) * PO] = make_float2(v.x, -v.y);
          }
        });
      }
    }
    block_sync<T>();
    // rows ky = 0 and N/2 from the packed row: V = F[0] + i F[N/2]
    for (int kx = threadIdx.x; kx <= H; kx += T) {
      const float2 v = vsd[kx * PO], cm = vsm[kx * PO];  // V[kx], conj(V[(N-kx)%N])
      tile[kx * PO] = make_float2(0.5f * (v.x + cm.x), 0.5f * (v.y + cm.y));
      tile[kx * PO + H] = make_float2(0.5f * (v.y - cm.y), 0.5f * (cm.x - v.x));
    }
    fence_async_smem();
    block_sync<T>();
    float* dst = out + (long long)b * out_sb;
    if (blk_planes) {
      // 4-bin blocks (contraction operands): 32-byte pieces, planes adjacent; two lanes per piece
      // (thread t keeps its half of the ky quad (t / 2) % QR and walks kx in steps of T / (2 QR): both
      // addresses advance by constants, and four reads are in flight before the first store)
      constexpr int QR = N / 4, KSTEP = T / (2 * QR), ROUNDS = (H + 1 + KSTEP - 1) / KSTEP;
      static_assert(T % (2 * QR) == 0, "a block covers whole stored rows per round");
      const int half = threadIdx.x & 1, quad = (threadIdx.x >> 1) % QR, kx0 = threadIdx.x / (2 * QR);
      const float2* src = tile + kx0 * PO + quad * 4 + half * 2;
      float* dstp = out + ((long long)(kx0 * QR + quad) * blk_planes + b) * 8 + half * 4;
      const long long dstep = (long long)KSTEP * QR * blk_planes * 8;
#pragma unroll 4
      for (int rd = 0; rd < ROUNDS; ++rd) {
        if (kx0 + rd * KSTEP <= H) {
          const float4 v = *reinterpret_cast<const float4*>(src + rd * KSTEP * PO);
          *reinterpret_cast<float4*>(dstp + rd * dstep) = v;
        }
      }
    } else {
      for (int kx = threadIdx.x; kx <= H; kx += T) bulk_s2g(dst + (long long)kx * (2 * N), smem_u32(tile + kx * PO), N * 8);
    }
    bulk_commit();
    if (IN_BULK) {
      // the next image is staged into the region the rows are leaving from
      bulk_wait_read();
      block_sync<T>();
      staged = false;
      if (b + gridDim.x < B) fetch(b + gridDim.x);
    }
  }
  bulk_wait_read();
}

// ------------------------------------------------------------------ inverse
// FULL: the output images are contiguous N x N with no crop offset (compile-time strides, no
// bounds predicates on the stores).  SKIP: small outputs such as weight gradients: a warp none of
// whose columns is kept by the crop skips its column transforms.
// NARROW (with SKIP, N = 128): only columns x < 16 are kept (weight gradients).  The row pass then needs 16
// of the 128 outputs of every line: G[x] = sum_s w128^(s x) T_s[x] with T_s the 16-point inverse transform
// of the inputs kx = 8 m + s -- four values of s per lane of the line's pair, the two partial sums added
// through one shuffle per value -- instead of the 64-point transform per lane with its radix-2 step.
// STAGE: output images with rows, crop offsets and strides in 16-byte units.  The rows of the result are
// parked in the shared memory the spectrum came through and leave by one bulk store per kept row (the
// crop is the store's start column and length) instead of 4-byte stores with bounds tests from every
// lane; the next spectrum is fetched after the stores have read the rows.
template <int N, bool FULL = false, bool SKIP = false, bool NARROW = false, bool STAGE = false>
__global__ void __launch_bounds__((N / 2) * CoopCfg<N>::Q, CoopCfg<N>::MIN_BLOCKS) fft2d_coop_inv_kernel(const float* __restrict__ in,
                                                                                long long in_sb, RealView out, int B,
                                                                                int padL, int padU, long long blk_planes) {
  constexpr int R = CoopCfg<N>::R, Q = CoopCfg<N>::Q, P = R / Q, LP = 32 / Q;
  constexpr int PM = CoopCfg<N>::PM, PO = CoopCfg<N>::PO;
  constexpr int H = N / 2, T = H * Q;
  extern __shared__ __align__(128) float2 smem[];
  constexpr int REGION = (H + 1) * PO > N * PM ? (H + 1) * PO : N * PM;
  float2* tile = smem;  // [H+1][PO]   spectrum rows as stored: tile[kx][ky]
  float2* mid = smem;   // [N][PM]     aliases the tile (consumed before mid is written)
  unsigned long long* bar_mem = reinterpret_cast<unsigned long long*>(smem + REGION);
  const unsigned bar = smem_u32(bar_mem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = lane / LP, item = warp * LP + (lane % LP);
  float2 lf[Q];
  lane_factors<Q, true>(q, lf);
  if (threadIdx.x == 0) mbar_init(bar, 1);
  fence_async_smem();
  block_sync<T>();
  unsigned phase = 0;
  auto fetch = [&](int b) {
    // all threads: earlier reads of the tile are done (caller synchronised)
    fence_async_smem();
    if (threadIdx.x == 0) mbar_expect_tx(bar, (unsigned)((H + 1) * N * 8));
    block_sync<T>();
    if (blk_planes) {
      // row blocks: stored row kx of plane b sits at ((kx * planes + b) * N) complex values
      for (int kx = threadIdx.x; kx <= H; kx += T)
        bulk_g2s(smem_u32(tile + kx * PO), in + ((long long)kx * blk_planes + b) * (2 * N), N * 8, bar);
    } else {
      const float* src = in + (long long)b * in_sb;
      for (int kx = threadIdx.x; kx <= H; kx += T) bulk_g2s(smem_u32(tile + kx * PO), src + (long long)kx * (2 * N), N * 8, bar);
    }
  };
  if (blockIdx.x < B) fetch(blockIdx.x);

  for (int b = blockIdx.x; b < B; b += gridDim.x) {
    float2 a[R];
    if (!mbar_wait(bar, phase, kErrCoopInvWait)) return;
    phase ^= 1;
    // Row 0 of pass B^-1 is the packed pair of rows ky = 0 and ky = H: P[kx] = F[0][kx] + i F[H][kx].
    // Rewrite columns 0 and H of the tile in place, tile[kx][0] = p + i h, tile[kx][H] = p - i h,
    // so that the general Hermitian fetch below (direct from column c1, mirrored and conjugated from
    // column c2) produces P for row 0 when it is pointed at columns (0, H).  The imaginary parts of
    // F[0][0] and F[H][0] carry nothing (both rows are transforms of real sequences) and are dropped.
    for (int kx = threadIdx.x; kx <= H; kx += T) {
      float2 p = tile[kx * PO], h = tile[kx * PO + H];
      if (kx == 0) p.y = 0.f, h.y = 0.f;
      tile[kx * PO] = make_float2(p.x - h.y, p.y + h.x);
      tile[kx * PO + H] = make_float2(p.x + h.y, p.y - h.x);
    }
    block_sync<T>();
    if constexpr (NARROW && N == 64) {
      // N = 64, only columns x < 8 are kept: G[x] = sum_s w64^(s x) T_s[x], T_s the 8-point inverse transform of
      // the inputs kx = 8 m + s (a lane holds a whole line)
      static_assert(!(NARROW && N == 64) || (Q == 1 && !FULL), "narrow outputs at N = 64");
      const int r = item;
      const float2* c1 = tile + r;
      const float2* c2 = tile + ((r == 0) ? H : N - r);
      float2 g[8];
#pragma unroll
      for (int x = 0; x < 8; ++x) g[x] = make_float2(0.f, 0.f);
      static_for<8>([&](auto sc) {
        constexpr int sft = decltype(sc)::value;
        float2 t[8];
        static_for<8>([&](auto mc) {
          constexpr int kx = 8 * decltype(mc)::value + sft;
          if constexpr (kx <= H) {
            t[decltype(mc)::value] = c1[kx * PO];
          } else {
            const float2 u = c2[(N - kx) * PO];
            t[decltype(mc)::value] = make_float2(u.x, -u.y);
          }
        });
        fft_bitrev<8, true, true>(t);
        static_for<8>([&](auto xc) {
          constexpr int x = decltype(xc)::value;
          const float2 v = mul_tw<sft * x, N, true>(t[brev(x, 8)]);
          g[x].x += v.x, g[x].y += v.y;
        });
      });
      block_sync<T>();  // the tile is consumed: mid may overwrite it
      float2* row1 = mid + r * PM;
      float2* row2 = mid + ((r == 0) ? H : N - r) * PM;
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        row1[x] = g[x];
        row2[x] = make_float2(g[x].x, -g[x].y);
      }
    } else if constexpr (NARROW) {
      static_assert(!NARROW || N == 64 || (N == 128 && Q == 2 && SKIP && !FULL), "narrow outputs: N = 128 weight gradients");
      const int r = item;
      const float2* c1 = tile + r;                                  // tile[kx][r]
      const float2* c2 = tile + ((r == 0) ? H : N - r);             // tile[N-kx][(N-r)%N]
      float2 g[16];
#pragma unroll
      for (int x = 0; x < 16; ++x) g[x] = make_float2(0.f, 0.f);
      static_for<4>([&](auto ic) {
        constexpr int i = decltype(ic)::value;
        const int sft = 4 * q + i;
        float2 t[16];
#pragma unroll
        for (int m = 0; m < 16; ++m) {
          const int kx = 8 * m + sft;
          if (kx <= H) {
            t[m] = c1[kx * PO];
          } else {
            const float2 u = c2[(N - kx) * PO];
            t[m] = make_float2(u.x, -u.y);
          }
        }
        fft_bitrev<16, true, true>(t);
        static_for<16>([&](auto xc) {
          constexpr int x = decltype(xc)::value;
          const float2 v = mul_tw<i * x, N, true>(t[brev(x, 16)]);
          g[x].x += v.x, g[x].y += v.y;
        });
      });
      if (q == 1) {  // the lane's factor w128^(4 x) = w32^x
        static_for<16>([&](auto xc) {
          constexpr int x = decltype(xc)::value;
          g[x] = mul_tw<x, 32, true>(g[x]);
        });
      }
#pragma unroll
      for (int x = 0; x < 16; ++x) {
        g[x].x += __shfl_xor_sync(0xffffffffu, g[x].x, LP);
        g[x].y += __shfl_xor_sync(0xffffffffu, g[x].y, LP);
      }
      block_sync<T>();  // the tile is consumed: mid may overwrite it
      // columns x >= 16 (and their partners x + H) are not kept: Z_x[ky] = G_x[ky], Z_x[N-ky] = conj(G_x[ky])
      float2* row1 = mid + r * PM;
      float2* row2 = mid + ((r == 0) ? H : N - r) * PM;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int x = 2 * j + q;
        const float2 v = q ? g[2 * j + 1] : g[2 * j];
        row1[x] = v;
        row2[x] = make_float2(v.x, -v.y);
      }
    } else {
      // ---- pass B^-1: row item along kx = jl + P*q + R*m.
      // F[ky][kx] = tile[kx][ky] for kx <= H, else conj(tile[N-kx][(N-ky)%N]).
      const int r = item;
      const float2* c1 = tile + r;                                  // tile[kx][r]
      const float2* c2 = tile + ((r == 0) ? H : N - r);             // tile[N-kx][(N-r)%N]
#pragma unroll
      for (int m = 0; m < Q; ++m) {
#pragma unroll
        for (int jl = 0; jl < P; ++jl) {
          const int kx = jl + P * q + R * m;
          if (kx <= H) {
            a[m * P + jl] = c1[kx * PO];
          } else {
            const float2 t = c2[(N - kx) * PO];
            a[m * P + jl] = make_float2(t.x, -t.y);
          }
        }
      }
      block_sync<T>();  // the tile is consumed: mid may overwrite it
      coop_fft<N, R, Q, true>(a, q, lf);
      // lane holds G[ky][x] at x = Q*k + q; columns x and x+H share a complex line:
      // Z_p[ky] = G_p[ky] + i G_{p+H}[ky], Z_p[N-ky] = conj(G_p[ky]) + i conj(G_{p+H}[ky]).
      // x + H = Q*(k + R/2) + q sits in the same lane.
      // Row 0 holds the packed pair (G[0], G[H]) = (re, im); it stores the same two combinations
      // into rows 0 and H, and pass A^-1 undoes them after loading.
      float2* row1 = mid + r * PM;
      float2* row2 = mid + ((r == 0) ? H : N - r) * PM;
      static_for<R / 2>([&](auto kc) {
        constexpr int k = decltype(kc)::value;
        const int p = Q * k + q;
        const float2 g0 = a[brev(k, R)], g1 = a[brev(k + R / 2, R)];
        row1[p] = make_float2(g0.x - g1.y, g0.y + g1.x);
        row2[p] = make_float2(g0.x + g1.y, g1.x - g0.y);
      });
    }
    block_sync<T>();
    if constexpr (NARROW && N == 64) {
      // ---- pass A^-1 for the 8 kept columns: 4 lanes a column (16 points each), ky = jl + 4 q4 + 16 m
      const int col = lane & 7, q4 = lane >> 3;
      float2 lf4[4];
      lane_factors<4, true>(q4, lf4);
      float2 c[16];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
#pragma unroll
        for (int jl = 0; jl < 4; ++jl) c[m * 4 + jl] = mid[(jl + 4 * q4 + 16 * m) * PM + col];
      }
      if (q4 == 0) {
        // ky = 0 sits at c[0] and ky = H at c[8] of the q4 = 0 lanes (see the general path below)
        const float2 A = c[0], Bv = c[8];
        c[0] = make_float2(0.5f * (A.x + Bv.x), 0.5f * (A.y + Bv.y));
        c[8] = make_float2(0.5f * (A.y - Bv.y), 0.5f * (Bv.x - A.x));
      }
      block_sync<T>();  // mid is consumed: fetch the next spectrum behind the last transform
      if (b + gridDim.x < B) fetch(b + gridDim.x);
      coop_fft<N, 16, 4, true>(c, q4, lf4);
      const unsigned x0 = (unsigned)(col - padL);
      if (x0 < (unsigned)out.w) {
        float* p0 = out.p + (long long)b * out.sb + (long long)x0 * out.sx + (long long)(q4 - padU) * out.sy;
        static_for<16>([&](auto kc) {
          constexpr int k = decltype(kc)::value;
          if ((unsigned)(4 * k + q4 - padU) < (unsigned)out.h) p0[(long long)(4 * k) * out.sy] = c[brev(k, 16)].x;
        });
      }
    } else if constexpr (NARROW && N == 128) {
      // ---- pass A^-1 for the 16 kept columns: 8 lanes a column (16 points each), ky = jl + 2 q8 + 16 m;
      // every warp takes 4 columns instead of the first warp all 16 with 64 points a lane
      const int col = warp * 4 + (lane & 3), q8 = lane >> 2;
      float2 lf8[8];
      lane_factors<8, true>(q8, lf8);
      float2 c[16];
#pragma unroll
      for (int m = 0; m < 8; ++m) {
#pragma unroll
        for (int jl = 0; jl < 2; ++jl) c[m * 2 + jl] = mid[(jl + 2 * q8 + 16 * m) * PM + col];
      }
      if (q8 == 0) {
        // ky = 0 sits at c[0] and ky = H at c[8] of the q8 = 0 lanes (see the general path below)
        const float2 A = c[0], Bv = c[8];
        c[0] = make_float2(0.5f * (A.x + Bv.x), 0.5f * (A.y + Bv.y));
        c[8] = make_float2(0.5f * (A.y - Bv.y), 0.5f * (Bv.x - A.x));
      }
      block_sync<T>();  // mid is consumed: fetch the next spectrum behind the last transform
      if (b + gridDim.x < B) fetch(b + gridDim.x);
      coop_fft<N, 16, 8, true>(c, q8, lf8);
      const unsigned x0 = (unsigned)(col - padL);
      if (x0 < (unsigned)out.w) {
        float* p0 = out.p + (long long)b * out.sb + (long long)x0 * out.sx + (long long)(q8 - padU) * out.sy;
        static_for<16>([&](auto kc) {
          constexpr int k = decltype(kc)::value;
          if ((unsigned)(8 * k + q8 - padU) < (unsigned)out.h) p0[(long long)(8 * k) * out.sy] = c[brev(k, 16)].x;
        });
      }
    } else {
      // ---- pass A^-1: column pair item along ky = jl + P*q + R*m
#pragma unroll
      for (int m = 0; m < Q; ++m) {
#pragma unroll
        for (int jl = 0; jl < P; ++jl) a[m * P + jl] = mid[(jl + P * q + R * m) * PM + item];
      }
      if (q == 0) {
        // ky = 0 sits at a[0] and ky = H at a[R/2] of the q = 0 lanes: A = (g0.x - g1.y, g0.y + g1.x),
        // B = (g0.x + g1.y, g1.x - g0.y) -> Z[0] = (g0.x, g1.x), Z[H] = (g0.y, g1.y)
        const float2 A = a[0], Bv = a[R / 2];
        a[0] = make_float2(0.5f * (A.x + Bv.x), 0.5f * (A.y + Bv.y));
        a[R / 2] = make_float2(0.5f * (A.y - Bv.y), 0.5f * (Bv.x - A.x));
      }
      block_sync<T>();  // mid is consumed: fetch the next spectrum behind the last transform
      if constexpr (!STAGE) {
        if (b + gridDim.x < B) fetch(b + gridDim.x);
      }
      const unsigned x0 = (unsigned)(item - padL), x1 = (unsigned)(item + H - padL);
      const bool ok0 = x0 < (unsigned)out.w, ok1 = x1 < (unsigned)out.w;
      if constexpr (SKIP) {
        if (__all_sync(0xffffffffu, !ok0 && !ok1)) continue;
      }
      coop_fft<N, R, Q, true>(a, q, lf);
      float* dst = out.p + (long long)b * out.sb;
      if constexpr (STAGE) {
        static_assert(!STAGE || (!FULL && !SKIP && !NARROW), "staged rows: the general crop");
        constexpr int PS = N + 4;  // floats per parked row
        float* rows = reinterpret_cast<float*>(smem);
        static_for<R>([&](auto kc) {
          constexpr int k = decltype(kc)::value;
          const float2 t = a[brev(k, R)];
          rows[(Q * k + q) * PS + item] = t.x;
          rows[(Q * k + q) * PS + item + H] = t.y;
        });
        fence_async_smem();
        block_sync<T>();
        for (int y = threadIdx.x; y < out.h; y += T)
          bulk_s2g(dst + (long long)y * out.sy, smem_u32(rows + (y + padU) * PS + padL), (unsigned)out.w * 4u);
        bulk_commit();
        bulk_wait_read();
        block_sync<T>();
        if (b + gridDim.x < B) fetch(b + gridDim.x);
      } else if constexpr (FULL) {
        float* p0 = dst + item + q * N;
        static_for<R>([&](auto kc) {
          constexpr int k = decltype(kc)::value;
          const float2 t = a[brev(k, R)];
          p0[Q * k * N] = t.x;
          p0[Q * k * N + H] = t.y;
        });
      } else {
        float* p0 = dst + (long long)x0 * out.sx + (long long)(q - padU) * out.sy;
        float* p1 = dst + (long long)x1 * out.sx + (long long)(q - padU) * out.sy;
        static_for<R>([&](auto kc) {
          constexpr int k = decltype(kc)::value;
          if ((unsigned)(Q * k + q - padU) < (unsigned)out.h) {
            const float2 t = a[brev(k, R)];
            if (ok0) p0[(long long)(Q * k) * out.sy] = t.x;
            if (ok1) p1[(long long)(Q * k) * out.sy] = t.y;
          }
        });
      }
    }
  }
}

// ------------------------------------------------------------------ convolution weights, N = 128, 4 planes a block
// Images of at most 16 x 16 at the canvas' origin into the contraction's 4-bin blocks.  In that layout the
// 32-byte piece (kx, 4 consecutive ky) of plane p sits between the same pieces of planes p - 1 and p + 1, so
// a block that transforms one plane writes isolated 32-byte sectors `planes * 32` bytes apart.  Here a block
// of 8 warps takes 4 adjacent planes and stores whole 128-byte lines:
//   rows     X1[y][kx] = sum_x img[y][x] w^(kx x), kx = 0..64, by direct sums (thread = kx and half of the rows;
//            the powers of w^kx by repeated multiplication);
//   columns  for a slab of 13 values of kx: X[kx][ky] = sum_y X1[y][kx] w^(ky y), a 128-point transform of 16
//            inputs = 8 independent 16-point transforms X[8 m + s], two per lane of the 4 lanes of a line
//            (s = 2 q + i), parked as slab[plane][kx][ky];
//   stores   the 8 lanes (plane, half) of a piece (kx, ky quad) write its 128 bytes of the 4 planes together.
constexpr int WG = 4, WKX = 13, WSLABS = 5, WPITCH = 130, WX1P = 66, WTHREADS = 256;
constexpr int kWeightsSmem = WG * 256 * 4 + 128 * 8 + WG * 16 * WX1P * 8 + WG * WKX * WPITCH * 8;

__global__ void __launch_bounds__(WTHREADS, 2) weights128_blocked_kernel(RealView in, float* __restrict__ out, int groups,
                                                                         long long blk_planes) {
  constexpr int N = 128, H = 64;
  extern __shared__ __align__(16) unsigned char wsm[];
  float* img = reinterpret_cast<float*>(wsm);                            // [WG][16][16]
  float2* stw = reinterpret_cast<float2*>(img + WG * 256);               // [128] roots of unity
  float2* x1 = stw + N;                                                  // [WG][16][WX1P]
  float2* slab = x1 + WG * 16 * WX1P;                                    // [WG][WKX][WPITCH]
  const int tid = threadIdx.x;
  for (int i = tid; i < N; i += WTHREADS) {
    float sn, cs;
    sincospif(-2.0f * (float)i / (float)N, &sn, &cs);
    stw[i] = make_float2(cs, sn);
  }
  // the group's 4 images travel through registers: the next group's loads are in flight during this group's work
  static_assert(WG * 256 == 4 * WTHREADS, "four image values a thread");
  auto load_images = [&](int g, float (&v)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = tid + j * WTHREADS, pl = i >> 8, y = (i >> 4) & 15, x = i & 15;
      v[j] = (g < groups && y < in.h && x < in.w)
                 ? __ldg(in.p + (long long)(WG * g + pl) * in.sb + (long long)y * in.sy + (long long)x * in.sx)
                 : 0.f;
    }
  };
  float pending[4];
  load_images(blockIdx.x, pending);
  for (int g = blockIdx.x; g < groups; g += gridDim.x) {
    __syncthreads();  // the previous group's stores have read the slab; stw is written
#pragma unroll
    for (int j = 0; j < 4; ++j) img[tid + j * WTHREADS] = pending[j];
    load_images(g + gridDim.x, pending);
    __syncthreads();
    {
      // rows: thread (kx = tid % 64, rows 4 (tid / 64) .. + 3) of every plane; kx = 64 (w = -1) by the first 64 threads
      const int kx = tid & 63, y0 = (tid >> 6) * 4;
      const float2 w1 = stw[kx];
      float2 wx[16];  // w^(kx x), x = 0..15, by repeated multiplication
      wx[0] = make_float2(1.f, 0.f);
#pragma unroll
      for (int x = 1; x < 16; ++x) wx[x] = make_float2(wx[x - 1].x * w1.x - wx[x - 1].y * w1.y, wx[x - 1].x * w1.y + wx[x - 1].y * w1.x);
#pragma unroll
      for (int pl = 0; pl < WG; ++pl) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4* row = reinterpret_cast<const float4*>(img + pl * 256 + (y0 + j) * 16);  // the same for all kx: a broadcast
          float2 acc = make_float2(0.f, 0.f);
#pragma unroll
          for (int x4 = 0; x4 < 4; ++x4) {
            const float4 v = row[x4];
            acc.x += v.x * wx[4 * x4].x + v.y * wx[4 * x4 + 1].x + v.z * wx[4 * x4 + 2].x + v.w * wx[4 * x4 + 3].x;
            acc.y += v.x * wx[4 * x4].y + v.y * wx[4 * x4 + 1].y + v.z * wx[4 * x4 + 2].y + v.w * wx[4 * x4 + 3].y;
          }
          x1[(pl * 16 + y0 + j) * WX1P + kx] = acc;
        }
      }
      if (tid < WG * 16) {
        const float* row = img + tid * 16;  // (plane, y) = tid
        float sum = 0.f;
#pragma unroll
        for (int x = 0; x < 16; ++x) sum += (x & 1) ? -row[x] : row[x];
        x1[tid * WX1P + H] = make_float2(sum, 0.f);
      }
    }
    __syncthreads();
    for (int sl = 0; sl < WSLABS; ++sl) {
      const int kx0 = sl * WKX;
      {
        // columns: line task = (plane, kx of the slab), 4 lanes a line
        const int task = tid >> 2, q = tid & 3;
        if (task < WG * WKX) {
          const int pl = task / WKX, kxl = task % WKX;
          float2 x[16];
#pragma unroll
          for (int n = 0; n < 16; ++n) {
            const float2 v = x1[(pl * 16 + n) * WX1P + kx0 + kxl];
            const float2 f = stw[(2 * q * n) & (N - 1)];  // the lane's factor w128^(2 q n)
            x[n] = make_float2(v.x * f.x - v.y * f.y, v.x * f.y + v.y * f.x);
          }
          float2* line = slab + (pl * WKX + kxl) * WPITCH;
          static_for<2>([&](auto ic) {
            constexpr int i = decltype(ic)::value;
            float2 t[16];
            static_for<16>([&](auto nc) {
              constexpr int n = decltype(nc)::value;
              t[n] = mul_tw<n * i, N, false>(x[n]);
            });
            fft_bitrev<16, false, true>(t);
            static_for<16>([&](auto mc) {
              constexpr int m = decltype(mc)::value;
              line[8 * m + 2 * q + i] = t[brev(m, 16)];
            });
          });
        }
      }
      __syncthreads();
      // stores: piece (kx, ky quad) of the 4 planes = 128 contiguous bytes, 8 lanes (plane, half)
      for (int e = tid; e < WKX * 32 * 8; e += WTHREADS) {
        const int sub = e & 7, ln = e >> 3, pl = sub >> 1, half = sub & 1;
        const int kxl = ln >> 5, quad = ln & 31;
        const float4 v = *reinterpret_cast<const float4*>(slab + (pl * WKX + kxl) * WPITCH + quad * 4 + half * 2);
        const long long piece = (long long)(kx0 + kxl) * 32 + quad;
        *reinterpret_cast<float4*>(out + (piece * blk_planes + WG * g + pl) * 8 + half * 4) = v;
      }
      __syncthreads();
    }
  }
}

template <int N>
constexpr int fwd_smem() {
  constexpr int mid = N * CoopCfg<N>::PM, tile = (N / 2 + 1) * CoopCfg<N>::PO;
  return (mid > tile ? mid : tile) * (int)sizeof(float2) + 16;
}
template <int N>
constexpr int inv_smem() {
  constexpr int mid = N * CoopCfg<N>::PM, tile = (N / 2 + 1) * CoopCfg<N>::PO;
  return (mid > tile ? mid : tile) * (int)sizeof(float2) + 16;
}

template <int N>
int launch_fwd(const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(fft2d_coop_fwd_kernel<N, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem<N>());
    cudaFuncSetAttribute(fft2d_coop_fwd_kernel<N, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem<N>());
    cudaFuncSetAttribute(fft2d_coop_fwd_kernel<N, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem<N>());
    cudaFuncSetAttribute(fft2d_coop_inv_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, inv_smem<N>());
    cudaFuncSetAttribute(fft2d_coop_inv_kernel<N, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, inv_smem<N>());
    cudaFuncSetAttribute(fft2d_coop_inv_kernel<N, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, inv_smem<N>());
    configured[dev] = true;
  }
  alignas(64) CUtensorMap cmap;
  std::memset(&cmap, 0, sizeof(cmap));
  const int cap = sm_count() * CoopCfg<N>::BLOCKS_PER_SM;
  const bool in_bulk = in.sx == 1 && in.sy == in.w && (B <= 1 || in.sb == (long long)in.h * in.w) && aligned16(in.p) &&
                       in.h <= N && in.w <= N && (long long)in.h * in.w * 4 + 32 <= fwd_smem<N>() - 16;
  if constexpr (N == 128) {
    if (out.blk_planes && in.h <= 16 && in.w <= 16 && padL == 0 && padU == 0 && B % WG == 0 && B == out.blk_planes) {
      // convolution weights into the contraction's blocks: 4 adjacent planes a block, whole 128-byte lines
      static bool weights_configured[64];
      if (dev >= 0 && dev < 64 && !weights_configured[dev]) {
        cudaFuncSetAttribute(weights128_blocked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWeightsSmem);
        weights_configured[dev] = true;
      }
      const int groups = B / WG, wcap = sm_count() * 2;
      weights128_blocked_kernel<<<groups < wcap ? groups : wcap, WTHREADS, kWeightsSmem, s>>>(in, out.p, groups, out.blk_planes);
      return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
    }
    if (in.h <= 16 && in.w + padL <= 16 && padL >= 0 && padU >= 0 && in.h + padU <= N) {
      // small images in the canvas' first 16 columns (convolution weights): direct column pass
      const int smem = fwd_smem<N>() + 1024 + N * 8 + 16;
      static bool small_configured[64];
      if (dev >= 0 && dev < 64 && !small_configured[dev]) {
        cudaFuncSetAttribute(fft2d_coop_fwd_kernel<N, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        small_configured[dev] = true;
      }
      fft2d_coop_fwd_kernel<N, false, false, true><<<B < cap ? B : cap, (N / 2) * CoopCfg<N>::Q, smem, s>>>(in, out.p, out.sb, B, padL, padU, out.blk_planes, cmap);
      return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
    }
  }
  if (in_bulk && !(in.h == N && in.w == N && padL == 0 && padU == 0) && in.w % 4 == 0 && in.w + padL <= N &&
      in.h + padU <= N) {
    // zero-padded images with rows of whole 16-byte units: the canvas arrives by one tensor copy per image
    const unsigned long long dims[3] = {(unsigned long long)in.w, (unsigned long long)in.h, (unsigned long long)B};
    const unsigned long long strides[2] = {(unsigned long long)in.w * 4, (unsigned long long)in.h * in.w * 4};
    const unsigned box[3] = {(unsigned)(N + 4), (unsigned)N, 1u};
    static bool canvas_configured[64];
    if (encode_tensor_map_f32(&cmap, in.p, 3, dims, strides, box)) {
      if (dev >= 0 && dev < 64 && !canvas_configured[dev]) {
        cudaFuncSetAttribute(fft2d_coop_fwd_kernel<N, true, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem<N>());
        canvas_configured[dev] = true;
      }
      fft2d_coop_fwd_kernel<N, true, false, false, true><<<B < cap ? B : cap, (N / 2) * CoopCfg<N>::Q, fwd_smem<N>(), s>>>(in, out.p, out.sb, B, padL, padU, out.blk_planes, cmap);
      return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
    }
  }
  if (in_bulk && in.h == N && in.w == N && padL == 0 && padU == 0) {
    fft2d_coop_fwd_kernel<N, true, true><<<B < cap ? B : cap, (N / 2) * CoopCfg<N>::Q, fwd_smem<N>(), s>>>(in, out.p, out.sb, B, padL, padU, out.blk_planes, cmap);
  } else if (in_bulk) {
    fft2d_coop_fwd_kernel<N, true><<<B < cap ? B : cap, (N / 2) * CoopCfg<N>::Q, fwd_smem<N>(), s>>>(in, out.p, out.sb, B, padL, padU, out.blk_planes, cmap);
  } else {
    fft2d_coop_fwd_kernel<N, false><<<B < cap ? B : cap, (N / 2) * CoopCfg<N>::Q, fwd_smem<N>(), s>>>(in, out.p, out.sb, B, padL, padU, out.blk_planes, cmap);
  }
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

template <int N>
int launch_inv(const CplxView& in, const RealView& out, int B, int padL, int padU, cudaStream_t s) {
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaFuncSetAttribute(fft2d_coop_fwd_kernel<N, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem<N>());
    cudaFuncSetAttribute(fft2d_coop_fwd_kernel<N, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem<N>());
    cudaFuncSetAttribute(fft2d_coop_fwd_kernel<N, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem<N>());
    cudaFuncSetAttribute(fft2d_coop_inv_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, inv_smem<N>());
    cudaFuncSetAttribute(fft2d_coop_inv_kernel<N, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, inv_smem<N>());
    cudaFuncSetAttribute(fft2d_coop_inv_kernel<N, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, inv_smem<N>());
    configured[dev] = true;
  }
  const int cap = sm_count() * CoopCfg<N>::BLOCKS_PER_SM;
  // (measured: the predicate-free stores gain at N = 128, 0.57 -> 0.78 of the copy bandwidth, and lose at N = 64)
  // (measured: full 128 x 128 outputs keep their direct stores, 0.76 against 0.71 of the copy bandwidth with parked rows)
  if (N == 128 && out.sx == 1 && out.sy == N && out.h == N && out.w == N && padL == 0 && padU == 0) {
    fft2d_coop_inv_kernel<N, true><<<B < cap ? B : cap, (N / 2) * CoopCfg<N>::Q, inv_smem<N>(), s>>>(in.p, in.sb, out, B, padL, padU, in.blk_planes);
  } else if (N == 64 && out.w + padL <= 8) {
    // weight gradients at N = 64: only the first 8 columns are kept
    if constexpr (N == 64) {
      static bool narrow64_configured[64];
      if (dev >= 0 && dev < 64 && !narrow64_configured[dev]) {
        cudaFuncSetAttribute(fft2d_coop_inv_kernel<N, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, inv_smem<N>());
        narrow64_configured[dev] = true;
      }
      fft2d_coop_inv_kernel<N, false, false, true><<<B < cap ? B : cap, (N / 2) * CoopCfg<N>::Q, inv_smem<N>(), s>>>(in.p, in.sb, out, B, padL, padU, in.blk_planes);
    }
  } else if (N == 128 && out.w + padL <= 16) {
    // weight gradients: only the first 16 columns are kept, the row pass computes nothing else
    if constexpr (N == 128) {
      static bool narrow_configured[64];
      if (dev >= 0 && dev < 64 && !narrow_configured[dev]) {
        cudaFuncSetAttribute(fft2d_coop_inv_kernel<N, false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, inv_smem<N>());
        narrow_configured[dev] = true;
      }
      fft2d_coop_inv_kernel<N, false, true, true><<<B < cap ? B : cap, (N / 2) * CoopCfg<N>::Q, inv_smem<N>(), s>>>(in.p, in.sb, out, B, padL, padU, in.blk_planes);
    }
  } else if (N == 128 && (out.w + padL) * 2 <= N) {
    // at most half of the column pairs survive the crop (measured on 13x13 weight gradients: 297 -> 227 us)
    fft2d_coop_inv_kernel<N, false, true><<<B < cap ? B : cap, (N / 2) * CoopCfg<N>::Q, inv_smem<N>(), s>>>(in.p, in.sb, out, B, padL, padU, in.blk_planes);
  } else if (out.sx == 1 && out.w >= 4 && out.w % 4 == 0 && padL % 4 == 0 && out.sy % 4 == 0 && (B <= 1 || out.sb % 4 == 0) &&
             aligned16(out.p) && padL + out.w <= N && padU + out.h <= N && !(N == 128 && (out.w + padL) * 2 <= N)) {
    // cropped images in 16-byte units: rows parked in shared memory, one bulk store per kept row
    static bool stage_configured[64];
    if (dev >= 0 && dev < 64 && !stage_configured[dev]) {
      cudaFuncSetAttribute(fft2d_coop_inv_kernel<N, false, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, inv_smem<N>());
      stage_configured[dev] = true;
    }
    fft2d_coop_inv_kernel<N, false, false, false, true><<<B < cap ? B : cap, (N / 2) * CoopCfg<N>::Q, inv_smem<N>(), s>>>(in.p, in.sb, out, B, padL, padU, in.blk_planes);
  } else {
    fft2d_coop_inv_kernel<N><<<B < cap ? B : cap, (N / 2) * CoopCfg<N>::Q, inv_smem<N>(), s>>>(in.p, in.sb, out, B, padL, padU, in.blk_planes);
  }
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

}  // namespace

bool fft2d_coop_supported(int n, const CplxView& c) {
  if (c.blk_planes) return (n == 64 || n == 128) && aligned16(c.p);
  return (n == 64 || n == 128) && c.sz == 1 && c.sc == 2 && c.sr == 2 * n && (c.sb % 4) == 0 && aligned16(c.p);
}

int fft2d_coop_forward(int n, const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s) {
  if (out.blk_planes && out.blk_bins != 4) return kUnsupportedDimension;  // forward transforms write 4-bin blocks
  if (n == 64) return launch_fwd<64>(in, out, B, padL, padU, s);
  return launch_fwd<128>(in, out, B, padL, padU, s);
}

int fft2d_coop_inverse(int n, const CplxView& in, const RealView& out, int B, int padL, int padU, cudaStream_t s) {
  if (in.blk_planes && in.blk_bins != n) return kUnsupportedDimension;  // inverse transforms read row blocks
  if (n == 64) return launch_inv<64>(in, out, B, padL, padU, s);
  return launch_inv<128>(in, out, B, padL, padU, s);
}

int read_device_error_coop() { return device_error_word_read(); }
int clear_device_error_coop() { return device_error_word_clear(); }

}  // namespace fbfft_b200
