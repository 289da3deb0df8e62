// Batched 2-D real-to-complex / complex-to-real FFTs for N in {8, 16, 32}.
//
// Replaces the reference's fbfft2DVertical_{8,16,32} / fbifft2DVertical_{8,16,32}
// kernels (fbfft/FFT2D32.cuh:361-533, dispatched from fbfft/FBFFT2D-inl.cuh:476-570
// and fbfft/FBIFFT2D-inl.cuh:591-682).  Output layout is the reference's for this
// size class: [B][ky in 0..N/2][kx in 0..N) complex, Hermitian half along the ROW
// frequency; the inverse is unnormalised (returns N*N*x) and crops at (padU, padL).
//
// Design: a warp owns 32/(N/2) images at a time and never synchronises with any
// other warp.  Both passes are length-N complex FFTs held entirely in one
// thread's registers (fft2d_small.cuh):
//   pass A  thread (image, l) takes columns l and l+N/2 as re/im of one complex
//           line, transforms it and separates the two real-input spectra; rows 0
//           and N/2 are real and travel packed as one complex row;
//   pass B  after a transpose through padded shared memory, thread (image, r)
//           transforms packed row r; row 0 is then unpacked into rows 0 and N/2.
// Data movement on the fast path (contiguous, 16-byte aligned tensors) is
// asynchronous: the raw images of the NEXT task are fetched with cp.async.bulk into
// a per-warp staging slot while the current task computes (completion on a
// per-warp mbarrier), and finished rows leave through bulk stores; neither costs
// issue slots or registers.  Strided or unaligned tensors take plain loads/stores
// with the same arithmetic.  No twiddle is ever shuffled or read from memory.
#include "fft2d_small.cuh"
#include "kernels.h"

namespace fbfft_b200 {

namespace {

constexpr int kSmallThreads = 128;
constexpr int kWarps = kSmallThreads / 32;

enum : int { kErrFwdWait = 101, kErrInvWait = 102 };

// ------------------------------------------------------------------ forward
// IN_BULK : real input is contiguous [B][h][w] with a 16-byte aligned base
// OUT_BULK: complex output is contiguous [B][N/2+1][N][2] with a 16-byte aligned base
// FULL    : (with IN_BULK) the images are N x N without padding: compile-time offsets, no predicates
// SINGLE  : (with IN_BULK and OUT_BULK) the staging slot aliases the warp's work buffer: the next task
//           is fetched only after the current rows have left, but 4 blocks fit an SM instead of 3
template <int N, bool IN_BULK, bool OUT_BULK, bool FULL = false, bool SINGLE = false>
__global__ void __launch_bounds__(kSmallThreads, SINGLE ? 4 : 3) fft2d_small_fwd_kernel(RealView in, CplxView out, int B, int padL,
                                                                          int padU, int ntasks, int slot_floats, int slot_pitch) {
  constexpr int T = N / 2, IPW = 32 / T, ROWS = T + 1;
  constexpr int RS = SmallCfg<N>::RS, IS = SmallCfg<N>::IS;
  extern __shared__ __align__(16) float2 smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float2* buf = smem + warp * (IPW * IS);
  const int li = lane / T, l = lane % T;
  float2* ib = buf + li * IS;
  // staging slots (IN_BULK) follow the work buffers; mbarriers follow the slots
  float* slot = SINGLE ? reinterpret_cast<float*>(buf)
                       : reinterpret_cast<float*>(smem + kWarps * (IPW * IS)) + warp * slot_floats;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(reinterpret_cast<float*>(smem + kWarps * (IPW * IS)) +
                                                                   (SINGLE ? 0 : kWarps * slot_floats));
  const unsigned bar = smem_u32(bars + warp);
  __shared__ float zero_storage;
  if (threadIdx.x == 0) zero_storage = 0.f;
  __syncthreads();
  const float* zero_word = &zero_storage;
  const long long img_floats = (long long)in.h * in.w;
  const long long total_bytes = (long long)B * img_floats * 4;

  const int first = blockIdx.x * kWarps + warp, stride = gridDim.x * kWarps;
  // bytes [lo, hi) of the 16-byte aligned window around the images of `task`;
  // returns false when the window would reach past the end of the tensor
  auto window = [&](int task, long long* lo, unsigned* bytes) {
    const long long g0 = (long long)task * IPW * img_floats * 4;
    long long g1 = g0 + IPW * img_floats * 4;
    if (g1 > total_bytes) g1 = total_bytes;
    *lo = g0 & ~15LL;
    const long long hi = (g1 + 15) & ~15LL;
    *bytes = (unsigned)(hi - *lo);
    return hi <= total_bytes || (total_bytes & 15) == 0;
  };
  // When an image is a whole number of 16-byte units every image gets its own copy into a slot
  // of pitch slot_pitch = h*w + N/2 floats, which puts the images of a warp N/2 banks apart (the
  // column reads of pass A are then conflict free); otherwise one copy brings the task's window.
  const bool per_image = slot_pitch != (int)img_floats;
  auto issue = [&](int task) -> bool {
    if (per_image) {
      int imgs = B - task * IPW;
      if (imgs > IPW) imgs = IPW;
      if (lane == 0) {
        fence_async_smem();
        mbar_expect_tx(bar, (unsigned)(imgs * img_floats * 4));
      }
      __syncwarp();
      if (lane < imgs)
        bulk_g2s(smem_u32(slot + lane * slot_pitch), in.p + (long long)(task * IPW + lane) * img_floats,
                 (unsigned)(img_floats * 4), bar);
      return true;
    }
    long long lo;
    unsigned bytes;
    const bool ok = window(task, &lo, &bytes);
    if (ok && lane == 0) {
      fence_async_smem();
      mbar_expect_tx(bar, bytes);
      bulk_g2s(smem_u32(slot), reinterpret_cast<const char*>(in.p) + lo, bytes, bar);
    }
    return ok;
  };
  unsigned phase = 0;
  bool staged = false;  // the slot holds (or will hold) the current task
  if (IN_BULK) {
    if (lane == 0) mbar_init(bar, 1);
    __syncwarp();
    if (first < ntasks) staged = issue(first);
  }

  for (int task = first; task < ntasks; task += stride) {
    const int b = task * IPW + li;
    const bool valid = b < B;
    {
      // ---- pass A
      float2 a[N];
      if (IN_BULK && staged) {
        if (!mbar_wait(bar, phase, kErrFwdWait)) return;
        phase ^= 1;
        const long long g0 = (long long)task * IPW * img_floats * 4;
        const int off0 = per_image ? 0 : (int)((g0 & 15) >> 2);
        if constexpr (FULL) {
          load_columns_full<N>(slot + li * (N * N + N / 2), l, a);  // per-image slots of pitch N*N + N/2
        } else {
          load_columns_staged<N>(slot + off0 + li * slot_pitch, zero_word, in.h, in.w, padL, padU, l, a);
        }
      } else {
        load_columns<N>(in.p + (long long)(valid ? b : 0) * in.sb, in.sy, in.sx, in.h, in.w, padL, padU, valid, l, a);
      }
      if (IN_BULK && !SINGLE) {
        // everything of this task is in registers: fetch the next task into the slot
        __syncwarp();
        const int next = task + stride;
        staged = false;
        if (next < ntasks) staged = issue(next);
      }
      if (SINGLE) __syncwarp();  // every lane has read the slot that the work buffer overwrites
      fft_bitrev<N, false>(a);
      if (OUT_BULK) {
        // rows of the previous task may still be leaving the work buffer
        bulk_wait_read();
        __syncwarp();
      }
      fwd_separate_store<N>(a, ib, l);
    }
    __syncwarp();
    fwd_rows_unpack<N>(ib, l);
    // ---- store IPW images x ROWS rows x N complex
    if (OUT_BULK) {
      fence_async_smem();
      __syncwarp();
      if (N >= 16 && out.blk_planes) {
        // 4-bin blocks: every 32-byte piece of a row goes next to the same piece of the neighbouring
        // planes; two lanes per piece, the images of the warp adjacent in memory
        constexpr int QR = N / 4;
        for (int e = lane; e < IPW * ROWS * QR * 2; e += 32) {
          const int half = e & 1, img = (e >> 1) % IPW, piece = (e >> 1) / IPW;  // piece = row * QR + quad in row
          const int bb = task * IPW + img;
          if (bb < B) {
            const float4 v = *reinterpret_cast<const float4*>(buf + img * IS + (piece / QR) * RS + (piece % QR) * 4 + half * 2);
            *reinterpret_cast<float4*>(out.p + ((long long)piece * out.blk_planes + bb) * 8 + half * 4) = v;
          }
        }
        __syncwarp();
      } else if (RS == N) {
        // rows are contiguous in shared memory: one copy per image
        if (lane < IPW && task * IPW + lane < B)
          bulk_s2g(out.p + (long long)(task * IPW + lane) * out.sb, smem_u32(buf + lane * IS), ROWS * N * 8);
      } else {
        for (int r = lane; r < IPW * ROWS; r += 32) {
          const int img = r / ROWS, row = r % ROWS;
          const int bb = task * IPW + img;
          if (bb < B)
            bulk_s2g(out.p + (long long)bb * out.sb + (long long)row * (2 * N), smem_u32(buf + img * IS + row * RS),
                     N * 8);
        }
      }
      bulk_commit();
      if constexpr (SINGLE) {
        // the rows have left the work buffer: the next task may land in it
        bulk_wait_read();
        __syncwarp();
        const int next = task + stride;
        staged = false;
        if (next < ntasks) staged = issue(next);
      }
    } else {
      constexpr int PER = ROWS * N;
      for (int e = lane; e < IPW * PER; e += 32) {
        const int img = e / PER, rem = e % PER, row = rem / N, c = rem % N;
        const int bb = task * IPW + img;
        if (bb < B) {
          const float2 t = buf[img * IS + row * RS + c];
          float* dst = out.p + (long long)bb * out.sb + (long long)row * out.sr + (long long)c * out.sc;
          dst[0] = t.x;
          dst[out.sz] = t.y;
        }
      }
      __syncwarp();
    }
  }
  if (OUT_BULK) bulk_wait_read();
}

// ------------------------------------------------------------------ inverse
// IN_BULK: complex input contiguous and 16-byte aligned; rows are fetched with bulk
// copies one task ahead into the second of two work buffers.
// FULL   : the output images are contiguous N x N without crop offset
// SINGLE : (with IN_BULK) one work buffer per warp instead of two: the next task's rows are fetched
//          into it as soon as the column pass holds the current task in registers.  Shorter
//          prefetch distance, but 5 resident blocks per SM instead of 3.
template <int N, bool IN_BULK, bool FULL = false, bool SINGLE = false>
__global__ void __launch_bounds__(kSmallThreads, SINGLE ? 5 : 3) fft2d_small_inv_kernel(CplxView in, RealView out, int B, int padL,
                                                                          int padU, int ntasks) {
  constexpr int T = N / 2, IPW = 32 / T, ROWS = T + 1;
  constexpr int RS = SmallCfg<N>::RS, IS = SmallCfg<N>::IS;
  constexpr int NBUF = (IN_BULK && !SINGLE) ? 2 : 1;
  extern __shared__ __align__(16) float2 smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float2* wbuf = smem + warp * (NBUF * IPW * IS);
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + kWarps * (NBUF * IPW * IS));
  const int li = lane / T, l = lane % T;
  const int first = blockIdx.x * kWarps + warp, stride = gridDim.x * kWarps;

  // issue the row copies of `task` into buffer `which`; completion on that buffer's barrier
  auto fetch = [&](int task, int which) {
    float2* dstbuf = wbuf + which * (IPW * IS);
    const unsigned bar = smem_u32(bars + warp * 2 + which);
    int imgs = B - task * IPW;
    if (imgs > IPW) imgs = IPW;
    fence_async_smem();
    __syncwarp();
    if (lane == 0) mbar_expect_tx(bar, (unsigned)(imgs * ROWS * N * 8));
    __syncwarp();
    if (N >= 16 && in.blk_planes) {
      // row blocks: stored row `row` of plane b sits at ((row * planes + b) * N) complex values
      for (int r = lane; r < imgs * ROWS; r += 32) {
        const int img = r / ROWS, row = r % ROWS;
        bulk_g2s(smem_u32(dstbuf + img * IS + row * RS),
                 in.p + ((long long)row * in.blk_planes + task * IPW + img) * (2 * N), N * 8, bar);
      }
    } else if (RS == N) {
      // rows are contiguous in shared memory: one copy per image
      if (lane < imgs)
        bulk_g2s(smem_u32(dstbuf + lane * IS), in.p + (long long)(task * IPW + lane) * in.sb, ROWS * N * 8, bar);
    } else {
      for (int r = lane; r < imgs * ROWS; r += 32) {
        const int img = r / ROWS, row = r % ROWS;
        bulk_g2s(smem_u32(dstbuf + img * IS + row * RS),
                 in.p + (long long)(task * IPW + img) * in.sb + (long long)row * (2 * N), N * 8, bar);
      }
    }
  };

  unsigned phase[2] = {0, 0};
  int cur = 0;
  if (IN_BULK) {
    if (lane == 0) {
      mbar_init(smem_u32(bars + warp * 2), 1);
      mbar_init(smem_u32(bars + warp * 2 + 1), 1);
    }
    __syncwarp();
    if (first < ntasks) fetch(first, 0);
  }

  for (int task = first; task < ntasks; task += stride) {
    float2* buf = wbuf + cur * (IPW * IS);
    float2* ib = buf + li * IS;
    if (IN_BULK) {
      if (!SINGLE && task + stride < ntasks) fetch(task + stride, cur ^ 1);
      if (!mbar_wait(smem_u32(bars + warp * 2 + cur), phase[cur], kErrInvWait)) return;
      phase[cur] ^= 1;
    } else {
      constexpr int PER = ROWS * N;
      for (int e = lane; e < IPW * PER; e += 32) {
        const int img = e / PER, rem = e % PER, row = rem / N, c = rem % N;
        const int bb = task * IPW + img;
        float2 t = make_float2(0.f, 0.f);
        if (bb < B) {
          const float* s = in.p + (long long)bb * in.sb + (long long)row * in.sr + (long long)c * in.sc;
          t = make_float2(__ldg(s), __ldg(s + in.sz));
        }
        buf[img * IS + row * RS + c] = t;
      }
      __syncwarp();
    }
    inv_pack_rows<N>(ib, l);
    {
      float2 z[N];
      inv_columns_load<N>(ib, l, z);
      if (IN_BULK && SINGLE) {
        // the whole task is in registers: its buffer takes the next task's rows
        __syncwarp();
        if (task + stride < ntasks) fetch(task + stride, 0);
      }
      fft_bitrev<N, true, true>(z);
      const int b = task * IPW + li;
      if (b < B) {
        if constexpr (FULL) {
          store_columns_full<N>(out.p + (long long)b * (N * N), l, z);
        } else {
          store_columns<N>(out.p + (long long)b * out.sb, out.sy, out.sx, out.h, out.w, padL, padU, l, z, 1.0f);
        }
      }
    }
    __syncwarp();
    cur ^= (IN_BULK && !SINGLE) ? 1 : 0;
  }
}

template <int N>
constexpr int work_floats() {
  return kWarps * (32 / (N / 2)) * SmallCfg<N>::IS * 2;
}

bool cplx_is_contiguous16(const CplxView& c, int cols) {
  if (c.blk_planes) return cols >= 16 && aligned16(c.p);
  return c.sz == 1 && c.sc == 2 && c.sr == 2 * cols && (c.sb % 4) == 0 && aligned16(c.p);
}
bool real_is_contiguous16(const RealView& r, int B) {
  return r.sx == 1 && r.sy == r.w && (B <= 1 || r.sb == (long long)r.h * r.w) && aligned16(r.p);
}

int grid_for(int ntasks, int per_sm) {
  const int want = (ntasks + kWarps - 1) / kWarps;
  const int cap = sm_count() * per_sm;
  return want < cap ? want : cap;
}

template <typename K>
void allow_smem(K kernel, int bytes) {
  if (bytes > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

template <int N>
int launch_fwd(const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s) {
  constexpr int IPW = 32 / (N / 2);
  const int ntasks = (B + IPW - 1) / IPW;
  const bool out_bulk = cplx_is_contiguous16(out, N);
  const int hw = in.h * in.w;
  // staging slot per warp: the raw images of one task plus alignment slack
  const int slot_pitch = (hw % 4 == 0) ? hw + N / 2 : hw;
  const int slot_floats = ((IPW * slot_pitch + 8 + 3) / 4) * 4;
  const bool in_bulk = real_is_contiguous16(in, B) && in.h <= N && in.w <= N;
  const int base = work_floats<N>() * 4;
  if (in_bulk) {
    const int smem = base + kWarps * slot_floats * 4 + kWarps * 8;
    const int grid = grid_for(ntasks, 3);
    // (measured: the predicate-free variant gains at N = 16 and loses a little at N = 8 and 32)
    // (measured on full images: the single-buffer variant gains at N = 32, 0.85 -> 0.99 of the copy
    // bandwidth with 16 instead of 12 resident warps, and loses at N = 8 and 16)
    if (N == 32 && out_bulk && !out.blk_planes && hw % 4 == 0) {
      const int smem1 = base + kWarps * 8;
      allow_smem(fft2d_small_fwd_kernel<N, true, true, false, true>, smem1);
      fft2d_small_fwd_kernel<N, true, true, false, true><<<grid_for(ntasks, 4), kSmallThreads, smem1, s>>>(in, out, B, padL, padU, ntasks, slot_floats, slot_pitch);
    } else if (N == 16 && out_bulk && in.h == N && in.w == N && padL == 0 && padU == 0) {
      allow_smem(fft2d_small_fwd_kernel<N, true, true, true>, smem);
      fft2d_small_fwd_kernel<N, true, true, true><<<grid, kSmallThreads, smem, s>>>(in, out, B, padL, padU, ntasks, slot_floats, slot_pitch);
    } else if (out_bulk) {
      allow_smem(fft2d_small_fwd_kernel<N, true, true>, smem);
      fft2d_small_fwd_kernel<N, true, true><<<grid, kSmallThreads, smem, s>>>(in, out, B, padL, padU, ntasks, slot_floats, slot_pitch);
    } else {
      allow_smem(fft2d_small_fwd_kernel<N, true, false>, smem);
      fft2d_small_fwd_kernel<N, true, false><<<grid, kSmallThreads, smem, s>>>(in, out, B, padL, padU, ntasks, slot_floats, slot_pitch);
    }
  } else {
    const int grid = grid_for(ntasks, 4);
    if (out_bulk) {
      fft2d_small_fwd_kernel<N, false, true><<<grid, kSmallThreads, base, s>>>(in, out, B, padL, padU, ntasks, 0, 0);
    } else {
      fft2d_small_fwd_kernel<N, false, false><<<grid, kSmallThreads, base, s>>>(in, out, B, padL, padU, ntasks, 0, 0);
    }
  }
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

template <int N>
int launch_inv(const CplxView& in, const RealView& out, int B, int padL, int padU, cudaStream_t s) {
  constexpr int IPW = 32 / (N / 2);
  const int ntasks = (B + IPW - 1) / IPW;
  const int base = work_floats<N>() * 4;
  if (cplx_is_contiguous16(in, N)) {
    const int smem = 2 * base + kWarps * 16;
    // (measured: gains at N = 16, loses at N = 8 and 32)
    const bool full = N == 16 && out.sx == 1 && out.sy == N && out.h == N && out.w == N && padL == 0 && padU == 0 &&
                      (B <= 1 || out.sb == (long long)N * N);
    if (full) {
      allow_smem(fft2d_small_inv_kernel<N, true, true>, smem);
      fft2d_small_inv_kernel<N, true, true><<<grid_for(ntasks, 3), kSmallThreads, smem, s>>>(in, out, B, padL, padU, ntasks);
    } else if (N == 8 || (N == 32 && (out.h < N || out.w < N))) {
      // (measured: the single-buffer variant gains at N = 8, 0.79 -> 0.82, and for cropped outputs at
      // N = 32, 27x27: 0.82 -> 0.92; it loses for full 32x32 outputs, 0.89 -> 0.86)
      const int smem1 = base + kWarps * 16;
      allow_smem(fft2d_small_inv_kernel<N, true, false, true>, smem1);
      fft2d_small_inv_kernel<N, true, false, true><<<grid_for(ntasks, 5), kSmallThreads, smem1, s>>>(in, out, B, padL, padU, ntasks);
    } else {
      allow_smem(fft2d_small_inv_kernel<N, true>, smem);
      fft2d_small_inv_kernel<N, true><<<grid_for(ntasks, 3), kSmallThreads, smem, s>>>(in, out, B, padL, padU, ntasks);
    }
  } else {
    fft2d_small_inv_kernel<N, false><<<grid_for(ntasks, 4), kSmallThreads, base, s>>>(in, out, B, padL, padU, ntasks);
  }
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

}  // namespace

int fft2d_small_forward(int n, const RealView& in, const CplxView& out, int B, int padL, int padU, cudaStream_t s) {
  if (B <= 0) return kSuccess;
  if (out.blk_planes && out.blk_bins != 4) return kUnsupportedDimension;  // forward transforms write 4-bin blocks
  if (n == 8 && fft2d_n8_supported(in, out, B, padL, padU)) {
    // whole groups of 32 full images: one thread per image; the rest below
    const int done = (B / 32) * 32;
    if (int rc = fft2d_n8(false, in.p, out.p, B / 32, s)) return rc;
    if (done == B) return kSuccess;
    RealView i2 = in;
    CplxView o2 = out;
    i2.p += (long long)done * in.sb, o2.p += (long long)done * out.sb;
    return launch_fwd<8>(i2, o2, B - done, padL, padU, s);
  }
  switch (n) {
    case 8:
      return launch_fwd<8>(in, out, B, padL, padU, s);
    case 16:
      return launch_fwd<16>(in, out, B, padL, padU, s);
    case 32:
      return launch_fwd<32>(in, out, B, padL, padU, s);
    default:
      return kUnsupportedSize;
  }
}

int fft2d_small_inverse(int n, const CplxView& in, const RealView& out, int B, int padL, int padU, cudaStream_t s) {
  if (B <= 0) return kSuccess;
  if (in.blk_planes && in.blk_bins != n) return kUnsupportedDimension;  // inverse transforms read row blocks
  if (n == 8 && fft2d_n8_supported(out, in, B, padL, padU)) {
    const int done = (B / 32) * 32;
    if (int rc = fft2d_n8(true, in.p, out.p, B / 32, s)) return rc;
    if (done == B) return kSuccess;
    CplxView i2 = in;
    RealView o2 = out;
    i2.p += (long long)done * in.sb, o2.p += (long long)done * out.sb;
    return launch_inv<8>(i2, o2, B - done, padL, padU, s);
  }
  switch (n) {
    case 8:
      return launch_inv<8>(in, out, B, padL, padU, s);
    case 16:
      return launch_inv<16>(in, out, B, padL, padU, s);
    case 32:
      return launch_inv<32>(in, out, B, padL, padU, s);
    default:
      return kUnsupportedSize;
  }
}

int read_device_error() { return device_error_word_read(); }
int clear_device_error() { return device_error_word_clear(); }

// ---------------------------------------------------------------- self-test of the bounded wait
// One thread waits, through the same mbar_wait the transforms use, on a barrier whose phase
// nothing ever completes.  The wait must run out, record its code and let the kernel return.
namespace {
constexpr int kErrSelftestWait = 901;
__device__ unsigned long long g_selftest_ns = 0;

__global__ void selftest_wait_kernel(int max_tries) {
  __shared__ __align__(8) unsigned long long bar_mem;
  if (threadIdx.x == 0) {
    const unsigned bar = smem_u32(&bar_mem);
    mbar_init(bar, 1);
    fence_async_smem();
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    const bool done = mbar_wait(bar, 0, kErrSelftestWait, max_tries);
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    g_selftest_ns = done ? 0ULL : (t1 - t0);
  }
}
}  // namespace

int selftest_bounded_wait(int max_tries, unsigned long long* elapsed_ns) {
  selftest_wait_kernel<<<1, 32>>>(max_tries);
  if (cudaPeekAtLastError() != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) return kCudaError;
  unsigned long long ns = 0;
  if (cudaMemcpyFromSymbol(&ns, g_selftest_ns, sizeof(ns)) != cudaSuccess) return kCudaError;
  if (elapsed_ns) *elapsed_ns = ns;
  return kSuccess;
}

}  // namespace fbfft_b200
