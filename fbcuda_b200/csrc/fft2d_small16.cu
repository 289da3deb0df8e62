// fbfft2D / fbifft2D for N in {8, 16, 32} with 16-bit storage (fp16 or bf16) of the images, of the
// spectra, or of both; arithmetic stays fp32 in registers.  The reference leaves this as
// "TODO: f16 implementation" in both directions (fbfft/FFT2D32.cuh:385, :451); layout, padding
// rule and normalisation are those of the fp32 transforms (fbfft/FFT2D32.cuh:361-470): spectrum
// [B][N/2+1][N] complex with ky the halved index, inverse unnormalised and cropped at (padU, padL).
//
// Same decomposition as fft2d_small.cu -- a warp owns 32/(N/2) images, every 1-D transform is a
// length-N complex FFT in one thread's registers, one transpose through padded shared memory --
// with the conversions at the edges: the stored bytes of the next task (images forward, spectra
// inverse) arrive by one cp.async.bulk per warp while the current task computes, are widened from
// shared memory into the fp32 canvas / rows, results leave as 16-byte vectors of four complex values
// (forward) or, narrowed in a shared-memory image first, as whole 4-byte words (inverse; a task's
// images start on a 4-byte boundary for every image size).
// Tensors must be contiguous.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fft2d_small.cuh"
#include "kernels.h"

namespace fbfft_b200 {

namespace {

constexpr int kThreads16 = 128;
constexpr int kWarps16 = kThreads16 / 32;

// ---- element access: T in {float, __half, __nv_bfloat16}
template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static constexpr int kPerWord = 1;  // elements per 4-byte word
  static __device__ __forceinline__ void unpack(unsigned w, float* lo, float* hi) { *lo = __uint_as_float(w), *hi = 0.f; }
  static __device__ __forceinline__ unsigned pack(float lo, float) { return __float_as_uint(lo); }
};
template <>
struct Elem<__half> {
  static constexpr int kPerWord = 2;
  static __device__ __forceinline__ void unpack(unsigned w, float* lo, float* hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    *lo = f.x, *hi = f.y;
  }
  static __device__ __forceinline__ unsigned pack(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&h);
  }
};
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kPerWord = 2;
  static __device__ __forceinline__ void unpack(unsigned w, float* lo, float* hi) {
    *lo = __uint_as_float(w << 16), *hi = __uint_as_float(w & 0xffff0000u);
  }
  static __device__ __forceinline__ unsigned pack(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&h);
  }
};

// four complex values (8 floats) <-> the storage type
template <typename T>
__device__ __forceinline__ void load_cplx4(const T* src, float4* a, float4* b) {
  if constexpr (Elem<T>::kPerWord == 1) {
    *a = *reinterpret_cast<const float4*>(src);
    *b = *reinterpret_cast<const float4*>(src + 4);
  } else {
    const uint4 w = *reinterpret_cast<const uint4*>(src);
    Elem<T>::unpack(w.x, &a->x, &a->y);
    Elem<T>::unpack(w.y, &a->z, &a->w);
    Elem<T>::unpack(w.z, &b->x, &b->y);
    Elem<T>::unpack(w.w, &b->z, &b->w);
  }
}
template <typename T>
__device__ __forceinline__ void store_cplx4(T* dst, float4 a, float4 b) {
  if constexpr (Elem<T>::kPerWord == 1) {
    *reinterpret_cast<float4*>(dst) = a;
    *reinterpret_cast<float4*>(dst + 4) = b;
  } else {
    *reinterpret_cast<uint4*>(dst) =
        make_uint4(Elem<T>::pack(a.x, a.y), Elem<T>::pack(a.z, a.w), Elem<T>::pack(b.x, b.y), Elem<T>::pack(b.z, b.w));
  }
}

enum : int { kErrFwd16Wait = 111, kErrInv16Wait = 112 };

// ------------------------------------------------------------------ forward
// in: [B][h][w] of TI, contiguous; out: [B][N/2+1][N][2] of TO, contiguous.
// The raw bytes of the NEXT task arrive by one cp.async.bulk (the 16-byte aligned window around the
// task's images, completion on the warp's mbarrier, bounded wait) while the current one computes.
template <int N, typename TI, typename TO>
__global__ void __launch_bounds__(kThreads16, 3) fft2d_small_fwd16_kernel(const TI* __restrict__ in, TO* __restrict__ out, int B,
                                                                         int h, int w, int padL, int padU, int ntasks,
                                                                         int slot_floats, int raw_bytes) {
  constexpr int T = N / 2, IPW = 32 / T, ROWS = T + 1, PW = Elem<TI>::kPerWord;
  constexpr int RS = SmallCfg<N>::RS, IS = SmallCfg<N>::IS;
  extern __shared__ __align__(16) float2 smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float2* buf = smem + warp * (IPW * IS);
  float* slot = reinterpret_cast<float*>(smem + kWarps16 * (IPW * IS)) + warp * slot_floats;
  unsigned char* raw = reinterpret_cast<unsigned char*>(reinterpret_cast<float*>(smem + kWarps16 * (IPW * IS)) + kWarps16 * slot_floats) +
                       warp * raw_bytes;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(
      reinterpret_cast<unsigned char*>(reinterpret_cast<float*>(smem + kWarps16 * (IPW * IS)) + kWarps16 * slot_floats) + kWarps16 * raw_bytes);
  const unsigned bar = smem_u32(bars + warp);
  __shared__ float zero_storage;
  if (threadIdx.x == 0) zero_storage = 0.f;
  if (lane == 0) mbar_init(bar, 1);
  fence_async_smem();
  __syncthreads();
  const int li = lane / T, l = lane % T;
  float2* ib = buf + li * IS;
  const int hw = h * w;
  const long long total = (long long)B * hw;  // elements of the whole input
  const long long total_bytes = total * (long long)sizeof(TI);
  const long long task_bytes = (long long)IPW * hw * (long long)sizeof(TI);  // a multiple of 4
  const unsigned* in_words = reinterpret_cast<const unsigned*>(in);
  const int first = blockIdx.x * kWarps16 + warp, stride = gridDim.x * kWarps16;
  // the 16-byte aligned window around the task's bytes; false when it would reach past the tensor
  auto issue = [&](int task) -> bool {
    const long long g0 = (long long)task * task_bytes;
    long long g1 = g0 + task_bytes;
    if (g1 > total_bytes) g1 = total_bytes;
    const long long lo = g0 & ~15LL, hi = (g1 + 15) & ~15LL;
    const bool ok = hi <= total_bytes || (total_bytes & 15) == 0;
    if (ok && lane == 0) {
      fence_async_smem();
      mbar_expect_tx(bar, (unsigned)(hi - lo));
      bulk_g2s(smem_u32(raw), reinterpret_cast<const char*>(in) + lo, (unsigned)(hi - lo), bar);
    }
    return ok;
  };
  unsigned phase = 0;
  bool staged = first < ntasks ? issue(first) : false;
  for (int task = first; task < ntasks; task += stride) {
    // ---- the task's images, widened into the slot (element e of the task at slot[e])
    const long long e0 = (long long)task * IPW * hw;  // a multiple of PW for every hw (IPW is even)
    long long cnt = total - e0;
    if (cnt > (long long)IPW * hw) cnt = (long long)IPW * hw;
    const int words = (int)((cnt + PW - 1) / PW);
    if (staged) {
      if (!mbar_wait(bar, phase, kErrFwd16Wait)) return;
      phase ^= 1;
      const unsigned* rw = reinterpret_cast<const unsigned*>(raw + (((long long)task * task_bytes) & 15));
#pragma unroll 4
      for (int i = lane; i < words; i += 32) {
        float lo, hi;
        Elem<TI>::unpack(rw[i], &lo, &hi);
        if (PW == 2) {
          *reinterpret_cast<float2*>(slot + 2 * i) = make_float2(lo, hi);
        } else {
          slot[i] = lo;
        }
      }
    } else {
      // (the tail of a tensor whose size is not a multiple of 16 bytes) plain loads
      const long long total_words = (total + PW - 1) / PW;
      for (int i = lane; i < words; i += 32) {
        const long long wi = e0 / PW + i;
        float lo = 0.f, hi = 0.f;
        if (wi < total_words) {
          if (PW == 2 && wi == total_words - 1 && (total & 1)) {
            // the tensor ends in the middle of this word: read the single element
            const unsigned short s = reinterpret_cast<const unsigned short*>(in)[total - 1];
            Elem<TI>::unpack((unsigned)s, &lo, &hi);
            hi = 0.f;
          } else {
            Elem<TI>::unpack(__ldg(in_words + wi), &lo, &hi);
          }
        }
        if (PW == 2) {
          *reinterpret_cast<float2*>(slot + 2 * i) = make_float2(lo, hi);
        } else {
          slot[i] = lo;
        }
      }
    }
    __syncwarp();
    // the raw bytes are consumed: fetch the next task
    staged = task + stride < ntasks ? issue(task + stride) : false;
    {
      float2 a[N];
      load_columns_staged<N>(slot + li * hw, &zero_storage, h, w, padL, padU, l, a);
      if (task * IPW + li >= B) {
#pragma unroll
        for (int y = 0; y < N; ++y) a[y] = make_float2(0.f, 0.f);
      }
      fft_bitrev<N, false>(a);
      fwd_separate_store<N>(a, ib, l);
    }
    __syncwarp();
    fwd_rows_unpack<N>(ib, l);
    // ---- IPW images x ROWS rows x N complex leave as vectors of four complex values
    constexpr int QR = N / 4;
#pragma unroll 2
    for (int e = lane; e < IPW * ROWS * QR; e += 32) {
      const int img = e / (ROWS * QR), rem = e % (ROWS * QR), row = rem / QR, q = rem % QR;
      const int b = task * IPW + img;
      if (b < B) {
        const float2* src = buf + img * IS + row * RS + q * 4;
        const float4 va = *reinterpret_cast<const float4*>(src), vb = *reinterpret_cast<const float4*>(src + 2);
        store_cplx4<TO>(out + (((long long)b * ROWS + row) * N + q * 4) * 2, va, vb);
      }
    }
    __syncwarp();
  }
}

// ------------------------------------------------------------------ inverse
// in: [B][N/2+1][N][2] of TI; out: [B][h][w] of TO, cropped at (padU, padL) of the canvas.
// The spectra of the next task arrive by one cp.async.bulk per task (they are contiguous and a
// multiple of 16 bytes) while the current one computes.
template <int N, typename TI, typename TO>
__global__ void __launch_bounds__(kThreads16, 3) fft2d_small_inv16_kernel(const TI* __restrict__ in, TO* __restrict__ out, int B,
                                                                         int h, int w, int padL, int padU, int ntasks,
                                                                         int slot_floats, int raw_bytes) {
  constexpr int T = N / 2, IPW = 32 / T, ROWS = T + 1, PW = Elem<TO>::kPerWord;
  constexpr int RS = SmallCfg<N>::RS, IS = SmallCfg<N>::IS;
  extern __shared__ __align__(16) float2 smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float2* buf = smem + warp * (IPW * IS);
  // the cropped fp32 image is staged in the work buffer itself, once the column pass holds it in registers
  float* slot = reinterpret_cast<float*>(buf);
  unsigned char* raw = reinterpret_cast<unsigned char*>(smem + kWarps16 * (IPW * IS)) + warp * raw_bytes;
  unsigned long long* bars =
      reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(smem + kWarps16 * (IPW * IS)) + kWarps16 * raw_bytes);
  const unsigned bar = smem_u32(bars + warp);
  if (lane == 0) mbar_init(bar, 1);
  fence_async_smem();
  __syncwarp();
  const int li = lane / T, l = lane % T;
  float2* ib = buf + li * IS;
  const int hw = h * w;
  const long long total = (long long)B * hw;
  unsigned* out_words = reinterpret_cast<unsigned*>(out);
  constexpr int IMG_ELEMS = ROWS * N * 2;  // storage elements per spectrum
  const int first = blockIdx.x * kWarps16 + warp, stride = gridDim.x * kWarps16;
  auto issue = [&](int task) {
    int imgs = B - task * IPW;
    if (imgs > IPW) imgs = IPW;
    if (lane == 0) {
      fence_async_smem();
      const unsigned bytes = (unsigned)(imgs * IMG_ELEMS * (int)sizeof(TI));
      mbar_expect_tx(bar, bytes);
      bulk_g2s(smem_u32(raw), in + (long long)task * IPW * IMG_ELEMS, bytes, bar);
    }
  };
  unsigned phase = 0;
  if (first < ntasks) issue(first);
  for (int task = first; task < ntasks; task += stride) {
    constexpr int QR = N / 4;
    if (!mbar_wait(bar, phase, kErrInv16Wait)) return;
    phase ^= 1;
    const TI* rsrc = reinterpret_cast<const TI*>(raw);
#pragma unroll 2
    for (int e = lane; e < IPW * ROWS * QR; e += 32) {
      const int img = e / (ROWS * QR), rem = e % (ROWS * QR), row = rem / QR, q = rem % QR;
      float4 va = make_float4(0.f, 0.f, 0.f, 0.f), vb = va;
      if (task * IPW + img < B) load_cplx4<TI>(rsrc + ((img * ROWS + row) * N + q * 4) * 2, &va, &vb);
      float2* dst = buf + img * IS + row * RS + q * 4;
      *reinterpret_cast<float4*>(dst) = va;
      *reinterpret_cast<float4*>(dst + 2) = vb;
    }
    __syncwarp();
    if (task + stride < ntasks) issue(task + stride);  // the raw spectra are consumed
    inv_pack_rows<N>(ib, l);
    {
      float2 z[N];
      inv_columns<N>(ib, l, z);
      __syncwarp();  // every lane holds its columns: the work buffer may take the image
      // the cropped image, still fp32, in the slot
      store_columns<N>(slot + li * hw, w, 1, h, w, padL, padU, l, z, 1.0f);
    }
    __syncwarp();
    const long long e0 = (long long)task * IPW * hw;
    long long cnt = total - e0;
    if (cnt > (long long)IPW * hw) cnt = (long long)IPW * hw;
    const int words = (int)(cnt / PW);
#pragma unroll 4
    for (int i = lane; i < words; i += 32) {
      out_words[e0 / PW + i] = PW == 2 ? Elem<TO>::pack(slot[2 * i], slot[2 * i + 1]) : Elem<TO>::pack(slot[i], 0.f);
    }
    if (PW == 2 && (cnt & 1) && lane == 0) {
      // the last element of a tensor with an odd element count
      const unsigned wv = Elem<TO>::pack(slot[cnt - 1], 0.f);
      reinterpret_cast<unsigned short*>(out)[e0 + cnt - 1] = (unsigned short)(wv & 0xffffu);
    }
    __syncwarp();
  }
}

template <int N, typename TI, typename TO>
int launch16(bool inverse, const void* src, void* dst, int B, int h, int w, int padL, int padU, cudaStream_t s) {
  constexpr int IPW = 32 / (N / 2), ROWS = N / 2 + 1;
  const int ntasks = (B + IPW - 1) / IPW;
  const int slot_floats = ((IPW * h * w + 3) / 4) * 4 + 4;
  // raw staging per warp: the task's images plus alignment slack (forward), the task's spectra (inverse)
  const int raw_bytes = inverse ? IPW * ROWS * N * 2 * (int)sizeof(TI) : ((IPW * h * w * (int)sizeof(TI) + 15) / 16) * 16 + 32;
  // (the inverse stages its fp32 image inside the work buffer: no slot of its own)
  const int smem = kWarps16 * (IPW * SmallCfg<N>::IS * 8 + (inverse ? 0 : slot_floats * 4) + raw_bytes + 8);
  const int want = (ntasks + kWarps16 - 1) / kWarps16, cap = sm_count() * 3;
  const int grid = want < cap ? want : cap;
  if (inverse) {
    auto k = fft2d_small_inv16_kernel<N, TI, TO>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    k<<<grid, kThreads16, smem, s>>>(static_cast<const TI*>(src), static_cast<TO*>(dst), B, h, w, padL, padU, ntasks, slot_floats,
                                     raw_bytes);
  } else {
    auto k = fft2d_small_fwd16_kernel<N, TI, TO>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    k<<<grid, kThreads16, smem, s>>>(static_cast<const TI*>(src), static_cast<TO*>(dst), B, h, w, padL, padU, ntasks, slot_floats,
                                     raw_bytes);
  }
  return cudaPeekAtLastError() == cudaSuccess ? kSuccess : kCudaError;
}

template <int N, typename TI>
int by_out(bool inverse, int out_type, const void* src, void* dst, int B, int h, int w, int padL, int padU, cudaStream_t s) {
  switch (out_type) {
    case FBFFT_STORAGE_F32:
      return launch16<N, TI, float>(inverse, src, dst, B, h, w, padL, padU, s);
    case FBFFT_STORAGE_F16:
      return launch16<N, TI, __half>(inverse, src, dst, B, h, w, padL, padU, s);
    default:
      return launch16<N, TI, __nv_bfloat16>(inverse, src, dst, B, h, w, padL, padU, s);
  }
}

template <int N>
int by_in(bool inverse, int in_type, int out_type, const void* src, void* dst, int B, int h, int w, int padL, int padU,
          cudaStream_t s) {
  switch (in_type) {
    case FBFFT_STORAGE_F32:
      return by_out<N, float>(inverse, out_type, src, dst, B, h, w, padL, padU, s);
    case FBFFT_STORAGE_F16:
      return by_out<N, __half>(inverse, out_type, src, dst, B, h, w, padL, padU, s);
    default:
      return by_out<N, __nv_bfloat16>(inverse, out_type, src, dst, B, h, w, padL, padU, s);
  }
}

}  // namespace

// src / dst are the real and complex tensors in the direction of the transform; types are FBFFT_STORAGE_*
int fft2d_small_storage(int n, bool inverse, int src_type, int dst_type, const void* src, void* dst, int B, int h, int w,
                        int padL, int padU, cudaStream_t s) {
  if (B <= 0) return kSuccess;
  switch (n) {
    case 8:
      return by_in<8>(inverse, src_type, dst_type, src, dst, B, h, w, padL, padU, s);
    case 16:
      return by_in<16>(inverse, src_type, dst_type, src, dst, B, h, w, padL, padU, s);
    case 32:
      return by_in<32>(inverse, src_type, dst_type, src, dst, B, h, w, padL, padU, s);
    default:
      return kUnsupportedSize;
  }
}

}  // namespace fbfft_b200
