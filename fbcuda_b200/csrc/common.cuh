// Shared host/device definitions for the fbfft kernels.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace fbfft_b200 {

// Numeric values of the reference's FBFFTParameters::ErrorCode
// (fbfft/FBFFTParameters.h:9-14).
enum ErrorCode : int {
  kSuccess = 0,
  kUnsupportedSize = 1,
  kUnsupportedDimension = 2,
  kCudaError = 3,
};

// A batch of real images: element (b, y, x) at p[b*sb + y*sy + x*sx].
struct RealView {
  float* p;
  long long sb;
  int sy, sx;
  int h, w;
};

// A batch of complex matrices stored as floats: element (b, r, c, z) at
// p[b*sb + r*sr + c*sc + z*sz], z = 0 (re) or 1 (im).
//
// blk_planes > 0 selects the bin-blocked layouts of the convolution workspace instead: the
// (N/2+1)*N stored bins of a plane are cut into blocks of blk_bins bins and block xb of plane b
// sits at p[((xb * blk_planes + b) * blk_bins + x % blk_bins) * 2], so that for a fixed block all
// planes are adjacent.  sb/sr/sc/sz are ignored then.  Two block sizes are in use:
//   blk_bins = 4   the contraction's operands (written by the forward transforms): a 4-bin tile of
//                  consecutive planes is one contiguous run;
//   blk_bins = N   the contraction's result (read by the inverse transforms): a block is one stored
//                  row of the spectrum, fetched by one bulk copy.
struct CplxView {
  float* p;
  long long sb;
  int sr, sc, sz;
  long long blk_planes = 0;
  int blk_bins = 4;
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device, cached per device (the reference caches
// cudaDeviceProp for its grid sizing, util/CachedDeviceProperties.cpp:45-64).
int sm_count();

void set_last_error(const char* msg);

}  // namespace fbfft_b200
