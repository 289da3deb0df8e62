// Error codes of the fbfft entry points, with the reference's numeric values
// (fbfft/FBFFTParameters.h:9-14).  The builder fields of the reference class are not read by
// any entry point and are not reproduced.
#pragma once
namespace facebook { namespace cuda { namespace fbfft {
class FBFFTParameters {
 public:
  enum ErrorCode { Success = 0, UnsupportedSize = 1, UnsupportedDimension = 2, CudaError = 3 };
};
}}}  // namespace facebook::cuda::fbfft
