// Internal interface of the data-parallel communicator (dp_nccl.cu), used by the
// convolution passes (conv.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

namespace fbfft_b200 {

struct Comm;
int comm_rank(const Comm* c);
int comm_world(const Comm* c);
// in-place sum over the ranks of `count` floats
int comm_all_reduce(Comm* c, float* buf, size_t count, cudaStream_t s);
// `rows` in-place reduce-scatters as one group: row i covers world * count floats from base + i * row_stride;
// this rank ends up with the sums of the floats at rank * count of every row
int comm_reduce_scatter_rows(Comm* c, float* base, int rows, size_t row_stride, size_t count, cudaStream_t s);
// in-place all-gather: every rank contributes the `count` floats at base + rank * count
int comm_all_gather(Comm* c, float* base, size_t count, cudaStream_t s);

}  // namespace fbfft_b200
