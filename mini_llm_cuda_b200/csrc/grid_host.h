// Host entry points of the whole-GPU batch-1 decode kernel (defined in grid.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

namespace mlb {
struct StepCtl;
struct GridParams;
// Resident CTAs per SM with `smem` bytes of dynamic shared memory (0: the kernel does not fit).
int grid_kernel_probe(int weight_dtype, int kv_dtype, size_t smem, int* per_sm);
// Cooperative launch of `ctas` CTAs on `st`.
cudaError_t grid_kernel_launch(int weight_dtype, int kv_dtype, int ctas, size_t smem, cudaStream_t st, const StepCtl& c,
                               const GridParams& p);
}  // namespace mlb
