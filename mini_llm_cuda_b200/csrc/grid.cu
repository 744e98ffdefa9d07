// Instantiations and launch of the whole-GPU batch-1 decode kernel (grid.cuh), in a translation
// unit of their own so that they build in parallel with the kernel chain.
#include <cstring>

#include "../../include/mlb.h"
#include "grid.cuh"
#include "grid_host.h"

namespace mlb {

template <typename T, typename T2, typename KVT>
static int probe_one(size_t smem, int* per_sm) {
    *per_sm = 0;
    if (cudaFuncSetAttribute(grid_decode_kernel<T, T2, KVT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, grid_decode_kernel<T, T2, KVT>, kRingThreads, smem) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    *per_sm = n;
    return 0;
}

template <typename T, typename T2, typename KVT>
static cudaError_t launch_one(int ctas, size_t smem, cudaStream_t st, const StepCtl& c, const GridParams& p) {
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(kRingThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // the CTAs wait on one another: all resident or no launch
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, grid_decode_kernel<T, T2, KVT>, c, p);
}

#define MLB_GRID_DISPATCH(fn, ...)                                                                   \
    if (wdt == MLB_DT_F32 && kvdt == MLB_DT_F32) return fn<float, float, float>(__VA_ARGS__);        \
    if (wdt == MLB_DT_F32 && kvdt == MLB_DT_BF16) return fn<float, float, bf16_t>(__VA_ARGS__);      \
    if (wdt == MLB_DT_BF16 && kvdt == MLB_DT_F32) return fn<bf16_t, bf16_t, float>(__VA_ARGS__);     \
    if (wdt == MLB_DT_BF16 && kvdt == MLB_DT_BF16) return fn<bf16_t, bf16_t, bf16_t>(__VA_ARGS__);   \
    if (wdt == MLB_DT_FP8_E4M3 && kvdt == MLB_DT_F32) return fn<fp8_t, bf16_t, float>(__VA_ARGS__);  \
    return fn<fp8_t, bf16_t, bf16_t>(__VA_ARGS__);

int grid_kernel_probe(int wdt, int kvdt, size_t smem, int* per_sm) { MLB_GRID_DISPATCH(probe_one, smem, per_sm) }

cudaError_t grid_kernel_launch(int wdt, int kvdt, int ctas, size_t smem, cudaStream_t st, const StepCtl& c, const GridParams& p) {
    MLB_GRID_DISPATCH(launch_one, ctas, smem, st, c, p)
}

}  // namespace mlb
