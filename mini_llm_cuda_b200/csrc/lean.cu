// Instantiations and launch of the shape-specialised whole-GPU decode kernel (lean.cuh).
#include <cstring>

#include "../../include/mlb.h"
#include "lean.cuh"
#include "lean_host.h"

namespace mlb {

// The shapes that are built. 128 CTAs: every row count of these models that must divide does.
using ShapeCfg1 = LeanShape<512, 1408, 8192, 8, 8, 64, 64, 64, 64, 128>;      // 1-GPU latency configuration (d=512, 8 heads x 64, ffn 1408, PLE 64)

template <typename S>
static LeanShapeInfo info_of() {
    LeanShapeInfo i;
    i.D = S::D; i.F = S::F; i.V = S::V; i.H = S::H; i.KVH = S::KVH; i.HD = S::HD; i.DK = S::DK; i.DV = S::DV; i.PLE = S::PLE; i.C = S::C;
    i.slot_x = lean_slot(S::RX); i.slot_qa = lean_slot(S::RQA); i.slot_qd = lean_slot(S::RQD); i.slot_parts = lean_slot(S::G * S::W);
    i.slot_a = lean_slot(S::RAD); i.slot_ah = lean_slot(S::HD); i.slot_h = lean_slot(S::RH);
    i.xs_floats = S::D > S::F ? S::D : S::F;
    if (S::NA_A > i.xs_floats) i.xs_floats = S::NA_A;
    const int s_cap = S::C / S::KVH;
    i.parts_floats = kLeanDirectWords > s_cap * S::W ? kLeanDirectWords : s_cap * S::W;
    if (2 * S::C > i.parts_floats) i.parts_floats = 2 * S::C;
    const int attn_n = S::G * S::HD + 2 * S::HD + kLeanWarps * S::W + ((S::G * S::W + 31) / 32) * 2 * kLeanWarps;
    const int dn_n = 2 * S::H * S::DK + ((S::RAD + 3) & ~3) + 2 * S::H + 8;
    i.mix_floats = attn_n > dn_n ? attn_n : dn_n;
    if (i.mix_floats < 64) i.mix_floats = 64;
    i.rx = S::RX;
    return i;
}

static const LeanShapeInfo kShapes[] = {info_of<ShapeCfg1>()};
static const int kNumShapes = 1;

int lean_find_shape(const mlb_config& c) {
    if (c.weight_dtype != MLB_DT_BF16 || c.qk_norm || c.query_gating) return -1;
    for (int i = 0; i < kNumShapes; ++i) {
        const LeanShapeInfo& s = kShapes[i];
        if (c.dim == s.D && c.ffn_dim == s.F && c.vocab == s.V && c.heads == s.H && c.kv_heads == s.KVH && c.head_dim == s.HD &&
            c.dn_key_dim == s.DK && c.dn_value_dim == s.DV && c.ple_dim == s.PLE)
            return i;
    }
    return -1;
}
const LeanShapeInfo& lean_shape_info(int idx) { return kShapes[idx]; }

template <typename S, typename KVT>
static int probe_one(size_t smem, int* per_sm) {
    *per_sm = 0;
    if (cudaFuncSetAttribute(lean_decode_kernel<S, KVT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, lean_decode_kernel<S, KVT>, kLeanThreads, smem) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    *per_sm = n;
    return 0;
}

template <typename S, typename KVT>
static cudaError_t launch_one(size_t smem, cudaStream_t st, const StepCtl& c, const LeanParams& p) {
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(S::C);
    cfg.blockDim = dim3(kLeanThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // the CTAs wait on one another: all resident or no launch
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, lean_decode_kernel<S, KVT>, c, p);
}

int lean_kernel_probe(int idx, int kvdt, size_t smem, int* per_sm) {
    if (idx != 0) { *per_sm = 0; return 0; }
    if (kvdt == MLB_DT_F32) return probe_one<ShapeCfg1, float>(smem, per_sm);
    return probe_one<ShapeCfg1, bf16_t>(smem, per_sm);
}

cudaError_t lean_kernel_launch(int idx, int kvdt, size_t smem, cudaStream_t st, const StepCtl& c, const LeanParams& p) {
    if (idx != 0) return cudaErrorInvalidValue;
    if (kvdt == MLB_DT_F32) return launch_one<ShapeCfg1, float>(smem, st, c, p);
    return launch_one<ShapeCfg1, bf16_t>(smem, st, c, p);
}

}  // namespace mlb
