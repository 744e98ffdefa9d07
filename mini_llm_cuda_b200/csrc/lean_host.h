// Host entry points of the shape-specialised whole-GPU decode kernel (defined in lean.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

struct mlb_config;

namespace mlb {
struct StepCtl;
struct LeanParams;
// What the host needs to lay out the exchange buffers and the shared memory of a built shape.
struct LeanShapeInfo {
    int D, F, V, H, KVH, HD, DK, DV, PLE, C;
    int slot_x, slot_qa, slot_qd, slot_parts, slot_a, slot_ah, slot_h;    // 8-byte words per producer slot of each exchanged vector
    int xs_floats, parts_floats, mix_floats, rx;                             // shared-memory areas (floats); rows of the residual stream per CTA
};
// Index of the built shape that matches the model, or -1 (the generic kernel serves it).
int lean_find_shape(const mlb_config& c);
const LeanShapeInfo& lean_shape_info(int idx);
// Resident CTAs per SM with `smem` bytes of dynamic shared memory (0: the kernel does not fit).
int lean_kernel_probe(int idx, int kv_dtype, size_t smem, int* per_sm);
// Cooperative launch of the shape's CTAs on `st`.
cudaError_t lean_kernel_launch(int idx, int kv_dtype, size_t smem, cudaStream_t st, const StepCtl& c, const LeanParams& p);
}  // namespace mlb
