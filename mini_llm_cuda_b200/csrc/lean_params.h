// Parameters of the shape-specialised whole-GPU decode kernel (lean.cuh), shared with the host code
// that lays out its shared memory and exchange buffers.
#pragma once
#include <cstdint>

namespace mlb {

struct StepLayer;

constexpr int kLeanWarps = 16;                       // consumer warps
constexpr int kLeanConsumers = kLeanWarps * 32;
constexpr int kLeanThreads = kLeanConsumers + 32;    // + the producer warp
constexpr int kLeanStage = 16 * 1024;                // ring stage
constexpr int kLeanDirectWords = 4096;
constexpr int kLeanTraceLen = 256;                 // events per CTA of the diagnostic trace

__host__ __device__ constexpr int lean_slot(int rpc) { return (rpc + 15) / 16 * 16; }

struct LeanParams {
    const StepLayer* layers;
    int n_layers;
    const void* E; const float* g_final; const float* rope; const int* page_table;
    float* logits;
    int* err;
    int with_lm_head, do_pick, tok_arg;
    unsigned int* epoch;
    // exchange buffers: C slots each (parts: one slot per attention item)
    unsigned long long *x, *xb, *pj, *parts, *a, *ah, *h, *lm;
    float eps, l2_eps;
    int pages_per_split;
    int n_stages;                  // ring stages of kLeanStage bytes
    long long* timers;             // [C][kGridTimerSlots] or null
    long long* trace;              // [C][kLeanTraceLen] (globaltimer << 8 | event) of the last step, or null
    // shared-memory float offsets
    int off_xs, xs_stride, off_xa, off_xb, off_parts, off_mix, off_pacc, off_red, off_layers, off_plan, off_timers, off_bar, off_ring;
};

}  // namespace mlb
