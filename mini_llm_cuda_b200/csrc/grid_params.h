// Parameters of the whole-GPU batch-1 decode kernel (grid.cuh), shared with the host code that
// lays out its shared memory and exchange buffers.
#pragma once
#include <cstdint>

namespace mlb {

struct MegaLayer;

// How the rows of a phase are finished: published as they are, added to the residual stream, kept
// as this CTA's per-layer-embedding contribution, SiLU(gate) * up, or logits with a running argmax.
enum { RJ_STORE = 0, RJ_RESID = 1, RJ_PACC = 2, RJ_SWIGLU = 3, RJ_LM = 4 };

// One phase of the step that streams weights: what to fetch first, what to normalise, which rows to
// multiply and how to finish them. The host fills the list once per session (the step is the same
// list every time); the kernel copies it to shared memory and adds this CTA's row range.
enum {
    GP_PAIR = 1,          // gate and up matrices, chunk-interleaved
    GP_T2 = 2,            // rows of a per-layer-embedding projection (its own element type)
    GP_PACC_IN = 4,       // add this CTA's per-layer-embedding contribution to the rows
    GP_FILL_PLE = 8,      // starts with the table row of the pending token
    GP_MIX_ATTN = 16,     // followed by the attention items and the split combine
    GP_MIX_DELTA = 32,    // followed by the gated delta-net update
    GP_SKIP_GATHER_IF_READY = 64,   // the input may already stand in shared memory (direct combine)
    GP_LM = 128           // the LM head (left out of the prompt chain)
};
struct alignas(16) GridPhase {
    const void* W; const void* W2;                    // row-major weights (W2: the up matrix)
    const float* scale; const float* scale2;          // FP8 row scales or null
    const float* gain; const void* ple_table;         // RMS-norm gain or null; per-layer-embedding table
    const unsigned long long* g_src; unsigned long long* dst;   // exchange words to fetch first / to publish
    float* logits; long long reserved;
    int N, K, row_bytes, mode;                        // rows of the matrix, row length, bytes per row, RJ_*
    int g_n, g_perm, g_e_off, g_dst_off;              // fetch: words, GEMV-layout vectors (0: linear), epoch, shared-memory offset
    int e_off, resid_off, xs_off, nsrc_off;           // epoch of the output; residual, input, norm source offsets (-1: none)
    int flags, layer, mix_e2_off, mix_ea_off;         // GP_*; layer; epochs of the mixer's partials and output
    int r0, rows, pad0, pad1;                         // this CTA's rows (filled in the kernel)
};
static_assert(sizeof(GridPhase) == 160, "GridPhase is copied in 16-byte words");

struct GridParams {
    const GridPhase* phases;
    int n_phases;                  // with the LM head as the last one
    int e_total, e_total_nolm;     // epochs one step takes (decode / prompt chain)
    int off_phases;                // shared-memory copy of the list (16-byte aligned)
    const MegaLayer* layers;
    int n_layers;
    int d, F, V, heads, kv_heads, hd, dk, dv, ple, qk_norm;
    float eps, l2_eps;
    const void* E; const float* Es; const float* g_final; const float* rope;
    const int* page_table; int pt_stride;
    float* logits;                 // [V]
    int* err;                      // device word: 0 = ok, else the code of the wait that ran out
    int with_lm_head;              // 0 in the prompt chain
    int do_pick;                   // greedy pick + advance inside the kernel
    // exchange buffers in global memory, 8-byte {value bits, epoch} words
    unsigned long long *ll_xa, *ll_xb, *ll_proj, *ll_parts, *ll_a, *ll_h, *ll_lm;
    unsigned int* epoch;           // epoch of the last phase of the previous step
    int s_max;                     // most context splits per kv head the partial buffers hold
    long long* timers;             // diagnostic: [CTA][kGridTimers] cycle counters, or null
    // shared-memory layout (float offsets), identical in every CTA
    int off_x, off_x2, off_xn, off_proj, off_parts, off_a, off_h, off_tmp, off_ple, off_pacc, off_red;
    int off_layers;                // copy of the per-layer table (8-byte aligned)
    int off_timers;                // kGridTimers 8-byte counters (8-byte aligned)
    int off_bar;                   // mbarriers: full[nst] then empty[nst] (8 bytes each)
    int off_ring;                  // ring stages (128-byte aligned)
    int n_stages, stage_bytes;
    int backoff_ns;                // the producer's pause between polls for a free ring stage
};

constexpr uint32_t kGridSpinLimit = 1u << 21;       // polls of one word group before giving up (~1 s)
constexpr int kGridAttnWarps = 8;
constexpr int kGridDirectWords = 4096;              // partials every CTA may fetch itself (else the heads' owners combine)
// Diagnostic cycle counters of thread 0 of every CTA, summed over the steps (kept only by a
// build with -DMLB_GRID_TIMERS): 0 whole step, 1 gathers, 2 norms, 3 rows, 4 attention items,
// 5 split combine, 6 delta-net phase, 8 phase set-up, 14 waiting for weight chunks, 15 repeated polls.
constexpr int kGridTimers = 16;

}  // namespace mlb
