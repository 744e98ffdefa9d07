// Parameters of the whole-GPU batch-1 decode kernel (grid.cuh), shared with the host code that
// lays out its shared memory and exchange buffers.
#pragma once
#include <cstdint>

namespace mlb {

struct StepLayer;

// One exchanged vector: N values made by the first P CTAs, CTA c owning the contiguous rows
// [r0(c), r0(c+1)) with r0(c) = floor(c * N / P). A producer's rows stand in a slot of its own
// (slotw 8-byte words, a multiple of 16: whole 128-byte lines), so that a line has one writer.
// Measured on B200: with the words packed densely (several writers per line) an all-to-all of 512
// words among 148 CTAs costs 2.4 us, with one slot per writer 1.2 us.
struct GridVec {
    unsigned long long* buf;
    int N, P;
    int rpc;               // most rows per producer, ceil(N / P)
    int slotw;             // 8-byte words per slot
    unsigned magic;        // q / rpc == __umulhi(q, magic) for every q < P * rpc (checked on the host); 0: rpc == 1
    int tab;               // shared-memory float offset of the row table r0[0..P] (ints, filled by the kernel)
    float inv_n;           // 1 / N
    int pad;
};
constexpr int kGridVecs = 8;   // the vectors of GridParams, vx first, stand one after the other

struct GridParams {
    const StepLayer* layers;
    int n_layers;
    int d, F, V, heads, kv_heads, hd, dk, dv, ple, qk_norm;
    float eps, l2_eps;
    const void* E; const float* Es; const float* g_final; const float* rope;
    const int* page_table;
    float* logits;                 // [V]
    int* err;                      // device word: 0 = ok, else the code of the wait that ran out
    int with_lm_head;              // 0 in the prompt chain
    int do_pick;                   // greedy pick + advance inside the kernel
    int tok_arg;                   // >= 0: the pending token, passed with the launch instead of read from StepCtl::tok
    unsigned int* epoch;           // epoch of the last phase of the previous step
    // exchanged vectors (kGridVecs of them, contiguous, vx first)
    GridVec vx, vxb;               // residual stream after the FFN / after the mixer (N = d)
    GridVec vproj_attn, vproj_dn;  // raw projections of an attention / a delta-net layer (N = n_qkv)
    GridVec vh;                    // FFN hidden (N = F)
    GridVec va_dn;                 // delta-net output (N = heads * dv)
    GridVec va_head;               // attention output combined by the heads' owners (N = heads * hd, P = heads)
    GridVec vlm;                   // per-CTA argmax pairs (N = 2 * C)
    unsigned long long* parts;     // flash-decode partials: item i at parts + i * parts_slotw, G * (hd + 2) words
    int parts_slotw;
    int vocab_tab;                 // row table of the LM head (shared-memory float offset)
    int s_max;                     // most context splits per kv head (two-level combine)
    int s_direct;                  // most splits whose partials every CTA fetches itself
    int pages_per_split;           // target pages per attention item
    long long* timers;             // diagnostic: [CTA][kGridTimerSlots] or null
    // shared-memory layout (float offsets), identical in every CTA
    int xs_stride;                 // floats between the two input buffers at off_xs
    int off_xs, off_xa, off_xb, off_parts, off_gate, off_mix, off_pacc, off_red, off_tabs, off_layers, off_timers, off_plan, off_obuf;
    int off_bar;                   // mbarriers: full[nst] then empty[nst] (8 bytes each)
    int off_ring;                  // ring stages (128-byte aligned)
    int n_stages, stage_bytes;
    int backoff_ns;                // the producer's pause between polls for a free ring stage
};

constexpr uint32_t kGridSpinLimit = 1u << 21;       // polls of one word group before giving up (~1 s)
constexpr int kGridDirectWords = 4096;              // partials every CTA may fetch itself (else the heads' owners combine)
// Diagnostic cycle counters of thread 0 of every CTA, summed over the steps (a session made with
// MLB_GRID_TIMERS=1 allocates them): per phase kind the cycles spent waiting for the input, and the cycles
// from the input's arrival to the end of the phase.
//   0 whole step   1 prologue
//   2/3 projection rows (wait / work)   4/5 attention items   6/7 head-owner combine   8/9 output projection
//   10/11 delta-net   12/13 gate+up   14/15 down   16/17 LM head   18 waiting for weight chunks
constexpr int kGridTimerSlots = 32;

}  // namespace mlb
