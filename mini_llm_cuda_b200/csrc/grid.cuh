// Batch-1 decode step as ONE persistent kernel over the whole GPU.
//
// A decode step of one sequence is a chain of ~5 dependent matrix-vector phases per layer. As a
// chain of kernels every phase pays a launch boundary; here one CTA per SM lives for the whole
// step and a phase boundary is one exchange of a few hundred values through L2.
//   * Every phase splits its output rows evenly over the CTAs. A CTA's rows of a weight matrix
//     are one contiguous slab, streamed by a producer warp with cp.async.bulk into a ring of
//     shared-memory stages. The producer depends on nothing but free stages, so it runs phases
//     ahead of the consumers: weights, the K/V pages of the CTA's attention item and its rows of
//     the delta-net state are in shared memory before the activations that need them arrive.
//   * Activations cross CTAs as 8-byte {value, epoch} words. A reader polls the words themselves
//     until they carry the epoch of the phase it waits for: no grid barrier, no flag, no fence.
//     Every producer writes into a slot of its own (whole 128-byte lines): a line polled by all
//     CTAs has exactly one writer. (Measured on B200: an all-to-all of 512 words among 148 CTAs
//     costs 2.4 us with densely packed words, 1.2 us with one slot per writer; the hop from one
//     SM's store to another SM's successful poll is 0.25 us within a die, 0.45 us across dies.)
//   * The RMS norm in front of a projection is applied after the dot products: the gathered
//     values are multiplied by the gain on their way into shared memory, every warp adds up the
//     squares while its dot products run, and a row's sum is scaled by one over the norm at the
//     end. One block barrier per phase instead of three.
//   * The attention phase works on (kv head, context split) items out of shared memory. The item
//     that holds the current position applies QK-norm and RoPE to the raw projections itself,
//     appends the K/V row to the paged pool and uses it from shared memory, so no CTA waits for
//     another one's pool write.
//   * Code size is a first-order cost. A step walks through its code once per layer and a warp
//     runs only a few hundred instructions per phase; on B200 about 32 KB of instructions stay
//     resident per SM, beyond that straight-line code is fetched at ~6 cycles per instruction and
//     every taken branch to a cold line stalls for an L2 round trip. With the phases inlined one
//     after the other (310 KB) a step took 330 us. So: ONE loop body serves all projection phases,
//     the fetch helpers are functions of their own, divisions / square roots / exponentials use
//     the hardware approximations (each exact form is 0.5-2 KB of code), and what depends on the
//     position only (the attention plan) is computed once per step.
// An exchange buffer is rewritten one layer after its last reader has left it: between the two,
// every CTA has produced rows that every CTA fetched (all projection phases have at least as many
// rows as there are CTAs), which orders the old reads before the new writes.
//
// The arithmetic of every phase is the one of the chain kernels in kernels.cuh (same reference
// citations); only the partition of rows and of the attention context differs, and the
// approximations named above (relative error ~1e-6, far inside the 1e-3 bound of the fp32 tests).
//
// The CTAs wait on one another, so the kernel is launched cooperatively (all CTAs co-resident
// or the launch fails). Every wait is bounded: when one runs out the kernel records an error
// code, stops waiting (later waits return at once) and still walks to the end, so it always
// terminates and the host reports MLB_E_TIMEOUT.
#pragma once
#include <type_traits>

#include "grid_params.h"
#include "ring.cuh"

#ifndef MLB_POLL_SLEEP
#define MLB_POLL_SLEEP 100
#endif

namespace mlb {

__device__ __forceinline__ void ll_store(unsigned long long* p, float v, uint32_t e) {
    const unsigned long long w = ((unsigned long long)e << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ll_load(const unsigned long long* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ float fast_sigmoid(float v) { return __fdividef(1.0f, 1.0f + __expf(-v)); }

// What depends on the position only, computed once per step by thread 0 (shared memory, ints).
// How the context is cut into attention items (kv head, split) and which item this CTA has.
struct GridPlan {
    int S, pps, direct;            // splits per kv head, pages per split, 1: every CTA combines the splits itself
    int has, kvh, split;           // this CTA's item (has = 0: none)
    int pg_begin, n_prev, pages_prev, cur_here;   // its first page, its earlier positions / pages holding them, 1: it holds the current position
    int pad0, pad1;
};

struct GridCtx {
    int C, rank, tok, pos, tid, lane, warp;
    uint32_t base;                 // epoch before this step
    float* smem;
    const int* tabs;               // shared memory seen as ints (row tables)
    volatile int* dead;
    int* err;
    const StepLayer* layers;       // the per-layer table in shared memory
    const GridPlan* plan;          // in shared memory
    long long* tm;                 // diagnostic counters in shared memory (thread 0 writes), or null
    long long tmark;
    Ring ring;
};

// thread 0: add the cycles since the last mark to counter i
__device__ __forceinline__ void grid_mark(GridCtx& k, int i) {
    if (k.tm != nullptr && k.tid == 0) {
        const long long n = clock64();
        k.tm[i] += n - k.tmark;
        k.tmark = n;
    }
}

// This CTA's rows of an exchanged vector (none for a CTA beyond the vector's producers).
__device__ __forceinline__ void vec_rows(const GridVec& v, const int* tabs, int rank, int& r0, int& r1) {
    r0 = tabs[v.tab + min(rank, v.P)];
    r1 = tabs[v.tab + min(rank + 1, v.P)];
}
__device__ __forceinline__ unsigned long long* vec_slot(const GridVec& v, int rank) { return v.buf + (size_t)rank * v.slotw; }

// Poll until the four words carry epoch `e`; at most kGridSpinLimit rounds. The caller passes
// four valid addresses (a thread with fewer words repeats one).
__device__ __forceinline__ void ll_poll4(const unsigned long long* s0, const unsigned long long* s1, const unsigned long long* s2,
                                         const unsigned long long* s3, unsigned long long (&w)[4], uint32_t e, volatile int* dead, int* err) {
    uint32_t spins = 0;
#pragma unroll 1
    for (;;) {
        w[0] = ll_load(s0);
        w[1] = ll_load(s1);
        w[2] = ll_load(s2);
        w[3] = ll_load(s3);
        const bool ok = (uint32_t)(w[0] >> 32) == e && (uint32_t)(w[1] >> 32) == e && (uint32_t)(w[2] >> 32) == e && (uint32_t)(w[3] >> 32) == e;
        if (ok) break;
        if (*dead) break;
        __nanosleep(MLB_POLL_SLEEP);
        if (++spins > kGridSpinLimit) {
            *dead = 1;
            atomicExch(err, 3);
            break;
        }
    }
}

// The whole vector. Row r goes to lin[r] (if lin) and, multiplied by gain[r] (if gain), to the GEMV
// layout of nvec weight vectors at xs. Returns the sum of squares of what this thread fetched.
// The gains are asked for before the polls start. `tabs`: shared memory seen as ints.
template <int EPV>
__device__ __noinline__ float ll_gather_vec(const GridVec* vp, uint32_t e, const float* __restrict__ gain, float* lin, float* xs, int nvec,
                                            const int* tabs, volatile int* dead, int* err) {
    const int P = vp->P, rpc = vp->rpc, slotw = vp->slotw, tab = vp->tab;
    const unsigned magic = vp->magic;
    const unsigned long long* buf = vp->buf;
    const int n = P * rpc;
    float ss = 0.f;
#pragma unroll 1
    for (int q0 = threadIdx.x; q0 < n; q0 += kRingConsumers * 4) {
        const unsigned long long* src[4];
        unsigned long long w[4];
        int row[4];
        float g[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            // slot q of the vector: producer c, its j-th word. A thread past the end, or on the unused last
            // word of a producer with one row less, repeats the producer's first word and drops it.
            const int q = min(q0 + u * kRingConsumers, n - 1);
            const int c = magic ? (int)__umulhi((unsigned)q, magic) : q;
            const int j = q - c * rpc;
            const int r0 = tabs[tab + c], r1 = tabs[tab + c + 1];
            const bool valid = q0 + u * kRingConsumers < n && r0 + j < r1;
            row[u] = valid ? r0 + j : -1;
            src[u] = buf + (size_t)c * slotw + (valid ? j : 0);
            g[u] = (gain != nullptr && valid) ? gain[r0 + j] : 1.0f;
        }
        ll_poll4(src[0], src[1], src[2], src[3], w, e, dead, err);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (row[u] >= 0) {
                const float val = __uint_as_float((uint32_t)w[u]);
                if (lin) lin[row[u]] = val;
                xs[xs_index<EPV>(row[u], nvec)] = val * g[u];
                ss = fmaf(val, val, ss);
            }
        }
    }
    return ss;
}

// Rows [row0, row0 + n) of a vector to dst[0..n).
static __device__ __noinline__ void ll_gather_rows(const GridVec* vp, int row0, int n, uint32_t e, float* dst, const int* tabs, volatile int* dead,
                                            int* err) {
    const int P = vp->P, slotw = vp->slotw, tab = vp->tab;
    const float pn = (float)P * vp->inv_n;
    const unsigned long long* buf = vp->buf;
#pragma unroll 1
    for (int i0 = threadIdx.x; i0 < n; i0 += kRingConsumers * 4) {
        const unsigned long long* src[4];
        unsigned long long w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int row = row0 + min(i0 + u * kRingConsumers, n - 1);
            // owner of a row under r0(c) = floor(c N / P) is floor(((row + 1) P - 1) / N): estimated in
            // floating point (off by one at most), settled against the row table
            int c = min(P - 1, (int)(((float)row + 0.5f) * pn));
            if (tabs[tab + c] > row) --c;
            else if (tabs[tab + c + 1] <= row) ++c;
            src[u] = buf + (size_t)c * slotw + (row - tabs[tab + c]);
        }
        ll_poll4(src[0], src[1], src[2], src[3], w, e, dead, err);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i0 + u * kRingConsumers < n) dst[i0 + u * kRingConsumers] = __uint_as_float((uint32_t)w[u]);
    }
}

template <typename KVT> __device__ __forceinline__ float round_kv(float v);
template <> __device__ __forceinline__ float round_kv<float>(float v) { return v; }
template <> __device__ __forceinline__ float round_kv<bf16_t>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// ---- rows of a projection out of the ring ----------------------------------------------------------
// One job = this CTA's rows of one weight matrix (or of the gate/up pair). Local row r belongs to
// warp r % 15 whatever chunk of the ring it arrives in; lane 0 of the warp finishes the row
// (weight scale, norm, residual, activation) and publishes it.
enum { RJ_STORE = 0, RJ_RESID = 1, RJ_SWIGLU = 2, RJ_LM = 3 };
struct RowsJob {
    int mode, rows, K, r0;
    const float* xs;               // input vector, GEMV layout
    const float* scale;            // per-row weight scale (FP8) or null, by global row
    const float* scale2;           // the up matrix's scale (RJ_SWIGLU)
    unsigned long long* dst;       // this CTA's slot of the output vector, by local row
    uint32_t epoch;
    const float* resid;            // RJ_RESID: residual stream in shared memory, by global row
    const float* pacc;             // RJ_RESID: addend per local row, or null
    float* logits;                 // RJ_LM
    int norm_n;                    // > 0: scale by 1 / sqrt(sum(red[0..479]) / norm_n + eps) (the RMS norm, applied late)
    float eps;
    const float* red;
    float* obuf;                   // finished rows of this phase, by local row (shared memory)
    int* ocnt;                     // how many of them are finished (shared memory, zero between phases)
};

template <typename T>
__device__ __forceinline__ float smem_row_dot(const T* row, int nvec, const float* xs, int lane) {
    constexpr int EPV = Elem<T>::EPV;
    const float4* xp = reinterpret_cast<const float4*>(xs);
    float a0 = 0.f, a1 = 0.f;
#pragma unroll 1
    for (int vi = lane; vi < nvec; vi += 32) {
        float w[EPV];
        Elem<T>::unpack(*reinterpret_cast<const uint4*>(row + (size_t)vi * EPV), w);
#pragma unroll
        for (int q = 0; q < EPV / 4; ++q) {
            const float4 t = xp[q * nvec + vi];
            a0 = fmaf(w[4 * q], t.x, a0); a1 = fmaf(w[4 * q + 1], t.y, a1);
            a0 = fmaf(w[4 * q + 2], t.z, a0); a1 = fmaf(w[4 * q + 3], t.w, a1);
        }
    }
    return warp_sum(a0 + a1);
}

template <typename T>
__device__ __forceinline__ void consume_rows(Ring& r, const RowsJob& j, bool pair, int warp, int lane, float& bv, int& bi, long long* tm) {
    (void)tm;
    constexpr int EPV = Elem<T>::EPV;
    constexpr int NW = kRingWarps;
    const int K = j.K, rows = j.rows, nvec = K / EPV;
    const int rpc = max(1, r.stage_bytes / (K * (int)sizeof(T)));
    // the norm of the input (inference.cu:24-50, :83-95): every warp adds up the threads' sums of squares
    float rn = 1.0f;
    if (j.norm_n > 0) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < NW; ++i) t += j.red[lane + 32 * i];
        rn = rsqrtf(__fdividef(warp_sum(t), (float)j.norm_n) + j.eps);
    }
    int wrow = warp;                       // this warp's next local row
#pragma unroll 1
    for (int c0 = 0; c0 < rows; c0 += rpc) {
        const int n = min(rpc, rows - c0);
        const int ia = r.idx;
        r.wait(r.full0 + 8u * r.idx, r.phase, 2);
        r.advance();
        int ib = ia;
        if (pair) {                        // gate and up chunks alternate in the ring
            ib = r.idx;
            r.wait(r.full0 + 8u * r.idx, r.phase, 2);
            r.advance();
        }
        const T* A = reinterpret_cast<const T*>(r.stages + (size_t)ia * r.stage_bytes);
        const T* Bm = reinterpret_cast<const T*>(r.stages + (size_t)ib * r.stage_bytes);
#pragma unroll 1
        for (; wrow < c0 + n; wrow += NW) {
            const size_t off = (size_t)(wrow - c0) * K;
            const int row = j.r0 + wrow;
            // the row's scales come from global memory: asked for before the dot products, used after
            const float sv = j.scale ? j.scale[row] : 1.0f;
            const float su = j.scale2 ? j.scale2[row] : 1.0f;
            float v = smem_row_dot<T>(A + off, nvec, j.xs, lane);
            float u = 0.f;
            if (pair) u = smem_row_dot<T>(Bm + off, nvec, j.xs, lane);
            // The finished rows are collected in shared memory and the warp that finishes the CTA's last
            // one publishes the whole slot with one store instruction per 32 rows: a line that every CTA
            // polls must change once. (Measured on B200: rows stored one by one by their warps, a few
            // dozen cycles apart, make an exchange cost 3-4 us instead of 1.2 us.)
            int last = 0;
            if (lane == 0) {
                v = (v * sv) * rn;
                if (j.mode == RJ_SWIGLU) {
                    // applySiluToFFN + hadamardMultiplyFFN, inference.cu:262-281
                    v = __fdividef(v, 1.0f + __expf(-v)) * ((u * su) * rn);
                } else if (j.mode == RJ_RESID) {
                    if (j.pacc) v += j.pacc[wrow];
                    v += j.resid[row];
                }
                if (j.mode == RJ_LM) {
                    j.logits[row] = v;
                    if (v > bv || (v == bv && row < bi)) { bv = v; bi = row; }
                } else {
                    j.obuf[wrow] = v;
                    __threadfence_block();
                    last = atomicAdd(j.ocnt, 1) == rows - 1;
                }
            }
            if (j.mode != RJ_LM) {
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence_block();
#pragma unroll 1
                    for (int q = lane; q < rows; q += 32) ll_store(j.dst + q, j.obuf[q], j.epoch);
                    if (lane == 0) *j.ocnt = 0;
                }
            }
        }
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(r.empty0 + 8u * ia);
            if (pair) mbar_arrive(r.empty0 + 8u * ib);
        }
    }
}

// ---- attention ---------------------------------------------------------------------------------------
// Thread 0, once per step: how the context is cut into items (kv head, split) and which one is
// this CTA's. From the position alone, so that every CTA arrives at the same answer.
__device__ __forceinline__ void grid_make_plan(const GridParams& p, int pos, int C, int rank, GridPlan* g) {
    const int npages = pos / kKvBlock + 1, cur_page = pos / kKvBlock;
    const int s_cap = max(1, min(p.s_max, C / p.kv_heads));
    const int s_dir = max(1, min(p.s_direct, s_cap));
    int S = min(s_cap, (npages + p.pages_per_split - 1) / p.pages_per_split);
    int direct = S <= s_dir;
    if (!direct && (npages + s_dir - 1) / s_dir <= 2 * p.pages_per_split) {
        S = s_dir;                          // a little more work per item beats a second exchange
        direct = 1;
    }
    const int pps = (npages + S - 1) / S;
    S = (npages + pps - 1) / pps;
    g->S = S; g->pps = pps; g->direct = direct;
    g->has = rank < p.kv_heads * S;
    g->kvh = rank / S;
    g->split = rank - g->kvh * S;
    g->pg_begin = g->split * pps;
    const int pg_end = min(npages, g->pg_begin + pps);
    g->cur_here = g->has && cur_page >= g->pg_begin && cur_page < pg_end;
    g->n_prev = g->has ? max(0, min(pos, pg_end * kKvBlock) - g->pg_begin * kKvBlock) : 0;
    g->pages_prev = (g->n_prev + kKvBlock - 1) / kKvBlock;
    g->pad0 = 0; g->pad1 = 0;
}

// Flash-decode of this CTA's item out of shared memory: 15/G warps per query head, the positions of a
// chunk interleaved among them. Publishes G partial vectors (hd values, maximum, sum) in the item's slot.
template <typename KVT, int HD>
__device__ __forceinline__ void grid_attention(const GridParams& p, const StepLayer& L, GridCtx& k, uint32_t e_proj, uint32_t e_out) {
    constexpr int EPL = 16 / (int)sizeof(KVT);        // elements per lane per row
    constexpr int LPR = HD / EPL;                     // lanes per row
    constexpr int PPI = 32 / LPR;                     // positions per warp iteration
    static_assert(LPR <= 32 && PPI >= 1, "head_dim does not fit one warp row");
    const GridPlan& it = *k.plan;
    const int pos = k.pos, tid = k.tid, lane = k.lane, warp = k.warp;
    const int G = p.heads / p.kv_heads;
    const int WPH = max(1, kRingWarps / G);           // warps per query head
    const int kvh = it.kvh;
    const int h0 = kvh * G;
    const int lr = lane % LPR, grp = lane / LPR;
    const float inv_div = rsqrtf((float)HD);          // scores are divided by sqrt(hd), inference.cu:154
    float* tq = k.smem + p.off_mix;                   // [G][HD] queries of the item's heads
    float* tk = tq + G * HD;                          // [HD] this step's key row
    float* tv = tk + HD;                              // [HD] this step's value row
    float* wpart = tv + HD;                           // [15][HD+2]
    KVT* kpool = reinterpret_cast<KVT*>(L.kpool);
    KVT* vpool = reinterpret_cast<KVT*>(L.vpool);
    const int g = warp / WPH, sub = warp - g * WPH;
    const bool scanner = g < G;
    Ring& ring = k.ring;

    // (a) raw projections of the item's query heads (+ this step's key and value row)
    ll_gather_rows(&p.vproj_attn, h0 * HD, G * HD, e_proj, tq, k.tabs, k.dead, k.err);
    if (it.cur_here) {
        ll_gather_rows(&p.vproj_attn, L.nq + kvh * HD, HD, e_proj, tk, k.tabs, k.dead, k.err);
        ll_gather_rows(&p.vproj_attn, L.nq + L.nk + kvh * HD, HD, e_proj, tv, k.tabs, k.dead, k.err);
    }
    consumer_sync();
    grid_mark(k, 4);
    // (b) per-head RMS norm (inference.cu:52-81, :97-111) and RoPE on adjacent pairs
    //     (inference.cu:113-134): one warp per vector; the new K/V row goes to the pool.
    {
        const int nvecs = G + (it.cur_here ? 1 : 0);
        const size_t row_off = it.cur_here ? (((size_t)p.page_table[pos / kKvBlock] * p.kv_heads + kvh) * kKvBlock + (pos % kKvBlock)) * HD : 0;
        if (warp < nvecs) {
            const bool is_k = warp >= G;
            float* vec = is_k ? tk : tq + warp * HD;
            const float* gain = is_k ? L.gk + (size_t)kvh * HD : L.gq + (size_t)(h0 + warp) * HD;
            float rs = 1.f;
            if (p.qk_norm) {
                float ss = 0.f;
#pragma unroll 1
                for (int r = lane; r < HD; r += 32) ss = fmaf(vec[r], vec[r], ss);
                rs = rsqrtf(warp_sum(ss) * (1.0f / (float)HD) + p.eps);
            }
#pragma unroll 1
            for (int pr = lane; pr < HD / 2; pr += 32) {
                const int r = 2 * pr;
                float a = vec[r], cc = vec[r + 1];
                if (p.qk_norm) {
                    a = (a * rs) * gain[r];
                    cc = (cc * rs) * gain[r + 1];
                }
                const float2 cssn = *reinterpret_cast<const float2*>(p.rope + (size_t)pos * HD + r);
                float ra = cssn.x * a - cssn.y * cc, rc = cssn.y * a + cssn.x * cc;
                if (is_k) {
                    Elem<KVT>::put(kpool, row_off + r, ra);
                    Elem<KVT>::put(kpool, row_off + r + 1, rc);
                    ra = round_kv<KVT>(ra);
                    rc = round_kv<KVT>(rc);
                }
                vec[r] = ra;
                vec[r + 1] = rc;
            }
        } else if (it.cur_here && warp == nvecs) {
#pragma unroll 1
            for (int r = lane; r < HD; r += 32) {
                const float v = tv[r];
                Elem<KVT>::put(vpool, row_off + r, v);
                tv[r] = round_kv<KVT>(v);
            }
        }
    }
    consumer_sync();
    // (c) online softmax of this warp's head over this warp's share of the positions
    float q[EPL], acc[EPL], m = kNegBig, l = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        q[e] = scanner ? tq[g * HD + lr * EPL + e] * inv_div : 0.f;
        acc[e] = 0.f;
    }
    {
        const int page_bytes = kKvBlock * HD * (int)sizeof(KVT);
        const int ppc = max(1, min(32, ring.stage_bytes / page_bytes));
#pragma unroll 1
        for (int c0 = 0; c0 < it.pages_prev; c0 += ppc) {
            const int ia = ring.idx;
            ring.wait(ring.full0 + 8u * ring.idx, ring.phase, 2);
            ring.advance();
            const int ib = ring.idx;
            ring.wait(ring.full0 + 8u * ring.idx, ring.phase, 2);
            ring.advance();
            const KVT* Ks = reinterpret_cast<const KVT*>(ring.stages + (size_t)ia * ring.stage_bytes);
            const KVT* Vs = reinterpret_cast<const KVT*>(ring.stages + (size_t)ib * ring.stage_bytes);
            const int cnt = min(ppc * kKvBlock, it.n_prev - c0 * kKvBlock);      // earlier positions in this chunk
            if (scanner) {
#pragma unroll 1
                for (int j0 = sub * PPI; j0 < cnt; j0 += WPH * PPI) {
                    const int j = j0 + grp;
                    const bool valid = j < cnt;
                    const int jj = valid ? j : 0;
                    float kv[EPL], vv[EPL];
                    Elem<KVT>::unpack(*reinterpret_cast<const uint4*>(Ks + (size_t)jj * HD + lr * EPL), kv);
                    Elem<KVT>::unpack(*reinterpret_cast<const uint4*>(Vs + (size_t)jj * HD + lr * EPL), vv);
                    float s = 0.f;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) s = fmaf(q[e], kv[e], s);
#pragma unroll
                    for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                    s = valid ? s : kNegBig;
                    const float mn = fmaxf(m, s);
                    const float sc = __expf(m - mn), pe = valid ? __expf(s - mn) : 0.f;
                    l = l * sc + pe;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) acc[e] = fmaf(pe, vv[e], acc[e] * sc);
                    m = mn;
                }
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(ring.empty0 + 8u * ia);
                mbar_arrive(ring.empty0 + 8u * ib);
            }
        }
    }
    if (scanner) {
        if (it.cur_here && sub == 0) {
            // the current position, from shared memory
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) s = fmaf(q[e], tk[lr * EPL + e], s);
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (grp == 0) {
                const float mn = fmaxf(m, s);
                const float sc = __expf(m - mn), pe = __expf(s - mn);
                l = l * sc + pe;
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[e] = acc[e] * sc + pe * tv[lr * EPL + e];
                m = mn;
            }
        }
        // merge the position groups of the warp
#pragma unroll 1
        for (int o = LPR; o < 32; o <<= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m, o);
            const float lo = __shfl_xor_sync(0xffffffffu, l, o);
            const float mn = fmaxf(m, mo);
            const float sa = __expf(m - mn), sb = __expf(mo - mn);
            l = l * sa + lo * sb;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                const float ao = __shfl_xor_sync(0xffffffffu, acc[e], o);
                acc[e] = acc[e] * sa + ao * sb;
            }
            m = mn;
        }
        if (grp == 0) {
            float* w = wpart + (size_t)warp * (HD + 2);
#pragma unroll
            for (int e = 0; e < EPL; ++e) w[lr * EPL + e] = acc[e];
            if (lr == 0) { w[HD] = m; w[HD + 1] = l; }
        }
    }
    consumer_sync();
    // merge the warps of each head; one thread per element of the item's partials
    unsigned long long* dst = p.parts + (size_t)k.rank * p.parts_slotw;
#pragma unroll 1
    for (int idx = tid; idx < G * (HD + 2); idx += kRingConsumers) {
        const int gg = idx / (HD + 2), e = idx - gg * (HD + 2);
        const float* w0 = wpart + (size_t)gg * WPH * (HD + 2);
        float mn = kNegBig;
#pragma unroll 1
        for (int w = 0; w < WPH; ++w) mn = fmaxf(mn, w0[(size_t)w * (HD + 2) + HD]);
        float val = mn;
        if (e != HD) {
            val = 0.f;
#pragma unroll 1
            for (int w = 0; w < WPH; ++w) val = fmaf(w0[(size_t)w * (HD + 2) + e], __expf(w0[(size_t)w * (HD + 2) + HD] - mn), val);
        }
        ll_store(dst + idx, val, e_out);
    }
    // no barrier here: the next writer of this scratch (the split combine) passes one first
}

// Combine the context splits of heads [h_first, h_first + h_count) (+ query gating,
// inference.cu:241-250): fetches their partials and the gate projections; element i of those heads
// goes to the GEMV layout at xs (if xs), else into the slot `dst` with epoch e_out.
// One warp per (head, split) partial fetches it; one thread per output element combines.
template <int EPV>
__device__ __forceinline__ void grid_combine(const GridParams& p, const StepLayer& L, GridCtx& k, int h_first, int h_count, uint32_t e_proj,
                                             uint32_t e_parts, float* xs, int nvec, unsigned long long* dst, uint32_t e_out) {
    const int hd = p.hd, tid = k.tid, lane = k.lane, warp = k.warp, W = hd + 2, S = k.plan->S, G = p.heads / p.kv_heads;
    float* parts = k.smem + p.off_parts;           // [h_count][S][hd+2]
    float* gate = k.smem + p.off_gate;             // [h_count][hd]
    // partial (hl, sp): hd + 2 words of item (kv head, sp); 5 words per lane cover hd = 128
    int hl = warp / S, sp = warp - hl * S;
#pragma unroll 1
    for (int pi = warp; pi < h_count * S; pi += kRingWarps) {
        const int h = h_first + hl;
        const unsigned long long* src = p.parts + (size_t)((h / G) * S + sp) * p.parts_slotw + (h % G) * W;
        float* out = parts + (size_t)pi * W;
        unsigned long long w[4];
        const int e0 = lane, e1 = lane + 32, e2 = min(lane + 64, W - 1), e3 = min(lane + 96, W - 1);
        ll_poll4(src + e0, src + e1, src + e2, src + e3, w, e_parts, k.dead, k.err);
        out[e0] = __uint_as_float((uint32_t)w[0]);
        out[e1] = __uint_as_float((uint32_t)w[1]);
        out[e2] = __uint_as_float((uint32_t)w[2]);
        out[e3] = __uint_as_float((uint32_t)w[3]);
        if (lane + 128 < W) {
            ll_poll4(src + lane + 128, src + lane + 128, src + lane + 128, src + lane + 128, w, e_parts, k.dead, k.err);
            out[lane + 128] = __uint_as_float((uint32_t)w[0]);
        }
        // next partial of this warp
        sp += kRingWarps;
        while (sp >= S) { sp -= S; ++hl; }
    }
    if (L.ng) ll_gather_rows(&p.vproj_attn, L.nq + L.nk + L.nv + h_first * hd, h_count * hd, e_proj, gate, k.tabs, k.dead, k.err);
    consumer_sync();
#pragma unroll 1
    for (int i = tid; i < h_count * hd; i += kRingConsumers) {
        const int hh = i / hd, el = i - hh * hd;
        const float* pp = parts + (size_t)hh * S * W;
        // the factor that brings a split's sums to the head's common maximum
        float mn = kNegBig;
#pragma unroll 1
        for (int s2 = 0; s2 < S; ++s2) mn = fmaxf(mn, pp[(size_t)s2 * W + hd]);
        float lt = 0.f, at = 0.f;
#pragma unroll 1
        for (int s2 = 0; s2 < S; ++s2) {
            const float sc = __expf(pp[(size_t)s2 * W + hd] - mn);
            lt = fmaf(pp[(size_t)s2 * W + hd + 1], sc, lt);
            at = fmaf(pp[(size_t)s2 * W + el], sc, at);
        }
        float o = __fdividef(at, lt);
        if (L.ng) o *= fast_sigmoid(gate[i]);      // sigmoid of the gate projection (inference.cu:248)
        if (xs) xs[xs_index<EPV>(i, nvec)] = o;
        else ll_store(dst + i, o, e_out);
    }
}

// Gated delta-net step on this CTA's rows of the state (the arithmetic of delta_net_kernel); the
// rows come out of the ring, the new rows go back to global memory.
__device__ __forceinline__ void grid_delta_net(const GridParams& p, const StepLayer& L, GridCtx& k, uint32_t e_proj, uint32_t e_out, float* obuf, int* ocnt) {
    constexpr int NW = kRingWarps;
    const int H = p.heads, dk = p.dk, dv = p.dv, lane = k.lane, warp = k.warp;
    int r0, r1;
    vec_rows(p.va_dn, k.tabs, k.rank, r0, r1);
    const int rows = r1 - r0;
    if (rows <= 0) return;
    const int h_lo = r0 / dv, h_hi = (r1 - 1) / dv, nh = h_hi - h_lo + 1;
    float* mix = k.smem + p.off_mix;
    float* qn = mix;                        // [nh][dk]
    float* kn = qn + nh * dk;               // [nh][dk]
    float* rv = kn + nh * dk;               // [rows]
    float* gates = rv + ((rows + 3) & ~3);  // beta[nh] then alpha[nh]
    const int seg_k = H * dk, seg_v = 2 * H * dk, seg_b = seg_v + H * dv, seg_a = seg_b + H;
    ll_gather_rows(&p.vproj_dn, h_lo * dk, nh * dk, e_proj, qn, k.tabs, k.dead, k.err);
    ll_gather_rows(&p.vproj_dn, seg_k + h_lo * dk, nh * dk, e_proj, kn, k.tabs, k.dead, k.err);
    ll_gather_rows(&p.vproj_dn, seg_v + r0, rows, e_proj, rv, k.tabs, k.dead, k.err);
    ll_gather_rows(&p.vproj_dn, seg_b + h_lo, nh, e_proj, gates, k.tabs, k.dead, k.err);
    ll_gather_rows(&p.vproj_dn, seg_a + h_lo, nh, e_proj, gates + nh, k.tabs, k.dead, k.err);
    consumer_sync();
    grid_mark(k, 10);
    // L2-normalise q and k of the heads this CTA touches: one warp per vector
#pragma unroll 1
    for (int hh = warp; hh < 2 * nh; hh += NW) {
        float* vec = mix + (size_t)hh * dk;
        float ss = 0.f;
#pragma unroll 1
        for (int e = lane; e < dk; e += 32) ss = fmaf(vec[e], vec[e], ss);
        const float rn = rsqrtf(warp_sum(ss) + p.l2_eps);
#pragma unroll 1
        for (int e = lane; e < dk; e += 32) vec[e] = vec[e] * rn;
    }
    consumer_sync();
    Ring& ring = k.ring;
    const int rpc = max(1, ring.stage_bytes / (dk * 4));
    unsigned long long* dst = vec_slot(p.va_dn, k.rank);
    int wrow = warp;
#pragma unroll 1
    for (int c0 = 0; c0 < rows; c0 += rpc) {
        const int n = min(rpc, rows - c0);
        const int ia = ring.idx;
        ring.wait(ring.full0 + 8u * ring.idx, ring.phase, 2);
        ring.advance();
        const float* Ss = reinterpret_cast<const float*>(ring.stages + (size_t)ia * ring.stage_bytes);
#pragma unroll 1
        for (; wrow < c0 + n; wrow += NW) {
            const int row = r0 + wrow;
            const int hl = row / dv - h_lo;
            const float* Sin = Ss + (size_t)(wrow - c0) * dk;
            float* Srow = L.state + (size_t)row * dk;                // sequence 0
            // beta, alpha = sigmoid of their projections
            const float beta = fast_sigmoid(gates[hl]), alpha = fast_sigmoid(gates[nh + hl]);
            float s[4], d1 = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kk = lane + 32 * e;
                s[e] = kk < dk ? Sin[kk] * alpha : 0.f;
                d1 = fmaf(s[e], kk < dk ? kn[hl * dk + kk] : 0.f, d1);
            }
            d1 = warp_sum(d1);
            const float cf = beta * (rv[wrow] - d1);
            float d2 = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kk = lane + 32 * e;
                if (kk < dk) {
                    s[e] = fmaf(cf, kn[hl * dk + kk], s[e]);
                    d2 = fmaf(s[e], qn[hl * dk + kk], d2);
                    Srow[kk] = s[e];
                }
            }
            d2 = warp_sum(d2);
            // the warp that finishes the CTA's last row publishes the slot (see consume_rows)
            int last = 0;
            if (lane == 0) {
                obuf[wrow] = d2;
                __threadfence_block();
                last = atomicAdd(ocnt, 1) == rows - 1;
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                __threadfence_block();
#pragma unroll 1
                for (int q = lane; q < rows; q += 32) ll_store(dst + q, obuf[q], e_out);
                if (lane == 0) *ocnt = 0;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(ring.empty0 + 8u * ia);
    }
}

// ---- the step ----------------------------------------------------------------------------------------
// Both roles walk the same sequence of phases: per layer QKV rows (0), [the mixer's data: K/V pages of
// the CTA's attention item, or its rows of the delta-net state] + O rows (1), gate/up rows (2), down
// rows (3); at the end the rows of the LM head (4). One loop body serves all of them.
enum { PH_PROJ = 0, PH_OPROJ = 1, PH_GATEUP = 2, PH_DOWN = 3, PH_LM = 4 };

// Producer (one warp): issues the copies in exactly the order in which the consumers wait for
// them. It depends on nothing but free ring stages.
template <typename T, typename KVT>
__device__ __forceinline__ void grid_producer(const GridParams& p, GridCtx& k) {
    const int lane = k.lane, rank = k.rank;
    Ring& ring = k.ring;
    const int esz = (int)sizeof(T);
    const int n_it = p.n_layers * 4 + (p.with_lm_head ? 1 : 0);
    const GridPlan& it = *k.plan;
#pragma unroll 1
    for (int itn = 0; itn < n_it; ++itn) {
        const int li = min(itn >> 2, p.n_layers - 1);
        const int ph = itn < p.n_layers * 4 ? (itn & 3) : PH_LM;
        const StepLayer& L = k.layers[li];
        const bool attn = L.type == 0;
        // job 1: rows [r0, r1) of matrix `a` (and of `b`: the gate/up pair); job 0, in front of the O rows:
        // this CTA's rows of the delta-net state, or the K and V pages of its attention item
        const unsigned char* a = reinterpret_cast<const unsigned char*>(p.E);
        const unsigned char* b = nullptr;
        const GridVec* vout = &p.vx;
        int row_bytes = p.d * esz;
        if (ph == PH_PROJ) {
            vout = attn ? &p.vproj_attn : &p.vproj_dn;
            a = reinterpret_cast<const unsigned char*>(L.Wqkv);
        } else if (ph == PH_OPROJ) {
            vout = &p.vxb;
            a = reinterpret_cast<const unsigned char*>(L.Wo);
            row_bytes = L.o_in * esz;
        } else if (ph == PH_GATEUP) {
            vout = &p.vh;
            a = reinterpret_cast<const unsigned char*>(L.W1a);
            b = reinterpret_cast<const unsigned char*>(L.W1b);
        } else if (ph == PH_DOWN) {
            a = reinterpret_cast<const unsigned char*>(L.W2);
            row_bytes = p.F * esz;
        }
        int r0, r1;
        if (ph == PH_LM) {
            r0 = k.tabs[p.vocab_tab + rank];
            r1 = k.tabs[p.vocab_tab + rank + 1];
        } else {
            vec_rows(*vout, k.tabs, rank, r0, r1);
        }
#pragma unroll 1
        for (int jb = ph == PH_OPROJ ? 0 : 1; jb < 2; ++jb) {
            const unsigned char* pa = a + (size_t)r0 * row_bytes;
            const unsigned char* pb = b ? b + (size_t)r0 * row_bytes : nullptr;
            int rows = r1 - r0, rb = row_bytes;
            const int* pt = nullptr;
            if (jb == 0) {
                pb = nullptr;
                if (attn) {
                    // chunks of whole pages: a K stage, then a V stage, one bulk copy per page
                    rows = it.has ? it.pages_prev : 0;
                    rb = kKvBlock * p.hd * (int)sizeof(KVT);
                    pa = reinterpret_cast<const unsigned char*>(L.kpool) + (size_t)it.kvh * rb;
                    pb = reinterpret_cast<const unsigned char*>(L.vpool) + (size_t)it.kvh * rb;
                    pt = p.page_table + it.pg_begin;
                } else {
                    int q0, q1;
                    vec_rows(p.va_dn, k.tabs, rank, q0, q1);
                    rows = q1 - q0;
                    rb = p.dk * 4;
                    pa = reinterpret_cast<const unsigned char*>(L.state) + (size_t)q0 * rb;
                }
            }
            int rpc = max(1, ring.stage_bytes / rb);
            if (pt) rpc = min(rpc, 32);             // one lane per page copy
#pragma unroll 1
            for (int c0 = 0; c0 < rows; c0 += rpc) {
                const int n = min(rpc, rows - c0);
                const int n_sub = pt ? n : 1;       // copies per stage: one per page, or the whole chunk at once
                const uint32_t sub_bytes = pt ? (uint32_t)rb : (uint32_t)n * (uint32_t)rb;
#pragma unroll 1
                for (int which = 0; which < (pb ? 2 : 1); ++which) {
                    int ok = 0;
                    if (lane == 0) {
                        ok = ring.wait(ring.empty0 + 8u * ring.idx, ring.phase ^ 1u, 1) ? 1 : 0;
                        if (ok) mbar_expect_tx(ring.full0 + 8u * ring.idx, (uint32_t)n * (uint32_t)rb);
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (ok && lane < n_sub) {
                        const unsigned char* base = which ? pb : pa;
                        const size_t src_off = pt ? (size_t)pt[c0 + lane] * p.kv_heads * rb : (size_t)c0 * rb;
                        const size_t dst_off = pt ? (size_t)lane * rb : 0;
                        bulk_g2s(smem_u32(ring.stages + (size_t)ring.idx * ring.stage_bytes + dst_off), base + src_off, sub_bytes,
                                 ring.full0 + 8u * ring.idx);
                    }
                    ring.advance();
                }
            }
        }
        __syncwarp();
    }
}

template <typename T, typename T2, typename KVT>
__device__ __forceinline__ void grid_consumer(const StepCtl& c, const GridParams& p, GridCtx& k) {
    constexpr int EPV = Elem<T>::EPV;
    const int C = k.C, rank = k.rank, tok = k.tok;
    const int tid = k.tid, lane = k.lane, warp = k.warp;
    float* smem = k.smem;
    // Input of a projection (GEMV layout) and the threads' sums of squares, two buffers each, used in
    // turn: a warp that is done with its rows of one phase fills the next phase's input while slower
    // warps still read the previous one; the block barrier after a gather is the only one of a phase.
    float* xsb[2] = {smem + p.off_xs, smem + p.off_xs + p.xs_stride};
    float* redb[2] = {smem + p.off_red, smem + p.off_red + kRingConsumers};
    float* xa = smem + p.off_xa;        // residual stream after the FFN (linear)
    float* xb = smem + p.off_xb;        // residual stream after the mixer (linear)
    float* pacc = smem + p.off_pacc;    // [layer][local row]: per-layer-embedding contribution to this CTA's rows of x
    Ring& ring = k.ring;
    const int d = p.d;
    uint32_t e = k.base;                // epochs used so far
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    const long long tstart = k.tm ? clock64() : 0;
    k.tmark = tstart;

    int xr0, xr1;                       // this CTA's rows of the residual stream
    vec_rows(p.vx, k.tabs, rank, xr0, xr1);
    const int xrows = xr1 - xr0;
    const int pacc_stride = p.vx.rpc;

    // ---- per-layer embeddings (no counterpart in the reference): pacc[l][j] = P_l[row] . T_l[tok] -------------
    // One warp per (layer, row of this CTA); all layers at once, before the first exchange.
    if (p.ple > 0) {
        const int n = p.n_layers * xrows;
#pragma unroll 1
        for (int i = warp; i < n; i += kRingWarps) {
            const int l = i / xrows, j = i - l * xrows;
            const StepLayer& L = k.layers[l];
            const T2* Pm = reinterpret_cast<const T2*>(L.pleP) + (size_t)(xr0 + j) * p.ple;
            const T2* Tb = reinterpret_cast<const T2*>(L.pleT) + (size_t)tok * p.ple;
            float a = 0.f;
#pragma unroll 1
            for (int q = lane; q < p.ple; q += 32) a = fmaf(Elem<T2>::get(Pm, q), Elem<T2>::get(Tb, q), a);
            a = warp_sum(a);
            if (lane == 0) pacc[l * pacc_stride + j] = a;
        }
        consumer_sync();
    }
    // ---- token embedding row, inference.cu:9-22: this CTA's rows, published like any other phase ----------------
    ++e;
    if (tid < xrows) {
        const T* E = reinterpret_cast<const T*>(p.E);
        float v = Elem<T>::get(E, (size_t)tok * d + xr0 + tid) * (p.Es ? p.Es[tok] : 1.0f);
        if (p.ple > 0) v += pacc[tid];
        ll_store(vec_slot(p.vx, rank) + tid, v, e);
    }
    grid_mark(k, 1);

    const int n_it = p.n_layers * 4 + (p.with_lm_head ? 1 : 0);
    int xi = 0, ri = 0;
    uint32_t e_in = e;                  // epoch of the next phase's input
    uint32_t e_proj = e;
    RowsJob job;
    job.eps = p.eps;
    job.logits = p.logits;
    job.ocnt = reinterpret_cast<int*>(smem + p.off_red + 2 * kRingConsumers + 1);
    job.obuf = smem + p.off_obuf;
#pragma unroll 1
    for (int itn = 0; itn < n_it; ++itn) {
        const int li = min(itn >> 2, p.n_layers - 1);
        const int ph = itn < p.n_layers * 4 ? (itn & 3) : PH_LM;
        const StepLayer& L = k.layers[li];
        const bool attn = L.type == 0;
        float* xs = xsb[xi];
        xi ^= 1;
        // ---- what this phase fetches, multiplies and publishes ------------------------------------------------------
        const GridVec* vin = &p.vx;
        const GridVec* vout = nullptr;
        const float* gain = nullptr;
        float* lin = nullptr;
        int K = d, tslot = 2;
        bool pair = false, do_gather = true;
        job.scale2 = nullptr;
        job.resid = nullptr;
        job.pacc = nullptr;
        if (ph == PH_PROJ) {
            gain = L.g1; lin = xa;
            vout = attn ? &p.vproj_attn : &p.vproj_dn;
            job.mode = RJ_STORE; job.scale = L.Sqkv;
        } else if (ph == PH_OPROJ) {
            K = L.o_in; tslot = 8;
            vout = &p.vxb;
            job.mode = RJ_RESID; job.scale = L.So; job.resid = xa;
            // ---- the mixer runs first (no weights): attention items + split combine, or the delta-net update ----
            if (attn) {
                const GridPlan& plan = *k.plan;
                const uint32_t e_parts = ++e;
                if (plan.has) {
                    if (p.hd == 64) grid_attention<KVT, 64>(p, L, k, e_proj, e_parts);
                    else grid_attention<KVT, 128>(p, L, k, e_proj, e_parts);
                    grid_mark(k, 5);
                }
                // few splits: every CTA combines all heads into its own input buffer; many: the owner of a
                // head combines it and publishes the result (a second exchange, but nobody fetches heads * S partials)
                if (plan.direct || rank < p.heads) {
                    grid_combine<EPV>(p, L, k, plan.direct ? 0 : rank, plan.direct ? p.heads : 1, e_proj, e_parts, plan.direct ? xs : nullptr,
                                      K / EPV, vec_slot(p.va_head, rank), e_parts + 1);
                    if (!plan.direct) grid_mark(k, 7);
                }
                if (plan.direct) {
                    do_gather = false;
                } else {
                    vin = &p.va_head;
                    e_in = ++e;
                }
            } else {
                e_in = ++e;
                grid_delta_net(p, L, k, e_proj, e_in, job.obuf, job.ocnt);
                grid_mark(k, 11);
                vin = &p.va_dn;
            }
        } else if (ph == PH_GATEUP) {
            tslot = 12;
            vin = &p.vxb; gain = L.g2; lin = xb;
            vout = &p.vh;
            pair = true;
            job.mode = RJ_SWIGLU; job.scale = L.S1a; job.scale2 = L.S1b;
        } else if (ph == PH_DOWN) {
            K = p.F; tslot = 14;
            vin = &p.vh;
            vout = &p.vx;
            job.mode = RJ_RESID; job.scale = L.S2; job.resid = xb;
            if (p.ple > 0 && li + 1 < p.n_layers) job.pacc = pacc + (li + 1) * pacc_stride;
        } else {
            tslot = 16;
            gain = p.g_final;
            job.mode = RJ_LM; job.scale = p.Es;
        }
        // ---- fetch the input; the RMS norm's sum of squares goes along ----------------------------------------------
        float* red = redb[ri];
        if (gain) ri ^= 1;
        float ss = 0.f;
        if (do_gather) ss = ll_gather_vec<EPV>(vin, e_in, gain, lin, xs, K / EPV, k.tabs, k.dead, k.err);
        if (gain) red[tid] = ss;
        consumer_sync();
        grid_mark(k, tslot);
        // ---- this CTA's rows ------------------------------------------------------------------------------------------
        int r0, r1;
        if (vout) {
            vec_rows(*vout, k.tabs, rank, r0, r1);
            job.dst = vec_slot(*vout, rank);
            job.epoch = ++e;
        } else {
            r0 = k.tabs[p.vocab_tab + rank];
            r1 = k.tabs[p.vocab_tab + rank + 1];
            job.dst = nullptr;
            job.epoch = 0;
        }
        job.rows = r1 - r0; job.K = K; job.r0 = r0; job.xs = xs;
        job.norm_n = gain ? d : 0; job.red = red;
        consume_rows<T>(ring, job, pair, warp, lane, bv, bi, k.tm);
        e_in = e;
        if (ph == PH_PROJ) e_proj = e;
        grid_mark(k, tslot + 1);
    }

    if (p.with_lm_head) {
        // reduce the warps' argmax picks (lane 0 of each warp holds them), then (in CTA 0) the grid's
        float* tmp = smem + p.off_mix;
        if (lane == 0) { tmp[2 * warp] = bv; tmp[2 * warp + 1] = __int_as_float(bi); }
        consumer_sync();
        ++e;
        if (tid == 0) {
            for (int w = 1; w < kRingWarps; ++w) {
                const float v = tmp[2 * w];
                const int ix = __float_as_int(tmp[2 * w + 1]);
                if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
            }
            tmp[0] = bv;
            tmp[1] = __int_as_float(bi);
        }
        __syncwarp();
        if (tid < 2) ll_store(vec_slot(p.vlm, rank) + tid, tmp[tid], e);      // one store instruction for the pair
    }
    if (k.tm != nullptr && tid == 0) {
        k.tm[0] += clock64() - tstart;
        if (p.timers)
            for (int i = 0; i < kGridTimerSlots; ++i) p.timers[(size_t)rank * kGridTimerSlots + i] += k.tm[i];
    }
    if (rank == 0) {
        if (p.with_lm_head) {
            float* lm = smem + p.off_parts;          // free by now
            ll_gather_rows(&p.vlm, 0, 2 * C, e, lm, k.tabs, k.dead, k.err);
            consumer_sync();
            if (warp == 0 && p.do_pick) {
                // lowest index among the largest values (the host loop of inference_orchestrator.cu:77-84 keeps the first)
                float best = -INFINITY;
                int at = 0x7fffffff;
                for (int r = lane; r < C; r += 32) {
                    const float v = lm[2 * r];
                    const int ix = __float_as_int(lm[2 * r + 1]);
                    if (v > best || (v == best && ix < at)) { best = v; at = ix; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float vo = __shfl_xor_sync(0xffffffffu, best, o);
                    const int io = __shfl_xor_sync(0xffffffffu, at, o);
                    if (vo > best || (vo == best && io < at)) { best = vo; at = io; }
                }
                if (lane == 0) advance_seq(c, 0, at);
            }
        } else if (tid == 0) {
            advance_seq(c, 0, -1);
        }
        // Every CTA read the epoch word when it started, and this CTA got here only through data
        // that all of them produced: the word is free to move on.
        if (tid == 0) *p.epoch = e;
    }
}

template <typename T, typename T2, typename KVT>
__global__ void __launch_bounds__(kRingThreads, 1) grid_decode_kernel(const __grid_constant__ StepCtl c, const __grid_constant__ GridParams p) {
    if (!seq_active(c, 0)) return;                    // uniform over the grid
    extern __shared__ __align__(128) float grid_smem[];
    float* smem = grid_smem;
    GridCtx k;
    k.C = (int)gridDim.x;
    k.rank = (int)blockIdx.x;
    k.tid = threadIdx.x;
    k.lane = threadIdx.x & 31;
    k.warp = threadIdx.x >> 5;
    k.smem = smem;
    k.tabs = reinterpret_cast<const int*>(smem);
    k.tok = p.tok_arg >= 0 ? p.tok_arg : c.tok[0];
    k.pos = c.pos[0];
    k.base = *p.epoch;
    int* dead = reinterpret_cast<int*>(smem + p.off_red + 2 * kRingConsumers);
    k.dead = dead;
    k.err = p.err;
    k.tm = p.timers ? reinterpret_cast<long long*>(smem + p.off_timers) : nullptr;
    k.tmark = 0;
    k.plan = reinterpret_cast<const GridPlan*>(smem + p.off_plan);
    k.ring.backoff_ns = (unsigned)p.backoff_ns;
    k.ring.full0 = smem_u32(smem + p.off_bar);
    k.ring.empty0 = k.ring.full0 + 8u * p.n_stages;
    k.ring.stages = reinterpret_cast<unsigned char*>(smem + p.off_ring);
    k.ring.nst = p.n_stages;
    k.ring.stage_bytes = p.stage_bytes;
    k.ring.idx = 0;
    k.ring.phase = 0;
    k.ring.dead = dead;
    k.ring.err = p.err;
    {
        // the per-layer table moves to shared memory: every phase reads a few of its fields
        const int n8 = p.n_layers * (int)(sizeof(StepLayer) / 8);
        const unsigned long long* src = reinterpret_cast<const unsigned long long*>(p.layers);
        unsigned long long* dstl = reinterpret_cast<unsigned long long*>(smem + p.off_layers);
#pragma unroll 1
        for (int i = threadIdx.x; i < n8; i += kRingThreads) dstl[i] = src[i];
        k.layers = reinterpret_cast<const StepLayer*>(dstl);
    }
    {
        // row tables r0[c] = floor(c N / P) of the exchanged vectors and of the LM head
        int* tabs = reinterpret_cast<int*>(smem);
        const GridVec* vs = &p.vx;                    // the vectors follow one another in GridParams
#pragma unroll 1
        for (int t = 0; t < kGridVecs; ++t) {
            const int N = vs[t].N, P = vs[t].P, tab = vs[t].tab;
#pragma unroll 1
            for (int i = threadIdx.x; i <= P; i += kRingThreads) tabs[tab + i] = (int)(((unsigned)i * (unsigned)N) / (unsigned)P);
        }
#pragma unroll 1
        for (int i = threadIdx.x; i <= k.C; i += kRingThreads) tabs[p.vocab_tab + i] = (int)(((unsigned)i * (unsigned)p.V) / (unsigned)k.C);
    }
    if (threadIdx.x == 0) {
        *dead = 0;
        dead[1] = 0;                     // the finished-row counter
        if (k.tm)
            for (int i = 0; i < kGridTimerSlots; ++i) k.tm[i] = 0;
        for (int i = 0; i < p.n_stages; ++i) {
            mbar_init(k.ring.full0 + 8u * i, 1);                    // the producer's expect_tx arrival
            mbar_init(k.ring.empty0 + 8u * i, kRingWarps);          // one arrival per consumer warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        grid_make_plan(p, k.pos, k.C, k.rank, reinterpret_cast<GridPlan*>(smem + p.off_plan));
    }
    __syncthreads();
    if (k.warp == kRingWarps) grid_producer<T, KVT>(p, k);
    else grid_consumer<T, T2, KVT>(c, p, k);
}

}  // namespace mlb
