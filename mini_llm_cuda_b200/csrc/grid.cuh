// Batch-1 decode step as ONE persistent kernel over the whole GPU.
//
// The kernel chain pays one launch boundary per projection (~40 per token) and every boundary
// drains the memory pipeline. Here one CTA per SM lives for the whole step:
//   * every phase splits its output rows evenly over the CTAs; a CTA's rows are one contiguous
//     slab of the row-major weight matrix, streamed by a producer warp with cp.async.bulk into a
//     ring of shared-memory stages (the code of the cluster step in mega.cuh). The producer
//     depends on nothing but free stages, so it runs phases ahead of the consumers and HBM stays
//     busy across phase boundaries;
//   * activations cross CTAs through global memory (L2) as 8-byte {value, epoch} words. A
//     reader polls the words themselves until they carry the epoch of the phase it waits for, so
//     a phase boundary costs ONE L2 round trip: there is no grid barrier and no separate flag.
//     An exchange buffer is rewritten two or more phases after its last reader has left it: a CTA
//     can write phase k+2 only after it saw every CTA's phase k+1 output, which each of them wrote
//     after it had finished reading phase k;
//   * the attention phase works on (kv head, context split) items; the item that holds the
//     current position applies QK-norm and RoPE to the raw projections itself, appends the K/V
//     row to the paged pool and uses it from shared memory, so no CTA waits for another one's
//     pool write.
// The arithmetic of every phase is the one of the chain kernels in kernels.cuh (same reference
// citations); only the partition of rows and of the attention context differs.
//
// The CTAs wait on one another, so the kernel is launched cooperatively (all CTAs co-resident
// or the launch fails). Every wait is bounded: when one runs out the kernel records an error
// code, stops waiting (later waits return at once) and still walks to the end, so it always
// terminates and the host reports MLB_E_TIMEOUT.
#pragma once
#include <type_traits>

#include "grid_params.h"
#include "mega.cuh"

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

struct GridCtx {
    int C, rank, tok, pos, tid, lane, warp;
    uint32_t base;                 // epoch before this step
    float* smem;
    volatile int* dead;
    int* err;
    const MegaLayer* layers;       // the per-layer table in shared memory
    const GridPhase* phases;       // the phase list in shared memory
    long long* tm;                 // diagnostic counters in shared memory (thread 0 writes)
    long long tmark;
    Ring ring;
};

#ifdef MLB_GRID_TIMERS
#define MLB_GT(i) if (k.tid == 0) { const long long n_ = clock64(); k.tm[i] += n_ - k.tmark; k.tmark = n_; }
#define MLB_GCOUNT(i) if (k.tid == 0) ++k.tm[i];
#else
#define MLB_GT(i)
#define MLB_GCOUNT(i)
#endif

// Consumer threads fetch words 0..n-1 of `src` that carry epoch `e` into shared memory: linearly,
// or (perm_nvec > 0) in the GEMV input layout of perm_nvec weight vectors of EPV elements.
// Returns the sum of squares of the values this thread fetched (for the RMS norm that follows).
template <int EPV>
__device__ __forceinline__ float ll_gather(const unsigned long long* src, int n, uint32_t e, float* dst, int perm_nvec, GridCtx& k) {
    constexpr int U = 4;               // words in flight per thread
    float ss = 0.f;
#pragma unroll 1
    for (int i0 = k.tid; i0 < n; i0 += kMegaConsumers * U) {
        unsigned long long w[U];
        uint32_t spins = 0;
        bool ok;
        do {
            ok = true;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + u * kMegaConsumers;
                w[u] = 0ull;
                if (i < n) {
                    w[u] = ll_load(src + i);
                    ok = ok && (uint32_t)(w[u] >> 32) == e;
                }
            }
            if (!ok) {
                MLB_GCOUNT(15)
                if (*k.dead) break;
                if (++spins > kGridSpinLimit) {
                    *k.dead = 1;
                    atomicExch(k.err, 3);
                    break;
                }
            }
        } while (!ok);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * kMegaConsumers;
            if (i < n) {
                const float v = __uint_as_float((uint32_t)w[u]);
                dst[perm_nvec > 0 ? xs_index<EPV>(i, perm_nvec) : i] = v;
                ss = fmaf(v, v, ss);
            }
        }
    }
    return ss;
}

template <typename KVT> __device__ __forceinline__ float round_kv(float v);
template <> __device__ __forceinline__ float round_kv<float>(float v) { return v; }
template <> __device__ __forceinline__ float round_kv<bf16_t>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Balanced row partition: every CTA gets floor(N/C) or ceil(N/C) rows, so with N >= C every CTA
// produces rows in every projection phase. The reuse rule of the exchange buffers rests on that:
// a CTA that only read would be waited for by nobody.
__device__ __forceinline__ void grid_rows(int N, int C, int rank, int& r0, int& r1) {
    r0 = (int)(((unsigned)rank * (unsigned)N) / (unsigned)C);          // rank * N stays far below 2^32
    r1 = (int)(((unsigned)(rank + 1) * (unsigned)N) / (unsigned)C);
}

// dst = (src / sqrt(mean(src^2)+eps)) * gain in the bank-conflict-free layout of a GEMV input
// (inference.cu:24-50, :83-95). `ss` is this thread's share of the sum of squares; the barrier
// inside also publishes `src`, which the caller has just written.
template <int EPV>
__device__ __forceinline__ void grid_norm(float ss, const float* src, float* dst, const float* __restrict__ gain, int n, float eps,
                                          float* red, int tid, int warp, int lane) {
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    consumer_sync();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kMegaWarps; ++w) tot += red[w];
    const float r = sqrtf(tot / (float)n + eps);
    const int nvec = n / EPV;
#pragma unroll 1
    for (int k = tid; k < n; k += kMegaConsumers) dst[xs_index<EPV>(k, nvec)] = (src[k] / r) * gain[k];
    consumer_sync();
}

// ---- rows of a projection out of the ring ----------------------------------------------------------
// One job = this CTA's rows of one weight matrix (or of the gate/up pair). Local row r belongs to
// warp r % 15 whatever chunk of the ring it arrives in, so consecutive chunks keep different warps
// busy; lane 0 of the warp finishes the row (scale, residual, activation) and publishes it.
struct RowsJob {
    int mode, rows, K, r0;
    const float* xs;               // input vector, GEMV layout
    const float* scale;            // per-row weight scale (FP8) or null, by global row
    const float* scale2;           // the up matrix's scale (RJ_SWIGLU)
    unsigned long long* dst;       // exchange buffer, by global row
    uint32_t epoch;
    const float* resid;            // RJ_RESID: residual stream in shared memory, by global row
    const float* pacc;             // RJ_RESID: addend per local row, or null
    float* out_s;                  // RJ_PACC: shared-memory destination per local row
    float* logits;                 // RJ_LM
};

template <typename T>
__device__ __forceinline__ float smem_row_dot(const T* row, int nvec, const float* xs, int lane) {
    constexpr int EPV = Elem<T>::EPV;
    const float4* xp = reinterpret_cast<const float4*>(xs);
    float a0 = 0.f, a1 = 0.f;
#pragma unroll 2
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

// Lane 0 of the row's warp: finish local row r (sv, su: the row's weight scales). (bv, bi): running
// argmax of RJ_LM.
__device__ __forceinline__ void row_done(const RowsJob& j, int r, float v, float u, float sv, float su, float& bv, int& bi) {
    const int row = j.r0 + r;
    v *= sv;
    if (j.mode == RJ_SWIGLU) {
        u *= su;
        // applySiluToFFN + hadamardMultiplyFFN, inference.cu:262-281
        ll_store(j.dst + row, (v / (1.0f + expf(-v))) * u, j.epoch);
        return;
    }
    if (j.mode == RJ_STORE) {
        ll_store(j.dst + row, v, j.epoch);
    } else if (j.mode == RJ_RESID) {
        if (j.pacc) v += j.pacc[r];
        ll_store(j.dst + row, v + j.resid[row], j.epoch);
    } else if (j.mode == RJ_PACC) {
        j.out_s[r] = v;
    } else {
        j.logits[row] = v;
        if (v > bv || (v == bv && row < bi)) { bv = v; bi = row; }
    }
}

template <typename T>
__device__ __forceinline__ void consume_rows(Ring& r, const RowsJob& j, bool pair, int warp, int lane, float& bv, int& bi) {
    constexpr int EPV = Elem<T>::EPV;
    constexpr int NW = kMegaWarps;
    const int K = j.K, rows = j.rows, nvec = K / EPV;
    const int rpc = max(1, r.stage_bytes / (K * (int)sizeof(T)));
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
            // the row's scales come from global memory: asked for before the dot products, used after
            const float sv = j.scale ? j.scale[j.r0 + wrow] : 1.0f;
            const float su = (pair && j.scale2) ? j.scale2[j.r0 + wrow] : 1.0f;
            const float a = smem_row_dot<T>(A + off, nvec, j.xs, lane);
            const float b = pair ? smem_row_dot<T>(Bm + off, nvec, j.xs, lane) : 0.f;
            if (lane == 0) row_done(j, wrow, a, b, sv, su, bv, bi);
        }
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(r.empty0 + 8u * ia);
            if (pair) mbar_arrive(r.empty0 + 8u * ib);
        }
    }
}

// Flash-decode items of one attention layer: (kv head, context split) over the CTAs. The warps of
// an item share its heads and pages: 8/G warps per query head, pages interleaved among them.
template <typename KVT, int HD>
__device__ __forceinline__ void grid_attention(const GridParams& p, const MegaLayer& L, GridCtx& k, uint32_t e_proj, uint32_t e_out, int S,
                                            int pps) {
    constexpr int EPL = 16 / (int)sizeof(KVT);        // elements per lane per row
    constexpr int LPR = HD / EPL;                     // lanes per row
    constexpr int PPI = 32 / LPR;                     // positions per warp iteration
    constexpr int ITERS = kKvBlock / PPI;
    constexpr int CH = ITERS < 4 ? ITERS : 4;         // iterations loaded together (2*CH 16-byte loads per lane in flight)
    static_assert(LPR <= 32 && PPI >= 1 && ITERS % CH == 0, "head_dim does not fit one warp row");
    const int C = k.C, rank = k.rank, pos = k.pos, tid = k.tid, lane = k.lane, warp = k.warp;
    const int G = p.heads / p.kv_heads;
    const int WPH = max(1, kGridAttnWarps / G);       // warps per query head
    const int npages = pos / kKvBlock + 1;
    const int cur_page = pos / kKvBlock;
    const int n_items = p.kv_heads * S;
    const int seg_q = L.nq, seg_k = L.nq + L.nk;
    const int lr = lane % LPR, grp = lane / LPR;
    const float div = sqrtf((float)HD);
    float* tq = k.smem + p.off_tmp;                   // [G][HD] queries of the item's heads
    float* tk = tq + G * HD;                          // [HD] this step's key row
    float* tv = tk + HD;                              // [HD] this step's value row
    float* wpart = tv + HD;                           // [kGridAttnWarps][HD+2]
    KVT* kpool = reinterpret_cast<KVT*>(L.kpool);
    KVT* vpool = reinterpret_cast<KVT*>(L.vpool);
    const int* pt = p.page_table;                     // sequence 0
    const int g = warp / WPH, sub = warp - g * WPH;
    const bool scanner = warp < kGridAttnWarps && g < G;

    for (int it = rank; it < n_items; it += C) {
        const int kvh = it / S, split = it - kvh * S;
        const int pg_begin = split * pps, pg_end = min(npages, pg_begin + pps);
        const bool cur_here = cur_page >= pg_begin && cur_page < pg_end;
        const int h0 = kvh * G;
        // (a) before anything arrives: the first positions of this warp's first page. Rows of earlier
        //     positions never change during the step, so they may come through L1 (read-only path).
        uint4 kr[CH], vr[CH];
        const int first_pg = pg_begin + sub;
        const bool has_first = scanner && first_pg < pg_end;
        int first_pgi = 0;
#pragma unroll
        for (int i = 0; i < CH; ++i) { kr[i] = make_uint4(0, 0, 0, 0); vr[i] = make_uint4(0, 0, 0, 0); }
        if (has_first) {
            first_pgi = pt[first_pg];
            const int cnt = min(kKvBlock, pos - first_pg * kKvBlock);
            const size_t base = ((size_t)first_pgi * p.kv_heads + kvh) * kKvBlock * HD;
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                const int j = i * PPI + grp;
                if (j < cnt) {
                    kr[i] = __ldg(reinterpret_cast<const uint4*>(kpool + base + (size_t)j * HD + lr * EPL));
                    vr[i] = __ldg(reinterpret_cast<const uint4*>(vpool + base + (size_t)j * HD + lr * EPL));
                }
            }
        }
        // (b) raw projections of the item's query heads (+ this step's key and value row)
        ll_gather<4>(p.ll_proj + (size_t)h0 * HD, G * HD, e_proj, tq, 0, k);
        if (cur_here) {
            ll_gather<4>(p.ll_proj + seg_q + (size_t)kvh * HD, HD, e_proj, tk, 0, k);
            ll_gather<4>(p.ll_proj + seg_k + (size_t)kvh * HD, HD, e_proj, tv, 0, k);
        }
        consumer_sync();
        // (c) per-head RMS norm (inference.cu:52-81, :97-111) and RoPE on adjacent pairs
        //     (inference.cu:113-134): one warp per vector; the new K/V row goes to the pool.
        {
            const int nvecs = G + (cur_here ? 1 : 0);
            const size_t row_off = (((size_t)pt[cur_page] * p.kv_heads + kvh) * kKvBlock + (pos % kKvBlock)) * HD;
            if (warp < nvecs) {
                const bool is_k = warp >= G;
                float* vec = is_k ? tk : tq + warp * HD;
                const float* gain = is_k ? L.gk + (size_t)kvh * HD : L.gq + (size_t)(h0 + warp) * HD;
                float rs = 1.f;
                if (p.qk_norm) {
                    float ss = 0.f;
#pragma unroll 1
                    for (int r = lane; r < HD; r += 32) ss = fmaf(vec[r], vec[r], ss);
                    rs = sqrtf(warp_sum(ss) / (float)HD + p.eps);
                }
#pragma unroll 1
                for (int pr = lane; pr < HD / 2; pr += 32) {
                    const int r = 2 * pr;
                    float a = vec[r], cc = vec[r + 1];
                    if (p.qk_norm) {
                        a = (a / rs) * gain[r];
                        cc = (cc / rs) * gain[r + 1];
                    }
                    const float cs = p.rope[(size_t)pos * HD + r], sn = p.rope[(size_t)pos * HD + r + 1];
                    float ra = cs * a - sn * cc, rc = sn * a + cs * cc;
                    if (is_k) {
                        Elem<KVT>::put(kpool, row_off + r, ra);
                        Elem<KVT>::put(kpool, row_off + r + 1, rc);
                        ra = round_kv<KVT>(ra);
                        rc = round_kv<KVT>(rc);
                    }
                    vec[r] = ra;
                    vec[r + 1] = rc;
                }
            } else if (cur_here && warp == nvecs) {
#pragma unroll 1
                for (int r = lane; r < HD; r += 32) {
                    const float v = tv[r];
                    Elem<KVT>::put(vpool, row_off + r, v);
                    tv[r] = round_kv<KVT>(v);
                }
            }
        }
        consumer_sync();
        // (d) online softmax of this warp's head over this warp's pages
        if (scanner) {
            float q[EPL], acc[EPL], m = kNegBig, l = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) { q[e] = tq[g * HD + lr * EPL + e]; acc[e] = 0.f; }
            for (int pg = first_pg; pg < pg_end; pg += WPH) {
                const bool first = pg == first_pg;
                const int cnt = min(kKvBlock, pos - pg * kKvBlock);      // earlier positions only
                if (cnt <= 0) break;
                const int pgi = first ? first_pgi : pt[pg];
                const size_t base = ((size_t)pgi * p.kv_heads + kvh) * kKvBlock * HD;
#pragma unroll
                for (int c0 = 0; c0 < ITERS; c0 += CH) {
                    uint4 kk[CH], vv4[CH];
#pragma unroll
                    for (int i = 0; i < CH; ++i) {
                        const int j = (c0 + i) * PPI + grp;
                        kk[i] = make_uint4(0, 0, 0, 0);
                        vv4[i] = make_uint4(0, 0, 0, 0);
                        if (c0 == 0 && first) {
                            kk[i] = kr[i];
                            vv4[i] = vr[i];
                        } else if (j < cnt) {
                            kk[i] = __ldg(reinterpret_cast<const uint4*>(kpool + base + (size_t)j * HD + lr * EPL));
                            vv4[i] = __ldg(reinterpret_cast<const uint4*>(vpool + base + (size_t)j * HD + lr * EPL));
                        }
                    }
                    // scores of the chunk's positions first (independent), then one rescale of the
                    // running sums and one exponential per position
                    float sv[CH];
#pragma unroll
                    for (int i = 0; i < CH; ++i) {
                        float kv[EPL];
                        Elem<KVT>::unpack(kk[i], kv);
                        float s = 0.f;
#pragma unroll
                        for (int e = 0; e < EPL; ++e) s = fmaf(q[e], kv[e], s);
#pragma unroll
                        for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                        s = s / div;                      // inference.cu:154
                        sv[i] = (c0 + i) * PPI + grp < cnt ? s : kNegBig;
                    }
                    float mn = m;
#pragma unroll
                    for (int i = 0; i < CH; ++i) mn = fmaxf(mn, sv[i]);
                    const float sc = expf(m - mn);
                    l *= sc;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) acc[e] *= sc;
#pragma unroll
                    for (int i = 0; i < CH; ++i) {
                        const float pe = (c0 + i) * PPI + grp < cnt ? expf(sv[i] - mn) : 0.f;
                        float vv[EPL];
                        Elem<KVT>::unpack(vv4[i], vv);
                        l += pe;
#pragma unroll
                        for (int e = 0; e < EPL; ++e) acc[e] = fmaf(pe, vv[e], acc[e]);
                    }
                    m = mn;
                }
            }
            if (cur_here && sub == 0) {
                // the current position, from shared memory
                float s = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) s = fmaf(q[e], tk[lr * EPL + e], s);
#pragma unroll
                for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                s = s / div;
                if (grp == 0) {
                    const float mn = fmaxf(m, s);
                    const float sc = expf(m - mn), pe = expf(s - mn);
                    l = l * sc + pe;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) acc[e] = acc[e] * sc + pe * tv[lr * EPL + e];
                    m = mn;
                }
            }
            // merge the position groups of the warp
#pragma unroll
            for (int o = LPR; o < 32; o <<= 1) {
                const float mo = __shfl_xor_sync(0xffffffffu, m, o);
                const float lo = __shfl_xor_sync(0xffffffffu, l, o);
                const float mn = fmaxf(m, mo);
                const float sa = expf(m - mn), sb = expf(mo - mn);
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
#pragma unroll 1
        for (int idx = tid; idx < G * (HD + 2); idx += kMegaConsumers) {
            const int gg = idx / (HD + 2), e = idx - gg * (HD + 2);
            const float* w0 = wpart + (size_t)gg * WPH * (HD + 2);
            float mn = kNegBig;
#pragma unroll 1
            for (int w = 0; w < WPH; ++w) mn = fmaxf(mn, w0[(size_t)w * (HD + 2) + HD]);
            float val;
            if (e == HD) {
                val = mn;
            } else {
                val = 0.f;
#pragma unroll 1
                for (int w = 0; w < WPH; ++w) val += w0[(size_t)w * (HD + 2) + e] * expf(w0[(size_t)w * (HD + 2) + HD] - mn);
            }
            ll_store(p.ll_parts + ((size_t)(h0 + gg) * S + split) * (HD + 2) + e, val, e_out);
        }
        consumer_sync();
    }
}

// Combine the context splits (+ query gating, inference.cu:241-250). Few splits: every CTA fetches
// all partials and builds the whole attention output in its own shared memory (`direct`, one
// exchange). Many splits: the owner of a head combines it and publishes the result (two exchanges,
// but nobody fetches heads * S partial vectors).
template <int EPV>
__device__ __forceinline__ void grid_combine(const GridParams& p, const MegaLayer& L, GridCtx& k, uint32_t e_proj, uint32_t e_parts,
                                             uint32_t e_out, int S, bool direct) {
    const int hd = p.hd, tid = k.tid;
    float* parts = k.smem + p.off_parts;
    float* gate = k.smem + p.off_proj;
    float* abuf = k.smem + p.off_a;
    float* scales = k.smem + p.off_tmp;       // [heads in this pass][S]
    const int seg_v = L.nq + L.nk + L.nv;
    const int n_a = p.heads * hd;
    const int h_first = direct ? 0 : k.rank, h_step = direct ? p.heads : k.C, h_count = direct ? p.heads : 1;
#pragma unroll 1
    for (int h0 = h_first; h0 < p.heads; h0 += h_step) {
        ll_gather<4>(p.ll_parts + (size_t)h0 * S * (hd + 2), h_count * S * (hd + 2), e_parts, parts, 0, k);
        if (L.ng) ll_gather<4>(p.ll_proj + seg_v + (size_t)h0 * hd, h_count * hd, e_proj, gate, 0, k);
        consumer_sync();
        // per (head, split): the factor that brings the split's sums to the head's common maximum
#pragma unroll 1
        for (int i = tid; i < h_count * S; i += kMegaConsumers) {
            const int hl = i / S;
            const float* pp = parts + (size_t)hl * S * (hd + 2);
            float mn = kNegBig;
#pragma unroll 1
            for (int s = 0; s < S; ++s) mn = fmaxf(mn, pp[(size_t)s * (hd + 2) + hd]);
            scales[i] = expf(parts[(size_t)i * (hd + 2) + hd] - mn);
        }
        consumer_sync();
#pragma unroll 1
        for (int i = tid; i < h_count * hd; i += kMegaConsumers) {
            const int hl = i / hd, e = i - hl * hd;
            const float* pp = parts + (size_t)hl * S * (hd + 2);
            const float* scl = scales + (size_t)hl * S;
            float lt = 0.f, at = 0.f;
#pragma unroll 4
            for (int s = 0; s < S; ++s) {
                const float sc = scl[s];
                lt = fmaf(pp[(size_t)s * (hd + 2) + hd + 1], sc, lt);
                at = fmaf(pp[(size_t)s * (hd + 2) + e], sc, at);
            }
            float o = at / lt;
            if (L.ng) o *= 1.0f / (1.0f + expf(-gate[i]));      // sigmoid of the gate projection (inference.cu:248)
            if (direct) abuf[xs_index<EPV>(i, n_a / EPV)] = o;
            else ll_store(p.ll_a + (size_t)h0 * hd + i, o, e_out);
        }
        consumer_sync();
    }
}

// Gated delta-net step on this CTA's rows of the state (the arithmetic of delta_net_kernel).
__device__ __forceinline__ void grid_delta_net(const GridParams& p, const MegaLayer& L, GridCtx& k, uint32_t e_out) {
    constexpr int NW = kMegaWarps;
    const int H = p.heads, dk = p.dk, dv = p.dv, tid = k.tid, lane = k.lane, warp = k.warp;
    float* proj = k.smem + p.off_proj;
    float* tmp = k.smem + p.off_tmp;
    float* qn = tmp;
    float* kn = tmp + H * dk;
    float* gates = tmp + 2 * H * dk;
#pragma unroll 1
    for (int hh = warp; hh < 2 * H; hh += NW) {
        const float* src = proj + (size_t)hh * dk;          // q heads then k heads
        float ss = 0.f;
#pragma unroll 1
        for (int e = lane; e < dk; e += 32) ss = fmaf(src[e], src[e], ss);
        ss = warp_sum(ss);
        const float n = sqrtf(ss + p.l2_eps);
#pragma unroll 1
        for (int e = lane; e < dk; e += 32) tmp[(size_t)hh * dk + e] = src[e] / n;
    }
#pragma unroll 1
    for (int i = tid; i < 2 * H; i += kMegaConsumers)
        gates[i] = 1.0f / (1.0f + expf(-proj[2 * H * dk + H * dv + i]));      // beta[H] then alpha[H]
    consumer_sync();
    const int rows = H * dv;
    int r0, r1;
    grid_rows(rows, k.C, k.rank, r0, r1);
    float* state = L.state;                                 // sequence 0
    const float* rv = proj + 2 * H * dk;
#pragma unroll 1
    for (int row = r0 + warp; row < r1; row += NW) {
        const int h = row / dv;
        float* Srow = state + (size_t)row * dk;
        const float beta = gates[h], alpha = gates[H + h];
        float s[4], d1 = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int kk = lane + 32 * e;
            s[e] = kk < dk ? Srow[kk] * alpha : 0.f;
            d1 = fmaf(s[e], kk < dk ? kn[h * dk + kk] : 0.f, d1);
        }
        d1 = warp_sum(d1);
        const float cf = beta * (rv[row] - d1);
        float d2 = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int kk = lane + 32 * e;
            if (kk < dk) {
                s[e] = fmaf(cf, kn[h * dk + kk], s[e]);
                d2 = fmaf(s[e], qn[h * dk + kk], d2);
                Srow[kk] = s[e];
            }
        }
        d2 = warp_sum(d2);
        if (lane == 0) ll_store(p.ll_a + row, d2, e_out);
    }
}

// ---- the step as a list of phases ---------------------------------------------------------------
// Both roles walk the same list (GridPhase): embedding rows (with per-layer embeddings), then per
// layer QKV rows, O rows, gate/up rows, the next layer's per-layer-embedding rows, down rows, and at
// the end the LM head; the mixer (attention items + combine, or the delta-net update) runs after the
// QKV rows. The list is interpreted by ONE loop whose body holds one copy of the gather, the norm
// and the row consumer: unrolled per phase, the kernel outgrew the instruction cache. The host
// fills the list, so that a phase starts with a few loads instead of a chain of decisions: the
// step is bound by the latency of its serial instructions, not by their throughput.

// Producer (one warp): issues the weight slabs in exactly the order in which the consumers wait
// for them. It depends on nothing but free ring stages.
__device__ __forceinline__ void grid_producer(const GridParams& p, GridCtx& k) {
    const int lane = k.lane;
    const int n_ph = p.with_lm_head ? p.n_phases : p.n_phases - 1;
    Ring& ring = k.ring;
#pragma unroll 1
    for (int pi = 0; pi < n_ph; ++pi) {
        const GridPhase& d = k.phases[pi];
        const unsigned char* a = reinterpret_cast<const unsigned char*>(d.W) + (size_t)d.r0 * d.row_bytes;
        if (d.W2) issue_slab_pair(ring, a, reinterpret_cast<const unsigned char*>(d.W2) + (size_t)d.r0 * d.row_bytes, d.rows, d.row_bytes, lane);
        else issue_slab(ring, a, d.rows, d.row_bytes, lane);
    }
}

template <typename T, typename T2, typename KVT>
__device__ __forceinline__ void grid_consumer(const StepCtl& c, const GridParams& p, GridCtx& k) {
    constexpr int EPV = Elem<T>::EPV;
    constexpr int EPV2 = Elem<T2>::EPV;
    constexpr bool kSameT2 = std::is_same<T, T2>::value;
    const int C = k.C, rank = k.rank, tok = k.tok, pos = k.pos;
    const int tid = k.tid, lane = k.lane, warp = k.warp;
    float* smem = k.smem;
    float* xa = smem + p.off_x;         // residual stream after the FFN (linear)
    float* xb = smem + p.off_x2;        // residual stream after the mixer (linear)
    float* xn = smem + p.off_xn;        // normalised input of the current projection (GEMV layout)
    float* proj = smem + p.off_proj;    // the raw delta-net projections, or the query gates
    float* tmp = smem + p.off_tmp;
    float* plerow = smem + p.off_ple;   // per-layer-embedding table row of the pending token (GEMV layout)
    float* pacc = smem + p.off_pacc;    // per-layer-embedding contribution to this CTA's rows of x
    float* red = smem + p.off_red;
    Ring& ring = k.ring;
    const int dim = p.d, hd = p.hd;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#ifdef MLB_GRID_TIMERS
    k.tmark = clock64();
    const long long tstart = k.tmark;
#endif

    // ---- token embedding row, inference.cu:9-22 ----------------------------------------------------------
    {
        const T* E = reinterpret_cast<const T*>(p.E);
        const float sc = p.Es ? p.Es[tok] : 1.0f;
        float* x0 = p.ple > 0 ? xb : xa;            // with per-layer embeddings the sum goes through ll_xa
#pragma unroll 1
        for (int i = tid; i < dim; i += kMegaConsumers) x0[i] = Elem<T>::get(E, (size_t)tok * dim + i) * sc;
    }

    // One pass of the loop body = one phase with weights: optional gather, optional norm, rows.
    const int n_ph = p.with_lm_head ? p.n_phases : p.n_phases - 1;
    const uint32_t base = k.base;
    bool abuf_ready = false;            // the mixer left its output in shared memory already
#pragma unroll 1
    for (int pi = 0; pi < n_ph; ++pi) {
        const GridPhase& d = k.phases[pi];
        const int flags = d.flags;
        if (flags & GP_FILL_PLE) {
            // the table row of the pending token, input of a per-layer-embedding projection
            const T2* Tb = reinterpret_cast<const T2*>(d.ple_table);
#pragma unroll 1
            for (int j = tid; j < p.ple; j += kMegaConsumers)
                plerow[xs_index<EPV2>(j, p.ple / EPV2)] = Elem<T2>::get(Tb, (size_t)tok * p.ple + j);
        }
        RowsJob job;
        job.mode = d.mode; job.rows = d.rows; job.K = d.K; job.r0 = d.r0;
        job.xs = smem + d.xs_off;
        job.scale = d.scale; job.scale2 = d.scale2;
        job.dst = d.dst; job.epoch = base + (uint32_t)d.e_off;
        job.resid = d.resid_off >= 0 ? smem + d.resid_off : nullptr;
        job.pacc = (flags & GP_PACC_IN) ? pacc : nullptr;
        job.out_s = pacc;
        job.logits = d.logits;
        const float* gain = d.gain;
        const float* nsrc = smem + d.nsrc_off;
        MLB_GT(8)

        // ---- the one copy of gather, norm, rows ------------------------------------------------------------
        float ss = 0.f;
        if (d.g_src && !(abuf_ready && (flags & GP_SKIP_GATHER_IF_READY))) {
            ss = ll_gather<EPV>(d.g_src, d.g_n, base + (uint32_t)d.g_e_off, smem + d.g_dst_off, d.g_perm, k);
        } else if (gain) {
            consumer_sync();            // the embedding row, written by other threads
#pragma unroll 1
            for (int i = tid; i < p.d; i += kMegaConsumers) ss = fmaf(nsrc[i], nsrc[i], ss);
        }
        MLB_GT(1)
        if (gain) grid_norm<EPV>(ss, nsrc, xn, gain, p.d, p.eps, red, tid, warp, lane);
        else consumer_sync();           // what was gathered (or pacc, plerow, the embedding row) is complete
        MLB_GT(2)
        if (!kSameT2 && (flags & GP_T2)) consume_rows<T2>(ring, job, false, warp, lane, bv, bi);
        else consume_rows<T>(ring, job, (flags & GP_PAIR) != 0, warp, lane, bv, bi);
        MLB_GT(3)

        // ---- the mixer (no weights) runs between the QKV rows and the O rows ---------------------------------
        if (flags & GP_MIX_ATTN) {
            // flash-decode items, then the split combine
            const MegaLayer& L = k.layers[d.layer];
            const uint32_t e1 = job.epoch, e2 = base + (uint32_t)d.mix_e2_off, e_a = base + (uint32_t)d.mix_ea_off;
            const int npages = pos / kKvBlock + 1;
            const int s_cap = max(1, min(p.s_max, C / p.kv_heads));
            int S = (npages + kGridAttnWarps - 1) / kGridAttnWarps;
            const bool direct = S <= s_cap && p.heads * S * (hd + 2) <= kGridDirectWords;
            int pps = kGridAttnWarps;
            if (!direct) {
                pps = (npages + s_cap - 1) / s_cap;
                S = (npages + pps - 1) / pps;
            }
            if (hd == 64) grid_attention<KVT, 64>(p, L, k, e1, e2, S, pps);
            else grid_attention<KVT, 128>(p, L, k, e1, e2, S, pps);
            MLB_GT(4)
            grid_combine<EPV>(p, L, k, e1, e2, e_a, S, direct);
            abuf_ready = direct;
            MLB_GT(5)
        } else if (flags & GP_MIX_DELTA) {
            // gated delta-net on this CTA's rows of the state
            const MegaLayer& L = k.layers[d.layer];
            ll_gather<EPV>(p.ll_proj, L.n_qkv, job.epoch, proj, 0, k);
            consumer_sync();
            grid_delta_net(p, L, k, base + (uint32_t)d.mix_ea_off);
            abuf_ready = false;
            MLB_GT(6)
        }
    }
    const uint32_t ph = base + (uint32_t)(p.with_lm_head ? p.e_total : p.e_total_nolm);

    if (p.with_lm_head) {
        // reduce the warps' picks (lane 0 of each warp holds them), then (in CTA 0) the grid's
        consumer_sync();
        if (lane == 0) { tmp[2 * warp] = bv; tmp[2 * warp + 1] = __int_as_float(bi); }
        consumer_sync();
        if (tid == 0) {
            for (int w = 1; w < kMegaWarps; ++w) {
                const float v = tmp[2 * w];
                const int ix = __float_as_int(tmp[2 * w + 1]);
                if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
            }
            ll_store(p.ll_lm + 2 * rank, bv, ph);
            ll_store(p.ll_lm + 2 * rank + 1, __int_as_float(bi), ph);
        }
    }
#ifdef MLB_GRID_TIMERS
    if (tid == 0) {
        k.tm[0] += clock64() - tstart;
        k.tm[14] += ring.wait_cycles;
        if (p.timers)
            for (int i = 0; i < kGridTimers; ++i) p.timers[(size_t)rank * kGridTimers + i] += k.tm[i];
    }
#endif
    if (rank == 0) {
        if (p.with_lm_head) {
            consumer_sync();
            float* lm = smem + p.off_parts;          // free by now
            ll_gather<4>(p.ll_lm, 2 * C, ph, lm, 0, k);
            consumer_sync();
            if (tid == 0 && p.do_pick) {
                float best = lm[0];
                int at = __float_as_int(lm[1]);
                for (int r = 1; r < C; ++r) {
                    const float v = lm[2 * r];
                    const int ix = __float_as_int(lm[2 * r + 1]);
                    if (v > best || (v == best && ix < at)) { best = v; at = ix; }
                }
                advance_seq(c, 0, at);
            }
        } else if (tid == 0) {
            advance_seq(c, 0, -1);
        }
        // Every CTA read the epoch word when it started, and this CTA got here only through data
        // that all of them produced: the word is free to move on.
        if (tid == 0) *p.epoch = ph;
    }
}

template <typename T, typename T2, typename KVT>
__global__ void __launch_bounds__(kMegaThreads, 1) grid_decode_kernel(StepCtl c, GridParams p) {
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
    k.tok = c.tok[0];
    k.pos = c.pos[0];
    k.base = *p.epoch;
    int* dead = reinterpret_cast<int*>(smem + p.off_red + kMegaWarps);
    k.dead = dead;
    k.err = p.err;
    k.tm = reinterpret_cast<long long*>(smem + p.off_timers);
    k.tmark = 0;
    k.ring.wait_cycles = 0;
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
        const int n8 = p.n_layers * (int)(sizeof(MegaLayer) / 8);
        const unsigned long long* src = reinterpret_cast<const unsigned long long*>(p.layers);
        unsigned long long* dstl = reinterpret_cast<unsigned long long*>(smem + p.off_layers);
#pragma unroll 1
        for (int i = threadIdx.x; i < n8; i += kMegaThreads) dstl[i] = src[i];
        k.layers = reinterpret_cast<const MegaLayer*>(dstl);
    }
    {
        // the phase list moves to shared memory too
        const int n16 = p.n_phases * (int)(sizeof(GridPhase) / 16);
        const uint4* src = reinterpret_cast<const uint4*>(p.phases);
        uint4* dstp = reinterpret_cast<uint4*>(smem + p.off_phases);
#pragma unroll 1
        for (int i = threadIdx.x; i < n16; i += kMegaThreads) dstp[i] = src[i];
        k.phases = reinterpret_cast<const GridPhase*>(dstp);
    }
    if (threadIdx.x == 0) {
        *dead = 0;
        for (int i = 0; i < kGridTimers; ++i) k.tm[i] = 0;
        for (int i = 0; i < p.n_stages; ++i) {
            mbar_init(k.ring.full0 + 8u * i, 1);                    // the producer's expect_tx arrival
            mbar_init(k.ring.empty0 + 8u * i, kMegaWarps);          // one arrival per consumer warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // this CTA's rows of every phase
    for (int i = threadIdx.x; i < p.n_phases; i += kMegaThreads) {
        GridPhase* d = const_cast<GridPhase*>(k.phases) + i;
        int r0, r1;
        grid_rows(d->N, k.C, k.rank, r0, r1);
        d->r0 = r0;
        d->rows = r1 - r0;
    }
    __syncthreads();
    if (k.warp == kMegaWarps) grid_producer(p, k);
    else grid_consumer<T, T2, KVT>(c, p, k);
}

}  // namespace mlb
