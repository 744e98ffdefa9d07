// The whole-GPU batch-1 decode step (grid.cuh) with every shape a compile-time constant.
//
// At batch 1 a warp runs a dependent chain of a few hundred instructions per phase, at 5-8 cycles
// per instruction; the generic kernel's index arithmetic (row tables, divisions by run-time row
// counts, run-time loop bounds, per-row mode switches) is most of that chain, and its code does
// not stay resident in the instruction caches. Here the model's dimensions, the CTA count and the
// rows per CTA are template parameters: a thread's exchange addresses are a shift and an add,
// the dot products are fully unrolled, a phase is ~100 instructions and the kernel is a few KB.
// Same structure and same arithmetic as grid.cuh (producer warp + ring, {value, epoch} words in
// per-producer slots, late-applied norm, attention items out of shared memory); the host takes
// this kernel when the session's model matches an instantiated shape, and grid.cuh otherwise.
//
// Restrictions of a shape: bf16 weights, no QK-norm, no query gating, d divisible by the CTA
// count (every CTA owns rows of the residual stream, which the reuse rule of the exchange buffers
// rests on), and the device must keep C CTAs resident (cooperative launch).
#pragma once
#include "grid.cuh"
#include "lean_params.h"

namespace mlb {

template <int D_, int F_, int V_, int H_, int KVH_, int HD_, int DK_, int DV_, int PLE_, int C_>
struct LeanShape {
    static constexpr int D = D_, F = F_, V = V_, H = H_, KVH = KVH_, HD = HD_, DK = DK_, DV = DV_, PLE = PLE_, C = C_;
    static constexpr int G = H / KVH;
    static constexpr int NQ_A = H * HD + 2 * KVH * HD;          // q | k | v rows of an attention layer
    static constexpr int NQ_D = 2 * H * DK + H * DV + 2 * H;    // q | k | v | beta | alpha rows of a delta-net layer
    static constexpr int NA_D = H * DV;                         // delta-net output
    static constexpr int NA_A = H * HD;                         // attention output
    static constexpr int RX = D / C;                            // rows of the residual stream per CTA (exact)
    static constexpr int RQA = (NQ_A + C - 1) / C, RQD = (NQ_D + C - 1) / C;
    static constexpr int RH = (F + C - 1) / C, RAD = (NA_D + C - 1) / C, RV = (V + C - 1) / C;
    static constexpr int W = HD + 2;                            // words of a flash-decode partial
    static_assert(D % C == 0, "every CTA must own rows of the residual stream");
    static_assert(H % KVH == 0 && (HD == 64 || HD == 128) && D % 8 == 0 && F % 8 == 0, "shape not supported");
};

// Bounded poll of up to NWORD words: returns once all carry epoch e (or a wait ran out).
template <int NWORD>
__device__ __forceinline__ void lean_poll(const unsigned long long* const (&src)[NWORD], unsigned long long (&w)[NWORD], uint32_t e,
                                          volatile int* dead, int* err) {
    uint32_t spins = 0;
#pragma unroll 1
    for (;;) {
        bool ok = true;
#pragma unroll
        for (int u = 0; u < NWORD; ++u) {
            w[u] = ll_load(src[u]);
            ok = ok && (uint32_t)(w[u] >> 32) == e;
        }
        if (ok) break;
        if ((++spins & 255u) == 0u) {
            if (*dead) break;
            if (spins > kGridSpinLimit) {
                *dead = 1;
                atomicExch(err, 3);
                break;
            }
        }
    }
}

// The whole vector of N values (RPC per producer) into the GEMV layout of K = N elements at xs
// (times gain, if gain), and linearly into lin (if lin). Returns this thread's sum of squares.
template <int N, int RPC, bool GAIN, bool LIN>
__device__ __forceinline__ float lean_gather(const unsigned long long* buf, uint32_t e, const float* __restrict__ gain, float* lin, float* xs,
                                             int tid, volatile int* dead, int* err) {
    constexpr int NW = (N + kLeanConsumers - 1) / kLeanConsumers;      // words per thread
    constexpr int SLOT = lean_slot(RPC);
    constexpr int NVEC = N / 8;
    const unsigned long long* src[NW];
    unsigned long long w[NW];
    float g[NW];
#pragma unroll
    for (int u = 0; u < NW; ++u) {
        const int q = min(tid + u * kLeanConsumers, N - 1);               // a thread past the end repeats the last word
        const int c = q / RPC, j = q - c * RPC;
        src[u] = buf + c * SLOT + j;
        g[u] = GAIN ? gain[q] : 1.0f;
    }
    lean_poll<NW>(src, w, e, dead, err);
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < NW; ++u) {
        const int q = tid + u * kLeanConsumers;
        if (N % kLeanConsumers == 0 || u + 1 < NW || q < N) {
            const float val = __uint_as_float((uint32_t)w[u]);
            if (LIN) lin[q] = val;
            xs[xs_index<8>(q, NVEC)] = val * g[u];
            ss = fmaf(val, val, ss);
        }
    }
    return ss;
}

// n consecutive rows of a vector starting at row0 (n <= 4 * 512) to dst[0..n).
template <int RPC>
__device__ __forceinline__ void lean_gather_rows(const unsigned long long* buf, int row0, int n, uint32_t e, float* dst, int tid,
                                                 volatile int* dead, int* err) {
    constexpr int SLOT = lean_slot(RPC);
#pragma unroll 1
    for (int i = tid; i < n; i += kLeanConsumers) {
        const int q = row0 + i;
        const int c = q / RPC, j = q - c * RPC;
        const unsigned long long* src[1] = {buf + c * SLOT + j};
        unsigned long long w[1];
        lean_poll<1>(src, w, e, dead, err);
        dst[i] = __uint_as_float((uint32_t)w[0]);
    }
}

// One over the RMS norm of the vector whose per-warp sums of squares stand in red[0..16).
template <int N>
__device__ __forceinline__ float lean_rnorm(const float* red, int lane, float eps) {
    float t = red[lane & (kLeanWarps - 1)];
#pragma unroll
    for (int o = kLeanWarps / 2; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return rsqrtf(t * (1.0f / (float)N) + eps);
}

// Dot product of a bf16 row of K elements in shared memory with the input at xs (GEMV layout).
template <int K>
__device__ __forceinline__ float lean_dot(const bf16_t* row, const float* xs, int lane) {
    constexpr int NVEC = K / 8;
    const float4* xp = reinterpret_cast<const float4*>(xs);
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int i = 0; i < (NVEC + 31) / 32; ++i) {
        const int vi = lane + 32 * i;
        if (NVEC % 32 == 0 || i + 1 < (NVEC + 31) / 32 || vi < NVEC) {
            float w[8];
            Elem<bf16_t>::unpack(*reinterpret_cast<const uint4*>(row + vi * 8), w);
            const float4 t0 = xp[vi], t1 = xp[NVEC + vi];
            a0 = fmaf(w[0], t0.x, a0); a1 = fmaf(w[1], t0.y, a1);
            a0 = fmaf(w[2], t0.z, a0); a1 = fmaf(w[3], t0.w, a1);
            a0 = fmaf(w[4], t1.x, a0); a1 = fmaf(w[5], t1.y, a1);
            a0 = fmaf(w[6], t1.z, a0); a1 = fmaf(w[7], t1.w, a1);
        }
    }
    return warp_sum(a0 + a1);
}

enum { LM_STORE = 0, LM_RESID = 1, LM_SWIGLU = 2, LM_LOGITS = 3 };

// This CTA's rows (at most ROWS, `rows` here) of a matrix with rows of K elements, out of the ring.
// Local row r belongs to warp r % 16. MODE says how a row is finished. The chunk geometry is the
// producer's: whole rows per 16 KB stage, gate and up chunks alternating (PAIR).
// The finished rows are collected in shared memory (`obuf`) and the warp that finishes the last one
// (`ocnt` counts them) publishes the whole slot with ONE store instruction: a line that all CTAs
// poll must change once. (Measured on B200: with the rows of a slot stored one by one by their warps,
// a few dozen cycles apart, an exchange costs 3-4 us instead of 1.2 us.)
template <int K, int ROWS, int MODE, bool PAIR, int ROPE_N = 0, int ROPE_HD = 64>
__device__ __forceinline__ void lean_rows(Ring& r, int rows, int row0, const float* xs, float rn, unsigned long long* dst, uint32_t e,
                                          const float* resid, const float* pacc, float* logits, float* obuf, int* ocnt, int warp, int lane, float& bv, int& bi,
                                          long long* tm = nullptr, const float* rope_row = nullptr) {
    constexpr int RPS = kLeanStage / (K * 2);        // rows per stage
    static_assert(RPS >= 1, "a row must fit a ring stage");
    constexpr int NCH = (ROWS + RPS - 1) / RPS;
    // RoPE factors of the row this lane would publish (whichever warp finishes last publishes): asked for now
    float rope_cs = 1.f, rope_sn = 0.f;
    if (ROPE_N > 0) {
        static_assert(ROPE_N == 0 || (ROWS % 2 == 0 && ROWS <= 32), "a RoPE pair must not straddle two CTAs");
        const int row = row0 + lane;
        if (lane < rows && row < ROPE_N) {
            const float2 t = *reinterpret_cast<const float2*>(rope_row + ((row & (ROPE_HD - 1)) & ~1));
            rope_cs = t.x;
            rope_sn = t.y;
        }
    }
#pragma unroll 1
    for (int ch = 0; ch < NCH; ++ch) {
        const int c0 = ch * RPS;
        if (c0 >= rows) break;
        const int n = min(RPS, rows - c0);
        const int ia = r.idx;
        const long long tw = tm ? clock64() : 0;
        r.wait(r.full0 + 8u * r.idx, r.phase, 2);
        r.advance();
        int ib = ia;
        if (PAIR) {
            ib = r.idx;
            r.wait(r.full0 + 8u * r.idx, r.phase, 2);
            r.advance();
        }
        const long long td = tm ? clock64() : 0;
        if (tm && threadIdx.x == 0) tm[18] += td - tw;
        const bf16_t* A = reinterpret_cast<const bf16_t*>(r.stages + (size_t)ia * kLeanStage);
        const bf16_t* Bm = reinterpret_cast<const bf16_t*>(r.stages + (size_t)ib * kLeanStage);
#pragma unroll 1
        for (int lr = warp; lr < n; lr += kLeanWarps) {
            const int wrow = c0 + lr;
            float v = lean_dot<K>(A + lr * K, xs, lane) * rn;
            if (PAIR) {
                const float u = lean_dot<K>(Bm + lr * K, xs, lane) * rn;
                v = __fdividef(v, 1.0f + __expf(-v)) * u;      // applySiluToFFN + hadamardMultiplyFFN, inference.cu:262-281
            }
            int last = 0;
            if (lane == 0) {
                if (MODE == LM_RESID) {
                    v += resid[row0 + wrow];
                    if (pacc) v += pacc[wrow];
                }
                if (MODE == LM_LOGITS) {
                    const int row = row0 + wrow;
                    logits[row] = v;
                    if (v > bv || (v == bv && row < bi)) { bv = v; bi = row; }
                } else {
                    obuf[wrow] = v;
                    __threadfence_block();
                    last = atomicAdd(ocnt, 1) == rows - 1;
                }
            }
            if (MODE != LM_LOGITS) {
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence_block();
#pragma unroll
                    for (int j0 = 0; j0 < ROWS; j0 += 32) {
                        if (j0 + lane < rows) {
                            float o = obuf[j0 + lane];
                            if (ROPE_N > 0) {
                                // RoPE on adjacent pairs of the q and k rows (inference.cu:113-134), applied where the
                                // slot is published: both rows of a pair stand in this slot (identity factors elsewhere)
                                const float other = obuf[(j0 + lane) ^ 1];
                                o = (lane & 1) ? rope_sn * other + rope_cs * o : rope_cs * o - rope_sn * other;
                            }
                            ll_store(dst + j0 + lane, o, e);
                        }
                    }
                    if (lane == 0) *ocnt = 0;
                }
            }
        }
        if (tm && threadIdx.x == 0) tm[19] += clock64() - td;
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(r.empty0 + 8u * ia);
            if (PAIR) mbar_arrive(r.empty0 + 8u * ib);
        }
    }
}

// Producer side of lean_rows: `rows` rows of K bf16 elements starting at `a` (and at `b`: the pair).
template <int K, int ROWS, bool PAIR>
__device__ __forceinline__ void lean_issue(Ring& r, const unsigned char* a, const unsigned char* b, int rows, int lane) {
    constexpr int RPS = kLeanStage / (K * 2);
    constexpr int NCH = (ROWS + RPS - 1) / RPS;
#pragma unroll 1
    for (int ch = 0; ch < NCH; ++ch) {
        const int c0 = ch * RPS;
        if (c0 >= rows) break;
        const uint32_t bytes = (uint32_t)min(RPS, rows - c0) * (uint32_t)(K * 2);
#pragma unroll
        for (int which = 0; which < (PAIR ? 2 : 1); ++which) {
            if (lane == 0 && r.wait(r.empty0 + 8u * r.idx, r.phase ^ 1u, 1)) {
                mbar_expect_tx(r.full0 + 8u * r.idx, bytes);
                bulk_g2s(smem_u32(r.stages + (size_t)r.idx * kLeanStage), (which ? b : a) + (size_t)c0 * (K * 2), bytes, r.full0 + 8u * r.idx);
            }
            r.advance();
        }
    }
}

// Flash-decode of this CTA's item out of shared memory (grid_attention with compile-time shapes,
// no QK-norm): 16/G warps per query head. Publishes G partials in the item's slot. The q and k
// rows arrive with RoPE applied (the QKV phase rotates them when it publishes its slot).
template <typename S, typename KVT, typename Mark>
__device__ __forceinline__ void lean_attention(const LeanParams& p, const StepLayer& L, const GridPlan& it, Ring& ring, float* mix, int rank,
                                               int pos, uint32_t e_proj, uint32_t e_out, int tid, volatile int* dead, int* err, Mark&& mark) {
    constexpr int HD = S::HD, G = S::G, W = S::W;
    constexpr int EPL = 16 / (int)sizeof(KVT), LPR = HD / EPL, PPI = 32 / LPR;
    constexpr int WPH = kLeanWarps / G;               // warps per query head
    static_assert(WPH >= 1 && WPH * G == kLeanWarps && G * W <= kLeanConsumers, "query heads per kv head must divide the warp count");
    constexpr int PAGE = kKvBlock * HD * (int)sizeof(KVT);
    constexpr int PPC = kLeanStage / PAGE < 32 ? kLeanStage / PAGE : 32;      // pages per stage
    const int lane = tid & 31, warp = tid >> 5;
    const int kvh = it.kvh, h0 = kvh * G;
    const int lr = lane % LPR, grp = lane / LPR;
    float* tq = mix;                                  // [G][HD]
    float* tk = tq + G * HD;                          // [HD]
    float* tv = tk + HD;                              // [HD]
    float* wpart = tv + HD;                           // [16][W]
    const int g = warp / WPH, sub = warp - g * WPH;

    lean_gather_rows<S::RQA>(p.pj, h0 * HD, G * HD, e_proj, tq, tid, dead, err);
    if (it.cur_here) {
        lean_gather_rows<S::RQA>(p.pj, S::H * HD + kvh * HD, HD, e_proj, tk, tid, dead, err);
        lean_gather_rows<S::RQA>(p.pj, S::H * HD + S::KVH * HD + kvh * HD, HD, e_proj, tv, tid, dead, err);
    }
    consumer_sync<kLeanWarps>();
    mark(20);
    const float inv_div = rsqrtf((float)HD);          // scores are divided by sqrt(hd), inference.cu:154
    float q[EPL], acc[EPL], m = kNegBig, l = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        q[e] = tq[g * HD + lr * EPL + e] * inv_div;
        acc[e] = 0.f;
    }
#pragma unroll 1
    for (int c0 = 0; c0 < it.pages_prev; c0 += PPC) {
        const int ia = ring.idx;
        ring.wait(ring.full0 + 8u * ring.idx, ring.phase, 2);
        ring.advance();
        const int ib = ring.idx;
        ring.wait(ring.full0 + 8u * ring.idx, ring.phase, 2);
        ring.advance();
        const KVT* Ks = reinterpret_cast<const KVT*>(ring.stages + (size_t)ia * kLeanStage);
        const KVT* Vs = reinterpret_cast<const KVT*>(ring.stages + (size_t)ib * kLeanStage);
        const int cnt = min(PPC * kKvBlock, it.n_prev - c0 * kKvBlock);      // earlier positions in this chunk
#pragma unroll 1
        for (int j0 = sub * PPI; j0 < cnt; j0 += WPH * PPI) {
            const int j = j0 + grp;
            const bool valid = j < cnt;
            const int jj = valid ? j : 0;
            float kv[EPL], vv[EPL];
            Elem<KVT>::unpack(*reinterpret_cast<const uint4*>(Ks + jj * HD + lr * EPL), kv);
            Elem<KVT>::unpack(*reinterpret_cast<const uint4*>(Vs + jj * HD + lr * EPL), vv);
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
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(ring.empty0 + 8u * ia);
            mbar_arrive(ring.empty0 + 8u * ib);
        }
    }
    mark(22);
    if (it.cur_here && sub == 0) {
        // the current position: its K/V row, rounded the way the cache stores it; the first warp also appends it to the pool
        float kc[EPL], vc[EPL];
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            kc[e] = tk[lr * EPL + e];
            vc[e] = tv[lr * EPL + e];
        }
        if (warp == 0 && grp == 0) {
            KVT* kpool = reinterpret_cast<KVT*>(L.kpool);
            KVT* vpool = reinterpret_cast<KVT*>(L.vpool);
            const size_t row_off = (((size_t)p.page_table[pos / kKvBlock] * S::KVH + kvh) * kKvBlock + (pos % kKvBlock)) * HD + lr * EPL;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                Elem<KVT>::put(kpool, row_off + e, kc[e]);
                Elem<KVT>::put(vpool, row_off + e, vc[e]);
            }
        }
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            kc[e] = round_kv<KVT>(kc[e]);
            vc[e] = round_kv<KVT>(vc[e]);
            s = fmaf(q[e], kc[e], s);
        }
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (grp == 0) {
            const float mn = fmaxf(m, s);
            const float sc = __expf(m - mn), pe = __expf(s - mn);
            l = l * sc + pe;
#pragma unroll
            for (int e = 0; e < EPL; ++e) acc[e] = acc[e] * sc + pe * vc[e];
            m = mn;
        }
    }
    // merge the position groups of the warp
#pragma unroll
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
        float* w = wpart + warp * W;
#pragma unroll
        for (int e = 0; e < EPL; ++e) w[lr * EPL + e] = acc[e];
        if (lr == 0) { w[HD] = m; w[HD + 1] = l; }
    }
    consumer_sync<kLeanWarps>();
    mark(23);
    // merge the warps of each head: every publishing warp works out the 16 warps' factors to their heads' common
    // maxima (its own copy in shared memory), then one thread per element of the item's partials
    constexpr int NSTORE = (G * W + 31) / 32;          // warps that publish
    if (warp < NSTORE) {
        float* wsc = wpart + kLeanWarps * W + warp * 2 * kLeanWarps;      // [16] factors, [16] maxima
        const int w16 = lane & (kLeanWarps - 1);
        const float mw = wpart[w16 * W + HD];
        float mx = mw;
#pragma unroll
        for (int o = WPH / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane < kLeanWarps) {
            wsc[lane] = __expf(mw - mx);
            wsc[kLeanWarps + lane] = mx;
        }
        __syncwarp();
        const int idx = tid;
        if (idx < G * W) {
            const int gg = idx / W, e = idx - gg * W;
            float val = wsc[kLeanWarps + gg * WPH];
            if (e != HD) {
                val = 0.f;
#pragma unroll
                for (int w = 0; w < WPH; ++w) val = fmaf(wpart[(gg * WPH + w) * W + e], wsc[gg * WPH + w], val);
            }
            ll_store(p.parts + (size_t)rank * lean_slot(G * W) + idx, val, e_out);
        }
    }
}

// Combine the context splits of heads [h_first, h_first + h_count): element i goes to the GEMV
// layout at xs (if xs), else into the slot `dst` with epoch e_out. One warp per partial fetches it.
template <typename S>
__device__ __forceinline__ void lean_combine(const LeanParams& p, int Ssp, int h_first, int h_count, uint32_t e_parts, float* parts, float* xs,
                                             unsigned long long* dst, uint32_t e_out, int tid, volatile int* dead, int* err) {
    constexpr int HD = S::HD, G = S::G, W = S::W, PSLOT = lean_slot(G * W);
    const int lane = tid & 31, warp = tid >> 5;
    int hl = warp / Ssp, sp = warp - hl * Ssp;
#pragma unroll 1
    for (int pi = warp; pi < h_count * Ssp; pi += kLeanWarps) {
        const int h = h_first + hl;
        const unsigned long long* base = p.parts + (size_t)((h / G) * Ssp + sp) * PSLOT + (h % G) * W;
        float* out = parts + pi * W;
        constexpr int NL = (W + 31) / 32;               // words per lane
        const unsigned long long* src[NL];
        unsigned long long w[NL];
#pragma unroll
        for (int u = 0; u < NL; ++u) src[u] = base + min(lane + 32 * u, W - 1);
        lean_poll<NL>(src, w, e_parts, dead, err);
#pragma unroll
        for (int u = 0; u < NL; ++u) out[min(lane + 32 * u, W - 1)] = __uint_as_float((uint32_t)w[u]);
        sp += kLeanWarps;
        while (sp >= Ssp) { sp -= Ssp; ++hl; }
    }
    consumer_sync<kLeanWarps>();
#pragma unroll 1
    for (int i = tid; i < h_count * HD; i += kLeanConsumers) {
        const int hh = i / HD, el = i - hh * HD;
        const float* pp = parts + hh * Ssp * W;
        float mn = kNegBig;
#pragma unroll 1
        for (int s2 = 0; s2 < Ssp; ++s2) mn = fmaxf(mn, pp[s2 * W + HD]);
        float lt = 0.f, at = 0.f;
#pragma unroll 1
        for (int s2 = 0; s2 < Ssp; ++s2) {
            const float sc = __expf(pp[s2 * W + HD] - mn);
            lt = fmaf(pp[s2 * W + HD + 1], sc, lt);
            at = fmaf(pp[s2 * W + el], sc, at);
        }
        const float o = __fdividef(at, lt);
        if (xs) xs[xs_index<8>(i, S::NA_A / 8)] = o;
        else ll_store(dst + i, o, e_out);
    }
}

// Gated delta-net step on this CTA's rows of the state (grid_delta_net with compile-time shapes).
template <typename S>
__device__ __forceinline__ void lean_delta_net(const LeanParams& p, const StepLayer& L, Ring& ring, float* mix, int rank, uint32_t e_proj,
                                               uint32_t e_out, float* obuf, int* ocnt, int tid, volatile int* dead, int* err) {
    constexpr int H = S::H, DK = S::DK, DV = S::DV, RAD = S::RAD;
    constexpr int RPS = kLeanStage / (DK * 4);
    static_assert(DK % 32 == 0 && DK <= 128 && RAD <= RPS, "delta-net shape not supported");
    const int lane = tid & 31, warp = tid >> 5;
    const int r0 = min(rank * RAD, S::NA_D), r1 = min(r0 + RAD, S::NA_D);
    const int rows = r1 - r0;
    if (rows <= 0) return;
    const int h_lo = r0 / DV, h_hi = (r1 - 1) / DV, nh = h_hi - h_lo + 1;
    float* qn = mix;                        // [nh][DK]
    float* kn = qn + nh * DK;               // [nh][DK]
    float* rv = kn + nh * DK;               // [rows]
    float* gates = rv + ((rows + 3) & ~3);  // beta[nh] then alpha[nh]
    constexpr int seg_k = H * DK, seg_v = 2 * H * DK, seg_b = seg_v + H * DV, seg_a = seg_b + H;
    lean_gather_rows<S::RQD>(p.pj, h_lo * DK, nh * DK, e_proj, qn, tid, dead, err);
    lean_gather_rows<S::RQD>(p.pj, seg_k + h_lo * DK, nh * DK, e_proj, kn, tid, dead, err);
    lean_gather_rows<S::RQD>(p.pj, seg_v + r0, rows, e_proj, rv, tid, dead, err);
    lean_gather_rows<S::RQD>(p.pj, seg_b + h_lo, nh, e_proj, gates, tid, dead, err);
    lean_gather_rows<S::RQD>(p.pj, seg_a + h_lo, nh, e_proj, gates + nh, tid, dead, err);
    consumer_sync<kLeanWarps>();
    // L2-normalise q and k of the heads this CTA touches: one warp per vector
#pragma unroll 1
    for (int hh = warp; hh < 2 * nh; hh += kLeanWarps) {
        float* vec = mix + hh * DK;
        float v[DK / 32], ss = 0.f;
#pragma unroll
        for (int i = 0; i < DK / 32; ++i) { v[i] = vec[lane + 32 * i]; ss = fmaf(v[i], v[i], ss); }
        const float rn = rsqrtf(warp_sum(ss) + p.l2_eps);
#pragma unroll
        for (int i = 0; i < DK / 32; ++i) vec[lane + 32 * i] = v[i] * rn;
    }
    consumer_sync<kLeanWarps>();
    unsigned long long* dst = p.a + (size_t)rank * lean_slot(RAD);
    const int ia = ring.idx;
    ring.wait(ring.full0 + 8u * ring.idx, ring.phase, 2);
    ring.advance();
    const float* Ss = reinterpret_cast<const float*>(ring.stages + (size_t)ia * kLeanStage);
#pragma unroll 1
    for (int wrow = warp; wrow < rows; wrow += kLeanWarps) {
        const int row = r0 + wrow;
        const int hl = row / DV - h_lo;
        const float* Sin = Ss + wrow * DK;
        float* Srow = L.state + (size_t)row * DK;                // sequence 0
        const float beta = fast_sigmoid(gates[hl]), alpha = fast_sigmoid(gates[nh + hl]);
        float s[DK / 32], kk[DK / 32], d1 = 0.f;
#pragma unroll
        for (int i = 0; i < DK / 32; ++i) {
            kk[i] = kn[hl * DK + lane + 32 * i];
            s[i] = Sin[lane + 32 * i] * alpha;
            d1 = fmaf(s[i], kk[i], d1);
        }
        d1 = warp_sum(d1);
        const float cf = beta * (rv[wrow] - d1);
        float d2 = 0.f;
#pragma unroll
        for (int i = 0; i < DK / 32; ++i) {
            s[i] = fmaf(cf, kk[i], s[i]);
            d2 = fmaf(s[i], qn[hl * DK + lane + 32 * i], d2);
            Srow[lane + 32 * i] = s[i];
        }
        d2 = warp_sum(d2);
        // the warp that finishes the CTA's last row publishes the slot with one store instruction
        int last = 0;
        if (lane == 0) {
            obuf[wrow] = d2;
            __threadfence_block();
            last = atomicAdd(ocnt, 1) == rows - 1;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
            __threadfence_block();
            for (int j = lane; j < rows; j += 32) ll_store(dst + j, obuf[j], e_out);
            if (lane == 0) *ocnt = 0;
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(ring.empty0 + 8u * ia);
}

// Thread 0, once per step: the attention plan (grid_make_plan with this shape's limits).
template <typename S>
__device__ __forceinline__ void lean_make_plan(int pages_per_split, int pos, int rank, GridPlan* g) {
    constexpr int s_cap = S::C / S::KVH;
    constexpr int s_dir_raw = kLeanDirectWords / (S::H * S::W);
    constexpr int s_dir = s_dir_raw < 1 ? 1 : (s_dir_raw > s_cap ? s_cap : s_dir_raw);
    const int npages = pos / kKvBlock + 1, cur_page = pos / kKvBlock;
    int Ssp = min(s_cap, (npages + pages_per_split - 1) / pages_per_split);
    int direct = Ssp <= s_dir;
    if (!direct && (npages + s_dir - 1) / s_dir <= 2 * pages_per_split) {
        Ssp = s_dir;
        direct = 1;
    }
    const int pps = (npages + Ssp - 1) / Ssp;
    Ssp = (npages + pps - 1) / pps;
    g->S = Ssp; g->pps = pps; g->direct = direct;
    g->has = rank < S::KVH * Ssp;
    g->kvh = rank / Ssp;
    g->split = rank - g->kvh * Ssp;
    g->pg_begin = g->split * pps;
    const int pg_end = min(npages, g->pg_begin + pps);
    g->cur_here = g->has && cur_page >= g->pg_begin && cur_page < pg_end;
    g->n_prev = g->has ? max(0, min(pos, pg_end * kKvBlock) - g->pg_begin * kKvBlock) : 0;
    g->pages_prev = (g->n_prev + kKvBlock - 1) / kKvBlock;
    g->pad0 = 0; g->pad1 = 0;
}

template <typename S, typename KVT>
__device__ __forceinline__ void lean_producer(const LeanParams& p, Ring& ring, const StepLayer* layers, const GridPlan& it, int rank, int lane) {
    constexpr int PAGE = kKvBlock * S::HD * (int)sizeof(KVT);
    constexpr int PPC = kLeanStage / PAGE < 32 ? kLeanStage / PAGE : 32;
#pragma unroll 1
    for (int li = 0; li < p.n_layers; ++li) {
        const StepLayer& L = layers[li];
        const bool attn = L.type == 0;
        if (attn) {
            const int r0 = min(rank * S::RQA, S::NQ_A), rows = min(S::RQA, S::NQ_A - r0);
            lean_issue<S::D, S::RQA, false>(ring, reinterpret_cast<const unsigned char*>(L.Wqkv) + (size_t)r0 * S::D * 2, nullptr, rows, lane);
            // the item's K and V pages: a K stage, then a V stage, one bulk copy per page
            const int n_pages = it.has ? it.pages_prev : 0;
            const unsigned char* kp = reinterpret_cast<const unsigned char*>(L.kpool) + (size_t)it.kvh * PAGE;
            const unsigned char* vp = reinterpret_cast<const unsigned char*>(L.vpool) + (size_t)it.kvh * PAGE;
#pragma unroll 1
            for (int c0 = 0; c0 < n_pages; c0 += PPC) {
                const int n = min(PPC, n_pages - c0);
                size_t src_off = 0;
                if (lane < n) src_off = (size_t)p.page_table[it.pg_begin + c0 + lane] * S::KVH * PAGE;
#pragma unroll
                for (int which = 0; which < 2; ++which) {
                    int ok = 0;
                    if (lane == 0) {
                        ok = ring.wait(ring.empty0 + 8u * ring.idx, ring.phase ^ 1u, 1) ? 1 : 0;
                        if (ok) mbar_expect_tx(ring.full0 + 8u * ring.idx, (uint32_t)n * PAGE);
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (ok && lane < n)
                        bulk_g2s(smem_u32(ring.stages + (size_t)ring.idx * kLeanStage + (size_t)lane * PAGE), (which ? vp : kp) + src_off, PAGE,
                                 ring.full0 + 8u * ring.idx);
                    ring.advance();
                }
            }
        } else {
            const int r0 = min(rank * S::RQD, S::NQ_D), rows = min(S::RQD, S::NQ_D - r0);
            lean_issue<S::D, S::RQD, false>(ring, reinterpret_cast<const unsigned char*>(L.Wqkv) + (size_t)r0 * S::D * 2, nullptr, rows, lane);
            // this CTA's rows of the state: one stage
            const int q0 = min(rank * S::RAD, S::NA_D), qrows = min(S::RAD, S::NA_D - q0);
            if (qrows > 0) {
                if (lane == 0 && ring.wait(ring.empty0 + 8u * ring.idx, ring.phase ^ 1u, 1)) {
                    const uint32_t bytes = (uint32_t)qrows * S::DK * 4;
                    mbar_expect_tx(ring.full0 + 8u * ring.idx, bytes);
                    bulk_g2s(smem_u32(ring.stages + (size_t)ring.idx * kLeanStage), reinterpret_cast<const unsigned char*>(L.state) + (size_t)q0 * S::DK * 4,
                             bytes, ring.full0 + 8u * ring.idx);
                }
                ring.advance();
            }
        }
        {
            constexpr int KO = S::NA_A;        // the mixer's output width (attention and delta-net outputs are equally wide here)
            const int r0 = rank * S::RX;
            lean_issue<KO, S::RX, false>(ring, reinterpret_cast<const unsigned char*>(L.Wo) + (size_t)r0 * KO * 2, nullptr, S::RX, lane);
        }
        {
            const int r0 = min(rank * S::RH, S::F), rows = min(S::RH, S::F - r0);
            lean_issue<S::D, S::RH, true>(ring, reinterpret_cast<const unsigned char*>(L.W1a) + (size_t)r0 * S::D * 2,
                                          reinterpret_cast<const unsigned char*>(L.W1b) + (size_t)r0 * S::D * 2, rows, lane);
        }
        lean_issue<S::F, S::RX, false>(ring, reinterpret_cast<const unsigned char*>(L.W2) + (size_t)rank * S::RX * S::F * 2, nullptr, S::RX, lane);
    }
    if (p.with_lm_head) {
        const int r0 = min(rank * S::RV, S::V), rows = min(S::RV, S::V - r0);
        lean_issue<S::D, S::RV, false>(ring, reinterpret_cast<const unsigned char*>(p.E) + (size_t)r0 * S::D * 2, nullptr, rows, lane);
    }
    __syncwarp();
}

template <typename S, typename KVT>
__global__ void __launch_bounds__(kLeanThreads, 1) lean_decode_kernel(const __grid_constant__ StepCtl c, const __grid_constant__ LeanParams p) {
    static_assert(S::NA_A == S::NA_D, "the output projection is instantiated for one input width");
    if (!seq_active(c, 0)) return;                    // uniform over the grid
    extern __shared__ __align__(128) float lean_smem[];
    float* smem = lean_smem;
    const int rank = (int)blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned long long g_entry = 0;
    if (p.trace != nullptr && tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g_entry));
    const int tok = p.tok_arg >= 0 ? p.tok_arg : c.tok[0];
    const int pos = c.pos[0];
    uint32_t e = *p.epoch;
    int* dead = reinterpret_cast<int*>(smem + p.off_red + 2 * kLeanWarps);
    GridPlan* plan = reinterpret_cast<GridPlan*>(smem + p.off_plan);
    Ring ring;
    ring.backoff_ns = 100;
    ring.full0 = smem_u32(smem + p.off_bar);
    ring.empty0 = ring.full0 + 8u * p.n_stages;
    ring.stages = reinterpret_cast<unsigned char*>(smem + p.off_ring);
    ring.nst = p.n_stages;
    ring.stage_bytes = kLeanStage;
    ring.idx = 0;
    ring.phase = 0;
    ring.dead = dead;
    ring.err = p.err;
    const StepLayer* layers;
    {
        const int n8 = p.n_layers * (int)(sizeof(StepLayer) / 8);
        const unsigned long long* src = reinterpret_cast<const unsigned long long*>(p.layers);
        unsigned long long* dstl = reinterpret_cast<unsigned long long*>(smem + p.off_layers);
#pragma unroll 1
        for (int i = tid; i < n8; i += kLeanThreads) dstl[i] = src[i];
        layers = reinterpret_cast<const StepLayer*>(dstl);
    }
    if (tid == 0) {
        *dead = 0;
        dead[1] = 0;                     // the finished-row counter
        for (int i = 0; i < p.n_stages; ++i) {
            mbar_init(ring.full0 + 8u * i, 1);
            mbar_init(ring.empty0 + 8u * i, kLeanWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        lean_make_plan<S>(p.pages_per_split, pos, rank, plan);
    }
    __syncthreads();
    if (warp == kLeanWarps) {
        lean_producer<S, KVT>(p, ring, layers, *plan, rank, lane);
        return;
    }
    // ---- consumers ------------------------------------------------------------------------------------------
    constexpr int D = S::D, F = S::F, RX = S::RX;
    float* xsb[2] = {smem + p.off_xs, smem + p.off_xs + p.xs_stride};
    float* redb[2] = {smem + p.off_red, smem + p.off_red + kLeanWarps};
    int* ocnt = reinterpret_cast<int*>(smem + p.off_red + 2 * kLeanWarps + 1);
    float* obuf = smem + p.off_red + 2 * kLeanWarps + 4;      // finished rows of the current phase
    float* xa = smem + p.off_xa;
    float* xb = smem + p.off_xb;
    float* pacc = smem + p.off_pacc;    // [layer][RX]
    float* parts = smem + p.off_parts;
    float* mix = smem + p.off_mix;
    long long* tm = p.timers ? reinterpret_cast<long long*>(smem + p.off_timers) : nullptr;
    long long tmark = 0, tstart = 0;
    if (tm) {
        if (tid == 0) for (int i = 0; i < kGridTimerSlots; ++i) tm[i] = 0;
        tstart = tmark = clock64();
    }
    int n_trace = 0;
    if (p.trace != nullptr && tid == 0) p.trace[(size_t)rank * kLeanTraceLen + n_trace++] = (long long)((g_entry << 8) | 30ull);
    auto mark = [&](int i) {
        if (tm != nullptr && tid == 0) {
            const long long n = clock64();
            tm[i] += n - tmark;
            tmark = n;
            if (p.trace != nullptr && n_trace < kLeanTraceLen) {
                unsigned long long g;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
                p.trace[(size_t)rank * kLeanTraceLen + n_trace++] = (long long)((g << 8) | (unsigned long long)i);
            }
        }
    };
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    const int xr0 = rank * RX;

    // per-layer embeddings: pacc[l][j] = P_l[xr0 + j] . T_l[tok]; 8 lanes per (layer, row), 16-byte loads, all
    // layers in one round of loads
    if (S::PLE > 0) {
        static_assert(S::PLE % 8 == 0, "per-layer embedding rows are read as 16-byte vectors");
        const int n = p.n_layers * RX;
        const int sub = lane & 7;
#pragma unroll 1
        for (int i = warp * 4 + (lane >> 3); i < (n + 3) / 4 * 4; i += kLeanWarps * 4) {
            float a = 0.f;
            if (i < n) {
                const int l = i / RX, j = i - l * RX;
                const bf16_t* Pm = reinterpret_cast<const bf16_t*>(layers[l].pleP) + (size_t)(xr0 + j) * S::PLE;
                const bf16_t* Tb = reinterpret_cast<const bf16_t*>(layers[l].pleT) + (size_t)tok * S::PLE;
#pragma unroll
                for (int q = 0; q < (S::PLE + 63) / 64; ++q) {
                    const int o = (sub + 8 * q) * 8;
                    if (S::PLE % 64 == 0 || o < S::PLE) {
                        float pw[8], tw[8];
                        Elem<bf16_t>::load_vec(Pm + o, pw);
                        Elem<bf16_t>::load_vec(Tb + o, tw);
#pragma unroll
                        for (int x = 0; x < 8; ++x) a = fmaf(pw[x], tw[x], a);
                    }
                }
            }
            a += __shfl_xor_sync(0xffffffffu, a, 1);
            a += __shfl_xor_sync(0xffffffffu, a, 2);
            a += __shfl_xor_sync(0xffffffffu, a, 4);
            if (sub == 0 && i < n) pacc[i] = a;
        }
        consumer_sync<kLeanWarps>();
    }
    // token embedding row (inference.cu:9-22): this CTA's rows, published like any other phase
    ++e;
    if (tid < RX) {
        float v = __bfloat162float(reinterpret_cast<const bf16_t*>(p.E)[(size_t)tok * D + xr0 + tid]);
        if (S::PLE > 0) v += pacc[tid];
        ll_store(p.x + (size_t)rank * lean_slot(RX) + tid, v, e);
    }
    mark(1);
    int xi = 0, ri = 0;
    uint32_t e_x = e;
#pragma unroll 1
    for (int li = 0; li < p.n_layers; ++li) {
        const StepLayer& L = layers[li];
        const bool attn = L.type == 0;
        // ---- QKV (or delta-net) projections of the normalised residual stream ----
        uint32_t e_proj;
        {
            float* xs = xsb[xi]; xi ^= 1;
            float* red = redb[ri]; ri ^= 1;
            float ss = lean_gather<D, RX, true, true>(p.x, e_x, L.g1, xa, xs, tid, dead, p.err);
            ss = warp_sum(ss);
            if (lane == 0) red[warp] = ss;
            consumer_sync<kLeanWarps>();
            mark(2);
            const float rn = lean_rnorm<D>(red, lane, p.eps);
            e_proj = ++e;
            if (attn) {
                const int r0 = min(rank * S::RQA, S::NQ_A), rows = min(S::RQA, S::NQ_A - r0);
                lean_rows<D, S::RQA, LM_STORE, false, S::H * S::HD + S::KVH * S::HD, S::HD>(
                    ring, rows, r0, xs, rn, p.pj + (size_t)rank * lean_slot(S::RQA), e_proj, nullptr, nullptr, nullptr, obuf, ocnt, warp, lane, bv, bi, tm,
                    p.rope + (size_t)pos * S::HD);
            } else {
                const int r0 = min(rank * S::RQD, S::NQ_D), rows = min(S::RQD, S::NQ_D - r0);
                lean_rows<D, S::RQD, LM_STORE, false>(ring, rows, r0, xs, rn, p.pj + (size_t)rank * lean_slot(S::RQD), e_proj,
                                                      nullptr, nullptr, nullptr, obuf, ocnt, warp, lane, bv, bi, tm);
            }
            mark(3);
        }
        // ---- mixer + output projection + residual ----
        {
            float* xs = xsb[xi]; xi ^= 1;
            if (attn) {
                const GridPlan& it = *plan;
                const uint32_t e_parts = ++e;
                if (it.has) {
                    lean_attention<S, KVT>(p, L, it, ring, mix, rank, pos, e_proj, e_parts, tid, dead, p.err, mark);
                    mark(5);
                }
                if (it.direct) {
                    lean_combine<S>(p, it.S, 0, S::H, e_parts, parts, xs, nullptr, 0, tid, dead, p.err);
                } else {
                    // many splits: the owner of a head combines it and publishes the result
                    ++e;
                    if (rank < S::H) lean_combine<S>(p, it.S, rank, 1, e_parts, parts, nullptr, p.ah + (size_t)rank * lean_slot(S::HD), e, tid, dead, p.err);
                    lean_gather<S::NA_A, S::HD, false, false>(p.ah, e, nullptr, nullptr, xs, tid, dead, p.err);
                }
            } else {
                const uint32_t e_a = ++e;
                lean_delta_net<S>(p, L, ring, mix, rank, e_proj, e_a, obuf, ocnt, tid, dead, p.err);
                mark(11);
                lean_gather<S::NA_D, S::RAD, false, false>(p.a, e_a, nullptr, nullptr, xs, tid, dead, p.err);
            }
            consumer_sync<kLeanWarps>();
            mark(8);
            ++e;
            lean_rows<S::NA_A, RX, LM_RESID, false>(ring, RX, xr0, xs, 1.0f, p.xb + (size_t)rank * lean_slot(RX), e, xa, nullptr, nullptr, obuf, ocnt, warp, lane, bv, bi, tm);
            mark(9);
        }
        // ---- FFN gate/up + SwiGLU ----
        {
            float* xs = xsb[xi]; xi ^= 1;
            float* red = redb[ri]; ri ^= 1;
            float ss = lean_gather<D, RX, true, true>(p.xb, e, L.g2, xb, xs, tid, dead, p.err);
            ss = warp_sum(ss);
            if (lane == 0) red[warp] = ss;
            consumer_sync<kLeanWarps>();
            mark(12);
            const float rn = lean_rnorm<D>(red, lane, p.eps);
            ++e;
            const int r0 = min(rank * S::RH, F), rows = min(S::RH, F - r0);
            lean_rows<D, S::RH, LM_SWIGLU, true>(ring, rows, r0, xs, rn, p.h + (size_t)rank * lean_slot(S::RH), e, nullptr, nullptr, nullptr, obuf, ocnt, warp, lane, bv, bi, tm);
            mark(13);
        }
        // ---- FFN down + residual (+ the next layer's per-layer embedding) ----
        {
            float* xs = xsb[xi]; xi ^= 1;
            lean_gather<F, S::RH, false, false>(p.h, e, nullptr, nullptr, xs, tid, dead, p.err);
            consumer_sync<kLeanWarps>();
            mark(14);
            ++e;
            lean_rows<F, RX, LM_RESID, false>(ring, RX, xr0, xs, 1.0f, p.x + (size_t)rank * lean_slot(RX), e, xb,
                                              (S::PLE > 0 && li + 1 < p.n_layers) ? pacc + (li + 1) * RX : nullptr, nullptr, obuf, ocnt, warp, lane, bv, bi, tm);
            e_x = e;
            mark(15);
        }
    }
    if (p.with_lm_head) {
        float* xs = xsb[xi];
        float* red = redb[ri];
        float ss = lean_gather<D, RX, true, false>(p.x, e_x, p.g_final, nullptr, xs, tid, dead, p.err);
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        consumer_sync<kLeanWarps>();
        mark(16);
        const float rn = lean_rnorm<D>(red, lane, p.eps);
        const int r0 = min(rank * S::RV, S::V), rows = min(S::RV, S::V - r0);
        lean_rows<D, S::RV, LM_LOGITS, false>(ring, rows, r0, xs, rn, nullptr, 0, nullptr, nullptr, p.logits, obuf, ocnt, warp, lane, bv, bi, tm);
        // reduce the warps' argmax picks (lane 0 of each warp holds them), then (in CTA 0) the grid's
        if (lane == 0) { mix[2 * warp] = bv; mix[2 * warp + 1] = __int_as_float(bi); }
        consumer_sync<kLeanWarps>();
        ++e;
        if (tid == 0) {
            for (int w = 1; w < kLeanWarps; ++w) {
                const float v = mix[2 * w];
                const int ix = __float_as_int(mix[2 * w + 1]);
                if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
            }
            mix[0] = bv;
            mix[1] = __int_as_float(bi);
        }
        __syncwarp();
        if (tid < 2) ll_store(p.lm + (size_t)rank * 16 + tid, mix[tid], e);      // one store instruction for the pair
        mark(17);
    }
    if (tm != nullptr && tid == 0) {
        tm[0] += clock64() - tstart;
        for (int i = 0; i < kGridTimerSlots; ++i) p.timers[(size_t)rank * kGridTimerSlots + i] += tm[i];
    }
    if (rank == 0) {
        if (p.with_lm_head) {
            lean_gather_rows<2>(p.lm, 0, 2 * S::C, e, parts, tid, dead, p.err);
            consumer_sync<kLeanWarps>();
            if (warp == 0 && p.do_pick) {
                // lowest index among the largest values (the host loop of inference_orchestrator.cu:77-84 keeps the first)
                float best = -INFINITY;
                int at = 0x7fffffff;
                for (int r = lane; r < S::C; r += 32) {
                    const float v = parts[2 * r];
                    const int ix = __float_as_int(parts[2 * r + 1]);
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
        if (tid == 0) *p.epoch = e;
        mark(31);
    }
}

}  // namespace mlb
