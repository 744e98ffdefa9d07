// Small-batch decode step as ONE kernel: a thread-block cluster per sequence, weights fed by
// TMA bulk copies.
//
// At batch 1 the kernel chain is bound by ~40 kernel boundaries and by the few bytes each SM
// keeps in flight, not by bandwidth. Here the CTAs of one cluster (16 by default) own one
// sequence for the whole step:
//   * every phase (projection, attention, FFN ...) splits its output rows over the CTAs; a CTA's
//     rows are one contiguous slab of the row-major weight matrix;
//   * a producer warp streams those slabs with cp.async.bulk (TMA; every CTA loads only its own data) into a ring of
//     shared-memory stages guarded by mbarriers, running ahead of the consumers across phase
//     boundaries, so that ~100+ KB per SM are in flight without holding registers;
//   * 15 consumer warps compute dot products out of shared memory, two rows per read of the
//     activation vector, and push each result into the shared memory of ALL CTAs of the cluster
//     (distributed shared memory); a hardware cluster barrier separates the phases.
// Activations never leave the SMs between phases and a phase boundary costs a cluster barrier
// instead of a kernel launch. One cluster per GPC can run at a time, so a few sequences decode
// side by side on weights shared through L2.
//
// The arithmetic of every phase is the one of the chain kernels in kernels.cuh (same reference
// citations); only the partition of rows and of the attention context differs.
//
// Safety: control flow is uniform across the cluster, so every cluster barrier is reached by
// every thread. Every mbarrier wait is bounded; when one runs out the kernel records an error
// code, stops waiting (later waits return at once) and still walks to the end, so it always
// terminates and the host reports MLB_E_TIMEOUT.
#pragma once
#include "kernels.cuh"

namespace mlb {

struct MegaLayer {
    int type;
    int n_qkv, nq, nk, nv, ng, o_in;
    const void* Wqkv; const float* Sqkv;
    const float *g1, *g2, *gq, *gk;
    const void* Wo; const float* So;
    const void *W1a, *W1b, *W2;
    const float *S1a, *S1b, *S2;
    const void *pleT, *pleP;
    void *kpool, *vpool;
    float* state;
};
static_assert(sizeof(MegaLayer) % 8 == 0, "MegaLayer is copied in 8-byte words");

struct MegaParams {
    const MegaLayer* layers;
    int n_layers;
    int d, F, V, heads, kv_heads, hd, dk, dv, ple, qk_norm;
    float eps, l2_eps;
    const void* E; const float* Es; const float* g_final; const float* rope;
    const int* page_table; int pt_stride;
    float* logits;                 // [B][V]
    int* err;                      // device word: 0 = ok, else the code of the wait that ran out
    int with_lm_head;              // 0 in the prompt chain
    int do_pick;                   // greedy pick + advance inside the kernel
    // shared-memory layout (float offsets), identical in every CTA
    int off_x, off_xn, off_proj, off_parts, off_a, off_h, off_tmp, off_ple, off_pacc, off_red, off_lm;
    int off_bar;                   // mbarriers: full[nst] then empty[nst] (8 bytes each)
    int off_ring;                  // ring stages (128-byte aligned)
    int n_stages, stage_bytes;
    int attn_splits;               // context splits per kv head
};

constexpr int kMegaConsumers = 480;                 // consumer threads (15 warps + 1 producer warp = 16: 128 registers each)
constexpr int kMegaWarps = kMegaConsumers / 32;
constexpr int kMegaThreads = kMegaConsumers + 32;   // + one producer warp
constexpr int kMegaAttnWarps = 8;
constexpr uint32_t kMegaSpinLimit = 1u << 24;

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t a, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t a, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t a) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t a, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    return ok != 0;
}
// TMA bulk copy global -> this CTA's shared memory, completion counted on an mbarrier; single destination CTA.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t mbar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(mbar)
                 : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
template <int NW = kMegaConsumers / 32>
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory"); }
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// generic address of `p` (a shared-memory pointer of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ float* map_rank(float* p, uint32_t rank) {
    uint64_t in = (uint64_t)p, out;
    asm volatile("mapa.u64 %0, %1, %2;" : "=l"(out) : "l"(in), "r"(rank));
    return (float*)out;
}

// Wait for a phase of an mbarrier, at most `limit` polls: every wait of the kernels here ends, with
// the data or with `false`, so that a kernel always terminates and the host can report the failure.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit, unsigned backoff_ns) {
#pragma unroll 1
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (backoff_ns) __nanosleep(backoff_ns);
    }
    return false;
}

// ---- ring of shared-memory stages -------------------------------------------------------------
struct Ring {
    uint32_t full0, empty0;        // shared addresses of the barrier arrays
    unsigned char* stages;
    int nst, stage_bytes;
    int idx;
    uint32_t phase;
    volatile int* dead;            // shared flag: a wait ran out somewhere in this CTA
    int* err;
    long long wait_cycles;         // diagnostic: cycles spent in wait()
    unsigned backoff_ns;           // producer: pause between polls for a free stage (0: none)
    __device__ __forceinline__ void advance() {
        if (++idx == nst) { idx = 0; phase ^= 1u; }
    }
    __device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, int code) {
        if (*dead) return false;
#ifdef MLB_GRID_TIMERS
        const long long t0 = clock64();
#endif
        // code 1 = the producer waiting for a free stage: it runs stages ahead, so while the ring is full
        // it polls at leisure and leaves the issue slots and the shared-memory pipe to the consumers
        const bool ok = mbar_wait_bounded(bar, parity, kMegaSpinLimit, code == 1 ? backoff_ns : 0u);
#ifdef MLB_GRID_TIMERS
        wait_cycles += clock64() - t0;
#endif
        if (ok) return true;
        *dead = 1;
        atomicExch(err, code);
        return false;
    }
};

// Producer (lane 0 of the producer warp): stream `rows` rows of `row_bytes` starting at `src`.
__device__ __forceinline__ void issue_slab(Ring& r, const unsigned char* src, int rows, int row_bytes, int lane) {
    const int rpc = max(1, r.stage_bytes / row_bytes);
    for (int r0 = 0; r0 < rows; r0 += rpc) {
        const int n = min(rpc, rows - r0);
        if (lane == 0) {
            if (r.wait(r.empty0 + 8u * r.idx, r.phase ^ 1u, 1)) {
                const uint32_t bytes = (uint32_t)n * (uint32_t)row_bytes;
                mbar_expect_tx(r.full0 + 8u * r.idx, bytes);
                bulk_g2s(smem_u32(r.stages + (size_t)r.idx * r.stage_bytes), src + (size_t)r0 * row_bytes, bytes,
                         r.full0 + 8u * r.idx);
            }
        }
        r.advance();
    }
    __syncwarp();
}

// Two slabs with the same row geometry, chunk-interleaved (gate and up matrices of the FFN).
__device__ __forceinline__ void issue_slab_pair(Ring& r, const unsigned char* a, const unsigned char* b, int rows, int row_bytes,
                                                int lane) {
    const int rpc = max(1, r.stage_bytes / row_bytes);
    for (int r0 = 0; r0 < rows; r0 += rpc) {
        const int n = min(rpc, rows - r0);
        for (int which = 0; which < 2; ++which) {
            if (lane == 0) {
                if (r.wait(r.empty0 + 8u * r.idx, r.phase ^ 1u, 1)) {
                    const uint32_t bytes = (uint32_t)n * (uint32_t)row_bytes;
                    mbar_expect_tx(r.full0 + 8u * r.idx, bytes);
                    bulk_g2s(smem_u32(r.stages + (size_t)r.idx * r.stage_bytes), (which ? b : a) + (size_t)r0 * row_bytes, bytes,
                             r.full0 + 8u * r.idx);
                }
            }
            r.advance();
        }
    }
    __syncwarp();
}

// ---- consumer side ------------------------------------------------------------------------------
// Two rows at a time against the activation vector in shared memory: one read of x serves both
// rows, so shared-memory traffic is 2 bytes per weight byte (fp32 x, bf16 weights) instead of 3.
template <typename T, bool PERM = false>
__device__ __forceinline__ void smem_rows_dot2(const T* row0, const T* row1, int nvec, const float* xs, int lane, float& a0,
                                               float& a1) {
    // PERM: xs is stored as [EPV/4][nvec] float4s (xs_f4_index), else linearly
    constexpr int EPV = Elem<T>::EPV;
    a0 = 0.f;
    a1 = 0.f;
#pragma unroll 2
    for (int vi = lane; vi < nvec; vi += 32) {
        float w0[EPV], w1[EPV];
        Elem<T>::unpack(*reinterpret_cast<const uint4*>(row0 + (size_t)vi * EPV), w0);
        Elem<T>::unpack(*reinterpret_cast<const uint4*>(row1 + (size_t)vi * EPV), w1);
        const float4* xp = reinterpret_cast<const float4*>(xs);
#pragma unroll
        for (int q = 0; q < EPV / 4; ++q) {
            const float4 t = PERM ? xp[q * nvec + vi] : xp[vi * (EPV / 4) + q];
            a0 = fmaf(w0[4 * q], t.x, a0); a0 = fmaf(w0[4 * q + 1], t.y, a0);
            a0 = fmaf(w0[4 * q + 2], t.z, a0); a0 = fmaf(w0[4 * q + 3], t.w, a0);
            a1 = fmaf(w1[4 * q], t.x, a1); a1 = fmaf(w1[4 * q + 1], t.y, a1);
            a1 = fmaf(w1[4 * q + 2], t.z, a1); a1 = fmaf(w1[4 * q + 3], t.w, a1);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a0 += __shfl_xor_sync(0xffffffffu, a0, o);
        a1 += __shfl_xor_sync(0xffffffffu, a1, o);
    }
}

// Consume a slab of `rows` rows of K elements: f(local_row, dot) runs in every lane of the warp
// that owns the row, with the full dot product.
template <typename T, int NW = kMegaWarps, bool PERM = false, typename F>
__device__ __forceinline__ void consume_slab(Ring& r, int rows, int K, const float* xs, int warp, int lane, F&& f) {
    const int nvec = K / Elem<T>::EPV;
    const int row_bytes = K * (int)sizeof(T);
    const int rpc = max(1, r.stage_bytes / row_bytes);
    for (int r0 = 0; r0 < rows; r0 += rpc) {
        const int n = min(rpc, rows - r0);
        r.wait(r.full0 + 8u * r.idx, r.phase, 2);
        const T* base = reinterpret_cast<const T*>(r.stages + (size_t)r.idx * r.stage_bytes);
        if (n >= 2 * NW) {
            for (int i = 2 * warp; i < n; i += 2 * NW) {
                const bool two = i + 1 < n;
                float a0, a1;
                smem_rows_dot2<T, PERM>(base + (size_t)i * K, base + (size_t)(two ? i + 1 : i) * K, nvec, xs, lane, a0, a1);
                f(r0 + i, a0);
                if (two) f(r0 + i + 1, a1);
            }
        } else {
            // few long rows in the chunk: one row per warp keeps more warps busy
            for (int i = warp; i < n; i += NW) {
                float a0, a1;
                smem_rows_dot2<T, PERM>(base + (size_t)i * K, base + (size_t)i * K, nvec, xs, lane, a0, a1);
                f(r0 + i, a0);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(r.empty0 + 8u * r.idx);
        r.advance();
    }
}

// Chunk-interleaved pair of slabs: f(local_row, dot_a, dot_b).
template <typename T, int NW = kMegaWarps, bool PERM = false, typename F>
__device__ __forceinline__ void consume_slab_pair(Ring& r, int rows, int K, const float* xs, int warp, int lane, F&& f) {
    const int nvec = K / Elem<T>::EPV;
    const int row_bytes = K * (int)sizeof(T);
    const int rpc = max(1, r.stage_bytes / row_bytes);
    for (int r0 = 0; r0 < rows; r0 += rpc) {
        const int n = min(rpc, rows - r0);
        const int ia = r.idx;
        r.wait(r.full0 + 8u * r.idx, r.phase, 2);
        r.advance();
        const int ib = r.idx;
        r.wait(r.full0 + 8u * r.idx, r.phase, 2);
        r.advance();
        const T* A = reinterpret_cast<const T*>(r.stages + (size_t)ia * r.stage_bytes);
        const T* Bm = reinterpret_cast<const T*>(r.stages + (size_t)ib * r.stage_bytes);
        for (int i = warp; i < n; i += NW) {
            float a0, a1;
            smem_rows_dot2<T, PERM>(A + (size_t)i * K, Bm + (size_t)i * K, nvec, xs, lane, a0, a1);
            f(r0 + i, a0, a1);
        }
        __syncwarp();
        if (lane == 0) { mbar_arrive(r.empty0 + 8u * ia); mbar_arrive(r.empty0 + 8u * ib); }
    }
}

// Sum over the consumer threads; every consumer gets the total. `red` holds kMegaWarps floats.
template <int NW = kMegaWarps>
__device__ __forceinline__ float consumer_sum(float v, float* red, int warp, int lane) {
    v = warp_sum(v);
    consumer_sync<NW>();                   // red may still be read from a previous use
    if (lane == 0) red[warp] = v;
    consumer_sync<NW>();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) t += red[w];
    return t;
}

// dst[k] = (src[k] / sqrt(mean(src^2)+eps)) * gain[k]   (inference.cu:24-50, :83-95)
__device__ __forceinline__ void rms_norm_local(const float* src, float* dst, const float* __restrict__ gain, int n, float eps,
                                               float* red, int tid, int warp, int lane) {
    float ss = 0.f;
    for (int k = tid; k < n; k += kMegaConsumers) ss = fmaf(src[k], src[k], ss);
    const float tot = consumer_sum(ss, red, warp, lane);
    const float r = sqrtf(tot / (float)n + eps);
    for (int k = tid; k < n; k += kMegaConsumers) dst[k] = (src[k] / r) * gain[k];
    consumer_sync();
}

struct MegaCtx {
    int C, rank, b, tok, pos, tid, lane, warp;
    float* smem;
    Ring ring;
};

// Phase barrier of the cluster. Consumers arrive and wait. The producer warp arrives as soon as
// it has issued the phase's copies and waits for that barrier only before it arrives at the next
// one: it runs one phase ahead and never blocks the consumers.
template <bool PRODUCER>
__device__ __forceinline__ void phase_barrier(bool& producer_pending) {
    __syncwarp();
    if (PRODUCER) {
        if (producer_pending) cluster_wait();
        cluster_arrive();
        producer_pending = true;
    } else {
        cluster_arrive();
        cluster_wait();
    }
}

// The one walk over the step that BOTH roles execute: the producer issues the weight slabs in
// exactly the order in which the consumers wait for them, and both meet the same barriers.
template <typename T, typename T2, typename KVT, bool PRODUCER>
__device__ __forceinline__ void mega_walk(const StepCtl& c, const MegaParams& p, MegaCtx& k) {
    const int C = k.C, rank = k.rank, b = k.b, tok = k.tok, pos = k.pos;
    const int tid = k.tid, lane = k.lane, warp = k.warp;
    float* smem = k.smem;
    float* x = smem + p.off_x;          // residual stream, replicated in every CTA
    float* xn = smem + p.off_xn;        // normalised input of the current projection (local)
    float* proj = smem + p.off_proj;    // q | . | . | gate   or the raw delta-net projections
    float* parts = smem + p.off_parts;  // flash-decode partials [heads][S][hd+2]
    float* abuf = smem + p.off_a;       // attention / delta-net output
    float* hbuf = smem + p.off_h;       // FFN hidden
    float* tmp = smem + p.off_tmp;      // one head of raw projection outputs; merge areas
    float* plerow = smem + p.off_ple;   // per-layer-embedding table row of the pending token
    float* pacc = smem + p.off_pacc;    // per-layer-embedding contribution to this CTA's rows of x
    float* red = smem + p.off_red;
    float* lmpart = smem + p.off_lm;    // [C][2] argmax partials (used in CTA 0)
    Ring& ring = k.ring;
    // lane r of a consumer warp addresses the shared memory of CTA r of the cluster
    float* rsm = map_rank(smem, lane < C ? lane : 0);
    const bool pusher = lane < C;
    const int d = p.d, F = p.F, hd = p.hd;
    const int esz = (int)sizeof(T);
    bool producer_pending = false;

    for (int li = 0; li < p.n_layers; ++li) {
        const MegaLayer& L = p.layers[li];
        if (!PRODUCER) rms_norm_local(x, xn, L.g1, d, p.eps, red, tid, warp, lane);
        const unsigned char* Wqkv = reinterpret_cast<const unsigned char*>(L.Wqkv);

        if (L.type == MLB_LAYER_ATTENTION) {
            // ---- phase 1: q | k | v | gate, one head (hd rows) per task --------------------------
            const int n_tasks = L.n_qkv / hd;
            const int seg_q = L.nq, seg_k = L.nq + L.nk, seg_v = seg_k + L.nv;
            KVT* kpool = reinterpret_cast<KVT*>(L.kpool);
            KVT* vpool = reinterpret_cast<KVT*>(L.vpool);
            for (int t = rank; t < n_tasks; t += C) {
                const int row0 = t * hd;
                if (PRODUCER) {
                    issue_slab(ring, Wqkv + (size_t)row0 * d * esz, hd, d * esz, lane);
                    continue;
                }
                consume_slab<T>(ring, hd, d, xn, warp, lane, [&](int r, float v) {
                    if (lane == 0) tmp[r] = L.Sqkv ? v * L.Sqkv[row0 + r] : v;
                });
                consumer_sync();
                const int page = p.page_table[(size_t)b * p.pt_stride + pos / kKvBlock];
                const int seg = row0 < seg_q ? 0 : (row0 < seg_k ? 1 : (row0 < seg_v ? 2 : 3));
                float rs = 1.f;
                if (p.qk_norm && seg < 2) {
                    // per-head RMS norm (inference.cu:52-81, :97-111)
                    float ss = 0.f;
                    for (int r = tid; r < hd; r += kMegaConsumers) ss = fmaf(tmp[r], tmp[r], ss);
                    rs = sqrtf(consumer_sum(ss, red, warp, lane) / (float)hd + p.eps);
                }
                // thread pr finishes pair pr of the head and pushes it to every CTA of the cluster
                for (int pr = tid; pr < hd / 2; pr += kMegaConsumers) {
                    const int r = 2 * pr;
                    float a = tmp[r], cc = tmp[r + 1];
                    const int row = row0 + r;
                    if (seg < 2) {
                        const int srow = seg == 0 ? row : row - seg_q;
                        if (p.qk_norm) {
                            const float* g = seg == 0 ? L.gq : L.gk;
                            a = (a / rs) * g[srow];
                            cc = (cc / rs) * g[srow + 1];
                        }
                        // RoPE on the adjacent pair (inference.cu:113-134)
                        const float cs = p.rope[(size_t)pos * hd + r], sn = p.rope[(size_t)pos * hd + r + 1];
                        const float ra = cs * a - sn * cc, rc = sn * a + cs * cc;
                        if (seg == 0) {
                            for (int rr = 0; rr < C; ++rr) {
                                float* dst = map_rank(smem, rr) + p.off_proj + row;
                                dst[0] = ra;
                                dst[1] = rc;
                            }
                        } else {
                            const int kvh = srow / hd;
                            const size_t off = (((size_t)page * p.kv_heads + kvh) * kKvBlock + (pos % kKvBlock)) * hd + r;
                            Elem<KVT>::put(kpool, off, ra);
                            Elem<KVT>::put(kpool, off + 1, rc);
                        }
                    } else if (seg == 2) {
                        const int srow = row - seg_k;
                        const int kvh = srow / hd;
                        const size_t off = (((size_t)page * p.kv_heads + kvh) * kKvBlock + (pos % kKvBlock)) * hd + r;
                        Elem<KVT>::put(vpool, off, a);
                        Elem<KVT>::put(vpool, off + 1, cc);
                    } else {
                        // sigmoid of the gate projection (inference.cu:248); stored after q|k|v
                        const float ga = 1.0f / (1.0f + expf(-a)), gc = 1.0f / (1.0f + expf(-cc));
                        for (int rr = 0; rr < C; ++rr) {
                            float* dst = map_rank(smem, rr) + p.off_proj + row;
                            dst[0] = ga;
                            dst[1] = gc;
                        }
                    }
                }
                consumer_sync();
            }
            if (!PRODUCER) __threadfence();      // this step's K/V row is read from global memory by other CTAs
            phase_barrier<PRODUCER>(producer_pending);

            // ---- phase 2: flash-decode, (kv head, context split) items over the CTAs (no weights) --
            if (!PRODUCER) {
                const int S = p.attn_splits;
                const int G = p.heads / p.kv_heads;
                const int n_items = p.kv_heads * S;
                const int ctx = pos + 1;
                const int npages = (ctx + kKvBlock - 1) / kKvBlock;
                const int pps = (npages + S - 1) / S;
                constexpr int EPL = 16 / (int)sizeof(KVT);
                const int LPR = hd / EPL, PPI = 32 / LPR;
                const int lr = lane % LPR, grp = lane / LPR;
                const float div = sqrtf((float)hd);
                for (int it = rank; it < n_items; it += C) {
                    const int kvh = it / S, split = it - kvh * S;
                    const int pg_begin = split * pps, pg_end = min(npages, pg_begin + pps);
                    for (int g = 0; g < G; ++g) {
                        const int h = kvh * G + g;
                        float q[8], acc[8], m = kNegBig, l = 0.f;
#pragma unroll
                        for (int e = 0; e < 8; ++e) { q[e] = e < EPL ? proj[h * hd + lr * EPL + e] : 0.f; acc[e] = 0.f; }
                        if (warp < kMegaAttnWarps) {
                            for (int pg = pg_begin + warp; pg < pg_end; pg += kMegaAttnWarps) {
                                const int pgi = p.page_table[(size_t)b * p.pt_stride + pg];
                                const int cnt = min(kKvBlock, ctx - pg * kKvBlock);
                                const size_t base = ((size_t)pgi * p.kv_heads + kvh) * kKvBlock * hd;
                                for (int j0 = 0; j0 < kKvBlock; j0 += PPI) {
                                    const int j = j0 + grp;
                                    const bool valid = j < cnt;
                                    float kv[8], vv[8];
#pragma unroll
                                    for (int e = 0; e < 8; ++e) { kv[e] = 0.f; vv[e] = 0.f; }
                                    if (valid) {
                                        Elem<KVT>::load_vec_cg(kpool + base + (size_t)j * hd + lr * EPL, kv);
                                        Elem<KVT>::load_vec_cg(vpool + base + (size_t)j * hd + lr * EPL, vv);
                                    }
                                    float s = 0.f;
#pragma unroll
                                    for (int e = 0; e < 8; ++e) s = fmaf(q[e], kv[e], s);
                                    for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                                    s = s / div;                      // inference.cu:154
                                    if (valid) {
                                        const float mn = fmaxf(m, s);
                                        const float sc = expf(m - mn), pe = expf(s - mn);
                                        l = l * sc + pe;
#pragma unroll
                                        for (int e = 0; e < 8; ++e) acc[e] = acc[e] * sc + pe * vv[e];
                                        m = mn;
                                    }
                                }
                            }
                            // merge the position groups of the warp
                            for (int o = LPR; o < 32; o <<= 1) {
                                const float mo = __shfl_xor_sync(0xffffffffu, m, o);
                                const float lo = __shfl_xor_sync(0xffffffffu, l, o);
                                const float mn = fmaxf(m, mo);
                                const float sa = expf(m - mn), sb = expf(mo - mn);
                                l = l * sa + lo * sb;
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    const float ao = __shfl_xor_sync(0xffffffffu, acc[e], o);
                                    acc[e] = acc[e] * sa + ao * sb;
                                }
                                m = mn;
                            }
                            if (grp == 0) {
                                float* w = tmp + (size_t)warp * (hd + 2);
                                for (int e = 0; e < EPL; ++e) w[lr * EPL + e] = acc[e];
                                if (lr == 0) { w[hd] = m; w[hd + 1] = l; }
                            }
                        }
                        consumer_sync();
                        // merge the warps; thread e owns one element of the item's partial and pushes it
                        for (int e = tid; e < hd + 2; e += kMegaConsumers) {
                            float mn = kNegBig;
                            for (int w = 0; w < kMegaAttnWarps; ++w) mn = fmaxf(mn, tmp[(size_t)w * (hd + 2) + hd]);
                            float val;
                            if (e == hd) {
                                val = mn;
                            } else {
                                val = 0.f;
                                for (int w = 0; w < kMegaAttnWarps; ++w)
                                    val += tmp[(size_t)w * (hd + 2) + e] * expf(tmp[(size_t)w * (hd + 2) + hd] - mn);
                            }
                            const size_t off = (size_t)p.off_parts + ((size_t)h * S + split) * (hd + 2) + e;
                            for (int rr = 0; rr < C; ++rr) map_rank(smem, rr)[off] = val;
                        }
                        consumer_sync();
                    }
                }
            }
            phase_barrier<PRODUCER>(producer_pending);
            if (!PRODUCER) {
                // combine the splits of every head locally (+ query gating, inference.cu:241-250)
                const int S = p.attn_splits;
                const float* gate = L.ng ? proj + seg_v : nullptr;
                for (int i = tid; i < p.heads * hd; i += kMegaConsumers) {
                    const int h = i / hd, e = i - h * hd;
                    const float* pp = parts + (size_t)h * S * (hd + 2);
                    float mn = kNegBig;
                    for (int s = 0; s < S; ++s) mn = fmaxf(mn, pp[(size_t)s * (hd + 2) + hd]);
                    float lt = 0.f, at = 0.f;
                    for (int s = 0; s < S; ++s) {
                        const float sc = expf(pp[(size_t)s * (hd + 2) + hd] - mn);
                        lt += pp[(size_t)s * (hd + 2) + hd + 1] * sc;
                        at += pp[(size_t)s * (hd + 2) + e] * sc;
                    }
                    float o = at / lt;
                    if (gate) o *= gate[i];
                    abuf[i] = o;
                }
                consumer_sync();
            }
        } else {
            // ---- gated delta-net: raw projections, then the state update row by row ----------------
            {
                const int N = L.n_qkv;
                const int rpc = (N + C - 1) / C;
                const int r_begin = min(N, rank * rpc), r_end = min(N, (rank + 1) * rpc);
                if (PRODUCER) {
                    issue_slab(ring, Wqkv + (size_t)r_begin * d * esz, r_end - r_begin, d * esz, lane);
                } else {
                    consume_slab<T>(ring, r_end - r_begin, d, xn, warp, lane, [&](int r, float v) {
                        const int row = r_begin + r;
                        if (pusher) rsm[p.off_proj + row] = L.Sqkv ? v * L.Sqkv[row] : v;
                    });
                }
            }
            phase_barrier<PRODUCER>(producer_pending);
            if (!PRODUCER) {
                const int H = p.heads, dk = p.dk, dv = p.dv;
                // L2-normalised q, k of every head and the two gates, locally (tmp: [2][H*dk] + [2H])
                float* qn = tmp;
                float* kn = tmp + H * dk;
                float* gates = tmp + 2 * H * dk;
                for (int hh = warp; hh < 2 * H; hh += kMegaWarps) {
                    const float* src = proj + (size_t)hh * dk;          // q heads then k heads
                    float ss = 0.f;
                    for (int e = lane; e < dk; e += 32) ss = fmaf(src[e], src[e], ss);
                    ss = warp_sum(ss);
                    const float n = sqrtf(ss + p.l2_eps);
                    for (int e = lane; e < dk; e += 32) tmp[(size_t)hh * dk + e] = src[e] / n;
                }
                for (int i = tid; i < 2 * H; i += kMegaConsumers)
                    gates[i] = 1.0f / (1.0f + expf(-proj[2 * H * dk + H * dv + i]));      // beta[H] then alpha[H]
                consumer_sync();
                const int rows = H * dv;
                const int rpc = (rows + C - 1) / C;
                const int r_begin = min(rows, rank * rpc), r_end = min(rows, (rank + 1) * rpc);
                float* state = L.state + (size_t)b * H * dv * dk;
                const float* rv = proj + 2 * H * dk;
                for (int row = r_begin + warp; row < r_end; row += kMegaWarps) {
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
                    if (pusher) rsm[p.off_a + row] = d2;
                }
            }
            phase_barrier<PRODUCER>(producer_pending);
        }

        // ---- output projection + residual (inference.cu:581-610) ---------------------------------
        {
            const int rpc = (d + C - 1) / C;
            const int r_begin = min(d, rank * rpc), r_end = min(d, (rank + 1) * rpc);
            if (PRODUCER) {
                issue_slab(ring, reinterpret_cast<const unsigned char*>(L.Wo) + (size_t)r_begin * L.o_in * esz, r_end - r_begin,
                           L.o_in * esz, lane);
            } else {
                consume_slab<T>(ring, r_end - r_begin, L.o_in, abuf, warp, lane, [&](int r, float v) {
                    const int row = r_begin + r;
                    if (L.So) v *= L.So[row];
                    if (pusher) rsm[p.off_x + row] = v + x[row];
                });
            }
        }
        phase_barrier<PRODUCER>(producer_pending);
        // ---- FFN gate/up + SwiGLU (inference.cu:612-672) ------------------------------------------
        if (!PRODUCER) rms_norm_local(x, xn, L.g2, d, p.eps, red, tid, warp, lane);
        {
            const int rpc = (F + C - 1) / C;
            const int r_begin = min(F, rank * rpc), r_end = min(F, (rank + 1) * rpc);
            if (PRODUCER) {
                issue_slab_pair(ring, reinterpret_cast<const unsigned char*>(L.W1a) + (size_t)r_begin * d * esz,
                                reinterpret_cast<const unsigned char*>(L.W1b) + (size_t)r_begin * d * esz, r_end - r_begin, d * esz,
                                lane);
            } else {
                consume_slab_pair<T>(ring, r_end - r_begin, d, xn, warp, lane, [&](int r, float g, float u) {
                    const int row = r_begin + r;
                    if (L.S1a) { g *= L.S1a[row]; u *= L.S1b[row]; }
                    // applySiluToFFN + hadamardMultiplyFFN, inference.cu:262-281
                    if (pusher) rsm[p.off_h + row] = (g / (1.0f + expf(-g))) * u;
                });
            }
        }
        phase_barrier<PRODUCER>(producer_pending);
        // ---- FFN down + residual + the next layer's per-layer embedding ------------------------
        {
            const bool ple_next = p.ple > 0 && li + 1 < p.n_layers;
            const int rpc = (d + C - 1) / C;
            const int r_begin = min(d, rank * rpc), r_end = min(d, (rank + 1) * rpc);
            if (ple_next) {
                const int psz = (int)sizeof(T2);
                if (PRODUCER) {
                    issue_slab(ring, reinterpret_cast<const unsigned char*>(p.layers[li + 1].pleP) + (size_t)r_begin * p.ple * psz,
                               r_end - r_begin, p.ple * psz, lane);
                } else {
                    const T2* Tn = reinterpret_cast<const T2*>(p.layers[li + 1].pleT);
                    for (int j = tid; j < p.ple; j += kMegaConsumers) plerow[j] = Elem<T2>::get(Tn, (size_t)tok * p.ple + j);
                    consumer_sync();
                    consume_slab<T2>(ring, r_end - r_begin, p.ple, plerow, warp, lane, [&](int r, float v) {
                        if (lane == 0) pacc[r] = v;
                    });
                    consumer_sync();      // the rows of the two slabs map to warps differently
                }
            }
            if (PRODUCER) {
                issue_slab(ring, reinterpret_cast<const unsigned char*>(L.W2) + (size_t)r_begin * F * esz, r_end - r_begin, F * esz,
                           lane);
            } else {
                consume_slab<T>(ring, r_end - r_begin, F, hbuf, warp, lane, [&](int r, float v) {
                    const int row = r_begin + r;
                    if (L.S2) v *= L.S2[row];
                    if (ple_next) v += pacc[r];
                    if (pusher) rsm[p.off_x + row] = v + x[row];
                });
            }
        }
        phase_barrier<PRODUCER>(producer_pending);
    }

    if (p.with_lm_head) {
        // ---- final norm, tied LM head, argmax (inference.cu:705-743; the host qsort of
        //      inference_orchestrator.cu:77-84 is replaced by an on-device pick) -----------------
        if (!PRODUCER) rms_norm_local(x, xn, p.g_final, d, p.eps, red, tid, warp, lane);
        const int V = p.V;
        const int rpc = (V + C - 1) / C;
        const int r_begin = min(V, rank * rpc), r_end = min(V, (rank + 1) * rpc);
        if (PRODUCER) {
            issue_slab(ring, reinterpret_cast<const unsigned char*>(p.E) + (size_t)r_begin * d * esz, r_end - r_begin, d * esz, lane);
        } else {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            float* lg = p.logits + (size_t)b * V;
            consume_slab<T>(ring, r_end - r_begin, d, xn, warp, lane, [&](int r, float v) {
                const int row = r_begin + r;
                if (p.Es) v *= p.Es[row];
                if (lane == 0) lg[row] = v;
                if (v > bv || (v == bv && row < bi)) { bv = v; bi = row; }
            });
            // every lane of a warp holds the same (bv, bi); reduce over the warps
            consumer_sync();
            if (lane == 0) { tmp[2 * warp] = bv; tmp[2 * warp + 1] = __int_as_float(bi); }
            consumer_sync();
            if (tid == 0) {
                for (int w = 1; w < kMegaWarps; ++w) {
                    const float v = tmp[2 * w];
                    const int ix = __float_as_int(tmp[2 * w + 1]);
                    if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
                }
                float* dst = map_rank(smem, 0) + p.off_lm + 2 * rank;
                dst[0] = bv;
                dst[1] = __int_as_float(bi);
            }
        }
        phase_barrier<PRODUCER>(producer_pending);
    }
    if (PRODUCER) {
        if (producer_pending) cluster_wait();        // the barrier this warp arrived at last
        return;
    }
    if (rank == 0 && tid == 0) {
        if (!p.with_lm_head) {
            advance_seq(c, b, -1);
        } else if (p.do_pick) {
            float bv = lmpart[0];
            int bi = __float_as_int(lmpart[1]);
            for (int r = 1; r < C; ++r) {
                const float v = lmpart[2 * r];
                const int ix = __float_as_int(lmpart[2 * r + 1]);
                if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
            }
            advance_seq(c, b, bi);
        }
    }
}

template <typename T, typename T2, typename KVT>
__global__ void __launch_bounds__(kMegaThreads, 1) mega_decode_kernel(StepCtl c, MegaParams p) {
    const int b = blockIdx.y;
    if (!seq_active(c, b)) return;                    // the whole cluster serves sequence b: uniform
    extern __shared__ __align__(128) float mega_smem[];
    float* smem = mega_smem;
    MegaCtx k;
    k.C = (int)cluster_nctarank();
    k.rank = (int)cluster_ctarank();
    k.b = b;
    k.tid = threadIdx.x;
    k.lane = threadIdx.x & 31;
    k.warp = threadIdx.x >> 5;
    k.smem = smem;
    k.tok = c.tok[b];
    k.pos = c.pos[b];
    int* dead = reinterpret_cast<int*>(smem + p.off_red + kMegaWarps);
    k.ring.full0 = smem_u32(smem + p.off_bar);
    k.ring.empty0 = k.ring.full0 + 8u * p.n_stages;
    k.ring.stages = reinterpret_cast<unsigned char*>(smem + p.off_ring);
    k.ring.nst = p.n_stages;
    k.ring.stage_bytes = p.stage_bytes;
    k.ring.idx = 0;
    k.ring.phase = 0;
    k.ring.dead = dead;
    k.ring.err = p.err;
    k.ring.wait_cycles = 0;
    k.ring.backoff_ns = 0;
    if (threadIdx.x == 0) {
        *dead = 0;
        for (int i = 0; i < p.n_stages; ++i) {
            mbar_init(k.ring.full0 + 8u * i, 1);                    // the producer's expect_tx arrival
            mbar_init(k.ring.empty0 + 8u * i, kMegaWarps);          // one arrival per consumer warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const bool producer = k.warp == kMegaWarps;
    if (!producer) {
        // ---- token embedding + first layer's PLE, redundantly in every CTA (inference.cu:9-22) ----
        float* x = smem + p.off_x;
        float* plerow = smem + p.off_ple;
        const T* E = reinterpret_cast<const T*>(p.E);
        const int d = p.d, tok = k.tok, tid = k.tid;
        const float sc = p.Es ? p.Es[tok] : 1.0f;
        for (int i = tid; i < d; i += kMegaConsumers) x[i] = Elem<T>::get(E, (size_t)tok * d + i) * sc;
        if (p.ple > 0) {
            const T2* T0 = reinterpret_cast<const T2*>(p.layers[0].pleT);
            const T2* P0 = reinterpret_cast<const T2*>(p.layers[0].pleP);
            for (int j = tid; j < p.ple; j += kMegaConsumers) plerow[j] = Elem<T2>::get(T0, (size_t)tok * p.ple + j);
            consumer_sync();
            constexpr int EPV2 = Elem<T2>::EPV;
            for (int i = tid; i < d; i += kMegaConsumers) {
                float a = 0.f;
                const T2* prow = P0 + (size_t)i * p.ple;
                for (int j = 0; j < p.ple; j += EPV2) {
                    float w[EPV2];
                    Elem<T2>::load_vec(prow + j, w);
#pragma unroll
                    for (int e = 0; e < EPV2; ++e) a = fmaf(w[e], plerow[j + e], a);
                }
                x[i] += a;
            }
        }
    }
    // Every CTA of the cluster is running before any remote shared memory is written.
    cluster_arrive();
    cluster_wait();
    if (producer) mega_walk<T, T2, KVT, true>(c, p, k);
    else mega_walk<T, T2, KVT, false>(c, p, k);
}

}  // namespace mlb
