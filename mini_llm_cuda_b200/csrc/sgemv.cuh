// Streaming GEMV for one sequence per CTA row: y[row] = sum_k W[row][k] * x[k], with the weights
// fed by TMA bulk copies instead of per-thread loads.
//
// The per-thread-load GEMV of kernels.cuh keeps ~30 KB in flight per SM and pays its latency chain
// (activations -> weights -> reduction) once per CTA of 8-16 rows; on multi-MB matrices that caps it
// at a tenth of the HBM bandwidth. Here the matrix is cut into one contiguous slab of rows per CTA
// (about one CTA per SM). A producer warp streams the slab with cp.async.bulk into a ring of
// shared-memory stages guarded by mbarriers - and it starts BEFORE griddepcontrol.wait, because
// weights do not depend on the predecessor kernel - while 15 consumer warps stage and normalise
// the activation vector once, then take dot products out of shared memory two rows at a time.
// Epilogues are the ones of gemv_kernel (same reference citations): plain store, residual (+ the
// next layer's per-layer embedding), SwiGLU of a gate/up slab pair, QKV with per-head norm / RoPE /
// KV append (one head per CTA), LM head with argmax partials and last-CTA pick.
// grid = (slabs, B); every mbarrier wait is bounded (Ring::wait).
#pragma once
#include "ring.cuh"

namespace mlb {

struct SgemvGeom {
    int rows_per_cta;
    int n_stages, stage_bytes;
    int off_xs, off_xs2, off_outs, off_pacc, off_red, off_bar, off_ring;   // float offsets
    int* err;
};

constexpr int kSgWarps = 31;                       // consumer warps (+ 1 producer warp = 1024 threads, 64 registers each)
constexpr int kSgConsumers = kSgWarps * 32;
constexpr int kSgThreads = kSgConsumers + 32;

template <typename T, typename T2, typename KVT, int MODE>
__global__ void __launch_bounds__(kSgThreads, 1) sgemv_kernel(StepCtl c, GemvParams p, SgemvGeom g) {
    extern __shared__ __align__(128) float sg_smem[];
    float* smem = sg_smem;
    float* xs = smem + g.off_xs;
    float* xs2 = smem + g.off_xs2;
    float* outs = smem + g.off_outs;
    float* pacc = smem + g.off_pacc;
    float* red = smem + g.off_red;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.y;
    const int K = p.K, Kp = p.Kp, N = p.N;
    const int esz = (int)sizeof(T);
    const int r_begin = min(N, (int)blockIdx.x * g.rows_per_cta);
    const int r_end = min(N, r_begin + g.rows_per_cta);
    const int rows = r_end - r_begin;

    Ring ring;
    int* dead = reinterpret_cast<int*>(red + kSgWarps);
    ring.full0 = smem_u32(smem + g.off_bar);
    ring.empty0 = ring.full0 + 8u * g.n_stages;
    ring.stages = reinterpret_cast<unsigned char*>(smem + g.off_ring);
    ring.nst = g.n_stages;
    ring.stage_bytes = g.stage_bytes;
    ring.idx = 0;
    ring.phase = 0;
    ring.dead = dead;
    ring.err = g.err;
    ring.backoff_ns = 0;
    if (tid == 0) {
        *dead = 0;
        for (int i = 0; i < g.n_stages; ++i) {
            mbar_init(ring.full0 + 8u * i, 1);
            mbar_init(ring.empty0 + 8u * i, kSgWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kSgWarps) {
        // ---- producer: weights only, nothing here depends on the predecessor kernel ------------
        if (Kp > 0)
            issue_slab(ring, reinterpret_cast<const unsigned char*>(p.P) + (size_t)r_begin * Kp * sizeof(T2), rows,
                       Kp * (int)sizeof(T2), lane);
        if (MODE == GEMV_SWIGLU)
            issue_slab_pair(ring, reinterpret_cast<const unsigned char*>(p.W) + (size_t)r_begin * K * esz,
                            reinterpret_cast<const unsigned char*>(p.Wb) + (size_t)r_begin * K * esz, rows, K * esz, lane);
        else
            issue_slab(ring, reinterpret_cast<const unsigned char*>(p.W) + (size_t)r_begin * K * esz, rows, K * esz, lane);
        return;
    }

    // ---- consumers ------------------------------------------------------------------------------
    pdl_wait();
    const bool active = seq_active(c, b);
    const int bg = min(b, c.B - 1);
    // stage (and RMS-normalise) the activation vector: inference.cu:24-50, :83-95
    {
        const float* xr = p.xin + (size_t)bg * K;
        constexpr int EPV = Elem<T>::EPV;
        const int nvec = K / EPV;
        float ss = 0.f;
        for (int k = tid; k < K; k += kSgConsumers) {
            const float v = xr[k];
            xs[xs_index<EPV>(k, nvec)] = v;              // bank-conflict-free layout for the dot products
            ss = fmaf(v, v, ss);
        }
        if (Kp > 0) {
            const int t = c.tok[bg];
            const T2* trow = reinterpret_cast<const T2*>(p.Ptab) + (size_t)t * Kp;
            for (int k = tid; k < Kp; k += kSgConsumers) xs2[xs_index<Elem<T2>::EPV>(k, Kp / Elem<T2>::EPV)] = Elem<T2>::get(trow, k);
        }
        if (p.do_norm) {
            const float tot = consumer_sum<kSgWarps>(ss, red, warp, lane);
            const float r = sqrtf(tot / (float)K + p.eps);
            for (int k = tid; k < K; k += kSgConsumers) {
                const int d = xs_index<EPV>(k, nvec);
                xs[d] = (xs[d] / r) * p.gain[k];
            }
        }
        consumer_sync<kSgWarps>();
    }
    if (Kp > 0) {
        consume_slab<T2, kSgWarps, true>(ring, rows, Kp, xs2, warp, lane, [&](int r, float v) {
            if (lane == 0) pacc[r] = v;
        });
        consumer_sync<kSgWarps>();
    }

    if (MODE == GEMV_SWIGLU) {
        consume_slab_pair<T, kSgWarps, true>(ring, rows, K, xs, warp, lane, [&](int r, float gt, float up) {
            const int row = r_begin + r;
            if (p.wscale) { gt *= p.wscale[row]; up *= p.wscale_b[row]; }
            // applySiluToFFN + hadamardMultiplyFFN, inference.cu:262-281
            if (lane == 0 && active) p.y[(size_t)b * N + row] = (gt / (1.0f + expf(-gt))) * up;
        });
    } else if (MODE == GEMV_RAW || MODE == GEMV_RESID) {
        consume_slab<T, kSgWarps, true>(ring, rows, K, xs, warp, lane, [&](int r, float v) {
            const int row = r_begin + r;
            if (p.wscale) v *= p.wscale[row];
            if (Kp > 0) v += pacc[r];
            if (lane == 0 && active) {
                // addResidualToOutputProj / addResidualToFFN, inference.cu:252-260, :283-291
                if (MODE == GEMV_RESID) v += p.resid[(size_t)b * N + row];
                p.y[(size_t)b * N + row] = v;
            }
        });
    } else if (MODE == GEMV_QKV) {
        // a CTA owns whole heads' worth of rows (rows_per_cta == hd) when the per-head norm is on,
        // else a 32-row group inside one head
        consume_slab<T, kSgWarps, true>(ring, rows, K, xs, warp, lane, [&](int r, float v) {
            if (lane == 0) outs[r] = p.wscale ? v * p.wscale[r_begin + r] : v;
        });
        consumer_sync<kSgWarps>();
        const int hd = p.hd;
        const int seg_q = p.nq, seg_k = p.nq + p.nk, seg_v = seg_k + p.nv;
        const int seg = r_begin < seg_q ? 0 : (r_begin < seg_k ? 1 : (r_begin < seg_v ? 2 : 3));
        float rs = 1.f;
        if (p.qk_norm && seg < 2) {
            // getRMSColSumsAcrossHeads + applyRMSNormAcrossHeads, inference.cu:52-81, :97-111
            float ss = 0.f;
            for (int r = tid; r < rows; r += kSgConsumers) ss = fmaf(outs[r], outs[r], ss);
            rs = sqrtf(consumer_sum<kSgWarps>(ss, red, warp, lane) / (float)hd + p.eps);
        }
        if (active) {
            const int pos = c.pos[b];
            KVT* kpool = reinterpret_cast<KVT*>(p.kpool);
            KVT* vpool = reinterpret_cast<KVT*>(p.vpool);
            for (int pr = tid; pr < rows / 2; pr += kSgConsumers) {
                const int r = 2 * pr, row = r_begin + r;
                float a = outs[r], cc = outs[r + 1];
                if (seg < 2) {
                    const int srow = seg == 0 ? row : row - seg_q;
                    if (p.qk_norm) {
                        const float* gg = seg == 0 ? p.gq : p.gk;
                        a = (a / rs) * gg[srow];
                        cc = (cc / rs) * gg[srow + 1];
                    }
                    // applyRoPE, inference.cu:113-134
                    const int e = srow % hd;                       // position of the pair inside its head
                    const float cs = p.rope[(size_t)pos * hd + e], sn = p.rope[(size_t)pos * hd + e + 1];
                    const float ra = cs * a - sn * cc, rc = sn * a + cs * cc;
                    if (seg == 0) {
                        p.qbuf[(size_t)b * p.nq + srow] = ra;
                        p.qbuf[(size_t)b * p.nq + srow + 1] = rc;
                    } else {
                        const int kvh = srow / hd;
                        const int page = p.page_table[(size_t)b * p.pt_stride + pos / kKvBlock];
                        const size_t off = (((size_t)page * p.kv_heads + kvh) * kKvBlock + (pos % kKvBlock)) * hd + e;
                        Elem<KVT>::put(kpool, off, ra);
                        Elem<KVT>::put(kpool, off + 1, rc);
                    }
                } else if (seg == 2) {
                    const int srow = row - seg_k;
                    const int kvh = srow / hd, e = srow % hd;
                    const int page = p.page_table[(size_t)b * p.pt_stride + pos / kKvBlock];
                    const size_t off = (((size_t)page * p.kv_heads + kvh) * kKvBlock + (pos % kKvBlock)) * hd + e;
                    Elem<KVT>::put(vpool, off, a);
                    Elem<KVT>::put(vpool, off + 1, cc);
                } else {
                    const int srow = row - seg_v;
                    p.gbuf[(size_t)b * p.ng + srow] = 1.0f / (1.0f + expf(-a));        // inference.cu:248
                    p.gbuf[(size_t)b * p.ng + srow + 1] = 1.0f / (1.0f + expf(-cc));
                }
            }
        }
    } else {
        // LM head: logits, argmax partial of this CTA, pick by the last CTA of the sequence
        // (inference.cu:720-743; host qsort of inference_orchestrator.cu:77-84 replaced)
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        consume_slab<T, kSgWarps, true>(ring, rows, K, xs, warp, lane, [&](int r, float v) {
            const int row = r_begin + r;
            if (p.wscale) v *= p.wscale[row];
            if (lane == 0 && active) p.y[(size_t)b * N + row] = v;
            if (v > bv || (v == bv && row < bi)) { bv = v; bi = row; }
        });
        consumer_sync<kSgWarps>();
        if (lane == 0) { outs[2 * warp] = bv; outs[2 * warp + 1] = __int_as_float(bi); }
        consumer_sync<kSgWarps>();
        __shared__ int is_last;
        const int nparts = gridDim.x;
        if (tid == 0) {
            for (int w = 1; w < kSgWarps; ++w) {
                const float v = outs[2 * w];
                const int ix = __float_as_int(outs[2 * w + 1]);
                if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
            }
            p.part_val[(size_t)b * nparts + blockIdx.x] = bv;
            p.part_idx[(size_t)b * nparts + blockIdx.x] = bi;
            __threadfence();
            const int t = atomicAdd(&p.ticket[b], 1);
            is_last = (t == nparts - 1);
        }
        consumer_sync<kSgWarps>();
        if (is_last && warp == 0) {
            __threadfence();
            float v2 = -INFINITY;
            int i2 = 0x7fffffff;
            for (int q = lane; q < nparts; q += 32) {
                const float v = __ldcg(&p.part_val[(size_t)b * nparts + q]);
                const int ix = __ldcg(&p.part_idx[(size_t)b * nparts + q]);
                if (v > v2 || (v == v2 && ix < i2)) { v2 = v; i2 = ix; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, v2, o);
                const int oi = __shfl_xor_sync(0xffffffffu, i2, o);
                if (ov > v2 || (ov == v2 && oi < i2)) { v2 = ov; i2 = oi; }
            }
            if (lane == 0) {
                p.ticket[b] = 0;
                if (p.do_pick && active) advance_seq(c, b, i2);
            }
        }
    }
}

}  // namespace mlb
