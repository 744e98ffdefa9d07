// Batched projections on the 5th-generation tensor cores: Y[b][n] = sum_k W[n][k] * X[b][k] for
// bf16 weights and bf16 activations with fp32 accumulation in tensor memory.
//
// Once the batch is large the decode step's projections are dense contractions. The operands
// are swapped so that the weight rows fill the MMA's M = 128 and the batch is the MMA's N
// (16..256): a CTA owns 128 output features for a tile of up to 256 sequences.
//   * one thread feeds a ring of shared-memory stages with TMA tensor loads (128-byte swizzle,
//     one destination CTA): a [128 x 64] weight tile (two for gate/up) and the [Nb x 64] activation tile;
//   * one thread issues tcgen05.mma (kind::f16, M128 x N=Nb x K16, four per stage) into TMEM and
//     tcgen05.commit's the stage back to the loader;
//   * all four warps read the accumulator with tcgen05.ld (warp w owns TMEM lanes 32w..32w+31 =
//     output features) and run the epilogue: plain store, residual add in place, or SwiGLU of
//     the two accumulators written as the bf16 input of the down projection.
// Reference ops replaced: the cublasGemmEx calls of inference.cu:401-465, :581-602, :623-695,
// :720-743 and the element-wise kernels fused behind them (inference.cu:252-291).
// Every mbarrier wait is bounded; a wait that runs out records an error code, the kernel still
// frees its tensor memory and returns.
#pragma once
#include <cuda.h>

#include "ring.cuh"   // mbarrier / TMA wrappers

namespace mlb {

constexpr int kTcM = 128;          // output features per CTA (UMMA M)
constexpr int kTcKB = 64;          // bf16 elements per k-block = one 128-byte swizzle row
constexpr uint32_t kTcSpin = 1u << 22;

enum GemmTcMode : int { TC_RAW = 0, TC_RESID = 1, TC_SWIGLU = 2 };

struct GemmTcParams {
    int N, K, B, Nb;               // Nb = batch tile = UMMA N (multiple of 16, <= 256)
    int stages;
    uint32_t tmem_cols;            // power of two >= 32 covering the accumulators
    float* y;                      // RAW / RESID: fp32 [B][N]
    const float* resid;            // RESID: fp32 [B][N] (may alias y)
    bf16_t* h16;                   // SWIGLU: bf16 [B][N]
    int* err;
};

__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, int* err, int code) {
    for (uint32_t i = 0; i < kTcSpin; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(err, code);
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t mbar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(mbar), "r"(c0), "r"(c1)
        : "memory");
}

// Shared-memory matrix descriptor: K-major tile of 128-byte rows, 128-byte swizzle, 8-row groups
// 1024 bytes apart (the layout a TMA load with CU_TENSOR_MAP_SWIZZLE_128B produces).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);     // start address / 16
    d |= (uint64_t)1 << 16;                           // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                           // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                           // 128-byte swizzle
    return d;
}

// Instruction descriptor of tcgen05.mma kind::f16: bf16 x bf16 -> fp32, both operands K-major.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 16 consecutive fp32 columns of this warp's 32 TMEM lanes: thread t gets lane (32*warp + t).
// The load is asynchronous: tmem_ld_wait() before the registers are read.
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

template <int MODE>
__global__ void __launch_bounds__(128, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA,
                                                          const __grid_constant__ CUtensorMap tmA2,
                                                          const __grid_constant__ CUtensorMap tmB, GemmTcParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int NA = MODE == TC_SWIGLU ? 2 : 1;
    const int a_bytes = kTcM * 128;
    const int b_bytes = p.Nb * 128;
    const int stage_bytes = NA * a_bytes + b_bytes;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int m0 = blockIdx.x * kTcM;
    const int b0 = blockIdx.y * p.Nb;
    const int nkb = (p.K + kTcKB - 1) / kTcKB;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)p.stages * stage_bytes);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = full0 + 8u * p.stages;
    const uint32_t accum = empty0 + 8u * p.stages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * p.stages + 1);

    if (tid == 0) {
        for (int i = 0; i < p.stages; ++i) {
            mbar_init(full0 + 8u * i, 1);
            mbar_init(empty0 + 8u * i, 1);
        }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    pdl_launch_dependents();
    if (warp == 0 && lane == 0) {
        // ---- TMA producer ---------------------------------------------------------------------
        // The weight tiles of the first stages depend on nothing: they are on their way before this
        // kernel waits for its predecessor, whose results only the activation tiles need.
        const uint32_t tx = (uint32_t)stage_bytes;
        const int pre = min(p.stages, nkb);
        for (int kb = 0; kb < pre; ++kb) {
            mbar_expect_tx(full0 + 8u * kb, tx);
            const uint32_t base = smem_u32(smem + (size_t)kb * stage_bytes);
            tma_load_2d(base, &tmA, kb * kTcKB, m0, full0 + 8u * kb);
            if (MODE == TC_SWIGLU) tma_load_2d(base + a_bytes, &tmA2, kb * kTcKB, m0, full0 + 8u * kb);
        }
        pdl_wait();                  // the activation operand comes from the predecessor kernel
        for (int kb = 0; kb < pre; ++kb)
            tma_load_2d(smem_u32(smem + (size_t)kb * stage_bytes) + NA * a_bytes, &tmB, kb * kTcKB, b0, full0 + 8u * kb);
        for (int kb = pre; kb < nkb; ++kb) {
            const int s = kb % p.stages;
            const uint32_t ph = (uint32_t)(kb / p.stages) & 1u;
            if (!tc_wait(empty0 + 8u * s, ph ^ 1u, p.err, 11)) break;
            mbar_expect_tx(full0 + 8u * s, tx);
            const uint32_t base = smem_u32(smem + (size_t)s * stage_bytes);
            tma_load_2d(base, &tmA, kb * kTcKB, m0, full0 + 8u * s);
            if (MODE == TC_SWIGLU) tma_load_2d(base + a_bytes, &tmA2, kb * kTcKB, m0, full0 + 8u * s);
            tma_load_2d(base + NA * a_bytes, &tmB, kb * kTcKB, b0, full0 + 8u * s);
        }
    } else {
        pdl_wait();
    }
    if (warp == 1 && lane == 0) {
        // ---- MMA issuer ------------------------------------------------------------------------
        const uint32_t idesc = umma_idesc_bf16(kTcM, p.Nb);
        for (int kb = 0; kb < nkb; ++kb) {
            const int s = kb % p.stages;
            const uint32_t ph = (uint32_t)(kb / p.stages) & 1u;
            if (!tc_wait(full0 + 8u * s, ph, p.err, 12)) break;
            tc_fence_after();
            const uint32_t base = smem_u32(smem + (size_t)s * stage_bytes);
            const uint64_t adesc = umma_desc_sw128(base);
            const uint64_t a2desc = umma_desc_sw128(base + a_bytes);
            const uint64_t bdesc = umma_desc_sw128(base + NA * a_bytes);
#pragma unroll
            for (int j = 0; j < kTcKB / 16; ++j) {
                // 16 bf16 = 32 bytes further along K inside the 128-byte swizzle row
                const uint32_t acc = (kb > 0 || j > 0) ? 1u : 0u;
                umma_bf16(tmem_base, adesc + 2u * j, bdesc + 2u * j, idesc, acc);
                if (MODE == TC_SWIGLU) umma_bf16(tmem_base + (uint32_t)p.Nb, a2desc + 2u * j, bdesc + 2u * j, idesc, acc);
            }
            umma_commit(empty0 + 8u * s);          // the stage is free once these MMAs have read it
        }
        umma_commit(accum);                        // the accumulators are complete
    }
    __syncwarp();

    // ---- epilogue: all four warps ------------------------------------------------------------------
    tc_wait(accum, 0, p.err, 13);
    tc_fence_after();
    const int row = m0 + warp * 32 + lane;            // output feature of this thread
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const bool row_ok = row < p.N;
    // residual values of the first chunk (RESID): fetched one chunk ahead of the stores, because
    // the output may alias the residual and the compiler must keep loads behind earlier stores
    float rnext[16];
    if (MODE == TC_RESID) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int b = b0 + j;
            rnext[j] = (row_ok && b < p.B) ? __ldcg(p.resid + (size_t)b * p.N + row) : 0.f;
        }
    }
    for (int c0 = 0; c0 < p.Nb; c0 += 16) {
        uint32_t v[16], u[16];
        tmem_ld16_issue(tmem_base + lane_base + (uint32_t)c0, v);
        if (MODE == TC_SWIGLU) tmem_ld16_issue(tmem_base + lane_base + (uint32_t)(p.Nb + c0), u);
        float rcur[16];
        if (MODE == TC_RESID) {
#pragma unroll
            for (int j = 0; j < 16; ++j) rcur[j] = rnext[j];
            if (c0 + 16 < p.Nb) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int b = b0 + c0 + 16 + j;
                    rnext[j] = (row_ok && b < p.B) ? __ldcg(p.resid + (size_t)b * p.N + row) : 0.f;
                }
            }
        }
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int b = b0 + c0 + j;
                if (b < p.B) {
                    const size_t o = (size_t)b * p.N + row;
                    const float acc = __uint_as_float(v[j]);
                    if (MODE == TC_RAW) {
                        p.y[o] = acc;
                    } else if (MODE == TC_RESID) {
                        p.y[o] = acc + rcur[j];            // inference.cu:252-260, :283-291
                    } else {
                        const float up = __uint_as_float(u[j]);
                        p.h16[o] = __float2bfloat16_rn((acc / (1.0f + expf(-acc))) * up);   // inference.cu:262-281
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
    }
}

// ---- small kernels around the GEMMs ---------------------------------------------------------------
// RMS norm (+ the layer's per-layer embedding added to the residual stream first) and conversion to
// the bf16 activation operand. One CTA per sequence. (inference.cu:24-50, :83-95)
// x[b] += P . T[tok_b]: the per-layer embedding of a large model as a launch of its own, one
// projection row per thread and the rows of a sequence spread over grid.y CTAs. Inside
// prep_bf16_kernel one CTA per sequence walks all d rows (25 us at d = 2048, ple = 128).
// grid = (B, ceil(d / 64)), block = 64, dynamic shared memory = ple floats.
template <typename T2>
__global__ void __launch_bounds__(64) ple_add_kernel(StepCtl c, float* __restrict__ x, int K, const T2* __restrict__ pleT,
                                                     const T2* __restrict__ pleP, int ple) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    if (!seq_active(c, b)) return;
    extern __shared__ __align__(16) float trow[];
    const int t = c.tok[b];
    for (int j = threadIdx.x; j < ple; j += blockDim.x) trow[j] = Elem<T2>::get(pleT, (size_t)t * ple + j);
    __syncthreads();
    constexpr int EPV2 = Elem<T2>::EPV;
    const int i = blockIdx.y * blockDim.x + threadIdx.x;
    if (i >= K) return;
    float a = 0.f;
    const T2* prow = pleP + (size_t)i * ple;
#pragma unroll 4
    for (int j = 0; j < ple; j += EPV2) {
        float w[EPV2];
        Elem<T2>::load_vec(prow + j, w);
#pragma unroll
        for (int e = 0; e < EPV2; ++e) a = fmaf(w[e], trow[j + e], a);
    }
    x[(size_t)b * K + i] += a;
}

template <typename T2>
__global__ void __launch_bounds__(256) prep_bf16_kernel(StepCtl c, float* __restrict__ x, int K, const float* __restrict__ gain,
                                                        float eps, const T2* __restrict__ pleT, const T2* __restrict__ pleP, int ple,
                                                        bf16_t* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    if (!seq_active(c, b)) return;
    extern __shared__ __align__(16) float sm[];
    float* xs = sm;                 // [K]
    float* trow = sm + K;           // [ple]
    __shared__ float red[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* xr = x + (size_t)b * K;
    if (ple > 0) {
        const int t = c.tok[b];
        for (int j = tid; j < ple; j += blockDim.x) trow[j] = Elem<T2>::get(pleT, (size_t)t * ple + j);
        __syncthreads();
    }
    float ss = 0.f;
    constexpr int EPV2 = Elem<T2>::EPV;
    for (int i = tid; i < K; i += blockDim.x) {
        float v = xr[i];
        if (ple > 0) {
            float a = 0.f;
            const T2* prow = pleP + (size_t)i * ple;
            for (int j = 0; j < ple; j += EPV2) {
                float w[EPV2];
                Elem<T2>::load_vec(prow + j, w);
#pragma unroll
                for (int e = 0; e < EPV2; ++e) a = fmaf(w[e], trow[j + e], a);
            }
            v += a;
            xr[i] = v;              // the residual stream carries the per-layer embedding on
        }
        xs[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (gain != nullptr) {
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
        const float r = sqrtf(tot / (float)K + eps);
        for (int i = tid; i < K; i += blockDim.x) out[(size_t)b * K + i] = __float2bfloat16_rn((xs[i] / r) * gain[i]);
    } else {
        for (int i = tid; i < K; i += blockDim.x) out[(size_t)b * K + i] = __float2bfloat16_rn(xs[i]);
    }
}

// Per-head QK RMS norm, RoPE, KV-cache append, sigmoid gate on the raw fp32 projections of a
// batched GEMM (inference.cu:52-134, :248). grid = (heads of q|k|v|gate, B), block = hd/2 threads.
struct QkvPostParams {
    const float* raw; int n_qkv;
    int nq, nk, nv, ng, hd, kv_heads, qk_norm;
    float eps;
    const float* gq; const float* gk; const float* rope;
    void* kpool; void* vpool;
    const int* page_table; int pt_stride;
    float* qbuf; float* gbuf;
};

template <typename KVT>
__global__ void __launch_bounds__(64) qkv_post_kernel(StepCtl c, QkvPostParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    if (!seq_active(c, b)) return;
    const int hd = p.hd, row0 = blockIdx.x * hd;
    const int pr = threadIdx.x, lane = pr & 31, warp = pr >> 5;
    const int seg_q = p.nq, seg_k = p.nq + p.nk, seg_v = seg_k + p.nv;
    const int seg = row0 < seg_q ? 0 : (row0 < seg_k ? 1 : (row0 < seg_v ? 2 : 3));
    const float* src = p.raw + (size_t)b * p.n_qkv + row0;
    const int r = 2 * pr;
    float a = src[r], cc = src[r + 1];
    const int pos = c.pos[b];
    __shared__ float red[2];
    if (p.qk_norm && seg < 2) {
        float ss = warp_sum(a * a + cc * cc);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = red[0];
        if (blockDim.x > 32) tot += red[1];
        const float rs = sqrtf(tot / (float)hd + p.eps);
        const int srow = seg == 0 ? row0 + r : row0 + r - seg_q;
        const float* g = seg == 0 ? p.gq : p.gk;
        a = (a / rs) * g[srow];
        cc = (cc / rs) * g[srow + 1];
    }
    if (seg < 2) {
        const float cs = p.rope[(size_t)pos * hd + r], sn = p.rope[(size_t)pos * hd + r + 1];
        const float ra = cs * a - sn * cc, rc = sn * a + cs * cc;
        if (seg == 0) {
            p.qbuf[(size_t)b * p.nq + row0 + r] = ra;
            p.qbuf[(size_t)b * p.nq + row0 + r + 1] = rc;
        } else {
            const int kvh = (row0 - seg_q) / hd;
            const int page = p.page_table[(size_t)b * p.pt_stride + pos / kKvBlock];
            const size_t off = (((size_t)page * p.kv_heads + kvh) * kKvBlock + (pos % kKvBlock)) * hd + r;
            Elem<KVT>::put(reinterpret_cast<KVT*>(p.kpool), off, ra);
            Elem<KVT>::put(reinterpret_cast<KVT*>(p.kpool), off + 1, rc);
        }
    } else if (seg == 2) {
        const int kvh = (row0 - seg_k) / hd;
        const int page = p.page_table[(size_t)b * p.pt_stride + pos / kKvBlock];
        const size_t off = (((size_t)page * p.kv_heads + kvh) * kKvBlock + (pos % kKvBlock)) * hd + r;
        Elem<KVT>::put(reinterpret_cast<KVT*>(p.vpool), off, a);
        Elem<KVT>::put(reinterpret_cast<KVT*>(p.vpool), off + 1, cc);
    } else {
        p.gbuf[(size_t)b * p.ng + (row0 - seg_v) + r] = 1.0f / (1.0f + expf(-a));
        p.gbuf[(size_t)b * p.ng + (row0 - seg_v) + r + 1] = 1.0f / (1.0f + expf(-cc));
    }
}

// Greedy pick over the fp32 logits of a batched LM-head GEMM: argmax, lowest index on ties
// (inference_orchestrator.cu:77-84, :112), then append. One CTA per sequence.
static __global__ void __launch_bounds__(256) argmax_advance_kernel(StepCtl c, const float* __restrict__ logits, int V) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    if (!seq_active(c, b)) return;
    const float* lg = logits + (size_t)b * V;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = lg[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    __shared__ float sv[8];
    __shared__ int si[8];
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
        advance_seq(c, b, bi);
    }
}

}  // namespace mlb
