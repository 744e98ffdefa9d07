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
//     output features) and run the epilogue.
// Nothing but these kernels, the attention / delta-net kernels and the pick runs between two steps'
// embeddings; what the reference does in element-wise kernels lives in the epilogues:
//   * RMS norm is deferred. The kernel that produces the residual stream x (embedding, o-projection,
//     down projection) also writes bf16(x * gain) - the next projection's activation operand - and,
//     per sequence and 128-feature tile, the sum of x^2. The consuming GEMM scales its accumulator
//     column b by 1 / sqrt(sum x_b^2 / K + eps): the same (x / rms) * gain . w up to rounding order.
//   * QKV mode: per-head QK norm, RoPE, KV-cache append and the sigmoid gate on the accumulator.
//   * SWIGLU mode: silu(gate) * up of two accumulators, written as the bf16 operand of the down projection.
//   * RESID mode: residual add in place; the per-layer embedding P . T[tok] of the next layer rides along
//     as extra k-blocks from a second operand pair ([W2 | P] . [h | T[tok]]).
// Reference ops replaced: the cublasGemmEx calls of inference.cu:401-465, :581-602, :623-695,
// :720-743 and the element-wise kernels around them (inference.cu:24-134, :248-291).
// Every mbarrier wait is bounded; a wait that runs out records an error code, the kernel still
// frees its tensor memory and returns.
#pragma once
#include <cuda.h>

#include "ring.cuh"   // mbarrier / TMA wrappers

namespace mlb {

constexpr int kTcM = 128;          // output features per CTA (UMMA M)
constexpr int kTcKB = 64;          // bf16 elements per k-block = one 128-byte swizzle row
constexpr uint32_t kTcSpin = 1u << 22;

enum GemmTcMode : int { TC_RAW = 0, TC_RESID = 1, TC_SWIGLU = 2, TC_QKV = 3 };

// Per-head QK RMS norm, RoPE, KV-cache append, sigmoid gate (inference.cu:52-134, :248) on the rows of a
// fused q|k|v|gate projection.
struct QkvPostParams {
    int nq, nk, nv, ng, hd, kv_heads, qk_norm;
    float eps;
    const float* gq; const float* gk; const float* rope;
    void* kpool; void* vpool;
    const int* page_table; int pt_stride;
    float* qbuf; float* gbuf;
};

struct GemmTcParams {
    int N, K, B, Nb;               // Nb = batch tile = UMMA N (multiple of 16, <= 256)
    int stages;                    // ring depth, a multiple of `group`
    int group;                     // k-blocks per refill of the ring: one tcgen05.commit frees `group` stages
    int nkb_x;                     // k-blocks taken from the second operand pair after the K / 64 of the first
    uint32_t tmem_cols;            // power of two >= 32 covering the accumulators
    float* y;                      // RAW / RESID: fp32 [B][N]
    const float* resid;            // RESID: fp32 [B][N] (may alias y)
    bf16_t* h16;                   // SWIGLU: bf16 [B][N]
    // deferred RMS norm of the activation operand: partial sums of squares [B][ssq_parts]; null = operand is used as is
    const float* ssq_in; int ssq_parts; float eps;
    // RESID: operand and partial sums for the next norm (null = not wanted)
    bf16_t* xg16; const float* gain_next; float* ssq_out;
    int* err;
    const float* sA; const float* sA2;   // FP8 weights: per-row scales of the weight tile(s), applied in the epilogue
    unsigned long long* trace;     // diagnostics: five %globaltimer stamps of CTA (0, 0, 0), or null
};

// vals[16] per lane -> the sum over the warp's 32 lanes of column (lane >> 1) & 15, in 16 shuffles
__device__ __forceinline__ float warp_colsum16(float (&v)[16], int lane) {
    {
        const bool hi = (lane & 16) != 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float send = hi ? v[j] : v[j + 8], keep = hi ? v[j + 8] : v[j];
            v[j] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
        }
    }
    {
        const bool hi = (lane & 8) != 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float send = hi ? v[j] : v[j + 4], keep = hi ? v[j + 4] : v[j];
            v[j] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
        }
    }
    {
        const bool hi = (lane & 4) != 0;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float send = hi ? v[j] : v[j + 2], keep = hi ? v[j + 2] : v[j];
            v[j] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
        }
    }
    {
        const bool hi = (lane & 2) != 0;
        const float send = hi ? v[0] : v[1], keep = hi ? v[1] : v[0];
        v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
    }
    return v[0] + __shfl_xor_sync(0xffffffffu, v[0], 1);
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Loads the compiler must issue where they are written (it otherwise sinks a prefetch to its first use, past
// the wait for the accumulator, and the epilogue pays one L2 latency per column: 0.5 us each, measured).
__device__ __forceinline__ float2 ld_nc_f2_now(const float2* p) {
    float2 v;
    asm volatile("ld.global.nc.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ float ld_cg_f32_now(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
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

constexpr int kTcThreads = 256;   // warp 0: TMA loader, warp 1: MMA issuer; all 8 warps run the epilogue (warps w and w + 4 share TMEM lanes)
constexpr int kTcHeadBytes = 9216;     // epilogue words (7680 B) and barriers
constexpr int kTcStageBytes = 32768;   // staging of the QKV epilogue
constexpr size_t kTcRingBytes = 184 * 1024;   // what is left of 227 KB for the ring of stages
constexpr int kTcEpiFloats = 256 + 4 * 256 + 8 * 16 + 2 * 256;   // column scales, per-warp column sums, per-warp head sums, positions, pages

// ---- thread-block cluster: the CTAs that share one output tile and split its k-blocks -----------------
// barrier over the four warps of one epilogue group (hardware barriers 1 and 2; 0 is __syncthreads)
__device__ __forceinline__ void group_sync(int grp) { asm volatile("bar.sync %0, 128;" ::"r"(grp + 1) : "memory"); }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Hardware barrier over the CTAs of the cluster; every CTA reaches every one of them (no early return in
// the kernel), so it needs no bound.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float cluster_ld_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

// two e4m3 codes -> two bf16 (exact: 3 mantissa bits, exponent range inside bf16's)
__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2(uint32_t two_codes) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)two_codes, __NV_E4M3);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
    const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
    return *reinterpret_cast<const uint32_t*>(&b);
}

// Four e4m3 codes (one 32-bit word) -> four bf16 in two words, with integer instructions: for a normal code the
// bf16 bit pattern is sign | ((code & 0x7f) << 4) + (120 << 7) (exponent rebias 7 -> 127, mantissa 3 -> 7 bits).
// Conversion instructions run at a quarter of the integer rate. Not valid for zeros and subnormal codes
// (exponent field 0, about one weight in 10^4): e4m3_word_has_exp0 tells, and the caller then converts exactly.
__device__ __forceinline__ void e4m3x4_to_bf16x4_normal(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t x0 = __byte_perm(w, 0u, 0x1404u);      // codes 0, 1 in the high bytes of the two halves
    const uint32_t x1 = __byte_perm(w, 0u, 0x3424u);      // codes 2, 3
    lo = (x0 & 0x80008000u) | (((x0 >> 4) & 0x07f007f0u) + 0x3c003c00u);
    hi = (x1 & 0x80008000u) | (((x1 >> 4) & 0x07f007f0u) + 0x3c003c00u);
}
// Nonzero iff one of the four codes has exponent field 0: subtracting 1 from the 4-bit field borrows into the
// (masked, hence clear) bit above it.
__device__ __forceinline__ uint32_t e4m3_word_has_exp0(uint32_t w) {
    const uint32_t e = w & 0x78787878u;
    return (e - 0x08080808u) & 0x80808080u;
}

// FP8 weights (WT = fp8_t): the weight tile arrives as e4m3 codes ([128 x 64] bytes by TMA, no swizzle) in a raw
// area of the stage; warps 4-7 widen it to bf16 into the swizzled operand tile the MMA reads (exact), and the
// per-row scale multiplies the accumulator row in the epilogue. Half the weight bytes of a bf16 copy, no copy.
// A bf16 extension operand (the per-layer embedding behind the down projection) then gets an accumulator of
// its own, since it must not be scaled.
// grid = (ceil(N / 128), ceil(B / Nb), split) with clusters of (1, 1, split) when split > 1: the `split`
// CTAs of a cluster take consecutive shares of the k-blocks of one output tile (a tcgen05.mma of these
// shapes costs about 0.1 us whatever its N, so the k-loop of a lone CTA is the time of the kernel), leave
// their partial accumulators in shared memory, and each finishes Nb / split columns of the tile from the
// partials of all of them, read over distributed shared memory in a fixed order.
template <int MODE, typename KVT, typename WT>
__global__ void __launch_bounds__(kTcThreads) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA,
                                                       const __grid_constant__ CUtensorMap tmA2,
                                                       const __grid_constant__ CUtensorMap tmB,
                                                       const __grid_constant__ CUtensorMap tmAx,
                                                       const __grid_constant__ CUtensorMap tmBx, GemmTcParams p,
                                                       StepCtl c, QkvPostParams q) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const bool tracing = p.trace != nullptr && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    if (tracing) p.trace[0] = globaltimer_ns();          // entry
    constexpr int NA = MODE == TC_SWIGLU ? 2 : 1;
    constexpr bool W8 = sizeof(WT) == 1;
    constexpr bool EXT2 = W8 && MODE == TC_RESID;
    constexpr int NACC = (MODE == TC_SWIGLU || EXT2) ? 2 : 1;      // accumulators of Nb columns each
    const int a_bytes = kTcM * 128;
    const int b_bytes = p.Nb * 128;
    const int raw_bytes = W8 ? NA * kTcM * kTcKB : 0;     // lands in the upper half of the operand tile it becomes
    const int stage_bytes = NA * a_bytes + b_bytes;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int m0 = blockIdx.x * kTcM;
    const int b0 = blockIdx.y * p.Nb;
    const int nkb1 = (p.K + kTcKB - 1) / kTcKB;
    const int split = (int)gridDim.z, rank = (int)blockIdx.z;      // cluster = the CTAs of one (x, y)
    // this CTA's k-blocks [kb_lo, kb_lo + nkb) of the nkb1 + nkb_x of the tile
    const int nkb_all = nkb1 + p.nkb_x;
    const int kb_lo = (int)(((long)nkb_all * rank) / split);
    const int nkb = (int)(((long)nkb_all * (rank + 1)) / split) - kb_lo;
    const int n_main = max(0, min(nkb, nkb1 - kb_lo));             // of them, k-blocks of the main operand pair (first)

    // shared memory: [epilogue words][barriers][ring stages | partial accumulators]; the offsets of the first
    // two are the same in every CTA of a cluster
    float* rinv_s = reinterpret_cast<float*>(smem);               // [256] scale of column b
    float* colsum_s = rinv_s + 256;                               // [4][256] per-warp sums of x^2 (RESID)
    float* head_s = colsum_s + 4 * 256;                           // [8][16] per-warp sums of a chunk (QK norm)
    int* pos_s = reinterpret_cast<int*>(head_s + 8 * 16);         // [256] position of column b, -1 = takes no part (QKV)
    int* page_s = pos_s + 256;                                    // [256] KV page its new row goes to (QKV)
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kTcEpiFloats * 4);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = full0 + 8u * p.stages;
    const uint32_t accum = empty0 + 8u * p.stages;
    const uint32_t rawfull0 = accum + 8u;                          // FP8: raw weight tile of a stage has landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * p.stages + 1);
    float* stage_s = reinterpret_cast<float*>(smem + kTcHeadBytes);                  // [2 groups][16][128] a chunk of the tile (QKV)
    float* rope_s = stage_s + 2 * 16 * kTcM;                                         // [2 groups][16][128] its RoPE factors (QKV)
    unsigned char* ring = smem + kTcHeadBytes + kTcStageBytes;    // 1024-aligned
    float* part = reinterpret_cast<float*>(ring);                 // [NA][Nb][128] partial accumulators (split > 1), over the ring

    if (tid == 0) {
        for (int i = 0; i < p.stages; ++i) {
            mbar_init(full0 + 8u * i, W8 ? 5 : 1);        // the loader, plus the four widening warps
            mbar_init(empty0 + 8u * i, 1);
            mbar_init(rawfull0 + 8u * i, 1);
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
    if (tracing) p.trace[1] = globaltimer_ns();          // barriers and tensor memory set up

    pdl_launch_dependents();
    if (warp == 0 && lane == 0) {
        // ---- TMA producer ---------------------------------------------------------------------
        // The weight tiles of the first stages depend on nothing: they are on their way before this
        // kernel waits for its predecessor, whose results only the activation tiles need.
        auto tx_of = [&](int kb) -> uint32_t {           // bytes that complete the stage's `full` barrier
            if (!W8) return (uint32_t)stage_bytes;
            return (uint32_t)(kb < n_main ? b_bytes : a_bytes + b_bytes);
        };
        auto load_a = [&](int kb, uint32_t base, uint32_t bar, uint32_t rbar) {
            const int k = kb_lo + kb;
            if (k < nkb1) {
                if (W8) {
                    mbar_expect_tx(rbar, (uint32_t)raw_bytes);
                    tma_load_2d(base + a_bytes / 2, &tmA, k * kTcKB, m0, rbar);
                    if (MODE == TC_SWIGLU) tma_load_2d(base + a_bytes + a_bytes / 2, &tmA2, k * kTcKB, m0, rbar);
                } else {
                    tma_load_2d(base, &tmA, k * kTcKB, m0, bar);
                    if (MODE == TC_SWIGLU) tma_load_2d(base + a_bytes, &tmA2, k * kTcKB, m0, bar);
                }
            } else {
                tma_load_2d(base, &tmAx, (k - nkb1) * kTcKB, m0, bar);
                if (W8) mbar_arrive(rbar);           // nothing to widen: the widening warps just pass
            }
        };
        auto load_b = [&](int kb, uint32_t base, uint32_t bar) {
            const int k = kb_lo + kb;
            if (k < nkb1) tma_load_2d(base + NA * a_bytes, &tmB, k * kTcKB, b0, bar);
            else tma_load_2d(base + NA * a_bytes, &tmBx, (k - nkb1) * kTcKB, b0, bar);
        };
        const int pre = min(p.stages, nkb);
        for (int kb = 0; kb < pre; ++kb) {
            mbar_expect_tx(full0 + 8u * kb, tx_of(kb));
            load_a(kb, smem_u32(ring + (size_t)kb * stage_bytes), full0 + 8u * kb, rawfull0 + 8u * kb);
        }
        pdl_wait();                  // the activation operand comes from the predecessor kernel
        if (tracing) p.trace[2] = globaltimer_ns();      // predecessor complete
        for (int kb = 0; kb < pre; ++kb) load_b(kb, smem_u32(ring + (size_t)kb * stage_bytes), full0 + 8u * kb);
        for (int kb = pre; kb < nkb; ++kb) {
            const int s = kb % p.stages;
            const uint32_t ph = (uint32_t)(kb / p.stages) & 1u;
            // the stages come back `group` at a time, on the barrier of the group's last stage
            if (kb % p.group == 0 && !tc_wait(empty0 + 8u * (s + p.group - 1), ph ^ 1u, p.err, 11)) break;
            mbar_expect_tx(full0 + 8u * s, tx_of(kb));
            const uint32_t base = smem_u32(ring + (size_t)s * stage_bytes);
            load_a(kb, base, full0 + 8u * s, rawfull0 + 8u * s);
            load_b(kb, base, full0 + 8u * s);
        }
    } else if (W8 && warp >= 4) {
        // ---- FP8: widen the raw weight tiles into the operand tiles ---------------------------------
        // Piece q of a tile = 8 codes = row q / 8, 16-byte chunk q % 8 of the bf16 row; consecutive lanes take
        // consecutive pieces (8-byte reads side by side, the 8 chunks of a row written by 8 lanes). The chunk
        // lands where the 128-byte swizzle of the MMA's descriptor expects it: chunk ^ (row % 8).
        const int t = tid - 128;
        bool dead = false;       // a wait ran out: stop waiting, but keep the four warps in step (they share a barrier)
        for (int kb = 0; kb < nkb; ++kb) {
            const int s = kb % p.stages;
            const uint32_t ph = (uint32_t)(kb / p.stages) & 1u;
            if (!dead && !tc_wait(rawfull0 + 8u * s, ph, p.err, 14)) dead = true;
            if (kb < n_main) {
                unsigned char* st_base = ring + (size_t)s * stage_bytes;
                const unsigned char* raw = st_base + a_bytes / 2;      // codes of tile a at raw + a * a_bytes
                uint2 w[NA * 8];
                uint32_t exp0 = 0;
#pragma unroll
                for (int i = 0; i < NA * 8; ++i) {
                    w[i] = *reinterpret_cast<const uint2*>(raw + (i >> 3) * a_bytes + (t + 128 * (i & 7)) * 8);
                    exp0 |= e4m3_word_has_exp0(w[i].x) | e4m3_word_has_exp0(w[i].y);
                }
                // every code is in registers before any bf16 lands on top of the raw tile
                asm volatile("bar.sync 3, 128;" ::: "memory");
                // one branch per k-block and thread (two loops the compiler cannot merge into predicated code)
                if (exp0 == 0) {
#pragma unroll
                    for (int i = 0; i < NA * 8; ++i) {
                        const int qd = t + 128 * (i & 7), r = qd >> 3, ch = qd & 7;
                        uint4 o;
                        e4m3x4_to_bf16x4_normal(w[i].x, o.x, o.y);
                        e4m3x4_to_bf16x4_normal(w[i].y, o.z, o.w);
                        *reinterpret_cast<uint4*>(st_base + (i >> 3) * a_bytes + (r >> 3) * 1024 + (r & 7) * 128 + ((ch ^ (r & 7)) << 4)) = o;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < NA * 8; ++i) {
                        const int qd = t + 128 * (i & 7), r = qd >> 3, ch = qd & 7;
                        const uint2 wi = w[i];
                        uint4 o;
                        o.x = e4m3x2_to_bf16x2(wi.x & 0xffffu);
                        o.y = e4m3x2_to_bf16x2(wi.x >> 16);
                        o.z = e4m3x2_to_bf16x2(wi.y & 0xffffu);
                        o.w = e4m3x2_to_bf16x2(wi.y >> 16);
                        *reinterpret_cast<uint4*>(st_base + (i >> 3) * a_bytes + (r >> 3) * 1024 + (r & 7) * 128 + ((ch ^ (r & 7)) << 4)) = o;
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic writes -> the MMA's reads
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(full0 + 8u * s);
        }
        pdl_wait();
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
            const uint32_t base = smem_u32(ring + (size_t)s * stage_bytes);
            const uint64_t adesc = umma_desc_sw128(base);
            const uint64_t a2desc = umma_desc_sw128(base + a_bytes);
            const uint64_t bdesc = umma_desc_sw128(base + NA * a_bytes);
#pragma unroll
            for (int j = 0; j < kTcKB / 16; ++j) {
                // 16 bf16 = 32 bytes further along K inside the 128-byte swizzle row
                if (EXT2 && kb >= n_main) {
                    // bf16 extension operand: its own accumulator (the main one is scaled per row afterwards)
                    umma_bf16(tmem_base + (uint32_t)p.Nb, adesc + 2u * j, bdesc + 2u * j, idesc, (kb > n_main || j > 0) ? 1u : 0u);
                } else {
                    const uint32_t acc = (kb > 0 || j > 0) ? 1u : 0u;
                    umma_bf16(tmem_base, adesc + 2u * j, bdesc + 2u * j, idesc, acc);
                    if (MODE == TC_SWIGLU) umma_bf16(tmem_base + (uint32_t)p.Nb, a2desc + 2u * j, bdesc + 2u * j, idesc, acc);
                }
            }
            // hand stages back only where the loader will refill them, a group at a time
            if (kb % p.group == p.group - 1 && kb - (p.group - 1) + p.stages < nkb) umma_commit(empty0 + 8u * s);
        }
        umma_commit(accum);                        // the accumulators are complete (at once, if there was no k-block)
    }
    if (warp >= 2 && !(W8 && warp >= 4)) {
        // scale of column b from the partial sums of squares its producer left (inference.cu:24-50)
        for (int j = tid - 64; j < p.Nb; j += (W8 ? 64 : kTcThreads - 64)) {
            float r = 1.0f;
            const int b = b0 + j;
            if (p.ssq_in != nullptr && b < p.B) {
                float tot = 0.f;
                for (int t = 0; t < p.ssq_parts; ++t) tot += __ldcg(p.ssq_in + (size_t)b * p.ssq_parts + t);
                r = 1.0f / sqrtf(tot / (float)p.K + p.eps);
            }
            rinv_s[j] = r;
            if (MODE == TC_QKV) {
                // position and KV page of the column: fetched here, off the epilogue's critical path
                int pos = -1, page = 0;
                if (seq_active(c, b)) {
                    pos = c.pos[b];
                    page = q.page_table[(size_t)b * q.pt_stride + pos / kKvBlock];
                }
                pos_s[j] = pos;
                page_s[j] = page;
            }
        }
    }
    __syncthreads();

    // ---- epilogue: all four warps ------------------------------------------------------------------
    // Two groups of four warps: group g takes every other chunk of 16 columns. The epilogue is a chain of
    // dependent instructions per thread, so its time follows the columns a thread owns.
    const int wq = warp & 3, grp = warp >> 2;
    const int row = m0 + wq * 32 + lane;              // output feature of this thread
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    const bool row_ok = row < p.N;
    // the columns this CTA finishes: all of the tile, or its share of them
    const int cb = split > 1 ? (p.Nb * rank) / split : 0;
    const int ce = split > 1 ? (p.Nb * (rank + 1)) / split : p.Nb;
    // residual values of the first chunk (RESID): fetched one chunk ahead of the stores, because
    // the output may alias the residual and the compiler must keep loads behind earlier stores
    float rnext[16];
    float gain = 0.f;
    if (MODE == TC_RESID) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int b = b0 + cb + 16 * grp + j;
            rnext[j] = (row_ok && cb + 16 * grp + j < ce && b < p.B) ? ld_cg_f32_now(p.resid + (size_t)b * p.N + row) : 0.f;
        }
        if (p.xg16 != nullptr && row_ok) gain = p.gain_next[row];
    }
    // QKV: which of q | k | v | gate this warp's 32 rows belong to (the parts are whole heads of 64 or 128 rows)
    const int seg_q = q.nq, seg_k = q.nq + q.nk, seg_v = seg_k + q.nv;
    int seg = 0, rloc = 0, kvh = 0, head_w0 = 0, head_wn = 1;
    float gn = 1.0f;
    if (MODE == TC_QKV) {
        const int wrow = m0 + wq * 32;
        seg = wrow < seg_q ? 0 : (wrow < seg_k ? 1 : (wrow < seg_v ? 2 : 3));
        rloc = row % q.hd;
        kvh = seg == 1 ? (row - seg_q) / q.hd : (seg == 2 ? (row - seg_k) / q.hd : 0);
        head_wn = q.hd / 32;
        head_w0 = grp * 4 + wq / head_wn * head_wn;
        if (q.qk_norm && seg < 2 && row_ok) gn = seg == 0 ? q.gq[row] : q.gk[row - seg_q];
    }
    // QKV: the chunk of 16 columns a group works on goes through shared memory, so that the per-column work is a
    // rolled loop: unrolled over the 16 accumulator registers it was 25 KB of code that every CTA ran once, from
    // a cold instruction cache (8 us per chunk, measured; 1 us this way). The RoPE factors of the chunk's
    // positions are staged the same way, for the first chunk before the accumulator is waited for.
    const int r128 = tid & 127;
    float* st = stage_s + grp * 16 * kTcM;
    float* rp = rope_s + grp * 16 * kTcM;
    float gn_other = 1.0f;
    float sa = 1.0f, sa2 = 1.0f;
    if (W8 && row_ok) {
        if (p.sA != nullptr) sa = p.sA[row];
        if (MODE == TC_SWIGLU && p.sA2 != nullptr) sa2 = p.sA2[row];
    }
    if (MODE == TC_QKV && q.qk_norm && seg < 2 && (row ^ 1) < p.N) gn_other = seg == 0 ? q.gq[row ^ 1] : q.gk[(row ^ 1) - seg_q];
    auto stage_rope = [&](int c0) {
        float t[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int pos = c0 + j < ce ? pos_s[c0 + j] : -1;
            t[j] = (pos >= 0 && row_ok && seg < 2) ? __ldg(q.rope + (size_t)pos * q.hd + rloc) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) rp[j * kTcM + r128] = t[j];
    };
    if (MODE == TC_QKV) stage_rope(cb + 16 * grp);
    tc_wait(accum, 0, p.err, 13);
    tc_fence_after();
    if (tracing) p.trace[3] = globaltimer_ns();          // accumulators complete
    if (split > 1) {
        // partial accumulators of all Nb columns into shared memory (the ring is idle: every MMA that read it
        // has completed), column-major so that a warp writes and later reads 128 consecutive bytes
        for (int c0 = 16 * grp; c0 < NACC * p.Nb; c0 += 32) {
            uint32_t t[16];
            tmem_ld16_issue(tmem_base + lane_base + (uint32_t)c0, t);
            tmem_ld_wait();
            // an accumulator no MMA of this CTA wrote holds nothing
            const bool written = EXT2 ? (c0 < p.Nb ? n_main > 0 : nkb > n_main) : nkb > 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) part[(size_t)(c0 + j) * kTcM + (tid & 127)] = written ? __uint_as_float(t[j]) : 0.f;
        }
        cluster_sync_all();
    }
    const uint32_t part_addr = smem_u32(part);
    // both groups run the same number of rounds; a round past the group's last chunk has all its columns masked
    for (int c0 = cb + 16 * grp; c0 - 16 * grp < ce; c0 += 32) {
        float v[16], u[16];
        float rcur[16];
        if (MODE == TC_RESID) {
#pragma unroll
            for (int j = 0; j < 16; ++j) rcur[j] = rnext[j];
            if (c0 + 32 < ce) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int b = b0 + c0 + 32 + j;
                    rnext[j] = (row_ok && c0 + 32 + j < ce && b < p.B) ? ld_cg_f32_now(p.resid + (size_t)b * p.N + row) : 0.f;
                }
            }
        }
        if (split > 1) {
#pragma unroll
            for (int j = 0; j < 16; ++j) { v[j] = 0.f; u[j] = 0.f; }
            for (int r = 0; r < split; ++r) {
                const uint32_t base = cluster_map(part_addr, (uint32_t)r) + (uint32_t)(tid & 127) * 4u;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (c0 + j < ce) {
                        v[j] += cluster_ld_f32(base + (uint32_t)(c0 + j) * (kTcM * 4u));
                        if (NACC == 2) u[j] += cluster_ld_f32(base + (uint32_t)(p.Nb + c0 + j) * (kTcM * 4u));
                    }
                }
            }
        } else {
            uint32_t t[16], t2[16];
            const uint32_t cc = (uint32_t)(c0 < ce ? c0 : cb);       // a masked round reads a valid chunk and drops it
            tmem_ld16_issue(tmem_base + lane_base + cc, t);
            if (NACC == 2) tmem_ld16_issue(tmem_base + lane_base + (uint32_t)p.Nb + cc, t2);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                v[j] = __uint_as_float(t[j]);
                if (NACC == 2) u[j] = (EXT2 && nkb <= n_main) ? 0.f : __uint_as_float(t2[j]);
            }
        }
        if (W8) {
            // per-row scales of the FP8 weights; the extension operand's accumulator is not scaled
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                v[j] *= sa;
                if (MODE == TC_SWIGLU) u[j] *= sa2;
                if (EXT2) v[j] += u[j];
            }
        }
        if (MODE == TC_QKV) {
            float vv[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                vv[j] = c0 + j < ce ? v[j] * rinv_s[c0 + j] : 0.f;
                st[j * kTcM + r128] = vv[j];
            }
            if (q.qk_norm) {
                float sq[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) sq[j] = (seg < 2 && row_ok) ? vv[j] * vv[j] : 0.f;
                const float tot = warp_colsum16(sq, lane);
                if (!(lane & 1)) head_s[warp * 16 + ((lane >> 1) & 15)] = tot;
            }
            group_sync(grp);
            const float inv_hd = 1.0f / (float)q.hd;
#pragma unroll 1
            for (int j = 0; j < 16; ++j) {
                const int pos = c0 + j < ce ? pos_s[c0 + j] : -1;
                if (!row_ok || pos < 0) continue;
                const int b = b0 + c0 + j;
                float val = st[j * kTcM + r128];
                if (seg < 2) {
                    float oth = st[j * kTcM + (r128 ^ 1)];
                    if (q.qk_norm) {
                        float t = 0.f;
                        for (int w = 0; w < head_wn; ++w) t += head_s[(head_w0 + w) * 16 + j];
                        const float sc = rsqrtf(t * inv_hd + q.eps);
                        val *= sc * gn;
                        oth *= sc * gn_other;
                    }
                    const float cs = rp[j * kTcM + (r128 & ~1)], sn = rp[j * kTcM + (r128 | 1)];
                    const float rot = (rloc & 1) ? fmaf(sn, oth, cs * val) : fmaf(cs, val, -(sn * oth));
                    if (seg == 0) {
                        q.qbuf[(size_t)b * q.nq + row] = rot;
                    } else {
                        const size_t off = (((size_t)page_s[c0 + j] * q.kv_heads + kvh) * kKvBlock + (pos % kKvBlock)) * q.hd + rloc;
                        Elem<KVT>::put(reinterpret_cast<KVT*>(q.kpool), off, rot);
                    }
                } else if (seg == 2) {
                    const size_t off = (((size_t)page_s[c0 + j] * q.kv_heads + kvh) * kKvBlock + (pos % kKvBlock)) * q.hd + rloc;
                    Elem<KVT>::put(reinterpret_cast<KVT*>(q.vpool), off, val);
                } else {
                    q.gbuf[(size_t)b * q.ng + (row - seg_v)] = __fdividef(1.0f, 1.0f + __expf(-val));
                }
            }
            group_sync(grp);                         // the staging is reused by the next chunk
            if (c0 + 32 < ce) stage_rope(c0 + 32);
        } else {
            float sq[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int b = b0 + c0 + j;
                sq[j] = 0.f;
                if (row_ok && c0 + j < ce && b < p.B) {
                    const size_t o = (size_t)b * p.N + row;
                    const float acc = v[j];
                    if (MODE == TC_RAW) {
                        p.y[o] = acc * rinv_s[c0 + j];
                    } else if (MODE == TC_RESID) {
                        const float xn = acc + rcur[j];    // inference.cu:252-260, :283-291
                        p.y[o] = xn;
                        if (p.xg16 != nullptr) {
                            p.xg16[o] = __float2bfloat16_rn(xn * gain);
                            sq[j] = xn * xn;
                        }
                    } else {
                        const float ri = rinv_s[c0 + j];
                        const float g = acc * ri, up = u[j] * ri;
                        p.h16[o] = __float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)) * up);   // inference.cu:262-281
                    }
                }
            }
            if (MODE == TC_RESID && p.xg16 != nullptr) {
                const float tot = warp_colsum16(sq, lane);
                const int col = c0 + ((lane >> 1) & 15);
                if (!(lane & 1) && col < ce) colsum_s[wq * 256 + col] = tot;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (MODE == TC_RESID && p.ssq_out != nullptr) {
        for (int j = cb + tid; j < ce; j += kTcThreads) {
            const int b = b0 + j;
            if (b < p.B)
                p.ssq_out[(size_t)b * gridDim.x + blockIdx.x] =
                    (colsum_s[j] + colsum_s[256 + j]) + (colsum_s[512 + j] + colsum_s[768 + j]);
        }
    }
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
    }
    if (tracing) p.trace[4] = globaltimer_ns();          // epilogue done
    if (split > 1) cluster_sync_all();      // the partial accumulators stay until every CTA of the cluster has read them
}

// ---- small kernels around the GEMMs ---------------------------------------------------------------
// Start of a step: token embedding plus the first layer's per-layer embedding into the fp32 residual
// stream (inference.cu:137-170), its bf16(x * gain) operand and partial sums of squares for the first
// projection, and the per-layer embedding rows T_l[tok] of the later layers gathered as bf16 operands of
// the down projections. grid = (B, ceil(d / 128)), block = 128: one feature per thread.
template <typename WT>
__global__ void __launch_bounds__(128) embed_tc_kernel(StepCtl c, const WT* __restrict__ E, const float* __restrict__ escale, int d,
                                                              const StepLayer* __restrict__ layers, int n_layers, int ple,
                                                              const float* __restrict__ gain, float* __restrict__ x,
                                                              bf16_t* __restrict__ xg16, float* __restrict__ ssq,
                                                              bf16_t* __restrict__ tple16) {
    pdl_launch_dependents();
    pdl_wait();                      // pos / tok come from the last kernel of the previous step
    const int b = blockIdx.x;
    if (!seq_active(c, b)) return;
    int t = c.tok[b];
    if (c.tok_src != nullptr) {
        t = c.tok_src[b];
        if (blockIdx.y == 0 && threadIdx.x == 0) c.tok[b] = t;
    }
    extern __shared__ __align__(16) float trow[];
    __shared__ float red[4];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (ple > 0) {
        const bf16_t* T0 = static_cast<const bf16_t*>(layers[0].pleT);
        for (int j = tid; j < ple; j += 128) trow[j] = __bfloat162float(T0[(size_t)t * ple + j]);
        for (int l = 1 + blockIdx.y; l < n_layers; l += gridDim.y) {
            const bf16_t* Tl = static_cast<const bf16_t*>(layers[l].pleT);
            for (int j = tid; j < ple; j += 128) tple16[((size_t)l * c.B + b) * ple + j] = Tl[(size_t)t * ple + j];
        }
        __syncthreads();
    }
    const int i = blockIdx.y * 128 + tid;
    float v = 0.f;
    if (i < d) {
        v = Elem<WT>::get(E, (size_t)t * d + i) * (escale ? escale[t] : 1.0f);
        if (ple > 0) {
            float a = 0.f;
            const bf16_t* prow = static_cast<const bf16_t*>(layers[0].pleP) + (size_t)i * ple;
#pragma unroll 4
            for (int j = 0; j < ple; j += 8) {
                float w[8];
                Elem<bf16_t>::load_vec(prow + j, w);
#pragma unroll
                for (int e = 0; e < 8; ++e) a = fmaf(w[e], trow[j + e], a);
            }
            v += a;
        }
        x[(size_t)b * d + i] = v;
        xg16[(size_t)b * d + i] = __float2bfloat16_rn(v * gain[i]);
    }
    const float ss = warp_sum(v * v);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (tid == 0) ssq[(size_t)b * gridDim.y + blockIdx.y] = (red[0] + red[1]) + (red[2] + red[3]);
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
