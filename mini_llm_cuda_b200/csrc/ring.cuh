// Shared pieces of the kernels that stream weights through shared memory: mbarrier / TMA-bulk
// wrappers, the ring of shared-memory stages with its bounded waits, the producer's slab issue
// and the consumers' dot products out of a stage. Used by the streamed GEMV (sgemv.cuh), the
// whole-GPU batch-1 step (grid.cuh), the tcgen05 GEMM (gemm_tc.cuh) and the operator tests (ops.cu).
#pragma once
#include "kernels.cuh"

namespace mlb {

// Per-layer pointers and row counts of the single-kernel step, as a device table.
struct StepLayer {
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
static_assert(sizeof(StepLayer) % 8 == 0, "StepLayer is copied in 8-byte words");

constexpr int kRingConsumers = 480;                 // consumer threads (15 warps + 1 producer warp = 16: 128 registers each)
constexpr int kRingWarps = kRingConsumers / 32;
constexpr int kRingThreads = kRingConsumers + 32;   // + one producer warp
constexpr uint32_t kRingSpinLimit = 1u << 24;

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
template <int NW = kRingConsumers / 32>
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory"); }

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
    unsigned backoff_ns;           // producer: pause between polls for a free stage (0: none)
    __device__ __forceinline__ void advance() {
        if (++idx == nst) { idx = 0; phase ^= 1u; }
    }
    __device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, int code) {
        if (*dead) return false;
        // code 1 = the producer waiting for a free stage: it runs stages ahead, so while the ring is full
        // it polls at leisure and leaves the issue slots and the shared-memory pipe to the consumers
        const bool ok = mbar_wait_bounded(bar, parity, kRingSpinLimit, code == 1 ? backoff_ns : 0u);
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
template <typename T, int NW = kRingWarps, bool PERM = false, typename F>
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
template <typename T, int NW = kRingWarps, bool PERM = false, typename F>
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

// Sum over the consumer threads; every consumer gets the total. `red` holds kRingWarps floats.
template <int NW = kRingWarps>
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


}  // namespace mlb
