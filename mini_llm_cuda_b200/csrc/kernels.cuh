// Decode-step kernels for sm_100a. One decode step of B independent sequences is a short
// chain of HBM-streaming kernels; every per-sequence quantity that changes between steps
// (position, pending token, page table) lives in device memory so that the chain can be
// replayed as a CUDA graph.
//
// Reference ops each kernel folds together are cited at the kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mlb {

typedef __nv_bfloat16 bf16_t;
struct fp8_t { uint8_t v; };   // e4m3 storage

constexpr int kKvBlock = 16;           // positions per KV page
constexpr float kNegBig = -1.0e30f;    // running-max seed (the reference seeds with -1e20, inference.cu:167)

// ------------------------------------------------------------------------------------
// Element / 16-byte vector access per storage type
// ------------------------------------------------------------------------------------
template <typename T> struct Elem;

template <> struct Elem<float> {
    static constexpr int EPV = 4;
    __device__ __forceinline__ static void unpack(const uint4& v, float* o) {
        o[0] = __uint_as_float(v.x); o[1] = __uint_as_float(v.y); o[2] = __uint_as_float(v.z); o[3] = __uint_as_float(v.w);
    }
    __device__ __forceinline__ static void load_vec(const float* p, float* o) {
        float4 v = __ldg(reinterpret_cast<const float4*>(p));
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
    __device__ __forceinline__ static void load_vec_cg(const float* p, float* o) {
        float4 v = __ldcg(reinterpret_cast<const float4*>(p));
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
    __device__ __forceinline__ static float get(const float* p, size_t i) { return p[i]; }
    __device__ __forceinline__ static void put(float* p, size_t i, float v) { p[i] = v; }
};

template <> struct Elem<bf16_t> {
    static constexpr int EPV = 8;
    __device__ __forceinline__ static void unpack(const uint4& v, float* o) {
        o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
        o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
        o[4] = __uint_as_float(v.z << 16); o[5] = __uint_as_float(v.z & 0xffff0000u);
        o[6] = __uint_as_float(v.w << 16); o[7] = __uint_as_float(v.w & 0xffff0000u);
    }
    __device__ __forceinline__ static void load_vec(const bf16_t* p, float* o) {
        unpack(__ldg(reinterpret_cast<const uint4*>(p)), o);
    }
    __device__ __forceinline__ static void load_vec_cg(const bf16_t* p, float* o) {
        unpack(__ldcg(reinterpret_cast<const uint4*>(p)), o);
    }
    __device__ __forceinline__ static float get(const bf16_t* p, size_t i) { return __bfloat162float(p[i]); }
    __device__ __forceinline__ static void put(bf16_t* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }
};

template <> struct Elem<fp8_t> {
    static constexpr int EPV = 16;
    __device__ __forceinline__ static void unpack_word(uint32_t w, float* o) {
        __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w & 0xffffu), __NV_E4M3);
        __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w >> 16), __NV_E4M3);
        float2 a = __half22float2(*reinterpret_cast<__half2*>(&lo));
        float2 b = __half22float2(*reinterpret_cast<__half2*>(&hi));
        o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
    }
    __device__ __forceinline__ static void unpack(const uint4& v, float* o) {
        unpack_word(v.x, o); unpack_word(v.y, o + 4); unpack_word(v.z, o + 8); unpack_word(v.w, o + 12);
    }
    __device__ __forceinline__ static void load_vec(const fp8_t* p, float* o) {
        unpack(__ldg(reinterpret_cast<const uint4*>(p)), o);
    }
    __device__ __forceinline__ static float get(const fp8_t* p, size_t i) {
        __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(p[i].v), __NV_E4M3);
        return __half2float(*reinterpret_cast<__half*>(&h));
    }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Layout of an activation vector staged in shared memory for a GEMV whose weights come as
// 16-byte vectors of EPV elements: lane l of a warp multiplies weight vector vi = l + 32 i with
// x[vi*EPV .. vi*EPV+EPV). Stored linearly, the lanes' float4 reads would be EPV*4 bytes apart
// (2-way bank conflicts for bf16 weights, 4-way for fp8). Stored as [EPV/4][nvec] float4s, the
// q-th float4 of 32 consecutive vectors is 512 contiguous bytes: conflict-free.
template <int EPV>
__device__ __forceinline__ int xs_f4_index(int j, int nvec) {      // j: float4 index in linear order
    constexpr int Q = EPV / 4;
    return (j % Q) * nvec + j / Q;
}
template <int EPV>
__device__ __forceinline__ int xs_index(int k, int nvec) {          // k: element index in linear order
    return xs_f4_index<EPV>(k >> 2, nvec) * 4 + (k & 3);
}

// Programmatic dependent launch (PDL): every kernel of the step lets its successor start
// launching at once and waits for its predecessor's results only where it first needs them, so
// that launch latency and the weight fetch (which depends on nothing) overlap the predecessor.
// Both instructions are no-ops for a kernel launched without the PDL attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ------------------------------------------------------------------------------------
// Per-step control block shared by all kernels of a step
// ------------------------------------------------------------------------------------
struct StepCtl {
    int B;
    int vocab;
    int* pos;            // [B] position of the pending token == tokens consumed so far
    int* tok;            // [B] pending token
    int* limit;          // [B] a sequence takes part in the step iff pos < limit
    int stop_token;      // a sequence that picks this id leaves the batch after appending it (limit = pos); -1 = none
    // prompt forcing (prefill chain) and output ring (decode chain)
    const int* prompt;   // [B][prompt_stride] or null
    int prompt_stride;
    int* out_ring;       // [B][out_cap]
    int* out_idx;        // [B]
    int out_cap;
    // one-token call: ids and the error word cross the bus inside the step's own kernels (pinned host
    // memory mapped into the device), instead of as copies queued around the step; all null otherwise
    const int* tok_src;  // [B] pending ids in host memory, read by the embedding kernel
    int* host_out;       // [B] picked ids, written where the sequence advances
    int* host_err;       // copy of *dev_err at the end of the step
    const int* dev_err;
};

__device__ __forceinline__ bool seq_active(const StepCtl& c, int b) {
    return b < c.B && c.pos[b] < c.limit[b];
}

// End of a step for one sequence: append the picked token (decode) or take the next prompt
// token (prefill). Stands in for inference_orchestrator.cu:149-154.
__device__ __forceinline__ void advance_seq(const StepCtl& c, int b, int sampled) {
    int p = c.pos[b];
    if (c.prompt != nullptr) {
        c.tok[b] = c.prompt[(size_t)b * c.prompt_stride + p + 1];
    } else {
        if ((unsigned)sampled >= (unsigned)c.vocab) sampled = 0;   // NaN logits leave no valid pick
        int oi = c.out_idx[b];
        if (oi < c.out_cap) c.out_ring[(size_t)b * c.out_cap + oi] = sampled;
        c.out_idx[b] = oi + 1;
        c.tok[b] = sampled;
        // the host may be polling host_out: the error word goes first
        if (c.host_err != nullptr && b == 0) {
            *c.host_err = *c.dev_err;
            __threadfence_system();
        }
        if (c.host_out != nullptr) c.host_out[b] = sampled;
        if (sampled == c.stop_token) c.limit[b] = p + 1;          // end of this sequence: later steps skip it
    }
    c.pos[b] = p + 1;
}

// Prefill chain has no LM head: a one-thread-per-sequence advance.
static __global__ void advance_kernel(StepCtl c) {
    pdl_launch_dependents();
    pdl_wait();
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < c.B && seq_active(c, b)) advance_seq(c, b, -1);
}

// ------------------------------------------------------------------------------------
// Token-embedding + first-layer PLE gather.   x[b] = E[tok] (+ P0 . T0[tok])
// Reference: setInputSeqEmbeddings, inference.cu:9-22 (gathers all L columns each step;
// here one row per sequence). PLE has no counterpart in the reference.
// ------------------------------------------------------------------------------------
template <typename T, typename T2>
__global__ void embed_kernel(StepCtl c, const T* __restrict__ E, const float* __restrict__ escale, int d,
                             const T2* __restrict__ pleT, const T2* __restrict__ pleP, int p,
                             float* __restrict__ x) {
    pdl_launch_dependents();
    pdl_wait();                      // pos / tok come from the last kernel of the previous step
    int b = blockIdx.x;
    if (!seq_active(c, b)) return;
    int t = c.tok[b];
    if (c.tok_src != nullptr) {
        // the pending id comes straight from host memory; later kernels of the step read the device copy
        t = c.tok_src[b];
        if (blockIdx.y == 0 && threadIdx.x == 0) c.tok[b] = t;
    }
    extern __shared__ __align__(16) float trow[];
    if (p > 0) {
        for (int j = threadIdx.x; j < p; j += blockDim.x) trow[j] = Elem<T2>::get(pleT, (size_t)t * p + j);
        __syncthreads();
    }
    float sc = escale ? escale[t] : 1.0f;
    constexpr int EPV2 = Elem<T2>::EPV;
    // grid.y CTAs share the rows of one sequence: a single CTA walking all of them was the
    // slowest launch of a batch-1 step
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < d; i += gridDim.y * blockDim.x) {
        float v = Elem<T>::get(E, (size_t)t * d + i) * sc;
        if (p > 0) {
            // one row of the projection per thread, 16-byte loads (p is a multiple of 8)
            float a = 0.f;
            const T2* prow = pleP + (size_t)i * p;
#pragma unroll 4
            for (int j = 0; j < p; j += EPV2) {
                float w[EPV2];
                Elem<T2>::load_vec(prow + j, w);
#pragma unroll
                for (int e = 0; e < EPV2; ++e) a = fmaf(w[e], trow[j + e], a);
            }
            v += a;
        }
        x[(size_t)b * d + i] = v;
    }
}

// ------------------------------------------------------------------------------------
// Batched GEMV  y[b][row] = sum_k W[row][k] * xin[b][k]  with fused prologue / epilogue.
//
// A CTA owns R consecutive output rows and a tile of BT sequences. The (optionally
// RMS-normalised) activations of the tile are staged once in shared memory; each warp
// streams RW weight rows at a time with 16-byte loads, every lane striding over K, and
// warp-shuffle-reduces the partial dot products. Results land in shared memory so that the
// epilogue can work on whole heads / pairs.
// ------------------------------------------------------------------------------------
enum GemvMode : int {
    GEMV_RAW = 0,      // y = acc
    GEMV_RESID = 1,    // y = acc + resid   (O projection / FFN down; optional PLE segment)
    GEMV_SWIGLU = 2,   // y = silu(Wa x) * (Wb x)
    GEMV_QKV = 3,      // per-head RMS norm, RoPE, KV-cache append, sigmoid gate
    GEMV_LMHEAD = 4    // logits + argmax partials + last-CTA pick
};

struct GemvParams {
    const void* W;         // [N][K]
    const void* Wb;        // SWIGLU: the up matrix
    const float* wscale;   // fp8: per-row scale (null otherwise)
    const float* wscale_b;
    int N, K, R;
    const float* xin;      // [B][K]
    const float* gain;     // [K] when do_norm
    float eps;
    int do_norm;
    // second K segment: per-layer embedding of the NEXT layer folded into the down projection
    const void* P;         // [N][Kp] (type T2)
    const void* Ptab;      // [vocab][Kp] (type T2)
    int Kp;
    float* y;              // [B][N]
    const float* resid;    // [B][N]
    // QKV epilogue
    int nq, nk, nv, ng;    // rows of the q | k | v | gate segments
    int hd, kv_heads, qk_norm;
    const float* gq; const float* gk;
    const float* rope;     // [max_context][hd] interleaved (cos, sin)
    void* kpool; void* vpool;          // this layer's pages: [page][kv_heads][16][hd]
    const int* page_table; int pt_stride;
    float* qbuf; float* gbuf;          // [B][nq]
    // LM head epilogue
    float* part_val; int* part_idx;    // [B][gridDim.x]
    int* ticket;                       // [gridDim.y]
    int do_pick;                       // greedy pick + advance in the last CTA
};

// Rows a warp streams per pass and 16-byte vectors per row it fetches BEFORE waiting for the
// predecessor kernel: 2 rows x 4 vectors at batch tile 1 (latency; deeper preloads cost occupancy
// and measured slower), 4 rows x 2 otherwise.
template <int BT> struct GemvShape {
    static constexpr int RW = (BT == 1) ? 2 : 4;
    static constexpr int PRE = (BT == 1) ? 4 : 2;
};

template <typename T, int RW>
__device__ __forceinline__ void row_pointers(const T* __restrict__ W, int N, int K, int row0, const T* (&wrow)[RW]) {
#pragma unroll
    for (int r = 0; r < RW; ++r) {
        int row = row0 + r;
        if (row > N - 1) row = N - 1;     // tail rows are computed on a duplicate and not stored
        wrow[r] = W + (size_t)row * K;
    }
}

template <typename T, int RW, int PRE>
__device__ __forceinline__ void preload_rows(const T* const (&wrow)[RW], int nvec, int lane, uint4 (&pre)[RW][PRE]) {
    constexpr int EPV = Elem<T>::EPV;
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
        const int v = lane + 32 * i;
#pragma unroll
        for (int r = 0; r < RW; ++r)
            pre[r][i] = v < nvec ? __ldg(reinterpret_cast<const uint4*>(wrow[r] + (size_t)v * EPV)) : make_uint4(0, 0, 0, 0);
    }
}

template <typename T, int BT, int RW>
__device__ __forceinline__ void fma_vec(const uint4 (&raw)[RW], const float* __restrict__ xs, int xs_stride, int v, int nvec,
                                        float (&acc)[RW][BT]) {
    constexpr int EPV = Elem<T>::EPV;
    float w[RW][EPV];
#pragma unroll
    for (int r = 0; r < RW; ++r) Elem<T>::unpack(raw[r], w[r]);
#pragma unroll
    for (int b = 0; b < BT; ++b) {
        const float4* xp = reinterpret_cast<const float4*>(xs + (size_t)b * xs_stride);
        float xv[EPV];
#pragma unroll
        for (int q = 0; q < EPV / 4; ++q) {
            float4 t = xp[q * nvec + v];                // [EPV/4][nvec] layout, see xs_f4_index
            xv[4 * q] = t.x; xv[4 * q + 1] = t.y; xv[4 * q + 2] = t.z; xv[4 * q + 3] = t.w;
        }
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int e = 0; e < EPV; ++e) acc[r][b] = fmaf(w[r][e], xv[e], acc[r][b]);
    }
}

// acc[r][b] += W[row r] . xs[b] over vectors [first_vec*32 + lane, nvec) of the rows
template <typename T, int BT, int RW>
__device__ __forceinline__ void warp_rows_dot(const T* const (&wrow)[RW], int nvec, int first_iter,
                                              const float* __restrict__ xs, int xs_stride, int lane,
                                              float (&acc)[RW][BT]) {
    constexpr int EPV = Elem<T>::EPV;
#pragma unroll 2
    for (int v = lane + 32 * first_iter; v < nvec; v += 32) {
        uint4 raw[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) raw[r] = __ldg(reinterpret_cast<const uint4*>(wrow[r] + (size_t)v * EPV));
        fma_vec<T, BT, RW>(raw, xs, xs_stride, v, nvec, acc);
    }
}

template <typename T, int BT, int RW, int PRE>
__device__ __forceinline__ void consume_preloaded(const uint4 (&pre)[RW][PRE], int nvec, const float* __restrict__ xs,
                                                  int xs_stride, int lane, float (&acc)[RW][BT]) {
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
        const int v = lane + 32 * i;
        if (v < nvec) {
            uint4 raw[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r) raw[r] = pre[r][i];
            fma_vec<T, BT, RW>(raw, xs, xs_stride, v, nvec, acc);
        }
    }
}

template <typename T, typename T2, typename KVT, int BT, int MODE>
__global__ void __launch_bounds__(256) gemv_kernel(StepCtl c, GemvParams p) {
    constexpr int RWF = GemvShape<BT>::RW;                           // weight rows per warp pass
    constexpr int RW = (MODE == GEMV_SWIGLU) ? RWF / 2 : RWF;        // output rows per warp pass
    constexpr int PRE = GemvShape<BT>::PRE;
    constexpr int EPV = Elem<T>::EPV;
    extern __shared__ __align__(16) float smem[];
    const int K = p.K, Kp = p.Kp, R = p.R;
    float* xs = smem;                                  // [BT][K]
    float* xs2 = xs + (size_t)BT * K;                  // [BT][Kp]
    float* outs = xs2 + (size_t)BT * Kp;               // [BT][R]
    float* rs = outs + (size_t)BT * R;                 // [BT]
    float* red = rs + BT;                              // [8][BT]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    const int b0 = blockIdx.y * BT;
    const int row0 = blockIdx.x * R;
    const int nvec = K / EPV;
    const T* W = reinterpret_cast<const T*>(p.W);
    const T* Wb = reinterpret_cast<const T*>(p.Wb);

    pdl_launch_dependents();
    // ---- weights of the first pass: fetched before the predecessor's results are needed ---
    const T* wrow[RW];
    const T* wrow_b[RW];
    uint4 pre[RW][PRE], pre_b[RW][PRE];
    const bool first_pass = warp * RW < R;
    if (first_pass) {
        row_pointers<T, RW>(W, p.N, K, row0 + warp * RW, wrow);
        preload_rows<T, RW, PRE>(wrow, nvec, lane, pre);
        if (MODE == GEMV_SWIGLU) {
            row_pointers<T, RW>(Wb, p.N, K, row0 + warp * RW, wrow_b);
            preload_rows<T, RW, PRE>(wrow_b, nvec, lane, pre_b);
        }
    }
    pdl_wait();

    // ---- prologue: stage (and RMS-normalise) the activations of the tile -------------
    // Reference: getRMSColSums + applyRMSNorm, inference.cu:24-50, :83-95 -
    // r = sqrt(mean(x^2) + eps); x / r, then times the gain.
    {
        float ss[BT];
#pragma unroll
        for (int b = 0; b < BT; ++b) {
            const int bg = min(b0 + b, c.B - 1);
            const float4* xr = reinterpret_cast<const float4*>(p.xin + (size_t)bg * K);
            float4* xd = reinterpret_cast<float4*>(xs + (size_t)b * K);
            float a = 0.f;
            for (int k = tid; k < K / 4; k += blockDim.x) {
                float4 v = xr[k];
                xd[xs_f4_index<EPV>(k, nvec)] = v;
                a = fmaf(v.x, v.x, a); a = fmaf(v.y, v.y, a); a = fmaf(v.z, v.z, a); a = fmaf(v.w, v.w, a);
            }
            ss[b] = a;
            if (Kp > 0) {
                const int t = c.tok[bg];
                const T2* trow = reinterpret_cast<const T2*>(p.Ptab) + (size_t)t * Kp;
                for (int k = tid; k < Kp; k += blockDim.x)
                    xs2[(size_t)b * Kp + xs_index<Elem<T2>::EPV>(k, Kp / Elem<T2>::EPV)] = Elem<T2>::get(trow, k);
            }
        }
        if (p.do_norm) {
#pragma unroll
            for (int b = 0; b < BT; ++b) {
                float a = warp_sum(ss[b]);
                if (lane == 0) red[warp * BT + b] = a;
            }
            __syncthreads();
#pragma unroll
            for (int b = 0; b < BT; ++b) {
                float tot = 0.f;
                for (int w = 0; w < nw; ++w) tot += red[w * BT + b];
                const float r = sqrtf(tot / (float)K + p.eps);
                float4* xd = reinterpret_cast<float4*>(xs + (size_t)b * K);
                const float4* gp = reinterpret_cast<const float4*>(p.gain);
                for (int k = tid; k < K / 4; k += blockDim.x) {
                    const int d = xs_f4_index<EPV>(k, nvec);
                    float4 v = xd[d], g = gp[k];
                    v.x = (v.x / r) * g.x; v.y = (v.y / r) * g.y; v.z = (v.z / r) * g.z; v.w = (v.w / r) * g.w;
                    xd[d] = v;
                }
            }
        }
    }
    __syncthreads();

    // ---- main loop: RW output rows per warp pass ---------------------------------------
    for (int rb = warp * RW; rb < R; rb += nw * RW) {
        const bool pre_ok = rb == warp * RW;            // the first pass has its first vectors in registers
        float acc[RW][BT];
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int b = 0; b < BT; ++b) acc[r][b] = 0.f;
        if (!pre_ok) row_pointers<T, RW>(W, p.N, K, row0 + rb, wrow);
        if (pre_ok) consume_preloaded<T, BT, RW, PRE>(pre, nvec, xs, K, lane, acc);
        warp_rows_dot<T, BT, RW>(wrow, nvec, pre_ok ? PRE : 0, xs, K, lane, acc);
        if (MODE == GEMV_SWIGLU) {
            float accb[RW][BT];
#pragma unroll
            for (int r = 0; r < RW; ++r)
#pragma unroll
                for (int b = 0; b < BT; ++b) accb[r][b] = 0.f;
            if (!pre_ok) row_pointers<T, RW>(Wb, p.N, K, row0 + rb, wrow_b);
            if (pre_ok) consume_preloaded<T, BT, RW, PRE>(pre_b, nvec, xs, K, lane, accb);
            warp_rows_dot<T, BT, RW>(wrow_b, nvec, pre_ok ? PRE : 0, xs, K, lane, accb);
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                int row = min(row0 + rb + r, p.N - 1);
                float sa = p.wscale ? p.wscale[row] : 1.f, sb = p.wscale_b ? p.wscale_b[row] : 1.f;
#pragma unroll
                for (int b = 0; b < BT; ++b) {
                    float g = warp_sum(acc[r][b]) * sa;
                    float u = warp_sum(accb[r][b]) * sb;
                    // applySiluToFFN + hadamardMultiplyFFN, inference.cu:262-281
                    if (lane == 0 && rb + r < R) outs[(size_t)b * R + rb + r] = (g / (1.0f + expf(-g))) * u;
                }
            }
        } else {
            if (Kp > 0) {
                float acc2[RW][BT];
#pragma unroll
                for (int r = 0; r < RW; ++r)
#pragma unroll
                    for (int b = 0; b < BT; ++b) acc2[r][b] = 0.f;
                const T2* prow[RW];
                row_pointers<T2, RW>(reinterpret_cast<const T2*>(p.P), p.N, Kp, row0 + rb, prow);
                warp_rows_dot<T2, BT, RW>(prow, Kp / Elem<T2>::EPV, 0, xs2, Kp, lane, acc2);
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    int row = min(row0 + rb + r, p.N - 1);
                    float sa = p.wscale ? p.wscale[row] : 1.f;
#pragma unroll
                    for (int b = 0; b < BT; ++b) acc[r][b] = acc[r][b] * sa + acc2[r][b];
                }
            } else if (p.wscale) {
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    float sa = p.wscale[min(row0 + rb + r, p.N - 1)];
#pragma unroll
                    for (int b = 0; b < BT; ++b) acc[r][b] *= sa;
                }
            }
#pragma unroll
            for (int r = 0; r < RW; ++r)
#pragma unroll
                for (int b = 0; b < BT; ++b) {
                    float v = warp_sum(acc[r][b]);
                    if (lane == 0 && rb + r < R) outs[(size_t)b * R + rb + r] = v;
                }
        }
    }
    __syncthreads();

    // ---- epilogues -----------------------------------------------------------------------
    if (MODE == GEMV_RAW || MODE == GEMV_SWIGLU || MODE == GEMV_RESID) {
        for (int i = tid; i < BT * R; i += blockDim.x) {
            int b = i / R, r = i - b * R;
            int bg = b0 + b, row = row0 + r;
            if (row < p.N && seq_active(c, bg)) {
                float v = outs[(size_t)b * R + r];
                // addResidualToOutputProj / addResidualToFFN, inference.cu:252-260, :283-291
                if (MODE == GEMV_RESID) v += p.resid[(size_t)bg * p.N + row];
                p.y[(size_t)bg * p.N + row] = v;
            }
        }
    } else if (MODE == GEMV_QKV) {
        // Segment of this CTA (R divides every segment and the head size).
        const int seg_q = p.nq, seg_k = p.nq + p.nk, seg_v = seg_k + p.nv;
        const int hd = p.hd;
        int seg = row0 < seg_q ? 0 : (row0 < seg_k ? 1 : (row0 < seg_v ? 2 : 3));
        if (p.qk_norm && seg < 2) {
            // getRMSColSumsAcrossHeads + applyRMSNormAcrossHeads, inference.cu:52-81, :97-111
            // (R == hd here: the CTA holds one whole head)
            for (int b = warp; b < BT; b += nw) {
                float ss = 0.f;
                for (int r = lane; r < R; r += 32) { float v = outs[(size_t)b * R + r]; ss = fmaf(v, v, ss); }
                ss = warp_sum(ss);
                if (lane == 0) rs[b] = sqrtf(ss / (float)hd + p.eps);
            }
            __syncthreads();
        }
        KVT* kpool = reinterpret_cast<KVT*>(p.kpool);
        KVT* vpool = reinterpret_cast<KVT*>(p.vpool);
        for (int i = tid; i < BT * (R / 2); i += blockDim.x) {
            int b = i / (R / 2), pr = i - b * (R / 2);
            int bg = b0 + b;
            if (!seq_active(c, bg)) continue;
            int r = 2 * pr, row = row0 + r;
            float a = outs[(size_t)b * R + r], cc = outs[(size_t)b * R + r + 1];
            int pos = c.pos[bg];
            if (seg < 2) {
                int srow = (seg == 0) ? row : row - seg_q;          // row inside q or k
                if (p.qk_norm) {
                    const float* g = (seg == 0) ? p.gq : p.gk;
                    a = (a / rs[b]) * g[srow];
                    cc = (cc / rs[b]) * g[srow + 1];
                }
                // applyRoPE, inference.cu:113-134: adjacent pair, table row = position
                int e = srow % hd;
                float cs = p.rope[(size_t)pos * hd + e], sn = p.rope[(size_t)pos * hd + e + 1];
                float ra = cs * a - sn * cc, rc = sn * a + cs * cc;
                if (seg == 0) {
                    p.qbuf[(size_t)bg * p.nq + srow] = ra;
                    p.qbuf[(size_t)bg * p.nq + srow + 1] = rc;
                } else {
                    int kvh = srow / hd;
                    int page = p.page_table[(size_t)bg * p.pt_stride + pos / kKvBlock];
                    size_t off = (((size_t)page * p.kv_heads + kvh) * kKvBlock + (pos % kKvBlock)) * hd + e;
                    Elem<KVT>::put(kpool, off, ra);
                    Elem<KVT>::put(kpool, off + 1, rc);
                }
            } else if (seg == 2) {
                int srow = row - seg_k;
                int kvh = srow / hd, e = srow % hd;
                int page = p.page_table[(size_t)bg * p.pt_stride + pos / kKvBlock];
                size_t off = (((size_t)page * p.kv_heads + kvh) * kKvBlock + (pos % kKvBlock)) * hd + e;
                Elem<KVT>::put(vpool, off, a);
                Elem<KVT>::put(vpool, off + 1, cc);
            } else {
                // sigmoid of the gate projection, inference.cu:248
                int srow = row - seg_v;
                p.gbuf[(size_t)bg * p.ng + srow] = 1.0f / (1.0f + expf(-a));
                p.gbuf[(size_t)bg * p.ng + srow + 1] = 1.0f / (1.0f + expf(-cc));
            }
        }
    } else if (MODE == GEMV_LMHEAD) {
        // Logits (vocabScores_DEVICE, inference.cu:720-743) and the greedy pick that the
        // reference does on the host with qsort (inference_orchestrator.cu:77-84, :112).
        for (int i = tid; i < BT * R; i += blockDim.x) {
            int b = i / R, r = i - b * R;
            int bg = b0 + b, row = row0 + r;
            if (row < p.N && seq_active(c, bg)) p.y[(size_t)bg * p.N + row] = outs[(size_t)b * R + r];
        }
        const int nparts = gridDim.x;
        for (int b = warp; b < BT; b += nw) {
            int bg = b0 + b;
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int r = lane; r < R; r += 32) {
                int row = row0 + r;
                if (row < p.N) {
                    float v = outs[(size_t)b * R + r];
                    if (v > bv || (v == bv && row < bi)) { bv = v; bi = row; }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0 && bg < c.B) {
                p.part_val[(size_t)bg * nparts + blockIdx.x] = bv;
                p.part_idx[(size_t)bg * nparts + blockIdx.x] = bi;
            }
        }
        // Last CTA of this batch tile reduces the partials (ticket pattern; no spinning).
        __shared__ int is_last;
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            int t = atomicAdd(&p.ticket[blockIdx.y], 1);
            is_last = (t == nparts - 1);
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            for (int b = warp; b < BT; b += nw) {
                int bg = b0 + b;
                if (!seq_active(c, bg)) continue;          // warp-uniform
                float bv = -INFINITY; int bi = 0x7fffffff;
                for (int q = lane; q < nparts; q += 32) {
                    float v = __ldcg(&p.part_val[(size_t)bg * nparts + q]);
                    int ix = __ldcg(&p.part_idx[(size_t)bg * nparts + q]);
                    if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
                }
                if (lane == 0 && p.do_pick) advance_seq(c, bg, bi);
            }
            if (tid == 0) p.ticket[blockIdx.y] = 0;        // ready for the next step
        }
    }
}

// ------------------------------------------------------------------------------------
// Split-K flash-decode over the paged KV cache, with the split combine and the query
// gating folded into the last-arriving CTA of each (sequence, kv head).
//
// Reference ops replaced: K^T Q GEMM, getHeadDimScaledMaskedAttn, the max / sum / apply
// softmax kernels, V P GEMM, applyGatingToValueScaledAttnPostSoftmax
// (inference.cu:510-579, kernels :136-250). Scores are divided by sqrtf(head_dim) as there.
// grid = (splits, kv_heads, B), block = 128.
// ------------------------------------------------------------------------------------
struct AttnParams {
    const void* kpool; const void* vpool;     // [page][kv_heads][16][hd]
    const int* page_table; int pt_stride;
    const float* qbuf;      // [B][heads*hd]
    const float* gbuf;      // [B][heads*hd] sigmoid gates or null
    float* abuf;            // [B][heads*hd]
    bf16_t* abuf16;         // same values as the bf16 operand of a tensor-core O projection, or null
    float* part;            // [B][heads][splits][hd+2]
    int* ticket;            // [B * gridDim.y]
    int heads, kv_heads;
    int hg;                 // CTAs per kv head along grid.y: each takes G of the kv head's query heads
    // A caller-owned page table (the operator entry points) is not trusted: with num_pages > 0 a sequence
    // whose position needs more than pt_stride pages is skipped (code 4 in *err) and a page id outside
    // [0, num_pages) is replaced by page 0 (code 5), so that nothing outside the caller's buffers is read.
    // The session passes 0: its own allocator filled the table.
    int num_pages;
    int* err;
    // A split is worth its partials and the combine only with enough positions in it: a sequence uses
    // min(grid splits, pages / min_pages_per_split) of them. 1 = every page may be a split.
    int min_pages_per_split;
};

template <typename KVT, int HD, int G>
__global__ void __launch_bounds__(128) attn_decode_kernel(StepCtl c, AttnParams p) {
    constexpr int EPL = 16 / sizeof(KVT);          // elements per lane per row
    constexpr int LPR = HD / EPL;                  // lanes per row
    constexpr int PPI = 32 / LPR;                  // positions per warp iteration
    constexpr int NW = 4;
    static_assert(LPR <= 32 && PPI >= 1, "head_dim too large for one warp row");
    // With many query heads per kv head one CTA would hold all their accumulators (160+ registers,
    // no room for a second chunk of loads in flight): hg CTAs share a kv head instead, G heads each;
    // the K/V rows they re-read come from L2.
    const int b = blockIdx.z, kvh = blockIdx.y / p.hg, split = blockIdx.x;
    const int tslot = b * (int)gridDim.y + (int)blockIdx.y;
    pdl_launch_dependents();
    pdl_wait();                                    // q and this step's K/V row come from the projection kernel
    if (!seq_active(c, b)) return;                 // uniform for all CTAs of this sequence
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int lr = lane % LPR, grp = lane / LPR;
    const int pos = c.pos[b];
    const int ctx = pos + 1;
    const int npages = (ctx + kKvBlock - 1) / kKvBlock;
    // The grid is sized for the longest context; a split needs at least one page, and the CTAs
    // beyond the page count leave at once (fewer partials for the combine to read). Every CTA of a
    // (sequence, kv head) computes the same S.
    if (p.num_pages > 0 && npages > p.pt_stride) {   // uniform for all CTAs of this sequence
        if (threadIdx.x == 0) atomicExch(p.err, 4);
        return;
    }
    const int S = max(1, min((int)gridDim.x, npages / max(1, p.min_pages_per_split)));
    const int SG = (int)gridDim.x;                 // stride of the partial buffer: fixed by the grid, not by S
    if (split >= S) return;
    const int pps = (npages + S - 1) / S;
    const int pg_begin = split * pps, pg_end = min(npages, pg_begin + pps);

    __shared__ float sq[G][HD];
    __shared__ float sred[NW][G][HD + 2];
    const int h0 = kvh * G * p.hg + ((int)blockIdx.y % p.hg) * G;
    for (int i = tid; i < G * HD; i += blockDim.x)
        sq[i / HD][i % HD] = p.qbuf[((size_t)b * p.heads + h0) * HD + i];
    __syncthreads();

    float q[G][EPL];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < EPL; ++e) q[g][e] = sq[g][lr * EPL + e];

    float m[G], l[G], acc[G][EPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = kNegBig; l[g] = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = 0.f;
    }
    const float inv_div = sqrtf((float)HD);
    const KVT* kpool = reinterpret_cast<const KVT*>(p.kpool);
    const KVT* vpool = reinterpret_cast<const KVT*>(p.vpool);

    // This warp's pages: pg_begin + warp + NW * i. Lane i holds the pool index of the i-th one
    // (refreshed every 32 pages), so that the page loop does not start with a dependent load.
    constexpr int ITERS = kKvBlock / PPI;
    constexpr int CH = ITERS < 4 ? ITERS : 4;      // positions per lane group handled together
    const int* pt = p.page_table + (size_t)b * p.pt_stride;
    const int span = pg_end - pg_begin - warp;
    const int npw = span > 0 ? (span + NW - 1) / NW : 0;
    int pidx = 0;
    constexpr int CPP = ITERS / CH;                // chunks per page
    const int nq = npw * CPP;                      // this warp's chunks, in order
    // All loads of a chunk first, then the scores of its positions (independent of one another), one
    // rescale of the running sums and one exponential per position.
    auto load_chunk = [&](int qi, uint4* kk, uint4* vv4, int& cnt, int& c0) {
        const int i = qi / CPP;
        c0 = (qi - i * CPP) * CH;
        if (c0 == 0 && (i & 31) == 0) {
            const int ii = i + lane;
            pidx = ii < npw ? pt[pg_begin + warp + NW * ii] : 0;
            if (p.num_pages > 0 && (unsigned)pidx >= (unsigned)p.num_pages) {
                atomicExch(p.err, 5);
                pidx = 0;
            }
        }
        const int pg = pg_begin + warp + NW * i;
        const int page = __shfl_sync(0xffffffffu, pidx, i & 31);
        cnt = min(kKvBlock, ctx - pg * kKvBlock);
        const size_t base = ((size_t)page * p.kv_heads + kvh) * kKvBlock * HD;
#pragma unroll
        for (int u = 0; u < CH; ++u) {
            const int j = (c0 + u) * PPI + grp;
            kk[u] = make_uint4(0, 0, 0, 0);
            vv4[u] = make_uint4(0, 0, 0, 0);
            if (j < cnt) {
                kk[u] = __ldcg(reinterpret_cast<const uint4*>(kpool + base + (size_t)j * HD + lr * EPL));
                vv4[u] = __ldcg(reinterpret_cast<const uint4*>(vpool + base + (size_t)j * HD + lr * EPL));
            }
        }
    };
    auto use_chunk = [&](const uint4* kk, const uint4* vv4, int cnt, int c0) {
        float sv[G][CH];
#pragma unroll
        for (int u = 0; u < CH; ++u) {
            const bool valid = (c0 + u) * PPI + grp < cnt;
            float kv[EPL];
            Elem<KVT>::unpack(kk[u], kv);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float sdot = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) sdot = fmaf(q[g][e], kv[e], sdot);
#pragma unroll
                for (int o = LPR / 2; o > 0; o >>= 1) sdot += __shfl_xor_sync(0xffffffffu, sdot, o);
                sv[g][u] = valid ? sdot / inv_div : kNegBig;
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float mn = m[g];
#pragma unroll
            for (int u = 0; u < CH; ++u) mn = fmaxf(mn, sv[g][u]);
            const float sc = expf(m[g] - mn);
            l[g] *= sc;
#pragma unroll
            for (int e = 0; e < EPL; ++e) acc[g][e] *= sc;
#pragma unroll
            for (int u = 0; u < CH; ++u) {
                const bool valid = (c0 + u) * PPI + grp < cnt;
                sv[g][u] = valid ? expf(sv[g][u] - mn) : 0.f;
                l[g] += sv[g][u];
            }
            m[g] = mn;
        }
#pragma unroll
        for (int u = 0; u < CH; ++u) {
            float vv[EPL];
            Elem<KVT>::unpack(vv4[u], vv);
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[g][e] = fmaf(sv[g][u], vv[e], acc[g][e]);
        }
    };
    if (G <= 2) {
        // few heads per CTA leave registers for a second chunk: the next chunk's loads are in flight
        // while the current one is used (twice the bytes in flight per warp)
        uint4 ka[CH], va[CH], kb[CH], vb[CH];
        int cnt_a = 0, c0_a = 0, cnt_b = 0, c0_b = 0;
        if (nq > 0) load_chunk(0, ka, va, cnt_a, c0_a);
        for (int qi = 0; qi < nq; qi += 2) {
            if (qi + 1 < nq) load_chunk(qi + 1, kb, vb, cnt_b, c0_b);
            use_chunk(ka, va, cnt_a, c0_a);
            if (qi + 1 < nq) {
                if (qi + 2 < nq) load_chunk(qi + 2, ka, va, cnt_a, c0_a);
                use_chunk(kb, vb, cnt_b, c0_b);
            }
        }
    } else {
        uint4 ka[CH], va[CH];
        int cnt_a = 0, c0_a = 0;
        for (int qi = 0; qi < nq; ++qi) {
            load_chunk(qi, ka, va, cnt_a, c0_a);
            use_chunk(ka, va, cnt_a, c0_a);
        }
    }
    // merge the PPI lane groups of the warp
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int o = LPR; o < 32; o <<= 1) {
            float mo = __shfl_xor_sync(0xffffffffu, m[g], o);
            float lo = __shfl_xor_sync(0xffffffffu, l[g], o);
            float mn = fmaxf(m[g], mo);
            float sa = expf(m[g] - mn), sb = expf(mo - mn);
            l[g] = l[g] * sa + lo * sb;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                float ao = __shfl_xor_sync(0xffffffffu, acc[g][e], o);
                acc[g][e] = acc[g][e] * sa + ao * sb;
            }
            m[g] = mn;
        }
        if (grp == 0) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) sred[warp][g][lr * EPL + e] = acc[g][e];
            if (lr == 0) { sred[warp][g][HD] = m[g]; sred[warp][g][HD + 1] = l[g]; }
        }
    }
    __syncthreads();
    // merge the warps; thread t < HD owns output dim t
    for (int i = tid; i < G * HD; i += blockDim.x) {
        int g = i / HD, e = i % HD;
        float mn = kNegBig;
#pragma unroll
        for (int w = 0; w < NW; ++w) mn = fmaxf(mn, sred[w][g][HD]);
        float lt = 0.f, at = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            float sc = expf(sred[w][g][HD] - mn);
            lt += sred[w][g][HD + 1] * sc;
            at += sred[w][g][e] * sc;
        }
        int h = h0 + g;
        if (S == 1) {
            float o = at / lt;
            if (p.gbuf) o *= p.gbuf[((size_t)b * p.heads + h) * HD + e];
            p.abuf[((size_t)b * p.heads + h) * HD + e] = o;
            if (p.abuf16) p.abuf16[((size_t)b * p.heads + h) * HD + e] = __float2bfloat16_rn(o);
        } else {
            float* pp = p.part + (((size_t)b * p.heads + h) * SG + split) * (HD + 2);
            pp[e] = at;
            if (e == 0) { pp[HD] = mn; pp[HD + 1] = lt; }
        }
    }
    if (S == 1) return;
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int t = atomicAdd(&p.ticket[tslot], 1);
        is_last = (t == S - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // Combine: one warp per head turns the splits' (max, sum) pairs into normalised weights once;
    // then every thread accumulates its output elements with independent loads.
    __shared__ float wsm[G][64];
    for (int g = warp; g < G; g += NW) {
        const float* pp = p.part + ((size_t)b * p.heads + h0 + g) * SG * (HD + 2);
        float m0 = kNegBig, l0 = 0.f, m1 = kNegBig, l1 = 0.f;
        if (lane < S) { m0 = __ldcg(pp + (size_t)lane * (HD + 2) + HD); l0 = __ldcg(pp + (size_t)lane * (HD + 2) + HD + 1); }
        if (lane + 32 < S) { m1 = __ldcg(pp + (size_t)(lane + 32) * (HD + 2) + HD); l1 = __ldcg(pp + (size_t)(lane + 32) * (HD + 2) + HD + 1); }
        float mx = fmaxf(m0, m1);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float w0 = expf(m0 - mx), w1 = expf(m1 - mx);
        const float lt = warp_sum(l0 * w0 + l1 * w1);
        wsm[g][lane] = w0 / lt;
        wsm[g][lane + 32] = w1 / lt;
    }
    __syncthreads();
    for (int i = tid; i < G * HD; i += blockDim.x) {
        int g = i / HD, e = i % HD, h = h0 + g;
        const float* pp = p.part + ((size_t)b * p.heads + h) * SG * (HD + 2) + e;
        float o = 0.f;
#pragma unroll 4
        for (int s = 0; s < S; ++s) o = fmaf(wsm[g][s], __ldcg(pp + (size_t)s * (HD + 2)), o);
        if (p.gbuf) o *= p.gbuf[((size_t)b * p.heads + h) * HD + e];
        p.abuf[((size_t)b * p.heads + h) * HD + e] = o;
        if (p.abuf16) p.abuf16[((size_t)b * p.heads + h) * HD + e] = __float2bfloat16_rn(o);
    }
    if (tid == 0) p.ticket[tslot] = 0;
}

// ------------------------------------------------------------------------------------
// Gated delta-net recurrent update (no counterpart in the reference):
//   S <- alpha S ; u = S k^ ; S <- S + beta (v - u) k^T ; o = S q^
// done row by row: a warp owns rows of S (dk floats each, spread over its lanes), so the
// state is read once and written once per step; the two dot products per row are
// warp-shuffle reductions. q^,k^ (L2-normalised), beta, alpha are prepared per CTA in
// shared memory from the raw projection outputs.
// raw layout per sequence: [q (H*dk) | k (H*dk) | v (H*dv) | beta (H) | alpha (H)]
// grid = (dv / rows_per_cta, H, B), block = 256 (8 warps x 4 rows).
// ------------------------------------------------------------------------------------
template <int DK>
__global__ void __launch_bounds__(256) delta_net_kernel(StepCtl c, const float* __restrict__ raw, int raw_stride,
                                                        float* __restrict__ state, int H, int dv,
                                                        float* __restrict__ abuf, bf16_t* __restrict__ abuf16, float l2_eps) {
    constexpr int EPL = DK / 32;
    constexpr int ROWS_PER_WARP = 4;
    const int b = blockIdx.z, h = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();
    // The state rows do not depend on this step's projections: fetch them before waiting.
    const int row0 = blockIdx.x * (8 * ROWS_PER_WARP) + warp * ROWS_PER_WARP;
    float* Sh = state + ((size_t)b * H + h) * (size_t)dv * DK;
    float s[ROWS_PER_WARP][EPL];
#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; ++i) {
        int row = row0 + i;
        if (row < dv) {
            // one vector load per lane and row: a warp reads the row's DK floats as one contiguous piece (element by
            // element, each instruction touched every sector of the row again: four L2 requests per sector at DK = 128)
            if (EPL == 4) {
                const float4 t = __ldcg(reinterpret_cast<const float4*>(&Sh[(size_t)row * DK + lane * 4]));
                s[i][0] = t.x; s[i][1] = t.y; s[i][2 % EPL] = t.z; s[i][3 % EPL] = t.w;
            } else {
                const float2 t = __ldcg(reinterpret_cast<const float2*>(&Sh[(size_t)row * DK + lane * 2]));
                s[i][0] = t.x; s[i][1] = t.y;
            }
        } else {
#pragma unroll
            for (int e = 0; e < EPL; ++e) s[i][e] = 0.f;
        }
    }
    pdl_wait();
    if (!seq_active(c, b)) return;
    __shared__ float sq[DK], sk[DK];
    __shared__ float sgate[2];
    const float* r = raw + (size_t)b * raw_stride;
    const float* rq = r + (size_t)h * DK;
    const float* rk = r + (size_t)H * DK + (size_t)h * DK;
    const float* rv = r + (size_t)2 * H * DK + (size_t)h * dv;
    if (warp < 2) {
        const float* src = warp == 0 ? rq : rk;
        float v[EPL], ss = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) { v[e] = src[lane * EPL + e]; ss = fmaf(v[e], v[e], ss); }
        ss = warp_sum(ss);
        float n = sqrtf(ss + l2_eps);
        float* dst = warp == 0 ? sq : sk;
#pragma unroll
        for (int e = 0; e < EPL; ++e) dst[lane * EPL + e] = v[e] / n;
    } else if (warp == 2 && lane < 2) {
        float g = r[(size_t)2 * H * DK + (size_t)H * dv + (size_t)lane * H + h];
        sgate[lane] = 1.0f / (1.0f + expf(-g));
    }
    __syncthreads();
    const float beta = sgate[0], alpha = sgate[1];
    float qn[EPL], kn[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) { qn[e] = sq[lane * EPL + e]; kn[e] = sk[lane * EPL + e]; }
#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; ++i) {
        int row = row0 + i;
        float d1 = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) { s[i][e] *= alpha; d1 = fmaf(s[i][e], kn[e], d1); }
        d1 = warp_sum(d1);
        float vi = row < dv ? rv[row] : 0.f;
        float cf = beta * (vi - d1);
        float d2 = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) { s[i][e] = fmaf(cf, kn[e], s[i][e]); d2 = fmaf(s[i][e], qn[e], d2); }
        d2 = warp_sum(d2);
        if (row < dv) {
            if (EPL == 4) *reinterpret_cast<float4*>(&Sh[(size_t)row * DK + lane * 4]) = make_float4(s[i][0], s[i][1], s[i][2 % EPL], s[i][3 % EPL]);
            else *reinterpret_cast<float2*>(&Sh[(size_t)row * DK + lane * 2]) = make_float2(s[i][0], s[i][1]);
            if (lane == 0) {
                abuf[((size_t)b * H + h) * dv + row] = d2;
                if (abuf16) abuf16[((size_t)b * H + h) * dv + row] = __float2bfloat16_rn(d2);
            }
        }
    }
}

// The same update for prompt columns: the columns of a chunk are consecutive tokens of one or
// several sequences (seq_of[col], grouped by sequence, positions ascending inside a sequence), and
// the recurrence S_t = f(S_{t-1}) runs over a sequence's columns in order.
//
// delta_cols_norm_kernel first turns the raw projections of every (column, head) into what the
// recurrence consumes - L2-normalised q and k, sigmoid gates - in place, in parallel over columns.
// grid = (H, columns), block = 64.
template <int DK>
__global__ void __launch_bounds__(64) delta_cols_norm_kernel(StepCtl c, float* __restrict__ raw, int raw_stride, int H, int dv,
                                                             float l2_eps) {
    constexpr int EPL = DK / 32;
    const int h = blockIdx.x, col = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_launch_dependents();
    pdl_wait();
    if (!seq_active(c, col)) return;
    float* r = raw + (size_t)col * raw_stride;
    float* vec = r + (size_t)(warp == 0 ? 0 : H) * DK + (size_t)h * DK;       // q heads, then k heads
    float v[EPL], ss = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) { v[e] = vec[lane * EPL + e]; ss = fmaf(v[e], v[e], ss); }
    ss = warp_sum(ss);
    const float n = sqrtf(ss + l2_eps);
#pragma unroll
    for (int e = 0; e < EPL; ++e) vec[lane * EPL + e] = v[e] / n;
    if (warp == 0 && lane < 2) {
        float* g = r + (size_t)2 * H * DK + (size_t)H * dv + (size_t)lane * H + h;       // beta[H] then alpha[H]
        *g = 1.0f / (1.0f + expf(-*g));
    }
}

// The recurrence itself. A warp owns 4 rows of one head's state and keeps them in registers
// across the columns of a sequence; the state is read and written once per sequence and chunk, and
// the next column's q, k, v and gates are requested while the current one is applied (no block
// barrier in the loop). The sequences of a chunk are independent: CTA z serves the run of columns
// that starts at column z, if a sequence starts there, and leaves otherwise.
// grid = (ceil(dv / 32), H, columns), block = 256.
template <int DK>
__global__ void __launch_bounds__(256) delta_net_cols_kernel(StepCtl c, const int* __restrict__ seq_of, int n_cols,
                                                             const float* __restrict__ raw, int raw_stride, float* __restrict__ state,
                                                             int H, int dv, float* __restrict__ abuf, bf16_t* __restrict__ abuf16) {
    constexpr int EPL = DK / 32;
    constexpr int ROWS_PER_WARP = 4;
    const int h = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();
    pdl_wait();
    const int row0 = blockIdx.x * (8 * ROWS_PER_WARP) + warp * ROWS_PER_WARP;
    const int first = blockIdx.z;
    if (first >= n_cols || !seq_active(c, first)) return;
    const int cur = seq_of[first];
    if (first > 0 && seq_active(c, first - 1) && seq_of[first - 1] == cur) return;     // not the start of a run
    if (row0 >= dv) return;
    float* Sh = state + ((size_t)cur * H + h) * (size_t)dv * DK;
    float s[ROWS_PER_WARP][EPL];
#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; ++i) {
#pragma unroll
        for (int e = 0; e < EPL; ++e) s[i][e] = 0.f;
        if (row0 + i < dv) {                     // one vector load per lane and row, as in delta_net_kernel
            if (EPL == 4) {
                const float4 t = __ldcg(reinterpret_cast<const float4*>(&Sh[(size_t)(row0 + i) * DK + lane * 4]));
                s[i][0] = t.x; s[i][1] = t.y; s[i][2 % EPL] = t.z; s[i][3 % EPL] = t.w;
            } else {
                const float2 t = __ldcg(reinterpret_cast<const float2*>(&Sh[(size_t)(row0 + i) * DK + lane * 2]));
                s[i][0] = t.x; s[i][1] = t.y;
            }
        }
    }
    // one column's inputs: normalised q and k of the head (EPL values per lane), the warp's 4 values
    // of v, the two gates
    float qn[EPL], kn[EPL], vr[ROWS_PER_WARP], beta, alpha;
    auto fetch = [&](int col, float* q_, float* k_, float* v_, float& b_, float& a_) {
        const float* r = raw + (size_t)col * raw_stride;
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            q_[e] = __ldcg(r + (size_t)h * DK + lane * EPL + e);
            k_[e] = __ldcg(r + (size_t)H * DK + (size_t)h * DK + lane * EPL + e);
        }
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i) v_[i] = row0 + i < dv ? __ldcg(r + (size_t)2 * H * DK + (size_t)h * dv + row0 + i) : 0.f;
        b_ = __ldcg(r + (size_t)2 * H * DK + (size_t)H * dv + h);
        a_ = __ldcg(r + (size_t)2 * H * DK + (size_t)H * dv + H + h);
    };
    fetch(first, qn, kn, vr, beta, alpha);
    for (int col = first; col < n_cols; ++col) {
        const bool more = col + 1 < n_cols && seq_active(c, col + 1) && seq_of[col + 1] == cur;
        float qx[EPL], kx[EPL], vx[ROWS_PER_WARP], bx = 0.f, ax = 0.f;
        if (more) fetch(col + 1, qx, kx, vx, bx, ax);
        float d1[ROWS_PER_WARP], d2[ROWS_PER_WARP];
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i) {
            d1[i] = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) { s[i][e] *= alpha; d1[i] = fmaf(s[i][e], kn[e], d1[i]); }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int i = 0; i < ROWS_PER_WARP; ++i) d1[i] += __shfl_xor_sync(0xffffffffu, d1[i], o);
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i) {
            const float cf = beta * (vr[i] - d1[i]);
            d2[i] = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) { s[i][e] = fmaf(cf, kn[e], s[i][e]); d2[i] = fmaf(s[i][e], qn[e], d2[i]); }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int i = 0; i < ROWS_PER_WARP; ++i) d2[i] += __shfl_xor_sync(0xffffffffu, d2[i], o);
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < ROWS_PER_WARP; ++i) {
                if (row0 + i < dv) {
                    abuf[((size_t)col * H + h) * dv + row0 + i] = d2[i];
                    if (abuf16) abuf16[((size_t)col * H + h) * dv + row0 + i] = __float2bfloat16_rn(d2[i]);
                }
            }
        }
        if (!more) break;
#pragma unroll
        for (int e = 0; e < EPL; ++e) { qn[e] = qx[e]; kn[e] = kx[e]; }
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i) vr[i] = vx[i];
        beta = bx;
        alpha = ax;
    }
#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; ++i)
        if (row0 + i < dv) {
            if (EPL == 4) *reinterpret_cast<float4*>(&Sh[(size_t)(row0 + i) * DK + lane * 4]) = make_float4(s[i][0], s[i][1], s[i][2 % EPL], s[i][3 % EPL]);
            else *reinterpret_cast<float2*>(&Sh[(size_t)(row0 + i) * DK + lane * 2]) = make_float2(s[i][0], s[i][1]);
        }
}

// ------------------------------------------------------------------------------------
// Temperature / top-k / Philox sampler (no counterpart in the reference). One CTA per
// sequence over the fp32 logits the LM head wrote: 4-pass radix select of the k-th largest
// value, candidates gathered and bitonic-sorted by (value desc, index asc), softmax over the
// kept set accumulated sequentially in that order, inverse CDF with one Philox4x32-10 draw
// keyed by the sequence seed at counter = position of the token being drawn.
// ------------------------------------------------------------------------------------
struct SampleParams {
    const float* logits; int V;
    int top_k; float temperature;
    const unsigned long long* seeds;   // [B]
};

__device__ __forceinline__ uint32_t philox_first_word(uint32_t c0, uint32_t k0, uint32_t k1) {
    uint32_t c[4] = {c0, 0u, 0u, 0u};
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
        uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
        uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return c[0];
}

__device__ __forceinline__ uint32_t float_order_key(float f) {
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // larger float -> larger key
}

constexpr int kSampleCap = 1024;       // max candidates kept in shared memory
constexpr int kSampleKeys = 8192;      // order keys of the first logits kept in shared memory between the passes

__device__ __forceinline__ float float_from_order_key(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}

// Temperature / top-k / Philox pick of one sequence per CTA (no counterpart in the reference, whose loop
// is greedy: inference_orchestrator.cu:77-84). The k largest logits are found by a radix select over
// order-preserving keys, most significant byte first. The keys of the first kSampleKeys logits are computed
// once (one division each) and kept in shared memory; a warp adds to a histogram bin once per distinct bin
// (__match_any_sync) - logits share their leading byte, and 8192 atomics on three or four words were most of
// the kernel's 52 us at 256 sequences.
static __global__ void __launch_bounds__(256) sample_topk_kernel(StepCtl c, SampleParams p) {
    const int b = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (!seq_active(c, b)) return;
    const int tid = threadIdx.x, lane = tid & 31;
    const float* lg = p.logits + (size_t)b * p.V;
    const float T = p.temperature;
    const int k = min(p.top_k, min(p.V, kSampleCap));
    __shared__ uint32_t hist[256];
    __shared__ uint32_t s_prefix, s_mask, s_need;
    __shared__ uint32_t skey[kSampleKeys];
    __shared__ float cval[kSampleCap];
    __shared__ int cidx[kSampleCap];
    __shared__ int s_count, s_overflow;
    if (tid == 0) { s_prefix = 0; s_mask = 0; s_need = (uint32_t)k; }
    __syncthreads();
    // after the four passes s_prefix is the key of the k-th largest element
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix, mask = s_mask;
        // The first digit (sign and exponent bits) is shared by most logits: lanes with the same bin add once
        // (__match_any_sync). From the second digit on only the few keys under the chosen prefix count and their
        // bins differ: plain atomics, no warp-wide exchange.
        auto count = [&](int i, uint32_t key) {
            const bool ok = i < p.V && (key & mask) == prefix;
            const uint32_t bin = (key >> shift) & 0xffu;
            if (pass == 0) {
                const unsigned act = __ballot_sync(0xffffffffu, ok);
                if (ok) {
                    const unsigned peers = __match_any_sync(act, bin);
                    if (lane == __ffs(peers) - 1) atomicAdd(&hist[bin], (uint32_t)__popc(peers));
                }
            } else if (ok) {
                atomicAdd(&hist[bin], 1u);
            }
        };
        // logits from global memory eight at a time per thread: one L2 latency per eight values instead of
        // one per value (the ballot below consumes a value as soon as it is there); keys of later passes come
        // from shared memory
        for (int base = 0; base < p.V; base += 8 * 256) {
            const bool from_global = pass == 0 || base + 8 * 256 > kSampleKeys;
            float v[8];
            if (from_global) {
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int i = base + u * 256 + tid;
                    v[u] = i < p.V ? lg[i] : 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * 256 + tid;
                uint32_t key = 0;
                if (from_global) {
                    key = float_order_key(v[u] / T);
                    if (pass == 0 && i < p.V && i < kSampleKeys) skey[i] = key;
                } else if (i < p.V) {
                    key = skey[i];
                }
                count(i, key);
            }
        }
        __syncthreads();
        if (tid < 32) {
            // the bin that holds the `need`-th largest key of this digit: lane l sums bins 255 - 8l .. 248 - 8l,
            // an exclusive scan over the lanes finds the lane, which then walks its eight bins
            const uint32_t need = s_need;
            uint32_t mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) mine += hist[255 - 8 * lane - j];
            uint32_t incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            const uint32_t before = incl - mine;
            // the last lane also takes the case of fewer than `need` candidates in all bins (k > count)
            const bool here = (before < need && need <= incl) || (lane == 31 && incl < need);
            if (here) {
                uint32_t left = need - before, bin = 255 - 8 * lane;
                for (int j = 0; j < 8; ++j, --bin) {
                    const uint32_t h = hist[bin];
                    if (h >= left || bin == 0) break;
                    left -= h;
                }
                s_need = left;
                s_prefix = prefix | (bin << shift);
                s_mask = mask | (0xffu << shift);
            }
        }
        __syncthreads();
    }
    const uint32_t kth = s_prefix;
    if (tid == 0) { s_count = 0; s_overflow = 0; }
    __syncthreads();
    for (int i = tid; i < p.V; i += blockDim.x) {
        const uint32_t key = i < kSampleKeys ? skey[i] : float_order_key(lg[i] / T);
        if (key >= kth) {
            int slot = atomicAdd(&s_count, 1);
            if (slot < kSampleCap) { cval[slot] = float_from_order_key(key); cidx[slot] = i; } else s_overflow = 1;
        }
    }
    __syncthreads();
    int n = min(s_count, kSampleCap);
    if (s_overflow) {
        // More than kSampleCap values tie at the threshold: keep the strictly larger ones and
        // refill ties in index order with one thread (degenerate inputs only).
        if (tid == 0) {
            int w = 0;
            for (int i = 0; i < p.V && w < kSampleCap; ++i) {
                float v = lg[i] / T;
                if (float_order_key(v) > kth) { cval[w] = v; cidx[w] = i; ++w; }
            }
            for (int i = 0; i < p.V && w < kSampleCap; ++i) {
                float v = lg[i] / T;
                if (float_order_key(v) == kth) { cval[w] = v; cidx[w] = i; ++w; }
            }
            s_count = w;
        }
        __syncthreads();
        n = s_count;
    }
    // pad to a power of two and bitonic sort: value descending, index ascending
    int np2 = 1;
    while (np2 < n) np2 <<= 1;
    for (int i = n + tid; i < np2; i += blockDim.x) { cval[i] = -INFINITY; cidx[i] = 0x7fffffff; }
    __syncthreads();
    for (int sz = 2; sz <= np2; sz <<= 1) {
        for (int st = sz >> 1; st > 0; st >>= 1) {
            for (int i = tid; i < np2; i += blockDim.x) {
                int j = i ^ st;
                if (j > i) {
                    bool up = ((i & sz) == 0);
                    float vi = cval[i], vj = cval[j];
                    int ii = cidx[i], ij = cidx[j];
                    bool i_first = (vi > vj) || (vi == vj && ii < ij);   // i belongs before j
                    if (i_first != up) { cval[i] = vj; cval[j] = vi; cidx[i] = ij; cidx[j] = ii; }
                }
            }
            __syncthreads();
        }
    }
    // the exponentials in parallel, their sums by one thread in descending order (the order is part of the result)
    const int kk = min(k, n);
    {
        const float v0 = cval[0];
        float e[(kSampleCap + 255) / 256];
#pragma unroll
        for (int r = 0; r < (kSampleCap + 255) / 256; ++r) {
            const int j = tid + 256 * r;
            e[r] = j < kk ? expf(cval[j] - v0) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < (kSampleCap + 255) / 256; ++r) {
            const int j = tid + 256 * r;
            if (j < kk) cval[j] = e[r];
        }
        __syncthreads();
    }
    if (tid == 0) {
        float total = 0.f;
        for (int j = 0; j < kk; ++j) total += cval[j];
        unsigned long long seed = p.seeds[b];
        uint32_t w0 = philox_first_word((uint32_t)(c.pos[b] + 1), (uint32_t)(seed & 0xffffffffull), (uint32_t)(seed >> 32));
        float u = (float)(w0 >> 8) * (1.0f / 16777216.0f);
        float target = u * total, cum = 0.f;
        int pick = kk - 1;
        for (int j = 0; j < kk; ++j) {
            cum += cval[j];
            if (cum > target) { pick = j; break; }
        }
        advance_seq(c, b, cidx[pick]);
    }
}

// Column softmax of the logits for the probability probe (getVocabMaxByCol_softmax,
// getVocabSumByCol_softmax, applySoftmaxToVocab, inference.cu:293-362). One CTA.
static __global__ void __launch_bounds__(256) softmax_probe_kernel(const float* __restrict__ logits, int V, float* __restrict__ out) {
    __shared__ float red[256];
    const int tid = threadIdx.x;
    float mx = -1.0e20f;
    for (int i = tid; i < V; i += blockDim.x) mx = fmaxf(mx, logits[i]);
    red[tid] = mx;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) { if (tid < s) red[tid] = fmaxf(red[tid], red[tid + s]); __syncthreads(); }
    mx = red[0];
    __syncthreads();
    float sum = 0.f;
    for (int i = tid; i < V; i += blockDim.x) { float e = expf(logits[i] - mx); out[i] = e; sum += e; }
    red[tid] = sum;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) { if (tid < s) red[tid] += red[tid + s]; __syncthreads(); }
    sum = red[0];
    for (int i = tid; i < V; i += blockDim.x) out[i] = out[i] / sum;
}

// ------------------------------------------------------------------------------------
// Load-time conversions
// ------------------------------------------------------------------------------------
static __global__ void cvt_f32_to_bf16_kernel(const float* __restrict__ src, bf16_t* __restrict__ dst, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] = __float2bfloat16_rn(src[i]);
}

// One warp per row: scale = max|row| / 448 (1 when the row is all zero), code = e4m3(w / scale).
static __global__ void quant_fp8_rows_kernel(const float* __restrict__ src, fp8_t* __restrict__ dst,
                                      float* __restrict__ scale, int rows, int cols) {
    int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* s = src + (size_t)row * cols;
    float amax = 0.f;
    for (int i = lane; i < cols; i += 32) amax = fmaxf(amax, fabsf(s[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float sc = amax > 0.f ? amax / 448.0f : 1.0f;
    if (lane == 0) scale[row] = sc;
    for (int i = lane; i < cols; i += 32)
        dst[(size_t)row * cols + i].v = (uint8_t)__nv_cvt_float_to_fp8(s[i] / sc, __NV_SATFINITE, __NV_E4M3);
}

// Writes a buffer larger than L2 so that the next timed step starts cold.
static __global__ void l2_flush_kernel(float4* __restrict__ buf, size_t n, float v) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) buf[i] = make_float4(v, v, v, v);
}

}  // namespace mlb
