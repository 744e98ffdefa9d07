// Stand-alone operator entry points over DEVICE pointers: single kernels of the decode step
// exposed for callers that own their buffers (and for kernel-level parity tests).
#include <atomic>
#include <cstdint>

#include "../../include/mlb.h"
#include "errors.h"
#include "kernels.cuh"
#include "ring.cuh"
#include "tc_host.h"

using namespace mlb;

#define CU(expr)                                                                              \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess)                                                               \
            return fail(MLB_E_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__); \
    } while (0)

namespace {

// Scratch of one flash-decode launch, carved from one byte range:
//   error word (zero before the launch) | tickets [B*kv_heads] int (zero before the launch) |
//   limits [B] int (never reached) | partials [B][heads][splits][hd+2] float
struct AttnScratch {
    int* err;
    int* ticket;
    int* limit;
    float* part;
};

size_t attn_scratch_ints(int B, int kv_heads) { return (1 + (size_t)B * kv_heads + (size_t)B + 63) / 64 * 64; }     // keeps the floats 256-byte aligned

size_t attn_scratch_bytes(int B, int heads, int kv_heads, int hd, int splits) {
    return attn_scratch_ints(B, kv_heads) * 4 + (size_t)B * heads * splits * (hd + 2) * 4;
}

AttnScratch carve(void* base, int B, int kv_heads) {
    AttnScratch s;
    s.err = static_cast<int*>(base);
    s.ticket = s.err + 1;
    s.limit = s.ticket + (size_t)B * kv_heads;
    s.part = reinterpret_cast<float*>(static_cast<int*>(base) + attn_scratch_ints(B, kv_heads));
    return s;
}

int check_attn_args(const void* kpool, const void* vpool, int kv_dtype, const int32_t* page_table, int pt_stride, int num_pages,
                    const int32_t* positions, const float* q, float* out, int batch, int heads, int kv_heads, int head_dim, int splits) {
    if (!kpool || !vpool || !page_table || !positions || !q || !out) return fail(MLB_E_INVALID, "attention op: null pointer");
    if (pt_stride < 1 || num_pages < 1) return fail(MLB_E_INVALID, "attention op: pt_stride and num_pages must be >= 1");
    if (kv_dtype != MLB_DT_F32 && kv_dtype != MLB_DT_BF16) return fail(MLB_E_INVALID, "attention op: kv_dtype must be float32 or bfloat16");
    if (batch < 1 || heads < 1 || kv_heads < 1 || heads % kv_heads) return fail(MLB_E_INVALID, "attention op: bad batch / head counts");
    const int g = heads / kv_heads;
    if (g != 1 && g != 2 && g != 4 && g != 8) return fail(MLB_E_UNSUPPORTED, "attention op: heads/kv_heads must be 1, 2, 4 or 8");
    if (head_dim != 64 && head_dim != 128) return fail(MLB_E_UNSUPPORTED, "attention op: head_dim must be 64 or 128");
    if (splits < 1 || splits > 64) return fail(MLB_E_INVALID, "attention op: splits must be in 1..64");
    return MLB_OK;
}

template <typename KVT, int HD>
cudaError_t launch_attn(const StepCtl& c, const AttnParams& p, int G, int splits, int B, cudaStream_t st) {
    dim3 grid(splits, p.kv_heads, B);
    switch (G) {
        case 1: attn_decode_kernel<KVT, HD, 1><<<grid, 128, 0, st>>>(c, p); break;
        case 2: attn_decode_kernel<KVT, HD, 2><<<grid, 128, 0, st>>>(c, p); break;
        case 4: attn_decode_kernel<KVT, HD, 4><<<grid, 128, 0, st>>>(c, p); break;
        default: attn_decode_kernel<KVT, HD, 8><<<grid, 128, 0, st>>>(c, p); break;
    }
    return cudaGetLastError();
}

// Clears the part of the scratch that must start at zero, then launches. No allocation.
int run_attn(void* scratch, const void* kpool, const void* vpool, int kv_dtype, const int32_t* page_table, int pt_stride, int num_pages,
             const int32_t* positions, const float* q, const float* gate, float* out, int batch, int heads, int kv_heads,
             int head_dim, int splits, cudaStream_t st) {
    AttnScratch sc = carve(scratch, batch, kv_heads);
    CU(cudaMemsetAsync(sc.err, 0, (1 + (size_t)batch * kv_heads) * 4, st));          // the error word and the tickets
    CU(cudaMemsetAsync(sc.limit, 0x7f, (size_t)batch * 4, st));          // 0x7f7f7f7f: every sequence takes part
    StepCtl c;
    c.B = batch; c.vocab = 0;
    c.pos = const_cast<int*>(positions); c.tok = nullptr; c.limit = sc.limit; c.stop_token = -1;
    c.prompt = nullptr; c.prompt_stride = 0; c.out_ring = nullptr; c.out_idx = nullptr; c.out_cap = 0;
    c.tok_src = nullptr; c.host_out = nullptr; c.host_err = nullptr; c.dev_err = nullptr;
    AttnParams p;
    p.kpool = kpool; p.vpool = vpool; p.page_table = page_table; p.pt_stride = pt_stride;
    p.qbuf = q; p.gbuf = gate; p.abuf = out; p.abuf16 = nullptr; p.part = sc.part; p.ticket = sc.ticket;
    p.heads = heads; p.kv_heads = kv_heads; p.hg = 1;
    p.num_pages = num_pages; p.err = sc.err; p.min_pages_per_split = 1;
    const int G = heads / kv_heads;
    cudaError_t e;
    if (kv_dtype == MLB_DT_F32)
        e = head_dim == 64 ? launch_attn<float, 64>(c, p, G, splits, batch, st) : launch_attn<float, 128>(c, p, G, splits, batch, st);
    else
        e = head_dim == 64 ? launch_attn<bf16_t, 64>(c, p, G, splits, batch, st) : launch_attn<bf16_t, 128>(c, p, G, splits, batch, st);
    if (e != cudaSuccess) return fail(MLB_E_CUDA, "attention op launch failed: %s", cudaGetErrorString(e));
    return MLB_OK;
}

}  // namespace

static const char* attn_err_text(int code) {
    return code == 4 ? "a position needs more pages than pt_stride (that sequence was skipped)"
                     : "the page table names a page outside [0, num_pages) (page 0 was read instead)";
}

extern "C" int mlb_op_attn_decode(const void* kpool, const void* vpool, int kv_dtype, const int32_t* page_table, int pt_stride,
                                  int num_pages, const int32_t* positions, const float* q, const float* gate_or_null, float* out,
                                  int batch, int heads, int kv_heads, int head_dim, int splits, void* stream) {
    int rc = check_attn_args(kpool, vpool, kv_dtype, page_table, pt_stride, num_pages, positions, q, out, batch, heads, kv_heads, head_dim,
                             splits);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    void* scratch = nullptr;
    cudaError_t e = cudaMalloc(&scratch, attn_scratch_bytes(batch, heads, kv_heads, head_dim, splits));
    if (e != cudaSuccess) return fail(MLB_E_NOMEM, "attention op: cudaMalloc of the scratch failed: %s", cudaGetErrorString(e));
    rc = run_attn(scratch, kpool, vpool, kv_dtype, page_table, pt_stride, num_pages, positions, q, gate_or_null, out, batch, heads,
                  kv_heads, head_dim, splits, st);
    cudaError_t se = cudaStreamSynchronize(st);       // the scratch must outlive the kernel
    int code = 0;
    if (rc == MLB_OK && se == cudaSuccess) se = cudaMemcpy(&code, scratch, 4, cudaMemcpyDeviceToHost);
    cudaFree(scratch);
    if (rc) return rc;
    if (se != cudaSuccess) return fail(MLB_E_CUDA, "attention op failed: %s", cudaGetErrorString(se));
    if (code) return fail(MLB_E_INVALID, "attention op: %s; the output is invalid", attn_err_text(code));
    return MLB_OK;
}

extern "C" int mlb_op_gemm_bf16(const void* W, const void* W_up_or_null, const void* X, const float* resid_or_null, void* out, int N,
                                int K, int batch, void* stream) {
    if (!W || !X || !out) return fail(MLB_E_INVALID, "gemm op: null pointer");
    if (N < 1 || K < 8 || K % 8 || batch < 1) return fail(MLB_E_INVALID, "gemm op: N >= 1, K a multiple of 8, batch >= 1");
    if (W_up_or_null && resid_or_null) return fail(MLB_E_INVALID, "gemm op: gate/up and residual are exclusive");
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return fail(MLB_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const int Nb = batch >= 256 ? 256 : (batch + 15) / 16 * 16;
    alignas(64) CUtensorMap tA, tA2, tB;
    int rc;
    if ((rc = make_bf16_map(enc, &tA, W, N, K, kTcM))) return rc;
    if ((rc = make_bf16_map(enc, &tA2, W_up_or_null ? W_up_or_null : W, N, K, kTcM))) return rc;
    if ((rc = make_bf16_map(enc, &tB, X, batch, K, Nb))) return rc;
    int* err = nullptr;
    CU(cudaMalloc(&err, 4));
    CU(cudaMemset(err, 0, 4));
    const int na = W_up_or_null ? 2 : 1;
    GemmTcParams p;
    p.N = N; p.K = K; p.B = batch; p.Nb = Nb;
    const size_t stage_bytes = (size_t)na * kTcM * 128 + (size_t)Nb * 128;
    p.stages = (int)(kTcRingBytes / stage_bytes);
    if (p.stages > 6) p.stages = 6;
    p.group = 1;
    p.trace = nullptr;
    p.sA = nullptr; p.sA2 = nullptr;
    uint32_t cols = 32;
    while (cols < (uint32_t)na * (uint32_t)Nb) cols <<= 1;
    p.tmem_cols = cols;
    p.y = static_cast<float*>(out); p.resid = resid_or_null; p.h16 = static_cast<bf16_t*>(out); p.err = err;
    // the plain operator: no deferred norm, no second operand pair, no outputs for a following norm
    p.nkb_x = 0; p.ssq_in = nullptr; p.ssq_parts = 0; p.eps = 0.f; p.xg16 = nullptr; p.gain_next = nullptr; p.ssq_out = nullptr;
    const StepCtl c0{};
    const QkvPostParams q0{};
    const size_t smem = 1024 + kTcHeadBytes + kTcStageBytes + (size_t)p.stages * stage_bytes;
    dim3 grid((N + kTcM - 1) / kTcM, (batch + Nb - 1) / Nb);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (W_up_or_null) {
        e = cudaFuncSetAttribute(gemm_tc_kernel<TC_SWIGLU, float, bf16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e == cudaSuccess) gemm_tc_kernel<TC_SWIGLU, float, bf16_t><<<grid, kTcThreads, smem, st>>>(tA, tA2, tB, tA, tB, p, c0, q0);
    } else if (resid_or_null) {
        e = cudaFuncSetAttribute(gemm_tc_kernel<TC_RESID, float, bf16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e == cudaSuccess) gemm_tc_kernel<TC_RESID, float, bf16_t><<<grid, kTcThreads, smem, st>>>(tA, tA2, tB, tA, tB, p, c0, q0);
    } else {
        e = cudaFuncSetAttribute(gemm_tc_kernel<TC_RAW, float, bf16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e == cudaSuccess) gemm_tc_kernel<TC_RAW, float, bf16_t><<<grid, kTcThreads, smem, st>>>(tA, tA2, tB, tA, tB, p, c0, q0);
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    int herr = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost);
    cudaFree(err);
    if (e != cudaSuccess) return fail(MLB_E_CUDA, "gemm op failed: %s", cudaGetErrorString(e));
    if (herr) return fail(MLB_E_TIMEOUT, "gemm op: a bounded wait ran out (code %d)", herr);
    return MLB_OK;
}

// ---------------------------------------------------------------------------------------
// mlb_op_attn_decode_static: the same flash-decode launch with its scratch in a fixed
// array that is part of the library image, for callers that must not allocate.
//
// Who needs this: a serving process that has handed ALL free device memory to its own pool
// (its KV cache, typically), where a cudaMalloc from inside a library call fails or steals
// from that budget; and a latency-critical token loop that cannot afford cudaMalloc /
// cudaFree at all, because both may synchronise the whole device and stall unrelated streams.
// Such callers already own q, the KV pools, the page table and the output; the only thing the
// operator still needed from the allocator was the split-combine scratch.
//
// The price: every GPU that loads the library carries kAttnStaticBytes of device memory
// until the process exits, sizes beyond it are refused, and because every call on a device
// uses the SAME array, two calls whose kernels overlap on the GPU (different streams, or
// different host threads) race on it - keep calls on one device ordered.
// ---------------------------------------------------------------------------------------
namespace {

constexpr size_t kAttnStaticBytes = 4u << 20;      // 4 MiB per device
// In host code this name is only a handle for the runtime, NOT a device address: the address
// that kernels can use comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_attn_static_scratch[kAttnStaticBytes];

constexpr int kMaxDevices = 64;
// per device, filled on the first call there. Atomic: two host threads may make their first call at once
// (both resolve the same address; either store wins).
std::atomic<void*> g_attn_static_ptr[kMaxDevices];

// One-time set-up for the CURRENT device: resolve the array's device address.
int attn_static_address(void** out) {
    int dev = -1;
    CU(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(MLB_E_UNSUPPORTED, "static attention op: device index %d not supported", dev);
    void* p = g_attn_static_ptr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        // With CUDA's lazy module loading this query is also what places the array on the device: a host
        // that has already given all device memory away gets an out-of-memory error here.
        cudaError_t e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
        if (e == cudaErrorMemoryAllocation)
            return fail(MLB_E_NOMEM, "static attention op: no device memory left for the library's %zu-byte array; make the first call on a "
                                     "device before the host claims all its memory, or set CUDA_MODULE_LOADING=EAGER", kAttnStaticBytes);
        if (e != cudaSuccess || p == nullptr)
            return fail(MLB_E_CUDA, "static attention op: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_attn_static_ptr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return MLB_OK;
}

}  // namespace

extern "C" size_t mlb_op_attn_decode_static_capacity(void) { return kAttnStaticBytes; }

extern "C" int mlb_op_attn_decode_static(const void* kpool, const void* vpool, int kv_dtype, const int32_t* page_table,
                                         int pt_stride, int num_pages, const int32_t* positions, const float* q,
                                         const float* gate_or_null, float* out, int batch, int heads, int kv_heads, int head_dim,
                                         int splits, void* stream) {
    int rc = check_attn_args(kpool, vpool, kv_dtype, page_table, pt_stride, num_pages, positions, q, out, batch, heads, kv_heads, head_dim,
                             splits);
    if (rc) return rc;
    const size_t need = attn_scratch_bytes(batch, heads, kv_heads, head_dim, splits);
    if (need > kAttnStaticBytes)
        return fail(MLB_E_UNSUPPORTED,
                    "static attention op: batch %d x heads %d x splits %d x head_dim %d needs %zu bytes of scratch, the "
                    "built-in array holds %zu; lower splits or batch, or use mlb_op_attn_decode",
                    batch, heads, splits, head_dim, need, kAttnStaticBytes);
    void* scratch = nullptr;
    if ((rc = attn_static_address(&scratch))) return rc;
    // The array keeps whatever the previous call left: run_attn clears the error word and the arrival
    // counters and rewrites the limits; the partials are fully overwritten before they are read.
    return run_attn(scratch, kpool, vpool, kv_dtype, page_table, pt_stride, num_pages, positions, q, gate_or_null, out, batch, heads,
                    kv_heads, head_dim, splits, static_cast<cudaStream_t>(stream));
}

// The call above returns before its kernel has run, so a page table that does not fit (see AttnParams)
// cannot be reported by it. This one waits for `stream` and reads the error word of the last call on the
// current device (a 4-byte copy out of the array: still no allocation).
extern "C" int mlb_op_attn_decode_static_status(void* stream) {
    void* scratch = nullptr;
    int rc = attn_static_address(&scratch);
    if (rc) return rc;
    CU(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    int code = 0;
    CU(cudaMemcpy(&code, scratch, 4, cudaMemcpyDeviceToHost));
    if (code) return fail(MLB_E_INVALID, "static attention op: %s; the output of that call is invalid", attn_err_text(code));
    return MLB_OK;
}

// ---- bounded-wait probe ------------------------------------------------------------------------
namespace {
// One thread waits, with the wait routine of the streaming kernels, for an mbarrier phase that
// nothing completes; when the polls run out it records code 2, as those kernels do.
__global__ void wait_probe_kernel(uint32_t max_polls, int* err) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t a = mlb::smem_u32(&bar);
    if (threadIdx.x == 0) {
        mlb::mbar_init(a, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!mlb::mbar_wait_bounded(a, 0, max_polls, 0)) atomicExch(err, 2);
    }
}
}  // namespace

extern "C" int mlb_op_wait_probe(int device, uint32_t max_polls) {
    if (max_polls < 1 || max_polls > (1u << 20)) return mlb::fail(MLB_E_INVALID, "max_polls must be in 1..2^20");
    CU(cudaSetDevice(device));
    int* err = nullptr;
    CU(cudaMalloc((void**)&err, 4));
    cudaError_t e = cudaMemset(err, 0, 4);
    int code = 0;
    if (e == cudaSuccess) {
        wait_probe_kernel<<<1, 32>>>(max_polls, err);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpy(&code, err, 4, cudaMemcpyDeviceToHost);      // waits for the kernel
    cudaFree(err);
    if (e != cudaSuccess) return mlb::fail(MLB_E_CUDA, "wait probe: %s", cudaGetErrorString(e));
    if (code != 0)
        return mlb::fail(MLB_E_TIMEOUT, "a bounded device-side wait ran out (code %d) after %u polls; the context stays usable", code,
                         max_polls);
    return MLB_OK;
}
