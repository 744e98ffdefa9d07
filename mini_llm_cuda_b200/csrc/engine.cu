// Host side of the decode path: model upload, session state (paged KV cache, delta-net
// state, step scratch), the launch chain of one decode step, CUDA-graph replay, and the C ABI
// declared in include/mlb.h.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <chrono>
#include <cstring>
#include <string>
#include <type_traits>
#include <mutex>
#include <vector>

#include "../../include/mlb.h"
#include "errors.h"
#include "kernels.cuh"
#include "gemm_tc.cuh"
#include "tc_host.h"
#include "ring.cuh"
#include "grid_params.h"
#include "grid_host.h"
#include "lean_params.h"
#include "lean_host.h"
#include "model_file.h"
#include "sgemv.cuh"

namespace mlb {

// --------------------------------------------------------------------------------------
// errors
// --------------------------------------------------------------------------------------
static thread_local std::string g_err;

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

#define CU(expr)                                                                              \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess)                                                               \
            return fail(MLB_E_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__); \
    } while (0)

static size_t elt_size(int dt) { return dt == MLB_DT_F32 ? 4 : (dt == MLB_DT_BF16 ? 2 : 1); }
static int ple_dtype(int wdt) { return wdt == MLB_DT_FP8_E4M3 ? MLB_DT_BF16 : wdt; }

// --------------------------------------------------------------------------------------
// KV page allocator (host only)
// --------------------------------------------------------------------------------------
}  // namespace mlb

struct mlb_kv_alloc {
    std::vector<int> free_list;                 // stack; back() is handed out next
    std::vector<std::vector<int>> seq_pages;
    int max_pages_per_seq = 0;
    int num_pages = 0;
};

namespace mlb {

static int kv_ensure(mlb_kv_alloc* a, int seq, int n_positions, int block) {
    if (!a || seq < 0 || seq >= (int)a->seq_pages.size() || block <= 0 || n_positions < 0)
        return fail(MLB_E_INVALID, "kv allocator: bad argument");
    int need = (n_positions + block - 1) / block;
    if (need > a->max_pages_per_seq)
        return fail(MLB_E_CONTEXT_FULL, "sequence %d needs %d pages, the page table holds %d", seq, need, a->max_pages_per_seq);
    auto& pages = a->seq_pages[seq];
    while ((int)pages.size() < need) {
        if (a->free_list.empty())
            return fail(MLB_E_KV_FULL, "KV page pool exhausted (%d pages) while growing sequence %d", a->num_pages, seq);
        pages.push_back(a->free_list.back());
        a->free_list.pop_back();
    }
    return MLB_OK;
}

// --------------------------------------------------------------------------------------
// model
// --------------------------------------------------------------------------------------
struct DevLayer {
    int type = MLB_LAYER_ATTENTION;
    float *g1 = nullptr, *g2 = nullptr, *gq = nullptr, *gk = nullptr;
    void* Wqkv = nullptr; float* Sqkv = nullptr; int n_qkv = 0;
    int nq = 0, nk = 0, nv = 0, ng = 0;
    void* Wo = nullptr; float* So = nullptr; int o_in = 0;
    void *W1a = nullptr, *W1b = nullptr, *W2 = nullptr;
    float *S1a = nullptr, *S1b = nullptr, *S2 = nullptr;
    void *pleT = nullptr, *pleP = nullptr;
};

}  // namespace mlb

struct mlb_model {
    mlb_config cfg;
    int device = 0;
    void* E = nullptr; float* Es = nullptr; float* g_final = nullptr; float* rope = nullptr;
    std::vector<mlb::DevLayer> layers;      // execution order
    uint64_t weight_bytes = 0;
    std::vector<void*> allocs;
    // FP8 models: the same weights as bf16 (code * row scale, rounded), made on first use for the
    // tensor-core steps that consume a prompt as columns; shares gains, RoPE table and PLE tensors
};

namespace mlb {

struct Uploader {
    mlb_model* m;
    const std::vector<unsigned char>* file;
    std::vector<float> hbuf;
    float* dstage = nullptr;
    size_t dstage_elems = 0;

    int dev_alloc(void** p, size_t bytes) {
        cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
        if (e != cudaSuccess) return fail(MLB_E_NOMEM, "cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
        m->allocs.push_back(*p);
        return MLB_OK;
    }
    // file tensor -> float32 on the device staging buffer
    int stage(const TensorDesc& t) {
        size_t n = (size_t)t.rows * t.cols;
        const unsigned char* src = file->data() + t.offset;
        const float* hsrc;
        if (t.dtype == FD_F32) {
            hsrc = reinterpret_cast<const float*>(src);
        } else {
            hbuf.resize(n);
            convert_to_f32(src, t.dtype, n, hbuf.data(), (uint64_t)t.cols);
            hsrc = hbuf.data();
        }
        CU(cudaMemcpy(dstage, hsrc, n * 4, cudaMemcpyHostToDevice));
        return MLB_OK;
    }
    // staged float32 [rows][cols] -> typed matrix rows [row_off, row_off+rows) of dst
    int emit(const TensorDesc& t, int dt, void* dst, size_t row_off, float* scale) {
        size_t n = (size_t)t.rows * t.cols;
        size_t off = row_off * (size_t)t.cols;
        if (dt == MLB_DT_F32) {
            CU(cudaMemcpy(static_cast<float*>(dst) + off, dstage, n * 4, cudaMemcpyDeviceToDevice));
        } else if (dt == MLB_DT_BF16) {
            cvt_f32_to_bf16_kernel<<<1024, 256>>>(dstage, static_cast<bf16_t*>(dst) + off, n);
            CU(cudaGetLastError());
        } else {
            int warps = 8;
            quant_fp8_rows_kernel<<<(t.rows + warps - 1) / warps, warps * 32>>>(dstage, static_cast<fp8_t*>(dst) + off,
                                                                              scale + row_off, t.rows, t.cols);
            CU(cudaGetLastError());
        }
        CU(cudaDeviceSynchronize());
        return MLB_OK;
    }
    int vec(const TensorDesc* t, float** out) {
        int rc = dev_alloc(reinterpret_cast<void**>(out), (size_t)t->rows * 4);
        if (rc) return rc;
        if ((rc = stage(*t))) return rc;
        CU(cudaMemcpy(*out, dstage, (size_t)t->rows * 4, cudaMemcpyDeviceToDevice));
        m->weight_bytes += (uint64_t)t->rows * 4;
        return MLB_OK;
    }
    // a matrix made of several file tensors stacked by rows
    int stacked(const std::vector<const TensorDesc*>& parts, int dt, void** W, float** S, int* total_rows) {
        int rows = 0, cols = parts[0]->cols;
        for (auto* t : parts) rows += t->rows;
        int rc = dev_alloc(W, (size_t)rows * cols * elt_size(dt));
        if (rc) return rc;
        *S = nullptr;
        if (dt == MLB_DT_FP8_E4M3 && (rc = dev_alloc(reinterpret_cast<void**>(S), (size_t)rows * 4))) return rc;
        size_t off = 0;
        for (auto* t : parts) {
            if (t->dtype == FD_FP8 && dt == MLB_DT_FP8_E4M3) {
                // quantised offline: the file's codes and per-row scales are the device's
                const unsigned char* src = file->data() + t->offset;
                const size_t n = (size_t)t->rows * t->cols;
                CU(cudaMemcpy(static_cast<fp8_t*>(*W) + off * (size_t)cols, src, n, cudaMemcpyHostToDevice));
                CU(cudaMemcpy(*S + off, src + n, (size_t)t->rows * 4, cudaMemcpyHostToDevice));
            } else {
                if ((rc = stage(*t))) return rc;
                if ((rc = emit(*t, dt, *W, off, *S))) return rc;
            }
            off += t->rows;
        }
        if (total_rows) *total_rows = rows;
        m->weight_bytes += (uint64_t)rows * cols * elt_size(dt) + (dt == MLB_DT_FP8_E4M3 ? (uint64_t)rows * 4 : 0);
        return MLB_OK;
    }
};

static int validate_for_kernels(const mlb_config& c) {
    const int gran = c.weight_dtype == MLB_DT_FP8_E4M3 ? 16 : (c.weight_dtype == MLB_DT_BF16 ? 8 : 4);
    if (c.dim % gran || c.ffn_dim % gran) return fail(MLB_E_UNSUPPORTED, "dim and ffn_dim must be multiples of %d for this weight type", gran);
    if (c.ple_dim % 8) return fail(MLB_E_UNSUPPORTED, "ple_dim must be a multiple of 8");
    bool has_attn = false, has_dn = false;
    for (int i = 0; i < c.layers; ++i) (c.layer_types[i] == MLB_LAYER_ATTENTION ? has_attn : has_dn) = true;
    if (has_attn) {
        if (c.head_dim != 64 && c.head_dim != 128) return fail(MLB_E_UNSUPPORTED, "attention head_dim must be 64 or 128 (got %d)", c.head_dim);
        int g = c.heads / c.kv_heads;
        if (g != 1 && g != 2 && g != 4 && g != 8) return fail(MLB_E_UNSUPPORTED, "heads/kv_heads must be 1, 2, 4 or 8 (got %d)", g);
        if ((c.heads * c.head_dim) % gran) return fail(MLB_E_UNSUPPORTED, "heads*head_dim must be a multiple of %d", gran);
    }
    if (has_dn) {
        if (c.dn_key_dim != 64 && c.dn_key_dim != 128) return fail(MLB_E_UNSUPPORTED, "delta-net key dim must be 64 or 128 (got %d)", c.dn_key_dim);
        if ((c.heads * c.dn_value_dim) % gran) return fail(MLB_E_UNSUPPORTED, "heads*dn_value_dim must be a multiple of %d", gran);
    }
    if (c.vocab < 2) return fail(MLB_E_INVALID, "vocabulary too small");
    return MLB_OK;
}

static void free_model(mlb_model* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    for (void* p : m->allocs) cudaFree(p);
    delete m;
}


}  // namespace mlb

using namespace mlb;

extern "C" void mlb_rope_table(float* table, int max_len, int head_dim, float base) {
    // Same host arithmetic as getPreComputedRopeTheta (inference.cu:364-374): float powf,
    // integer position times the float frequency, cosf / sinf.
    const int pairs = head_dim / 2;
    for (int pos = 0; pos < max_len; ++pos) {
        for (int i = 0; i < pairs; ++i) {
            float theta = pos * powf(base, (-2.0f * i / head_dim));
            table[(size_t)pos * head_dim + 2 * i] = cosf(theta);
            table[(size_t)pos * head_dim + 2 * i + 1] = sinf(theta);
        }
    }
}

extern "C" int mlb_file_inspect(const char* path, const mlb_config* ov, mlb_config* out, uint64_t* n_params) {
    if (!path || !out) return fail(MLB_E_INVALID, "null argument");
    std::vector<unsigned char> buf;
    std::string err;
    int rc = read_file(path, &buf, &err);
    if (rc) return fail(rc, "%s", err.c_str());
    ParsedModel pm;
    rc = parse_model_header(buf.data(), buf.size(), buf.size(), ov, &pm, &err);
    if (rc) return fail(rc, "%s", err.c_str());
    *out = pm.cfg;
    if (n_params) *n_params = pm.n_params;
    return MLB_OK;
}

extern "C" int mlb_model_load(const char* path, int device, const mlb_config* ov, mlb_model** out) {
    if (!path || !out) return fail(MLB_E_INVALID, "null argument");
    *out = nullptr;
    std::vector<unsigned char> buf;
    std::string err;
    int rc = read_file(path, &buf, &err);
    if (rc) return fail(rc, "%s", err.c_str());
    ParsedModel pm;
    rc = parse_model_header(buf.data(), buf.size(), buf.size(), ov, &pm, &err);
    if (rc) return fail(rc, "%s", err.c_str());
    if ((rc = validate_for_kernels(pm.cfg))) return rc;
    int ndev = 0;
    cudaError_t ce = cudaGetDeviceCount(&ndev);
    if (ce != cudaSuccess || ndev == 0)
        return fail(MLB_E_CUDA, "no CUDA device available (%s); this library has no CPU path", cudaGetErrorString(ce));
    if (device < 0 || device >= ndev) return fail(MLB_E_INVALID, "device %d out of range (0..%d)", device, ndev - 1);
    CU(cudaSetDevice(device));

    mlb_model* m = new mlb_model();
    m->cfg = pm.cfg;
    m->device = device;
    const mlb_config& c = m->cfg;
    const int wdt = c.weight_dtype, pdt = ple_dtype(wdt);
    Uploader up;
    up.m = m;
    up.file = &buf;
    size_t max_elems = 0;
    for (auto& t : pm.tensors) max_elems = std::max(max_elems, (size_t)t.rows * t.cols);
    up.dstage_elems = max_elems;
    if (cudaMalloc(reinterpret_cast<void**>(&up.dstage), max_elems * 4) != cudaSuccess) {
        free_model(m);
        return fail(MLB_E_NOMEM, "cudaMalloc of the %zu-byte staging buffer failed", max_elems * 4);
    }
#define UP(expr) do { int r__ = (expr); if (r__) { cudaFree(up.dstage); free_model(m); return r__; } } while (0)
    UP(up.stacked({pm.find(-1, "tokenEmbeddings")}, wdt, &m->E, &m->Es, nullptr));
    UP(up.vec(pm.find(-1, "finalRMSNormGamma"), &m->g_final));
    m->layers.resize(c.layers);
    for (int i = 0; i < c.layers; ++i) {
        const int blk = c.layers - 1 - i;               // block N-1 runs first (inference.cu:384-385)
        DevLayer& L = m->layers[i];
        L.type = c.layer_types[i];
        UP(up.vec(pm.find(blk, "rmsGamma"), &L.g1));
        UP(up.vec(pm.find(blk, "rmsGamma2"), &L.g2));
        std::vector<const TensorDesc*> parts = {pm.find(blk, "queryWeights"), pm.find(blk, "keyWeights"), pm.find(blk, "valueWeights")};
        L.nq = parts[0]->rows; L.nk = parts[1]->rows; L.nv = parts[2]->rows; L.ng = 0;
        if (L.type == MLB_LAYER_ATTENTION) {
            if (c.query_gating) { parts.push_back(pm.find(blk, "gatedQueryWeights")); L.ng = parts.back()->rows; }
            if (c.qk_norm) {
                UP(up.vec(pm.find(blk, "queryRMSGamma"), &L.gq));
                UP(up.vec(pm.find(blk, "keyRMSGamma"), &L.gk));
            }
        } else {
            parts.push_back(pm.find(blk, "betaWeights"));
            parts.push_back(pm.find(blk, "decayWeights"));
        }
        UP(up.stacked(parts, wdt, &L.Wqkv, &L.Sqkv, &L.n_qkv));
        const TensorDesc* wo = pm.find(blk, "outputProjectionWeights");
        L.o_in = wo->cols;
        UP(up.stacked({wo}, wdt, &L.Wo, &L.So, nullptr));
        UP(up.stacked({pm.find(blk, "feedForwardWeights1A")}, wdt, &L.W1a, &L.S1a, nullptr));
        UP(up.stacked({pm.find(blk, "feedForwardWeights1B")}, wdt, &L.W1b, &L.S1b, nullptr));
        UP(up.stacked({pm.find(blk, "feedForwardWeights2")}, wdt, &L.W2, &L.S2, nullptr));
        if (c.ple_dim > 0) {
            float* unused = nullptr;
            UP(up.stacked({pm.find(blk, "pleTable")}, pdt, &L.pleT, &unused, nullptr));
            UP(up.stacked({pm.find(blk, "pleProjection")}, pdt, &L.pleP, &unused, nullptr));
            // only one table row per sequence is read per step, not the whole table
            m->weight_bytes -= (uint64_t)c.vocab * c.ple_dim * elt_size(pdt);
        }
    }
    {
        std::vector<float> tab((size_t)c.max_context * c.head_dim);
        mlb_rope_table(tab.data(), c.max_context, c.head_dim, c.rope_theta);
        UP(up.dev_alloc(reinterpret_cast<void**>(&m->rope), tab.size() * 4));
        cudaError_t e = cudaMemcpy(m->rope, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { cudaFree(up.dstage); free_model(m); return fail(MLB_E_CUDA, "rope table upload: %s", cudaGetErrorString(e)); }
    }
#undef UP
    cudaFree(up.dstage);
    *out = m;
    return MLB_OK;
}

extern "C" int mlb_model_get_config(const mlb_model* m, mlb_config* out) {
    if (!m || !out) return fail(MLB_E_INVALID, "null argument");
    *out = m->cfg;
    return MLB_OK;
}
extern "C" uint64_t mlb_model_weight_bytes(const mlb_model* m) { return m ? m->weight_bytes : 0; }
extern "C" void mlb_model_free(mlb_model* m) { free_model(m); }

// --------------------------------------------------------------------------------------
// session
// --------------------------------------------------------------------------------------
namespace mlb {
enum ChainKind { CHAIN_PREFILL = 0, CHAIN_GREEDY = 1, CHAIN_TOPK = 2 };

struct LaunchRec {
    const char* name;
    uint64_t bytes, flops;
    cudaEvent_t e0, e1;
};
struct Recorder {
    cudaStream_t st;
    std::vector<LaunchRec> recs;
    int begin(const char* name, uint64_t bytes, uint64_t flops) {
        LaunchRec r{name, bytes, flops, nullptr, nullptr};
        CU(cudaEventCreate(&r.e0));
        CU(cudaEventCreate(&r.e1));
        CU(cudaEventRecord(r.e0, st));
        recs.push_back(r);
        return MLB_OK;
    }
    int end() {
        CU(cudaEventRecord(recs.back().e1, st));
        return MLB_OK;
    }
};
}  // namespace mlb

struct TcShape { int nb, split, stages, group; size_t smem; uint32_t tmem_cols; };

struct mlb_session {
    mlb_model* m = nullptr;
    int B = 0, max_ctx = 0, max_pages = 0, kv_pages = 0;
    cudaStream_t stream = nullptr;
    int *pos = nullptr, *tok = nullptr, *limit_prefill = nullptr, *limit_decode = nullptr;
    int *prompt = nullptr, *out_ring = nullptr, *out_idx = nullptr, *page_table = nullptr;
    unsigned long long* seeds = nullptr;
    float *x = nullptr, *qbuf = nullptr, *gbuf = nullptr, *abuf = nullptr, *hbuf = nullptr, *raw = nullptr;
    float *logits = nullptr, *part = nullptr, *part_val = nullptr, *probe = nullptr;
    int *part_idx = nullptr, *attn_ticket = nullptr, *lm_ticket = nullptr;
    std::vector<void*> kpool, vpool;
    std::vector<float*> state;
    std::vector<void*> allocs;
    // host mirrors
    std::vector<int> h_pos;
    std::vector<char> h_stopped;            // the sequence drew the stop token: it takes no further step
    int stop_token = -1;
    std::vector<int> h_table;
    bool table_dirty = true;
    bool have_logits = false;
    mlb_kv_alloc alloc;
    int attn_min_pps = 11;                    // KV pages a flash-decode split must hold before a sequence uses it
    int splits = 1, lm_rows = 32, lm_parts = 1, raw_stride = 0, max_q = 0;
    // graphs
    cudaGraphExec_t graphs[3] = {nullptr, nullptr, nullptr};
    int g_topk = -1; float g_temp = 0.f;
    int cur_topk = 50; float cur_temp = 1.f;
    int launches_per_step[3] = {0, 0, 0};
    // one-token call as ONE graph: upload of the pending ids, the step, read-back of ids and error word
    cudaGraphExec_t tgraphs[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};     // [kind][with input ids]
    int tg_topk[2] = {-1, -1}; float tg_temp[2] = {0.f, 0.f};
    int* pinned_out = nullptr;
    int ctl_host_io = 0;                    // while the one-token graph is captured: 1 = ids and error word to the host, 2 = + ids from the host
    int tok_arg = -1;                       // single-kernel step: the pending id travels with the launch (>= 0), else it is read from `tok`
    float4* flush_buf = nullptr; size_t flush_n = 0;
    int* pinned_tok = nullptr;
    bool use_pdl = true;
    bool use_sgemv = false;                 // TMA-streamed GEMV for very small batches and large matrices
    bool force_sgemv = false;               // MLB_GEMV=stream: also for small matrices (tests)
    int sg_stage_kb = 48, sg_max_stages = 8; // ring geometry of the streamed GEMV (MLB_SG_STAGE_KB, MLB_SG_STAGES)
    int sm_count = 148;
    mlb::StepLayer* step_layers = nullptr;   // device table of per-layer pointers (single-kernel step)
    int* dev_err = nullptr;                 // set by a kernel whose bounded wait ran out
    // whole-GPU single-kernel step (batch 1)
    bool use_grid = false;
    int grid_ctas = 0;
    size_t grid_smem = 0;
    mlb::GridParams grid;
    // the same step with compile-time shapes, for the models it is built for
    bool use_lean = false;
    int lean_idx = -1;
    size_t lean_smem = 0;
    mlb::LeanParams lean;
    // tensor-core projections (bf16 weights, batch >= 16)
    bool use_tc = false;
    int tc_nb = 0, tc_stages = 0, tc_stages_swiglu = 0;
    int tc_max_split = 8;                     // largest cluster that may split a GEMM's k-blocks
    bool tc_split_forced = false;             // MLB_TC_SPLIT given: take it as the limit without the k-blocks-per-CTA rule
    int tc_cluster_cap[4] = {0, 0, 0, 0};     // clusters of 1, 2, 4, 8 GEMM CTAs that can be resident at once
    unsigned long long* tc_trace = nullptr;   // MLB_TC_TRACE=1: [64][8] timer stamps of the step's GEMM launches
    int tc_trace_n = 0;
    TcShape tc_shape_down{};                  // launch shape of the down projection (its per-layer embedding map has this batch tile)
    mlb::bf16_t *xn16 = nullptr, *a16 = nullptr, *h16 = nullptr;
    float* rawq = nullptr;
    struct alignas(64) TcLayerMaps { CUtensorMap qkv, o, w1a, w1b, w2, pleP, pleT; };   // pleP / pleT: [d][ple] projection, gathered [B][ple] rows
    float* tc_ssq = nullptr;                 // [B][ceil(d / 128)] partial sums of squares of the residual stream
    mlb::bf16_t* tple16 = nullptr;           // [layers][B][ple] per-layer embedding rows of the step's tokens
    std::vector<TcLayerMaps> tc_maps;
    // activation operand maps per batch tile 16, 32, 64, 128, 256 (index log2(Nb/16))
    struct alignas(64) TcGlobalMaps { CUtensorMap E, xn[5], a_attn[5], a_dn[5], h[5]; } tc_g;
    int* pinned_err = nullptr;
    // prompt columns: a second set of step buffers, `B` columns wide, that shares this session's KV
    // pool, delta-net state and stream; a column is one prompt token of one sequence
    mlb_session* cols = nullptr;            // owned by the session it serves
    mlb_session* parent = nullptr;          // set in the column set
    bool cols_tried = false;
    int* seq_of = nullptr;                  // [B] in the column set: column -> sequence of the parent
};

namespace mlb {

static int sess_alloc(mlb_session* s, void** p, size_t bytes, bool zero) {
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
    if (e != cudaSuccess) return fail(MLB_E_NOMEM, "cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    s->allocs.push_back(*p);
    if (zero) CU(cudaMemset(*p, 0, bytes ? bytes : 16));
    return MLB_OK;
}

// Queue the read-back of the device error word; call before the stream synchronisation.
static int queue_err_readback(mlb_session* s) {
    CU(cudaMemcpyAsync(s->pinned_err, s->dev_err, 4, cudaMemcpyDeviceToHost, s->stream));
    return MLB_OK;
}
// After the synchronisation: a bounded device-side wait ran out somewhere in the step.
static int check_err_readback(mlb_session* s) {
    if (*s->pinned_err == 0) return MLB_OK;
    const int code = *s->pinned_err;
    *s->pinned_err = 0;
    cudaMemsetAsync(s->dev_err, 0, 4, s->stream);
    cudaStreamSynchronize(s->stream);
    return fail(MLB_E_TIMEOUT, "a bounded device-side wait ran out (code %d: %s); the results of this call are invalid", code,
                code == 1 ? "producer waiting for a free ring stage"
                          : (code == 2 ? "consumer waiting for a weight chunk" : "consumer waiting for another CTA's results"));
}

static void free_session(mlb_session* s) {
    if (!s) return;
    cudaSetDevice(s->m->device);
    if (s->stream) cudaStreamSynchronize(s->stream);
    if (s->cols) free_session(s->cols);
    for (auto& g : s->graphs) if (g) cudaGraphExecDestroy(g);
    for (auto& g : s->tgraphs) if (g) cudaGraphExecDestroy(g);
    for (void* p : s->allocs) cudaFree(p);
    if (s->pinned_tok) cudaFreeHost(s->pinned_tok);
    if (s->pinned_out) cudaFreeHost(s->pinned_out);
    if (s->pinned_err) cudaFreeHost(s->pinned_err);
    if (s->stream && !s->parent) cudaStreamDestroy(s->stream);      // a column set runs on its parent's stream
    delete s;
}

// Host mirror of seq_active for the decode chains.
static bool seq_live(const mlb_session* s, int b) { return s->h_pos[b] < s->max_ctx && !s->h_stopped[b]; }
// After a decode call returned `n` ids of sequence b (ring order): advance the mirror, stop at the stop token,
// blank what lies behind it.
static void note_outputs(mlb_session* s, int b, int32_t* out, int n) {
    int room = seq_live(s, b) ? std::min(n, s->max_ctx - s->h_pos[b]) : 0;
    for (int i = 0; i < room; ++i) {
        if (s->stop_token >= 0 && out[i] == s->stop_token) {
            room = i + 1;
            s->h_stopped[b] = 1;
            break;
        }
    }
    for (int i = room; i < n; ++i) out[i] = -1;
    s->h_pos[b] += room;
}

static StepCtl make_ctl(mlb_session* s, int kind) {
    StepCtl c;
    c.B = s->B;
    c.vocab = s->m->cfg.vocab;
    c.pos = s->pos;
    c.tok = s->tok;
    c.limit = kind == CHAIN_PREFILL ? s->limit_prefill : s->limit_decode;
    c.stop_token = kind == CHAIN_PREFILL ? -1 : s->stop_token;
    c.prompt = kind == CHAIN_PREFILL ? s->prompt : nullptr;
    c.prompt_stride = s->max_ctx;
    c.out_ring = s->out_ring;
    c.out_idx = s->out_idx;
    c.out_cap = s->parent ? 0 : s->max_ctx;     // a column set has no output ring
    c.tok_src = s->ctl_host_io == 2 ? s->pinned_tok : nullptr;
    c.host_out = s->ctl_host_io ? s->pinned_out : nullptr;
    c.host_err = s->ctl_host_io ? s->pinned_err : nullptr;
    c.dev_err = s->dev_err;
    return c;
}

static int pick_bt(int B, size_t per_seq_floats) {
    int bt = B >= 8 ? 8 : (B >= 4 ? 4 : (B >= 2 ? 2 : 1));
    while (bt > 1 && (size_t)bt * per_seq_floats * 4 > 200 * 1024) bt >>= 1;
    return bt;
}

// Launch with the programmatic-dependent-launch attribute: the kernel may start while its
// predecessor in the stream still runs and orders itself with griddepcontrol.wait.
template <typename... KArgs, typename... Args>
static cudaError_t launch_chain(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                Args... args) {
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// launch_chain for a grid whose z extent is one thread-block cluster (cluster_z CTAs share an output tile).
template <typename... KArgs, typename... Args>
static cudaError_t launch_cluster(bool pdl, int cluster_z, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args... args) {
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = (unsigned)cluster_z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Shape of one tensor-core GEMM launch: batch tile (UMMA N), how many CTAs of a cluster split the k-blocks of
// an output tile, and the ring. Measured on B200: a tcgen05.mma of M = 128 costs about 0.1 us whatever its N
// (16..128), so a CTA's k-loop takes 0.4 us per 64-wide k-block (0.8 with two weight tiles) whatever the ring
// depth, and is the time of the kernel unless the k-blocks are spread over CTAs. Exchanging partial
// accumulators through distributed shared memory costs 2-3 us per launch with clusters of 4 and 8, more than
// it saves at cfg1's sizes (8-23 k-blocks per tile); pairs pay off at small batches (cfg1 step at 32 sequences:
// 452 -> 424 us) and are neutral at 256. Larger clusters are taken only where a CTA keeps 8 k-blocks or more
// (cfg4: 32-90 k-blocks per tile and few tiles). MLB_TC_SPLIT sets the limit by hand. One wave of CTAs per
// launch where possible.
static TcShape tc_pick_shape(const mlb_session* s, int N, int nkb_all, int na, bool w8, int nacc) {
    const int tiles_m = (N + kTcM - 1) / kTcM;
    const int cap = std::min(256, (s->B + 15) / 16 * 16);
    TcShape best{};
    double best_cost = -1.0;
    for (int nb = 16; nb <= cap && nacc * nb <= 512; nb <<= 1) {
        for (int li = 0; li < 4; ++li) {
            const int S = 1 << li;
            if (S > s->tc_max_split || S > nkb_all) break;
            // clusters of 4 and 8 only where a CTA keeps 8 k-blocks or more: their exchange costs 2-3 us
            if (S > 2 && !s->tc_split_forced && (nkb_all + S - 1) / S < 8) break;
            if (S > 1 && (nb % S != 0 || s->tc_cluster_cap[li] <= 0)) continue;
            const size_t stage_bytes = (size_t)na * kTcM * 128 + (size_t)nb * 128;      // FP8 codes land inside the operand tile
            const int kpc = (nkb_all + S - 1) / S;
            int st = (int)std::max<size_t>(1, std::min<size_t>(std::min(kpc, 12), kTcRingBytes / stage_bytes));
            const int g = st >= kpc ? 1 : (st >= 8 ? 4 : (st >= 4 ? 2 : 1));
            st -= st % g;
            const size_t body = std::max((size_t)st * stage_bytes, S > 1 ? (size_t)nacc * nb * kTcM * 4 : (size_t)0);
            const size_t smem = 1024 + kTcHeadBytes + kTcStageBytes + body;
            if (smem > 227 * 1024) continue;
            const long ctas = (long)tiles_m * ((s->B + nb - 1) / nb) * S;
            const long resident = S == 1 ? s->sm_count : (long)s->tc_cluster_cap[li] * S;
            const long waves = (ctas + resident - 1) / resident;
            const double t_loop = 0.4 * na * kpc;
            const double t_red = S > 2 ? 2.5 + (double)nacc * nb * 512.0 / 65536.0 : (S > 1 ? 0.5 + (double)nacc * nb * 512.0 / 65536.0 : 0.0);
            const double t_epi = 0.25 * ((nb / S + 15) / 16);
            const double cost = (double)waves * (t_loop + t_red + t_epi + 0.5);
            if (best_cost < 0 || cost < best_cost) {
                best_cost = cost;
                uint32_t cols = 32;
                while (cols < (uint32_t)(nacc * nb)) cols <<= 1;
                best = TcShape{nb, S, st, g, smem, cols};
            }
        }
    }
    return best;
}
static int nb_index(int nb) { return nb == 16 ? 0 : nb == 32 ? 1 : nb == 64 ? 2 : nb == 128 ? 3 : 4; }

template <typename T, typename T2, typename KVT>
struct Chain {
    // TMA-streamed variant: one contiguous slab of rows per CTA (one head per CTA for QKV).
    template <int MODE>
    static int sgemv(mlb_session* s, const StepCtl& c, GemvParams p, Recorder* rec, const char* name, bool* done) {
        *done = false;
        // Worth it only when the matrix is large: below a few MB the per-thread-load kernel's
        // shorter latency chain wins (measured on the 1-GPU latency configuration).
        const size_t mat_bytes = (size_t)p.N * p.K * sizeof(T) * (MODE == GEMV_SWIGLU ? 2 : 1);
        if (!s->force_sgemv && mat_bytes < (4u << 20)) return MLB_OK;
        SgemvGeom g;
        g.stage_bytes = s->sg_stage_kb * 1024;
        if ((size_t)p.K * sizeof(T) > (size_t)g.stage_bytes || (size_t)p.Kp * sizeof(T2) > (size_t)g.stage_bytes) return MLB_OK;
        int grid_x;
        if (MODE == GEMV_QKV) {
            // whole heads when the per-head norm needs them, else 32-row groups (RoPE pairs stay together)
            g.rows_per_cta = p.qk_norm ? p.hd : 32;
            grid_x = p.N / g.rows_per_cta;
        } else {
            const int n_ctas = std::max(1, std::min(s->sm_count, (p.N + 3) / 4));
            g.rows_per_cta = (p.N + n_ctas - 1) / n_ctas;
            grid_x = (p.N + g.rows_per_cta - 1) / g.rows_per_cta;
        }
        auto up4 = [](int v) { return (v + 3) / 4 * 4; };
        int off = 0;
        g.off_xs = off; off += up4(p.K);
        g.off_xs2 = off; off += up4(std::max(p.Kp, 4));
        g.off_outs = off; off += up4(std::max(p.hd, 64));
        g.off_pacc = off; off += up4(g.rows_per_cta + 4);
        g.off_red = off; off += 64;
        off = (off + 31) / 32 * 32;
        g.off_bar = off; off += 8 * 4;
        off = (off + 31) / 32 * 32;
        g.off_ring = off;
        const size_t fixed = (size_t)off * 4;
        if (fixed + 3 * (size_t)g.stage_bytes > 210 * 1024) return MLB_OK;
        g.n_stages = (int)std::min<size_t>(s->sg_max_stages, (210 * 1024 - fixed) / g.stage_bytes);
        g.err = s->dev_err;
        const size_t smem = fixed + (size_t)g.n_stages * g.stage_bytes;
        if (rec) {
            const uint64_t wbytes = (uint64_t)p.N * p.K * sizeof(T) * (MODE == GEMV_SWIGLU ? 2 : 1) +
                                    (uint64_t)p.N * p.Kp * sizeof(T2) + (p.wscale ? (uint64_t)p.N * 4 : 0);
            const uint64_t abytes = (uint64_t)s->B * ((uint64_t)p.K + p.N) * 4;
            int rc = rec->begin(name, wbytes + abytes, 2ull * p.N * (p.K + p.Kp) * s->B * (MODE == GEMV_SWIGLU ? 2 : 1));
            if (rc) return rc;
        }
        cudaError_t e = launch_chain(s->use_pdl, sgemv_kernel<T, T2, KVT, MODE>, dim3(grid_x, s->B), dim3(kSgThreads), smem,
                                     s->stream, c, p, g);
        if (e != cudaSuccess) return fail(MLB_E_CUDA, "launch of %s (streamed) failed: %s", name, cudaGetErrorString(e));
        *done = true;
        if (rec) return rec->end();
        return MLB_OK;
    }

    template <int MODE>
    static int gemv(mlb_session* s, const StepCtl& c, GemvParams p, int R, Recorder* rec, const char* name) {
        if (s->use_sgemv) {
            bool done = false;
            int rc = sgemv<MODE>(s, c, p, rec, name, &done);
            if (rc || done) return rc;
        }
        p.R = R;
        const size_t per_seq = (size_t)p.K + p.Kp + R + 1 + 8;
        const int BT = pick_bt(s->B, per_seq);
        if (per_seq * 4 > 200 * 1024) return fail(MLB_E_UNSUPPORTED, "projection input of %d floats does not fit shared memory", p.K);
        const int rwf = BT == 1 ? 2 : 4;                                  // GemvShape<BT>::RW
        const int rw = MODE == GEMV_SWIGLU ? rwf / 2 : rwf;
        const int warps = std::max(1, std::min(8, (R + rw - 1) / rw));
        dim3 grid((p.N + R - 1) / R, (s->B + BT - 1) / BT);
        const size_t smem = (size_t)BT * per_seq * 4;
        if (rec) {
            const uint64_t wbytes = (uint64_t)p.N * p.K * sizeof(T) * (MODE == GEMV_SWIGLU ? 2 : 1) +
                                    (uint64_t)p.N * p.Kp * sizeof(T2) + (p.wscale ? (uint64_t)p.N * 4 : 0);
            const uint64_t abytes = (uint64_t)s->B * ((uint64_t)p.K + p.N) * 4;
            int rc = rec->begin(name, wbytes + abytes, 2ull * p.N * (p.K + p.Kp) * s->B * (MODE == GEMV_SWIGLU ? 2 : 1));
            if (rc) return rc;
        }
        cudaError_t e;
        switch (BT) {
            case 1: e = launch_chain(s->use_pdl, gemv_kernel<T, T2, KVT, 1, MODE>, grid, dim3(warps * 32), smem, s->stream, c, p); break;
            case 2: e = launch_chain(s->use_pdl, gemv_kernel<T, T2, KVT, 2, MODE>, grid, dim3(warps * 32), smem, s->stream, c, p); break;
            case 4: e = launch_chain(s->use_pdl, gemv_kernel<T, T2, KVT, 4, MODE>, grid, dim3(warps * 32), smem, s->stream, c, p); break;
            default: e = launch_chain(s->use_pdl, gemv_kernel<T, T2, KVT, 8, MODE>, grid, dim3(warps * 32), smem, s->stream, c, p); break;
        }
        if (e != cudaSuccess) return fail(MLB_E_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e));
        if (rec) return rec->end();
        return MLB_OK;
    }

    template <int MODE>
    static int configure_mode() {
        const int big = 200 * 1024;
        CU(cudaFuncSetAttribute(sgemv_kernel<T, T2, KVT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 212 * 1024));
        CU(cudaFuncSetAttribute(gemv_kernel<T, T2, KVT, 1, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
        CU(cudaFuncSetAttribute(gemv_kernel<T, T2, KVT, 2, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
        CU(cudaFuncSetAttribute(gemv_kernel<T, T2, KVT, 4, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
        CU(cudaFuncSetAttribute(gemv_kernel<T, T2, KVT, 8, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
        return MLB_OK;
    }
    static int configure() {
        int rc;
        if ((rc = configure_mode<GEMV_RAW>())) return rc;
        if ((rc = configure_mode<GEMV_RESID>())) return rc;
        if ((rc = configure_mode<GEMV_SWIGLU>())) return rc;
        if ((rc = configure_mode<GEMV_QKV>())) return rc;
        if ((rc = configure_mode<GEMV_LMHEAD>())) return rc;
        return MLB_OK;
    }

    template <int HD>
    static int attn_g(mlb_session* s, const StepCtl& c, const AttnParams& p0, int G) {
        AttnParams p = p0;
        p.hg = 1;
        // few CTAs (small batch): two query heads per CTA, G/2 CTAs per kv head (cfg4 at batch 1: 1.28 -> 1.14 ms
        // per step); with the GPU already full the extra CTAs only re-read K/V (62 -> 69 us at 64 sequences)
        if (G >= 4 && G % 2 == 0 && s->splits * p.kv_heads * s->B < 2 * s->sm_count) { p.hg = G / 2; G = 2; }
        dim3 grid(s->splits, p.kv_heads * p.hg, s->B);
        cudaError_t e;
        switch (G) {
            case 1: e = launch_chain(s->use_pdl, attn_decode_kernel<KVT, HD, 1>, grid, dim3(128), 0, s->stream, c, p); break;
            case 2: e = launch_chain(s->use_pdl, attn_decode_kernel<KVT, HD, 2>, grid, dim3(128), 0, s->stream, c, p); break;
            case 4: e = launch_chain(s->use_pdl, attn_decode_kernel<KVT, HD, 4>, grid, dim3(128), 0, s->stream, c, p); break;
            default: e = launch_chain(s->use_pdl, attn_decode_kernel<KVT, HD, 8>, grid, dim3(128), 0, s->stream, c, p); break;
        }
        if (e != cudaSuccess) return fail(MLB_E_CUDA, "attention launch failed: %s", cudaGetErrorString(e));
        return MLB_OK;
    }

    // Launch shape of the embedding kernel: with per-layer embeddings and a small batch, the rows
    // of a sequence are spread over several CTAs of 64 threads (one projection row per thread).
    static int embed_split(int B, int d, int ple) {
        if (ple <= 0) return 1;
        return std::max(1, std::min((d + 63) / 64, 1024 / std::max(1, B)));
    }
    static dim3 embed_grid(int B, int d, int ple) { return dim3(B, embed_split(B, d, ple)); }
    static dim3 embed_block(int B, int d, int ple) { return dim3(embed_split(B, d, ple) > 1 ? 64 : 256); }

    // One decode (or prefill) step of a batch-1 session as a single cooperative kernel over all
    // SMs (plus the sampler for top-k).
    static int run_grid(mlb_session* s, int kind, const StepCtl& c, Recorder* rec, int* n_launches) {
        int rc, launches = 0;
        if (rec) {
            uint64_t w, kv, st, rows;
            mlb_session_step_bytes(s, &w, &kv, &st, &rows);
            if ((rc = rec->begin(s->use_lean ? "lean_decode_step" : "grid_decode_step", w + kv + st + rows, 0))) return rc;
        }
        if (s->use_lean) {
            LeanParams lp = s->lean;
            lp.tok_arg = s->tok_arg;
            lp.with_lm_head = kind == CHAIN_PREFILL ? 0 : 1;
            lp.do_pick = kind == CHAIN_GREEDY ? 1 : 0;
            CU(lean_kernel_launch(s->lean_idx, s->m->cfg.kv_dtype, s->lean_smem, s->stream, c, lp));
        } else {
            GridParams gp = s->grid;
            gp.tok_arg = s->tok_arg;
            gp.with_lm_head = kind == CHAIN_PREFILL ? 0 : 1;
            gp.do_pick = kind == CHAIN_GREEDY ? 1 : 0;
            CU(grid_kernel_launch(s->m->cfg.weight_dtype, s->m->cfg.kv_dtype, s->grid_ctas, s->grid_smem, s->stream, c, gp));
        }
        if (rec && (rc = rec->end())) return rc;
        ++launches;
        if (kind == CHAIN_TOPK) {
            SampleParams sp;
            sp.logits = s->logits; sp.V = s->m->cfg.vocab; sp.top_k = s->cur_topk; sp.temperature = s->cur_temp; sp.seeds = s->seeds;
            if (rec && (rc = rec->begin("sample_topk_philox", (uint64_t)s->B * s->m->cfg.vocab * 4 * 5, 0))) return rc;
            CU(launch_chain(false, sample_topk_kernel, dim3(s->B), dim3(256), 0, s->stream, c, sp));
            if (rec && (rc = rec->end())) return rc;
            ++launches;
        }
        if (n_launches) *n_launches = launches;
        return MLB_OK;
    }

    // One tensor-core projection. `normed`: the activation operand is bf16(x * gain) and the accumulator
    // columns are scaled by 1 / rms(x) from the partial sums its producer left. `next_gain` (RESID): also
    // write the operand and the partial sums for the next norm. `ext`: the per-layer embedding pair whose
    // k-blocks follow the main operands' (RESID of the down projection).
    template <int MODE>
    static int gemm_tc(mlb_session* s, const StepCtl& c, const CUtensorMap& A, const CUtensorMap& A2, const CUtensorMap* Bmaps, int N, int K,
                       float* y, bf16_t* h16, bool normed, const float* next_gain, const mlb_session::TcLayerMaps* ext,
                       const QkvPostParams* q, const float* sA, const float* sA2, Recorder* rec, const char* name) {
        GemmTcParams p;
        const int ple = s->m->cfg.ple_dim;
        const int na = MODE == TC_SWIGLU ? 2 : 1;
        p.nkb_x = ext ? (ple + kTcKB - 1) / kTcKB : 0;
        constexpr bool w8 = sizeof(T) == 1;
        const int nacc = (MODE == TC_SWIGLU || (w8 && MODE == TC_RESID)) ? 2 : 1;
        const TcShape sh = ext ? s->tc_shape_down : tc_pick_shape(s, N, (K + kTcKB - 1) / kTcKB, na, w8, nacc);
        if (sh.nb == 0) return fail(MLB_E_UNSUPPORTED, "%s: no launch shape fits", name);
        const int nb = sh.nb;
        p.N = N; p.K = K; p.B = s->B; p.Nb = nb;
        p.stages = sh.stages; p.group = sh.group; p.tmem_cols = sh.tmem_cols;
        p.y = y; p.resid = MODE == TC_RESID ? y : nullptr; p.h16 = h16; p.err = s->dev_err;
        p.sA = sA; p.sA2 = sA2;
        p.trace = s->tc_trace ? s->tc_trace + 8 * (size_t)(s->tc_trace_n++ % 64) : nullptr;
        p.ssq_in = normed ? s->tc_ssq : nullptr; p.ssq_parts = (s->m->cfg.dim + kTcM - 1) / kTcM; p.eps = s->m->cfg.rms_eps;
        p.xg16 = next_gain ? s->xn16 : nullptr; p.gain_next = next_gain; p.ssq_out = next_gain ? s->tc_ssq : nullptr;
        const size_t smem = sh.smem;
        dim3 grid((N + kTcM - 1) / kTcM, (s->B + nb - 1) / nb, sh.split);
        int rc;
        if (rec && (rc = rec->begin(name, ((uint64_t)N * K * sizeof(T) + (uint64_t)N * (ext ? ple : 0) * 2) * na + (uint64_t)s->B * K * 2 + (uint64_t)s->B * N * 4,
                                    2ull * N * (K + (ext ? ple : 0)) * s->B * na)))
            return rc;
        QkvPostParams q0{};
        const CUtensorMap& Ax = ext ? ext->pleP : A;
        const CUtensorMap& Bx = ext ? ext->pleT : A;
        cudaError_t e = launch_cluster(s->use_pdl, sh.split, gemm_tc_kernel<MODE, KVT, T>, grid, dim3(kTcThreads), smem, s->stream, A, A2, Bmaps[nb_index(nb)], Ax, Bx, p,
                                       c, q ? *q : q0);
        if (e != cudaSuccess) return fail(MLB_E_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e));
        if (rec) return rec->end();
        return MLB_OK;
    }

    // Large-batch step: projections as tcgen05 GEMMs on bf16 operands with the element-wise work in their
    // epilogues; per layer: projection, attention / delta-net, o-projection, gate-up, down.
    static int run_tc(mlb_session* s, int kind, const StepCtl& c, Recorder* rec, int* n_launches) {
        if (std::is_same<T, float>::value) return fail(MLB_E_UNSUPPORTED, "tensor-core projections need bf16 or FP8 weights");
        const mlb_model* m = s->m;
        const mlb_config& cfg = m->cfg;
        const int d = cfg.dim, F = cfg.ffn_dim, B = s->B, ple = cfg.ple_dim;
        int launches = 0, rc;
        if (rec && (rc = rec->begin("embed_ple_gather_norm", (uint64_t)B * d * 8 + (uint64_t)B * ple * 2 * cfg.layers, 0))) return rc;
        CU(launch_chain(s->use_pdl, embed_tc_kernel<T>, dim3(B, (d + kTcM - 1) / kTcM), dim3(128), (size_t)ple * 4, s->stream, c,
                        static_cast<const T*>(m->E), static_cast<const float*>(m->Es), d, static_cast<const StepLayer*>(s->step_layers), cfg.layers, ple,
                        static_cast<const float*>(m->layers[0].g1), s->x, s->xn16, s->tc_ssq, s->tple16));
        if (rec && (rc = rec->end())) return rc;
        ++launches;
        for (int i = 0; i < cfg.layers; ++i) {
            const DevLayer& L = m->layers[i];
            const mlb_session::TcLayerMaps& M = s->tc_maps[i];
            if (L.type == MLB_LAYER_ATTENTION) {
                QkvPostParams q;
                q.nq = L.nq; q.nk = L.nk; q.nv = L.nv; q.ng = L.ng; q.hd = cfg.head_dim;
                q.kv_heads = cfg.kv_heads; q.qk_norm = cfg.qk_norm; q.eps = cfg.rms_eps; q.gq = L.gq; q.gk = L.gk; q.rope = m->rope;
                q.kpool = s->kpool[i]; q.vpool = s->vpool[i]; q.page_table = s->page_table; q.pt_stride = s->max_pages;
                q.qbuf = s->qbuf; q.gbuf = s->gbuf;
                if ((rc = gemm_tc<TC_QKV>(s, c, M.qkv, M.qkv, s->tc_g.xn, L.n_qkv, d, nullptr, nullptr, true, nullptr, nullptr, &q, L.Sqkv, nullptr, rec,
                                          "qkv_gemm_tcgen05_norm_rope_kvappend")))
                    return rc;
                ++launches;
                AttnParams a;
                a.kpool = s->kpool[i]; a.vpool = s->vpool[i];
                a.page_table = s->page_table; a.pt_stride = s->max_pages;
                a.qbuf = s->qbuf; a.gbuf = L.ng ? s->gbuf : nullptr; a.abuf = s->abuf; a.abuf16 = s->a16;
                a.part = s->part; a.ticket = s->attn_ticket;
                a.heads = cfg.heads; a.kv_heads = cfg.kv_heads; a.num_pages = 0; a.err = nullptr; a.min_pages_per_split = s->attn_min_pps;
                if (rec) {
                    uint64_t kvb = 0, fl = 0;
                    for (int b = 0; b < B; ++b) {
                        if (!seq_live(s, b)) continue;
                        kvb += 2ull * cfg.kv_heads * cfg.head_dim * sizeof(KVT) * (s->h_pos[b] + 1);
                        fl += 4ull * cfg.heads * cfg.head_dim * (s->h_pos[b] + 1);
                    }
                    if ((rc = rec->begin("attn_flash_decode_paged", kvb, fl))) return rc;
                }
                const int G = cfg.heads / cfg.kv_heads;
                if (cfg.head_dim == 64) rc = attn_g<64>(s, c, a, G); else rc = attn_g<128>(s, c, a, G);
                if (rc) return rc;
                if (rec && (rc = rec->end())) return rc;
                ++launches;
            } else {
                if ((rc = gemm_tc<TC_RAW>(s, c, M.qkv, M.qkv, s->tc_g.xn, L.n_qkv, d, s->raw, nullptr, true, nullptr, nullptr, nullptr, L.Sqkv, nullptr, rec,
                                          "deltanet_proj_gemm_tcgen05")))
                    return rc;
                ++launches;
                const int dk = cfg.dn_key_dim, dv = cfg.dn_value_dim, H = cfg.heads;
                if (rec && (rc = rec->begin("deltanet_state_update", (uint64_t)B * 2ull * H * dk * dv * 4, (uint64_t)B * 6ull * H * dk * dv))) return rc;
                if (s->parent) {
                    // prompt columns: the recurrence runs over the columns of a sequence in order
                    dim3 ngrid(H, B), grid((dv + 31) / 32, H, B);
                    if (dk == 64) {
                        CU(launch_chain(s->use_pdl, delta_cols_norm_kernel<64>, ngrid, dim3(64), 0, s->stream, c, s->raw, s->raw_stride, H, dv, 1e-6f));
                        CU(launch_chain(s->use_pdl, delta_net_cols_kernel<64>, grid, dim3(256), 0, s->stream, c, static_cast<const int*>(s->seq_of), B, static_cast<const float*>(s->raw), s->raw_stride, s->state[i], H, dv, s->abuf, s->a16));
                    } else {
                        CU(launch_chain(s->use_pdl, delta_cols_norm_kernel<128>, ngrid, dim3(64), 0, s->stream, c, s->raw, s->raw_stride, H, dv, 1e-6f));
                        CU(launch_chain(s->use_pdl, delta_net_cols_kernel<128>, grid, dim3(256), 0, s->stream, c, static_cast<const int*>(s->seq_of), B, static_cast<const float*>(s->raw), s->raw_stride, s->state[i], H, dv, s->abuf, s->a16));
                    }
                    ++launches;
                } else {
                    dim3 grid((dv + 31) / 32, H, B);
                    if (dk == 64) CU(launch_chain(s->use_pdl, delta_net_kernel<64>, grid, dim3(256), 0, s->stream, c, static_cast<const float*>(s->raw), s->raw_stride, s->state[i], H, dv, s->abuf, s->a16, 1e-6f));
                    else CU(launch_chain(s->use_pdl, delta_net_kernel<128>, grid, dim3(256), 0, s->stream, c, static_cast<const float*>(s->raw), s->raw_stride, s->state[i], H, dv, s->abuf, s->a16, 1e-6f));
                }
                if (rec && (rc = rec->end())) return rc;
                ++launches;
            }
            const CUtensorMap* amap = L.type == MLB_LAYER_ATTENTION ? s->tc_g.a_attn : s->tc_g.a_dn;
            if ((rc = gemm_tc<TC_RESID>(s, c, M.o, M.o, amap, d, L.o_in, s->x, nullptr, false, L.g2, nullptr, nullptr, L.So, nullptr, rec,
                                        "oproj_gemm_tcgen05_residual_norm")))
                return rc;
            ++launches;
            if ((rc = gemm_tc<TC_SWIGLU>(s, c, M.w1a, M.w1b, s->tc_g.xn, F, d, nullptr, s->h16, true, nullptr, nullptr, nullptr, L.S1a, L.S1b, rec,
                                         "ffn_gateup_gemm_tcgen05_swiglu")))
                return rc;
            ++launches;
            const bool last = i + 1 == cfg.layers;
            const float* g_next = last ? m->g_final : m->layers[i + 1].g1;
            if ((rc = gemm_tc<TC_RESID>(s, c, M.w2, M.w2, s->tc_g.h, d, F, s->x, nullptr, false, g_next,
                                        (!last && ple > 0) ? &s->tc_maps[i + 1] : nullptr, nullptr, L.S2, nullptr, rec, "ffn_down_gemm_tcgen05_residual_ple_norm")))
                return rc;
            ++launches;
        }
        if (kind == CHAIN_PREFILL && s->parent) {
            // prompt columns: positions and tokens of the next chunk come from the host
        } else if (kind == CHAIN_PREFILL) {
            if (rec && (rc = rec->begin("advance_prompt", (uint64_t)B * 12, 0))) return rc;
            CU(launch_chain(s->use_pdl, advance_kernel, dim3((B + 127) / 128), dim3(128), 0, s->stream, c));
            if (rec && (rc = rec->end())) return rc;
            ++launches;
        } else {
            if ((rc = gemm_tc<TC_RAW>(s, c, s->tc_g.E, s->tc_g.E, s->tc_g.xn, cfg.vocab, d, s->logits, nullptr, true, nullptr, nullptr, nullptr, static_cast<const float*>(m->Es), nullptr, rec,
                                      "lmhead_gemm_tcgen05")))
                return rc;
            ++launches;
            if (kind == CHAIN_GREEDY) {
                if (rec && (rc = rec->begin("argmax_pick", (uint64_t)B * cfg.vocab * 4, 0))) return rc;
                CU(launch_chain(s->use_pdl, argmax_advance_kernel, dim3(B), dim3(256), 0, s->stream, c, static_cast<const float*>(s->logits), cfg.vocab));
                if (rec && (rc = rec->end())) return rc;
            } else {
                SampleParams sp;
                sp.logits = s->logits; sp.V = cfg.vocab; sp.top_k = s->cur_topk; sp.temperature = s->cur_temp; sp.seeds = s->seeds;
                if (rec && (rc = rec->begin("sample_topk_philox", (uint64_t)B * cfg.vocab * 4 * 5, 0))) return rc;
                CU(launch_chain(s->use_pdl, sample_topk_kernel, dim3(B), dim3(256), 0, s->stream, c, sp));
                if (rec && (rc = rec->end())) return rc;
            }
            ++launches;
        }
        if (n_launches) *n_launches = launches;
        return MLB_OK;
    }

    // One decode (or prefill) step as a chain of launches on the session's stream.
    static int run(mlb_session* s, int kind, Recorder* rec, int* n_launches) {
        const mlb_model* m = s->m;
        const mlb_config& cfg = m->cfg;
        const StepCtl c = make_ctl(s, kind);
        const int d = cfg.dim, F = cfg.ffn_dim, B = s->B, p = cfg.ple_dim;
        int launches = 0, rc;
        if (s->use_lean || s->use_grid) return run_grid(s, kind, c, rec, n_launches);
        if (s->use_tc) return run_tc(s, kind, c, rec, n_launches);

        if (rec && (rc = rec->begin("embed_ple_gather", (uint64_t)B * (d * sizeof(T) + (uint64_t)p * sizeof(T2) + (uint64_t)d * 4) + (uint64_t)d * p * sizeof(T2), 0))) return rc;
        CU(launch_chain(s->use_pdl, embed_kernel<T, T2>, embed_grid(B, d, p), embed_block(B, d, p), (size_t)p * 4, s->stream, c,
                        static_cast<const T*>(m->E), static_cast<const float*>(m->Es), d, static_cast<const T2*>(m->layers[0].pleT),
                        static_cast<const T2*>(m->layers[0].pleP), p, s->x));
        if (rec && (rc = rec->end())) return rc;
        ++launches;

        for (int i = 0; i < cfg.layers; ++i) {
            const DevLayer& L = m->layers[i];
            GemvParams g;
            std::memset(&g, 0, sizeof g);
            g.W = L.Wqkv; g.wscale = L.Sqkv; g.N = L.n_qkv; g.K = d;
            g.xin = s->x; g.gain = L.g1; g.eps = cfg.rms_eps; g.do_norm = 1;
            if (L.type == MLB_LAYER_ATTENTION) {
                g.nq = L.nq; g.nk = L.nk; g.nv = L.nv; g.ng = L.ng;
                g.hd = cfg.head_dim; g.kv_heads = cfg.kv_heads; g.qk_norm = cfg.qk_norm;
                g.gq = L.gq; g.gk = L.gk; g.rope = m->rope;
                g.kpool = s->kpool[i]; g.vpool = s->vpool[i];
                g.page_table = s->page_table; g.pt_stride = s->max_pages;
                g.qbuf = s->qbuf; g.gbuf = s->gbuf;
                const int R = cfg.qk_norm ? cfg.head_dim : 16;
                if ((rc = gemv<GEMV_QKV>(s, c, g, R, rec, "qkv_gemv_norm_rope_kvappend"))) return rc;
                ++launches;
                AttnParams a;
                a.kpool = s->kpool[i]; a.vpool = s->vpool[i];
                a.page_table = s->page_table; a.pt_stride = s->max_pages;
                a.qbuf = s->qbuf; a.gbuf = L.ng ? s->gbuf : nullptr; a.abuf = s->abuf; a.abuf16 = nullptr;
                a.part = s->part; a.ticket = s->attn_ticket;
                a.heads = cfg.heads; a.kv_heads = cfg.kv_heads; a.num_pages = 0; a.err = nullptr; a.min_pages_per_split = s->attn_min_pps;
                if (rec) {
                    uint64_t kvb = 0, fl = 0;
                    for (int b = 0; b < B; ++b) {
                        if (!seq_live(s, b)) continue;
                        kvb += 2ull * cfg.kv_heads * cfg.head_dim * sizeof(KVT) * (s->h_pos[b] + 1);
                        fl += 4ull * cfg.heads * cfg.head_dim * (s->h_pos[b] + 1);
                    }
                    if ((rc = rec->begin("attn_flash_decode_paged", kvb, fl))) return rc;
                }
                const int G = cfg.heads / cfg.kv_heads;
                if (cfg.head_dim == 64) rc = attn_g<64>(s, c, a, G); else rc = attn_g<128>(s, c, a, G);
                if (rc) return rc;
                if (rec && (rc = rec->end())) return rc;
                ++launches;
            } else {
                g.y = s->raw;
                if ((rc = gemv<GEMV_RAW>(s, c, g, 16, rec, "deltanet_proj_gemv_norm"))) return rc;
                ++launches;
                const int dk = cfg.dn_key_dim, dv = cfg.dn_value_dim, H = cfg.heads;
                if (rec && (rc = rec->begin("deltanet_state_update", (uint64_t)B * 2ull * H * dk * dv * 4, (uint64_t)B * 6ull * H * dk * dv))) return rc;
                dim3 grid((dv + 31) / 32, H, B);
                if (dk == 64) CU(launch_chain(s->use_pdl, delta_net_kernel<64>, grid, dim3(256), 0, s->stream, c, static_cast<const float*>(s->raw), s->raw_stride, s->state[i], H, dv, s->abuf, static_cast<bf16_t*>(nullptr), 1e-6f));
                else CU(launch_chain(s->use_pdl, delta_net_kernel<128>, grid, dim3(256), 0, s->stream, c, static_cast<const float*>(s->raw), s->raw_stride, s->state[i], H, dv, s->abuf, static_cast<bf16_t*>(nullptr), 1e-6f));
                if (rec && (rc = rec->end())) return rc;
                ++launches;
            }
            // output projection + residual (in place on the residual stream)
            std::memset(&g, 0, sizeof g);
            g.W = L.Wo; g.wscale = L.So; g.N = d; g.K = L.o_in;
            g.xin = s->abuf; g.y = s->x; g.resid = s->x;
            if ((rc = gemv<GEMV_RESID>(s, c, g, d <= 1024 ? 8 : 16, rec, "oproj_gemv_residual"))) return rc;
            ++launches;
            // FFN gate/up with RMS norm prologue and SwiGLU epilogue
            std::memset(&g, 0, sizeof g);
            g.W = L.W1a; g.Wb = L.W1b; g.wscale = L.S1a; g.wscale_b = L.S1b; g.N = F; g.K = d;
            g.xin = s->x; g.gain = L.g2; g.eps = cfg.rms_eps; g.do_norm = 1; g.y = s->hbuf;
            if ((rc = gemv<GEMV_SWIGLU>(s, c, g, 8, rec, "ffn_gateup_gemv_norm_swiglu"))) return rc;
            ++launches;
            // FFN down + residual (+ the next layer's per-layer embedding)
            std::memset(&g, 0, sizeof g);
            g.W = L.W2; g.wscale = L.S2; g.N = d; g.K = F;
            g.xin = s->hbuf; g.y = s->x; g.resid = s->x;
            if (p > 0 && i + 1 < cfg.layers) { g.P = m->layers[i + 1].pleP; g.Ptab = m->layers[i + 1].pleT; g.Kp = p; }
            if ((rc = gemv<GEMV_RESID>(s, c, g, d <= 1024 ? 8 : 16, rec, "ffn_down_gemv_residual_ple"))) return rc;
            ++launches;
        }
        if (kind == CHAIN_PREFILL) {
            if (rec && (rc = rec->begin("advance_prompt", (uint64_t)B * 12, 0))) return rc;
            CU(launch_chain(s->use_pdl, advance_kernel, dim3((B + 127) / 128), dim3(128), 0, s->stream, c));
            if (rec && (rc = rec->end())) return rc;
            ++launches;
        } else {
            GemvParams g;
            std::memset(&g, 0, sizeof g);
            g.W = m->E; g.wscale = m->Es; g.N = cfg.vocab; g.K = d;
            g.xin = s->x; g.gain = m->g_final; g.eps = cfg.rms_eps; g.do_norm = 1; g.y = s->logits;
            g.part_val = s->part_val; g.part_idx = s->part_idx; g.ticket = s->lm_ticket;
            g.do_pick = kind == CHAIN_GREEDY ? 1 : 0;
            if ((rc = gemv<GEMV_LMHEAD>(s, c, g, s->lm_rows, rec, "lmhead_gemv_norm_argmax"))) return rc;
            ++launches;
            if (kind == CHAIN_TOPK) {
                SampleParams sp;
                sp.logits = s->logits; sp.V = cfg.vocab; sp.top_k = s->cur_topk; sp.temperature = s->cur_temp; sp.seeds = s->seeds;
                if (rec && (rc = rec->begin("sample_topk_philox", (uint64_t)B * cfg.vocab * 4 * 5, 0))) return rc;
                CU(launch_chain(s->use_pdl, sample_topk_kernel, dim3(B), dim3(256), 0, s->stream, c, sp));
                if (rec && (rc = rec->end())) return rc;
                ++launches;
            }
        }
        if (n_launches) *n_launches = launches;
        return MLB_OK;
    }
};

static int chain_run(mlb_session* s, int kind, Recorder* rec, int* n_launches) {
    const int w = s->m->cfg.weight_dtype, k = s->m->cfg.kv_dtype;
    if (w == MLB_DT_F32 && k == MLB_DT_F32) return Chain<float, float, float>::run(s, kind, rec, n_launches);
    if (w == MLB_DT_F32 && k == MLB_DT_BF16) return Chain<float, float, bf16_t>::run(s, kind, rec, n_launches);
    if (w == MLB_DT_BF16 && k == MLB_DT_F32) return Chain<bf16_t, bf16_t, float>::run(s, kind, rec, n_launches);
    if (w == MLB_DT_BF16 && k == MLB_DT_BF16) return Chain<bf16_t, bf16_t, bf16_t>::run(s, kind, rec, n_launches);
    if (w == MLB_DT_FP8_E4M3 && k == MLB_DT_F32) return Chain<fp8_t, bf16_t, float>::run(s, kind, rec, n_launches);
    return Chain<fp8_t, bf16_t, bf16_t>::run(s, kind, rec, n_launches);
}
static int chain_configure(mlb_session* s) {
    const int w = s->m->cfg.weight_dtype, k = s->m->cfg.kv_dtype;
    if (w == MLB_DT_F32 && k == MLB_DT_F32) return Chain<float, float, float>::configure();
    if (w == MLB_DT_F32 && k == MLB_DT_BF16) return Chain<float, float, bf16_t>::configure();
    if (w == MLB_DT_BF16 && k == MLB_DT_F32) return Chain<bf16_t, bf16_t, float>::configure();
    if (w == MLB_DT_BF16 && k == MLB_DT_BF16) return Chain<bf16_t, bf16_t, bf16_t>::configure();
    if (w == MLB_DT_FP8_E4M3 && k == MLB_DT_F32) return Chain<fp8_t, bf16_t, float>::configure();
    return Chain<fp8_t, bf16_t, bf16_t>::configure();
}

// Device copy of the per-layer pointer table of the single-kernel steps.
static int build_step_layers(mlb_session* s) {
    if (s->step_layers) return MLB_OK;
    const mlb_config& c = s->m->cfg;
    std::vector<StepLayer> hl(c.layers);
    for (int i = 0; i < c.layers; ++i) {
        const DevLayer& L = s->m->layers[i];
        StepLayer& M = hl[i];
        std::memset(&M, 0, sizeof M);
        M.type = L.type; M.n_qkv = L.n_qkv; M.nq = L.nq; M.nk = L.nk; M.nv = L.nv; M.ng = L.ng; M.o_in = L.o_in;
        M.Wqkv = L.Wqkv; M.Sqkv = L.Sqkv; M.g1 = L.g1; M.g2 = L.g2; M.gq = L.gq; M.gk = L.gk;
        M.Wo = L.Wo; M.So = L.So; M.W1a = L.W1a; M.W1b = L.W1b; M.W2 = L.W2; M.S1a = L.S1a; M.S1b = L.S1b; M.S2 = L.S2;
        M.pleT = L.pleT; M.pleP = L.pleP; M.kpool = s->kpool[i]; M.vpool = s->vpool[i]; M.state = s->state[i];
    }
    int rc = sess_alloc(s, (void**)&s->step_layers, hl.size() * sizeof(StepLayer), false);
    if (rc) return rc;
    CU(cudaMemcpy(s->step_layers, hl.data(), hl.size() * sizeof(StepLayer), cudaMemcpyHostToDevice));
    return MLB_OK;
}

// The whole-GPU step with compile-time shapes (lean.cuh), for batch-1 sessions of the models it is built
// for. MLB_DECODE_PATH = auto (this kernel where it fits, else the generic one) | lean | grid | chain.
static int setup_lean_path(mlb_session* s) {
    const mlb_config& c = s->m->cfg;
    const char* env = std::getenv("MLB_DECODE_PATH");
    const std::string mode = env ? env : "auto";
    s->use_lean = false;
    if (mode != "lean" && mode != "auto") return MLB_OK;
    auto no = [&](const char* why) {
        if (mode == "lean") return fail(MLB_E_UNSUPPORTED, "MLB_DECODE_PATH=lean: %s", why);
        return (int)MLB_OK;
    };
    if (s->B != 1) return no("the whole-GPU step serves batch 1 only");
    const int idx = lean_find_shape(c);
    if (idx < 0) return no("no specialised kernel is built for this model's shape");
    const LeanShapeInfo& si = lean_shape_info(idx);
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, s->m->device);
    if (!coop || s->sm_count < si.C) return no("the device cannot keep the kernel's CTAs resident");
    for (const DevLayer& L : s->m->layers)
        if (L.o_in != si.H * si.HD) return no("a layer's output projection has another input width");
    auto up4 = [](int v) { return (v + 3) / 4 * 4; };
    LeanParams lp;
    std::memset(&lp, 0, sizeof lp);
    int off = 0;
    lp.xs_stride = up4(si.xs_floats);
    lp.off_xs = off; off += 2 * lp.xs_stride;
    lp.off_xa = off; off += up4(si.D);
    lp.off_xb = off; off += up4(si.D);
    lp.off_parts = off; off += up4(si.parts_floats);
    lp.off_mix = off; off += up4(si.mix_floats);
    lp.off_pacc = off; off += up4(std::max(1, c.layers * si.rx));
    lp.off_red = off; off += 2 * kLeanWarps + 4 + 128;      // + the dead flag, the finished-row counter, the finished rows
    off = (off + 1) / 2 * 2;
    lp.off_layers = off; off += up4((int)(c.layers * sizeof(StepLayer) / 4));
    lp.off_timers = off; off += 2 * kGridTimerSlots;
    lp.off_plan = off; off += 12;
    off = (off + 31) / 32 * 32;
    const int max_stages = 12;
    lp.off_bar = off; off += max_stages * 2 * 2;
    off = (off + 31) / 32 * 32;
    lp.off_ring = off;
    const size_t fixed = (size_t)off * 4;
    if (fixed + 4 * (size_t)kLeanStage > 208 * 1024) return no("too little shared memory is left for the weight ring");
    lp.n_stages = (int)std::min<size_t>(max_stages, (208 * 1024 - fixed) / kLeanStage);
    const size_t smem = fixed + (size_t)lp.n_stages * kLeanStage;
    int per_sm = 0, rc;
    if ((rc = lean_kernel_probe(idx, c.kv_dtype, smem, &per_sm))) return rc;
    if (per_sm < 1) return no("the kernel does not fit an SM");
    if ((rc = build_step_layers(s))) return rc;
    // exchange buffers (zeroed: epoch 0 is never produced)
    const size_t C = (size_t)si.C;
    const size_t n_ll = C * (2 * (size_t)si.slot_x + si.slot_qa + si.slot_qd + si.slot_parts + si.slot_a + si.slot_ah + si.slot_h + 16) + 64;
    unsigned long long* ll = nullptr;
    if ((rc = sess_alloc(s, (void**)&ll, n_ll * 8, true))) return rc;
    lp.x = ll; ll += C * si.slot_x;
    lp.xb = ll; ll += C * si.slot_x;
    lp.pj = ll; ll += C * std::max(si.slot_qa, si.slot_qd);
    ll += C * std::min(si.slot_qa, si.slot_qd);
    lp.parts = ll; ll += C * si.slot_parts;
    lp.a = ll; ll += C * si.slot_a;
    lp.ah = ll; ll += C * si.slot_ah;
    lp.h = ll; ll += C * si.slot_h;
    lp.lm = ll; ll += C * 16;
    if ((rc = sess_alloc(s, (void**)&lp.epoch, 16, true))) return rc;
    if (const char* t = std::getenv("MLB_GRID_TIMERS"))
        if (t[0] == '1' && (rc = sess_alloc(s, (void**)&lp.timers, C * kGridTimerSlots * 8, true))) return rc;
    if (lp.timers && (rc = sess_alloc(s, (void**)&lp.trace, C * kLeanTraceLen * 8, true))) return rc;
    lp.layers = s->step_layers; lp.n_layers = c.layers;
    lp.E = s->m->E; lp.g_final = s->m->g_final; lp.rope = s->m->rope; lp.page_table = s->page_table;
    lp.logits = s->logits; lp.err = s->dev_err;
    lp.tok_arg = -1;
    lp.eps = c.rms_eps; lp.l2_eps = 1e-6f;
    lp.pages_per_split = 4;       // 64 positions per attention item: one round of the 16 warps (measured: 4 beats 16 by 4 us per step at a context of 150)
    if (const char* v = std::getenv("MLB_GRID_PAGES_PER_SPLIT")) lp.pages_per_split = std::max(1, std::min(256, std::atoi(v)));
    s->lean = lp;
    s->lean_idx = idx;
    s->lean_smem = smem;
    s->grid_ctas = si.C;
    s->use_lean = true;
    return MLB_OK;
}

// Geometry of one exchanged vector of the whole-GPU step: N values from P producers, a slot of whole
// 128-byte lines per producer (grid_params.h). `tab` is the shared-memory offset of its row table, -1
// when every producer owns exactly N / P rows.
static GridVec grid_vec(int N, int P, int tab) {
    GridVec v;
    std::memset(&v, 0, sizeof v);
    v.N = N;
    v.P = P;
    v.rpc = (N + P - 1) / P;
    v.slotw = (v.rpc + 15) / 16 * 16;
    v.tab = tab;
    v.inv_n = 1.0f / (float)N;
    v.magic = 0;
    if (v.rpc > 1) {
        // q / rpc as one multiply-high, exact over the range the kernel uses (q < P * rpc < 2^16 * rpc)
        v.magic = (unsigned)(((1ull << 32) + (unsigned)v.rpc - 1) / (unsigned)v.rpc);
        for (unsigned q = 0; q < (unsigned)(P * v.rpc); ++q)
            if ((unsigned)(((unsigned long long)q * v.magic) >> 32) != q / (unsigned)v.rpc) { v.N = -1; break; }     // never seen; the caller refuses
    }
    return v;
}

// Decides whether the whole-GPU single-kernel step serves this session (batch 1) and lays out
// its shared memory and exchange buffers. MLB_DECODE_PATH = chain | grid | auto; auto takes it
// whenever the model fits its constraints.
static int setup_grid_path(mlb_session* s) {
    const mlb_config& c = s->m->cfg;
    const char* env = std::getenv("MLB_DECODE_PATH");
    const std::string mode = env ? env : "auto";
    s->use_grid = false;
    if (mode != "grid" && mode != "auto") return MLB_OK;
    auto no = [&](const char* why) {
        if (mode == "grid") return fail(MLB_E_UNSUPPORTED, "MLB_DECODE_PATH=grid: %s", why);
        return (int)MLB_OK;
    };
    if (s->B != 1) return no("the whole-GPU step serves batch 1 only");
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, s->m->device);
    if (!coop) return no("the device has no cooperative launch");
    const int epv = 16 / (int)elt_size(c.weight_dtype);
    bool has_attn = false, has_dn = false;
    int nqkv_attn = 0, nqkv_dn = 0, min_rows = std::min(c.dim, c.ffn_dim), a_dim = 16;
    for (const DevLayer& L : s->m->layers) {
        min_rows = std::min(min_rows, L.n_qkv);
        a_dim = std::max(a_dim, L.o_in);
        if (L.type == MLB_LAYER_ATTENTION) { has_attn = true; nqkv_attn = L.n_qkv; }
        else { has_dn = true; nqkv_dn = L.n_qkv; }
        if (L.o_in % epv) return no("a projection width is not a multiple of the weight vector");
    }
    if (c.dim % epv || c.ffn_dim % epv) return no("a projection width is not a multiple of the weight vector");
    if (has_attn && c.head_dim != 64 && c.head_dim != 128) return no("head_dim must be 64 or 128");
    if (has_attn && (c.heads % c.kv_heads || c.heads / c.kv_heads > 8)) return no("more than 8 query heads per kv head");
    if (has_dn && c.dn_key_dim > 128) return no("delta-net key dim above 128");
    if (has_dn) min_rows = std::min(min_rows, c.heads * c.dn_value_dim);
    min_rows = std::min(min_rows, c.vocab);
    // Every CTA must own rows in every projection phase (the reuse rule of the exchange buffers)
    int C = std::min(s->sm_count, min_rows);
    if (const char* v = std::getenv("MLB_GRID_CTAS")) C = std::max(8, std::min(C, std::atoi(v)));
    if (C < 8) return no("the model is too small to split over the SMs");
    if (has_attn && c.heads > C) return no("more heads than CTAs");
    const int G = has_attn ? c.heads / c.kv_heads : 1;
    auto up4 = [](int v) { return (v + 3) / 4 * 4; };
    GridParams gp;
    std::memset(&gp, 0, sizeof gp);
    // context splits per kv head: at most one item per CTA; a head's partials fit 32 KB of shared memory
    gp.s_max = has_attn ? std::max(1, std::min(C / c.kv_heads, 8192 / (c.head_dim + 2))) : 1;
    gp.s_direct = has_attn ? std::max(1, std::min(gp.s_max, kGridDirectWords / (c.heads * (c.head_dim + 2)))) : 1;
    gp.pages_per_split = 4;        // 64 positions per attention item (measured: the large GQA model 1.07 -> 0.99 ms per token against 16, the reference-shaped fp32 model 207 -> 198 us)
    if (const char* v = std::getenv("MLB_GRID_PAGES_PER_SPLIT")) gp.pages_per_split = std::max(1, std::min(256, std::atoi(v)));
    const int rpc_d = (c.dim + C - 1) / C;
    const int rpc_a = has_dn ? (c.heads * c.dn_value_dim + C - 1) / C : 0;
    int off = 0;
    // row tables (ints) of the vectors whose rows do not divide evenly
    const int tab_d = off; off += up4(C + 1);
    const int tab_f = off; off += up4(C + 1);
    const int tab_qa = off; off += up4(C + 1);
    const int tab_qd = off; off += up4(C + 1);
    const int tab_a = off; off += up4(C + 1);
    const int tab_ah = off; off += up4(C + 1);
    const int tab_lm = off; off += up4(C + 1);
    gp.vocab_tab = off; off += up4(C + 1);
    gp.off_tabs = 0;
    gp.xs_stride = up4(std::max(std::max(c.dim, c.ffn_dim), a_dim));
    gp.off_xs = off; off += 2 * gp.xs_stride;
    gp.off_xa = off; off += up4(c.dim);
    gp.off_xb = off; off += up4(c.dim);
    gp.off_parts = off; off += up4(std::max(has_attn ? std::max(gp.s_max * (c.head_dim + 2), kGridDirectWords) : 0, 2 * C));
    gp.off_gate = off; off += up4(has_attn ? c.heads * c.head_dim : 4);
    {
        const int attn_n = has_attn ? G * c.head_dim + 2 * c.head_dim + kRingWarps * (c.head_dim + 2) : 0;
        const int comb_n = has_attn ? std::max(c.heads * gp.s_direct, gp.s_max) : 0;
        const int dn_n = has_dn ? 2 * c.heads * c.dn_key_dim + up4(rpc_a) + 2 * c.heads + 8 : 0;
        gp.off_mix = off; off += up4(std::max(std::max(attn_n, comb_n), std::max(dn_n, 64)));
    }
    gp.off_pacc = off; off += up4(std::max(1, c.layers * rpc_d));
    gp.off_red = off; off += 2 * kRingConsumers + 8;      // + the dead flag and the finished-row counter
    gp.off_obuf = off; off += up4(std::max(std::max((nqkv_attn + C - 1) / C, (nqkv_dn + C - 1) / C), std::max((c.ffn_dim + C - 1) / C, std::max(rpc_d, rpc_a))) + 4);
    off = (off + 1) / 2 * 2;
    gp.off_layers = off; off += up4((int)(c.layers * sizeof(StepLayer) / 4));
    gp.off_timers = off; off += 2 * kGridTimerSlots;
    gp.off_plan = off; off += 12;
    off = (off + 31) / 32 * 32;
    const int max_stages = 12;
    gp.off_bar = off; off += max_stages * 2 * 2;              // 8-byte barriers: full[] then empty[]
    off = (off + 31) / 32 * 32;
    gp.off_ring = off;
    // ring: stages of whole rows (and whole KV pages), 16 KB unless a row is longer, as many as fit below ~208 KB
    size_t widest = (size_t)std::max(std::max(c.dim, c.ffn_dim), a_dim) * elt_size(c.weight_dtype);
    if (has_attn) widest = std::max(widest, (size_t)kKvBlock * c.head_dim * elt_size(c.kv_dtype));
    if (has_dn) widest = std::max(widest, (size_t)c.dn_key_dim * 4);
    gp.stage_bytes = (int)std::max<size_t>(16 * 1024, (widest + 1023) / 1024 * 1024);
    if (const char* v = std::getenv("MLB_GRID_STAGE_KB")) gp.stage_bytes = std::max(gp.stage_bytes, std::min(64, std::atoi(v)) * 1024);
    const size_t fixed = (size_t)off * 4;
    if (fixed + 3 * (size_t)gp.stage_bytes > 208 * 1024) return no("the activations leave too little shared memory for the weight ring");
    gp.n_stages = (int)std::min<size_t>(max_stages, (208 * 1024 - fixed) / gp.stage_bytes);
    const size_t smem = fixed + (size_t)gp.n_stages * gp.stage_bytes;
    int per_sm = 0, rc;
    if ((rc = grid_kernel_probe(c.weight_dtype, c.kv_dtype, smem, &per_sm))) return rc;
    if (per_sm < 1) return no("the kernel does not fit an SM");
    if ((rc = build_step_layers(s))) return rc;
    // exchanged vectors and their buffers (zeroed: epoch 0 is never produced)
    gp.vx = grid_vec(c.dim, C, tab_d);
    gp.vxb = grid_vec(c.dim, C, tab_d);
    gp.vproj_attn = grid_vec(std::max(nqkv_attn, C), C, tab_qa);
    gp.vproj_dn = grid_vec(std::max(nqkv_dn, C), C, tab_qd);
    gp.vh = grid_vec(c.ffn_dim, C, tab_f);
    gp.va_dn = grid_vec(has_dn ? c.heads * c.dn_value_dim : C, C, tab_a);
    gp.va_head = grid_vec(has_attn ? c.heads * c.head_dim : 16, has_attn ? c.heads : 1, tab_ah);
    gp.vlm = grid_vec(2 * C, C, tab_lm);
    gp.parts_slotw = (G * (c.head_dim + 2) + 15) / 16 * 16;
    GridVec* vecs[] = {&gp.vx, &gp.vxb, &gp.vproj_attn, &gp.vproj_dn, &gp.vh, &gp.va_dn, &gp.va_head, &gp.vlm};
    size_t n_ll = (size_t)C * gp.parts_slotw + 64;
    for (GridVec* v : vecs) {
        if (v->N < 0) return no("a row split has no exact multiply-high divisor");
        n_ll += (size_t)v->P * v->slotw;
    }
    unsigned long long* ll = nullptr;
    if ((rc = sess_alloc(s, (void**)&ll, n_ll * 8, true))) return rc;
    for (GridVec* v : vecs) { v->buf = ll; ll += (size_t)v->P * v->slotw; }
    gp.parts = ll;
    if ((rc = sess_alloc(s, (void**)&gp.epoch, 16, true))) return rc;
    if (const char* t = std::getenv("MLB_GRID_TIMERS"))
        if (t[0] == '1' && (rc = sess_alloc(s, (void**)&gp.timers, (size_t)C * kGridTimerSlots * 8, true))) return rc;
    gp.layers = s->step_layers; gp.n_layers = c.layers;
    gp.d = c.dim; gp.F = c.ffn_dim; gp.V = c.vocab; gp.heads = c.heads; gp.kv_heads = c.kv_heads; gp.hd = c.head_dim;
    gp.dk = c.dn_key_dim; gp.dv = c.dn_value_dim; gp.ple = c.ple_dim; gp.qk_norm = c.qk_norm;
    gp.eps = c.rms_eps; gp.l2_eps = 1e-6f;
    gp.E = s->m->E; gp.Es = s->m->Es; gp.g_final = s->m->g_final; gp.rope = s->m->rope;
    gp.page_table = s->page_table; gp.logits = s->logits;
    gp.err = s->dev_err;
    gp.tok_arg = -1;
    gp.backoff_ns = 100;
    if (const char* v = std::getenv("MLB_GRID_BACKOFF_NS")) gp.backoff_ns = std::max(0, std::min(10000, std::atoi(v)));
    s->grid = gp;
    s->grid_ctas = C;
    s->grid_smem = smem;
    s->use_grid = true;
    return MLB_OK;
}

template <typename KVT, typename WT>
static int tc_allow_big_smem_t() {
    const int big = 227 * 1024;
    CU(cudaFuncSetAttribute(gemm_tc_kernel<TC_RAW, KVT, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    CU(cudaFuncSetAttribute(gemm_tc_kernel<TC_RESID, KVT, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    CU(cudaFuncSetAttribute(gemm_tc_kernel<TC_SWIGLU, KVT, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    CU(cudaFuncSetAttribute(gemm_tc_kernel<TC_QKV, KVT, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    return MLB_OK;
}
static int tc_allow_big_smem(int wdt, int kvdt) {
    if (wdt == MLB_DT_FP8_E4M3) return kvdt == MLB_DT_BF16 ? tc_allow_big_smem_t<bf16_t, fp8_t>() : tc_allow_big_smem_t<float, fp8_t>();
    return kvdt == MLB_DT_BF16 ? tc_allow_big_smem_t<bf16_t, bf16_t>() : tc_allow_big_smem_t<float, bf16_t>();
}

// Tensor-core projections for batches of 4 sequences or more with bf16 weights (MLB_GEMM=simt turns it off).
static int setup_tc_path(mlb_session* s) {
    const mlb_config& c = s->m->cfg;
    s->use_tc = false;
    const char* env = std::getenv("MLB_GEMM");
    const std::string mode = env ? env : "auto";
    if (!s->parent && (mode == "simt" || s->use_grid || s->use_lean)) return MLB_OK;
    if (c.weight_dtype != MLB_DT_BF16 && c.weight_dtype != MLB_DT_FP8_E4M3) {
        if (mode == "tc") return fail(MLB_E_UNSUPPORTED, "MLB_GEMM=tc needs bf16 or FP8 weights");
        return MLB_OK;
    }
    const bool w8 = c.weight_dtype == MLB_DT_FP8_E4M3;
    // auto: from 4 sequences on. The GEMV kernels re-read nothing, but their time grows with the batch
    // (cfg1: 169 us at 1 sequence, 369 at 4, 537 at 8, 635 at 12), while the tensor-core step costs
    // 360-390 us for any batch up to 16 (its floor is its 60 launches).
    if (!s->parent && mode == "auto" && s->B < 4) return MLB_OK;
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) {
        if (mode == "tc") return fail(MLB_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        return MLB_OK;
    }
    const int B = s->B;
    s->tc_nb = std::min(256, (B + 15) / 16 * 16);
    const size_t budget = 200 * 1024;
    s->tc_stages = (int)std::max<size_t>(2, std::min<size_t>(6, budget / ((size_t)kTcM * 128 + (size_t)s->tc_nb * 128)));
    s->tc_stages_swiglu = (int)std::max<size_t>(2, std::min<size_t>(6, budget / ((size_t)2 * kTcM * 128 + (size_t)s->tc_nb * 128)));
    const int nq = c.heads * c.head_dim, a_dn = c.heads * c.dn_value_dim;
    int rc;
    if (c.ple_dim > 0 && ple_dtype(c.weight_dtype) != MLB_DT_BF16) return MLB_OK;
    if ((rc = build_step_layers(s))) return rc;
    if (const char* v = std::getenv("MLB_TC_TRACE"))
        if (v[0] == '1' && (rc = sess_alloc(s, (void**)&s->tc_trace, 64 * 8 * 8, true))) return rc;
    s->tc_max_split = 8;
    if (const char* v = std::getenv("MLB_TC_SPLIT")) {
        s->tc_max_split = std::max(1, std::min(8, std::atoi(v)));
        s->tc_split_forced = true;
    }
    {
        // how many clusters of GEMM CTAs fit on the GPU at once (a 100 KB CTA, typical of a split launch)
        const int big = 227 * 1024;
        void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, GemmTcParams, StepCtl, QkvPostParams) =
            gemm_tc_kernel<TC_RESID, float, bf16_t>;
        CU(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
        s->tc_cluster_cap[0] = s->sm_count;
        for (int li = 1; li < 4; ++li) {
            cudaLaunchConfig_t cfg;
            std::memset(&cfg, 0, sizeof cfg);
            cfg.gridDim = dim3(1, 1, 1u << li);
            cfg.blockDim = dim3(kTcThreads);
            cfg.dynamicSmemBytes = 100 * 1024;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1u << li;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
            s->tc_cluster_cap[li] = n;
        }
    }
    s->tc_shape_down = tc_pick_shape(s, c.dim, (c.ffn_dim + kTcKB - 1) / kTcKB + (c.ple_dim + kTcKB - 1) / kTcKB, 1, w8, w8 ? 2 : 1);
    const int parts = (c.dim + kTcM - 1) / kTcM;
    if ((rc = sess_alloc(s, (void**)&s->xn16, (size_t)B * c.dim * 2, true))) return rc;
    if ((rc = sess_alloc(s, (void**)&s->a16, (size_t)B * std::max(nq, a_dn) * 2, true))) return rc;
    if ((rc = sess_alloc(s, (void**)&s->h16, (size_t)B * c.ffn_dim * 2, true))) return rc;
    if ((rc = sess_alloc(s, (void**)&s->tc_ssq, (size_t)B * parts * 4, true))) return rc;
    if (c.ple_dim > 0 && (rc = sess_alloc(s, (void**)&s->tple16, (size_t)c.layers * B * c.ple_dim * 2, true))) return rc;
    s->tc_maps.resize(c.layers);
    for (int i = 0; i < c.layers; ++i) {
        const DevLayer& L = s->m->layers[i];
        auto& M = s->tc_maps[i];
        auto wmap = w8 ? make_u8_map : make_bf16_map;       // FP8: e4m3 codes, widened in the kernel
        if ((rc = wmap(enc, &M.qkv, L.Wqkv, L.n_qkv, c.dim, kTcM))) return rc;
        if ((rc = wmap(enc, &M.o, L.Wo, c.dim, L.o_in, kTcM))) return rc;
        if ((rc = wmap(enc, &M.w1a, L.W1a, c.ffn_dim, c.dim, kTcM))) return rc;
        if ((rc = wmap(enc, &M.w1b, L.W1b, c.ffn_dim, c.dim, kTcM))) return rc;
        if ((rc = wmap(enc, &M.w2, L.W2, c.dim, c.ffn_dim, kTcM))) return rc;
        if (c.ple_dim > 0) {
            // operands of the per-layer embedding folded into the previous layer's down projection
            if ((rc = make_bf16_map(enc, &M.pleP, L.pleP, c.dim, c.ple_dim, kTcM))) return rc;
            if ((rc = make_bf16_map(enc, &M.pleT, s->tple16 + (size_t)i * B * c.ple_dim, B, c.ple_dim, s->tc_shape_down.nb))) return rc;
        }
    }
    if ((rc = (w8 ? make_u8_map : make_bf16_map)(enc, &s->tc_g.E, s->m->E, c.vocab, c.dim, kTcM))) return rc;
    for (int i = 0; i < 5; ++i) {
        const uint32_t nb = 16u << i;
        if ((rc = make_bf16_map(enc, &s->tc_g.xn[i], s->xn16, B, c.dim, nb))) return rc;
        if ((rc = make_bf16_map(enc, &s->tc_g.a_attn[i], s->a16, B, nq, nb))) return rc;
        if ((rc = make_bf16_map(enc, &s->tc_g.a_dn[i], s->a16, B, a_dn, nb))) return rc;
        if ((rc = make_bf16_map(enc, &s->tc_g.h[i], s->h16, B, c.ffn_dim, nb))) return rc;
    }
    if ((rc = tc_allow_big_smem(c.weight_dtype, c.kv_dtype))) return rc;
    s->use_tc = true;
    return MLB_OK;
}

// Capture the chain once per kind; sampling parameters are baked into the top-k graph.
static int ensure_graph(mlb_session* s, int kind) {
    if (kind == CHAIN_TOPK && s->graphs[kind] && (s->g_topk != s->cur_topk || s->g_temp != s->cur_temp)) {
        cudaGraphExecDestroy(s->graphs[kind]);
        s->graphs[kind] = nullptr;
    }
    if (s->graphs[kind]) return MLB_OK;
    if (s->use_grid || s->use_lean) {
        // one cooperative launch per step (plus the sampler): launched directly, nothing to capture
        s->launches_per_step[kind] = kind == CHAIN_TOPK ? 2 : 1;
        if (kind == CHAIN_TOPK) { s->g_topk = s->cur_topk; s->g_temp = s->cur_temp; }
        return MLB_OK;
    }
    cudaGraph_t graph = nullptr;
    CU(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
    int n = 0;
    int rc = chain_run(s, kind, nullptr, &n);
    cudaError_t e = cudaStreamEndCapture(s->stream, &graph);
    if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (e != cudaSuccess) return fail(MLB_E_CUDA, "cudaStreamEndCapture failed: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(&s->graphs[kind], graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return fail(MLB_E_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
    s->launches_per_step[kind] = n;
    if (kind == CHAIN_TOPK) { s->g_topk = s->cur_topk; s->g_temp = s->cur_temp; }
    return MLB_OK;
}

// The one-token call (mlb_decode_step) as a single graph of the step's own kernels: the embedding
// kernel reads the pending ids from pinned host memory, the kernel that advances a sequence writes
// the picked id and the error word there. One launch and one synchronisation per token, no copy
// queued around the step (as graph nodes such copies cost more than the enqueues they replaced:
// 199 vs 188 us per token). The error word is copied when sequence 0 advances: a wait that runs out
// in the very last kernel of a step may be reported one call late.
static int ensure_token_graph(mlb_session* s, int kind, bool with_input) {
    const int idx = kind * 2 + (with_input ? 1 : 0);
    if (kind == CHAIN_TOPK && s->tgraphs[idx] && (s->tg_topk[with_input] != s->cur_topk || s->tg_temp[with_input] != s->cur_temp)) {
        cudaGraphExecDestroy(s->tgraphs[idx]);
        s->tgraphs[idx] = nullptr;
    }
    if (s->tgraphs[idx]) return MLB_OK;
    cudaGraph_t graph = nullptr;
    CU(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
    int n = 0;
    s->ctl_host_io = with_input ? 2 : 1;
    int rc = chain_run(s, kind, nullptr, &n);
    s->ctl_host_io = 0;
    cudaError_t e = cudaStreamEndCapture(s->stream, &graph);
    if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (e != cudaSuccess) return fail(MLB_E_CUDA, "capture of the one-token graph failed: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(&s->tgraphs[idx], graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return fail(MLB_E_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
    s->launches_per_step[kind] = n;
    if (kind == CHAIN_TOPK) { s->tg_topk[with_input] = s->cur_topk; s->tg_temp[with_input] = s->cur_temp; }
    return MLB_OK;
}

// One step on the session's stream: the captured chain, or the single cooperative kernel.
static int launch_step(mlb_session* s, int kind) {
    if (s->use_grid || s->use_lean) return chain_run(s, kind, nullptr, nullptr);
    CU(cudaGraphLaunch(s->graphs[kind], s->stream));
    return MLB_OK;
}

static int sync_page_table(mlb_session* s) {
    if (!s->table_dirty) return MLB_OK;
    for (int b = 0; b < s->B; ++b) {
        const auto& pg = s->alloc.seq_pages[b];
        for (size_t i = 0; i < pg.size(); ++i) s->h_table[(size_t)b * s->max_pages + i] = pg[i];
    }
    CU(cudaMemcpyAsync(s->page_table, s->h_table.data(), s->h_table.size() * 4, cudaMemcpyHostToDevice, s->stream));
    CU(cudaStreamSynchronize(s->stream));      // h_table may be rewritten by the next call
    s->table_dirty = false;
    return MLB_OK;
}

static int grow_pages(mlb_session* s, int extra_steps) {
    bool has_attn = false;
    for (auto* p : s->kpool) if (p) has_attn = true;
    if (!has_attn) return MLB_OK;
    for (int b = 0; b < s->B; ++b) {
        int want = s->h_stopped[b] ? s->h_pos[b] : std::min(s->h_pos[b] + extra_steps, s->max_ctx);
        size_t before = s->alloc.seq_pages[b].size();
        int rc = kv_ensure(&s->alloc, b, want, kKvBlock);
        if (s->alloc.seq_pages[b].size() != before) s->table_dirty = true;
        if (rc) return rc;
    }
    return sync_page_table(s);
}

static int apply_sampling(mlb_session* s, const mlb_sampling* sp, int* kind) {
    *kind = CHAIN_GREEDY;
    if (!sp || sp->mode == 0) return MLB_OK;
    if (sp->mode != 1) return fail(MLB_E_INVALID, "unknown sampling mode %d", sp->mode);
    if (sp->top_k < 1 || sp->top_k > kSampleCap) return fail(MLB_E_INVALID, "top_k must be in 1..%d", kSampleCap);
    if (!(sp->temperature > 0.f)) return fail(MLB_E_INVALID, "temperature must be > 0");
    s->cur_topk = sp->top_k;
    s->cur_temp = sp->temperature;
    std::vector<unsigned long long> seeds(s->B);
    for (int b = 0; b < s->B; ++b) seeds[b] = sp->seeds ? sp->seeds[b] : (unsigned long long)b;
    CU(cudaMemcpyAsync(s->seeds, seeds.data(), (size_t)s->B * 8, cudaMemcpyHostToDevice, s->stream));
    CU(cudaStreamSynchronize(s->stream));
    *kind = CHAIN_TOPK;
    return MLB_OK;
}

}  // namespace mlb

// A session, or (parent != null) the column set of one: `batch` columns of step buffers on the
// parent's KV pool, delta-net state and stream, always on the tensor-core step.
static int session_create(mlb_model* m, int batch, int max_context, int kv_block, int kv_pages, mlb_session* parent, mlb_session** out) {
    if (!m || !out) return fail(MLB_E_INVALID, "null argument");
    *out = nullptr;
    if (batch < 1) return fail(MLB_E_INVALID, "batch must be >= 1");
    if (kv_block != 0 && kv_block != kKvBlock) return fail(MLB_E_UNSUPPORTED, "kv_block must be %d", kKvBlock);
    if (max_context <= 0) max_context = m->cfg.max_context;
    if (max_context > m->cfg.max_context) return fail(MLB_E_INVALID, "max_context %d exceeds the model's %d (RoPE table size)", max_context, m->cfg.max_context);
    CU(cudaSetDevice(m->device));
    const mlb_config& c = m->cfg;
    mlb_session* s = new mlb_session();
    s->m = m;
    s->B = batch;
    s->max_ctx = max_context;
    s->max_pages = (max_context + kKvBlock - 1) / kKvBlock;
    s->kv_pages = kv_pages > 0 ? kv_pages : batch * s->max_pages;
    s->parent = parent;
    if (parent) s->kv_pages = parent->kv_pages;
#define SA(expr) do { int r__ = (expr); if (r__) { free_session(s); return r__; } } while (0)
#define SCU(expr) do { cudaError_t e__ = (expr); if (e__ != cudaSuccess) { free_session(s); return fail(MLB_E_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)); } } while (0)
    if (parent) s->stream = parent->stream;
    else SCU(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
    const size_t B = batch;
    const size_t ctx_rows = parent ? 1 : (size_t)max_context;      // a column set has no prompt / output ring of its own
    SA(sess_alloc(s, (void**)&s->pos, B * 4, true));
    SA(sess_alloc(s, (void**)&s->tok, B * 4, true));
    SA(sess_alloc(s, (void**)&s->limit_prefill, B * 4, true));
    SA(sess_alloc(s, (void**)&s->limit_decode, B * 4, true));
    SA(sess_alloc(s, (void**)&s->prompt, B * ctx_rows * 4, true));
    SA(sess_alloc(s, (void**)&s->out_ring, B * ctx_rows * 4, true));
    if (parent) SA(sess_alloc(s, (void**)&s->seq_of, B * 4, true));
    SA(sess_alloc(s, (void**)&s->out_idx, B * 4, true));
    SA(sess_alloc(s, (void**)&s->page_table, B * s->max_pages * 4, true));
    SA(sess_alloc(s, (void**)&s->seeds, B * 8, true));
    const int nq = c.heads * c.head_dim;
    const int a_dim = std::max(nq, c.heads * c.dn_value_dim);
    s->max_q = nq;
    s->raw_stride = 2 * c.heads * c.dn_key_dim + c.heads * c.dn_value_dim + 2 * c.heads;
    SA(sess_alloc(s, (void**)&s->x, B * c.dim * 4, true));
    SA(sess_alloc(s, (void**)&s->qbuf, B * nq * 4, true));
    SA(sess_alloc(s, (void**)&s->gbuf, B * nq * 4, true));
    SA(sess_alloc(s, (void**)&s->abuf, B * a_dim * 4, true));
    SA(sess_alloc(s, (void**)&s->hbuf, B * c.ffn_dim * 4, true));
    SA(sess_alloc(s, (void**)&s->raw, B * s->raw_stride * 4, true));
    SA(sess_alloc(s, (void**)&s->logits, B * c.vocab * 4, true));
    SA(sess_alloc(s, (void**)&s->probe, (size_t)c.vocab * 4, true));
    // split count of the flash-decode: enough CTAs to cover the GPU at small batch, at least
    // four pages of work per split at full context
    int sm_count = 148;
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, m->device);
    int want = (4 * sm_count + c.kv_heads * batch - 1) / (c.kv_heads * batch);
    s->splits = std::max(1, std::min(std::min(want, 32), std::max(1, s->max_pages / 4)));
    if (const char* v = std::getenv("MLB_ATTN_SPLITS")) s->splits = std::max(1, std::min(32, std::atoi(v)));
    // pages a split must hold before a sequence uses it (the grid above already caps the splits at about four
    // CTAs per SM). Measured: cfg1 at 32 / 64 sequences and a context of 260, one split beats two (12.6 vs 15.5,
    // 16.3 vs 22.8 us per launch); the GQA model at 64 sequences and a context of 576, three splits of 11 pages
    // beat two of 18 and four of 9 (63 vs 78 and 74 us).
    s->attn_min_pps = 11;
    if (const char* v = std::getenv("MLB_ATTN_MIN_PAGES")) s->attn_min_pps = std::max(1, std::atoi(v));
    SA(sess_alloc(s, (void**)&s->part, B * c.heads * s->splits * (c.head_dim + 2) * 4, true));
    SA(sess_alloc(s, (void**)&s->attn_ticket, B * c.heads * 4, true));
    s->lm_rows = 16;
    // argmax partials per sequence: one per LM-head CTA of either GEMV form (the streamed form
    // launches up to one CTA per SM, whatever the vocabulary size)
    s->lm_parts = std::max((c.vocab + s->lm_rows - 1) / s->lm_rows, 2 * sm_count);
    SA(sess_alloc(s, (void**)&s->part_val, B * s->lm_parts * 4, true));
    SA(sess_alloc(s, (void**)&s->part_idx, B * s->lm_parts * 4, true));
    SA(sess_alloc(s, (void**)&s->lm_ticket, (B + 7) / 1 * 4, true));
    s->kpool.assign(c.layers, nullptr);
    s->vpool.assign(c.layers, nullptr);
    s->state.assign(c.layers, nullptr);
    const size_t kv_elt = elt_size(c.kv_dtype);
    for (int i = 0; i < c.layers; ++i) {
        if (parent) {
            s->kpool[i] = parent->kpool[i];
            s->vpool[i] = parent->vpool[i];
            s->state[i] = parent->state[i];
        } else if (c.layer_types[i] == MLB_LAYER_ATTENTION) {
            size_t bytes = (size_t)s->kv_pages * c.kv_heads * kKvBlock * c.head_dim * kv_elt;
            SA(sess_alloc(s, &s->kpool[i], bytes, true));
            SA(sess_alloc(s, &s->vpool[i], bytes, true));
        } else {
            SA(sess_alloc(s, (void**)&s->state[i], B * c.heads * c.dn_value_dim * c.dn_key_dim * 4, true));
        }
    }
    if (!parent) {
        s->flush_n = (192ull << 20) / 16;
        SA(sess_alloc(s, (void**)&s->flush_buf, s->flush_n * 16, false));
    }
    SCU(cudaMallocHost((void**)&s->pinned_tok, B * 4));
    SCU(cudaMallocHost((void**)&s->pinned_out, B * 4));
    SCU(cudaMallocHost((void**)&s->pinned_err, 4));
    *s->pinned_err = 0;
    s->alloc.num_pages = s->kv_pages;
    s->alloc.max_pages_per_seq = s->max_pages;
    s->alloc.seq_pages.assign(batch, {});
    for (int p = s->kv_pages - 1; p >= 0; --p) s->alloc.free_list.push_back(p);
    s->h_pos.assign(batch, 0);
    s->h_stopped.assign(batch, 0);
    s->h_table.assign(B * s->max_pages, 0);
    std::vector<int> lim(batch, max_context);
    SCU(cudaMemcpy(s->limit_decode, lim.data(), B * 4, cudaMemcpyHostToDevice));
    {
        const char* e = std::getenv("MLB_NO_PDL");     // measurement switch: plain stream-ordered launches
        s->use_pdl = !(e && e[0] == '1');
        const char* gv = std::getenv("MLB_GEMV");      // stream | thread | auto (stream for batch <= 4)
        const std::string gmode = gv ? gv : "auto";
        s->use_sgemv = gmode == "stream" || (gmode == "auto" && batch <= 4);
        s->force_sgemv = gmode == "stream";
        if (const char* v = std::getenv("MLB_SG_STAGE_KB")) s->sg_stage_kb = std::max(8, std::min(96, std::atoi(v)));
        if (const char* v = std::getenv("MLB_SG_STAGES")) s->sg_max_stages = std::max(2, std::min(8, std::atoi(v)));
        cudaDeviceGetAttribute(&s->sm_count, cudaDevAttrMultiProcessorCount, m->device);
    }
    SA(sess_alloc(s, (void**)&s->dev_err, 4, true));
    SA(chain_configure(s));
    if (!parent) {
        SA(setup_lean_path(s));
        if (!s->use_lean) SA(setup_grid_path(s));
    }
    SA(setup_tc_path(s));
    if (parent && !s->use_tc) {
        free_session(s);
        return fail(MLB_E_UNSUPPORTED, "prompt columns need the tensor-core step (bf16 weights)");
    }
#undef SA
#undef SCU
    *out = s;
    return MLB_OK;
}

extern "C" int mlb_session_new(mlb_model* m, int batch, int max_context, int kv_block, int kv_pages, mlb_session** out) {
    if (!m || !out) return fail(MLB_E_INVALID, "null argument");
    return session_create(m, batch, max_context, kv_block, kv_pages, nullptr, out);
}

extern "C" int mlb_session_reset(mlb_session* s) {
    if (!s) return fail(MLB_E_INVALID, "null session");
    CU(cudaSetDevice(s->m->device));
    CU(cudaStreamSynchronize(s->stream));
    const size_t B = s->B;
    CU(cudaMemsetAsync(s->pos, 0, B * 4, s->stream));
    CU(cudaMemsetAsync(s->tok, 0, B * 4, s->stream));
    CU(cudaMemsetAsync(s->limit_prefill, 0, B * 4, s->stream));
    CU(cudaMemsetAsync(s->out_idx, 0, B * 4, s->stream));
    {
        // a sequence that stopped had its decode limit lowered on the device
        const std::vector<int> lim(B, s->max_ctx);
        CU(cudaMemcpyAsync(s->limit_decode, lim.data(), B * 4, cudaMemcpyHostToDevice, s->stream));
        CU(cudaStreamSynchronize(s->stream));
    }
    const mlb_config& c = s->m->cfg;
    for (int i = 0; i < c.layers; ++i)
        if (s->state[i]) CU(cudaMemsetAsync(s->state[i], 0, B * c.heads * c.dn_value_dim * c.dn_key_dim * 4, s->stream));
    CU(cudaStreamSynchronize(s->stream));
    for (int b = 0; b < s->B; ++b) {
        for (int pg : s->alloc.seq_pages[b]) s->alloc.free_list.push_back(pg);
        s->alloc.seq_pages[b].clear();
        s->h_pos[b] = 0;
        s->h_stopped[b] = 0;
    }
    s->table_dirty = true;
    s->have_logits = false;
    return MLB_OK;
}

extern "C" void mlb_session_free(mlb_session* s) { free_session(s); }

// Prompt by columns. The token loop consumes a prompt one token per step and sequence: a
// 512-token prompt costs 511 steps. Here the prompt tokens of all sequences become the columns of
// tensor-core steps (bf16 weights): the projections of up to kPromptCols (256) tokens are one GEMM each,
// every column appends its K/V row and attends to the rows before it (same kernels as a decode
// step, the column's page-table row is its sequence's), and the delta-net recurrence walks the
// columns of a sequence in order (delta_net_cols_kernel). All tokens but the last of each prompt
// are consumed; the last one stays pending, as after the token loop. MLB_PREFILL = auto | step |
// chunk: auto takes this path from 64 prompt tokens on (its activations are bf16, so the cache
// differs from the token loop's within the low-precision tolerance); `*done` tells whether it ran.
static const int kPromptCols = 256;
// score_out != null: the scoring forward instead (mlb_score_tokens): every token of sequence 0 is a
// column, the LM head runs on the columns too, and the logits of each chunk go to score_out.
static int prefill_columns(mlb_session* s, const int32_t* tokens, const int32_t* lens, int stride, bool* done, float* score_out = nullptr) {
    *done = false;
    const char* env = std::getenv("MLB_PREFILL");
    const std::string mode = score_out ? "chunk" : (env ? env : "auto");
    if (mode == "step") return MLB_OK;
    const int B = score_out ? 1 : s->B;
    const int keep = score_out ? 0 : 1;            // tokens per prompt that stay pending
    const int kind = score_out ? CHAIN_GREEDY : CHAIN_PREFILL;
    long total = 0;
    for (int b = 0; b < B; ++b) total += lens[b] - keep;
    if (total < 1 || (mode == "auto" && total < 64)) return MLB_OK;
    if (s->m->cfg.weight_dtype != MLB_DT_BF16 && s->m->cfg.weight_dtype != MLB_DT_FP8_E4M3) {
        if (mode == "chunk") return fail(MLB_E_UNSUPPORTED, "MLB_PREFILL=chunk needs bf16 or FP8 weights");
        return MLB_OK;
    }
    if (!s->cols && !s->cols_tried) {
        s->cols_tried = true;
        int rc = session_create(s->m, kPromptCols, s->max_ctx, 0, 0, s, &s->cols);
        if (rc) {
            s->cols = nullptr;
            if (mode == "chunk") return rc;
        }
    }
    mlb_session* cs = s->cols;
    if (!cs) return MLB_OK;
    const int T = cs->B, MP = s->max_pages;
    int rc;
    if ((rc = ensure_graph(cs, kind))) return rc;
    const size_t V = (size_t)s->m->cfg.vocab;
    size_t scored = 0;
    std::vector<int> h_tok(T), h_pos(T), h_lim(T), h_seq(T), h_tab((size_t)T * MP);
    // A chunk takes the next tokens of as many sequences as it can, an equal share each: the
    // delta-net recurrence is serial along a sequence and parallel across sequences, so 64 sequences
    // with 2 columns each beat 1 sequence with 128. Columns stay grouped by sequence, positions ascending.
    std::vector<int> cursor(B, 0);
    long left = total;
    while (left > 0) {
        int n_active = 0;
        for (int b = 0; b < B; ++b) n_active += cursor[b] < lens[b] - keep ? 1 : 0;
        const int share = std::max(1, T / n_active);
        int n = 0;
        for (int b = 0; b < B && n < T; ++b) {
            const int take = std::min(std::min(share, lens[b] - keep - cursor[b]), T - n);
            for (int i = 0; i < take; ++i, ++n) {
                const int t = cursor[b] + i;
                h_tok[n] = tokens[(size_t)b * stride + t];
                h_pos[n] = t;
                h_lim[n] = t + 1;        // active: pos < limit
                h_seq[n] = b;
                std::memcpy(&h_tab[(size_t)n * MP], &s->h_table[(size_t)b * MP], (size_t)MP * 4);
            }
            if (take > 0) cursor[b] += take;
        }
        left -= n;
        for (int i = n; i < T; ++i) { h_tok[i] = 0; h_pos[i] = 0; h_lim[i] = 0; h_seq[i] = 0; }      // idle columns
        CU(cudaMemcpyAsync(cs->tok, h_tok.data(), (size_t)T * 4, cudaMemcpyHostToDevice, s->stream));
        CU(cudaMemcpyAsync(cs->pos, h_pos.data(), (size_t)T * 4, cudaMemcpyHostToDevice, s->stream));
        CU(cudaMemcpyAsync(kind == CHAIN_PREFILL ? cs->limit_prefill : cs->limit_decode, h_lim.data(), (size_t)T * 4, cudaMemcpyHostToDevice, s->stream));
        CU(cudaMemcpyAsync(cs->seq_of, h_seq.data(), (size_t)T * 4, cudaMemcpyHostToDevice, s->stream));
        CU(cudaMemcpyAsync(cs->page_table, h_tab.data(), h_tab.size() * 4, cudaMemcpyHostToDevice, s->stream));
        CU(cudaGraphLaunch(cs->graphs[kind], s->stream));
        if (score_out) {
            // one sequence: the columns of a chunk are its next n positions, in order
            CU(cudaMemcpyAsync(score_out + scored * V, cs->logits, (size_t)n * V * 4, cudaMemcpyDeviceToHost, s->stream));
            scored += (size_t)n;
        }
        CU(cudaStreamSynchronize(s->stream));          // the host arrays are rewritten for the next chunk
    }
    if (!score_out) {
        // what the token loop would have left: position len-1 with the last prompt token pending
        std::vector<int> pos(B), last(B);
        for (int i = 0; i < B; ++i) { pos[i] = lens[i] - 1; last[i] = tokens[(size_t)i * stride + lens[i] - 1]; }
        CU(cudaMemcpyAsync(s->pos, pos.data(), (size_t)B * 4, cudaMemcpyHostToDevice, s->stream));
        CU(cudaMemcpyAsync(s->tok, last.data(), (size_t)B * 4, cudaMemcpyHostToDevice, s->stream));
    }
    if ((rc = queue_err_readback(cs))) return rc;
    CU(cudaStreamSynchronize(s->stream));
    *done = true;
    return check_err_readback(cs);
}

extern "C" int mlb_prefill(mlb_session* s, const int32_t* tokens, const int32_t* lens, int stride) {
    if (!s || !tokens || !lens) return fail(MLB_E_INVALID, "null argument");
    CU(cudaSetDevice(s->m->device));
    const int B = s->B, V = s->m->cfg.vocab;
    int max_len = 0;
    for (int b = 0; b < B; ++b) {
        if (lens[b] < 1) return fail(MLB_E_INVALID, "sequence %d: prompt length must be >= 1 (got %d)", b, lens[b]);
        if (lens[b] > s->max_ctx) return fail(MLB_E_CONTEXT_FULL, "sequence %d: prompt of %d tokens exceeds max_context %d", b, lens[b], s->max_ctx);
        if (lens[b] > stride) return fail(MLB_E_INVALID, "sequence %d: length %d exceeds stride %d", b, lens[b], stride);
        for (int i = 0; i < lens[b]; ++i) {
            int t = tokens[(size_t)b * stride + i];
            if (t < 0 || t >= V) return fail(MLB_E_INVALID, "sequence %d: token %d at position %d is outside the vocabulary (%d)", b, t, i, V);
        }
        max_len = std::max(max_len, lens[b]);
    }
    int rc = mlb_session_reset(s);
    if (rc) return rc;
    std::vector<int> hp((size_t)B * s->max_ctx, 0), first(B), lim(B);
    for (int b = 0; b < B; ++b) {
        std::memcpy(&hp[(size_t)b * s->max_ctx], &tokens[(size_t)b * stride], (size_t)lens[b] * 4);
        first[b] = tokens[(size_t)b * stride];
        lim[b] = lens[b] - 1;
    }
    // pages for the whole prompt before any launch
    for (int b = 0; b < B; ++b) s->h_pos[b] = 0;
    bool has_attn = false;
    for (auto* p : s->kpool) if (p) has_attn = true;
    if (has_attn) {
        for (int b = 0; b < B; ++b) {
            if ((rc = kv_ensure(&s->alloc, b, lens[b], kKvBlock))) return rc;
        }
        s->table_dirty = true;
        if ((rc = sync_page_table(s))) return rc;
    }
    CU(cudaMemcpyAsync(s->prompt, hp.data(), hp.size() * 4, cudaMemcpyHostToDevice, s->stream));
    CU(cudaMemcpyAsync(s->tok, first.data(), (size_t)B * 4, cudaMemcpyHostToDevice, s->stream));
    CU(cudaMemcpyAsync(s->limit_prefill, lim.data(), (size_t)B * 4, cudaMemcpyHostToDevice, s->stream));
    CU(cudaStreamSynchronize(s->stream));
    bool by_columns = false;
    if ((rc = prefill_columns(s, tokens, lens, stride, &by_columns))) return rc;
    if (!by_columns && max_len > 1) {
        if ((rc = ensure_graph(s, CHAIN_PREFILL))) return rc;
        for (int t = 0; t < max_len - 1; ++t)
            if ((rc = launch_step(s, CHAIN_PREFILL))) return rc;
    }
    if ((rc = queue_err_readback(s))) return rc;
    CU(cudaStreamSynchronize(s->stream));
    for (int b = 0; b < B; ++b) s->h_pos[b] = lens[b] - 1;
    return check_err_readback(s);
}

extern "C" int mlb_score_tokens(mlb_session* s, const int32_t* tokens, int len, float* logits_out) {
    if (!s || !tokens || !logits_out) return fail(MLB_E_INVALID, "null argument");
    if (len < 1) return fail(MLB_E_INVALID, "len must be >= 1");
    if (len > s->max_ctx) return fail(MLB_E_CONTEXT_FULL, "%d tokens exceed max_context %d", len, s->max_ctx);
    CU(cudaSetDevice(s->m->device));
    const int V = s->m->cfg.vocab;
    for (int i = 0; i < len; ++i)
        if (tokens[i] < 0 || tokens[i] >= V) return fail(MLB_E_INVALID, "token %d at position %d is outside the vocabulary (%d)", tokens[i], i, V);
    const char* mode = std::getenv("MLB_SCORE");
    const bool by_steps = (mode && std::string(mode) == "step") ||
                          (s->m->cfg.weight_dtype != MLB_DT_BF16 && s->m->cfg.weight_dtype != MLB_DT_FP8_E4M3);
    if (by_steps) {
        // fp32 weights (or MLB_SCORE=step): the token loop with the given ids forced in, fp32 activations, the
        // logits of every step copied out - what the reference's trainer reads after runInference(L)
        // (training_orchestrator.cu:308), within the fp32 bound of the decode path
        std::vector<int32_t> first(s->B, 0), lens(s->B, 1), in(s->B, 0), out(s->B, 0);
        first[0] = tokens[0];
        int rc = mlb_prefill(s, first.data(), lens.data(), 1);
        if (rc) return rc;
        std::vector<float> row((size_t)s->B * V);
        for (int t = 0; t < len; ++t) {
            in[0] = tokens[t];
            if ((rc = mlb_decode_step(s, nullptr, in.data(), out.data()))) return rc;
            if ((rc = mlb_get_logits(s, row.data()))) return rc;
            std::memcpy(logits_out + (size_t)t * V, row.data(), (size_t)V * 4);
        }
        return mlb_session_reset(s);
    }
    int rc = mlb_session_reset(s);
    if (rc) return rc;
    bool has_attn = false;
    for (auto* p : s->kpool) if (p) has_attn = true;
    if (has_attn) {
        if ((rc = kv_ensure(&s->alloc, 0, len, kKvBlock))) return rc;
        s->table_dirty = true;
        if ((rc = sync_page_table(s))) return rc;
    }
    bool done = false;
    const int32_t lens[1] = {len};
    rc = prefill_columns(s, tokens, lens, len, &done, logits_out);
    const int rc2 = mlb_session_reset(s);          // the cache holds the scored sequence: not a state to decode from
    if (rc) return rc;
    if (!done) return fail(MLB_E_UNSUPPORTED, "the scoring forward could not set up its tensor-core columns");
    return rc2;
}

extern "C" int mlb_session_set_stop_token(mlb_session* s, int token_id) {
    if (!s) return fail(MLB_E_INVALID, "null session");
    if (token_id >= s->m->cfg.vocab) return fail(MLB_E_INVALID, "stop token %d is outside the vocabulary of %d", token_id, s->m->cfg.vocab);
    if (token_id < 0) token_id = -1;
    if (token_id == s->stop_token) return MLB_OK;
    CU(cudaSetDevice(s->m->device));
    CU(cudaStreamSynchronize(s->stream));
    // the id is an argument of the captured launches: capture again on next use
    for (auto& g : s->graphs) if (g) { cudaGraphExecDestroy(g); g = nullptr; }
    for (auto& g : s->tgraphs) if (g) { cudaGraphExecDestroy(g); g = nullptr; }
    s->stop_token = token_id;
    return MLB_OK;
}

extern "C" int mlb_session_stopped(mlb_session* s, int32_t* out_flags) {
    if (!s || !out_flags) return fail(MLB_E_INVALID, "null argument");
    for (int b = 0; b < s->B; ++b) out_flags[b] = s->h_stopped[b] ? 1 : 0;
    return MLB_OK;
}

namespace mlb {
// Shared body of the decode entry points. step_ms != null times each step.
static int decode_impl(mlb_session* s, const mlb_sampling* sp, int n, const int32_t* in_tokens, int32_t* out_tokens,
                       float* step_ms, float* total_ms, int flush_l2) {
    if (!s || !out_tokens) return fail(MLB_E_INVALID, "null argument");
    if (n < 1) return fail(MLB_E_INVALID, "n must be >= 1");
    CU(cudaSetDevice(s->m->device));
    const int B = s->B;
    bool any = false;
    for (int b = 0; b < B; ++b) any = any || seq_live(s, b);
    if (!any) return fail(MLB_E_CONTEXT_FULL, "every sequence is at max_context %d or has drawn the stop token", s->max_ctx);
    if (n > s->max_ctx) n = std::min(n, s->max_ctx);
    int kind, rc;
    if ((rc = apply_sampling(s, sp, &kind))) return rc;
    if ((rc = grow_pages(s, n))) return rc;
    if (in_tokens) {
        const int V = s->m->cfg.vocab;
        for (int b = 0; b < B; ++b) {
            if (in_tokens[b] < 0 || in_tokens[b] >= V) return fail(MLB_E_INVALID, "sequence %d: token %d is outside the vocabulary", b, in_tokens[b]);
            s->pinned_tok[b] = in_tokens[b];
        }
    }
    if (n == 1 && !step_ms && !s->use_grid && !s->use_lean) {
        // the one-token call: one graph launch, one synchronisation
        if ((rc = ensure_token_graph(s, kind, in_tokens != nullptr))) return rc;
        // The kernel that advances a sequence writes its id to pinned host memory (the error word first, by
        // sequence 0): the host polls those words instead of synchronising the stream, which wakes it later.
        const bool poll = seq_live(s, 0);
        volatile int* words = s->pinned_out;
        if (poll)
            for (int b = 0; b < B; ++b) words[b] = seq_live(s, b) ? -2 : -1;
        CU(cudaGraphLaunch(s->tgraphs[kind * 2 + (in_tokens ? 1 : 0)], s->stream));
        bool arrived = false;
        if (poll) {
            const auto t0 = std::chrono::steady_clock::now();
            for (unsigned spins = 0; !arrived; ++spins) {
                arrived = true;
                for (int b = 0; b < B; ++b)
                    if (words[b] == -2) { arrived = false; break; }
                if (!arrived && (spins & 0xfffu) == 0xfffu && std::chrono::steady_clock::now() - t0 > std::chrono::seconds(5)) break;
            }
        }
        if (!arrived) CU(cudaStreamSynchronize(s->stream));
        for (int b = 0; b < B; ++b) {
            out_tokens[b] = s->pinned_out[b];
            note_outputs(s, b, &out_tokens[b], 1);
        }
        s->have_logits = true;
        return check_err_readback(s);
    }
    if (n == 1 && !step_ms && B == 1 && (s->use_grid || s->use_lean) && seq_live(s, 0)) {
        // The one-token call of the single-kernel step: the pending id travels as a launch argument, the
        // kernel that advances the sequence writes the picked id and the error word to pinned host memory,
        // and the host polls that word instead of synchronising the stream (which costs 5-10 us more).
        if ((rc = ensure_graph(s, kind))) return rc;
        volatile int* word = s->pinned_out;
        *word = -2;
        s->ctl_host_io = 1;
        s->tok_arg = in_tokens ? in_tokens[0] : -1;
        rc = chain_run(s, kind, nullptr, nullptr);
        s->ctl_host_io = 0;
        s->tok_arg = -1;
        if (rc) return rc;
        const auto t0 = std::chrono::steady_clock::now();
        for (unsigned spins = 0; *word == -2; ++spins) {
            if ((spins & 0xffffu) == 0xffffu && std::chrono::steady_clock::now() - t0 > std::chrono::seconds(5)) break;
        }
        if (*word == -2) CU(cudaStreamSynchronize(s->stream));       // a wait ran out on the device, or the launch failed late
        if (*word == -2) return fail(MLB_E_CUDA, "the decode step ended without a token");
        out_tokens[0] = *word;
        note_outputs(s, 0, &out_tokens[0], 1);
        s->have_logits = true;
        return check_err_readback(s);
    }
    if ((rc = ensure_graph(s, kind))) return rc;
    if (in_tokens) CU(cudaMemcpyAsync(s->tok, s->pinned_tok, (size_t)B * 4, cudaMemcpyHostToDevice, s->stream));
    CU(cudaMemsetAsync(s->out_idx, 0, (size_t)B * 4, s->stream));
    std::vector<cudaEvent_t> ev;
    if (step_ms) {
        ev.resize(2 * (size_t)n);
        for (auto& e : ev) CU(cudaEventCreate(&e));
    }
    for (int i = 0; i < n; ++i) {
        if (step_ms) {
            if (flush_l2) {
                l2_flush_kernel<<<1184, 256, 0, s->stream>>>(s->flush_buf, s->flush_n, (float)i);
                CU(cudaGetLastError());
            }
            CU(cudaEventRecord(ev[2 * i], s->stream));
        }
        if ((rc = launch_step(s, kind))) return rc;
        if (step_ms) CU(cudaEventRecord(ev[2 * i + 1], s->stream));
    }
    // result: ring [B][max_ctx] -> out [B][n]
    if ((rc = queue_err_readback(s))) return rc;
    if (n == 1) {
        // one id per sequence: gather through the pinned buffer
        CU(cudaMemcpy2DAsync(s->pinned_tok, 4, s->out_ring, (size_t)s->max_ctx * 4, 4, B, cudaMemcpyDeviceToHost, s->stream));
        CU(cudaStreamSynchronize(s->stream));
        for (int b = 0; b < B; ++b) out_tokens[b] = s->pinned_tok[b];
    } else {
        std::vector<int> ring((size_t)B * n);
        CU(cudaMemcpy2DAsync(ring.data(), (size_t)n * 4, s->out_ring, (size_t)s->max_ctx * 4, (size_t)n * 4, B, cudaMemcpyDeviceToHost, s->stream));
        CU(cudaStreamSynchronize(s->stream));
        std::memcpy(out_tokens, ring.data(), ring.size() * 4);
    }
    if (step_ms) {
        for (int i = 0; i < n; ++i) CU(cudaEventElapsedTime(&step_ms[i], ev[2 * i], ev[2 * i + 1]));
        if (total_ms) CU(cudaEventElapsedTime(total_ms, ev[0], ev[2 * (size_t)n - 1]));
        for (auto& e : ev) cudaEventDestroy(e);
    }
    for (int b = 0; b < B; ++b) note_outputs(s, b, &out_tokens[(size_t)b * n], n);
    s->have_logits = true;
    return check_err_readback(s);
}
}  // namespace mlb

extern "C" int mlb_decode_step(mlb_session* s, const mlb_sampling* sp, const int32_t* in_tokens, int32_t* out_tokens) {
    return decode_impl(s, sp, 1, in_tokens, out_tokens, nullptr, nullptr, 0);
}
extern "C" int mlb_decode_n(mlb_session* s, const mlb_sampling* sp, int n, int32_t* out_tokens) {
    return decode_impl(s, sp, n, nullptr, out_tokens, nullptr, nullptr, 0);
}
extern "C" int mlb_decode_timed(mlb_session* s, const mlb_sampling* sp, int n, int flush_l2, float* step_ms, float* total_ms,
                                int32_t* out_tokens) {
    if (!step_ms) return fail(MLB_E_INVALID, "null step_ms");
    return decode_impl(s, sp, n, nullptr, out_tokens, step_ms, total_ms, flush_l2);
}

extern "C" int mlb_profile_decode(mlb_session* s, const mlb_sampling* sp, int n, int flush_l2, mlb_kernel_stat* stats,
                                  int max_stats, int* n_stats) {
    if (!s || !stats || !n_stats) return fail(MLB_E_INVALID, "null argument");
    CU(cudaSetDevice(s->m->device));
    int kind, rc;
    if ((rc = apply_sampling(s, sp, &kind))) return rc;
    if ((rc = grow_pages(s, n))) return rc;
    CU(cudaMemsetAsync(s->out_idx, 0, (size_t)s->B * 4, s->stream));
    Recorder rec;
    rec.st = s->stream;
    for (int i = 0; i < n; ++i) {
        bool any = false;
        for (int b = 0; b < s->B; ++b) any = any || seq_live(s, b);
        if (!any) break;
        if (flush_l2) {
            l2_flush_kernel<<<1184, 256, 0, s->stream>>>(s->flush_buf, s->flush_n, (float)i);
            CU(cudaGetLastError());
        }
        if ((rc = chain_run(s, kind, &rec, nullptr))) return rc;
        for (int b = 0; b < s->B; ++b) if (seq_live(s, b)) s->h_pos[b] += 1;
    }
    CU(cudaStreamSynchronize(s->stream));
    if (s->stop_token >= 0) {
        // no ids came back: take positions and who stopped from the device
        std::vector<int> dp(s->B), dl(s->B);
        CU(cudaMemcpy(dp.data(), s->pos, (size_t)s->B * 4, cudaMemcpyDeviceToHost));
        CU(cudaMemcpy(dl.data(), s->limit_decode, (size_t)s->B * 4, cudaMemcpyDeviceToHost));
        for (int b = 0; b < s->B; ++b) {
            s->h_pos[b] = std::min(dp[b], s->max_ctx);
            s->h_stopped[b] = dl[b] < s->max_ctx;
        }
    }
    s->have_logits = true;
    int count = 0;
    for (auto& r : rec.recs) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, r.e0, r.e1);
        cudaEventDestroy(r.e0);
        cudaEventDestroy(r.e1);
        int j = 0;
        for (; j < count; ++j) if (std::strcmp(stats[j].name, r.name) == 0) break;
        if (j == count) {
            if (count >= max_stats) continue;
            std::memset(&stats[j], 0, sizeof stats[j]);
            std::strncpy(stats[j].name, r.name, sizeof(stats[j].name) - 1);
            ++count;
        }
        stats[j].launches += 1;
        stats[j].total_ms += ms;
        stats[j].bytes += r.bytes;
        stats[j].flops += r.flops;
    }
    *n_stats = count;
    return MLB_OK;
}

extern "C" int mlb_get_logits(mlb_session* s, float* out) {
    if (!s || !out) return fail(MLB_E_INVALID, "null argument");
    if (!s->have_logits) return fail(MLB_E_INVALID, "no decode step has run since the last prefill/reset");
    CU(cudaSetDevice(s->m->device));
    CU(cudaMemcpyAsync(out, s->logits, (size_t)s->B * s->m->cfg.vocab * 4, cudaMemcpyDeviceToHost, s->stream));
    CU(cudaStreamSynchronize(s->stream));
    return MLB_OK;
}

extern "C" int mlb_get_probs_col(mlb_session* s, int seq, float* out) {
    if (!s || !out) return fail(MLB_E_INVALID, "null argument");
    if (seq < 0 || seq >= s->B) return fail(MLB_E_INVALID, "sequence index out of range");
    if (!s->have_logits) return fail(MLB_E_INVALID, "no decode step has run since the last prefill/reset");
    CU(cudaSetDevice(s->m->device));
    const int V = s->m->cfg.vocab;
    softmax_probe_kernel<<<1, 256, 0, s->stream>>>(s->logits + (size_t)seq * V, V, s->probe);
    CU(cudaGetLastError());
    CU(cudaMemcpyAsync(out, s->probe, (size_t)V * 4, cudaMemcpyDeviceToHost, s->stream));
    CU(cudaStreamSynchronize(s->stream));
    return MLB_OK;
}

extern "C" int mlb_session_positions(mlb_session* s, int32_t* out) {
    if (!s || !out) return fail(MLB_E_INVALID, "null argument");
    CU(cudaSetDevice(s->m->device));
    CU(cudaMemcpyAsync(out, s->pos, (size_t)s->B * 4, cudaMemcpyDeviceToHost, s->stream));
    CU(cudaStreamSynchronize(s->stream));
    return MLB_OK;
}

extern "C" int mlb_session_step_bytes(mlb_session* s, uint64_t* weights, uint64_t* kv, uint64_t* state, uint64_t* rows) {
    if (!s) return fail(MLB_E_INVALID, "null session");
    const mlb_config& c = s->m->cfg;
    uint64_t kvb = 0, st = 0, rw = 0;
    const uint64_t kv_elt = elt_size(c.kv_dtype), w_elt = elt_size(c.weight_dtype), p_elt = elt_size(ple_dtype(c.weight_dtype));
    for (int b = 0; b < s->B; ++b) {
        if (!seq_live(s, b)) continue;
        for (int i = 0; i < c.layers; ++i) {
            if (c.layer_types[i] == MLB_LAYER_ATTENTION) kvb += 2ull * c.kv_heads * c.head_dim * kv_elt * (s->h_pos[b] + 1);
            else st += 2ull * c.heads * c.dn_key_dim * c.dn_value_dim * 4;
        }
        rw += (uint64_t)c.dim * w_elt + (uint64_t)c.layers * c.ple_dim * p_elt;
    }
    if (weights) *weights = s->m->weight_bytes;   // the tied table is streamed once (LM head)
    if (kv) *kv = kvb;
    if (state) *state = st;
    if (rows) *rows = rw;
    return MLB_OK;
}

extern "C" int mlb_session_grid_timers(mlb_session* s, long long* out, int cap) {
    if (!s || !out) return fail(MLB_E_INVALID, "null argument");
    long long* timers = s->use_lean ? s->lean.timers : (s->use_grid ? s->grid.timers : nullptr);
    if (!timers) return 0;
    CU(cudaSetDevice(s->m->device));
    const int n = s->grid_ctas * kGridTimerSlots;
    if (cap < n) return fail(MLB_E_INVALID, "room for %d counters needed, %d given", n, cap);
    CU(cudaStreamSynchronize(s->stream));
    CU(cudaMemcpy(out, timers, (size_t)n * 8, cudaMemcpyDeviceToHost));
    CU(cudaMemset(timers, 0, (size_t)n * 8));
    return s->grid_ctas;
}

extern "C" int mlb_session_grid_trace(mlb_session* s, long long* out, int cap) {
    if (!s || !out) return fail(MLB_E_INVALID, "null argument");
    if (s->tc_trace) {
        // tensor-core step: 8 words per GEMM launch of the last step (entry, set up, predecessor complete,
        // accumulators complete, epilogue done), 64 launches at most
        if (cap < 512) return fail(MLB_E_INVALID, "room for 512 words needed, %d given", cap);
        CU(cudaSetDevice(s->m->device));
        CU(cudaStreamSynchronize(s->stream));
        CU(cudaMemcpy(out, s->tc_trace, 512 * 8, cudaMemcpyDeviceToHost));
        return 64;
    }
    if (!s->use_lean || !s->lean.trace) return 0;
    CU(cudaSetDevice(s->m->device));
    const int n = s->grid_ctas * kLeanTraceLen;
    if (cap < n) return fail(MLB_E_INVALID, "room for %d events needed, %d given", n, cap);
    CU(cudaStreamSynchronize(s->stream));
    CU(cudaMemcpy(out, s->lean.trace, (size_t)n * 8, cudaMemcpyDeviceToHost));
    return s->grid_ctas;
}

extern "C" int mlb_session_launches_per_step(mlb_session* s) {
    if (!s) return fail(MLB_E_INVALID, "null session");
    int rc = ensure_graph(s, CHAIN_GREEDY);
    if (rc) return rc;
    return s->launches_per_step[CHAIN_GREEDY];
}

// ---- host-only allocator entry points --------------------------------------------------
extern "C" int mlb_kv_alloc_new(int num_pages, int batch, int max_pages_per_seq, mlb_kv_alloc** out) {
    if (!out || num_pages < 0 || batch < 1 || max_pages_per_seq < 1) return fail(MLB_E_INVALID, "kv allocator: bad argument");
    mlb_kv_alloc* a = new mlb_kv_alloc();
    a->num_pages = num_pages;
    a->max_pages_per_seq = max_pages_per_seq;
    a->seq_pages.assign(batch, {});
    for (int p = num_pages - 1; p >= 0; --p) a->free_list.push_back(p);
    *out = a;
    return MLB_OK;
}
extern "C" int mlb_kv_alloc_ensure(mlb_kv_alloc* a, int seq, int n_positions, int block) { return kv_ensure(a, seq, n_positions, block); }
extern "C" int mlb_kv_alloc_table(const mlb_kv_alloc* a, int seq, int32_t* out, int max_entries) {
    if (!a || !out || seq < 0 || seq >= (int)a->seq_pages.size()) return fail(MLB_E_INVALID, "kv allocator: bad argument");
    const auto& pg = a->seq_pages[seq];
    int n = std::min((int)pg.size(), max_entries);
    for (int i = 0; i < n; ++i) out[i] = pg[i];
    return (int)pg.size();
}
extern "C" int mlb_kv_alloc_free_pages(const mlb_kv_alloc* a) { return a ? (int)a->free_list.size() : fail(MLB_E_INVALID, "null allocator"); }
extern "C" void mlb_kv_alloc_release(mlb_kv_alloc* a, int seq) {
    if (!a || seq < 0 || seq >= (int)a->seq_pages.size()) return;
    for (int pg : a->seq_pages[seq]) a->free_list.push_back(pg);
    a->seq_pages[seq].clear();
}
extern "C" void mlb_kv_alloc_free(mlb_kv_alloc* a) { delete a; }

extern "C" const char* mlb_last_error(void) { return g_err.c_str(); }
extern "C" const char* mlb_version(void) { return "mini-llm-b200 0.1 (sm_100a)"; }
