#include "model_file.h"

#include <cmath>
#include <cstdio>
#include <cstring>

#include "json_min.h"

namespace mlb {

namespace {

const char* const kBaseKeys[] = {"rmsGamma", "queryWeights", "keyWeights", "valueWeights",
                                 "outputProjectionWeights", "rmsGamma2", "feedForwardWeights1A",
                                 "feedForwardWeights1B", "feedForwardWeights2",
                                 // config-guarded tensors follow the nine base ones (load_model.cu:442-450)
                                 "queryRMSGamma", "keyRMSGamma", "gatedQueryWeights"};

bool parse_meta(const JsonValue& v, TensorDesc* t, std::string* err) {
    // parseTensorMeta, load_model.cu:24-61
    const JsonValue* shape = v.get("shape");
    const JsonValue* dtype = v.get("dtype");
    if (!shape || !shape->is(JsonValue::Array) || !dtype || !dtype->is(JsonValue::String)) {
        *err = "tensor '" + t->name + "' lacks shape/dtype";
        return false;
    }
    t->ndim = static_cast<int>(shape->items.size());
    if (t->ndim < 1 || t->ndim > 2) {
        *err = "tensor '" + t->name + "': unsupported number of dimensions";
        return false;
    }
    double r = shape->items[0].num, c = t->ndim == 2 ? shape->items[1].num : 1.0;
    if (!(r >= 1 && r <= 2147483647.0) || !(c >= 1 && c <= 2147483647.0)) {
        *err = "tensor '" + t->name + "': bad shape";
        return false;
    }
    t->rows = static_cast<int>(r);
    t->cols = static_cast<int>(c);
    uint64_t n = static_cast<uint64_t>(t->rows) * static_cast<uint64_t>(t->cols);
    if (dtype->str == "float32") { t->dtype = FD_F32; t->nbytes = 4 * n; }
    else if (dtype->str == "float64") { t->dtype = FD_F64; t->nbytes = 8 * n; }
    else if (dtype->str == "bfloat16") { t->dtype = FD_BF16; t->nbytes = 2 * n; }
    else if (dtype->str == "float8_e4m3") {
        if (t->ndim != 2) {
            *err = "tensor '" + t->name + "': float8_e4m3 needs a matrix (codes with one scale per row)";
            return false;
        }
        t->dtype = FD_FP8;
        t->nbytes = n + 4 * static_cast<uint64_t>(t->rows);
    }
    else {
        *err = "Unsupported dtype: " + dtype->str;     // load_model.cu:55-57
        return false;
    }
    return true;
}

int json_int(const JsonValue* v, int dflt) {
    if (!v) return dflt;
    if (v->is(JsonValue::Number)) return static_cast<int>(v->num);
    if (v->is(JsonValue::Bool)) return v->b ? 1 : 0;
    return dflt;
}

int dtype_from_string(const std::string& s) {
    if (s == "float32") return MLB_DT_F32;
    if (s == "bfloat16") return MLB_DT_BF16;
    if (s == "float8_e4m3") return MLB_DT_FP8_E4M3;
    return -1;
}

}  // namespace

const TensorDesc* ParsedModel::find(int block, const char* name) const {
    for (const auto& t : tensors)
        if (t.block == block && t.name == name) return &t;
    return nullptr;
}

int read_file(const char* path, std::vector<unsigned char>* out, std::string* err) {
    FILE* f = std::fopen(path, "rb");
    if (!f) {
        *err = std::string("Model file not found at '") + path + "'";
        return MLB_E_IO;
    }
    std::fseek(f, 0, SEEK_END);
    long sz = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    if (sz < 0) { std::fclose(f); *err = "cannot size file"; return MLB_E_IO; }
    try {
        out->resize(static_cast<size_t>(sz));
    } catch (...) {
        std::fclose(f);
        *err = "out of host memory reading the model file";
        return MLB_E_NOMEM;
    }
    size_t got = sz ? std::fread(out->data(), 1, static_cast<size_t>(sz), f) : 0;
    std::fclose(f);
    if (got != static_cast<size_t>(sz)) { *err = "Failed to read file."; return MLB_E_IO; }
    return MLB_OK;
}

float e4m3_to_f32(unsigned char code) {
    const int e = (code >> 3) & 15, m = code & 7;
    float v;
    if (e == 15 && m == 7) v = std::nanf("");
    else if (e == 0) v = std::ldexp(static_cast<float>(m), -9);              // subnormal: m / 8 * 2^-6
    else v = std::ldexp(1.0f + static_cast<float>(m) / 8.0f, e - 7);
    return (code & 0x80) ? -v : v;
}

void convert_to_f32(const unsigned char* src, FileDtype dt, uint64_t n, float* dst, uint64_t cols) {
    if (dt == FD_FP8) {
        const uint64_t rows = cols ? n / cols : 0;
        for (uint64_t r = 0; r < rows; ++r) {
            float sc;
            std::memcpy(&sc, src + n + 4 * r, 4);
            for (uint64_t c = 0; c < cols; ++c) dst[r * cols + c] = e4m3_to_f32(src[r * cols + c]) * sc;
        }
        return;
    }
    if (dt == FD_F32) {
        std::memcpy(dst, src, n * 4);
    } else if (dt == FD_F64) {
        for (uint64_t i = 0; i < n; ++i) {       // narrowing as load_model.cu:81-85
            double d;
            std::memcpy(&d, src + 8 * i, 8);
            dst[i] = static_cast<float>(d);
        }
    } else {
        for (uint64_t i = 0; i < n; ++i) {
            uint16_t h;
            std::memcpy(&h, src + 2 * i, 2);
            uint32_t u = static_cast<uint32_t>(h) << 16;
            std::memcpy(&dst[i], &u, 4);
        }
    }
}

int parse_model_header(const unsigned char* data, uint64_t avail, uint64_t file_size,
                       const mlb_config* ov, ParsedModel* out, std::string* err) {
    if (avail < 8) { *err = "file shorter than its 8-byte header length"; return MLB_E_FORMAT; }
    uint64_t hlen = 0;
    for (int i = 0; i < 8; ++i) hlen |= static_cast<uint64_t>(data[i]) << (8 * i);   // load_model.cu:320-324
    if (hlen > file_size || 8 + hlen > file_size || 8 + hlen > avail) {
        *err = "Header length specified in file is larger than the file itself.";
        return MLB_E_FORMAT;
    }
    JsonValue root;
    JsonParser parser(reinterpret_cast<const char*>(data + 8), static_cast<size_t>(hlen));
    if (!parser.parse(&root) || !root.is(JsonValue::Object)) {
        *err = "Error parsing JSON header: " + parser.error();
        return MLB_E_FORMAT;
    }
    uint64_t off = 8 + hlen;
    off += (8 - off % 8) % 8;                                  // load_model.cu:341-343
    out->tensors.clear();
    out->n_params = 0;
    out->file_size = file_size;

    auto add = [&](const JsonValue& meta, const std::string& name, int block) -> int {
        TensorDesc t;
        t.name = name;
        t.block = block;
        if (!parse_meta(meta, &t, err)) return MLB_E_FORMAT;
        t.offset = off;
        if (off + t.nbytes > file_size) {
            *err = "Attempting to read past buffer end (tensor '" + name + "').";   // load_model.cu:69-72
            return MLB_E_FORMAT;
        }
        off += t.nbytes;
        out->n_params += static_cast<uint64_t>(t.rows) * t.cols;
        out->tensors.push_back(t);
        return MLB_OK;
    };

    const JsonValue* emb = root.get("tokenEmbeddings");
    const JsonValue* fin = root.get("finalRMSNormGamma");
    const JsonValue* blocks = root.get("transformerBlocks");
    if (!emb || !fin || !blocks || !blocks->is(JsonValue::Array)) {
        *err = "header lacks tokenEmbeddings / finalRMSNormGamma / transformerBlocks";
        return MLB_E_FORMAT;
    }
    int rc;
    if ((rc = add(*emb, "tokenEmbeddings", -1)) != MLB_OK) return rc;
    if ((rc = add(*fin, "finalRMSNormGamma", -1)) != MLB_OK) return rc;
    const int n_blocks = static_cast<int>(blocks->items.size());
    if (n_blocks < 1 || n_blocks > MLB_MAX_LAYERS) { *err = "unsupported number of transformer blocks"; return MLB_E_FORMAT; }
    for (int b = 0; b < n_blocks; ++b) {
        const JsonValue& blk = blocks->items[b];
        if (!blk.is(JsonValue::Object)) { *err = "Expected transformer block object."; return MLB_E_FORMAT; }
        for (const char* key : kBaseKeys) {
            const JsonValue* m = blk.get(key);
            if (!m) continue;                                  // a missing key does not advance (load_model.cu:436-438)
            if ((rc = add(*m, key, b)) != MLB_OK) return rc;
        }
    }
    if (const JsonValue* ext = root.get("ext")) {
        if (!ext->is(JsonValue::Array)) { *err = "'ext' must be an array"; return MLB_E_FORMAT; }
        for (const JsonValue& e : ext->items) {
            const JsonValue* nm = e.get("name");
            const JsonValue* bl = e.get("block");
            if (!nm || !nm->is(JsonValue::String) || !bl || !bl->is(JsonValue::Number)) {
                *err = "'ext' entry lacks name/block";
                return MLB_E_FORMAT;
            }
            int b = static_cast<int>(bl->num);
            if (b < 0 || b >= n_blocks) { *err = "'ext' entry names a block that does not exist"; return MLB_E_FORMAT; }
            if ((rc = add(e, nm->str, b)) != MLB_OK) return rc;
        }
    }

    // ---- configuration: shapes, then the file's "config", then the caller's override ----
    mlb_config& c = out->cfg;
    mlb_config_init(&c);
    const TensorDesc* te = out->find(-1, "tokenEmbeddings");
    if (te->ndim != 2) { *err = "tokenEmbeddings must be 2-D [vocab, dim]"; return MLB_E_FORMAT; }
    c.vocab = te->rows;
    c.dim = te->cols;
    c.layers = n_blocks;
    const TensorDesc* f1 = out->find(0, "feedForwardWeights1A");
    if (!f1) { *err = "block 0 lacks feedForwardWeights1A"; return MLB_E_FORMAT; }
    c.ffn_dim = f1->rows;
    const JsonValue* jc = root.get("config");
    if (jc && jc->is(JsonValue::Object)) {
        c.heads = json_int(jc->get("heads"), -1);
        c.kv_heads = json_int(jc->get("kv_heads"), -1);
        c.head_dim = json_int(jc->get("head_dim"), -1);
        c.max_context = json_int(jc->get("max_context"), -1);
        c.ple_dim = json_int(jc->get("ple_dim"), -1);
        c.qk_norm = json_int(jc->get("qk_norm"), -1);
        c.query_gating = json_int(jc->get("query_gating"), -1);
        c.dn_key_dim = json_int(jc->get("dn_key_dim"), -1);
        c.dn_value_dim = json_int(jc->get("dn_value_dim"), -1);
        if (const JsonValue* v = jc->get("rope_theta")) if (v->is(JsonValue::Number)) c.rope_theta = static_cast<float>(v->num);
        if (const JsonValue* v = jc->get("rms_eps")) if (v->is(JsonValue::Number)) c.rms_eps = static_cast<float>(v->num);
        if (const JsonValue* v = jc->get("weight_dtype")) if (v->is(JsonValue::String)) c.weight_dtype = dtype_from_string(v->str);
        if (const JsonValue* v = jc->get("kv_dtype")) if (v->is(JsonValue::String)) c.kv_dtype = dtype_from_string(v->str);
        if (const JsonValue* lt = jc->get("layer_types")) {
            if (!lt->is(JsonValue::Array) || static_cast<int>(lt->items.size()) != n_blocks) {
                *err = "config.layer_types must list one entry per block";
                return MLB_E_FORMAT;
            }
            for (int i = 0; i < n_blocks; ++i) {
                const std::string& s = lt->items[i].str;
                if (s == "attention") c.layer_types[i] = MLB_LAYER_ATTENTION;
                else if (s == "delta_net") c.layer_types[i] = MLB_LAYER_DELTA_NET;
                else { *err = "unknown layer type '" + s + "'"; return MLB_E_FORMAT; }
            }
            c.layer_types_set = 1;
        }
    }
    if (ov) {
        if (ov->heads >= 0) c.heads = ov->heads;
        if (ov->kv_heads >= 0) c.kv_heads = ov->kv_heads;
        if (ov->head_dim >= 0) c.head_dim = ov->head_dim;
        if (ov->max_context >= 0) c.max_context = ov->max_context;
        if (ov->ple_dim >= 0) c.ple_dim = ov->ple_dim;
        if (ov->qk_norm >= 0) c.qk_norm = ov->qk_norm;
        if (ov->query_gating >= 0) c.query_gating = ov->query_gating;
        if (ov->dn_key_dim >= 0) c.dn_key_dim = ov->dn_key_dim;
        if (ov->dn_value_dim >= 0) c.dn_value_dim = ov->dn_value_dim;
        if (ov->weight_dtype > 0) c.weight_dtype = ov->weight_dtype;
        if (ov->kv_dtype > 0) c.kv_dtype = ov->kv_dtype;
        if (!std::isnan(ov->rope_theta)) c.rope_theta = ov->rope_theta;
        if (!std::isnan(ov->rms_eps)) c.rms_eps = ov->rms_eps;
        if (ov->layer_types_set) {
            std::memcpy(c.layer_types, ov->layer_types, sizeof(c.layer_types));
            c.layer_types_set = 1;
        }
    }
    if (c.heads <= 0 || c.head_dim <= 0) {
        *err = "heads/head_dim are not derivable from tensor shapes: the file needs a 'config' key or the caller an override";
        return MLB_E_INVALID;
    }
    if (c.kv_heads <= 0) c.kv_heads = c.heads;
    if (c.max_context <= 0) c.max_context = 1024;
    if (c.ple_dim < 0) c.ple_dim = 0;
    if (c.qk_norm < 0) c.qk_norm = out->find(0, "queryRMSGamma") || out->find(n_blocks - 1, "queryRMSGamma") ? 1 : 0;
    if (c.query_gating < 0) c.query_gating = out->find(0, "gatedQueryWeights") || out->find(n_blocks - 1, "gatedQueryWeights") ? 1 : 0;
    if (c.dn_key_dim <= 0) c.dn_key_dim = c.head_dim;
    if (c.dn_value_dim <= 0) c.dn_value_dim = c.head_dim;
    if (c.weight_dtype <= 0) c.weight_dtype = MLB_DT_F32;
    if (c.kv_dtype <= 0) c.kv_dtype = MLB_DT_F32;
    if (std::isnan(c.rope_theta)) c.rope_theta = 10000.0f;     // ropeDenomBase, network_meta.h:7
    if (std::isnan(c.rms_eps)) c.rms_eps = 1e-8f;              // inference.cu:48
    if (!c.layer_types_set) {
        for (int i = 0; i < n_blocks; ++i) c.layer_types[i] = MLB_LAYER_ATTENTION;
        c.layer_types_set = 1;
    }
    if (c.heads % c.kv_heads != 0) { *err = "heads must be a multiple of kv_heads"; return MLB_E_INVALID; }
    if (c.kv_dtype != MLB_DT_F32 && c.kv_dtype != MLB_DT_BF16) { *err = "kv_dtype must be float32 or bfloat16"; return MLB_E_INVALID; }
    if (c.weight_dtype < MLB_DT_F32 || c.weight_dtype > MLB_DT_FP8_E4M3) { *err = "unknown weight_dtype"; return MLB_E_INVALID; }

    // ---- shape validation per block ----
    auto expect = [&](int block, const char* name, int rows, int cols, bool required) -> int {
        const TensorDesc* t = out->find(block, name);
        if (!t) {
            if (!required) return MLB_OK;
            char buf[160];
            std::snprintf(buf, sizeof buf, "Weight '%s' not found in block %d", name, block);
            *err = buf;
            return MLB_E_FORMAT;
        }
        if (t->rows != rows || t->cols != cols) {
            char buf[200];
            std::snprintf(buf, sizeof buf, "block %d '%s' has shape [%d, %d], expected [%d, %d]", block, name,
                          t->rows, t->cols, rows, cols);
            *err = buf;
            return MLB_E_FORMAT;
        }
        return MLB_OK;
    };
    const int d = c.dim, F = c.ffn_dim;
    if ((rc = expect(-1, "finalRMSNormGamma", d, 1, true)) != MLB_OK) return rc;
    for (int b = 0; b < n_blocks; ++b) {
        const int type = c.layer_types[n_blocks - 1 - b];      // block b runs at execution index N-1-b
        int q_out, k_out, v_out;
        if (type == MLB_LAYER_ATTENTION) {
            q_out = c.heads * c.head_dim;
            k_out = v_out = c.kv_heads * c.head_dim;
        } else {
            q_out = k_out = c.heads * c.dn_key_dim;
            v_out = c.heads * c.dn_value_dim;
        }
        const int o_in = type == MLB_LAYER_ATTENTION ? q_out : v_out;
        if ((rc = expect(b, "rmsGamma", d, 1, true)) != MLB_OK) return rc;
        if ((rc = expect(b, "queryWeights", q_out, d, true)) != MLB_OK) return rc;
        if ((rc = expect(b, "keyWeights", k_out, d, true)) != MLB_OK) return rc;
        if ((rc = expect(b, "valueWeights", v_out, d, true)) != MLB_OK) return rc;
        if ((rc = expect(b, "outputProjectionWeights", d, o_in, true)) != MLB_OK) return rc;
        if ((rc = expect(b, "rmsGamma2", d, 1, true)) != MLB_OK) return rc;
        if ((rc = expect(b, "feedForwardWeights1A", F, d, true)) != MLB_OK) return rc;
        if ((rc = expect(b, "feedForwardWeights1B", F, d, true)) != MLB_OK) return rc;
        if ((rc = expect(b, "feedForwardWeights2", d, F, true)) != MLB_OK) return rc;
        if (type == MLB_LAYER_ATTENTION) {
            if ((rc = expect(b, "queryRMSGamma", q_out, 1, c.qk_norm != 0)) != MLB_OK) return rc;
            if ((rc = expect(b, "keyRMSGamma", k_out, 1, c.qk_norm != 0)) != MLB_OK) return rc;
            if ((rc = expect(b, "gatedQueryWeights", q_out, d, c.query_gating != 0)) != MLB_OK) return rc;
        } else {
            if ((rc = expect(b, "betaWeights", c.heads, d, true)) != MLB_OK) return rc;
            if ((rc = expect(b, "decayWeights", c.heads, d, true)) != MLB_OK) return rc;
        }
        if (c.ple_dim > 0) {
            if ((rc = expect(b, "pleTable", c.vocab, c.ple_dim, true)) != MLB_OK) return rc;
            if ((rc = expect(b, "pleProjection", d, c.ple_dim, true)) != MLB_OK) return rc;
        }
    }
    return MLB_OK;
}

}  // namespace mlb

extern "C" void mlb_config_init(mlb_config* cfg) {
    if (!cfg) return;
    std::memset(cfg, 0, sizeof(*cfg));
    cfg->dim = cfg->layers = cfg->heads = cfg->kv_heads = cfg->head_dim = cfg->ffn_dim = -1;
    cfg->vocab = cfg->max_context = cfg->ple_dim = cfg->qk_norm = cfg->query_gating = -1;
    cfg->dn_key_dim = cfg->dn_value_dim = -1;
    cfg->weight_dtype = cfg->kv_dtype = 0;
    cfg->layer_types_set = 0;
    cfg->rope_theta = std::nanf("");
    cfg->rms_eps = std::nanf("");
}
