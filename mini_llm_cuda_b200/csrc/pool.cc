// Several GPUs of one box behind one handle: sequences are sharded over the devices in contiguous
// blocks, each device has a full weight replica, one mlb_session for its block, one stream and one
// host thread per call. Decode has no dependency between sequences, so the token path has no
// collective and no device-to-device traffic; the host only splits the inputs and joins the ids.
// The reference runs on device 0 only (memory_allocation.cu:329 allocates there, no cudaSetDevice
// anywhere); its runInferenceLoop is the batch-1, one-device case of this.
// Host-only C++ on the C ABI of mlb.h.
#include <algorithm>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../../include/mlb.h"
#include "errors.h"

using mlb::fail;

struct mlb_pool {
    struct Shard {
        int device = 0, begin = 0, end = 0;      // sequences [begin, end) of the pool
        mlb_model* model = nullptr;
        mlb_session* session = nullptr;
    };
    std::vector<Shard> shards;
    int batch = 0;
};

extern "C" int mlb_shard_range(int n_items, int n_shards, int shard, int* begin, int* end) {
    if (!begin || !end || n_shards < 1 || shard < 0 || shard >= n_shards || n_items < 0) return fail(MLB_E_INVALID, "bad shard arguments");
    const int base = n_items / n_shards, extra = n_items % n_shards;
    *begin = shard * base + std::min(shard, extra);              // the first n_items % n_shards shards hold one more
    *end = *begin + base + (shard < extra ? 1 : 0);
    return MLB_OK;
}

namespace {

// Runs fn(shard index) on one thread per shard that has sequences; the first failure wins.
template <typename Fn>
int for_each_shard(mlb_pool* p, Fn fn) {
    const size_t n = p->shards.size();
    std::vector<int> rcs(n, MLB_OK);
    std::vector<std::string> msgs(n);
    std::vector<std::thread> threads;
    auto body = [&](size_t i) {
        rcs[i] = fn((int)i);
        if (rcs[i] != MLB_OK) msgs[i] = mlb_last_error();        // the message is per thread: carry it over
    };
    for (size_t i = 1; i < n; ++i)
        if (p->shards[i].end > p->shards[i].begin) threads.emplace_back(body, i);
    if (p->shards[0].end > p->shards[0].begin) body(0);          // the caller's thread serves the first shard
    for (auto& t : threads) t.join();
    for (size_t i = 0; i < n; ++i)
        if (rcs[i] != MLB_OK) return fail(rcs[i], "device %d: %s", p->shards[i].device, msgs[i].c_str());
    return MLB_OK;
}

}  // namespace

extern "C" void mlb_pool_free(mlb_pool* p) {
    if (!p) return;
    for (auto& s : p->shards) {
        if (s.session) mlb_session_free(s.session);
        if (s.model) mlb_model_free(s.model);
    }
    delete p;
}

extern "C" int mlb_pool_new(const char* model_path, const int* devices, int n_devices, int batch, int max_context,
                            const mlb_config* override_or_null, mlb_pool** out) {
    if (!model_path || !devices || !out) return fail(MLB_E_INVALID, "null argument");
    if (n_devices < 1 || n_devices > 64) return fail(MLB_E_INVALID, "1..64 devices, %d given", n_devices);
    if (batch < 1) return fail(MLB_E_INVALID, "batch must be >= 1");
    for (int i = 0; i < n_devices; ++i)
        if (devices[i] < 0) return fail(MLB_E_INVALID, "device index %d", devices[i]);
    mlb_pool* p = new mlb_pool();
    p->batch = batch;
    p->shards.resize(n_devices);
    for (int i = 0; i < n_devices; ++i) {
        p->shards[i].device = devices[i];
        mlb_shard_range(batch, n_devices, i, &p->shards[i].begin, &p->shards[i].end);
    }
    const int rc = for_each_shard(p, [&](int i) -> int {
        mlb_pool::Shard& s = p->shards[i];
        int r = mlb_model_load(model_path, s.device, override_or_null, &s.model);
        if (r != MLB_OK) return r;
        return mlb_session_new(s.model, s.end - s.begin, max_context, 16, 0, &s.session);
    });
    if (rc != MLB_OK) {
        const std::string msg = mlb_last_error();
        mlb_pool_free(p);
        return fail(rc, "%s", msg.c_str());
    }
    *out = p;
    return MLB_OK;
}

extern "C" int mlb_pool_shards(const mlb_pool* p, int* devices, int* begins, int* ends, int cap) {
    if (!p) return fail(MLB_E_INVALID, "null pool");
    const int n = (int)p->shards.size();
    for (int i = 0; i < n && i < cap; ++i) {
        if (devices) devices[i] = p->shards[i].device;
        if (begins) begins[i] = p->shards[i].begin;
        if (ends) ends[i] = p->shards[i].end;
    }
    return n;
}

extern "C" int mlb_pool_set_stop_token(mlb_pool* p, int token_id) {
    if (!p) return fail(MLB_E_INVALID, "null pool");
    return for_each_shard(p, [&](int i) { return mlb_session_set_stop_token(p->shards[i].session, token_id); });
}

extern "C" int mlb_pool_prefill(mlb_pool* p, const int32_t* tokens, const int32_t* lens, int stride) {
    if (!p || !tokens || !lens) return fail(MLB_E_INVALID, "null argument");
    return for_each_shard(p, [&](int i) {
        const mlb_pool::Shard& s = p->shards[i];
        return mlb_prefill(s.session, tokens + (size_t)s.begin * stride, lens + s.begin, stride);
    });
}

extern "C" int mlb_pool_decode_n(mlb_pool* p, const mlb_sampling* sampling, int n, int32_t* out_tokens) {
    if (!p || !out_tokens) return fail(MLB_E_INVALID, "null argument");
    if (n < 1) return fail(MLB_E_INVALID, "n must be >= 1");
    // Philox keys default to the sequence index within a session: give every shard the pool-wide indices, so
    // that a draw does not depend on how many devices serve the batch
    std::vector<uint64_t> keys;
    if (sampling && sampling->mode != 0 && !sampling->seeds) {
        keys.resize(p->batch);
        for (int b = 0; b < p->batch; ++b) keys[b] = (uint64_t)b;
    }
    return for_each_shard(p, [&](int i) {
        const mlb_pool::Shard& s = p->shards[i];
        mlb_sampling local;
        const mlb_sampling* sp = nullptr;
        if (sampling) {
            local = *sampling;
            const uint64_t* seeds = sampling->seeds ? sampling->seeds : (keys.empty() ? nullptr : keys.data());
            local.seeds = seeds ? seeds + s.begin : nullptr;
            sp = &local;
        }
        // the rows of a shard are consecutive in out_tokens [batch][n]
        return mlb_decode_n(s.session, sp, n, out_tokens + (size_t)s.begin * n);
    });
}
