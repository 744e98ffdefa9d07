// The reference's decode-path entry points (inference_orchestrator.h:17-18, inference.h:3-4,
// load_model.h:3-6, memory_allocation.h:5, loadStoryContext of main.cu:45) implemented on the
// C ABI of mlb.h. Host-only C++; every device operation goes through mlb_* calls.
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/mini_llm_compat.h"
#include "json_min.h"
#include "model_file.h"

int* seqTokenIndices = nullptr;

namespace {

struct CompatState {
    mlb_config override_cfg;
    bool has_override = false;
    int device = 0;
    mlb_model* model = nullptr;
    mlb_session* session = nullptr;
    int max_context = 0, vocab = 0;
    int token_capacity = 0;
    std::vector<int> cached;                 // tokens whose K/V (or state) the session holds
    std::vector<float> probs;
    std::vector<std::string> vocab_tokens;
    std::vector<char> vocab_present;
    std::unordered_map<std::string, int> vocab_index;
    double last_loop_ms = 0.0;
    int pending_pick = -1;                   // device pick of the last runInference
    int stop_token = -1;                     // generation also ends when this id is picked (-1: only at maxL)
    bool streaming = false;                  // print each generated token as it arrives
};

CompatState& st() {
    static CompatState s;
    static bool init = false;
    if (!init) { mlb_config_init(&s.override_cfg); init = true; }
    return s;
}

void ensure_token_capacity(int n) {
    CompatState& s = st();
    if (n <= s.token_capacity && seqTokenIndices) return;
    int* fresh = static_cast<int*>(std::calloc(static_cast<size_t>(n), sizeof(int)));
    if (seqTokenIndices && s.token_capacity > 0) std::memcpy(fresh, seqTokenIndices, sizeof(int) * static_cast<size_t>(s.token_capacity));
    std::free(seqTokenIndices);
    seqTokenIndices = fresh;
    s.token_capacity = n;
}

void print_token(const char* t) {
    if (!t) return;
    if (std::strcmp(t, "\n") == 0) std::printf("[\\n]");
    else if (std::strcmp(t, "\t") == 0) std::printf("[\\t]");
    else std::printf("%s", t);
}

int load_model_path(const char* path) {
    CompatState& s = st();
    if (s.session) { mlb_session_free(s.session); s.session = nullptr; }
    if (s.model) { mlb_model_free(s.model); s.model = nullptr; }
    std::printf("\n--- Loading model weights from %s ---\n", path);
    int rc = mlb_model_load(path, s.device, s.has_override ? &s.override_cfg : nullptr, &s.model);
    if (rc != MLB_OK) {
        std::printf("Error: %s\n", mlb_last_error());
        return 0;
    }
    mlb_config c;
    mlb_model_get_config(s.model, &c);
    rc = mlb_session_new(s.model, 1, c.max_context, 16, 0, &s.session);
    if (rc != MLB_OK) {
        std::printf("Error: %s\n", mlb_last_error());
        mlb_model_free(s.model);
        s.model = nullptr;
        return 0;
    }
    s.max_context = c.max_context;
    s.vocab = c.vocab;
    if (s.stop_token >= c.vocab) s.stop_token = -1;
    s.cached.clear();
    s.probs.assign(static_cast<size_t>(c.vocab), 0.f);
    ensure_token_capacity(c.max_context + 1);
    std::printf("--- Model loaded: dim %d, %d layers, vocab %d, max context %d ---\n\n", c.dim, c.layers, c.vocab, c.max_context);
    return 1;
}

}  // namespace

extern "C" int mlb_compat_configure(const mlb_config* ov, int device) {
    CompatState& s = st();
    if (ov) { s.override_cfg = *ov; s.has_override = true; }
    if (device >= 0) s.device = device;
    return MLB_OK;
}

void allocateMemory(bool /*allocateTraining*/) {
    // The reference allocates every buffer at maxL capacity here (memory_allocation.cu:326-557).
    // Device buffers of this path are sized from the model file in loadModel; only the host
    // token array exists before that.
    CompatState& s = st();
    int cap = s.has_override && s.override_cfg.max_context > 0 ? s.override_cfg.max_context + 1 : 65537;
    ensure_token_capacity(cap);
}

int loadModel(const char* modelName) {
    char filepath[1024];
    std::snprintf(filepath, sizeof filepath, "./model/%s.bin", modelName);      // load_model.cu:288
    return load_model_path(filepath);
}

int loadVocab(const char* vocabPath) {
    CompatState& s = st();
    std::printf("--- Loading vocabulary from %s ---\n", vocabPath);
    std::vector<unsigned char> buf;
    std::string err;
    if (mlb::read_file(vocabPath, &buf, &err) != MLB_OK) {
        std::printf("Error: Vocabulary file not found at '%s'\n", vocabPath);
        return 0;
    }
    mlb::JsonValue root;
    mlb::JsonParser parser(reinterpret_cast<const char*>(buf.data()), buf.size());
    if (!parser.parse(&root)) {
        std::printf("Error: Failed to parse vocabulary JSON (%s).\n", parser.error().c_str());
        return 0;
    }
    if (!root.is(mlb::JsonValue::Array)) {
        std::printf("Error: Vocabulary JSON is not an array.\n");
        return 0;
    }
    const int n = static_cast<int>(root.items.size());
    if (s.vocab > 0 && n != s.vocab)
        std::printf("Warning: Vocabulary size (%d) differs from the model's vocabulary (%d)\n", n, s.vocab);
    const int keep = s.vocab > 0 ? s.vocab : n;      // the reference keeps vocabSize slots (load_model.cu:243-263)
    s.vocab_tokens.assign(static_cast<size_t>(keep), std::string());
    s.vocab_present.assign(static_cast<size_t>(keep), 0);
    s.vocab_index.clear();
    int loaded = 0;
    for (int i = 0; i < n && i < keep; ++i) {
        if (!root.items[i].is(mlb::JsonValue::String)) continue;
        s.vocab_tokens[i] = root.items[i].str;
        s.vocab_present[i] = 1;
        s.vocab_index[root.items[i].str] = i;        // a later duplicate wins, as chaining at the front does (load_model.cu:165-173)
        ++loaded;
    }
    std::printf("Loaded %d vocabulary tokens.\n\n", loaded);
    return 1;
}

int vocabLookup(const char* token) {
    CompatState& s = st();
    if (!token) return -1;
    auto it = s.vocab_index.find(token);
    return it == s.vocab_index.end() ? -1 : it->second;
}

const char* vocabGetToken(int index) {
    CompatState& s = st();
    if (index < 0 || index >= static_cast<int>(s.vocab_tokens.size()) || !s.vocab_present[index]) return nullptr;
    return s.vocab_tokens[index].c_str();
}

void getPreComputedRopeTheta(float* table, int maxL_) {
    CompatState& s = st();
    mlb_config c;
    int hd = 64;
    float base = 10000.0f;
    if (s.model && mlb_model_get_config(s.model, &c) == MLB_OK) { hd = c.head_dim; base = c.rope_theta; }
    else if (s.has_override && s.override_cfg.head_dim > 0) hd = s.override_cfg.head_dim;
    mlb_rope_table(table, maxL_, hd, base);
}

int loadStoryContext(const char* storiesPath, int storyIndex, int percentage) {
    CompatState& s = st();
    std::printf("--- Loading story context from %s ---\n", storiesPath);
    std::printf("Story index: %d, Context percentage: %d%%\n", storyIndex, percentage);
    if (s.max_context <= 0) {
        std::printf("Error: load a model before the story context.\n");
        return 0;
    }
    std::vector<unsigned char> buf;
    std::string err;
    if (mlb::read_file(storiesPath, &buf, &err) != MLB_OK) {
        std::printf("Error: Stories file not found at '%s'\n", storiesPath);
        return 0;
    }
    mlb::JsonValue root;
    mlb::JsonParser parser(reinterpret_cast<const char*>(buf.data()), buf.size());
    if (!parser.parse(&root)) { std::printf("Error: Failed to parse stories JSON.\n"); return 0; }
    if (!root.is(mlb::JsonValue::Array)) { std::printf("Error: Stories JSON is not an array.\n"); return 0; }
    const int numStories = static_cast<int>(root.items.size());
    if (storyIndex < 0 || storyIndex >= numStories) {
        std::printf("Error: Story index %d out of range (0-%d).\n", storyIndex, numStories - 1);
        return 0;
    }
    const mlb::JsonValue& story = root.items[storyIndex];
    if (!story.is(mlb::JsonValue::Array)) { std::printf("Error: Story at index %d is not an array.\n", storyIndex); return 0; }
    const int total = static_cast<int>(story.items.size());
    if (total == 0) { std::printf("Error: Story at index %d has no tokens.\n", storyIndex); return 0; }
    int contextLength = (total * percentage) / 100;             // main.cu:114-120
    if (contextLength < 1) contextLength = 1;
    if (contextLength > s.max_context + 1) {
        std::printf("Warning: Context length %d exceeds max capacity (maxL+1=%d), truncating.\n", contextLength, s.max_context + 1);
        contextLength = s.max_context + 1;
    }
    std::printf("Story has %d tokens, using %d tokens as context.\n\n=== Story Context ===\n", total, contextLength);
    ensure_token_capacity(s.max_context + 1);
    for (int i = 0; i < contextLength; ++i) {
        const mlb::JsonValue& item = story.items[i];
        if (!item.is(mlb::JsonValue::String)) { std::printf("\nError: Token at position %d is not a string.\n", i); return 0; }
        int idx = vocabLookup(item.str.c_str());
        if (idx < 0) { std::printf("\nError: Token '%s' not found in vocabulary.\n", item.str.c_str()); return 0; }
        seqTokenIndices[i] = idx;
        print_token(item.str.c_str());
    }
    std::printf("\n=====================\n\n");
    return contextLength;
}

int runInference(int L) {
    CompatState& s = st();
    if (!s.session || L < 1 || L > s.max_context) return 1;
    // longest prefix of seqTokenIndices[0..L-1) already consumed by the session
    size_t keep = 0;
    const size_t want = static_cast<size_t>(L - 1);
    while (keep < s.cached.size() && keep < want && s.cached[keep] == seqTokenIndices[keep]) ++keep;
    if (keep != s.cached.size() || s.cached.size() > want || (s.cached.empty() && want >= 2)) {
        // the cached prefix diverged (or is longer), or nothing is cached yet: ingest the prompt in one call
        int len = L;
        if (mlb_prefill(s.session, seqTokenIndices, &len, s.max_context + 1) != MLB_OK) return 1;
        s.cached.assign(seqTokenIndices, seqTokenIndices + (L - 1));
    }
    int pick = -1;
    while (static_cast<int>(s.cached.size()) < L) {
        int t = seqTokenIndices[s.cached.size()];
        if (mlb_decode_step(s.session, nullptr, &t, &pick) != MLB_OK) return 1;
        s.cached.push_back(t);
    }
    s.pending_pick = pick;
    if (mlb_get_probs_col(s.session, 0, s.probs.data()) != MLB_OK) return 1;
    return 0;
}

int runInferenceLoop(const char* storiesPath, int storyIndex, int contextPercent, bool skipUserInput, bool verboseOutput) {
    CompatState& s = st();
    int L = loadStoryContext(storiesPath, storyIndex, contextPercent);
    if (L <= 0) { std::printf("Failed to load story context.\n"); return 1; }
    const int maxL = s.max_context;
    if (L >= maxL) {
        std::printf("Sequence already at maxL=%d tokens (loaded %d). No generation needed.\n", maxL, L);
        return 0;
    }
    int generated = 0;
    std::printf("\n========================================\n");
    std::printf("Starting text generation (max %d new tokens)\n", maxL - L);
    std::printf("========================================\n\n");
    auto t0 = std::chrono::high_resolution_clock::now();
    if (skipUserInput && !verboseOutput) {
        // No host decision between tokens: ingest the prompt, then let the device run the
        // whole loop (the reference's per-token D2H / qsort / H2D, inference_orchestrator.cu:68-154,
        // is replaced by an on-device argmax and a 4-byte id per token).
        // the device ends the sequence at the stop token only inside this loop: runInference() feeds given tokens
        if (s.stop_token >= 0) mlb_session_set_stop_token(s.session, s.stop_token);
        int len = L;
        if (mlb_prefill(s.session, seqTokenIndices, &len, maxL + 1) != MLB_OK) { std::printf("Error: %s\n", mlb_last_error()); return 1; }
        const int n = maxL - L;
        // Without a stop token and without streaming the whole loop is one call. Otherwise the tokens come a
        // chunk at a time (one per call when streaming, so that each is printed as soon as it exists), and the
        // loop ends where the device took the sequence out of the batch.
        const int chunk = s.streaming ? 1 : (s.stop_token >= 0 ? 64 : n);
        std::vector<int> outv(static_cast<size_t>(chunk));
        bool stopped = false;
        while (L < maxL && !stopped) {
            const int m = std::min(chunk, maxL - L);
            const int rc = m == 1 ? mlb_decode_step(s.session, nullptr, nullptr, outv.data()) : mlb_decode_n(s.session, nullptr, m, outv.data());
            if (rc != MLB_OK) { std::printf("Error: %s\n", mlb_last_error()); return 1; }
            for (int i = 0; i < m; ++i) {
                if (outv[i] < 0) { stopped = true; break; }
                seqTokenIndices[L++] = outv[i];
                ++generated;
                if (s.streaming) { print_token(vocabGetToken(outv[i])); std::fflush(stdout); }
                if (outv[i] == s.stop_token) { stopped = true; break; }
            }
        }
        if (s.streaming) std::printf("\n");
        s.cached.assign(seqTokenIndices, seqTokenIndices + (L - 1));
        if (s.stop_token >= 0) {
            mlb_session_set_stop_token(s.session, -1);
            if (stopped) s.cached.clear();       // the session holds an ended sequence: the next call ingests again
        }
    } else {
        while (L < maxL) {
            if (runInference(L) != 0) { std::printf("Error: %s\n", mlb_last_error()); return 1; }
            int next = s.pending_pick;
            if (verboseOutput) {
                std::vector<TokenProb> tp(static_cast<size_t>(s.vocab));
                for (int i = 0; i < s.vocab; ++i) { tp[i].tokenIdx = i; tp[i].prob = s.probs[i]; }
                const int top = std::min(10, s.vocab);
                std::partial_sort(tp.begin(), tp.begin() + top, tp.end(), [](const TokenProb& a, const TokenProb& b) {
                    return a.prob > b.prob || (a.prob == b.prob && a.tokenIdx < b.tokenIdx);
                });
                std::printf("\n--- Top 10 Most Probable Next Tokens (position %d) ---\n", L);
                for (int i = 0; i < top; ++i) {
                    const char* t = vocabGetToken(tp[i].tokenIdx);
                    std::printf("%2d. ", i + 1);
                    if (t && std::strlen(t) == 0) std::printf("[EMPTY]"); else print_token(t);
                    std::printf(" (idx: %5d, prob: %.6f)\n", tp[i].tokenIdx, tp[i].prob);
                }
                std::printf("-------------------------------------------------------\n");
                std::printf("\nMost probable token: ");
                print_token(vocabGetToken(next));
                std::printf(" (index: %d)\n", next);
            }
            if (!skipUserInput) {
                std::printf("\nPress Enter to add this token and continue, or 'q' + Enter to quit: ");
                std::fflush(stdout);
                char input[10];
                if (std::fgets(input, sizeof input, stdin) == nullptr) break;
                if (input[0] == 'q' || input[0] == 'Q') { std::printf("Generation stopped by user.\n"); break; }
            }
            seqTokenIndices[L] = next;
            ++L;
            ++generated;
            if (s.streaming && !verboseOutput) { print_token(vocabGetToken(next)); std::fflush(stdout); }
            if (next == s.stop_token) { std::printf("\nStop token reached.\n"); break; }
            if (verboseOutput) std::printf("\n[Token added. Total context: %d tokens, generated: %d]\n", L, generated);
        }
    }
    auto t1 = std::chrono::high_resolution_clock::now();
    s.last_loop_ms = std::chrono::duration<double>(t1 - t0).count() * 1000.0;
    std::printf("Generation took %f ms\n", s.last_loop_ms);
    std::printf("\n========================================\n");
    std::printf("Generation complete. Generated %d new tokens.\n", generated);
    std::printf("Final sequence length: %d tokens\n", L);
    std::printf("========================================\n\n=== Final Generated Sequence ===\n");
    for (int i = 0; i < L; ++i) print_token(vocabGetToken(seqTokenIndices[i]));
    std::printf("\n================================\n");
    return 0;
}

extern "C" {
int mlb_compat_load_model(const char* modelName) { return loadModel(modelName); }
int mlb_compat_load_model_path(const char* path) { return load_model_path(path); }
int mlb_compat_load_vocab(const char* vocabPath) { return loadVocab(vocabPath); }
int mlb_compat_vocab_lookup(const char* token) { return vocabLookup(token); }
const char* mlb_compat_vocab_token(int index) { return vocabGetToken(index); }
int mlb_compat_load_story_context(const char* p, int i, int pct) { return loadStoryContext(p, i, pct); }
int mlb_compat_run_inference(int L) { return runInference(L); }
int mlb_compat_run_inference_loop(const char* p, int i, int pct, int skip, int verbose) {
    return runInferenceLoop(p, i, pct, skip != 0, verbose != 0);
}
int mlb_compat_set_stop_token(const char* token_or_null, int token_id) {
    CompatState& s = st();
    if (token_or_null) token_id = vocabLookup(token_or_null);
    if (token_or_null && token_id < 0) return MLB_E_INVALID;
    s.stop_token = token_id < 0 ? -1 : token_id;
    return MLB_OK;
}
void mlb_compat_set_streaming(int on) { st().streaming = on != 0; }
int mlb_compat_max_context(void) { return st().max_context; }
int mlb_compat_vocab_size(void) { return st().vocab; }
int* mlb_compat_tokens(void) { return seqTokenIndices; }
int mlb_compat_set_tokens(const int* ids, int n) {
    if (!ids || n < 0) return MLB_E_INVALID;
    ensure_token_capacity(std::max(n, st().max_context + 1));
    std::memcpy(seqTokenIndices, ids, sizeof(int) * static_cast<size_t>(n));
    return MLB_OK;
}
const float* mlb_compat_last_probs(void) { return st().probs.data(); }
double mlb_compat_last_loop_ms(void) { return st().last_loop_ms; }
void mlb_compat_shutdown(void) {
    CompatState& s = st();
    if (s.session) { mlb_session_free(s.session); s.session = nullptr; }
    if (s.model) { mlb_model_free(s.model); s.model = nullptr; }
    s.cached.clear();
}
}
