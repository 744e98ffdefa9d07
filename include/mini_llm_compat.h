/*
 * mini_llm_compat.h - the reference's own entry points for the decode path, kept with their
 * signatures, C++ linkage and return conventions, implemented on top of the C ABI in mlb.h.
 * A program written against the reference's headers for this path (a `main` that calls
 * allocateMemory / loadModel / loadVocab / runInferenceLoop) links against
 * libmini_llm_b200.so instead of the reference's objects.
 *
 * What differs, because the reference fixes it at compile time (network_meta.h:3-20):
 * dims come from the model file; heads / head_dim for files without a "config" key, and the
 * device, are given once through mlb_compat_configure() before loadModel().
 */
#ifndef MINI_LLM_COMPAT_H_
#define MINI_LLM_COMPAT_H_

#include "mlb.h"

/* inference_orchestrator.h:4-7 */
typedef struct {
    int tokenIdx;
    float prob;
} TokenProb;

/* inference_orchestrator.h:17-18 - returns 0 on success, non-zero on failure. */
int runInferenceLoop(const char* storiesPath, int storyIndex, int contextPercent,
                     bool skipUserInput, bool verboseOutput);
/* inference.h:3 - forward for positions 0..L-1 of seqTokenIndices; always returns 0 in the
 * reference, here non-zero on a failed launch. Afterwards the probabilities of column L-1
 * (the only column the loop reads, inference_orchestrator.cu:74) are available through
 * mlb_compat_last_probs(). Only the tokens not yet in the KV cache are run. */
int runInference(int L);
/* inference.h:4 - host table [maxL_][headDim] of interleaved (cos, sin). */
void getPreComputedRopeTheta(float* preComputedRopeTheta, int maxL_);
/* load_model.h:3-6 - 1 on success, 0 on failure. loadModel reads ./model/<modelName>.bin. */
int loadVocab(const char* vocabPath);
const char* vocabGetToken(int index);
int vocabLookup(const char* token);
int loadModel(const char* modelName);
/* memory_allocation.h:5 */
void allocateMemory(bool allocateTraining);
/* main.cu:45 - returns the number of context tokens loaded (0 on failure). */
int loadStoryContext(const char* storiesPath, int storyIndex, int percentage);

/* network_globals.h:147 - host token ids, capacity max context + 1. */
extern int* seqTokenIndices;

extern "C" {
/* Runtime stand-in for the compile-time configuration; all arguments optional (NULL / <0). */
int mlb_compat_configure(const mlb_config* override_or_null, int device);
/* Same entry points with C linkage for FFI callers (ctypes, cgo, JNI). */
int mlb_compat_load_model(const char* modelName);
int mlb_compat_load_model_path(const char* path);
int mlb_compat_load_vocab(const char* vocabPath);
int mlb_compat_vocab_lookup(const char* token);
const char* mlb_compat_vocab_token(int index);
int mlb_compat_load_story_context(const char* storiesPath, int storyIndex, int percentage);
int mlb_compat_run_inference(int L);
int mlb_compat_run_inference_loop(const char* storiesPath, int storyIndex, int contextPercent,
                                  int skipUserInput, int verboseOutput);
/* Additions to the reference's loop, which ends only at maxL and prints the text once at the end
 * (inference_orchestrator.cu:64, :168-183). Stop token: by vocabulary string (after loadVocab) or by id
 * (token_or_null == NULL; -1 clears it); runInferenceLoop then also ends when that token is generated (it is
 * kept in the sequence). Streaming: each generated token is printed as soon as it exists. Both default off. */
int mlb_compat_set_stop_token(const char* token_or_null, int token_id);
void mlb_compat_set_streaming(int on);
int mlb_compat_max_context(void);
int mlb_compat_vocab_size(void);
int* mlb_compat_tokens(void);                 /* == seqTokenIndices */
int mlb_compat_set_tokens(const int* ids, int n);
/* Probabilities of the last runInference column, [vocab] floats, host memory owned by the library. */
const float* mlb_compat_last_probs(void);
double mlb_compat_last_loop_ms(void);         /* wall time of the last generation loop */
void mlb_compat_shutdown(void);
}

#endif /* MINI_LLM_COMPAT_H_ */
