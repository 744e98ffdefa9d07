// TEST / BASELINE INFRASTRUCTURE - driver `main` for the UNMODIFIED reference sources.
//
// The reference's own main.cu runs the training loop (main.cu:223) and keeps the inference
// call commented out (main.cu:215). This file replaces main.cu only: it provides `main` and
// `loadStoryContext` (which main.cu defines and inference_orchestrator.cu:26 declares extern)
// and then calls the reference's allocateMemory, loadModel and runInferenceLoop as they are.
// build_ref.py compiles it together with the reference's .cu files (taken from the reference
// checkout where they lie, with network_meta.h regenerated for the wanted dims).
//
// usage: ref_decode <modelName> <prompt.i32> <out_prefix> <tf32: 0|1> [col ...]
//   ./model/<modelName>.bin must exist relative to the working directory.
//   prompt.i32: little-endian int32 token ids. The loop generates until maxL.
//   writes <out_prefix>.tokens.i32 (maxL ids) and <out_prefix>.logits.f32 (the requested
//   columns of vocabScores_DEVICE after the last forward, each vocabSize floats) and prints
//   one line `REF_RESULT prompt=<n> generated=<n> loop_ms=<chrono ms of runInferenceLoop>`.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include <cuda_runtime.h>
#include <cublas_v2.h>

#include "network_meta.h"
#include "network_globals.h"
#include "load_model.h"
#include "inference.h"
#include "inference_orchestrator.h"
#include "memory_allocation.h"

static std::vector<int> g_prompt;

// Same contract as main.cu:45-175: fill seqTokenIndices (+ device copy), return the count.
int loadStoryContext(const char* /*storiesPath*/, int /*storyIndex*/, int /*percentage*/) {
    int n = (int)g_prompt.size();
    if (n > maxL + 1) n = maxL + 1;
    for (int i = 0; i < n; ++i) seqTokenIndices[i] = g_prompt[i];
    cudaMemcpy(seqTokenIndices_DEVICE, seqTokenIndices, n * sizeof(int), cudaMemcpyHostToDevice);
    return n;
}

int main(int argc, char** argv) {
    if (argc < 5) {
        fprintf(stderr, "usage: %s modelName prompt.i32 out_prefix tf32 [col ...]\n", argv[0]);
        return 2;
    }
    FILE* f = fopen(argv[2], "rb");
    if (!f) { fprintf(stderr, "cannot open %s\n", argv[2]); return 2; }
    int v;
    while (fread(&v, 4, 1, f) == 1) g_prompt.push_back(v);
    fclose(f);
    for (int t : g_prompt) if (t < 0 || t >= vocabSize) { fprintf(stderr, "token out of range\n"); return 2; }

    cublasCreate(&handle);                                       // main.cu:178
    if (atoi(argv[4])) cublasSetMathMode(handle, CUBLAS_TF32_TENSOR_OP_MATH);   // main.cu:179
    allocateMemory(false);
    if (!loadModel(argv[1])) return 3;
    if (cudaDeviceSynchronize() != cudaSuccess) { fprintf(stderr, "CUDA error after load\n"); return 4; }

    auto t0 = std::chrono::high_resolution_clock::now();
    int rc = runInferenceLoop("", 0, 100, /*skipUserInput=*/true, /*verboseOutput=*/false);
    cudaError_t ce = cudaDeviceSynchronize();
    auto t1 = std::chrono::high_resolution_clock::now();
    if (rc != 0 || ce != cudaSuccess) { fprintf(stderr, "reference loop failed rc=%d cuda=%s\n", rc, cudaGetErrorString(ce)); return 5; }
    double ms = std::chrono::duration<double>(t1 - t0).count() * 1000.0;

    char path[1024];
    snprintf(path, sizeof path, "%s.tokens.i32", argv[3]);
    f = fopen(path, "wb");
    fwrite(seqTokenIndices, 4, maxL, f);
    fclose(f);
    // The last forward ran over maxL-1 tokens: column c holds the logits after c+1 tokens.
    snprintf(path, sizeof path, "%s.logits.f32", argv[3]);
    f = fopen(path, "wb");
    std::vector<float> col(vocabSize);
    for (int i = 5; i < argc; ++i) {
        int c = atoi(argv[i]);
        if (c < 0 || c > maxL - 2) { fprintf(stderr, "column %d out of range\n", c); return 2; }
        cudaMemcpy(col.data(), vocabScores_DEVICE + (size_t)c * vocabSize, sizeof(float) * vocabSize, cudaMemcpyDeviceToHost);
        fwrite(col.data(), 4, vocabSize, f);
    }
    fclose(f);
    int prompt_n = (int)g_prompt.size() > maxL + 1 ? maxL + 1 : (int)g_prompt.size();
    printf("REF_RESULT prompt=%d generated=%d loop_ms=%f\n", prompt_n, maxL - prompt_n, ms);
    return 0;
}
