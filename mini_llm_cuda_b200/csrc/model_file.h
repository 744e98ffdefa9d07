// Host-side parser of the model.bin container (layout read by load_model.cu:286-481 and
// pytorch_verification/load_model_weights.py:135-351). Produces a list of tensor
// descriptors with byte offsets; the device upload lives in engine.cu.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/mlb.h"

namespace mlb {

// FD_FP8: e4m3 codes [rows][cols] followed by one float32 scale per row (value = code * scale[row]); written
// by the offline converter for the matrices a float8_e4m3 model keeps in that form on the device. The
// reference's loader knows float32, float64 and bfloat16 only (load_model.cu:24-61).
enum FileDtype { FD_F32 = 0, FD_F64 = 1, FD_BF16 = 2, FD_FP8 = 3 };

struct TensorDesc {
    std::string name;      // JSON key, e.g. "queryWeights"
    int block = -1;        // file block index, -1 for the two global tensors
    int rows = 0, cols = 0;  // 1-D tensors: rows = length, cols = 1
    int ndim = 0;
    FileDtype dtype = FD_F32;
    uint64_t offset = 0;   // byte offset in the file
    uint64_t nbytes = 0;
};

struct ParsedModel {
    mlb_config cfg;
    std::vector<TensorDesc> tensors;
    uint64_t n_params = 0;
    uint64_t file_size = 0;
    const TensorDesc* find(int block, const char* name) const;
};

// Fills `out` from the header of `data` (whole file or at least header; `file_size` is the
// real size used for bounds checks). Returns an mlb_status; message in *err.
int parse_model_header(const unsigned char* data, uint64_t avail, uint64_t file_size,
                       const mlb_config* override_cfg, ParsedModel* out, std::string* err);

// Reads the whole file into memory. Returns an mlb_status.
int read_file(const char* path, std::vector<unsigned char>* out, std::string* err);

// Converts `n` elements at `src` of the given file dtype to float32 (FD_FP8: rows of `cols` codes, the scales
// behind them).
void convert_to_f32(const unsigned char* src, FileDtype dt, uint64_t n, float* dst, uint64_t cols = 0);
// Value of one e4m3 code (no infinities; 0x7f / 0xff are NaN).
float e4m3_to_f32(unsigned char code);

}  // namespace mlb
