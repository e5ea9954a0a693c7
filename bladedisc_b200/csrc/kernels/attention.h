// Masked self-attention over packed sequences, fused: softmax(Q K^T * scale) V
// with the scores kept on chip, for the encoder the quantized path runs in
// (head size 64, up to 512 keys per sequence, no causal mask).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace disc_b200 {

constexpr int kAttnHeadDim = 64;
constexpr int kAttnMaxKeys = 512;
constexpr int kAttnRowsPerBlock = 128;

// One entry per work item: `nq` consecutive blocks of 128 query rows of one sequence (one thread block per
// item and head; the keys and values of the sequence are fetched once per item).
struct AttnBlock {
  int32_t tok0;  // first token (row of qkv) of the sequence
  int32_t len;   // tokens of the sequence (1 .. 512)
  int32_t q0;    // first query row of the item inside the sequence (multiple of 128)
  int32_t nq;    // query blocks of the item (0 is read as 1); q0 + 128 * nq covers at most the sequence
};

struct AttentionParams {
  const void* qkv;   // f16 [tokens, 3 * hidden]: q | k | v, head h in columns h * 64 .. of each third
  int64_t tokens;
  int64_t ld_qkv;    // row stride of qkv in elements (>= 3 * hidden, multiple of 8)
  int32_t heads;     // hidden = heads * 64
  const AttnBlock* blocks;  // device array
  int32_t num_blocks;
  float scale;       // multiplies q . k before the softmax
  void* out;         // [tokens, hidden]: int8 (quantized at *out_scale) or f16
  int64_t ld_out;    // row stride of out in elements
  const float* out_scale;  // device scalar; null = f16 output
};

// Launches on `stream`; returns the first error, `err` gets a static description of argument errors.
cudaError_t attention_launch(const AttentionParams& p, cudaStream_t stream, const char** err);

// Reads and clears the status word the kernel sets when one of its bounded waits ran out (0 = ok).
int attention_status_fetch_and_clear();

}  // namespace disc_b200
