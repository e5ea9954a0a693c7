// Bandwidth-bound kernels around the quantized linear: activation quantize /
// dequantize and the row-reduction fusions (LayerNorm, RMSNorm, softmax) that
// the reference compiler emits as generated kLoop / kStitch kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace disc_b200 {

enum ElemType : int { kF32 = 0, kF16 = 1 };

// q = clamp(rne(x / scale + zero_point), qmin, qmax) -> int8.
// scale / zero_point: one value (per-tensor) or `channels` values applied along
// an axis of a tensor viewed as [outer, channels, inner].  zero_point may be null (0).
struct QuantizeParams {
  const void* x;
  int8_t* q;
  int64_t numel;
  int in_type;  // ElemType
  const float* scale;
  const int32_t* zero_point;
  int64_t channels;  // 1 = per-tensor
  int64_t inner;     // elements between consecutive channels (1 = last axis)
  int qmin, qmax;
};
cudaError_t quantize_launch(const QuantizeParams& p, cudaStream_t s, const char** err);

// y = float(q - zero_point) * scale -> f32 / f16.
struct DequantizeParams {
  const int8_t* q;
  void* y;
  int64_t numel;
  int out_type;
  const float* scale;
  const int32_t* zero_point;
  int64_t channels;
  int64_t inner;
};
cudaError_t dequantize_launch(const DequantizeParams& p, cudaStream_t s, const char** err);

// Per-row (per-token) symmetric quantize: scale[r] = max(max|x[r,:]| / 127, eps),
// q = clamp(rne(x / scale[r]), -128, 127).  The row stays in registers between
// the reduction and the write.
struct DynQuantParams {
  const void* x;
  int8_t* q;
  float* row_scale;
  int64_t rows, cols;
  int in_type;
};
cudaError_t dynamic_quantize_launch(const DynQuantParams& p, cudaStream_t s, const char** err);

// y = LayerNorm(x [+ residual]) * gamma + beta over the last axis.
// Optional second output: int8 copy quantized with a static per-tensor scale
// (feeds the next quantized linear without another pass over y).
// rms != 0 selects RMSNorm (no mean subtraction, beta ignored).
// sum_out (optional) receives x + residual (the updated residual stream).
// q_row_scale (optional, with q_out and no q_scale): per-row dynamic quantize of y.
struct NormParams {
  const void* x;
  const void* residual;
  const void* gamma;
  const void* beta;
  void* y;        // may be null when only the quantized output is wanted
  void* sum_out;  // may be null
  int8_t* q_out;  // may be null
  const float* q_scale;
  float* q_row_scale;
  int64_t rows, cols;
  float eps;
  int type;  // ElemType of x / residual / gamma / beta / y
  int rms;
  // x stored as column slabs, the layout an all-gather of column-parallel
  // outputs leaves: element (r, c) at x[(c / x_slab_cols) * x_slab_stride +
  // r * x_slab_cols + c % x_slab_cols].  0 = plain row-major.  Needs 16-byte
  // aligned rows and x_slab_cols a multiple of the 16-byte vector.
  int64_t x_slab_cols;
  int64_t x_slab_stride;
};
cudaError_t norm_launch(const NormParams& p, cudaStream_t s, const char** err);

// Per-row symmetric quantization of h = up ? silu(gate) * up : gate in two
// passes, for rows whose columns are spread over several GPUs: pass 0 writes
// row_scale[r] = max(max|h[r, :]| / 127, eps) of the local columns, the caller
// takes the maximum over the GPUs, pass 1 writes q = sat(rne(h / row_scale[r])).
// Both passes compute h with the same instructions, so the scale always covers
// the values that are quantized.  gate / up are [rows, cols] with row stride ld
// (two column halves of one buffer when a merged gate-up linear produced them),
// q has row stride ldq.
struct GatedQuantParams {
  const void* gate;
  const void* up;  // may be null
  int64_t ld;
  int8_t* q;  // pass 1
  int64_t ldq;
  float* row_scale;
  int64_t rows, cols;
  int type;  // ElemType of gate / up
  int pass;  // 0, 1, or 2 = both at once (rows that are whole on this GPU)
};
cudaError_t gated_quantize_launch(const GatedQuantParams& p, cudaStream_t s, const char** err);

// y = softmax(x * scale + mask) over the last axis.  Row r belongs to batch
// r / rows_per_batch; `lens` (optional) gives the valid length per batch
// (columns >= len get probability 0), `mask` (optional, [batches, cols], same
// type as x) is added before the max.
struct SoftmaxParams {
  const void* x;
  void* y;
  int64_t rows, cols;
  int64_t rows_per_batch;
  const int32_t* lens;
  const void* mask;
  float scale;
  int type;
  int log_softmax;
};
cudaError_t softmax_launch(const SoftmaxParams& p, cudaStream_t s, const char** err);

// Rotary position embedding of q and k inside the fused QKV output, and the
// append of k and v to the cache, in one pass (decoder glue around the
// quantized linears; elementwise, one read and one write per element).
//   qkv      fp16 [batch * seq, 3, heads, dim]: q is rotated in place
//   k_cache, v_cache fp16 [batch, heads, cache_len, dim]: positions pos0 .. pos0 + seq - 1 are written
//   cos, sin fp32 [>= pos0 + seq, dim / 2]
// Pairs (i, i + dim / 2) are rotated: out1 = x1 * cos - x2 * sin, out2 = x2 * cos + x1 * sin,
// every product and sum rounded to fp32 separately (as an unfused elementwise graph computes them).
// dim must be a multiple of 16.
struct RopeParams {
  void* qkv;
  void* k_cache;
  void* v_cache;
  const float* cos;
  const float* sin;
  int64_t batch, seq, heads, dim;
  int64_t pos0, cache_len;
};
cudaError_t rope_kv_append_launch(const RopeParams& p, cudaStream_t s, const char** err);

// Status word of the row kernels' bounded waits (0 = none ran out); cleared by
// the read.  The caller has synchronised the device.
int rowops_status_fetch_and_clear();

}  // namespace disc_b200
