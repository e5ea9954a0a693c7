// Weight-only quantized linear: floating-point activations times uint8 weights
// that are dequantized inside the kernel,
//   out[m, n] = sum_k x[m, k] * (w[k, n] - zp[n]) * scale[n] + bias[n].
// The decode-time path of a weight-only quantized model: a few rows of
// activations, the whole weight matrix streamed once from HBM.
//
// Reference: custom call ral_pdll_weight_only_qgemm, emitted by
// pytorch_blade/tests/disc/pdl/pdll_files/gpu/weight_only_qgemm.pdll:2-106 with
// operands (input, weight transposed to [K, N], [bias,] weight_scale,
// weight_zero_point).  The reference ships no open kernel for it; its compiler
// pre-permutes the weights for a closed sm_75/80 kernel
// (tao_compiler/mlir/disc/transforms/disc_transform_weight_data_layout_for_weight_only_gemm.cc:36-110).
// Here the weights stay in the plain [K, N] row-major layout the pattern
// produces: a warp reads whole rows, which is already the best HBM pattern.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace disc_b200 {

struct WoqGemmParams {
  const void* x;        // [M, K], row stride ldx (elements); f16 or f32 (`type`)
  const uint8_t* w;     // [K, N] row-major, row stride ldw (bytes)
  const void* scale;    // [N], same type as x
  const int32_t* zp;    // [N]; null = 0
  const void* bias;     // [N], same type as x; null = none
  void* out;            // [M, N], row stride ldo, same type as x
  int64_t M, N, K;
  int64_t ldx, ldw, ldo;
  int type;             // ElemType of rowops.h: 0 = f32, 1 = f16
  // Device scratch of at least woq_gemm_scratch_bytes(M, N, K) bytes.  Its first
  // 16 KiB are arrival counters: zero before the first use, left zero; launches
  // that share it must not overlap on the GPU.
  void* ws;
  int64_t ws_bytes;
};

int64_t woq_gemm_scratch_bytes(int64_t M, int64_t N, int64_t K);
cudaError_t woq_gemm_launch(const WoqGemmParams& p, cudaStream_t s, const char** err);

}  // namespace disc_b200
