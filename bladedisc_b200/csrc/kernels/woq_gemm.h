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
// produces: a warp reads whole row segments, which is already the best HBM pattern.
// Needs no scratch memory: partial sums are exchanged inside thread-block clusters.
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
  int path = 0;         // 0 = chosen by shape, 1 = streaming kernel, 2 = tensor cores (f16 only)
};

constexpr int kWoqPathAuto = 0, kWoqPathStream = 1, kWoqPathTensor = 2;
// Rows from which the tensor-core kernel is chosen when `path` is 0.
constexpr int kWoqTensorMinRows = 5;

// The weights are constants of the model: the kernel may start reading them before
// the kernel launched ahead of it on the stream has finished.
// How a problem would be launched on a GPU of `sm_count` SMs with weights aligned to
// `align` (4, 8 or 16) bytes: {rows per pass, padded rows, bytes per lane and load, strips
// along N, cluster size along K, k rows per block, dynamic shared memory}.  Host only.
// 0 = ok, 1 = bad argument, 2 = K too large for shared memory.
int woq_gemm_plan_describe(int64_t m, int64_t n, int64_t k, int align, int sm_count, int64_t out7[7]);

cudaError_t woq_gemm_launch(const WoqGemmParams& p, cudaStream_t s, const char** err);

// The tensor-core kernel (woq_gemm_tc.cu): fp16 activations, N a multiple of 16, weights and
// activations 16-byte aligned with row pitches to match; zero points within [-1024, 1024].
bool woq_gemm_tc_usable(const WoqGemmParams& p);
cudaError_t woq_gemm_tc_launch(const WoqGemmParams& p, cudaStream_t s, const char** err);
// Reads and clears the status word the kernel sets when one of its bounded waits ran out (0 = ok).
int woq_tc_status_fetch_and_clear();

}  // namespace disc_b200
