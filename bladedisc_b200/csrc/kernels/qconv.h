// Quantized 2-D convolution, int8 x int8 -> int8:
//   out[n, o, y, x] = sat_s8(rne( acc * (s_x * s_w(o) / s_out) )),
//   acc = sum over (ky, kx, c) of in[n, c, y*sh - pt + ky*dh, x*sw - pl + kx*dw] * w[o, c, ky, kx]
// with zero outside the input (symmetric quantization: zero points are 0).
//
// Reference: ral_qconv on "gpu" (cuDNN int8 forward convolution with
// scale = s_in * s_w / s_out, tao_compiler/mlir/ral/context/stream_executor_based_impl.cc:1832-1950)
// and ral_pdll_qconv2d (per-channel weight scales,
// tao_compiler/mlir/ral/context/common_context_impl_quantization.cc:363-607).
//
// Here the product with its requantizing epilogue is the quantized linear of qgemm.h
// (tcgen05 int8 tensor-core path) over [batch * out_h * out_w, k_h * k_w * in_ch]:
//   * channels-last input, in_ch a multiple of 64, kernel already [out, y, x, in]:
//     implicit GEMM, the linear's producer fetches 128 positions x 128 (or 64) channels per
//     K block from the image with TMA in im2col mode (padding and strides live in the
//     tensor map, positions outside the image read as zero);
//   * 1 x 1 window, unit strides, no padding, dense channels-last input: the input is
//     the matrix;
//   * otherwise the receptive fields are gathered into a row-major int8 matrix (K
//     padded to 16) and the kernel is used as, or packed into, [out_ch, the same K].
// Channels-last output is written by the GEMM itself; other layouts through a
// scatter pass.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace disc_b200 {

// A 2-D convolution in logical terms: sizes and element strides of every operand
// by role (batch / channel / y / x), whatever the memory layout.
struct ConvGeometry {
  int64_t batch = 0, in_ch = 0, in_h = 0, in_w = 0;
  int64_t out_ch = 0, k_h = 0, k_w = 0, out_h = 0, out_w = 0;
  int64_t x_stride[4] = {0, 0, 0, 0};  // input:  batch, channel, y, x
  int64_t w_stride[4] = {0, 0, 0, 0};  // kernel: out feature, in feature, y, x
  int64_t o_stride[4] = {0, 0, 0, 0};  // output: batch, channel, y, x
  int64_t stride_h = 1, stride_w = 1, dil_h = 1, dil_w = 1;
  int64_t pad_top = 0, pad_bottom = 0, pad_left = 0, pad_right = 0;
};

struct QConvParams {
  ConvGeometry g;
  const int8_t* x;
  const int8_t* w;
  int8_t* out;
  const float* x_scale;    // device, one value
  const float* w_scale;    // device, one value or out_ch values
  int w_scale_per_channel;
  const float* out_scale;  // device, one value
  void* workspace;         // device, at least qconv_workspace_bytes(g)
  int64_t workspace_bytes;
  int32_t* splitk_ws;      // scratch of the few-row quantized linear (see qgemm.h)
  int64_t splitk_ws_bytes;
};

int64_t qconv_workspace_bytes(const ConvGeometry& g);
cudaError_t qconv_launch(const QConvParams& p, cudaStream_t stream, const char** err);

}  // namespace disc_b200
