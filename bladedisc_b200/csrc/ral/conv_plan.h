// Host-side geometry of a quantized convolution: what the attributes of
// ral_pdll_qconv2d or the metadata of ral_qconv say about layouts, strides,
// dilations and padding, and the result shape that follows.  No device code.
//
// Reference semantics:
//   attributes -> padding / metadata / result shape:
//     tao_compiler/mlir/ral/context/common_context_impl_quantization.h:27-215
//   metadata layout (5 * rank - 4 integers, + 1 "weight is constant" in the
//   attribute form): tao_compiler/mlir/ral/context/stream_executor_based_impl.cc:1127-1152
//     input  : batch dim, channel dim, spatial dims
//     kernel : input-feature dim, output-feature dim, spatial dims
//     output : batch dim, channel dim, spatial dims
//     strides (per spatial dim), dilations (per spatial dim)
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../kernels/qconv.h"

namespace disc_b200 {
namespace ral {

using ::disc_b200::ConvGeometry;

// Attribute form (rank 4).  `data_format` is "NHWC" or "NCHW"; strides / dilations
// have 1, 2 or 4 entries (4: indexed like the data format); padding is "SAME",
// "VALID" or "EXPLICIT" (then explicit_paddings has 4 or 8 entries); the kernel is
// [out, y, x, in].  Outputs: padding (lo, hi per spatial dim), result sizes in the
// data format, metadata in the reference's order (17 entries).  Empty string on
// success, else what is wrong.
std::string plan_conv2d_from_attrs(const std::string& data_format, const std::vector<int64_t>& strides,
                                   const std::vector<int64_t>& dilations, const std::string& padding,
                                   const std::vector<int64_t>& explicit_paddings, bool weight_is_const,
                                   const int64_t input_sizes[4], const int64_t weight_sizes[4],
                                   int32_t padding_out[4], int64_t result_sizes[4], int32_t metadata_out[17]);

// Geometry from operand shapes (dense row-major operands), padding and metadata
// (16 or 17 entries), as ral_qconv receives them.  Checks that the output shape is
// the one the convolution produces and that there is one group.
std::string conv2d_geometry(const int64_t input_sizes[4], const int64_t kernel_sizes[4],
                            const int64_t output_sizes[4], const int32_t* padding, const int32_t* metadata,
                            int64_t metadata_len, ConvGeometry* geo);

}  // namespace ral
}  // namespace disc_b200
