#include "conv_plan.h"

#include <algorithm>

namespace disc_b200 {
namespace ral {
namespace {

// spatial dims first, then batch, then channel: positions in the data format
bool reorder_dims(const std::string& fmt, int out[4]) {
  const size_t b = fmt.find('N'), c = fmt.find('C');
  if (fmt.size() != 4 || b == std::string::npos || c == std::string::npos) return false;
  int idx = 0;
  for (int i = 0; i < 4; ++i) {
    if (i == static_cast<int>(b) || i == static_cast<int>(c)) continue;
    out[idx++] = i;
  }
  if (idx != 2) return false;
  out[2] = static_cast<int>(b);
  out[3] = static_cast<int>(c);
  return true;
}

bool per_spatial(const std::vector<int64_t>& v, const int order[4], int64_t out[2]) {
  if (v.size() == 1) {
    out[0] = out[1] = v[0];
  } else if (v.size() == 2) {
    out[0] = v[0];
    out[1] = v[1];
  } else if (v.size() == 4) {
    out[0] = v[order[0]];
    out[1] = v[order[1]];
  } else {
    return false;
  }
  return out[0] > 0 && out[1] > 0;
}

void dense_strides(const int64_t sizes[4], int64_t strides[4]) {
  int64_t s = 1;
  for (int i = 3; i >= 0; --i) {
    strides[i] = s;
    s *= sizes[i];
  }
}

}  // namespace

std::string plan_conv2d_from_attrs(const std::string& data_format, const std::vector<int64_t>& strides,
                                   const std::vector<int64_t>& dilations, const std::string& padding,
                                   const std::vector<int64_t>& explicit_paddings, bool weight_is_const,
                                   const int64_t input_sizes[4], const int64_t weight_sizes[4],
                                   int32_t padding_out[4], int64_t result_sizes[4], int32_t metadata_out[17]) {
  int order[4];
  if (!reorder_dims(data_format, order)) return "fail to generate spatial dims";
  int64_t st[2], dl[2];
  if (!per_spatial(strides, order, st) || !per_spatial(dilations, order, dl)) {
    return "fail to generate strides and dilations";
  }
  if (padding == "SAME") {
    // TensorFlow's rule: pad so that the output has ceil(in / stride) positions
    for (int i = 0; i < 2; ++i) {
      const int64_t in = input_sizes[order[i]];
      const int64_t window = (weight_sizes[i + 1] - 1) * dl[i] + 1;
      const int64_t total = in % st[i] == 0 ? std::max<int64_t>(window - st[i], 0)
                                            : std::max<int64_t>(window - in % st[i], 0);
      padding_out[2 * i] = static_cast<int32_t>(total / 2);
      padding_out[2 * i + 1] = static_cast<int32_t>(total - total / 2);
    }
  } else if (padding == "VALID") {
    for (int i = 0; i < 4; ++i) padding_out[i] = 0;
  } else if (padding == "EXPLICIT") {
    if (explicit_paddings.size() == 4) {
      for (int i = 0; i < 4; ++i) padding_out[i] = static_cast<int32_t>(explicit_paddings[i]);
    } else if (explicit_paddings.size() == 8) {
      for (int i = 0; i < 2; ++i) {
        padding_out[2 * i] = static_cast<int32_t>(explicit_paddings[2 * order[i]]);
        padding_out[2 * i + 1] = static_cast<int32_t>(explicit_paddings[2 * order[i] + 1]);
      }
    } else {
      return "fail to generate explicit paddings";
    }
  } else {
    return "fail to generate paddings";
  }
  for (int i = 0; i < 2; ++i) {
    const int64_t in = input_sizes[order[i]], k = weight_sizes[i + 1];
    result_sizes[order[i]] = (in + padding_out[2 * i] + padding_out[2 * i + 1] - k * dl[i] + dl[i] + st[i] - 1) / st[i];
  }
  result_sizes[order[2]] = input_sizes[order[2]];
  result_sizes[order[3]] = weight_sizes[0];
  int idx = 0;
  for (int rep = 0; rep < 3; ++rep) {
    if (rep == 1) {  // kernel: [out, y, x, in]
      metadata_out[idx++] = 3;
      metadata_out[idx++] = 0;
      metadata_out[idx++] = 1;
      metadata_out[idx++] = 2;
    } else {
      metadata_out[idx++] = order[2];
      metadata_out[idx++] = order[3];
      metadata_out[idx++] = order[0];
      metadata_out[idx++] = order[1];
    }
  }
  metadata_out[idx++] = static_cast<int32_t>(st[0]);
  metadata_out[idx++] = static_cast<int32_t>(st[1]);
  metadata_out[idx++] = static_cast<int32_t>(dl[0]);
  metadata_out[idx++] = static_cast<int32_t>(dl[1]);
  metadata_out[idx++] = weight_is_const ? 1 : 0;
  return "";
}

std::string conv2d_geometry(const int64_t input_sizes[4], const int64_t kernel_sizes[4],
                            const int64_t output_sizes[4], const int32_t* padding, const int32_t* metadata,
                            int64_t metadata_len, ConvGeometry* g) {
  if (!padding || !metadata || (metadata_len != 16 && metadata_len != 17)) return "invalid conv params";
  for (int i = 0; i < 12; ++i) {
    if (metadata[i] < 0 || metadata[i] > 3) return "invalid conv params";
  }
  for (int part = 0; part < 3; ++part) {  // each layout is a permutation of the four dims
    int seen = 0;
    for (int i = 0; i < 4; ++i) seen |= 1 << metadata[4 * part + i];
    if (seen != 15) return "invalid conv params";
  }
  const int32_t* in = metadata;
  const int32_t* ker = metadata + 4;
  const int32_t* out = metadata + 8;
  int64_t xs[4], ws[4], os[4];
  dense_strides(input_sizes, xs);
  dense_strides(kernel_sizes, ws);
  dense_strides(output_sizes, os);
  g->batch = input_sizes[in[0]];
  g->in_ch = input_sizes[in[1]];
  g->in_h = input_sizes[in[2]];
  g->in_w = input_sizes[in[3]];
  for (int i = 0; i < 4; ++i) g->x_stride[i] = xs[in[i]];
  const int64_t k_in = kernel_sizes[ker[0]];
  g->out_ch = kernel_sizes[ker[1]];
  g->k_h = kernel_sizes[ker[2]];
  g->k_w = kernel_sizes[ker[3]];
  g->w_stride[0] = ws[ker[1]];
  g->w_stride[1] = ws[ker[0]];
  g->w_stride[2] = ws[ker[2]];
  g->w_stride[3] = ws[ker[3]];
  g->out_h = output_sizes[out[2]];
  g->out_w = output_sizes[out[3]];
  for (int i = 0; i < 4; ++i) g->o_stride[i] = os[out[i]];
  g->stride_h = metadata[12];
  g->stride_w = metadata[13];
  g->dil_h = metadata[14];
  g->dil_w = metadata[15];
  g->pad_top = padding[0];
  g->pad_bottom = padding[1];
  g->pad_left = padding[2];
  g->pad_right = padding[3];
  if (g->stride_h <= 0 || g->stride_w <= 0 || g->dil_h <= 0 || g->dil_w <= 0 || g->pad_top < 0 || g->pad_bottom < 0 ||
      g->pad_left < 0 || g->pad_right < 0) {
    return "invalid conv params";
  }
  if (k_in != g->in_ch) return "invalid conv params: grouped convolution is not supported";
  if (output_sizes[out[0]] != g->batch || output_sizes[out[1]] != g->out_ch) return "invalid conv params";
  const int64_t span_h = g->in_h + g->pad_top + g->pad_bottom - ((g->k_h - 1) * g->dil_h + 1);
  const int64_t span_w = g->in_w + g->pad_left + g->pad_right - ((g->k_w - 1) * g->dil_w + 1);
  const int64_t want_h = span_h < 0 ? 0 : span_h / g->stride_h + 1;
  const int64_t want_w = span_w < 0 ? 0 : span_w / g->stride_w + 1;
  if (g->out_h != want_h || g->out_w != want_w) return "invalid conv params: output shape does not match the convolution";
  return "";
}

}  // namespace ral
}  // namespace disc_b200
