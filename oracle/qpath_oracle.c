/* TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement of the arithmetic of BladeDISC's quantized-inference path,
 * used only as the checker in tests/, in __graft_entry__.smoke() and as the
 * "port" CPU baseline of bench.py.  Nothing under bladedisc_b200/ may call it.
 *
 * Parity pins: checked in tests/test_oracle.py against the reference's own
 * known-answer vectors (12.0 and 128.0 cases of its qgemm feature tests) and
 * against fixtures under tests/golden/ generated here by torch's
 * fake_quantize / layer_norm / softmax and by the reference's torch_quant
 * observers (script: tests/golden/make_golden.py).
 *
 * Every function cites the reference file:line it restates (paths inside
 * alibaba/BladeDISC).  Build: make -C oracle  (gcc -O2 -ffp-contract=off, so
 * that a*b+c stays two roundings unless fmaf is written out).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* q = convert(clamp(round_half_even(x / scale + zero_point), qmin, qmax)).
 * tao_compiler/mlir/disc/transforms/disc_lower_quantize_and_dequantize.cc:77-93
 * (divide, add, round per round_mode, clamp, convert); the torch front end
 * selects RoundHalfToEven (pytorch_blade/pytorch_blade/torch-mlir/lib/Conversion/
 * TorchToMhlo/DiscConvertTorchToDiscMhlo.cpp:115-117).
 * The tensor is viewed as [outer, channels, inner]; channels == 1 is per-tensor. */
ORACLE_API void oracle_quantize_f32(const float* x, int64_t numel, const float* scale,
                                    const int32_t* zero_point, int64_t channels, int64_t inner,
                                    int32_t qmin, int32_t qmax, int8_t* q) {
  if (channels < 1) channels = 1;
  if (inner < 1) inner = 1;
  for (int64_t i = 0; i < numel; ++i) {
    const int64_t c = channels == 1 ? 0 : (i / inner) % channels;
    const float zp = zero_point ? (float)zero_point[c] : 0.f;
    float t = x[i] / scale[c];
    t = t + zp;
    t = rintf(t); /* default rounding mode: to nearest, ties to even */
    t = clampf(t, (float)qmin, (float)qmax);
    q[i] = (int8_t)(int32_t)t;
  }
}

/* y = float(q - zero_point) * scale.
 * disc_lower_quantize_and_dequantize.cc:131-136. */
ORACLE_API void oracle_dequantize_f32(const int8_t* q, int64_t numel, const float* scale,
                                      const int32_t* zero_point, int64_t channels, int64_t inner,
                                      float* y) {
  if (channels < 1) channels = 1;
  if (inner < 1) inner = 1;
  for (int64_t i = 0; i < numel; ++i) {
    const int64_t c = channels == 1 ? 0 : (i / inner) % channels;
    const int32_t zp = zero_point ? zero_point[c] : 0;
    y[i] = (float)((int32_t)q[i] - zp) * scale[c];
  }
}

/* Offline constant (weight) quantisation, done by the compiler in double:
 * q = clamp(round(double(w) / double(s[c]) + zp[c]), qmin, qmax), half-to-even.
 * tao_compiler/mlir/disc/IR/hlo_disc_ops.cc:149-340 (QuantizeOp::fold). */
ORACLE_API void oracle_quantize_weight_f64(const float* w, int64_t rows, int64_t cols,
                                           const float* scale, const int32_t* zero_point,
                                           int per_channel, int32_t qmin, int32_t qmax, int8_t* q) {
  for (int64_t r = 0; r < rows; ++r) {
    const int64_t c = per_channel ? r : 0;
    const double s = (double)scale[c];
    const double zp = zero_point ? (double)zero_point[c] : 0.0;
    for (int64_t j = 0; j < cols; ++j) {
      double t = rint((double)w[r * cols + j] / s + zp);
      if (t < (double)qmin) t = (double)qmin;
      if (t > (double)qmax) t = (double)qmax;
      q[r * cols + j] = (int8_t)(int32_t)t;
    }
  }
}

/* The golden of the reference's own e2e tests: torch.fake_quantize_per_tensor_affine
 * / per_channel_affine (pytorch_blade/tests/disc/pdl/test_e2e/test_quantization.py:357-460;
 * tools/torch_quant/torch_quant/observer.py:181-208):
 * fq(x) = (clamp(nearbyint(x * (1/s)) + zp, qmin, qmax) - zp) * s. */
ORACLE_API void oracle_fake_quant_f32(const float* x, int64_t numel, const float* scale,
                                      const int32_t* zero_point, int64_t channels, int64_t inner,
                                      int32_t qmin, int32_t qmax, float* y) {
  if (channels < 1) channels = 1;
  if (inner < 1) inner = 1;
  for (int64_t i = 0; i < numel; ++i) {
    const int64_t c = channels == 1 ? 0 : (i / inner) % channels;
    const int32_t zp = zero_point ? zero_point[c] : 0;
    const float inv = 1.0f / scale[c];
    float t = nearbyintf(x[i] * inv) + (float)zp;
    t = clampf(t, (float)qmin, (float)qmax);
    y[i] = (t - (float)zp) * scale[c];
  }
}

/* acc[m, n] = sum_k a[m, k] * w[n, k] in int32: the COMPUTE_32I product the GPU
 * path asks cuBLASLt for (tao_compiler/mlir/ral/context/
 * quantized_gpu_kernel_impl.cc:57-100, 418-420; weight is [N, K], "n x k col major"
 * at :323-327). */
ORACLE_API void oracle_qgemm_acc(const int8_t* a, const int8_t* w, int64_t M, int64_t N, int64_t K,
                                 int32_t* acc) {
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
  for (int64_t m = 0; m < M; ++m) {
    const int8_t* ar = a + m * K;
    for (int64_t n = 0; n < N; ++n) {
      const int8_t* wr = w + n * K;
      int32_t s = 0;
      for (int64_t k = 0; k < K; ++k) s += (int32_t)ar[k] * (int32_t)wr[k];
      acc[m * N + n] = s;
    }
  }
}

static inline float act_apply(float v, int act) {
  if (act == 1) return 0.5f * v * (1.f + erff(v * 0.70710678118654752440f)); /* exact GELU */
  if (act == 2) return v / (1.f + expf(-v));                                  /* SiLU */
  return v;
}

static inline int8_t sat_s8(float v) {
  float r = rintf(v);
  r = clampf(r, -128.f, 127.f);
  return (int8_t)(int32_t)r;
}

enum { SCALE_NONE = 0, SCALE_SCALAR = 1, SCALE_PER_COL = 2, SCALE_PER_ROW = 3 };
enum { BIAS_NONE = 0, BIAS_F32 = 1, BIAS_I8 = 2 };
enum { OUT_I8 = 0, OUT_F16 = 1, OUT_F32 = 2, OUT_I32 = 3 };

/* General epilogue on an int32 accumulator matrix; produces float values
 * (before the final store conversion) and, for OUT_I8, the int8 result.
 *
 *   cs = x_scale(n) * w_scale(n) [/ out_scale(n) when fold_out]
 *   v  = fmaf(float(acc) [* x_scale[m]], cs, bias[n]); v = act(v); [v /= out_scale]
 *
 * With fold_out = 1, act = 0 and scalar scales this is ral_pdll_qgemm:
 * kernel_scale = input_scale * weight_scale / result_scale computed in fp32 in
 * that order (quantized_gpu_kernel_impl.cc:382), alpha * acc + bias, saturating
 * round-to-nearest conversion to int8 (cuBLASLt epilogue, :130-159).  With
 * per-column scales it is ral_pdll_qgemm_per_channel (:267-270).  With
 * div_out it is dequantize -> bias -> activation -> quantize of the lowered
 * graph (disc_lower_quantize_and_dequantize.cc:77-93,131-136). */
ORACLE_API void oracle_qgemm_epilogue(const int32_t* acc, int64_t M, int64_t N, const float* x_scale,
                                      int x_kind, const float* w_scale, int w_kind,
                                      const float* out_scale, int o_kind, const void* bias,
                                      int bias_kind, int fold_out, int div_out, int act,
                                      float* out_f32, int8_t* out_i8) {
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t n = 0; n < N; ++n) {
      float sx = 1.f, sw = 1.f;
      if (x_kind == SCALE_SCALAR) sx = x_scale[0];
      else if (x_kind == SCALE_PER_COL) sx = x_scale[n];
      if (w_kind == SCALE_SCALAR) sw = w_scale[0];
      else if (w_kind == SCALE_PER_COL) sw = w_scale[n];
      float cs = sx * sw;
      if (fold_out) cs = cs / (o_kind == SCALE_PER_COL ? out_scale[n] : out_scale[0]);
      float cb = 0.f;
      if (bias_kind == BIAS_F32) cb = ((const float*)bias)[n];
      else if (bias_kind == BIAS_I8) cb = (float)((const int8_t*)bias)[n];
      float t = (float)acc[m * N + n];
      if (x_kind == SCALE_PER_ROW) t = t * x_scale[m];
      float v = fmaf(t, cs, cb);
      v = act_apply(v, act);
      if (div_out) v = v / out_scale[0];
      if (out_f32) out_f32[m * N + n] = v;
      if (out_i8) out_i8[m * N + n] = sat_s8(v);
    }
  }
}

/* x86 (oneDNN) form of the same custom call: the f32 bias is first rounded to
 * s32 at the accumulator scale, then one per-channel output scale is applied:
 *   bias_s32[n] = rne(bias[n] * (1 / (s_x * s_w[n])))
 *   out = sat_s8(rne(float(acc + bias_s32[n]) * ((s_x * s_w[n]) / s_out)))
 * tao_compiler/mlir/ral/context/mkldnn/ideep/ideep/operators/matmul.hpp:527-536
 * (bias_scales, op_scales) and :556-565 (bias as s32); call site
 * tao_compiler/mlir/ral/context/common_context_impl_quantization.cc:1268-1400. */
ORACLE_API void oracle_qgemm_x86(const int32_t* acc, int64_t M, int64_t N, float s_x,
                                 const float* s_w, int w_per_channel, float s_out,
                                 const float* bias, int8_t* out) {
  for (int64_t n = 0; n < N; ++n) {
    const float sw = w_per_channel ? s_w[n] : s_w[0];
    const float bias_scale = 1.0f / (s_x * sw);
    const float op_scale = (s_x * sw) / s_out;
    int32_t b32 = 0;
    if (bias) {
      float br = rintf(bias[n] * bias_scale);
      if (br > 2147483520.f) br = 2147483520.f;
      if (br < -2147483648.f) br = -2147483648.f;
      b32 = (int32_t)br;
    }
    for (int64_t m = 0; m < M; ++m) {
      const float v = (float)(acc[m * N + n] + b32) * op_scale;
      out[m * N + n] = sat_s8(v);
    }
  }
}

/* Per-row symmetric quantisation of activations (an extension: the reference
 * quantize op rejects use_dynamic, disc_lower_quantize_and_dequantize.cc:41-43):
 * scale[r] = max(max|x[r,:]| / 127, FLT_EPSILON), q = quantize(x, scale[r]). */
ORACLE_API void oracle_dynamic_quantize_f32(const float* x, int64_t rows, int64_t cols, int8_t* q,
                                            float* row_scale) {
  for (int64_t r = 0; r < rows; ++r) {
    float m = 0.f;
    for (int64_t c = 0; c < cols; ++c) {
      const float a = fabsf(x[r * cols + c]);
      if (a > m) m = a;
    }
    float s = m / 127.f;
    if (s < 1.1920928955078125e-07f) s = 1.1920928955078125e-07f;
    row_scale[r] = s;
    for (int64_t c = 0; c < cols; ++c) {
      float t = rintf(x[r * cols + c] / s);
      t = clampf(t, -128.f, 127.f);
      q[r * cols + c] = (int8_t)(int32_t)t;
    }
  }
}

/* LayerNorm / RMSNorm over the last axis, as eager PyTorch computes it (the
 * golden of pytorch_blade/tests/disc/ops/test_layer_norm.py); statistics in
 * double so that the restatement itself adds no error.
 * y = (x + residual - mean) / sqrt(var + eps) * gamma + beta. */
ORACLE_API void oracle_norm_f32(const float* x, const float* residual, const float* gamma,
                                const float* beta, int64_t rows, int64_t cols, float eps, int rms,
                                float* y, float* sum_out) {
  double* buf = (double*)malloc(sizeof(double) * (size_t)cols);
  for (int64_t r = 0; r < rows; ++r) {
    double mean = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
      float v = x[r * cols + c];
      if (residual) v = v + residual[r * cols + c];
      if (sum_out) sum_out[r * cols + c] = v;
      buf[c] = (double)v;
      mean += buf[c];
    }
    mean = rms ? 0.0 : mean / (double)cols;
    double var = 0.0;
    for (int64_t c = 0; c < cols; ++c) var += (buf[c] - mean) * (buf[c] - mean);
    var /= (double)cols;
    const double rstd = 1.0 / sqrt(var + (double)eps);
    for (int64_t c = 0; c < cols; ++c) {
      double v = (buf[c] - mean) * rstd * (double)gamma[c];
      if (!rms && beta) v += (double)beta[c];
      y[r * cols + c] = (float)v;
    }
  }
  free(buf);
}

/* softmax(x * scale + mask) over the last axis with an optional valid length
 * per batch (columns >= len get probability 0): eager PyTorch's softmax, the
 * golden of pytorch_blade/tests/disc/ops/test_nn_ops.py:30-90. */
ORACLE_API void oracle_softmax_f32(const float* x, int64_t rows, int64_t cols, int64_t rows_per_batch,
                                   const int32_t* lens, const float* mask, float scale,
                                   int log_softmax, float* y) {
  if (rows_per_batch <= 0) rows_per_batch = rows;
  for (int64_t r = 0; r < rows; ++r) {
    const int64_t b = r / rows_per_batch;
    int64_t len = lens ? lens[b] : cols;
    if (len > cols) len = cols;
    double mx = -INFINITY;
    for (int64_t c = 0; c < len; ++c) {
      double v = (double)(x[r * cols + c] * scale);
      if (mask) v = (double)(x[r * cols + c] * scale + mask[b * cols + c]);
      if (v > mx) mx = v;
    }
    double sum = 0.0;
    for (int64_t c = 0; c < len; ++c) {
      float v = x[r * cols + c] * scale;
      if (mask) v = v + mask[b * cols + c];
      sum += exp((double)v - mx);
    }
    for (int64_t c = 0; c < cols; ++c) {
      if (c >= len) {
        y[r * cols + c] = log_softmax ? -INFINITY : 0.f;
        continue;
      }
      float v = x[r * cols + c] * scale;
      if (mask) v = v + mask[b * cols + c];
      const double d = (double)v - mx;
      y[r * cols + c] = (float)(log_softmax ? d - log(sum) : exp(d) / sum);
    }
  }
}

/* Convenience for timing (bench.py "port" baseline): int32 product plus the
 * ral_pdll_qgemm epilogue, blocked over rows so that OpenMP (if the file is
 * built with -fopenmp) can spread it.  Same arithmetic as the two functions
 * above. */
ORACLE_API void oracle_qgemm_ral_i8(const int8_t* a, const int8_t* w, int64_t M, int64_t N, int64_t K,
                                    float s_x, const float* s_w, int w_per_channel, float s_out,
                                    const float* bias, int8_t* out) {
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
  for (int64_t m = 0; m < M; ++m) {
    const int8_t* ar = a + m * K;
    for (int64_t n = 0; n < N; ++n) {
      const int8_t* wr = w + n * K;
      int32_t s = 0;
      for (int64_t k = 0; k < K; ++k) s += (int32_t)ar[k] * (int32_t)wr[k];
      const float sw = w_per_channel ? s_w[n] : s_w[0];
      const float cs = (s_x * sw) / s_out;
      out[m * N + n] = sat_s8(fmaf((float)s, cs, bias ? bias[n] : 0.f));
    }
  }
}

/* ---- configuration 4 (column-parallel decoder): the glue around the linears.
 * None of this exists as named code in the reference (its quantize op rejects
 * dynamic scales, disc_lower_quantize_and_dequantize.cc:41-43; RoPE and SwiGLU
 * reach it as generated elementwise kernels), so these restate the defining
 * formulas -- parity unpinned against the reference for these three, pinned to
 * numpy / eager torch in tests/test_oracle.py -- and the collective itself is
 * ral_all_gather's rank-major concatenation
 * (tao_compiler/mlir/ral/collective.cu.cc:226-309). */

/* h = up ? silu(gate) * up : gate, per-row symmetric int8:
 * row_scale[r] = max(max|h[r,:]| / 127, FLT_EPSILON), q = sat(rne(h / row_scale[r])).
 * gate / up are [rows, cols] with row stride ld.  silu in double, so that the
 * restatement adds no error of its own (the GPU kernel uses the approximate
 * exponential and reciprocal: compare within 1 LSB). */
ORACLE_API void oracle_gated_quantize_f32(const float* gate, const float* up, int64_t rows, int64_t cols,
                                          int64_t ld, int8_t* q, float* row_scale) {
  for (int64_t r = 0; r < rows; ++r) {
    float m = 0.f;
    for (int64_t c = 0; c < cols; ++c) {
      const double g = gate[r * ld + c];
      const float h = up ? (float)(g / (1.0 + exp(-g)) * (double)up[r * ld + c]) : (float)g;
      if (fabsf(h) > m) m = fabsf(h);
    }
    float s = m / 127.f;
    if (s < 1.1920928955078125e-07f) s = 1.1920928955078125e-07f;
    row_scale[r] = s;
    for (int64_t c = 0; c < cols; ++c) {
      const double g = gate[r * ld + c];
      const float h = up ? (float)(g / (1.0 + exp(-g)) * (double)up[r * ld + c]) : (float)g;
      q[r * cols + c] = (int8_t)(int32_t)clampf(rintf(h / s), -128.f, 127.f);
    }
  }
}

/* Rotary position embedding of x [tokens, heads, dim] at positions pos[token]:
 * pairs (i, i + dim/2), out1 = x1 cos - x2 sin, out2 = x2 cos + x1 sin with
 * cos / sin [positions, dim/2]; every product and sum rounded to fp32 on its own
 * (this file is built with -ffp-contract=off), as an unfused elementwise graph
 * computes them. */
ORACLE_API void oracle_rope_f32(const float* x, const int64_t* pos, const float* cos_t, const float* sin_t,
                                int64_t tokens, int64_t heads, int64_t dim, float* y) {
  const int64_t half = dim / 2;
  for (int64_t t = 0; t < tokens; ++t) {
    const float* cs = cos_t + pos[t] * half;
    const float* sn = sin_t + pos[t] * half;
    for (int64_t h = 0; h < heads; ++h) {
      const float* xr = x + (t * heads + h) * dim;
      float* yr = y + (t * heads + h) * dim;
      for (int64_t i = 0; i < half; ++i) {
        const float a = xr[i] * cs[i];
        const float b = xr[i + half] * sn[i];
        const float c = xr[i + half] * cs[i];
        const float d = xr[i] * sn[i];
        yr[i] = a - b;
        yr[i + half] = c + d;
      }
    }
  }
}

/* What an all-gather of column-parallel results leaves on every rank: slot r of
 * out [ranks, rows, cols / ranks] holds columns [r * cols / ranks, ...) of the
 * row-major matrix x [rows, cols] (byte-wise; elem = element size). */
ORACLE_API void oracle_gathered_layout(const void* x, int64_t rows, int64_t cols, int64_t ranks, int64_t elem,
                                       void* out) {
  const int64_t share = cols / ranks;
  const char* src = (const char*)x;
  char* dst = (char*)out;
  for (int64_t r = 0; r < ranks; ++r)
    for (int64_t m = 0; m < rows; ++m)
      memcpy(dst + ((r * rows + m) * share) * elem, src + (m * cols + r * share) * elem, (size_t)(share * elem));
}

/* ---- Weight-only quantized linear.
 * The reference has the front end and the custom call name but no open kernel
 * (pytorch_blade/tests/disc/pdl/pdll_files/gpu/weight_only_qgemm.pdll:2-106), so
 * the definition restated here is the model its tests compile
 * (pytorch_blade/tests/disc/pdl/test_torchscipt_to_mhlo/test_quantization.py:501-618):
 *   F.linear(x, fake_quantize_per_channel_affine(weight, scale, zp, 0, 0, 255), bias)
 * i.e. out[m, n] = sum_k x[m, k] * ((q[k, n] - zp[n]) * scale[n]) + bias[n] with
 * q the uint8 weight, stored transposed [K, N] as the pattern passes it.  The sum
 * is taken in double over the exact products x * (q - zp); scale and bias are
 * applied once, in float.  Pinned to that eager torch model on the CPU in
 * tests/test_oracle.py; there is no reference kernel output to pin to. */
ORACLE_API void oracle_weight_only_qgemm_f32(const float* x, const uint8_t* w, const float* scale, const int32_t* zp,
                                             const float* bias, int64_t m, int64_t n, int64_t k, float* out) {
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      const int32_t z = zp ? zp[j] : 0;
      double acc = 0.0;
      for (int64_t t = 0; t < k; ++t) acc += (double)x[i * k + t] * (double)((int32_t)w[t * n + j] - z);
      const float v = (float)acc * scale[j];
      out[i * n + j] = bias ? v + bias[j] : v;
    }
  }
}

/* ---- Quantized 2-D convolution, int8 x int8 -> int8, symmetric.
 * out = sat_s8(rne( acc * (s_x * s_w[o] / s_out) )), acc the int32 convolution sum,
 * zero outside the input.  Restates what ral_qconv computes through cuDNN with
 * scale = s_in * s_w / s_out (tao_compiler/mlir/ral/context/stream_executor_based_impl.cc:1866-1873)
 * and ral_pdll_qconv2d with per-channel weight scales
 * (common_context_impl_quantization.cc:363-607).  Operands by role: element strides
 * for (batch, channel, y, x) of input and output and (out, in, y, x) of the kernel,
 * so that every layout of the reference's tests (NHWC / NCHW data, OHWI kernel) is
 * one code path.  Pinned to the known answers of
 * tao_compiler/mlir/disc/tests/pdll/quantized_conv2d.cc in tests/test_oracle.py. */
ORACLE_API void oracle_qconv2d_s8(const int8_t* x, const int8_t* w, int8_t* out, const int64_t* dims9,
                                  const int64_t* x_stride4, const int64_t* w_stride4, const int64_t* o_stride4,
                                  const int64_t* conv8, float x_scale, const float* w_scale, int w_scale_per_channel,
                                  float out_scale) {
  const int64_t batch = dims9[0], in_ch = dims9[1], in_h = dims9[2], in_w = dims9[3];
  const int64_t out_ch = dims9[4], k_h = dims9[5], k_w = dims9[6], out_h = dims9[7], out_w = dims9[8];
  const int64_t sh = conv8[0], sw = conv8[1], dh = conv8[2], dw = conv8[3], pt = conv8[4], pl = conv8[6];
  for (int64_t n = 0; n < batch; ++n) {
    for (int64_t o = 0; o < out_ch; ++o) {
      /* the "kernel scale" in the reference's order: (s_x * s_w) / s_out, in float */
      const float cs = x_scale * w_scale[w_scale_per_channel ? o : 0] / out_scale;
      for (int64_t oy = 0; oy < out_h; ++oy) {
        for (int64_t ox = 0; ox < out_w; ++ox) {
          int32_t acc = 0;
          for (int64_t ky = 0; ky < k_h; ++ky) {
            const int64_t iy = oy * sh - pt + ky * dh;
            if (iy < 0 || iy >= in_h) continue;
            for (int64_t kx = 0; kx < k_w; ++kx) {
              const int64_t ix = ox * sw - pl + kx * dw;
              if (ix < 0 || ix >= in_w) continue;
              for (int64_t c = 0; c < in_ch; ++c) {
                acc += (int32_t)x[n * x_stride4[0] + c * x_stride4[1] + iy * x_stride4[2] + ix * x_stride4[3]] *
                       (int32_t)w[o * w_stride4[0] + c * w_stride4[1] + ky * w_stride4[2] + kx * w_stride4[3]];
              }
            }
          }
          out[n * o_stride4[0] + o * o_stride4[1] + oy * o_stride4[2] + ox * o_stride4[3]] =
              sat_s8(fmaf((float)acc, cs, 0.f));
        }
      }
    }
  }
}
