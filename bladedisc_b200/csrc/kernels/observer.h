// Calibration observers on the GPU: running minimum / maximum of what flows
// through a tensor (per tensor or per channel) and the quantization parameters
// that follow from them.  The state stays on the device between batches; nothing
// is read back while calibrating.
//
// Reference: MinMaxObserver / PerChannelMinMaxObserver and
// Observer._calculate_qparams (tools/torch_quant/torch_quant/observer.py:134-165,
// 230-297), which run as eager torch ops.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace disc_b200 {

// min_val[c] = min(min_val[c], min over x[:, c, :]), max_val likewise, x viewed as
// [outer, channels, inner] (channels = 1: the whole tensor).  The caller starts
// the state at +inf / -inf, as the reference's buffers do.  `scratch` holds at
// least minmax_scratch_floats(...) floats.  NaN inputs are not propagated.
struct MinMaxParams {
  const void* x;
  int type;  // ElemType of rowops.h: 0 = f32, 1 = f16
  int64_t outer, channels, inner;
  float* min_val;
  float* max_val;
  float* scratch;
  int64_t scratch_floats;
};
int64_t minmax_scratch_floats(int64_t outer, int64_t channels, int64_t inner);
cudaError_t minmax_observe_launch(const MinMaxParams& p, cudaStream_t s, const char** err);

// scale / zero point from the observed range, n channels:
//   lo = min(min_val, 0), hi = max(max_val, 0)
//   symmetric: scale = max(max(-lo, hi) / ((qmax - qmin) / 2), eps), zp = symmetric_zero_point
//   affine:    scale = max((hi - lo) / (qmax - qmin), eps), zp = clamp(qmin - rne(lo / scale), qmin, qmax)
// with eps the float32 machine epsilon; a range that was never observed
// (min > max) gives scale 1, zero point 0.
struct QParamsParams {
  const float* min_val;
  const float* max_val;
  int64_t n;
  int qmin, qmax;
  int symmetric;
  int symmetric_zero_point;  // 0 for signed types, 128 for quint8
  float* scale;
  int32_t* zero_point;
};
cudaError_t minmax_qparams_launch(const QParamsParams& p, cudaStream_t s, const char** err);

// counts[b] += number of x in bin b of `bins` equal bins over [lo, hi], the binning torch.histc does
// (HistogramObserver, observer.py:447-744, calls it once per batch): bin (int)((x - lo) * bins / (hi - lo)) in
// float32, the last bin includes hi; values outside [lo, hi] and NaN are not counted.  bins <= 4096.
struct HistogramParams {
  const void* x;
  int type;  // 0 = f32, 1 = f16
  int64_t n;
  float lo, hi;
  int bins;
  uint32_t* counts;     // [bins], accumulated into
};
cudaError_t histogram_observe_launch(const HistogramParams& p, cudaStream_t s, const char** err);

}  // namespace disc_b200
