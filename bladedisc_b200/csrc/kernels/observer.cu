// Min / max observers (see observer.h).  One read of the tensor: blocks reduce
// slices of a channel to partial (min, max) pairs, a second small kernel folds the
// partials into the running state in a fixed order.  No floating-point atomics, so
// the state does not depend on scheduling.
#include "observer.h"

#include <cuda_fp16.h>
#include <float.h>

#include <algorithm>

#include "rowops.h"
#include "sm100_ptx.cuh"

namespace disc_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxBlocksPerChannel = 1024;
constexpr int64_t kElemsPerBlock = 16384;  // per block and channel before another block is added

template <typename T>
__device__ __forceinline__ float load_f32(const T* p, int64_t i);
template <>
__device__ __forceinline__ float load_f32<float>(const float* p, int64_t i) { return __ldg(p + i); }
template <>
__device__ __forceinline__ float load_f32<__half>(const __half* p, int64_t i) { return __half2float(__ldg(p + i)); }

__device__ __forceinline__ void block_min_max(float& lo, float& hi, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    smem[warp] = lo;
    smem[kThreads / 32 + warp] = hi;
  }
  __syncthreads();
  if (warp == 0) {
    lo = lane < kThreads / 32 ? smem[lane] : __int_as_float(0x7f800000);
    hi = lane < kThreads / 32 ? smem[kThreads / 32 + lane] : __int_as_float(0xff800000);
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
  }
}

// grid (blocks per channel, channels): block b of channel c covers elements
// j = b * per_block .. of the channel's outer * inner elements.
template <typename T>
__global__ void __launch_bounds__(kThreads) minmax_partial_kernel(MinMaxParams p, int64_t per_block) {
  __shared__ float smem[2 * kThreads / 32];
  grid_dep_launch();
  grid_dep_wait();
  const T* x = static_cast<const T*>(p.x);
  const int64_t c = blockIdx.y;
  const int64_t count = p.outer * p.inner;
  const int64_t begin = static_cast<int64_t>(blockIdx.x) * per_block;
  const int64_t end = min(count, begin + per_block);
  float lo = __int_as_float(0x7f800000), hi = __int_as_float(0xff800000);  // +inf, -inf
  if (p.outer == 1 || p.channels == 1) {
    // the channel's elements are one contiguous run
    const int64_t base = p.channels == 1 ? 0 : c * p.inner;
    for (int64_t j = begin + threadIdx.x; j < end; j += kThreads) {
      const float v = load_f32<T>(x, base + j);
      lo = fminf(lo, v);
      hi = fmaxf(hi, v);
    }
  } else {
    for (int64_t j = begin + threadIdx.x; j < end; j += kThreads) {
      const int64_t o = j / p.inner;
      const float v = load_f32<T>(x, (o * p.channels + c) * p.inner + (j - o * p.inner));
      lo = fminf(lo, v);
      hi = fmaxf(hi, v);
    }
  }
  block_min_max(lo, hi, smem);
  if (threadIdx.x == 0) {
    float* part = p.scratch + 2 * (c * gridDim.x + blockIdx.x);
    part[0] = lo;
    part[1] = hi;
  }
}

// one block per channel: partials (in block order) and the running state -> the running state
__global__ void __launch_bounds__(kThreads) minmax_fold_kernel(MinMaxParams p, int blocks) {
  __shared__ float smem[2 * kThreads / 32];
  grid_dep_launch();
  grid_dep_wait();
  const int64_t c = blockIdx.x;
  float lo = __int_as_float(0x7f800000), hi = __int_as_float(0xff800000);
  for (int b = threadIdx.x; b < blocks; b += kThreads) {
    const float* part = p.scratch + 2 * (c * blocks + b);
    lo = fminf(lo, part[0]);
    hi = fmaxf(hi, part[1]);
  }
  block_min_max(lo, hi, smem);
  if (threadIdx.x == 0) {
    p.min_val[c] = fminf(p.min_val[c], lo);
    p.max_val[c] = fmaxf(p.max_val[c], hi);
  }
}

__global__ void __launch_bounds__(kThreads) minmax_qparams_kernel(QParamsParams p) {
  grid_dep_launch();
  grid_dep_wait();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= p.n) return;
  const float mn = p.min_val[i], mx = p.max_val[i];
  float scale = 1.f;
  int32_t zp = 0;
  if (mn <= mx) {
    const float lo = fminf(mn, 0.f), hi = fmaxf(mx, 0.f);
    if (p.symmetric) {
      const float half_range = static_cast<float>(p.qmax - p.qmin) / 2.f;
      scale = fmaxf(__fdiv_rn(fmaxf(-lo, hi), half_range), FLT_EPSILON);
      zp = p.symmetric_zero_point;
    } else {
      scale = fmaxf(__fdiv_rn(hi - lo, static_cast<float>(p.qmax - p.qmin)), FLT_EPSILON);
      const float z = static_cast<float>(p.qmin) - rintf(__fdiv_rn(lo, scale));
      zp = static_cast<int32_t>(fminf(fmaxf(z, static_cast<float>(p.qmin)), static_cast<float>(p.qmax)));
    }
  }
  p.scale[i] = scale;
  p.zero_point[i] = zp;
}

int blocks_per_channel(int64_t count) {
  const int64_t b = (count + kElemsPerBlock - 1) / kElemsPerBlock;
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(b, kMaxBlocksPerChannel)));
}

}  // namespace

int64_t minmax_scratch_floats(int64_t outer, int64_t channels, int64_t inner) {
  if (outer <= 0 || channels <= 0 || inner <= 0) return 0;
  return 2 * channels * blocks_per_channel(outer * inner);
}

cudaError_t minmax_observe_launch(const MinMaxParams& p, cudaStream_t s, const char** err) {
  static const char* none = "";
  const char** e = err ? err : &none;
  if (p.outer < 0 || p.channels < 0 || p.inner < 0) {
    *e = "observer: negative size";
    return cudaErrorInvalidValue;
  }
  if (p.outer == 0 || p.channels == 0 || p.inner == 0) return cudaSuccess;  // nothing observed
  if (!p.x || !p.min_val || !p.max_val) {
    *e = "observer: null operand";
    return cudaErrorInvalidValue;
  }
  if (p.channels > 65535) {
    *e = "observer: more than 65535 channels";
    return cudaErrorInvalidValue;
  }
  const int blocks = blocks_per_channel(p.outer * p.inner);
  if (!p.scratch || p.scratch_floats < 2 * p.channels * blocks) {
    *e = "observer: scratch missing or smaller than minmax_scratch_floats";
    return cudaErrorInvalidValue;
  }
  const int64_t per_block = (p.outer * p.inner + blocks - 1) / blocks;
  cudaError_t st;
  const dim3 grid(blocks, static_cast<unsigned>(p.channels));
  if (p.type == kF32) {
    st = launch_dependent(minmax_partial_kernel<float>, grid, dim3(kThreads), 0, s, p, per_block);
  } else if (p.type == kF16) {
    st = launch_dependent(minmax_partial_kernel<__half>, grid, dim3(kThreads), 0, s, p, per_block);
  } else {
    *e = "observer: element type must be f32 or f16";
    return cudaErrorInvalidValue;
  }
  if (st != cudaSuccess) return st;
  return launch_dependent(minmax_fold_kernel, dim3(static_cast<unsigned>(p.channels)), dim3(kThreads), 0, s, p, blocks);
}

cudaError_t minmax_qparams_launch(const QParamsParams& p, cudaStream_t s, const char** err) {
  static const char* none = "";
  const char** e = err ? err : &none;
  if (p.n < 0 || p.qmax <= p.qmin) {
    *e = "observer: invalid channel count or quantized range";
    return cudaErrorInvalidValue;
  }
  if (p.n == 0) return cudaSuccess;
  if (!p.min_val || !p.max_val || !p.scale || !p.zero_point) {
    *e = "observer: null operand";
    return cudaErrorInvalidValue;
  }
  return launch_dependent(minmax_qparams_kernel, dim3(static_cast<unsigned>((p.n + kThreads - 1) / kThreads)),
                          dim3(kThreads), 0, s, p);
}

// --------------------------------------------------------------------- histogram
namespace {
constexpr int kHistMaxBins = 4096;

// One read of the tensor.  A private histogram sits in shared memory; a block adds its counts to the
// global ones once, at the end.  A thread walks 16-byte vectors with a grid stride.
template <typename T>
__global__ void __launch_bounds__(kThreads) histogram_kernel(HistogramParams p) {
  extern __shared__ uint32_t hist_smem[];
  uint32_t* h = hist_smem;   // [bins]
  grid_dep_launch();
  grid_dep_wait();
  for (int i = threadIdx.x; i < p.bins; i += kThreads) h[i] = 0;
  __syncthreads();
  const float lo = p.lo, hi = p.hi;
  const float span = hi - lo;
  const float fbins = static_cast<float>(p.bins);

  auto count = [&](float v) {
    if (!(v >= lo && v <= hi)) return;   // outside the range, or NaN
    // the order of operations of the CPU kernel: (x - lo) * bins, then / (hi - lo), truncated
    int pos = static_cast<int>(__fdiv_rn(__fmul_rn(__fsub_rn(v, lo), fbins), span));
    if (pos == p.bins) pos -= 1;         // the last bin is closed on the right
    if (pos >= 0 && pos < p.bins) atomicAdd(&h[pos], 1u);
  };

  constexpr int V = 16 / static_cast<int>(sizeof(T));
  const T* x = static_cast<const T*>(p.x);
  const int64_t nvec = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) ? p.n / V : 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < nvec; i += stride) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x) + i);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < V; ++j) count(static_cast<float>(e[j]));
  }
  for (int64_t i = nvec * V + static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < p.n; i += stride) {
    count(static_cast<float>(x[i]));
  }
  __syncthreads();
  for (int i = threadIdx.x; i < p.bins; i += kThreads) {
    if (h[i]) atomicAdd(&p.counts[i], h[i]);
  }
}
}  // namespace

cudaError_t histogram_observe_launch(const HistogramParams& p, cudaStream_t s, const char** err) {
  static const char* none = "";
  const char** e = err ? err : &none;
  if (p.n <= 0) return cudaSuccess;
  if (!p.x || !p.counts || p.bins < 1 || p.bins > kHistMaxBins || !(p.lo <= p.hi)) {
    *e = "observer: histogram needs x, counts, lo <= hi and 1 .. 4096 bins";
    return cudaErrorInvalidValue;
  }
  const size_t smem = static_cast<size_t>(p.bins) * 4;
  int sms = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t want = (p.n / 8 + kThreads - 1) / kThreads;
  const unsigned blocks = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(want, 8LL * sms)));
  if (p.type == kF32) return launch_dependent(histogram_kernel<float>, dim3(blocks), dim3(kThreads), smem, s, p);
  if (p.type == kF16) return launch_dependent(histogram_kernel<__half>, dim3(blocks), dim3(kThreads), smem, s, p);
  *e = "observer: element type must be f32 or f16";
  return cudaErrorInvalidValue;
}

}  // namespace disc_b200
