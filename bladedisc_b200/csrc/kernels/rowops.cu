// Bandwidth-bound kernels of the quantized path, hand-written for sm_100a.
//
// In the reference these are compiler-generated: quantize / dequantize are
// lowered to elementwise mhlo (tao_compiler/mlir/disc/transforms/
// disc_lower_quantize_and_dequantize.cc:36-139) and codegen'd as kLoop
// kernels; LayerNorm / softmax become kRowReduction / kStitch kernels with one
// of two schedules, one warp per row or one block per row
// (tao_compiler/mlir/disc/transforms/lhlo_legalize_roots_to_loops.cc:1263-1289,
// 1678-1716; choice at disc_specialize_fusion_with_speculation.cc:393-452).
// Here the same two schedules exist, but a row is read once with 16-byte
// loads, kept in registers across the reductions, and written once.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <float.h>

#include "rowops.h"

namespace disc_b200 {
namespace {

constexpr int kBlock = 256;

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

__device__ __forceinline__ int8_t quant_one(float x, float s, float zp, float qmin, float qmax) {
  // divide, add zero point, round half to even, clamp, convert: the order of the reference.
  float t = __fadd_rn(__fdiv_rn(x, s), zp);
  t = rintf(t);
  t = fminf(fmaxf(t, qmin), qmax);
  return static_cast<int8_t>(static_cast<int>(t));
}

// 8 consecutive elements as floats.
template <typename T>
struct Pack8;
template <>
struct Pack8<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
  static __device__ __forceinline__ float get(const float* p) { return *p; }
  static __device__ __forceinline__ void put(float* p, float v) { *p = v; }
};
template <>
struct Pack8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float* v) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__half* p, const float* v) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
  static __device__ __forceinline__ float get(const __half* p) { return __half2float(*p); }
  static __device__ __forceinline__ void put(__half* p, float v) { *p = __float2half_rn(v); }
};

__device__ __forceinline__ void store_q8(int8_t* p, const int8_t* q) {
  uint2 u;
  u.x = static_cast<uint8_t>(q[0]) | (static_cast<uint8_t>(q[1]) << 8) |
        (static_cast<uint8_t>(q[2]) << 16) | (static_cast<uint32_t>(static_cast<uint8_t>(q[3])) << 24);
  u.y = static_cast<uint8_t>(q[4]) | (static_cast<uint8_t>(q[5]) << 8) |
        (static_cast<uint8_t>(q[6]) << 16) | (static_cast<uint32_t>(static_cast<uint8_t>(q[7])) << 24);
  *reinterpret_cast<uint2*>(p) = u;
}

// ------------------------------------------------------ elementwise quantize
// Per-tensor, 16 elements per thread per step: 16-byte int8 stores.
template <typename T>
__global__ void __launch_bounds__(kBlock)
quantize_tensor_kernel(const T* __restrict__ x, int8_t* __restrict__ q, int64_t numel,
                       const float* __restrict__ scale, const int32_t* __restrict__ zero_point,
                       float qmin, float qmax, int aligned) {
  const float s = __ldg(scale);
  const float zp = zero_point ? static_cast<float>(__ldg(zero_point)) : 0.f;
  const int64_t nvec = aligned ? numel / 16 : 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; v < nvec; v += stride) {
    float f[16];
    Pack8<T>::load(x + v * 16, f);
    Pack8<T>::load(x + v * 16 + 8, f + 8);
    int8_t o[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i] = quant_one(f[i], s, zp, qmin, qmax);
    uint4 u;
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[i] = static_cast<uint8_t>(o[4 * i]) | (static_cast<uint8_t>(o[4 * i + 1]) << 8) |
             (static_cast<uint8_t>(o[4 * i + 2]) << 16) |
             (static_cast<uint32_t>(static_cast<uint8_t>(o[4 * i + 3])) << 24);
    }
    *reinterpret_cast<uint4*>(q + v * 16) = u;
  }
  for (int64_t i = nvec * 16 + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < numel;
       i += stride) {
    q[i] = quant_one(Pack8<T>::get(x + i), s, zp, qmin, qmax);
  }
}

// Per-axis: scale index = (i / inner) % channels.
template <typename T>
__global__ void __launch_bounds__(kBlock)
quantize_axis_kernel(const T* __restrict__ x, int8_t* __restrict__ q, int64_t numel,
                     const float* __restrict__ scale, const int32_t* __restrict__ zero_point,
                     int64_t channels, int64_t inner, float qmin, float qmax) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < numel; i += stride) {
    const int64_t c = (i / inner) % channels;
    const float zp = zero_point ? static_cast<float>(__ldg(zero_point + c)) : 0.f;
    q[i] = quant_one(Pack8<T>::get(x + i), __ldg(scale + c), zp, qmin, qmax);
  }
}

template <typename T>
__global__ void __launch_bounds__(kBlock)
dequantize_kernel(const int8_t* __restrict__ q, T* __restrict__ y, int64_t numel,
                  const float* __restrict__ scale, const int32_t* __restrict__ zero_point,
                  int64_t channels, int64_t inner, int aligned) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (channels == 1) {
    const float s = __ldg(scale);
    const int zp = zero_point ? __ldg(zero_point) : 0;
    const int64_t nvec = aligned ? numel / 16 : 0;
    for (int64_t v = tid; v < nvec; v += stride) {
      const uint4 u = *reinterpret_cast<const uint4*>(q + v * 16);
      const int8_t* b = reinterpret_cast<const int8_t*>(&u);
      float f[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = __fmul_rn(static_cast<float>(static_cast<int>(b[i]) - zp), s);
      Pack8<T>::store(y + v * 16, f);
      Pack8<T>::store(y + v * 16 + 8, f + 8);
    }
    for (int64_t i = nvec * 16 + tid; i < numel; i += stride) {
      Pack8<T>::put(y + i, __fmul_rn(static_cast<float>(static_cast<int>(q[i]) - zp), s));
    }
  } else {
    for (int64_t i = tid; i < numel; i += stride) {
      const int64_t c = (i / inner) % channels;
      const int zp = zero_point ? __ldg(zero_point + c) : 0;
      Pack8<T>::put(y + i, __fmul_rn(static_cast<float>(static_cast<int>(q[i]) - zp), __ldg(scale + c)));
    }
  }
}

// ------------------------------------------------------------- row kernels
// A row is shared by G threads (32 = one warp per row, 256 = one block per
// row).  Thread t of the group owns 8-element vectors t, t+G, t+2G, ... up to
// MAXV of them, all kept in registers.
template <int G>
__device__ __forceinline__ float group_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (G > 32) {
    const int w = threadIdx.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[w] = v;
    __syncthreads();
    v = red[0];
#pragma unroll
    for (int i = 1; i < G / 32; ++i) v += red[i];
  }
  return v;
}
template <int G>
__device__ __forceinline__ float group_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if (G > 32) {
    const int w = threadIdx.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[w] = v;
    __syncthreads();
    v = red[0];
#pragma unroll
    for (int i = 1; i < G / 32; ++i) v = fmaxf(v, red[i]);
  }
  return v;
}

template <typename T, int G, int MAXV>
__device__ __forceinline__ void row_load(const T* row, int cols, int t, bool aligned, float fill,
                                         float (&x)[MAXV * 8]) {
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int base = (t + i * G) * 8;
    if (aligned) {
      if (base < cols) {
        Pack8<T>::load(row + base, &x[i * 8]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[i * 8 + j] = fill;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[i * 8 + j] = (base + j < cols) ? Pack8<T>::get(row + base + j) : fill;
    }
  }
}

template <typename T, int G, int MAXV>
__device__ __forceinline__ void row_store(T* row, int cols, int t, bool aligned,
                                          const float (&x)[MAXV * 8]) {
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int base = (t + i * G) * 8;
    if (aligned) {
      if (base < cols) Pack8<T>::store(row + base, &x[i * 8]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (base + j < cols) Pack8<T>::put(row + base + j, x[i * 8 + j]);
    }
  }
}

template <int G, int MAXV>
__device__ __forceinline__ void row_store_q8(int8_t* row, int cols, int t, bool aligned,
                                             const int8_t (&q)[MAXV * 8]) {
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int base = (t + i * G) * 8;
    if (aligned) {
      if (base < cols) store_q8(row + base, &q[i * 8]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (base + j < cols) row[base + j] = q[i * 8 + j];
    }
  }
}

template <typename T, int G, int MAXV>
__global__ void __launch_bounds__(kBlock)
norm_kernel(NormParams p, int aligned) {
  __shared__ float red[8];
  const int t = threadIdx.x % G;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (kBlock / G) + threadIdx.x / G;
  const bool active = row < p.rows;  // whole groups are active or not
  if (G == 32 && !active) return;    // warp-per-row: no block-level sync is used
  const int cols = static_cast<int>(p.cols);
  const bool al = aligned != 0;
  const int64_t off = (active ? row : 0) * p.cols;
  float x[MAXV * 8];
  row_load<T, G, MAXV>(reinterpret_cast<const T*>(p.x) + off, cols, t, al, 0.f, x);
  if (p.residual) {
    float r[MAXV * 8];
    row_load<T, G, MAXV>(reinterpret_cast<const T*>(p.residual) + off, cols, t, al, 0.f, r);
#pragma unroll
    for (int i = 0; i < MAXV * 8; ++i) x[i] += r[i];
    if (p.sum_out) {
      // Round the stream to its storage type once, and normalise what was stored.
#pragma unroll
      for (int i = 0; i < MAXV * 8; ++i) {
        if (sizeof(T) == 2) x[i] = __half2float(__float2half_rn(x[i]));
      }
      if (active) row_store<T, G, MAXV>(reinterpret_cast<T*>(p.sum_out) + off, cols, t, al, x);
    }
  }
  const float inv_n = 1.f / static_cast<float>(cols);
  float mean = 0.f;
  if (!p.rms) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV * 8; ++i) s += x[i];
    mean = group_sum<G>(s, red) * inv_n;
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = (t + i * G) * 8 + j;
      const float d = (c < cols) ? x[i * 8 + j] - mean : 0.f;
      ss += d * d;
    }
  }
  const float var = group_sum<G>(ss, red) * inv_n;
  const float rstd = 1.f / sqrtf(var + p.eps);
  float g[MAXV * 8];
  row_load<T, G, MAXV>(reinterpret_cast<const T*>(p.gamma), cols, t, al, 0.f, g);
#pragma unroll
  for (int i = 0; i < MAXV * 8; ++i) x[i] = (x[i] - mean) * rstd * g[i];
  if (!p.rms && p.beta) {
    row_load<T, G, MAXV>(reinterpret_cast<const T*>(p.beta), cols, t, al, 0.f, g);
#pragma unroll
    for (int i = 0; i < MAXV * 8; ++i) x[i] += g[i];
  }
  if (sizeof(T) == 2) {
    // What the next op sees is the stored half value; quantize that one.
#pragma unroll
    for (int i = 0; i < MAXV * 8; ++i) x[i] = __half2float(__float2half_rn(x[i]));
  }
  if (p.y && active) row_store<T, G, MAXV>(reinterpret_cast<T*>(p.y) + off, cols, t, al, x);
  if (p.q_out) {
    float s;
    if (p.q_scale) {
      s = __ldg(p.q_scale);
    } else {
      float m = 0.f;
#pragma unroll
      for (int i = 0; i < MAXV * 8; ++i) m = fmaxf(m, fabsf(x[i]));  // padding holds 0
      m = group_max<G>(m, red);
      s = fmaxf(__fdiv_rn(m, 127.f), FLT_EPSILON);
      if (t == 0 && active && p.q_row_scale) p.q_row_scale[row] = s;
    }
    int8_t q[MAXV * 8];
#pragma unroll
    for (int i = 0; i < MAXV * 8; ++i) q[i] = quant_one(x[i], s, 0.f, -128.f, 127.f);
    if (active) row_store_q8<G, MAXV>(p.q_out + off, cols, t, al, q);
  }
}

template <typename T, int G, int MAXV>
__global__ void __launch_bounds__(kBlock)
dynquant_kernel(DynQuantParams p, int aligned) {
  __shared__ float red[8];
  const int t = threadIdx.x % G;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (kBlock / G) + threadIdx.x / G;
  const bool active = row < p.rows;
  if (G == 32 && !active) return;
  const int cols = static_cast<int>(p.cols);
  const bool al = aligned != 0;
  const int64_t off = (active ? row : 0) * p.cols;
  float x[MAXV * 8];
  row_load<T, G, MAXV>(reinterpret_cast<const T*>(p.x) + off, cols, t, al, 0.f, x);
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV * 8; ++i) m = fmaxf(m, fabsf(x[i]));
  m = group_max<G>(m, red);
  const float s = fmaxf(__fdiv_rn(m, 127.f), FLT_EPSILON);
  if (t == 0 && active) p.row_scale[row] = s;
  int8_t q[MAXV * 8];
#pragma unroll
  for (int i = 0; i < MAXV * 8; ++i) q[i] = quant_one(x[i], s, 0.f, -128.f, 127.f);
  if (active) row_store_q8<G, MAXV>(p.q + off, cols, t, al, q);
}

template <typename T, int G, int MAXV>
__global__ void __launch_bounds__(kBlock)
softmax_kernel(SoftmaxParams p, int aligned) {
  __shared__ float red[8];
  const int t = threadIdx.x % G;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (kBlock / G) + threadIdx.x / G;
  const bool active = row < p.rows;
  if (G == 32 && !active) return;
  const int cols = static_cast<int>(p.cols);
  const bool al = aligned != 0;
  const int64_t r = active ? row : 0;
  const int64_t batch = r / p.rows_per_batch;
  const int len = p.lens ? min(cols, __ldg(p.lens + batch)) : cols;
  float x[MAXV * 8];
  row_load<T, G, MAXV>(reinterpret_cast<const T*>(p.x) + r * p.cols, cols, t, al, 0.f, x);
#pragma unroll
  for (int i = 0; i < MAXV * 8; ++i) x[i] *= p.scale;
  if (p.mask) {
    float mk[MAXV * 8];
    row_load<T, G, MAXV>(reinterpret_cast<const T*>(p.mask) + batch * p.cols, cols, t, al, 0.f, mk);
#pragma unroll
    for (int i = 0; i < MAXV * 8; ++i) x[i] += mk[i];
  }
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = (t + i * G) * 8 + j;
      if (c >= len) x[i * 8 + j] = -INFINITY;
      mx = fmaxf(mx, x[i * 8 + j]);
    }
  }
  mx = group_max<G>(mx, red);
  if (mx == -INFINITY) mx = 0.f;  // empty row: all probabilities 0
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV * 8; ++i) {
    const float d = x[i] - mx;
    const float e = expf(d);  // exp(-inf) = 0 for masked columns
    sum += e;
    x[i] = p.log_softmax ? d : e;
  }
  sum = group_sum<G>(sum, red);
  if (p.log_softmax) {
    const float l = logf(sum);
#pragma unroll
    for (int i = 0; i < MAXV * 8; ++i) x[i] -= l;
  } else {
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
#pragma unroll
    for (int i = 0; i < MAXV * 8; ++i) x[i] *= inv;
  }
  if (active) row_store<T, G, MAXV>(reinterpret_cast<T*>(p.y) + r * p.cols, cols, t, al, x);
}

bool is_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Picks (G, MAXV) for a row length: one warp per row up to 1024 columns, one
// block per row up to 16384.
#define DISC_ROW_DISPATCH(KERNEL, T, cols, rows, stream, ...)                              \
  do {                                                                                     \
    if ((cols) <= 512) {                                                                   \
      KERNEL<T, 32, 2><<<static_cast<unsigned>(((rows) + 7) / 8), kBlock, 0, stream>>>(__VA_ARGS__); \
    } else if ((cols) <= 1024) {                                                           \
      KERNEL<T, 32, 4><<<static_cast<unsigned>(((rows) + 7) / 8), kBlock, 0, stream>>>(__VA_ARGS__); \
    } else if ((cols) <= 4096) {                                                           \
      KERNEL<T, 256, 2><<<static_cast<unsigned>(rows), kBlock, 0, stream>>>(__VA_ARGS__);  \
    } else {                                                                               \
      KERNEL<T, 256, 8><<<static_cast<unsigned>(rows), kBlock, 0, stream>>>(__VA_ARGS__);  \
    }                                                                                      \
  } while (0)

bool row_shape_ok(int64_t rows, int64_t cols, const char** err) {
  if (cols > 16384) {
    if (err) *err = "row kernel: more than 16384 columns is not supported";
    return false;
  }
  if (rows > 0x7fffffff) {
    if (err) *err = "row kernel: too many rows";
    return false;
  }
  return true;
}

int elem_grid(int64_t work_items) {
  int64_t blocks = (work_items + kBlock - 1) / kBlock;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace

cudaError_t quantize_launch(const QuantizeParams& p, cudaStream_t s, const char** err) {
  if (err) *err = nullptr;
  if (p.numel <= 0) return cudaSuccess;
  if (!p.x || !p.q || !p.scale) {
    if (err) *err = "quantize: null operand";
    return cudaErrorInvalidValue;
  }
  const float qmin = static_cast<float>(p.qmin), qmax = static_cast<float>(p.qmax);
  if (p.channels <= 1) {
    const int aligned = is_aligned16(p.x) && is_aligned16(p.q);
    const int grid = elem_grid((p.numel + 15) / 16);
    if (p.in_type == kF32)
      quantize_tensor_kernel<float><<<grid, kBlock, 0, s>>>(reinterpret_cast<const float*>(p.x), p.q,
                                                            p.numel, p.scale, p.zero_point, qmin,
                                                            qmax, aligned);
    else
      quantize_tensor_kernel<__half><<<grid, kBlock, 0, s>>>(reinterpret_cast<const __half*>(p.x),
                                                             p.q, p.numel, p.scale, p.zero_point,
                                                             qmin, qmax, aligned);
  } else {
    const int grid = elem_grid(p.numel);
    const int64_t inner = p.inner > 0 ? p.inner : 1;
    if (p.in_type == kF32)
      quantize_axis_kernel<float><<<grid, kBlock, 0, s>>>(reinterpret_cast<const float*>(p.x), p.q,
                                                          p.numel, p.scale, p.zero_point, p.channels,
                                                          inner, qmin, qmax);
    else
      quantize_axis_kernel<__half><<<grid, kBlock, 0, s>>>(reinterpret_cast<const __half*>(p.x), p.q,
                                                           p.numel, p.scale, p.zero_point,
                                                           p.channels, inner, qmin, qmax);
  }
  return cudaGetLastError();
}

cudaError_t dequantize_launch(const DequantizeParams& p, cudaStream_t s, const char** err) {
  if (err) *err = nullptr;
  if (p.numel <= 0) return cudaSuccess;
  if (!p.q || !p.y || !p.scale) {
    if (err) *err = "dequantize: null operand";
    return cudaErrorInvalidValue;
  }
  const int aligned = is_aligned16(p.q) && is_aligned16(p.y);
  const int64_t ch = p.channels > 1 ? p.channels : 1;
  const int64_t inner = p.inner > 0 ? p.inner : 1;
  const int grid = elem_grid(ch == 1 ? (p.numel + 15) / 16 : p.numel);
  if (p.out_type == kF32)
    dequantize_kernel<float><<<grid, kBlock, 0, s>>>(p.q, reinterpret_cast<float*>(p.y), p.numel,
                                                     p.scale, p.zero_point, ch, inner, aligned);
  else
    dequantize_kernel<__half><<<grid, kBlock, 0, s>>>(p.q, reinterpret_cast<__half*>(p.y), p.numel,
                                                      p.scale, p.zero_point, ch, inner, aligned);
  return cudaGetLastError();
}

cudaError_t dynamic_quantize_launch(const DynQuantParams& p, cudaStream_t s, const char** err) {
  if (err) *err = nullptr;
  if (p.rows <= 0 || p.cols <= 0) return cudaSuccess;
  if (!p.x || !p.q || !p.row_scale) {
    if (err) *err = "dynamic quantize: null operand";
    return cudaErrorInvalidValue;
  }
  if (!row_shape_ok(p.rows, p.cols, err)) return cudaErrorInvalidValue;
  const int aligned = (p.cols % 8 == 0) && is_aligned16(p.x) && ((reinterpret_cast<uintptr_t>(p.q) & 7) == 0);
  if (p.in_type == kF32)
    DISC_ROW_DISPATCH(dynquant_kernel, float, p.cols, p.rows, s, p, aligned);
  else
    DISC_ROW_DISPATCH(dynquant_kernel, __half, p.cols, p.rows, s, p, aligned);
  return cudaGetLastError();
}

cudaError_t norm_launch(const NormParams& p, cudaStream_t s, const char** err) {
  if (err) *err = nullptr;
  if (p.rows <= 0 || p.cols <= 0) return cudaSuccess;
  if (!p.x || !p.gamma || (!p.y && !p.q_out)) {
    if (err) *err = "norm: null operand";
    return cudaErrorInvalidValue;
  }
  if (p.q_out && !p.q_scale && !p.q_row_scale) {
    if (err) *err = "norm: quantized output needs q_scale or q_row_scale";
    return cudaErrorInvalidValue;
  }
  if (!row_shape_ok(p.rows, p.cols, err)) return cudaErrorInvalidValue;
  const int aligned = (p.cols % 8 == 0) && is_aligned16(p.x) && is_aligned16(p.gamma) &&
                      (!p.residual || is_aligned16(p.residual)) && (!p.beta || is_aligned16(p.beta)) &&
                      (!p.y || is_aligned16(p.y)) && (!p.sum_out || is_aligned16(p.sum_out)) &&
                      (!p.q_out || (reinterpret_cast<uintptr_t>(p.q_out) & 7) == 0);
  if (p.type == kF32)
    DISC_ROW_DISPATCH(norm_kernel, float, p.cols, p.rows, s, p, aligned);
  else
    DISC_ROW_DISPATCH(norm_kernel, __half, p.cols, p.rows, s, p, aligned);
  return cudaGetLastError();
}

cudaError_t softmax_launch(const SoftmaxParams& p, cudaStream_t s, const char** err) {
  if (err) *err = nullptr;
  if (p.rows <= 0 || p.cols <= 0) return cudaSuccess;
  if (!p.x || !p.y) {
    if (err) *err = "softmax: null operand";
    return cudaErrorInvalidValue;
  }
  if (!row_shape_ok(p.rows, p.cols, err)) return cudaErrorInvalidValue;
  SoftmaxParams q = p;
  if (q.rows_per_batch <= 0) q.rows_per_batch = q.rows;
  const int aligned = (p.cols % 8 == 0) && is_aligned16(p.x) && is_aligned16(p.y) &&
                      (!p.mask || is_aligned16(p.mask));
  if (p.type == kF32)
    DISC_ROW_DISPATCH(softmax_kernel, float, q.cols, q.rows, s, q, aligned);
  else
    DISC_ROW_DISPATCH(softmax_kernel, __half, q.cols, q.rows, s, q, aligned);
  return cudaGetLastError();
}

}  // namespace disc_b200
