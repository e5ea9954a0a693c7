// Weight-only quantized linear for a few rows of activations (see woq_gemm.h).
//
// The work is reading K x N bytes of weights once; everything is arranged around
// that stream:
//   * a block owns a strip of 32*C columns and a chunk of k rows; its 8 warps take
//     interleaved groups of U rows, every lane C adjacent columns, so a warp reads
//     whole 32*C-byte row segments and has U of them in flight per lane;
//   * a byte becomes a float with one byte permute (the byte dropped into the
//     mantissa of 2^23) and one subtraction of the column's (2^23 + zero point),
//     which yields w - zp exactly; the activation comes from shared memory as a
//     warp broadcast; products and sums are fp32, so a product is exact and the
//     result differs from real arithmetic only by the order of the fp32 sums;
//   * warps of a block reduce through shared memory; blocks that share a strip
//     (split over k to fill the GPU) leave fp32 partials in scratch and the last
//     one to arrive adds them in k order and applies scale and bias, so the
//     result does not depend on scheduling.
// Instruction budget per weight byte: 2 + MT (MT = rows of activations, padded to
// 1/2/4/8/16), against about 5.5 per byte that a B200 SM can issue at full HBM
// rate: memory-bound up to 4 rows, issue-bound beyond.
#include "woq_gemm.h"

#include <cuda_fp16.h>

#include <algorithm>

#include "rowops.h"
#include "sm100_ptx.cuh"

namespace disc_b200 {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int64_t kCounterBytes = 16 * 1024;
constexpr int kMaxStrips = static_cast<int>(kCounterBytes / sizeof(int));

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// 2^23 + byte `i` of `word`, exactly.
template <int I>
__device__ __forceinline__ float byte_plus_magic(uint32_t word) {
  return __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7650u | I));
}

struct Plan {
  int mt;       // rows of activations per launch, padded (1, 2, 4, 8, 16)
  int c;        // columns per lane (8 or 4)
  int u;        // rows in flight per lane
  int strips;   // blocks along N
  int ksplit;   // blocks along K
  int kc;       // k rows per block, a multiple of kWarps * u
  bool vec;     // the vector kernel applies (alignment), else the simple kernel
  size_t smem;
  int64_t ws_bytes;
};

Plan make_plan(int64_t m, int64_t n, int64_t k, int sm_count) {
  Plan pl{};
  pl.mt = m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16;
  pl.c = pl.mt <= 4 ? 8 : 4;
  pl.u = pl.mt <= 4 ? 8 : 16;
  const int strip_w = 32 * pl.c;
  pl.strips = static_cast<int>((n + strip_w - 1) / strip_w);
  const int step = kWarps * pl.u;
  const int64_t target = static_cast<int64_t>(sm_count) * 3;
  int64_t ks = std::max<int64_t>(1, (target + pl.strips - 1) / pl.strips);
  ks = std::min<int64_t>(ks, (k + step - 1) / step);
  int64_t kc = (k + ks - 1) / ks;
  kc = (kc + step - 1) / step * step;
  pl.kc = static_cast<int>(kc);
  pl.ksplit = static_cast<int>((k + kc - 1) / kc);
  pl.smem = sizeof(float) * (static_cast<size_t>(pl.mt) * pl.kc + static_cast<size_t>(kWarps) * pl.mt * strip_w);
  pl.ws_bytes = kCounterBytes +
                (pl.ksplit > 1 ? static_cast<int64_t>(pl.ksplit) * pl.strips * pl.mt * strip_w * 4 : 0);
  return pl;
}

template <typename T, int MT, int C, int U>
__global__ void __launch_bounds__(kThreads)
woq_gemm_kernel(WoqGemmParams p, int64_t m0, int kc, int ksplit) {
  constexpr int STRIP = 32 * C;
  constexpr int WORDS = C / 4;
  extern __shared__ __align__(16) float woq_smem[];
  float* xs = woq_smem;                                  // [MT][kc]
  float* red = woq_smem + static_cast<size_t>(MT) * kc;  // [kWarps][MT][STRIP]
  __shared__ int last_block;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int strip = blockIdx.x;
  const int ks = blockIdx.y;
  const int64_t k_begin = static_cast<int64_t>(ks) * kc;
  const int64_t n0 = static_cast<int64_t>(strip) * STRIP + lane * C;
  const bool active = n0 < p.N;  // N is a multiple of C: a lane is wholly inside or outside
  const int rows = static_cast<int>(min(static_cast<int64_t>(MT), p.M - m0));

  grid_dep_launch();
  grid_dep_wait();

  // activations of this k chunk as fp32; zero beyond M and K, so that padding rows and
  // the tail of the last chunk add nothing
  const T* x = static_cast<const T*>(p.x);
  for (int i = threadIdx.x; i < MT * kc; i += kThreads) {
    const int m = i / kc;
    const int64_t k = k_begin + (i - m * kc);
    xs[i] = (m < rows && k < p.K) ? to_f32<T>(x[(m0 + m) * p.ldx + k]) : 0.f;
  }
  float zpm[C];
#pragma unroll
  for (int c = 0; c < C; ++c) {
    zpm[c] = 8388608.f + ((active && p.zp) ? static_cast<float>(__ldg(p.zp + n0 + c)) : 0.f);
  }
  __syncthreads();

  float acc[MT][C];
#pragma unroll
  for (int m = 0; m < MT; ++m) {
#pragma unroll
    for (int c = 0; c < C; ++c) acc[m][c] = 0.f;
  }
  const uint8_t* wcol = p.w + n0;
  for (int kk0 = warp * U; kk0 < kc; kk0 += kWarps * U) {
    uint32_t raw[U][WORDS];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t k = k_begin + kk0 + u;
      if (active && k < p.K) {
        if constexpr (WORDS == 2) {
          const uint2 v = __ldcs(reinterpret_cast<const uint2*>(wcol + k * p.ldw));
          raw[u][0] = v.x;
          raw[u][1] = v.y;
        } else {
          raw[u][0] = __ldcs(reinterpret_cast<const uint32_t*>(wcol + k * p.ldw));
        }
      } else {
#pragma unroll
        for (int j = 0; j < WORDS; ++j) raw[u][j] = 0u;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float wv[C];
#pragma unroll
      for (int j = 0; j < WORDS; ++j) {
        wv[4 * j + 0] = byte_plus_magic<0>(raw[u][j]) - zpm[4 * j + 0];
        wv[4 * j + 1] = byte_plus_magic<1>(raw[u][j]) - zpm[4 * j + 1];
        wv[4 * j + 2] = byte_plus_magic<2>(raw[u][j]) - zpm[4 * j + 2];
        wv[4 * j + 3] = byte_plus_magic<3>(raw[u][j]) - zpm[4 * j + 3];
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float xv = xs[m * kc + kk0 + u];
#pragma unroll
        for (int c = 0; c < C; ++c) acc[m][c] = fmaf(xv, wv[c], acc[m][c]);
      }
    }
  }

  // warps -> block
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    float* dst = red + (static_cast<size_t>(warp) * MT + m) * STRIP + lane * C;
#pragma unroll
    for (int c = 0; c < C; c += 4) {
      *reinterpret_cast<float4*>(dst + c) = make_float4(acc[m][c], acc[m][c + 1], acc[m][c + 2], acc[m][c + 3]);
    }
  }
  __syncthreads();

  const T* scale = static_cast<const T*>(p.scale);
  const T* bias = static_cast<const T*>(p.bias);
  T* out = static_cast<T*>(p.out);
  float* partials = reinterpret_cast<float*>(static_cast<uint8_t*>(p.ws) + kCounterBytes);
  const size_t tile = static_cast<size_t>(MT) * STRIP;
  float* mine = partials + (static_cast<size_t>(ks) * gridDim.x + strip) * tile;
  for (int i = threadIdx.x; i < MT * STRIP; i += kThreads) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) v += red[static_cast<size_t>(w) * tile + i];
    if (ksplit > 1) {
      mine[i] = v;
    } else {
      const int m = i / STRIP;
      const int64_t n = static_cast<int64_t>(strip) * STRIP + (i - m * STRIP);
      if (m < rows && n < p.N) {
        v = v * to_f32<T>(scale[n]) + (bias ? to_f32<T>(bias[n]) : 0.f);
        out[(m0 + m) * p.ldo + n] = from_f32<T>(v);
      }
    }
  }
  if (ksplit == 1) return;

  // blocks of a strip -> result: the last block to arrive adds the partials in k order
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = static_cast<int*>(p.ws) + strip;
    const int before = atomicAdd(counter, 1);
    last_block = before == ksplit - 1;
    if (last_block) atomicExch(counter, 0);  // everyone has arrived: leave the counter as it was found
  }
  __syncthreads();
  if (!last_block) return;
  __threadfence();
  for (int i = threadIdx.x; i < MT * STRIP; i += kThreads) {
    const int m = i / STRIP;
    const int64_t n = static_cast<int64_t>(strip) * STRIP + (i - m * STRIP);
    if (m >= rows || n >= p.N) continue;
    float v = 0.f;
    for (int j = 0; j < ksplit; ++j) v += __ldcg(partials + (static_cast<size_t>(j) * gridDim.x + strip) * tile + i);
    v = v * to_f32<T>(scale[n]) + (bias ? to_f32<T>(bias[n]) : 0.f);
    out[(m0 + m) * p.ldo + n] = from_f32<T>(v);
  }
}

// Any shape and alignment: one thread per output element, k in order.
template <typename T>
__global__ void __launch_bounds__(256) woq_gemm_simple_kernel(WoqGemmParams p) {
  grid_dep_launch();
  grid_dep_wait();
  const int64_t n = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t m = blockIdx.y;
  if (n >= p.N) return;
  const T* x = static_cast<const T*>(p.x) + m * p.ldx;
  const float zp = p.zp ? static_cast<float>(p.zp[n]) : 0.f;
  float acc = 0.f;
  for (int64_t k = 0; k < p.K; ++k) {
    acc = fmaf(to_f32<T>(x[k]), static_cast<float>(p.w[k * p.ldw + n]) - zp, acc);
  }
  const T* scale = static_cast<const T*>(p.scale);
  const T* bias = static_cast<const T*>(p.bias);
  acc = acc * to_f32<T>(scale[n]) + (bias ? to_f32<T>(bias[n]) : 0.f);
  static_cast<T*>(p.out)[m * p.ldo + n] = from_f32<T>(acc);
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      n = 148;
    }
  }
  return n;
}

template <typename T, int MT, int C, int U>
cudaError_t launch_tile(const WoqGemmParams& p, int64_t m0, const Plan& pl, cudaStream_t s) {
  auto kern = woq_gemm_kernel<T, MT, C, U>;
  static bool configured = false;  // per instantiation; the attribute is per function, set once
  if (!configured) {
    cudaError_t st = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (st != cudaSuccess) return st;
    configured = true;
  }
  return launch_dependent(kern, dim3(pl.strips, pl.ksplit), dim3(kThreads), pl.smem, s, p, m0, pl.kc, pl.ksplit);
}

template <typename T>
cudaError_t launch_typed(const WoqGemmParams& p, cudaStream_t s, const char** err) {
  const bool aligned8 = p.N % 8 == 0 && p.ldw % 8 == 0 && reinterpret_cast<uintptr_t>(p.w) % 8 == 0;
  const bool aligned4 = p.N % 4 == 0 && p.ldw % 4 == 0 && reinterpret_cast<uintptr_t>(p.w) % 4 == 0;
  if (p.K == 0 || !aligned4 || (p.M <= 4 && !aligned8)) {
    if (p.M > 65535) {
      *err = "weight-only qgemm: more than 65535 rows with a weight matrix that is not 8-byte aligned";
      return cudaErrorInvalidValue;
    }
    return launch_dependent(woq_gemm_simple_kernel<T>, dim3(static_cast<unsigned>((p.N + 255) / 256),
                                                           static_cast<unsigned>(p.M)),
                            dim3(256), 0, s, p);
  }
  // more than 16 rows: 16 at a time, the weights re-read for each group
  for (int64_t m0 = 0; m0 < p.M; m0 += 16) {
    const int64_t rows = std::min<int64_t>(16, p.M - m0);
    const Plan pl = make_plan(rows, p.N, p.K, sm_count());
    if (pl.strips > kMaxStrips) {
      *err = "weight-only qgemm: N too large for the arrival counters";
      return cudaErrorInvalidValue;
    }
    if (pl.smem > 160 * 1024) {
      *err = "weight-only qgemm: k chunk does not fit shared memory";
      return cudaErrorInvalidValue;
    }
    if (pl.ws_bytes > kCounterBytes && (!p.ws || p.ws_bytes < pl.ws_bytes)) {
      *err = "weight-only qgemm: scratch missing or smaller than woq_gemm_scratch_bytes";
      return cudaErrorInvalidValue;
    }
    cudaError_t st;
    switch (pl.mt) {
      case 1: st = launch_tile<T, 1, 8, 8>(p, m0, pl, s); break;
      case 2: st = launch_tile<T, 2, 8, 8>(p, m0, pl, s); break;
      case 4: st = launch_tile<T, 4, 8, 8>(p, m0, pl, s); break;
      case 8: st = launch_tile<T, 8, 4, 16>(p, m0, pl, s); break;
      default: st = launch_tile<T, 16, 4, 16>(p, m0, pl, s); break;
    }
    if (st != cudaSuccess) return st;
  }
  return cudaSuccess;
}

}  // namespace

int64_t woq_gemm_scratch_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return kCounterBytes;
  // the device's SM count is not known to a caller without a GPU context: size for the
  // largest split any B200-class part would choose
  int64_t worst = kCounterBytes;
  for (int64_t rows : {std::min<int64_t>(M, 16), M % 16 == 0 ? int64_t{16} : M % 16}) {
    for (int sms : {148, 160, 192}) worst = std::max(worst, make_plan(rows, N, K, sms).ws_bytes);
  }
  return worst;
}

cudaError_t woq_gemm_launch(const WoqGemmParams& p, cudaStream_t s, const char** err) {
  static const char* none = "";
  const char** e = err ? err : &none;
  if (p.M < 0 || p.N < 0 || p.K < 0) {
    *e = "weight-only qgemm: negative size";
    return cudaErrorInvalidValue;
  }
  if (p.M == 0 || p.N == 0) return cudaSuccess;
  if (!p.x || !p.w || !p.scale || !p.out) {
    if (p.K == 0 && p.scale && p.out) {
      // no k: the result is the bias (or zero); the simple kernel handles it
    } else {
      *e = "weight-only qgemm: null operand";
      return cudaErrorInvalidValue;
    }
  }
  if (p.ldx < p.K || p.ldw < p.N || p.ldo < p.N) {
    *e = "weight-only qgemm: row stride smaller than the row";
    return cudaErrorInvalidValue;
  }
  if (p.type == kF16) return launch_typed<__half>(p, s, e);
  if (p.type == kF32) return launch_typed<float>(p, s, e);
  *e = "weight-only qgemm: element type must be f32 or f16";
  return cudaErrorInvalidValue;
}

}  // namespace disc_b200
