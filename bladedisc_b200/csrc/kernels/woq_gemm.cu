// Weight-only quantized linear for a few rows of activations (see woq_gemm.h).
//
// The work is reading K x N bytes of weights once; everything is arranged around
// that stream, and around the fact that on the SIMT pipes the cost is counted in
// instructions per weight byte (a B200 SM issues about 5.5 per byte at full HBM
// rate):
//   * a block owns a strip of 128 columns and a chunk of k rows.  A lane loads C
//     adjacent bytes of one row (C = 16, 8 or 4: the widest the alignment and the
//     accumulator registers allow), so 128 / C lanes cover the strip's 128-byte
//     row segment and a warp load spans R = C / 4 rows; wide loads keep the
//     address arithmetic at a fraction of an instruction per byte;
//   * no predicates in the loop: rows past K are clamped to the last row (their
//     activations are staged as zero), lanes past N to column 0 (never stored);
//   * the loads of the next group of U warp loads are issued before the current
//     group is consumed, so the memory system never waits for the arithmetic (a
//     variant that streamed through asynchronous copies into a shared-memory ring
//     measured the same from 2 rows on and slower for 1 row, and was dropped);
//   * a byte becomes a float with one byte permute (the byte dropped into the
//     mantissa of 2^23) and one subtraction of the column's (2^23 + zero point),
//     which yields w - zp exactly; the activation comes from shared memory;
//     products and sums are fp32, so a product is exact and the result differs
//     from real arithmetic only by the order of the fp32 sums;
//   * the k range is split over the blocks of a thread-block cluster (up to 8) to
//     fill the GPU.  Lanes that hold different rows of the same columns combine by
//     shuffles, warps through shared memory, blocks of a cluster through
//     distributed shared memory: every block leaves its tile in its own shared
//     memory, and after a cluster barrier each block adds, in rank order, one
//     slice of the tile and applies scale and bias.  No partial sums travel
//     through global memory, nothing depends on scheduling, and there is no flag
//     to wait on (only hardware barriers).
// Per weight byte: 2 (convert) + MT (multiply-add; MT = rows of activations padded
// to 1/2/4/8/16) + about 0.3 (loads, addresses): memory-bound up to 2 rows,
// issue-bound beyond.
#include "woq_gemm.h"

#include "device_info.h"

#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "rowops.h"
#include "sm100_ptx.cuh"

namespace cg = cooperative_groups;

namespace disc_b200 {
namespace {

constexpr int kMaxCluster = 8;  // portable cluster size
constexpr int kStrip = 128;     // columns per block
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

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

template <int WORDS>
struct RawVec;
template <>
struct RawVec<1> {
  using type = uint32_t;
  static __device__ __forceinline__ void split(uint32_t v, uint32_t (&o)[1]) { o[0] = v; }
};
template <>
struct RawVec<2> {
  using type = uint2;
  static __device__ __forceinline__ void split(uint2 v, uint32_t (&o)[2]) { o[0] = v.x; o[1] = v.y; }
};
template <>
struct RawVec<4> {
  using type = uint4;
  static __device__ __forceinline__ void split(uint4 v, uint32_t (&o)[4]) { o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
};

// Bytes per lane and load, and warp loads per group, by rows of activations: the
// accumulators (MT * C) and two groups of raw words (2 * U * C / 4) have to leave
// the compiler room to keep the next group's loads in flight across the arithmetic
// (with 64 accumulators it stopped doing so and exposed the memory latency).
__host__ __device__ constexpr int widest_for(int mt) { return mt <= 2 ? 16 : mt <= 4 ? 8 : 4; }
__host__ __device__ constexpr int group_for(int mt, int c) {
  return c == 16 ? 8 : c == 8 ? 8 : (mt <= 8 ? 16 : 8);
}

constexpr size_t kSmemLimit = 200 * 1024;

struct Plan {
  int mt;       // rows of activations per launch, padded (1, 2, 4, 8, 16)
  int c;        // bytes per lane and load (16, 8 or 4)
  int strips;   // blocks along N
  int cluster;  // blocks along K = cluster size (1, 2, 4, 8)
  int kc;       // k rows per block, a multiple of the rows the block covers per step
  size_t smem;
};

Plan make_plan(int64_t m, int64_t n, int64_t k, int align, int sm_count) {
  Plan pl{};
  pl.mt = m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16;
  pl.c = std::min(widest_for(pl.mt), align);
  pl.strips = static_cast<int>((n + kStrip - 1) / kStrip);
  const int step = kWarps * (pl.c / 4) * group_for(pl.mt, pl.c);  // rows a block covers per step
  // How far to split k: two blocks fit an SM; the time is about (waves of blocks) x (rows per
  // block + a fixed cost worth ~512 rows: launch, staging, the two cluster barriers).
  const int64_t slots = 2 * static_cast<int64_t>(sm_count);
  int best = 1;
  int64_t best_cost = -1;
  for (int cs = 1; cs <= kMaxCluster; cs *= 2) {
    if (cs > 1 && k <= static_cast<int64_t>(cs / 2) * step) break;  // every block keeps at least one step
    const int64_t blocks = static_cast<int64_t>(pl.strips) * cs;
    const int64_t waves = (blocks + slots - 1) / slots;
    const int64_t rows = (k + cs - 1) / cs;
    // fewer blocks than SMs leave SMs idle: count the missing share as extra time
    const int64_t idle = blocks < sm_count ? (sm_count + blocks - 1) / blocks : 1;
    const int64_t cost = waves * (rows + 512) * idle;
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = cs;
    }
  }
  const size_t tile = sizeof(float) * pl.mt * kStrip;
  const size_t red = sizeof(float) * kWarps * pl.mt * kStrip;
  for (;;) {
    int64_t kc = (k + best - 1) / best;
    kc = std::max<int64_t>(step, (kc + step - 1) / step * step);
    pl.cluster = best;
    pl.kc = static_cast<int>(kc);
    pl.smem = tile + std::max(sizeof(float) * pl.mt * static_cast<size_t>(kc), red);
    // a k chunk whose activations do not fit shared memory: split further before giving up rows
    if (pl.smem <= kSmemLimit || best == kMaxCluster || k <= static_cast<int64_t>(best) * step) break;
    best *= 2;
  }
  return pl;
}

// Rows of activations per pass: 16, or fewer when the fp32 copy of a k chunk of that many
// rows would not fit shared memory (K beyond ~25k); 0 if not even one row fits.
int64_t rows_per_pass(int64_t m, int64_t n, int64_t k, int align, int sms) {
  int64_t group = 16;
  while (group > 1 && make_plan(std::min(group, m), n, k, align, sms).smem > kSmemLimit) group /= 2;
  return make_plan(std::min(group, m), n, k, align, sms).smem > kSmemLimit ? 0 : group;
}

template <typename T, int MT, int C>
__global__ void __launch_bounds__(kThreads, 2)
woq_gemm_kernel(WoqGemmParams p, int64_t m0, int kc) {
  constexpr int U = group_for(MT, C);
  constexpr int WORDS = C / 4;
  constexpr int LPR = kStrip / C;  // lanes per row segment
  constexpr int R = 32 / LPR;      // rows per warp load
  constexpr int TILE = MT * kStrip;
  using Vec = typename RawVec<WORDS>::type;
  extern __shared__ __align__(16) float woq_smem[];
  float* tile = woq_smem;        // [MT][128], read by the other blocks of the cluster
  float* xs = woq_smem + TILE;   // [MT][kc]; reused as red [kWarps][MT][128] after the k loop
  float* red = xs;

  cg::cluster_group cluster = cg::this_cluster();
  const int rank = static_cast<int>(cluster.block_rank());   // == blockIdx.y: the cluster spans y
  const int csize = static_cast<int>(cluster.num_blocks());
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int strip = blockIdx.x;
  const int col = (lane % LPR) * C;  // within the strip
  const int sub = lane / LPR;        // row within a warp load
  const int k_begin = rank * kc;
  const int64_t n0 = static_cast<int64_t>(strip) * kStrip + col;
  const bool active = n0 < p.N;  // N is a multiple of C: a lane is wholly inside or outside
  const int rows = static_cast<int>(min(static_cast<int64_t>(MT), p.M - m0));
  const int last_row = static_cast<int>(p.K) - 1;
  const uint8_t* wcol = p.w + (active ? n0 : 0);

  // group of U warp loads starting at row kk0 (relative to the chunk) of this warp
  auto load_group = [&](Vec (&raw)[U], int kk0) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = min(k_begin + kk0 + u * R + sub, last_row);
      raw[u] = __ldcs(reinterpret_cast<const Vec*>(wcol + static_cast<int64_t>(k) * p.ldw));
    }
  };

  // the weights do not depend on the kernel before this one: the first group is on its way
  // while the activations are staged
  Vec cur[U];
  load_group(cur, warp * (R * U));

  grid_dep_launch();
  grid_dep_wait();

  // activations of this k chunk as fp32; zero beyond M and K, so that padding rows and
  // clamped weight rows add nothing
  const T* x = static_cast<const T*>(p.x);
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const T* xr = x + (m0 + m) * p.ldx + k_begin;
    for (int kk = threadIdx.x; kk < kc; kk += kThreads) {
      xs[m * kc + kk] = (m < rows && k_begin + kk <= last_row) ? to_f32<T>(xr[kk]) : 0.f;
    }
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
  for (int kk0 = warp * (R * U); kk0 < kc; kk0 += kWarps * R * U) {
    Vec next[U];
    if (kk0 + kWarps * R * U < kc) load_group(next, kk0 + kWarps * R * U);  // warp-uniform
    const float* xrow = xs + kk0 + sub;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      uint32_t words[WORDS];
      RawVec<WORDS>::split(cur[u], words);
      float wv[C];
#pragma unroll
      for (int j = 0; j < WORDS; ++j) {
        wv[4 * j + 0] = byte_plus_magic<0>(words[j]) - zpm[4 * j + 0];
        wv[4 * j + 1] = byte_plus_magic<1>(words[j]) - zpm[4 * j + 1];
        wv[4 * j + 2] = byte_plus_magic<2>(words[j]) - zpm[4 * j + 2];
        wv[4 * j + 3] = byte_plus_magic<3>(words[j]) - zpm[4 * j + 3];
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float xv = xrow[m * kc + u * R];
#pragma unroll
        for (int c = 0; c < C; ++c) acc[m][c] = fmaf(xv, wv[c], acc[m][c]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) cur[u] = next[u];
  }

  // lanes that hold other rows of the same columns -> the lanes of the first row
  if constexpr (R > 1) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
      for (int c = 0; c < C; ++c) {
#pragma unroll
        for (int o = LPR; o < 32; o <<= 1) acc[m][c] += __shfl_xor_sync(0xffffffffu, acc[m][c], o);
      }
    }
  }
  // warps -> block (the activations are no longer needed: their space takes the partials)
  __syncthreads();
  if (sub == 0) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float* dst = red + (warp * MT + m) * kStrip + col;
#pragma unroll
      for (int c = 0; c < C; c += 4) {
        *reinterpret_cast<float4*>(dst + c) = make_float4(acc[m][c], acc[m][c + 1], acc[m][c + 2], acc[m][c + 3]);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < TILE; i += kThreads) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) v += red[w * TILE + i];
    tile[i] = v;
  }

  // blocks -> result: every block adds its slice of the tile over the cluster, in rank order
  cluster.sync();
  const T* scale = static_cast<const T*>(p.scale);
  const T* bias = static_cast<const T*>(p.bias);
  T* out = static_cast<T*>(p.out);
  const int slice = TILE / csize;  // csize is a power of two <= 8, TILE a multiple of 128
  for (int i = rank * slice + threadIdx.x; i < (rank + 1) * slice; i += kThreads) {
    const int m = i / kStrip;
    const int64_t n = static_cast<int64_t>(strip) * kStrip + (i - m * kStrip);
    float v = 0.f;
    for (int j = 0; j < csize; ++j) v += cluster.map_shared_rank(tile, j)[i];
    if (m < rows && n < p.N) {
      v = v * to_f32<T>(scale[n]) + (bias ? to_f32<T>(bias[n]) : 0.f);
      out[(m0 + m) * p.ldo + n] = from_f32<T>(v);
    }
  }
  cluster.sync();  // no block leaves while its tile may still be read
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

int sm_count() { return device_sm_count(); }

template <typename T, int MT, int C>
cudaError_t launch_tile(const WoqGemmParams& p, int64_t m0, const Plan& pl, cudaStream_t s) {
  auto kern = woq_gemm_kernel<T, MT, C>;
  // the attribute belongs to the function on the current device: set on every launch (cheap), never cached
  cudaError_t st = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemLimit));
  if (st != cudaSuccess) return st;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pl.strips, pl.cluster);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = s;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 1;
  attrs[0].val.clusterDim.y = pl.cluster;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kern, p, m0, pl.kc);
}

template <typename T, int MT>
cudaError_t launch_mt(const WoqGemmParams& p, int64_t m0, const Plan& pl, cudaStream_t s) {
  if constexpr (widest_for(MT) >= 16) {
    if (pl.c == 16) return launch_tile<T, MT, 16>(p, m0, pl, s);
  }
  if constexpr (widest_for(MT) >= 8) {
    if (pl.c == 8) return launch_tile<T, MT, 8>(p, m0, pl, s);
  }
  return launch_tile<T, MT, 4>(p, m0, pl, s);
}

template <typename T>
cudaError_t launch_typed(const WoqGemmParams& p, cudaStream_t s, const char** err) {
  int align = 16;  // bytes a lane may load at once: columns, row pitch and base all multiples of it
  while (align >= 4 && (p.N % align != 0 || p.ldw % align != 0 || reinterpret_cast<uintptr_t>(p.w) % align != 0)) {
    align /= 2;
  }
  if (p.K == 0 || align < 4 || p.K > (int64_t{1} << 30)) {
    if (p.M > 65535) {
      *err = "weight-only qgemm: more than 65535 rows with a weight matrix that is not 4-byte aligned";
      return cudaErrorInvalidValue;
    }
    return launch_dependent(woq_gemm_simple_kernel<T>, dim3(static_cast<unsigned>((p.N + 255) / 256),
                                                           static_cast<unsigned>(p.M)),
                            dim3(256), 0, s, p);
  }
  // more rows than one pass takes: a group at a time, the weights re-read for each group
  const int64_t group = rows_per_pass(p.M, p.N, p.K, align, sm_count());
  if (group == 0) {
    *err = "weight-only qgemm: K too large for the shared-memory staging of the activations";
    return cudaErrorInvalidValue;
  }
  for (int64_t m0 = 0; m0 < p.M; m0 += group) {
    const int64_t rows = std::min<int64_t>(group, p.M - m0);
    const Plan pl = make_plan(rows, p.N, p.K, align, sm_count());
    cudaError_t st;
    switch (pl.mt) {
      case 1: st = launch_mt<T, 1>(p, m0, pl, s); break;
      case 2: st = launch_mt<T, 2>(p, m0, pl, s); break;
      case 4: st = launch_mt<T, 4>(p, m0, pl, s); break;
      case 8: st = launch_mt<T, 8>(p, m0, pl, s); break;
      default: st = launch_mt<T, 16>(p, m0, pl, s); break;
    }
    if (st != cudaSuccess) return st;
  }
  return cudaSuccess;
}

}  // namespace

int woq_gemm_plan_describe(int64_t m, int64_t n, int64_t k, int align, int sm_count, int64_t out7[7]) {
  if (m <= 0 || n <= 0 || k <= 0 || (align != 4 && align != 8 && align != 16) || sm_count <= 0) return 1;
  const int64_t group = rows_per_pass(m, n, k, align, sm_count);
  if (group == 0) return 2;
  const Plan pl = make_plan(std::min(group, m), n, k, align, sm_count);
  out7[0] = group;
  out7[1] = pl.mt;
  out7[2] = pl.c;
  out7[3] = pl.strips;
  out7[4] = pl.cluster;
  out7[5] = pl.kc;
  out7[6] = static_cast<int64_t>(pl.smem);
  return 0;
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
  if (p.path == kWoqPathTensor ||
      (p.path == kWoqPathAuto && p.type == kF16 && p.M >= kWoqTensorMinRows && woq_gemm_tc_usable(p))) {
    return woq_gemm_tc_launch(p, s, e);
  }
  if (p.type == kF16) return launch_typed<__half>(p, s, e);
  if (p.type == kF32) return launch_typed<float>(p, s, e);
  *e = "weight-only qgemm: element type must be f32 or f16";
  return cudaErrorInvalidValue;
}

}  // namespace disc_b200
