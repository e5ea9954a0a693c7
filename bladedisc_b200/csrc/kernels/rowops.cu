// Bandwidth-bound kernels of the quantized path, hand-written for sm_100a.
//
// In the reference these are compiler-generated: quantize / dequantize are
// lowered to elementwise mhlo (tao_compiler/mlir/disc/transforms/
// disc_lower_quantize_and_dequantize.cc:36-139) and codegen'd as kLoop
// kernels; LayerNorm / softmax become kRowReduction / kStitch kernels with one
// of two schedules, one warp per row or one block per row
// (tao_compiler/mlir/disc/transforms/lhlo_legalize_roots_to_loops.cc:1263-1289,
// 1678-1716; choice at disc_specialize_fusion_with_speculation.cc:393-452).
//
// Here a row is read once with 16-byte loads and written once.  What decides
// the speed of such kernels on B200 is how many bytes each SM keeps in flight
// (about 6.5 TB/s x 1 us / 148 SMs = 45 KB at the least), so:
//   * rows stay in registers in their storage type (packed 16-byte vectors),
//     converted to fp32 on the fly in each pass, which halves the registers a
//     fp16 row needs and lets more warps be resident;
//   * a group of G threads (8, 16 or 32 lanes of a warp, or a 256-thread
//     block for long rows) works on R rows at once, so that R x NV loads per
//     thread are issued before the first reduction starts;
//   * per-column parameters (gamma, beta) are fetched per vector from L1/L2
//     instead of being kept for the whole row.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <float.h>

#include "device_info.h"
#include "rowops.h"
#include "sm100_ptx.cuh"

namespace disc_b200 {
namespace {

constexpr int kBlock = 256;
constexpr float kRoundMagic = 12582912.f;  // 1.5 * 2^23: (x + m) - m rounds half-to-even for |x| < 2^22

int sm_count() { return device_sm_count(); }

// x / s wherever the exact IEEE quotient decides the integer result.  The
// product with the (correctly rounded) reciprocal is within 2 ulp of the true
// quotient; only a quotient that close to a rounding tie (k + 0.5) can round to
// a different integer, and anything beyond +-1024 saturates whatever its last
// bits are.  So ties within 1e-3 (and small magnitudes only) take the real
// division, kept out of line because it is rare and long: unrolled copies of
// it were what overflowed the instruction cache.
__device__ __noinline__ float slow_div(float x, float s) { return __fdiv_rn(x, s); }

struct Divisor {
  float s, inv;
  bool fast;
};
__device__ __forceinline__ Divisor make_divisor(float s) {
  Divisor d;
  d.s = s;
  d.inv = __frcp_rn(s);
  const float a = fabsf(s);
  d.fast = a > 1e-15f && a < 1e15f;
  return d;
}
__device__ __forceinline__ float div_exact_for_rounding(float x, const Divisor& d) {
  if (!d.fast) return slow_div(x, d.s);
  float q = x * d.inv;
  const float frac = fabsf(q - ((q + kRoundMagic) - kRoundMagic));
  if (fabsf(frac - 0.5f) < 1e-3f && fabsf(q) < 1024.f) q = slow_div(x, d.s);
  return q;
}

// divide, add zero point, round half to even, clamp: the order of the reference
// (clamping to integer bounds before rounding gives the same result as after).
// Returns the value still carrying the rounding constant: its low byte is the int8.
__device__ __forceinline__ float quant_biased(float x, const Divisor& d, float zp, float qmin, float qmax) {
  const float t = __fadd_rn(div_exact_for_rounding(x, d), zp);
  return fminf(fmaxf(t, qmin), qmax) + kRoundMagic;
}
__device__ __forceinline__ int8_t quant_one(float x, const Divisor& d, float zp, float qmin, float qmax) {
  return static_cast<int8_t>(__float_as_uint(quant_biased(x, d, zp, qmin, qmax)) & 0xffu);
}
// Four values from quant_biased -> packed bytes.
__device__ __forceinline__ uint32_t pack4(float a, float b, float c, float d) {
  const uint32_t ab = __byte_perm(__float_as_uint(a), __float_as_uint(b), 0x0040);
  const uint32_t cd = __byte_perm(__float_as_uint(c), __float_as_uint(d), 0x0040);
  return __byte_perm(ab, cd, 0x5410);
}

// ------------------------------------------------------------ 16-byte vectors
template <typename T>
struct VecT;
template <>
struct VecT<float> {
  static constexpr int kElems = 4;
  static __device__ __forceinline__ float get(const uint4& v, int j) {
    return __uint_as_float(j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w)));
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ float load1(const float* p) { return *p; }
  static __device__ __forceinline__ void store1(float* p, float v) { *p = v; }
  static __device__ __forceinline__ float round_to_storage(float v) { return v; }
};
template <>
struct VecT<__half> {
  static constexpr int kElems = 8;
  static __device__ __forceinline__ float get(const uint4& v, int j) {
    const uint32_t w = (j >> 1) == 0 ? v.x : ((j >> 1) == 1 ? v.y : ((j >> 1) == 2 ? v.z : v.w));
    const __half2 h = *reinterpret_cast<const __half2*>(&w);
    return (j & 1) ? __high2float(h) : __low2float(h);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint4 u;
    __half2 h0 = __floats2half2_rn(f[0], f[1]), h1 = __floats2half2_rn(f[2], f[3]);
    __half2 h2 = __floats2half2_rn(f[4], f[5]), h3 = __floats2half2_rn(f[6], f[7]);
    u.x = *reinterpret_cast<uint32_t*>(&h0);
    u.y = *reinterpret_cast<uint32_t*>(&h1);
    u.z = *reinterpret_cast<uint32_t*>(&h2);
    u.w = *reinterpret_cast<uint32_t*>(&h3);
    return u;
  }
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    }
  }
  static __device__ __forceinline__ float load1(const __half* p) { return __half2float(*p); }
  static __device__ __forceinline__ void store1(__half* p, float v) { *p = __float2half_rn(v); }
  static __device__ __forceinline__ float round_to_storage(float v) { return __half2float(__float2half_rn(v)); }
};

// Vector `v` (16 bytes) of a row of `cols` elements; elements past the row read as `fill`.
template <typename T>
__device__ __forceinline__ uint4 load_vec(const T* row, int cols, int v, bool aligned, float fill) {
  constexpr int E = VecT<T>::kElems;
  const int base = v * E;
  if (aligned) {
    if (base < cols) return *reinterpret_cast<const uint4*>(row + base);
    float f[E];
#pragma unroll
    for (int j = 0; j < E; ++j) f[j] = fill;
    return VecT<T>::pack(f);
  }
  float f[E];
#pragma unroll
  for (int j = 0; j < E; ++j) f[j] = (base + j < cols) ? VecT<T>::load1(row + base + j) : fill;
  return VecT<T>::pack(f);
}
template <typename T>
__device__ __forceinline__ void store_vec(T* row, int cols, int v, bool aligned, const uint4& u) {
  constexpr int E = VecT<T>::kElems;
  const int base = v * E;
  if (base >= cols) return;
  if (aligned) {
    *reinterpret_cast<uint4*>(row + base) = u;
  } else {
#pragma unroll
    for (int j = 0; j < E; ++j)
      if (base + j < cols) VecT<T>::store1(row + base + j, VecT<T>::get(u, j));
  }
}
// E int8 values of vector v, as produced by quant_biased.
template <int E>
__device__ __forceinline__ void store_q(int8_t* row, int cols, int v, bool aligned, const float* q) {
  const int base = v * E;
  if (base >= cols) return;
  if (aligned) {
    if (E == 8) {
      *reinterpret_cast<uint2*>(row + base) = make_uint2(pack4(q[0], q[1], q[2], q[3]), pack4(q[4], q[5], q[6], q[7]));
    } else {
      *reinterpret_cast<uint32_t*>(row + base) = pack4(q[0], q[1], q[2], q[3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < E; ++j)
      if (base + j < cols) row[base + j] = static_cast<int8_t>(__float_as_uint(q[j]) & 0xffu);
  }
}

// ------------------------------------------------------ group reductions
// G lanes of a warp (8, 16, 32) reduce with shuffles; G = 256 is a whole block
// and goes through shared memory.  R values are reduced together.
template <int G, int R, bool IS_MAX>
__device__ __forceinline__ void group_reduce(float (&v)[R], float* red) {
  constexpr int kLanes = G < 32 ? G : 32;
#pragma unroll
  for (int o = kLanes / 2; o > 0; o >>= 1) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float other = __shfl_xor_sync(0xffffffffu, v[r], o);
      v[r] = IS_MAX ? fmaxf(v[r], other) : v[r] + other;
    }
  }
  if (G > 32) {
    // groups of 2, 4 or 8 warps: partials meet in shared memory; every group of the
    // block runs the same sequence, so block-wide barriers serve all of them
    constexpr int kWarps = G > 32 ? G / 32 : 1;
    const int w = threadIdx.x >> 5;
    const int grp = w / kWarps;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) red[r * 8 + w] = v[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float a = red[r * 8 + grp * kWarps];
#pragma unroll
      for (int i = 1; i < kWarps; ++i)
        a = IS_MAX ? fmaxf(a, red[r * 8 + grp * kWarps + i]) : a + red[r * 8 + grp * kWarps + i];
      v[r] = a;
    }
  }
}

// ------------------------------------------------------ elementwise quantize
template <typename T>
__global__ void __launch_bounds__(kBlock)
quantize_tensor_kernel(const T* __restrict__ x, int8_t* __restrict__ q, int64_t numel,
                       const float* __restrict__ scale, const int32_t* __restrict__ zero_point,
                       float qmin, float qmax, int aligned) {
  constexpr int E = VecT<T>::kElems;
  constexpr int NVEC = 16 / E;  // input vectors per 16 output bytes
  const Divisor d = make_divisor(__ldg(scale));
  const float zp = zero_point ? static_cast<float>(__ldg(zero_point)) : 0.f;
  const int64_t nchunk = aligned ? numel / 16 : 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  for (int64_t c = tid; c < nchunk; c += stride) {
    uint4 in[NVEC];
#pragma unroll
    for (int i = 0; i < NVEC; ++i) in[i] = *reinterpret_cast<const uint4*>(x + c * 16 + i * E);
    float o[16];
#pragma unroll
    for (int i = 0; i < NVEC; ++i)
#pragma unroll
      for (int j = 0; j < E; ++j) o[i * E + j] = quant_biased(VecT<T>::get(in[i], j), d, zp, qmin, qmax);
    *reinterpret_cast<uint4*>(q + c * 16) =
        make_uint4(pack4(o[0], o[1], o[2], o[3]), pack4(o[4], o[5], o[6], o[7]),
                   pack4(o[8], o[9], o[10], o[11]), pack4(o[12], o[13], o[14], o[15]));
  }
  for (int64_t i = nchunk * 16 + tid; i < numel; i += stride) {
    q[i] = quant_one(VecT<T>::load1(x + i), d, zp, qmin, qmax);
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
    q[i] = quant_one(VecT<T>::load1(x + i), make_divisor(__ldg(scale + c)), zp, qmin, qmax);
  }
}

template <typename T>
__global__ void __launch_bounds__(kBlock)
dequantize_kernel(const int8_t* __restrict__ q, T* __restrict__ y, int64_t numel,
                  const float* __restrict__ scale, const int32_t* __restrict__ zero_point,
                  int64_t channels, int64_t inner, int aligned) {
  constexpr int E = VecT<T>::kElems;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (channels == 1) {
    const float s = __ldg(scale);
    const int zp = zero_point ? __ldg(zero_point) : 0;
    const int64_t nchunk = aligned ? numel / 16 : 0;
    for (int64_t c = tid; c < nchunk; c += stride) {
      const uint4 u = *reinterpret_cast<const uint4*>(q + c * 16);
      const int8_t* b = reinterpret_cast<const int8_t*>(&u);
      float f[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = __fmul_rn(static_cast<float>(static_cast<int>(b[i]) - zp), s);
#pragma unroll
      for (int i = 0; i < 16 / E; ++i) *reinterpret_cast<uint4*>(y + c * 16 + i * E) = VecT<T>::pack(f + i * E);
    }
    for (int64_t i = nchunk * 16 + tid; i < numel; i += stride) {
      VecT<T>::store1(y + i, __fmul_rn(static_cast<float>(static_cast<int>(q[i]) - zp), s));
    }
  } else {
    for (int64_t i = tid; i < numel; i += stride) {
      const int64_t c = (i / inner) % channels;
      const int zp = zero_point ? __ldg(zero_point + c) : 0;
      VecT<T>::store1(y + i, __fmul_rn(static_cast<float>(static_cast<int>(q[i]) - zp), __ldg(scale + c)));
    }
  }
}

// ------------------------------------------------------------- row kernels
// Thread t of a group owns vectors t, t + G, ... (NV of them) of each of its R rows.
template <int G, int R>
struct RowIndex {
  int t;
  int64_t row0;  // first of the R rows of this group
  __device__ __forceinline__ RowIndex() : RowIndex(blockIdx.x) {}
  __device__ __forceinline__ explicit RowIndex(int64_t blk) {
    t = threadIdx.x % G;
    row0 = (blk * (kBlock / G) + threadIdx.x / G) * R;
  }
};
// Blocks of work for `rows` rows: the row kernels walk them with a stride of
// gridDim.x (a grid sized to what the GPU holds at once) and fetch the next
// block's rows into registers before they work on the current one, so that
// loads stay in flight while a warp computes.
template <int G, int R>
__device__ __forceinline__ int64_t row_blocks(int64_t rows) {
  constexpr int64_t kRowsPerBlock = static_cast<int64_t>(kBlock / G) * R;
  return (rows + kRowsPerBlock - 1) / kRowsPerBlock;
}

// The reciprocal form for quantization fused behind another row operation (zero
// point 0, int8 range): one fused multiply-add forms x * (1 / s) under the
// rounding constant -- a single rounding, to nearest even, so a quotient that is
// exactly a tie (power-of-two scales on fp16 data produce many) goes where the
// division sends it -- and the clamp works on the biased value.  Three
// instructions per value against seven with the tie test above.  The rounded
// reciprocal instead of the division can move a value whose quotient lies
// within an ulp of a rounding tie to the neighbouring level, never further.
struct RecipQuant {
  float inv;
};
__device__ __forceinline__ RecipQuant make_recip_quant(float s) {
  RecipQuant u;
  u.inv = __frcp_rn(s);
  return u;
}
__device__ __forceinline__ float quant_recip(float x, const RecipQuant& u) {
  return fminf(fmaxf(__fmaf_rn(x, u.inv, kRoundMagic), kRoundMagic - 128.f), kRoundMagic + 127.f);
}
template <int E>
__device__ __forceinline__ void quant_vec_recip(const float* y, const RecipQuant& u, float* q) {
#pragma unroll
  for (int j = 0; j < E; ++j) q[j] = quant_recip(y[j], u);
}

// LayerNorm / RMSNorm over rows held in registers, with optional residual add,
// sum output and int8 second output.  ALIGNED rows (16-byte aligned, length a
// multiple of the vector) need no per-element bounds: a vector is either inside
// the row or entirely outside it.
template <typename T, int G, int NV, int R, bool ALIGNED>
__global__ void __launch_bounds__(kBlock, (NV * R <= 4 ? 3 : (NV * R <= 8 ? 2 : 1)))
norm_kernel(NormParams p) {
  grid_dep_launch();  // the next kernel may begin its own set-up
  constexpr int E = VecT<T>::kElems;
  __shared__ float red[R * 8];
  const RowIndex<G, R> ix;
  const int t = ix.t;
  const int cols = static_cast<int>(p.cols);
  const T* xb = reinterpret_cast<const T*>(p.x);
  const T* rb = reinterpret_cast<const T*>(p.residual);
  // gamma and beta are parameters of the model, final long before this launch: short rows fetch them
  // while the kernel before this one may still be running, which takes their latency (one more trip to
  // L2 after the reductions) off the critical path of a launch that is a few microseconds long.
  constexpr bool kEarlyParams = NV <= 4;
  const T* gb = reinterpret_cast<const T*>(p.gamma);
  const T* bb = (!p.rms && p.beta) ? reinterpret_cast<const T*>(p.beta) : nullptr;
  uint4 gvs[kEarlyParams ? NV : 1], bvs[kEarlyParams ? NV : 1];
  if (kEarlyParams) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      gvs[i] = load_vec<T>(gb, cols, t + i * G, ALIGNED, 0.f);
      bvs[i] = bb ? load_vec<T>(bb, cols, t + i * G, ALIGNED, 0.f) : make_uint4(0, 0, 0, 0);
    }
  }
  grid_dep_wait();    // the kernel before this one has finished and its writes are visible
  uint4 raw[R][NV];
  bool live[R];
  float mean[R], var[R];
  // number of valid elements of vector i of this thread: E, 0, or (unaligned rows) in between
  auto nvalid = [&](int i) {
    const int n = cols - (t + i * G) * E;
    return ALIGNED ? (n > 0 ? E : 0) : n;
  };
#pragma unroll
  for (int r = 0; r < R; ++r) {
    live[r] = ix.row0 + r < p.rows;
    const int64_t row = live[r] ? ix.row0 + r : 0;
    if (ALIGNED && p.x_slab_cols > 0) {
      // column slabs: vector v starts at column v * E of the logical row
      const int sc = static_cast<int>(p.x_slab_cols);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = (t + i * G) * E;
        const int slab = c / sc;
        raw[r][i] = load_vec<T>(xb + slab * p.x_slab_stride + row * sc - static_cast<int64_t>(slab) * sc, cols,
                                t + i * G, true, 0.f);
      }
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) raw[r][i] = load_vec<T>(xb + row * p.cols, cols, t + i * G, ALIGNED, 0.f);
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int64_t off = (live[r] ? ix.row0 + r : 0) * p.cols;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float f[E];
      if (rb) {
        const uint4 rv = load_vec<T>(rb + off, cols, t + i * G, ALIGNED, 0.f);
#pragma unroll
        for (int j = 0; j < E; ++j) f[j] = VecT<T>::get(raw[r][i], j) + VecT<T>::get(rv, j);
        raw[r][i] = VecT<T>::pack(f);  // the sum lives in the storage type, as a separate add would leave it
        if (p.sum_out && live[r])
          store_vec<T>(reinterpret_cast<T*>(p.sum_out) + off, cols, t + i * G, ALIGNED, raw[r][i]);
      } else {
#pragma unroll
        for (int j = 0; j < E; ++j) f[j] = VecT<T>::get(raw[r][i], j);
      }
#pragma unroll
      for (int j = 0; j < E; ++j) s += f[j];  // padding holds 0
    }
    mean[r] = s;
  }
  const float inv_n = 1.f / static_cast<float>(cols);
  if (!p.rms) {
    group_reduce<G, R, false>(mean, red);
#pragma unroll
    for (int r = 0; r < R; ++r) mean[r] *= inv_n;
  } else {
#pragma unroll
    for (int r = 0; r < R; ++r) mean[r] = 0.f;
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int nv = nvalid(i);
      if (ALIGNED && nv == 0) continue;
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const float dlt = VecT<T>::get(raw[r][i], j) - mean[r];
        if (ALIGNED || j < nv) ss = __fmaf_rn(dlt, dlt, ss);
      }
    }
    var[r] = ss;
  }
  group_reduce<G, R, false>(var, red);
  float rstd[R];
#pragma unroll
  for (int r = 0; r < R; ++r) rstd[r] = 1.f / sqrtf(var[r] * inv_n + p.eps);

  const bool dyn = p.q_out && !p.q_scale;
  // normalise in place: raw becomes y in the storage type (what the next op reads)
  float qs[R];
#pragma unroll
  for (int r = 0; r < R; ++r) qs[r] = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const uint4 gv = kEarlyParams ? gvs[i] : load_vec<T>(gb, cols, t + i * G, ALIGNED, 0.f);
    const uint4 bv = kEarlyParams ? bvs[i] : (bb ? load_vec<T>(bb, cols, t + i * G, ALIGNED, 0.f) : make_uint4(0, 0, 0, 0));
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float y[E];
#pragma unroll
      for (int j = 0; j < E; ++j) {
        y[j] = (VecT<T>::get(raw[r][i], j) - mean[r]) * rstd[r] * VecT<T>::get(gv, j);
        if (bb) y[j] += VecT<T>::get(bv, j);
      }
      raw[r][i] = VecT<T>::pack(y);
      if (p.y && live[r])
        store_vec<T>(reinterpret_cast<T*>(p.y) + (ix.row0 + r) * p.cols, cols, t + i * G, ALIGNED, raw[r][i]);
      if (dyn) {
#pragma unroll
        for (int j = 0; j < E; ++j) qs[r] = fmaxf(qs[r], fabsf(VecT<T>::get(raw[r][i], j)));  // padding: gamma fill 0
      }
    }
  }
  if (!p.q_out) return;
  if (dyn) {
    group_reduce<G, R, true>(qs, red);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      qs[r] = fmaxf(__fdiv_rn(qs[r], 127.f), FLT_EPSILON);
      if (t == 0 && live[r] && p.q_row_scale) p.q_row_scale[ix.row0 + r] = qs[r];
    }
  } else {
    const float s = __ldg(p.q_scale);
#pragma unroll
    for (int r = 0; r < R; ++r) qs[r] = s;
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (!live[r]) continue;
    const RecipQuant d = make_recip_quant(qs[r]);
    const int64_t off = (ix.row0 + r) * p.cols;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float y[E], q[E];
      VecT<T>::unpack(raw[r][i], y);
      quant_vec_recip<E>(y, d, q);
      store_q<E>(p.q_out + off, cols, t + i * G, ALIGNED, q);
    }
  }
}

template <typename T, int G, int NV, int R>
__global__ void __launch_bounds__(kBlock, (NV * R <= 4 ? 3 : (NV * R <= 8 ? 2 : 1)))
dynquant_kernel(DynQuantParams p, int aligned) {
  grid_dep_launch();  // the next kernel may begin its own set-up
  grid_dep_wait();    // the kernel before this one has finished and its writes are visible
  constexpr int E = VecT<T>::kElems;
  __shared__ float red[R * 8];
  const RowIndex<G, R> ix;
  const int t = ix.t;
  const int cols = static_cast<int>(p.cols);
  const bool al = aligned != 0;
  const T* xb = reinterpret_cast<const T*>(p.x);
  uint4 raw[R][NV];
  bool live[R];
  float m[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    live[r] = ix.row0 + r < p.rows;
    const int64_t off = (live[r] ? ix.row0 + r : 0) * p.cols;
#pragma unroll
    for (int i = 0; i < NV; ++i) raw[r][i] = load_vec<T>(xb + off, cols, t + i * G, al, 0.f);
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int j = 0; j < E; ++j) a = fmaxf(a, fabsf(VecT<T>::get(raw[r][i], j)));
    m[r] = a;
  }
  group_reduce<G, R, true>(m, red);
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (!live[r]) continue;
    const float s = fmaxf(__fdiv_rn(m[r], 127.f), FLT_EPSILON);
    if (t == 0) p.row_scale[ix.row0 + r] = s;
    const RecipQuant d = make_recip_quant(s);
    const int64_t off = (ix.row0 + r) * p.cols;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float y[E], q[E];
      VecT<T>::unpack(raw[r][i], y);
      quant_vec_recip<E>(y, d, q);
      store_q<E>(p.q + off, cols, t + i * G, al, q);
    }
  }
}

// h of the two-pass gated quantization; one definition for both passes, so that
// the scale of pass 0 always covers the values pass 1 quantizes.  silu(g) * u as
// (g * u) * rcp(1 + 2^(-g log2 e)) with the approximate exponential and
// reciprocal: two special-function ops and four multiply-adds per element.  An
// IEEE division here costs ten more instructions and a branch per element, and
// the kernel is bound by instruction issue (measured: 49 instructions per
// element and 23 % of the memory rate with it).
__device__ __forceinline__ float ex2_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_ftz(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float swiglu_value(float g, float u) {
  const float e = ex2_ftz(g * -1.4426950408889634f);
  return (g * u) * rcp_ftz(1.f + e);
}

// PASS 0: local row scale.  PASS 1: quantize with the (agreed) row scale.
// PASS 2: both in one go, for rows that are whole on this GPU.
template <typename T, int G, int NV, int R, int PASS>
__global__ void __launch_bounds__(kBlock, (NV * R <= 4 ? 3 : (NV * R <= 8 ? 2 : 1)))
gated_quant_kernel(GatedQuantParams p, int aligned) {
  grid_dep_launch();  // the next kernel may begin its own set-up
  grid_dep_wait();    // the kernel before this one has finished and its writes are visible
  constexpr int E = VecT<T>::kElems;
  __shared__ float red[R * 8];
  const RowIndex<G, R> ix;
  const int t = ix.t;
  const int cols = static_cast<int>(p.cols);
  const bool al = aligned != 0;
  const bool has_up = p.up != nullptr;
  const T* gb = reinterpret_cast<const T*>(p.gate);
  const T* ub = reinterpret_cast<const T*>(p.up);
  uint4 graw[R][NV], uraw[R][NV];
  bool live[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    live[r] = ix.row0 + r < p.rows;
    const int64_t off = (live[r] ? ix.row0 + r : 0) * p.ld;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      graw[r][i] = load_vec<T>(gb + off, cols, t + i * G, al, 0.f);
      if (has_up) uraw[r][i] = load_vec<T>(ub + off, cols, t + i * G, al, 0.f);
    }
  }
  // h of vector i of row r (padding gives h(0, 0) = 0)
  auto values = [&](int r, int i, float* h) {
    VecT<T>::unpack(graw[r][i], h);
    if (has_up) {
      float u[E];
      VecT<T>::unpack(uraw[r][i], u);
#pragma unroll
      for (int j = 0; j < E; ++j) h[j] = swiglu_value(h[j], u[j]);
    }
  };
  float m[R];
  if (PASS != 1) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float a = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        float h[E];
        values(r, i, h);
#pragma unroll
        for (int j = 0; j < E; ++j) a = fmaxf(a, fabsf(h[j]));
      }
      m[r] = a;
    }
    group_reduce<G, R, true>(m, red);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      m[r] = fmaxf(__fdiv_rn(m[r], 127.f), FLT_EPSILON);
      if (live[r] && t == 0) p.row_scale[ix.row0 + r] = m[r];
    }
  }
  if (PASS != 0) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (!live[r]) continue;
      const RecipQuant d = make_recip_quant(PASS == 1 ? __ldg(p.row_scale + ix.row0 + r) : m[r]);
      const int64_t off = (ix.row0 + r) * p.ldq;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        if ((t + i * G) * E >= cols) continue;
        float h[E], q[E];
        values(r, i, h);
        quant_vec_recip<E>(h, d, q);
        store_q<E>(p.q + off, cols, t + i * G, al, q);
      }
    }
  }
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// softmax over rows held in registers.  exp(x * scale - max) is evaluated as
// ex2(x * k - max * k) with k = scale * log2(e): one fused multiply-add and one
// special-function op per element and pass; the maximum is taken on the raw
// values (a positive scale keeps the order; a negative one turns it into the
// minimum).  Columns at and beyond the valid length are skipped by a
// per-vector count instead of a per-element index.
template <typename T, int G, int NV, int R>
__global__ void __launch_bounds__(kBlock, (NV * R <= 4 ? 3 : (NV * R <= 8 ? 2 : 1)))
softmax_kernel(SoftmaxParams p, int aligned) {
  grid_dep_launch();  // the next kernel may begin its own set-up
  grid_dep_wait();    // the kernel before this one has finished and its writes are visible
  // Issue bound unless lean: the logits are unpacked once, the exponentials are
  // kept (one special-function op per element, not one per pass), whole vectors
  // inside the valid length take a path without per-element predicates.
  constexpr int E = VecT<T>::kElems;
  constexpr float kLog2e = 1.4426950408889634f;
  __shared__ float red[R * 8];
  const int cols = static_cast<int>(p.cols);
  const bool al = aligned != 0;
  const T* xb = reinterpret_cast<const T*>(p.x);
  const T* mb = reinterpret_cast<const T*>(p.mask);
  const int64_t nblk = row_blocks<G, R>(p.rows);
  uint4 nxt[R][NV];
  auto fetch = [&](int64_t blk) {
    const RowIndex<G, R> fx(blk);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int64_t row = fx.row0 + r < p.rows ? fx.row0 + r : 0;
#pragma unroll
      for (int i = 0; i < NV; ++i) nxt[r][i] = load_vec<T>(xb + row * p.cols, cols, fx.t + i * G, al, 0.f);
    }
  };
  if (blockIdx.x < nblk) fetch(blockIdx.x);
  for (int64_t blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
  const RowIndex<G, R> ix(blk);
  const int t = ix.t;
  float f[R][NV][E];
  bool live[R];
  int len[R];
  {
    uint4 raw[R][NV];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int i = 0; i < NV; ++i) raw[r][i] = nxt[r][i];
    if (blk + gridDim.x < nblk) fetch(blk + gridDim.x);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      live[r] = ix.row0 + r < p.rows;
      const int64_t row = live[r] ? ix.row0 + r : 0;
      const int64_t batch = row / p.rows_per_batch;
      len[r] = p.lens ? min(cols, __ldg(p.lens + batch)) : cols;
      if (mb) {
        // fold the additive mask in once; the biased logits replace the raw values in the
        // storage type (as an unfused add would leave them) and carry the scale already
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const uint4 mv = load_vec<T>(mb + batch * p.cols, cols, t + i * G, al, 0.f);
          float a[E], b[E];
          VecT<T>::unpack(raw[r][i], a);
          VecT<T>::unpack(mv, b);
#pragma unroll
          for (int j = 0; j < E; ++j) a[j] = a[j] * p.scale + b[j];
          raw[r][i] = VecT<T>::pack(a);
        }
      }
#pragma unroll
      for (int i = 0; i < NV; ++i) VecT<T>::unpack(raw[r][i], f[r][i]);
    }
  }
  const float scale = mb ? 1.f : p.scale;
  const float k = scale * kLog2e;
  const float sgn = scale < 0.f ? -1.f : 1.f;  // a negative scale turns the maximum into the minimum
  float mx[R], sum[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float a = -INFINITY;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int nvalid = len[r] - (t + i * G) * E;  // valid elements of this vector (may be <= 0 or >= E)
      if (nvalid >= E) {
        if (sgn > 0.f) {
#pragma unroll
          for (int j = 0; j < E; ++j) a = fmaxf(a, f[r][i][j]);
        } else {
#pragma unroll
          for (int j = 0; j < E; ++j) a = fmaxf(a, -f[r][i][j]);
        }
      } else if (nvalid > 0) {
#pragma unroll
        for (int j = 0; j < E; ++j)
          if (j < nvalid) a = fmaxf(a, sgn * f[r][i][j]);
      }
    }
    mx[r] = a;
  }
  group_reduce<G, R, true>(mx, red);
  const bool want_log = p.log_softmax != 0;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    // mx holds max(x) (or max(-x) for a negative scale); the largest logit is |scale| * mx
    const float top = mx[r] == -INFINITY ? 0.f : mx[r] * fabsf(scale);
    mx[r] = top;                  // largest logit (0 for an empty row: every probability 0)
    const float bias = -top * kLog2e;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int nvalid = len[r] - (t + i * G) * E;
      if (nvalid >= E) {
#pragma unroll
        for (int j = 0; j < E; ++j) {
          const float e = ex2_approx(__fmaf_rn(f[r][i][j], k, bias));
          s += e;
          if (!want_log) f[r][i][j] = e;
        }
      } else {
#pragma unroll
        for (int j = 0; j < E; ++j) {
          const float e = j < nvalid ? ex2_approx(__fmaf_rn(f[r][i][j], k, bias)) : 0.f;
          s += e;
          if (!want_log) f[r][i][j] = e;
        }
      }
    }
    sum[r] = s;
  }
  group_reduce<G, R, false>(sum, red);
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (!live[r]) continue;
    const float inv = sum[r] > 0.f ? 1.f / sum[r] : 0.f;
    const int64_t off = (ix.row0 + r) * p.cols;
    if (!want_log) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        float y[E];
#pragma unroll
        for (int j = 0; j < E; ++j) y[j] = f[r][i][j] * inv;  // masked columns hold 0
        store_vec<T>(reinterpret_cast<T*>(p.y) + off, cols, t + i * G, al, VecT<T>::pack(y));
      }
    } else {
      const float lsum = logf(sum[r]);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int nvalid = len[r] - (t + i * G) * E;
        float y[E];
#pragma unroll
        for (int j = 0; j < E; ++j) y[j] = j < nvalid ? __fmaf_rn(f[r][i][j], scale, -mx[r]) - lsum : -INFINITY;
        store_vec<T>(reinterpret_cast<T*>(p.y) + off, cols, t + i * G, al, VecT<T>::pack(y));
      }
    }
  }
  }  // block loop
}

bool is_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ------------------------------------------------------------ rope + kv append
// One thread rotates eight pairs (i, i + dim/2) of one (token, head) of q and of
// k, and moves the matching sixteen values of v.
__global__ void __launch_bounds__(kBlock) rope_kv_kernel(RopeParams p) {
  const int half = static_cast<int>(p.dim / 2);
  const int chunks = half / 8;  // threads per (token, head)
  const int64_t total = p.batch * p.seq * p.heads * chunks;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(kBlock) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * kBlock) {
    const int c = static_cast<int>(idx % chunks);
    const int64_t th = idx / chunks;
    const int h = static_cast<int>(th % p.heads);
    const int64_t tok = th / p.heads;
    const int64_t b = tok / p.seq, s = tok % p.seq;
    const int64_t pos = p.pos0 + s;
    __half* q = reinterpret_cast<__half*>(p.qkv) + ((tok * 3 + 0) * p.heads + h) * p.dim + c * 8;
    __half* k = reinterpret_cast<__half*>(p.qkv) + ((tok * 3 + 1) * p.heads + h) * p.dim + c * 8;
    const __half* v = reinterpret_cast<const __half*>(p.qkv) + ((tok * 3 + 2) * p.heads + h) * p.dim + c * 8;
    const int64_t coff = ((b * p.heads + h) * p.cache_len + pos) * p.dim + c * 8;
    __half* kc = reinterpret_cast<__half*>(p.k_cache) + coff;
    __half* vc = reinterpret_cast<__half*>(p.v_cache) + coff;
    float cs[8], sn[8];
    {
      const float4* cp = reinterpret_cast<const float4*>(p.cos + pos * half + c * 8);
      const float4* sp = reinterpret_cast<const float4*>(p.sin + pos * half + c * 8);
      const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
      cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
      sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    }
    auto rotate = [&](const __half* src, __half* dst_lo, __half* dst_hi) {
      float x1[8], x2[8], o1[8], o2[8];
      VecT<__half>::unpack(*reinterpret_cast<const uint4*>(src), x1);
      VecT<__half>::unpack(*reinterpret_cast<const uint4*>(src + half), x2);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o1[j] = __fsub_rn(__fmul_rn(x1[j], cs[j]), __fmul_rn(x2[j], sn[j]));
        o2[j] = __fadd_rn(__fmul_rn(x2[j], cs[j]), __fmul_rn(x1[j], sn[j]));
      }
      *reinterpret_cast<uint4*>(dst_lo) = VecT<__half>::pack(o1);
      *reinterpret_cast<uint4*>(dst_hi) = VecT<__half>::pack(o2);
    };
    rotate(q, q, q + half);
    rotate(k, kc, kc + half);
    *reinterpret_cast<uint4*>(vc) = *reinterpret_cast<const uint4*>(v);
    *reinterpret_cast<uint4*>(vc + half) = *reinterpret_cast<const uint4*>(v + half);
  }
}

#include "rownorm_staged.inl"

// (G, NV, R) for a row of `nvec` 16-byte vectors: sub-warp groups for short
// rows, one warp up to 8 vectors per lane, one block above; R chosen so that a
// thread has 4 to 8 loads in flight.
#define DISC_ROW_LAUNCH(KERNEL, T, G, NV, R, rows, stream, ...)                                        \
  do {                                                                                                 \
    const int64_t groups_per_block = kBlock / (G);                                                     \
    const int64_t rows_per_block = groups_per_block * (R);                                             \
    const unsigned grid = static_cast<unsigned>(((rows) + rows_per_block - 1) / rows_per_block);       \
    launch_dependent(KERNEL<T, G, NV, R>, dim3(grid), dim3(kBlock), 0, stream, __VA_ARGS__);           \
  } while (0)

#define DISC_ROW_DISPATCH(KERNEL, T, nvec, rows, stream, ...)                                          \
  do {                                                                                                 \
    if ((nvec) <= 8) DISC_ROW_LAUNCH(KERNEL, T, 8, 1, 4, rows, stream, __VA_ARGS__);                   \
    else if ((nvec) <= 16) DISC_ROW_LAUNCH(KERNEL, T, 8, 2, 2, rows, stream, __VA_ARGS__);             \
    else if ((nvec) <= 32) DISC_ROW_LAUNCH(KERNEL, T, 16, 2, 2, rows, stream, __VA_ARGS__);            \
    else if ((nvec) <= 64) DISC_ROW_LAUNCH(KERNEL, T, 32, 2, 2, rows, stream, __VA_ARGS__);            \
    else if ((nvec) <= 96) DISC_ROW_LAUNCH(KERNEL, T, 32, 3, 1, rows, stream, __VA_ARGS__);            \
    else if ((nvec) <= 128) DISC_ROW_LAUNCH(KERNEL, T, 32, 4, 1, rows, stream, __VA_ARGS__);           \
    else if ((nvec) <= 192) DISC_ROW_LAUNCH(KERNEL, T, 32, 6, 1, rows, stream, __VA_ARGS__);           \
    else if ((nvec) <= 256) DISC_ROW_LAUNCH(KERNEL, T, 32, 8, 1, rows, stream, __VA_ARGS__);           \
    else if ((nvec) <= 512) DISC_ROW_LAUNCH(KERNEL, T, 256, 2, 1, rows, stream, __VA_ARGS__);          \
    else if ((nvec) <= 1024) DISC_ROW_LAUNCH(KERNEL, T, 256, 4, 1, rows, stream, __VA_ARGS__);         \
    else if ((nvec) <= 2048) DISC_ROW_LAUNCH(KERNEL, T, 256, 8, 1, rows, stream, __VA_ARGS__);         \
    else DISC_ROW_LAUNCH(KERNEL, T, 256, 16, 1, rows, stream, __VA_ARGS__);                            \
  } while (0)

// The same for kernels that walk row blocks with a stride of gridDim.x and
// prefetch: the grid is what the GPU holds at once.
#define DISC_ROW_LAUNCH_P(KERNEL, T, G, NV, R, rows, stream, ...)                                      \
  do {                                                                                                 \
    const int64_t groups_per_block = kBlock / (G);                                                     \
    const int64_t rows_per_block = groups_per_block * (R);                                             \
    int64_t grid = ((rows) + rows_per_block - 1) / rows_per_block;                                     \
    static int resident = 0; /* blocks of this instantiation one SM holds */                          \
    if (resident == 0) {                                                                               \
      int n = 0;                                                                                       \
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, KERNEL<T, G, NV, R>, kBlock, 0) != cudaSuccess || n < 1) \
        n = 1;                                                                                         \
      resident = n;                                                                                    \
    }                                                                                                  \
    const int64_t cap = static_cast<int64_t>(sm_count()) * resident;                                   \
    if (grid > cap) grid = cap;                                                                        \
    launch_dependent(KERNEL<T, G, NV, R>, dim3(static_cast<unsigned>(grid)), dim3(kBlock), 0, stream,  \
                     __VA_ARGS__);                                                                     \
  } while (0)

#define DISC_ROW_DISPATCH_P(KERNEL, T, nvec, rows, stream, ...)                                        \
  do {                                                                                                 \
    if ((nvec) <= 8) DISC_ROW_LAUNCH_P(KERNEL, T, 8, 1, 4, rows, stream, __VA_ARGS__);                 \
    else if ((nvec) <= 16) DISC_ROW_LAUNCH_P(KERNEL, T, 8, 2, 2, rows, stream, __VA_ARGS__);           \
    else if ((nvec) <= 32) DISC_ROW_LAUNCH_P(KERNEL, T, 16, 2, 2, rows, stream, __VA_ARGS__);          \
    else if ((nvec) <= 64) DISC_ROW_LAUNCH_P(KERNEL, T, 32, 2, 2, rows, stream, __VA_ARGS__);          \
    else if ((nvec) <= 96) DISC_ROW_LAUNCH_P(KERNEL, T, 32, 3, 1, rows, stream, __VA_ARGS__);          \
    else if ((nvec) <= 128) DISC_ROW_LAUNCH_P(KERNEL, T, 32, 4, 1, rows, stream, __VA_ARGS__);         \
    else if ((nvec) <= 192) DISC_ROW_LAUNCH_P(KERNEL, T, 32, 6, 1, rows, stream, __VA_ARGS__);         \
    else if ((nvec) <= 256) DISC_ROW_LAUNCH_P(KERNEL, T, 32, 8, 1, rows, stream, __VA_ARGS__);         \
    else if ((nvec) <= 512) DISC_ROW_LAUNCH_P(KERNEL, T, 256, 2, 1, rows, stream, __VA_ARGS__);        \
    else if ((nvec) <= 1024) DISC_ROW_LAUNCH_P(KERNEL, T, 256, 4, 1, rows, stream, __VA_ARGS__);       \
    else if ((nvec) <= 2048) DISC_ROW_LAUNCH_P(KERNEL, T, 256, 8, 1, rows, stream, __VA_ARGS__);       \
    else DISC_ROW_LAUNCH_P(KERNEL, T, 256, 16, 1, rows, stream, __VA_ARGS__);                          \
  } while (0)

template <typename T, int G, int NV, int R>
constexpr auto NORM_ALIGNED = norm_kernel<T, G, NV, R, true>;
template <typename T, int G, int NV, int R>
constexpr auto NORM_RAGGED = norm_kernel<T, G, NV, R, false>;

template <typename T, int G, int NV, int R>
constexpr auto GATED_SCALE = gated_quant_kernel<T, G, NV, R, 0>;
template <typename T, int G, int NV, int R>
constexpr auto GATED_QUANT = gated_quant_kernel<T, G, NV, R, 1>;
template <typename T, int G, int NV, int R>
constexpr auto GATED_BOTH = gated_quant_kernel<T, G, NV, R, 2>;

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

template <typename T>
int64_t vectors_per_row(int64_t cols) {
  return (cols + VecT<T>::kElems - 1) / VecT<T>::kElems;
}

}  // namespace

cudaError_t rope_kv_append_launch(const RopeParams& p, cudaStream_t s, const char** err) {
  if (err) *err = nullptr;
  if (p.batch <= 0 || p.seq <= 0 || p.heads <= 0) return cudaSuccess;
  if (!p.qkv || !p.k_cache || !p.v_cache || !p.cos || !p.sin) {
    if (err) *err = "rope: null operand";
    return cudaErrorInvalidValue;
  }
  if (p.dim <= 0 || p.dim % 16 != 0 || p.pos0 < 0 || p.pos0 + p.seq > p.cache_len) {
    if (err) *err = "rope: head dim must be a multiple of 16 and the positions must fit the cache";
    return cudaErrorInvalidValue;
  }
  if (!is_aligned16(p.qkv) || !is_aligned16(p.k_cache) || !is_aligned16(p.v_cache) || !is_aligned16(p.cos) ||
      !is_aligned16(p.sin)) {
    if (err) *err = "rope: operands must be 16-byte aligned";
    return cudaErrorInvalidValue;
  }
  const int64_t total = p.batch * p.seq * p.heads * (p.dim / 16);
  rope_kv_kernel<<<elem_grid(total), kBlock, 0, s>>>(p);
  return cudaGetLastError();
}

int rowops_status_fetch_and_clear() {
  int h = 0;
  if (cudaMemcpyFromSymbol(&h, g_rowops_status, sizeof(int)) != cudaSuccess) return -1;
  if (h != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_rowops_status, &z, sizeof(int));
  }
  return h;
}

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
  if (p.in_type == kF32) {
    const int aligned = (p.cols % 4 == 0) && is_aligned16(p.x) && ((reinterpret_cast<uintptr_t>(p.q) & 3) == 0);
    DISC_ROW_DISPATCH(dynquant_kernel, float, vectors_per_row<float>(p.cols), p.rows, s, p, aligned);
  } else {
    const int aligned = (p.cols % 8 == 0) && is_aligned16(p.x) && ((reinterpret_cast<uintptr_t>(p.q) & 7) == 0);
    DISC_ROW_DISPATCH(dynquant_kernel, __half, vectors_per_row<__half>(p.cols), p.rows, s, p, aligned);
  }
  return cudaGetLastError();
}

cudaError_t gated_quantize_launch(const GatedQuantParams& p, cudaStream_t s, const char** err) {
  if (err) *err = nullptr;
  if (p.rows <= 0 || p.cols <= 0) return cudaSuccess;
  if (!p.gate || !p.row_scale || (p.pass != 0 && !p.q) || p.pass < 0 || p.pass > 2) {
    if (err) *err = "gated quantize: null operand or unknown pass";
    return cudaErrorInvalidValue;
  }
  if (p.ld < p.cols || (p.pass != 0 && p.ldq < p.cols)) {
    if (err) *err = "gated quantize: row stride smaller than the row";
    return cudaErrorInvalidValue;
  }
  if (!row_shape_ok(p.rows, p.cols, err)) return cudaErrorInvalidValue;
  const int epv = p.type == kF32 ? 4 : 8;
  const int aligned = (p.cols % epv == 0) && (p.ld % epv == 0) && is_aligned16(p.gate) &&
                      (!p.up || is_aligned16(p.up)) &&
                      (p.pass == 0 || ((p.ldq % epv == 0) && (reinterpret_cast<uintptr_t>(p.q) & (epv - 1)) == 0));
  // pass 2 = pass 0 and pass 1 in one kernel (row scale written and used at once)
  if (p.type == kF32) {
    if (p.pass == 0) DISC_ROW_DISPATCH(GATED_SCALE, float, vectors_per_row<float>(p.cols), p.rows, s, p, aligned);
    else if (p.pass == 1) DISC_ROW_DISPATCH(GATED_QUANT, float, vectors_per_row<float>(p.cols), p.rows, s, p, aligned);
    else DISC_ROW_DISPATCH(GATED_BOTH, float, vectors_per_row<float>(p.cols), p.rows, s, p, aligned);
  } else {
    if (p.pass == 0) DISC_ROW_DISPATCH(GATED_SCALE, __half, vectors_per_row<__half>(p.cols), p.rows, s, p, aligned);
    else if (p.pass == 1) DISC_ROW_DISPATCH(GATED_QUANT, __half, vectors_per_row<__half>(p.cols), p.rows, s, p, aligned);
    else DISC_ROW_DISPATCH(GATED_BOTH, __half, vectors_per_row<__half>(p.cols), p.rows, s, p, aligned);
  }
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
  const int epv = p.type == kF32 ? 4 : 8;
  if (p.x_slab_cols > 0 &&
      (p.x_slab_cols % epv != 0 || p.cols % p.x_slab_cols != 0 || p.x_slab_stride % epv != 0 ||
       p.cols % epv != 0 || !is_aligned16(p.x))) {
    if (err) *err = "norm: slabbed x needs 16-byte aligned slabs whose width divides the row";
    return cudaErrorInvalidValue;
  }
  const int aligned = (p.cols % epv == 0) && is_aligned16(p.x) && is_aligned16(p.gamma) &&
                      (!p.residual || is_aligned16(p.residual)) && (!p.beta || is_aligned16(p.beta)) &&
                      (!p.y || is_aligned16(p.y)) && (!p.sum_out || is_aligned16(p.sum_out)) &&
                      (!p.q_out || (reinterpret_cast<uintptr_t>(p.q_out) & (epv - 1)) == 0);
  // long fp16 rows: a warp per row over a copy of the row in shared memory
  if (p.type == kF16 && aligned && p.cols >= 2048 && p.cols <= 8192) {
    const size_t row_bytes = static_cast<size_t>(p.cols) * 2;
    const size_t smem = 2 * row_bytes + kStagedWarps * (p.residual ? 2 : 1) * row_bytes + kStagedWarps * 8 + 16;
    auto kern = p.rms ? norm_staged_f16_kernel<true> : norm_staged_f16_kernel<false>;
    cudaError_t st = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (st != cudaSuccess) return st;
    int64_t per_sm = static_cast<int64_t>((227 * 1024) / (smem + 1024));
    if (per_sm > 12) per_sm = 12;
    if (per_sm < 1) per_sm = 1;
    int64_t grid = (p.rows + kStagedWarps - 1) / kStagedWarps;
    const int64_t cap = per_sm * sm_count();
    if (grid > cap) grid = cap;
    kern<<<static_cast<unsigned>(grid), kStagedWarps * 32, smem, s>>>(p);
    return cudaGetLastError();
  }
  if (p.type == kF32) {
    if (aligned) DISC_ROW_DISPATCH(NORM_ALIGNED, float, vectors_per_row<float>(p.cols), p.rows, s, p);
    else DISC_ROW_DISPATCH(NORM_RAGGED, float, vectors_per_row<float>(p.cols), p.rows, s, p);
  } else {
    if (aligned) DISC_ROW_DISPATCH(NORM_ALIGNED, __half, vectors_per_row<__half>(p.cols), p.rows, s, p);
    else DISC_ROW_DISPATCH(NORM_RAGGED, __half, vectors_per_row<__half>(p.cols), p.rows, s, p);
  }
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
  const int epv = p.type == kF32 ? 4 : 8;
  const int aligned = (p.cols % epv == 0) && is_aligned16(p.x) && is_aligned16(p.y) &&
                      (!p.mask || is_aligned16(p.mask));
  if (p.type == kF32)
    DISC_ROW_DISPATCH_P(softmax_kernel, float, vectors_per_row<float>(q.cols), q.rows, s, q, aligned);
  else
    DISC_ROW_DISPATCH_P(softmax_kernel, __half, vectors_per_row<__half>(q.cols), q.rows, s, q, aligned);
  return cudaGetLastError();
}

}  // namespace disc_b200
