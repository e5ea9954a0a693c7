// Int8 quantized linear for sm_100a: out = epilogue(A[M,K] . W[N,K]^T).
//
// This is the arithmetic of the reference's GPU custom call ral_pdll_qgemm
// (tao_compiler/mlir/ral/context/quantized_gpu_kernel_impl.cc:328-422, a
// cuBLASLt int8 GEMM with alpha and a bias epilogue) plus the dequantize /
// GELU / quantize elementwise kernels DISC generates after it
// (tao_compiler/mlir/disc/transforms/disc_lower_quantize_and_dequantize.cc:77-136),
// done in one pass: the int32 accumulator never leaves the SM.
//
// Three paths, all computing the same function:
//   tiled   (M > 64)  persistent CTAs, 128 x BN output tiles, TMA -> 128B-swizzled
//                     smem ring -> tcgen05.mma kind::i8 -> two TMEM accumulators so
//                     the epilogue of tile i overlaps the MMAs of tile i+1.
//   small-M (M <= 64) operands swapped: 128 output channels sit on the MMA M
//                     dimension, the few activation rows on the MMA N dimension, so
//                     the weight streams at HBM rate; K may be split across CTAs,
//                     partial sums meet in global scratch (plain stores, the last
//                     CTA of a channel block adds them: integer, order-free, exact).
//   simt              one thread per output; only for shapes TMA cannot address
//                     (K not a multiple of 16, unaligned base) such as the
//                     reference's 25x71 known-answer case.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>
#include <type_traits>

#include "attention.h"
#include "device_info.h"
#include "qgemm.h"
#include "rowops.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"
#include "woq_gemm.h"

namespace disc_b200 {

__device__ int g_kernel_status = 0;

namespace {

struct EpiParams {
  void* out;
  int64_t ldo;
  int64_t M, N;
  const float* x_scale;
  const float* w_scale;
  const float* out_scale;
  const void* bias;
  int x_kind, w_kind, o_kind, bias_kind, fold_out, div_out, div_exact, act, out_kind;
};

// Where K block `kb` of the two operands starts when the activation is stored
// as column slabs (kb_per_slab == 0: plain row-major, x = 128 * kb for both).
// Geometry the producer of the tiled kernel needs when the activation tiles are fetched in im2col mode
// (enabled = 0: plain 2-D tiles).
struct Im2colDev {
  int enabled;
  int pixels_per_image;  // out_h * out_w
  int out_w;
  int k_w, cblks;        // window width; channel blocks per window position
  int kb_bytes;          // channels (= bytes) per K block: 128, or 64 with 64-byte-swizzled tiles and two MMAs per block
  int stride_h, stride_w, dil_h, dil_w, pad_top, pad_left;
};

struct SlabA {
  int kb_per_slab;  // K blocks per slab = ceil(slab_cols / 128)
  int slab_rows;    // rows of the activation tensor map between two slabs
  int slab_cols;    // K extent of one slab
};
struct KCoord {
  int ax, ay, wx;  // activation x, activation row offset, weight x
};
__device__ __forceinline__ KCoord k_coord(const SlabA& s, int kb) {
  KCoord c;
  if (s.kb_per_slab == 0) {
    c.ax = c.wx = kb * 128;
    c.ay = 0;
  } else {
    const int slab = kb / s.kb_per_slab;
    const int kin = kb - slab * s.kb_per_slab;
    c.ax = kin * 128;
    c.ay = slab * s.slab_rows;
    c.wx = slab * s.slab_cols + kin * 128;  // the tail of a ragged slab meets zeros of the activation
  }
  return c;
}

__device__ __forceinline__ float col_scale(const EpiParams& e, int64_t n) {
  float sx = 1.f;
  if (e.x_kind == kScaleScalar) sx = __ldg(e.x_scale);
  else if (e.x_kind == kScalePerCol) sx = __ldg(e.x_scale + n);
  float sw = 1.f;
  if (e.w_kind == kScaleScalar) sw = __ldg(e.w_scale);
  else if (e.w_kind == kScalePerCol) sw = __ldg(e.w_scale + n);
  float s = __fmul_rn(sx, sw);
  if (e.fold_out) {
    const float so = (e.o_kind == kScalePerCol) ? __ldg(e.out_scale + n) : __ldg(e.out_scale);
    s = __fdiv_rn(s, so);
  }
  return s;
}

__device__ __forceinline__ float col_bias(const EpiParams& e, int64_t n) {
  if (e.bias_kind == kBiasF32) return __ldg(reinterpret_cast<const float*>(e.bias) + n);
  if (e.bias_kind == kBiasI8)
    return static_cast<float>(__ldg(reinterpret_cast<const int8_t*>(e.bias) + n));
  return 0.f;
}

// erf(x) to 3e-7 absolute (Abramowitz & Stegun 7.1.28): 1 - (1 + a1 t + ... + a6 t^6)^-16 for t = |x|, six
// fused multiply-adds, four squarings and one reciprocal.  libdevice's erff is exact to an ulp at about twice
// the instructions, which the epilogue of a short-K tile cannot hide; 3e-7 is far inside every tolerance the
// outputs are held to (the int8 step of a GELU output is four orders of magnitude larger).
__device__ __forceinline__ float erf_fast(float x) {
  const float t = fabsf(x);
  float p = 0.0000430638f;
  p = __fmaf_rn(p, t, 0.0002765672f);
  p = __fmaf_rn(p, t, 0.0001520143f);
  p = __fmaf_rn(p, t, 0.0092705272f);
  p = __fmaf_rn(p, t, 0.0422820123f);
  p = __fmaf_rn(p, t, 0.0705230784f);
  p = __fmaf_rn(p, t, 1.f);
  p *= p;
  p *= p;
  p *= p;
  p *= p;   // overflows to +inf for |x| > ~13, where erf is 1 to every bit
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(p));
  return copysignf(1.f - r, x);
}
__device__ __forceinline__ float gelu_erf(float v) {
  return 0.5f * v * (1.f + erf_fast(v * 0.70710678118654752440f));
}

__device__ __forceinline__ float act_apply(float v, int act) {
  if (act == kActGelu) return gelu_erf(v);
  if (act == kActSilu) return v / (1.f + __expf(-v));
  return v;
}

// Per-thread constants of the epilogue.
struct EpiCtx {
  float rs;      // row scale (per-token quantization) or 1
  float so;      // output scale when the result is divided by it
  float so_inv;  // correctly rounded 1 / so
  int act;
  bool has_rs;
  float k1, k0;   // unit form: u = v * k1 + k0 with k1 = (1 / so) / 255, k0 = 128 / 255
  int div;        // kDivNone, kDivRecip (product with 1 / so) or kDivExact (the IEEE quotient)
  bool folded;    // kDivRecip without an activation: the factor already sits in the column constants
  bool unit;      // kDivRecip with int8 output: values travel as u = (q + 128) / 255, see below
  bool div_fast;  // so is in the range where the reciprocal sequence below is safe
};

// How the value is brought to the output scale before rounding to int8.
//   kDivRecip  v * (1 / so) with the correctly rounded reciprocal: a few ulp from
//              the quotient, so the int8 result can differ from the divide-based
//              formula only for quotients that close to a rounding tie, and then
//              by one level (the tolerance the quantized path states for
//              requantized outputs).  Without an activation the factor is folded
//              into the column scale and bias and costs nothing per element.
//              (Holds while so and 1 / so are normal floats, 2^-126 <= |so| <=
//              2^126; a scale outside that range wants kDivExact.)
//              With int8 output the value is carried as u = (q + 128) / 255: the
//              saturating fused multiply-add clamps u to [0, 1], which is the
//              clamp of q to [-128, 127], and one more fused multiply-add,
//              255 u - 128 + 1.5 * 2^23, leaves the rounded (half to even) int8
//              in the low byte of the sum.  Two instructions on the FMA pipe
//              replace two min/max, an add and the reciprocal product; every
//              kernel uses the same sequence, so all paths agree bit for bit.
//   kDivExact  bit for bit what the reference's divide-based quantize computes.
enum DivMode : int { kDivNone = 0, kDivRecip = 1, kDivExact = 2 };

__device__ __forceinline__ EpiCtx make_epi_ctx(const EpiParams& e) {
  EpiCtx c;
  c.rs = 1.f;
  c.has_rs = e.x_kind == kScalePerRow;
  c.act = e.act;
  c.div = e.div_out ? (e.div_exact ? kDivExact : kDivRecip) : kDivNone;
  c.so = c.div != kDivNone ? __ldg(e.out_scale) : 1.f;
  c.so_inv = __frcp_rn(c.so);
  const float a = fabsf(c.so);
  c.div_fast = a > 1e-15f && a < 1e15f;
  c.folded = c.div == kDivRecip && c.act == kActNone;
  c.unit = c.div == kDivRecip && e.out_kind == kOutI8;
  c.k1 = c.unit ? __fdiv_rn(c.so_inv, 255.f) : c.so_inv;
  c.k0 = c.unit ? __fdiv_rn(128.f, 255.f) : 0.f;
  return c;
}

// Scale and bias of output channel n as the epilogue uses them.
__device__ __forceinline__ void col_consts(const EpiParams& e, const EpiCtx& c, int64_t n, float& cs, float& cb) {
  cs = col_scale(e, n);
  cb = col_bias(e, n);
  if (c.folded) {
    cs = __fmul_rn(cs, c.k1);
    cb = __fmaf_rn(cb, c.k1, c.k0);
  }
}

// The same in two steps for kernels that walk many tiles: the loads of the next
// tile's constants are issued before the current tile's arithmetic and finished
// (products, the folded division) after it, so their latency stays off the
// epilogue warps' critical path.
struct ColRaw {
  float sx, sw, so, b;
};
__device__ __forceinline__ ColRaw col_raw_load(const EpiParams& e, int64_t n) {
  ColRaw r;
  r.sx = 1.f;
  if (e.x_kind == kScaleScalar) r.sx = __ldg(e.x_scale);
  else if (e.x_kind == kScalePerCol) r.sx = __ldg(e.x_scale + n);
  r.sw = 1.f;
  if (e.w_kind == kScaleScalar) r.sw = __ldg(e.w_scale);
  else if (e.w_kind == kScalePerCol) r.sw = __ldg(e.w_scale + n);
  r.so = 1.f;
  if (e.fold_out) r.so = (e.o_kind == kScalePerCol) ? __ldg(e.out_scale + n) : __ldg(e.out_scale);
  r.b = 0.f;
  if (e.bias_kind == kBiasF32) r.b = __ldg(reinterpret_cast<const float*>(e.bias) + n);
  else if (e.bias_kind == kBiasI8) r.b = static_cast<float>(__ldg(reinterpret_cast<const int8_t*>(e.bias) + n));
  return r;
}
__device__ __forceinline__ void col_raw_finish(const EpiParams& e, const EpiCtx& c, const ColRaw& r, bool ok,
                                               float& cs, float& cb) {
  float s = __fmul_rn(r.sx, r.sw);
  if (e.fold_out) s = __fdiv_rn(s, r.so);
  float b = r.b;
  if (c.folded) {
    s = __fmul_rn(s, c.k1);
    b = __fmaf_rn(b, c.k1, c.k0);
  }
  cs = ok ? s : 0.f;
  cb = ok ? b : 0.f;
}

// v / so, correctly rounded wherever it decides the int8 result.  One IEEE
// division per output is the most expensive instruction sequence of the whole
// epilogue, so the quotient is first formed from the (correctly rounded)
// reciprocal with one residual correction: q0 = v * r, q = q0 + (v - q0 * so) * r.
// That is within one ulp of the true quotient; only a quotient that close to a
// rounding tie (k + 0.5) could round to a different integer, so those rare
// values alone are recomputed with the IEEE division the reference uses.
// The IEEE division is kept out of line: it runs for a few outputs in a
// thousand, and inlined into every unrolled epilogue slot it multiplies the
// code a CTA has to fetch.
__device__ __noinline__ float ieee_div(float v, float so) { return __fdiv_rn(v, so); }

__device__ __forceinline__ float div_out_scale(float v, const EpiCtx& c) {
  if (!c.div_fast) return ieee_div(v, c.so);
  const float q0 = v * c.so_inv;
  float q = __fmaf_rn(__fmaf_rn(-q0, c.so, v), c.so_inv, q0);
  // (q + 1.5 * 2^23) - 1.5 * 2^23 is q rounded half-to-even for |q| < 2^22: two
  // additions instead of a conversion-rate round instruction.
  const float frac = fabsf(q - ((q + 12582912.f) - 12582912.f));
  if (fabsf(frac - 0.5f) < 1e-3f && fabsf(q) < 256.f) q = ieee_div(v, c.so);
  return q;
}

// acc -> real value, shared by every path.
__device__ __forceinline__ float epi_value(int32_t acc, float cs, float cb, const EpiCtx& c) {
  float t = __int2float_rn(acc);
  if (c.has_rs) t = __fmul_rn(t, c.rs);
  float v = __fmaf_rn(t, cs, cb);
  v = act_apply(v, c.act);
  if (c.div == kDivExact) v = div_out_scale(v, c);
  else if (c.div == kDivRecip && !c.folded) v = __fmaf_rn(v, c.k1, c.k0);
  if (c.unit) v = __saturatef(v);
  return v;
}

// The same arithmetic with the mode fixed at compile time.  The tiled kernels
// run the epilogue of a whole tile inside one case of a switch over the mode,
// so the instructions a launch actually fetches are a short straight-line
// loop instead of sixteen unrolled copies of every branch (erf, exp, the
// division fix-up): with 18 warps in three roles the instruction cache was
// the first thing to run out.
// float(acc), correctly rounded like the conversion instruction, from integer and
// floating-point adds only.  acc = hi * 2048 + lo with hi = acc >> 11 (|hi| < 2^20)
// and lo = acc & 2047; both become floats exactly through the mantissa of a
// magic constant, and one fused multiply-add rounds their exact sum once.  The
// conversion instruction runs on the 16-lane special-function pipe; tile
// epilogues convert every other value this way so that neither pipe limits them.
__device__ __forceinline__ float int2float_by_adds(int32_t acc) {
  const float lo = __uint_as_float((static_cast<uint32_t>(acc) & 0x7FFu) | 0x4B000000u) - 8388608.f;
  const float hi = __int_as_float((acc >> 11) + 0x4B400000) - 12582912.f;
  return __fmaf_rn(hi, 2048.f, lo);
}

template <int ACT, int DIV, bool RS, bool UNIT, bool CVT_BY_ADDS = false>
__device__ __forceinline__ float epi_value_t(int32_t acc, float cs, float cb, const EpiCtx& c) {
  float t = CVT_BY_ADDS ? int2float_by_adds(acc) : __int2float_rn(acc);
  if (RS) t = __fmul_rn(t, c.rs);
  float v = __fmaf_rn(t, cs, cb);
  if (ACT == kActGelu) v = gelu_erf(v);
  if (ACT == kActSilu) v = v / (1.f + __expf(-v));
  if (DIV == kDivExact) v = div_out_scale(v, c);
  if (DIV == kDivRecip && ACT != kActNone) v = __fmaf_rn(v, c.k1, c.k0);  // folded into cs / cb otherwise
  if (DIV == kDivRecip && UNIT) v = __saturatef(v);
  return v;
}

__device__ __forceinline__ int epi_mode(const EpiCtx& c) {
  return c.act | (c.div << 2) | (c.has_rs ? 16 : 0);
}

// Calls BODY with ACT / DIV / RS bound as compile-time constants for `mode`.
#define DISC_EPI_CASE(A, D, R, BODY)                 \
  case ((A) | ((D) << 2) | ((R) ? 16 : 0)): {        \
    constexpr int ACT = (A);                         \
    constexpr int DIV = (D);                         \
    constexpr bool RS = (R);                         \
    BODY;                                            \
  } break;
// Whether values of this (output type, division form) travel in unit form.
template <typename OutT, int DIV>
inline constexpr bool kUnitForm = std::is_same_v<OutT, int8_t> && DIV == kDivRecip;
#define DISC_EPI_CASES_RS(R, BODY)                                                         \
  DISC_EPI_CASE(0, 0, R, BODY) DISC_EPI_CASE(1, 0, R, BODY) DISC_EPI_CASE(2, 0, R, BODY)   \
  DISC_EPI_CASE(0, 1, R, BODY) DISC_EPI_CASE(1, 1, R, BODY) DISC_EPI_CASE(2, 1, R, BODY)   \
  DISC_EPI_CASE(0, 2, R, BODY) DISC_EPI_CASE(1, 2, R, BODY) DISC_EPI_CASE(2, 2, R, BODY)
#define DISC_EPI_SWITCH(mode, BODY)                                                        \
  switch (mode) {                                                                          \
    DISC_EPI_CASES_RS(false, BODY)                                                         \
    DISC_EPI_CASES_RS(true, BODY)                                                          \
    default: break;                                                                        \
  }

__device__ __forceinline__ int8_t to_s8(float v) {
  int r = __float2int_rn(v);
  r = max(-128, min(127, r));
  return static_cast<int8_t>(r);
}

// A word whose low byte is the int8 result.  Plain form: clamp to [-128, 127],
// then adding 1.5 * 2^23 leaves the rounded integer in the low mantissa bits
// (the add itself rounds to nearest even), so the low byte of the sum is the
// two's-complement result; no float-to-int conversion.  Unit form (u in [0, 1]
// stands for 255 u - 128): the same magic sum in one fused multiply-add.
template <bool UNIT>
__device__ __forceinline__ uint32_t s8_word(float v) {
  const float kMagic = 12582912.f;
  if (UNIT) return __float_as_uint(__fmaf_rn(v, 255.f, kMagic - 128.f));
  return __float_as_uint(fminf(fmaxf(v, -128.f), 127.f) + kMagic);
}

// Four of them packed into one word.
template <bool UNIT = false>
__device__ __forceinline__ uint32_t pack4_s8(float a, float b, float c, float d) {
  const uint32_t ab = __byte_perm(s8_word<UNIT>(a), s8_word<UNIT>(b), 0x0040);
  const uint32_t cd = __byte_perm(s8_word<UNIT>(c), s8_word<UNIT>(d), 0x0040);
  return __byte_perm(ab, cd, 0x5410);
}

// UNIT: `v` of an int8 output is in unit form (see DivMode).
template <typename OutT, bool UNIT = false>
__device__ __forceinline__ void store_one(OutT* p, float v, int32_t acc) {
  if constexpr (std::is_same_v<OutT, int8_t>) {
    *p = UNIT ? static_cast<int8_t>(s8_word<true>(v) & 0xFFu) : to_s8(v);
  } else if constexpr (std::is_same_v<OutT, __half>) {
    *p = __float2half_rn(v);
  } else if constexpr (std::is_same_v<OutT, float>) {
    *p = v;
  } else {
    *p = acc;
  }
}
// The same for kernels that learn the mode at run time.
template <typename OutT>
__device__ __forceinline__ void store_one_rt(OutT* p, float v, int32_t acc, const EpiCtx& c) {
  if (std::is_same_v<OutT, int8_t> && c.unit) store_one<OutT, true>(p, v, acc);
  else store_one<OutT, false>(p, v, acc);
}

// Stores 16 consecutive outputs of one row with 16-byte stores.
template <typename OutT, bool UNIT = false>
__device__ __forceinline__ void store_row16_vec(OutT* p, const float* v, const uint32_t* acc) {
  if constexpr (std::is_same_v<OutT, int8_t>) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = pack4_s8<UNIT>(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  } else if constexpr (std::is_same_v<OutT, __half>) {
    uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      __half2 h0 = __floats2half2_rn(v[8 * i + 0], v[8 * i + 1]);
      __half2 h1 = __floats2half2_rn(v[8 * i + 2], v[8 * i + 3]);
      __half2 h2 = __floats2half2_rn(v[8 * i + 4], v[8 * i + 5]);
      __half2 h3 = __floats2half2_rn(v[8 * i + 6], v[8 * i + 7]);
      q[i] = make_uint4(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1),
                        *reinterpret_cast<uint32_t*>(&h2), *reinterpret_cast<uint32_t*>(&h3));
    }
  } else if constexpr (std::is_same_v<OutT, float>) {
    float4* q = reinterpret_cast<float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
    uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = make_uint4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
  }
}

// ------------------------------------------------------------------ tiled
constexpr int kTileM = 128;        // MMA M, rows of the 128-row operand tile
constexpr int kTileKBytes = 128;   // one 128-byte swizzle row of int8 = 128 k
constexpr int kMmaK = 32;          // k per tcgen05.mma kind::i8
// Tiled kernel: warps [0, 16) run the epilogue, four per TMEM lane quadrant
// (a warp may only read the quadrant warp_id % 4), each owning a quarter of the
// tile's columns; warp 16 issues TMA, warp 17 owns TMEM and issues the MMAs.
// Four epilogue warps per scheduler hide the latency of the conversion /
// activation / division chain, which one warp per scheduler could not.
constexpr int kEpiWarps = 16;
constexpr int kEpiGroups = kEpiWarps / 4;
constexpr int kTiledThreads = (kEpiWarps + 2) * 32;
constexpr int kThreads = 576;      // small-M kernel: warp 0 TMA, warp 1 MMA, warps 2-17 epilogue

template <int BN, int STAGES>
struct TiledSmem {
  static constexpr int kABytes = kTileM * kTileKBytes;
  static constexpr int kBBytes = BN * kTileKBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  static constexpr int kNumBars = 2 * STAGES + 4;
  static constexpr int kMiscOffset = kBarOffset + kNumBars * 8;  // tmem slot, abort flag
  static constexpr int kScaleOffset = kMiscOffset + 16;
  static constexpr int kColsPerWarp = BN / kEpiGroups;
  static constexpr int kTotal = kScaleOffset + kEpiWarps * 2 * kColsPerWarp * 4;  // per warp: cs[], cb[]
  static constexpr int kDynamic = kTotal + 1024;  // slack to align the base to 1024
};

// One epilogue warp's share of a tile: CW columns of its 32 rows, 16 columns
// per TMEM load, converted and stored straight from registers.
template <typename OutT, int ACT, int DIV, bool RS, int CW>
__device__ __forceinline__ void tiled_epilogue_cols(uint32_t t_row, const float* cs, const float* cb,
                                                    const EpiCtx& ctx, OutT* out, int64_t m,
                                                    bool row_ok, int64_t col0, int64_t N,
                                                    int64_t ldo, int vec_ok) {
#pragma unroll 1
  for (int c = 0; c < CW / 16; ++c) {
    const int64_t n0 = col0 + c * 16;
    if (n0 >= N) break;  // uniform across the warp
    uint32_t r[16];
    tmem_ld_x16(t_row + c * 16, r);
    tmem_ld_wait();
    if (row_ok) {
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        v[j] = epi_value_t<ACT, DIV, RS, kUnitForm<OutT, DIV>>(static_cast<int32_t>(r[j]), cs[c * 16 + j],
                                                               cb[c * 16 + j], ctx);
      }
      OutT* dst = out + m * ldo + n0;
      if (vec_ok && n0 + 16 <= N) {
        store_row16_vec<OutT, kUnitForm<OutT, DIV>>(dst, v, r);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (n0 + j < N) store_one<OutT, kUnitForm<OutT, DIV>>(dst + j, v[j], static_cast<int32_t>(r[j]));
        }
      }
    }
  }
}

template <int BN, int STAGES, typename OutT>
__global__ void __launch_bounds__(kTiledThreads, 1)
qgemm_tiled_kernel(const __grid_constant__ CUtensorMap tmap_a,
                   const __grid_constant__ CUtensorMap tmap_w, EpiParams ep, int num_kb, int tiles_m,
                   int tiles_n, int vec_ok, SlabA slab, Im2colDev ic) {
  using L = TiledSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOffset);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOffset + 4);
  float* s_scale = reinterpret_cast<float*>(smem + L::kScaleOffset);  // [warp][2][kColsPerWarp]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = 2 * BN;  // 128, 256 or 512: a power of two >= 32
  constexpr int kProducerWarp = kEpiWarps;
  constexpr int kMmaWarp = kEpiWarps + 1;

  if (threadIdx.x == kProducerWarp * 32) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_w);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), kEpiWarps);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // the set-up above ran while the kernel before this one may still have been
  // finishing; everything below reads or writes what that kernel may touch
  grid_dep_launch();
  grid_dep_wait();

  const int num_tiles = tiles_m * tiles_n;

  if (warp == kProducerWarp) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m_blk = tile / tiles_n;
        const int n_blk = tile % tiles_n;
        // im2col mode: base position of the tile's first output pixel in the image, and the window
        // position / channel block of the K block, kept by increments
        int img = 0, w_base = 0, h_base = 0, ky = 0, kx = 0, cb = 0;
        if (ic.enabled) {
          const int m0 = m_blk * kTileM;
          img = m0 / ic.pixels_per_image;
          const int rem = m0 - img * ic.pixels_per_image;
          const int oy = rem / ic.out_w;
          h_base = oy * ic.stride_h - ic.pad_top;
          w_base = (rem - oy * ic.out_w) * ic.stride_w - ic.pad_left;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, &g_kernel_status,
                         kStatusTimeoutEmpty);
          if (!ok) break;
          mbar_arrive_expect_tx(full_bar(stage), ic.enabled ? (kTileM + BN) * ic.kb_bytes : L::kStageBytes);
          const uint32_t a_dst = smem_base + stage * L::kStageBytes;
          if (ic.enabled) {
            tma_load_im2col_4d(a_dst, &tmap_a, full_bar(stage), cb * ic.kb_bytes, w_base, h_base, img,
                               static_cast<uint16_t>(kx * ic.dil_w), static_cast<uint16_t>(ky * ic.dil_h));
            tma_load_2d(a_dst + L::kABytes, &tmap_w, full_bar(stage), kb * ic.kb_bytes, n_blk * BN);
            if (++cb == ic.cblks) {
              cb = 0;
              if (++kx == ic.k_w) {
                kx = 0;
                ++ky;
              }
            }
          } else {
          const KCoord kc = k_coord(slab, kb);
          tma_load_2d(a_dst, &tmap_a, full_bar(stage), kc.ax, kc.ay + m_blk * kTileM);
          tma_load_2d(a_dst + L::kABytes, &tmap_w, full_bar(stage), kc.wx, n_blk * BN);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_i8_idesc(kTileM, BN);
      // everything of the shared-memory descriptors but the address.  Image tiles of 64 channels have rows of
      // 64 bytes with 64-byte swizzle and take two MMAs per K block; all other tiles 128 bytes and four.
      const bool half = ic.enabled && ic.kb_bytes == 64;
      const uint64_t desc_hi = (half ? make_kmajor_sw64_desc(0) : make_kmajor_sw128_desc(0));
      const int mmas_per_kb = half ? 2 : kTileKBytes / kMmaK;
      int stage = 0;
      uint32_t phase = 0;
      int acc_buf = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        ok = mbar_wait(tempty_bar(acc_buf), acc_phase ^ 1, abort_flag, &g_kernel_status,
                       kStatusTimeoutTmemEmpty);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc_buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(full_bar(stage), phase, abort_flag, &g_kernel_status, kStatusTimeoutFull);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * L::kStageBytes;
          const uint64_t a_desc = desc_hi | static_cast<uint64_t>((a_addr & 0x3FFFF) >> 4);
          const uint64_t b_desc = desc_hi | static_cast<uint64_t>(((a_addr + L::kABytes) & 0x3FFFF) >> 4);
#pragma unroll
          for (int k = 0; k < kTileKBytes / kMmaK; ++k) {
            if (k < mmas_per_kb) umma_i8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc_buf));
        acc_buf ^= 1;
        if (acc_buf == 0) acc_phase ^= 1;
      }
    }
  } else {
    // Epilogue warp: TMEM lane quadrant q = 32-row slice of the tile, column
    // group g = a quarter of the tile's columns.  Each warp keeps its own copy
    // of its columns' scale / bias, so epilogue warps never wait on one another.
    constexpr int CW = L::kColsPerWarp;
    const int q = warp & 3;
    const int g = warp >> 2;
    float* cs = s_scale + warp * 2 * CW;
    float* cb = cs + CW;
    int acc_buf = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    EpiCtx ctx = make_epi_ctx(ep);
    OutT* out = reinterpret_cast<OutT*>(ep.out);
    // Column constants of the tile after the current one travel in registers:
    // requested before the current tile's arithmetic, finished after it.
    constexpr int CPL = (CW + 31) / 32;  // columns per lane
    ColRaw raw[CPL];
    auto request_consts = [&](int tile) {
      const int64_t c0 = static_cast<int64_t>(tile % tiles_n) * BN + g * CW;
#pragma unroll
      for (int i = 0; i < CPL; ++i) {
        const int64_t n = c0 + lane + 32 * i;
        raw[i] = col_raw_load(ep, n < ep.N ? n : ep.N - 1);
      }
    };
    if (static_cast<int>(blockIdx.x) < num_tiles) request_consts(blockIdx.x);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m_blk = tile / tiles_n;
      const int n_blk = tile % tiles_n;
      const int64_t col0 = static_cast<int64_t>(n_blk) * BN + g * CW;  // first column of this warp
      __syncwarp();
#pragma unroll
      for (int i = 0; i < CPL; ++i) {
        const int j = lane + 32 * i;
        if (j < CW) col_raw_finish(ep, ctx, raw[i], col0 + j < ep.N, cs[j], cb[j]);
      }
      __syncwarp();
      if (tile + static_cast<int>(gridDim.x) < num_tiles) request_consts(tile + gridDim.x);
      ok = mbar_wait(tfull_bar(acc_buf), acc_phase, abort_flag, &g_kernel_status,
                     kStatusTimeoutTmemFull);
      if (!ok) break;
      tc_fence_after();
      const int64_t m = static_cast<int64_t>(m_blk) * kTileM + q * 32 + lane;
      const bool row_ok = m < ep.M;
      if (ctx.has_rs) ctx.rs = row_ok ? __ldg(ep.x_scale + m) : 1.f;
      const uint32_t t_row =
          tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc_buf * BN + g * CW;
      const int mode = std::is_same_v<OutT, int32_t> ? 0 : epi_mode(ctx);
      DISC_EPI_SWITCH(mode, (tiled_epilogue_cols<OutT, ACT, DIV, RS, CW>(t_row, cs, cb, ctx, out, m, row_ok,
                                                                         col0, ep.N, ep.ldo, vec_ok)))
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc_buf));
      acc_buf ^= 1;
      if (acc_buf == 0) acc_phase ^= 1;
    }
  }

  // Wind-down.  After an abort, give copies still in flight time to land
  // before the shared memory is handed back.
  __syncwarp();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

#include "qgemm_pair.inl"

// ---------------------------------------------------------------- small M
constexpr int kSmallMaxStages = 8;
constexpr int kSmallMaxSplit = 8;   // K splits per channel block
constexpr int kSplitCounterWords = 4096;  // int32 arrival counters at the front of the scratch
constexpr int kSmallBarOffset = 200 * 1024;  // stages live below this offset
constexpr int kSmallDynamic = kSmallBarOffset + 256 + 1024;

// grid = (channel blocks of 128, K splits).  MT = activation rows padded to
// 16/32/64/128 = the MMA N dimension.
template <typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
qgemm_smallm_kernel(const __grid_constant__ CUtensorMap tmap_w,
                    const __grid_constant__ CUtensorMap tmap_x, EpiParams ep, int MT, int stages,
                    int num_kb, int32_t* ws, int32_t* counters, int kbs, int box_rows) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + kSmallBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kSmallMaxStages + s); };
  const uint32_t tfull_bar = bar_base + 8u * (2 * kSmallMaxStages);
  const uint32_t stored_bar = bar_base + 8u * (2 * kSmallMaxStages + 1);   // 16 warps stored partials
  const uint32_t counted_bar = bar_base + 8u * (2 * kSmallMaxStages + 2);  // arrival count taken
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kSmallBarOffset + 8 * (2 * kSmallMaxStages + 3));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_blk = blockIdx.x;
  const int split = gridDim.y;
  const int ks = blockIdx.y;
  const int kb_begin = static_cast<int>((static_cast<int64_t>(ks) * num_kb) / split);
  const int kb_end = static_cast<int>((static_cast<int64_t>(ks + 1) * num_kb) / split);
  const uint32_t w_bytes = kTileM * kTileKBytes;
  const uint32_t x_bytes = static_cast<uint32_t>(MT) * kTileKBytes;
  const uint32_t stage_bytes = kbs * (w_bytes + x_bytes);  // multiples of 1024 (MT >= 16)
  const uint32_t tmem_cols = MT < 32 ? 32u : static_cast<uint32_t>(MT);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    mbar_init(stored_bar, 16);
    mbar_init(counted_bar, 1);
    *abort_flag = 0;
    *last_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      // A stage holds `kbs` consecutive K blocks.  The weight boxes are issued
      // row group by row group, the K blocks of a group back to back, so that
      // requests for neighbouring 128-byte pieces of one weight row (one DRAM
      // page) leave the SM close together.
      for (int kb0 = kb_begin; kb0 < kb_end; kb0 += kbs) {
        const int nk = kb_end - kb0 < kbs ? kb_end - kb0 : kbs;
        if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, &g_kernel_status,
                       kStatusTimeoutEmpty))
          break;
        mbar_arrive_expect_tx(full_bar(stage), nk * (w_bytes + x_bytes));
        const uint32_t w_dst = smem_base + stage * stage_bytes;
        const uint32_t x_dst = w_dst + kbs * w_bytes;
        for (int r0 = 0; r0 < kTileM; r0 += box_rows) {
          for (int c = 0; c < nk; ++c) {
            tma_load_2d(w_dst + c * w_bytes + r0 * kTileKBytes, &tmap_w, full_bar(stage),
                        (kb0 + c) * kTileKBytes, n_blk * kTileM + r0);
          }
        }
        for (int c = 0; c < nk; ++c) {
          tma_load_2d(x_dst + c * x_bytes, &tmap_x, full_bar(stage), (kb0 + c) * kTileKBytes, 0);
        }
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_i8_idesc(kTileM, MT);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb0 = kb_begin; kb0 < kb_end; kb0 += kbs) {
        const int nk = kb_end - kb0 < kbs ? kb_end - kb0 : kbs;
        ok = mbar_wait(full_bar(stage), phase, abort_flag, &g_kernel_status, kStatusTimeoutFull);
        if (!ok) break;
        tc_fence_after();
        const uint32_t w_addr = smem_base + stage * stage_bytes;
        const uint32_t x_addr = w_addr + kbs * w_bytes;
        for (int c = 0; c < nk; ++c) {
          const uint64_t a_desc = make_kmajor_sw128_desc(w_addr + c * w_bytes);
          const uint64_t b_desc = make_kmajor_sw128_desc(x_addr + c * x_bytes);
#pragma unroll
          for (int k = 0; k < kTileKBytes / kMmaK; ++k) {
            umma_i8(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc,
                    (kb0 + c != kb_begin || k != 0) ? 1u : 0u);
          }
        }
        umma_commit(empty_bar(stage));
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit(tfull_bar);
    }
  } else {
    // Sixteen epilogue warps: warp w reads TMEM lane quadrant w & 3 (its 32
    // channels) and activation rows 16 * g + [0, 16) (+64 when MT is 128),
    // g = (w - 2) >> 2.  One warp per quadrant would walk all MT rows alone
    // and, with nothing else resident to hide its latencies, cost more than
    // the whole weight stream.
    const int q = warp & 3;
    const int ew = warp - 2;  // 0..15
    const int g = ew >> 2;
    const int et = threadIdx.x - 64;
    const int64_t n = static_cast<int64_t>(n_blk) * kTileM + q * 32 + lane;  // this thread's channel
    const bool n_ok = n < ep.N;
    const int64_t n_pad = static_cast<int64_t>(gridDim.x) * kTileM;
    EpiCtx ctx = make_epi_ctx(ep);
    OutT* out = reinterpret_cast<OutT*>(ep.out);
    const int Mrows = static_cast<int>(ep.M);

    // Column constants are fetched while the weight still streams.  With one
    // split a thread finishes channel n; after a split-K sum it finishes the
    // four channels n4 .. n4 + 3.
    const int64_t n4 = static_cast<int64_t>(n_blk) * kTileM + lane * 4;
    float cs = 0.f, cb = 0.f, cs4[4], cb4[4];
    if (split == 1) {
      if (n_ok) col_consts(ep, ctx, n, cs, cb);
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const bool c_ok = n4 + c < ep.N;
        cs4[c] = cb4[c] = 0.f;
        if (c_ok) col_consts(ep, ctx, n4 + c, cs4[c], cb4[c]);
      }
    }

    bool ok = mbar_wait(tfull_bar, 0, abort_flag, &g_kernel_status, kStatusTimeoutTmemFull);
    if (ok) {
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      if (split == 1) {
#pragma unroll 1
        for (int c = g; c < MT / 16; c += 4) {
          if (c * 16 >= Mrows) break;
          uint32_t r[16];
          tmem_ld_x16(t_row + c * 16, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c * 16 + j;
            if (m < Mrows && n_ok) {
              if (ctx.has_rs) ctx.rs = __ldg(ep.x_scale + m);
              const int32_t acc = static_cast<int32_t>(r[j]);
              store_one_rt<OutT>(out + static_cast<int64_t>(m) * ep.ldo + n, epi_value(acc, cs, cb, ctx), acc, ctx);
            }
          }
        }
      } else {
        // Partial sums: ws[ks][m][n_pad]; every slot this launch reads is
        // written first, so the scratch needs no clearing between launches.
        int32_t* my_ws = ws + static_cast<int64_t>(ks) * Mrows * n_pad;
        const int64_t n_ws = static_cast<int64_t>(n_blk) * kTileM + q * 32 + lane;
#pragma unroll 1
        for (int c = g; c < MT / 16; c += 4) {
          if (c * 16 >= Mrows) break;
          uint32_t r[16];
          tmem_ld_x16(t_row + c * 16, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c * 16 + j;
            if (m < Mrows) __stcg(my_ws + static_cast<int64_t>(m) * n_pad + n_ws, static_cast<int32_t>(r[j]));
          }
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(stored_bar);
        if (et == 0) {
          if (mbar_wait(stored_bar, 0, abort_flag, &g_kernel_status, kStatusTimeoutSplitK)) {
            const int old = atomicAdd(counters + n_blk, 1);
            *last_flag = (old == split - 1) ? 1 : 0;
            __threadfence_block();
            mbar_arrive(counted_bar);
          }
        }
        ok = mbar_wait(counted_bar, 0, abort_flag, &g_kernel_status, kStatusTimeoutSplitK);
        if (ok && *last_flag) {
          __threadfence();
          // The sum is latency bound (the partials sit in L2), so every thread
          // keeps many independent 16-byte loads in flight: it owns four
          // consecutive channels, the sixteen warps interleave rows, and all
          // splits of a row are read at once.
          const int64_t slab = static_cast<int64_t>(Mrows) * n_pad;
          for (int m0 = ew; m0 < Mrows; m0 += 32) {
            int4 acc[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) acc[r] = make_int4(0, 0, 0, 0);
#pragma unroll
            for (int s = 0; s < kSmallMaxSplit; ++s) {
              if (s < split) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                  const int m = m0 + 16 * r;
                  if (m < Mrows) {
                    const int4 v = __ldcg(reinterpret_cast<const int4*>(
                        ws + s * slab + static_cast<int64_t>(m) * n_pad + n4));
                    acc[r].x += v.x;
                    acc[r].y += v.y;
                    acc[r].z += v.z;
                    acc[r].w += v.w;
                  }
                }
              }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              const int m = m0 + 16 * r;
              if (m < Mrows) {
                if (ctx.has_rs) ctx.rs = __ldg(ep.x_scale + m);
                const int32_t a4[4] = {acc[r].x, acc[r].y, acc[r].z, acc[r].w};
                OutT* orow = out + static_cast<int64_t>(m) * ep.ldo + n4;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  if (n4 + c < ep.N) store_one_rt<OutT>(orow + c, epi_value(a4[c], cs4[c], cb4[c], ctx), a4[c], ctx);
                }
              }
            }
          }
          if (et == 0) counters[n_blk] = 0;  // ready for the next launch
        }
      }
    }
  }

  __syncwarp();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// -------------------------------------------------------------------- simt
template <typename OutT>
__global__ void qgemm_simt_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ w,
                                  int64_t K, int64_t lda, int64_t ldw, EpiParams ep,
                                  int64_t slab_cols, int64_t slab_stride) {
  const int64_t n = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t m = blockIdx.y;
  if (n >= ep.N || m >= ep.M) return;
  const int8_t* ar = a + m * lda;
  const int8_t* wr = w + n * ldw;
  int32_t acc = 0;
  if (slab_cols > 0) {
    for (int64_t k = 0; k < K; ++k) {
      const int64_t s = k / slab_cols;
      acc += static_cast<int32_t>(ar[s * slab_stride + (k - s * slab_cols)]) * static_cast<int32_t>(wr[k]);
    }
  } else {
    for (int64_t k = 0; k < K; ++k) acc += static_cast<int32_t>(ar[k]) * static_cast<int32_t>(wr[k]);
  }
  EpiCtx ctx = make_epi_ctx(ep);
  if (ctx.has_rs) ctx.rs = ep.x_scale[m];
  float cs, cb;
  col_consts(ep, ctx, n, cs, cb);
  store_one_rt<OutT>(reinterpret_cast<OutT*>(ep.out) + m * ep.ldo + n, epi_value(acc, cs, cb, ctx), acc, ctx);
}

// ------------------------------------------------------------------- host
EncodeTiledFn get_encode_fn() { return tensor_map_encode_fn(); }

// int8 [rows, K] row-major (row stride ld bytes), box = box_rows x 128 bytes, 128B swizzle (or 64 and 64).
bool make_tmap(CUtensorMap* tm, const int8_t* base, int64_t rows, int64_t K, int64_t ld,
               int box_rows, int box_bytes = kTileKBytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// int8 image {C, W, H, N} (channels-last), fetched in im2col mode: 128 output positions x `kb_bytes` (128 or
// 64) channels per load, swizzled over the row length (the tile the MMA's K-major descriptor expects).  The
// bounding box of the base positions starts `pad` before the image and ends where the last window still begins.
bool make_im2col_tmap(CUtensorMap* tm, const Im2colA& g, int kb_bytes) {
  EncodeIm2colFn fn = tensor_map_encode_im2col_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(g.in_ch), static_cast<cuuint64_t>(g.in_w),
                        static_cast<cuuint64_t>(g.in_h), static_cast<cuuint64_t>(g.batch)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(g.stride_w), static_cast<cuuint64_t>(g.stride_h),
                           static_cast<cuuint64_t>(g.stride_n)};
  int lower[2] = {-g.pad_left, -g.pad_top};
  int upper[2] = {g.pad_right - (g.k_w - 1) * g.dil_w, g.pad_bottom - (g.k_h - 1) * g.dil_h};
  cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(g.conv_stride_w), static_cast<cuuint32_t>(g.conv_stride_h), 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t*>(g.x), dims, strides, lower, upper,
                  /*channelsPerPixel=*/static_cast<cuuint32_t>(kb_bytes), /*pixelsPerColumn=*/static_cast<cuuint32_t>(kTileM),
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  kb_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int sm_count() { return device_sm_count(); }

EpiParams make_epi(const QGemmParams& p) {
  EpiParams e;
  e.out = p.out;
  e.ldo = p.ldo;
  e.M = p.M;
  e.N = p.N;
  e.x_scale = p.x_scale;
  e.w_scale = p.w_scale;
  e.out_scale = p.out_scale;
  e.bias = p.bias;
  e.x_kind = p.x_scale_kind;
  e.w_kind = p.w_scale_kind;
  e.o_kind = p.out_scale_kind;
  e.bias_kind = p.bias_kind;
  e.fold_out = p.fold_out_scale;
  e.div_out = p.div_out_scale;
  e.div_exact = p.div_exact;
  e.out_kind = p.out_dtype;
  e.act = p.act;
  return e;
}

int out_elem_bytes(int dt) { return dt == kOutI8 ? 1 : (dt == kOutF16 ? 2 : 4); }

bool tma_ok(const QGemmParams& p) {
  if (p.lda <= 0 || p.ldw <= 0) return false;
  if (p.a_slabs > 1 && (p.a_slab_cols % 16 != 0 || p.a_slab_stride % p.lda != 0)) return false;
  return p.K % 16 == 0 && p.lda % 16 == 0 && p.ldw % 16 == 0 &&
         (reinterpret_cast<uintptr_t>(p.a) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.w) & 15) == 0;
}

// The same int8 [rows, K] operand seen as [K / 128 blocks][rows][128 bytes] (K a
// multiple of 128): one box = `box_kb` consecutive K blocks of `box_rows` rows,
// which land in shared memory as `box_kb` consecutive 128B-swizzled tiles.
bool make_tmap_kblocks(CUtensorMap* tm, const int8_t* base, int64_t rows, int64_t K, int64_t ld,
                       int box_rows, int box_kb) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn || K % kTileKBytes != 0) return false;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(kTileKBytes), static_cast<cuuint64_t>(rows),
                        static_cast<cuuint64_t>(K / kTileKBytes)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld), static_cast<cuuint64_t>(kTileKBytes)};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(kTileKBytes), static_cast<cuuint32_t>(box_rows),
                       static_cast<cuuint32_t>(box_kb)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Host view of the slab layout of the activation operand.
bool has_slabs(const QGemmParams& p) { return p.a_slabs > 1; }
SlabA slab_of(const QGemmParams& p) {
  SlabA s = {0, 0, 0};
  if (has_slabs(p)) {
    s.kb_per_slab = static_cast<int>((p.a_slab_cols + kTileKBytes - 1) / kTileKBytes);
    s.slab_rows = static_cast<int>(p.a_slab_stride / p.lda);
    s.slab_cols = static_cast<int>(p.a_slab_cols);
  }
  return s;
}
int num_k_blocks(const QGemmParams& p) {
  if (has_slabs(p)) return p.a_slabs * slab_of(p).kb_per_slab;
  return static_cast<int>((p.K + kTileKBytes - 1) / kTileKBytes);
}
// Activation tensor map: plain [M, K], or all slabs stacked along the rows,
// [(a_slabs - 1) * slab_rows + M, a_slab_cols] (rows past M of a slab are the
// next slab's; they only reach accumulator rows that are never stored).
bool make_a_tmap(CUtensorMap* tm, const QGemmParams& p, int box_rows) {
  if (!has_slabs(p)) return make_tmap(tm, p.a, p.M, p.K, p.lda, box_rows);
  const int64_t rows = (p.a_slabs - 1) * (p.a_slab_stride / p.lda) + p.M;
  return make_tmap(tm, p.a, rows, p.a_slab_cols, p.lda, box_rows);
}

int small_mt(int64_t M) { return M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128)); }

int small_split(const QGemmParams& p) {
  const int num_kb = static_cast<int>((p.K + kTileKBytes - 1) / kTileKBytes);
  if (p.split_k > 0) {
    const int want = p.split_k < kSmallMaxSplit ? p.split_k : kSmallMaxSplit;
    return want < num_kb ? want : num_kb;
  }
  const int tiles_n = static_cast<int>((p.N + kTileM - 1) / kTileM);
  int s = sm_count() / tiles_n;
  if (s < 1) s = 1;
  if (s > kSmallMaxSplit) s = kSmallMaxSplit;
  if (s > num_kb) s = num_kb;
  return s;
}

template <typename OutT, int BN, int STAGES>
cudaError_t launch_tiled_t(const QGemmParams& p, cudaStream_t stream, const char** err) {
  using L = TiledSmem<BN, STAGES>;
  CUtensorMap ta, tw;
  Im2colDev ic{};
  const int kb_bytes = (p.im2col && p.im2col->in_ch % 128 != 0) ? 64 : 128;
  if (p.im2col) {
    if (!make_im2col_tmap(&ta, *p.im2col, kb_bytes)) {
      if (err) *err = "cuTensorMapEncodeIm2col failed or unavailable";
      return cudaErrorInvalidValue;
    }
    const Im2colA& g = *p.im2col;
    ic.enabled = 1;
    ic.pixels_per_image = g.out_h * g.out_w;
    ic.out_w = g.out_w;
    ic.k_w = g.k_w;
    ic.cblks = static_cast<int>(g.in_ch / kb_bytes);
    ic.kb_bytes = kb_bytes;
    ic.stride_h = g.conv_stride_h;
    ic.stride_w = g.conv_stride_w;
    ic.dil_h = g.dil_h;
    ic.dil_w = g.dil_w;
    ic.pad_top = g.pad_top;
    ic.pad_left = g.pad_left;
  } else if (!make_a_tmap(&ta, p, kTileM)) {
    if (err) *err = "cuTensorMapEncodeTiled failed";
    return cudaErrorInvalidValue;
  }
  if (!make_tmap(&tw, p.w, p.N, p.K, p.ldw, BN, kb_bytes)) {
    if (err) *err = "cuTensorMapEncodeTiled failed";
    return cudaErrorInvalidValue;
  }
  auto kern = qgemm_tiled_kernel<BN, STAGES, OutT>;
  cudaError_t st =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
  if (st != cudaSuccess) return st;
  const int tiles_m = static_cast<int>((p.M + kTileM - 1) / kTileM);
  const int tiles_n = static_cast<int>((p.N + BN - 1) / BN);
  const int num_kb = p.im2col ? static_cast<int>(p.K / kb_bytes) : num_k_blocks(p);
  const int64_t tiles = static_cast<int64_t>(tiles_m) * tiles_n;
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  const int eb = out_elem_bytes(p.out_dtype);
  const int vec_ok = ((p.ldo * eb) % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
  return launch_dependent(kern, dim3(grid), dim3(kTiledThreads), L::kDynamic, stream, ta, tw, make_epi(p), num_kb,
                          tiles_m, tiles_n, vec_ok, slab_of(p), ic);
}

template <typename OutT>
cudaError_t launch_tiled(const QGemmParams& p, cudaStream_t stream, const char** err) {
  const int64_t tiles256 = ((p.M + kTileM - 1) / kTileM) * ((p.N + 255) / 256);
  if (tiles256 >= sm_count()) return launch_tiled_t<OutT, 256, 4>(p, stream, err);
  return launch_tiled_t<OutT, 128, 6>(p, stream, err);
}

// Output described in bytes: [M rows, N * elem bytes], box = 32 rows x 64 bytes, 64-byte swizzle.
bool make_out_tmap(CUtensorMap* tm, void* base, int64_t rows, int64_t row_bytes, int64_t ld_bytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_bytes)};
  cuuint32_t box[2] = {64, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <typename OutT>
int pair_max_clusters() {
  static std::atomic<int> cache[kMaxDeviceOrdinals];  // per instantiation and device
  const int dev = current_device_ordinal();
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74);
    cfg.blockDim = dim3(kTiledThreads);
    cfg.dynamicSmemBytes = PairSmem::kDynamic;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int c = 0;
    // every mode of one output type has the same launch shape and resource use
    if (cudaOccupancyMaxActiveClusters(&c, qgemm_pair_kernel<OutT, kActNone, kDivNone, false>, &cfg) != cudaSuccess ||
        c <= 0) {
      (void)cudaGetLastError();
      c = sm_count() / 2;
    }
    n = c;
    cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

template <typename OutT, int ACT, int DIV, bool RS>
cudaError_t launch_pair_mode(const QGemmParams& p, cudaStream_t stream, const char** err) {
  CUtensorMap ta, tw, to;
  if (!make_a_tmap(&ta, p, kTileM) || !make_tmap(&tw, p.w, p.N, p.K, p.ldw, kTileM)) {
    if (err) *err = "cuTensorMapEncodeTiled failed";
    return cudaErrorInvalidValue;
  }
  const int eb = out_elem_bytes(p.out_dtype);
  const bool out_aligned =
      ((p.ldo * eb) % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
  int use_tma_store = out_aligned ? 1 : 0;
  if (!use_tma_store || !make_out_tmap(&to, p.out, p.M, p.N * eb, p.ldo * eb)) {
    use_tma_store = 0;
    to = ta;  // never dereferenced when stores are direct
  }
  auto kern = qgemm_pair_kernel<OutT, ACT, DIV, RS>;
  cudaError_t st =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::kDynamic);
  if (st != cudaSuccess) return st;
  const int tiles_m = static_cast<int>((p.M + 2 * kTileM - 1) / (2 * kTileM));
  const int tiles_n = static_cast<int>((p.N + kPairBN - 1) / kPairBN);
  const int num_kb = num_k_blocks(p);
  const int64_t tiles = static_cast<int64_t>(tiles_m) * tiles_n;
  const int max_clusters = pair_max_clusters<OutT>();
  const int clusters = static_cast<int>(tiles < max_clusters ? tiles : max_clusters);
  return launch_dependent(kern, dim3(2 * clusters), dim3(kTiledThreads), PairSmem::kDynamic, stream, ta, tw, to,
                          make_epi(p), num_kb, tiles_m, tiles_n, use_tma_store, out_aligned ? 1 : 0, slab_of(p));
}

// Host-side view of the epilogue mode a launch asks for.
int host_epi_mode(const QGemmParams& p) {
  const int div = p.div_out_scale ? (p.div_exact ? kDivExact : kDivRecip) : kDivNone;
  return p.act | (div << 2) | (p.x_scale_kind == kScalePerRow ? 16 : 0);
}

// The pair kernel exists for the modes each output type is used with: every
// mode for int8, no division for the floating-point outputs, the raw sum for
// int32 (qgemm_choose_path sends other combinations to the single-CTA kernel).
template <typename OutT>
cudaError_t launch_pair(const QGemmParams& p, cudaStream_t stream, const char** err) {
  if constexpr (std::is_same_v<OutT, int32_t>) {
    return launch_pair_mode<OutT, kActNone, kDivNone, false>(p, stream, err);
  } else if constexpr (std::is_same_v<OutT, int8_t>) {
    DISC_EPI_SWITCH(host_epi_mode(p), return (launch_pair_mode<OutT, ACT, DIV, RS>(p, stream, err)))
  } else {
    switch (host_epi_mode(p)) {
      DISC_EPI_CASE(0, 0, false, return (launch_pair_mode<OutT, ACT, DIV, RS>(p, stream, err)))
      DISC_EPI_CASE(1, 0, false, return (launch_pair_mode<OutT, ACT, DIV, RS>(p, stream, err)))
      DISC_EPI_CASE(2, 0, false, return (launch_pair_mode<OutT, ACT, DIV, RS>(p, stream, err)))
      DISC_EPI_CASE(0, 0, true, return (launch_pair_mode<OutT, ACT, DIV, RS>(p, stream, err)))
      DISC_EPI_CASE(1, 0, true, return (launch_pair_mode<OutT, ACT, DIV, RS>(p, stream, err)))
      DISC_EPI_CASE(2, 0, true, return (launch_pair_mode<OutT, ACT, DIV, RS>(p, stream, err)))
      default: break;
    }
  }
  if (err) *err = "pair qgemm path: epilogue mode not available for this output type";
  return cudaErrorInvalidValue;
}

template <typename OutT>
cudaError_t launch_smallm(const QGemmParams& p, cudaStream_t stream, const char** err) {
  const int MT = small_mt(p.M);
  const int split = small_split(p);
  const int tiles_n = static_cast<int>((p.N + kTileM - 1) / kTileM);
  const int num_kb = static_cast<int>((p.K + kTileKBytes - 1) / kTileKBytes);
  const int kbs = 4;            // K blocks per pipeline stage
  const int box_rows = kTileM;  // weight rows per TMA box
  const int stage_bytes = kbs * (kTileM + MT) * kTileKBytes;
  int stages = kSmallBarOffset / stage_bytes;
  if (stages > kSmallMaxStages) stages = kSmallMaxStages;
  int32_t* ws = nullptr;
  int32_t* counters = nullptr;
  if (split > 1) {
    const int64_t n_pad = static_cast<int64_t>(tiles_n) * kTileM;
    const int64_t need = (static_cast<int64_t>(split) * p.M * n_pad + kSplitCounterWords) * 4;
    if (!p.splitk_ws || p.splitk_ws_bytes < need || tiles_n > kSplitCounterWords) {
      if (err) *err = "small-M qgemm: split-K scratch missing or too small";
      return cudaErrorInvalidValue;
    }
    // The arrival counters own a fixed region at the front (they must stay zero
    // between launches); partial sums of any launch shape live behind it.
    counters = p.splitk_ws;
    ws = p.splitk_ws + kSplitCounterWords;
  }
  CUtensorMap tw, tx;
  if (!make_tmap(&tw, p.w, p.N, p.K, p.ldw, box_rows) || !make_tmap(&tx, p.a, p.M, p.K, p.lda, MT)) {
    if (err) *err = "cuTensorMapEncodeTiled failed";
    return cudaErrorInvalidValue;
  }
  auto kern = qgemm_smallm_kernel<OutT>;
  cudaError_t st =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmallDynamic);
  if (st != cudaSuccess) return st;
  dim3 grid(tiles_n, split);
  kern<<<grid, kThreads, kSmallDynamic, stream>>>(tw, tx, make_epi(p), MT, stages, num_kb, ws,
                                                  counters, kbs, box_rows);
  return cudaGetLastError();
}

template <typename OutT>
cudaError_t launch_simt(const QGemmParams& p, cudaStream_t stream, const char** err) {
  if (p.M > 65535) {
    if (err) *err = "simt qgemm path: M too large";
    return cudaErrorInvalidValue;
  }
  dim3 block(128);
  dim3 grid(static_cast<unsigned>((p.N + 127) / 128), static_cast<unsigned>(p.M));
  qgemm_simt_kernel<OutT><<<grid, block, 0, stream>>>(p.a, p.w, p.K, p.lda, p.ldw, make_epi(p),
                                                      p.a_slabs > 1 ? p.a_slab_cols : 0, p.a_slab_stride);
  return cudaGetLastError();
}

#include "qgemm_gemv.inl"
#include "qgemm_skinny.inl"

// Channels per CTA of the few-row path: one wave of CTAs over N (per row tile).
int skinny_bn(const QGemmParams& p) {
  const int64_t tiles_m = (p.M + kTileM - 1) / kTileM;
  int64_t ctas = sm_count() / tiles_m;
  if (ctas < 1) ctas = 1;
  int64_t bn = (p.N + ctas - 1) / ctas;
  bn = (bn + 15) / 16 * 16;
  if (bn < 16) bn = 16;
  // Blocks wider than 128 channels where they save a wave: one row tile whose N would otherwise take a second
  // wave here, or several row tiles whose 256 x 256 pair tiles would take a second wave there
  // (333 x 4096 x 11008: 86 pair tiles on 74 SM pairs, 26.5 us; 138 blocks of 240 channels here, 20.3 us).
  // With one wave of pair tiles the pair kernel is ahead (256 x 4096 x 11008: 17.0 against 18.2 us).
  const int64_t pair_tiles = ((p.M + 255) / 256) * ((p.N + 255) / 256);
  const int64_t cap = (tiles_m == 1 || pair_tiles > sm_count() / 2) ? kSkinnyMaxBN : 128;
  if (bn > cap) bn = cap;
  return static_cast<int>(bn);
}

// Clusters of `ks` blocks of the few-row kernel the current device holds at once (asked once per device and size).
template <typename OutT>
int skinny_max_clusters(int ks) {
  static std::atomic<int> cache[kMaxDeviceOrdinals][5];
  const int dev = current_device_ordinal();
  int n = cache[dev][ks].load(std::memory_order_relaxed);
  if (n != 0) return n < 0 ? 0 : n;
  auto kern = qgemm_skinny_kernel<OutT>;
  int active = 0;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSkinnyDynamic) == cudaSuccess) {
    cudaLaunchConfig_t q{};
    q.gridDim = dim3(1, 1, static_cast<unsigned>(ks));
    q.blockDim = dim3(kThreads);
    q.dynamicSmemBytes = kSkinnyDynamic;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 1;
    qa[0].val.clusterDim.y = 1;
    qa[0].val.clusterDim.z = static_cast<unsigned>(ks);
    q.attrs = qa;
    q.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&active, kern, &q) != cudaSuccess) {
      (void)cudaGetLastError();
      active = 0;
    }
  }
  cache[dev][ks].store(active > 0 ? active : -1, std::memory_order_relaxed);
  return active;
}

template <typename OutT>
cudaError_t launch_skinny(const QGemmParams& p, cudaStream_t stream, const char** err) {
  const int MT = p.M > 64 ? kTileM : small_mt(p.M);
  int BN = skinny_bn(p);
  // Long K, few tiles: a block's time is its K range (0.2 - 0.35 us per 128-byte K block, whatever the tile's
  // width), so K is cut over a thread-block cluster of 4, 3 or 2 blocks with 128 channels each, as long as every
  // cluster is resident at once.  The exchange costs about 3 us, so fewer ranks need a longer K to pay
  // (measured, f16 out: 64 x 4096 x 4096 over 4: 9.4 -> 8.2 us; 64 x 11008 x 4096 over 4: 20.0 -> 13.1 us;
  // 64 x 8192 x 8192 over 2: 20.5 -> 16.7 us; 64 x 4096 x 5120 over 3: 9.5 -> 10.0 us, not taken; several row
  // tiles: 256 x 11008 x 2048 over 4: 25.8 -> 15.1 us, 512 x 8192 x 1024 over 4: 19.9 -> 12.8 us,
  // 256 x 11008 x 4096 over 2: 26.5 -> 23.3 us).  More blocks than SMs lose to the exchange at every K measured.
  int ksplit = 1;
  const int64_t tiles_m = (p.M + kTileM - 1) / kTileM;
  if (!has_slabs(p)) {
    static constexpr int64_t kMinK[5] = {0, 0, 8192, 6144, 4096};
    const int64_t strips = ((p.N + 127) / 128) * tiles_m;
    for (int ks = 4; ks >= 2; --ks) {
      if (p.K >= kMinK[ks] && strips * ks <= sm_count() && strips <= skinny_max_clusters<OutT>(ks)) {
        ksplit = ks;
        BN = 128;
        break;
      }
    }
  }
  // K blocks per stage: as many as leave at least three stages in flight.
  int kbs = 4;
  while (kbs > 1 && 3 * kbs * (BN + MT) * kTileKBytes > kSkinnyStageRegion) kbs >>= 1;
  int stages = kSkinnyStageRegion / (kbs * (BN + MT) * kTileKBytes);
  if (stages > 4) stages = 4;  // 100+ KB in flight per SM is plenty; more only delays the start
  CUtensorMap tx, tw;
  // One box per operand and stage when K is a whole number of 128-byte blocks.
  const int k3d = (p.K % kTileKBytes == 0 && !has_slabs(p)) ? 1 : 0;
  const bool maps_ok =
      k3d ? (make_tmap_kblocks(&tx, p.a, p.M, p.K, p.lda, MT, kbs) &&
             make_tmap_kblocks(&tw, p.w, p.N, p.K, p.ldw, BN, kbs))
          : (make_a_tmap(&tx, p, MT) && make_tmap(&tw, p.w, p.N, p.K, p.ldw, BN));
  if (!maps_ok) {
    if (err) *err = "cuTensorMapEncodeTiled failed";
    return cudaErrorInvalidValue;
  }
  auto kern = qgemm_skinny_kernel<OutT>;
  cudaError_t st =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSkinnyDynamic);
  if (st != cudaSuccess) return st;
  const int num_kb = num_k_blocks(p);
  const int eb = out_elem_bytes(p.out_dtype);
  const int vec_ok = ((p.ldo * eb) % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
  const int kb_per_rank = ((num_kb + ksplit - 1) / ksplit + kbs - 1) / kbs * kbs;  // whole stages
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>((p.N + BN - 1) / BN), static_cast<unsigned>((p.M + kTileM - 1) / kTileM),
                     static_cast<unsigned>(ksplit));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSkinnyDynamic;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = 1;
  attrs[1].id = cudaLaunchAttributeClusterDimension;
  attrs[1].val.clusterDim.x = 1;
  attrs[1].val.clusterDim.y = 1;
  attrs[1].val.clusterDim.z = static_cast<unsigned>(ksplit);
  cfg.attrs = attrs;
  cfg.numAttrs = ksplit > 1 ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, tx, tw, make_epi(p), MT, BN, stages, kbs, num_kb, vec_ok, k3d, slab_of(p),
                            p.weights_static ? 1 : 0, kb_per_rank);
}

template <typename OutT>
cudaError_t dispatch(const QGemmParams& p, int path, cudaStream_t stream, const char** err) {
  switch (path) {
    case kPathGemv: return launch_gemv<OutT>(p, stream, err);
    case kPathSkinny: return launch_skinny<OutT>(p, stream, err);
    case kPathTiled: return launch_tiled<OutT>(p, stream, err);
    case kPathSmallM: return launch_smallm<OutT>(p, stream, err);
    case kPathPair: return launch_pair<OutT>(p, stream, err);
    default: return launch_simt<OutT>(p, stream, err);
  }
}

}  // namespace

// The CTA-pair kernel is built for the epilogue modes in use (see launch_pair).
static bool pair_mode_ok(const QGemmParams& p) {
  if (p.act < kActNone || p.act > kActSilu) return false;
  return p.out_dtype == kOutI8 || !p.div_out_scale;
}

int qgemm_choose_path(const QGemmParams& p) {
  if (p.im2col) return kPathTiled;  // the only kernel whose producer fetches image tiles
  if (!tma_ok(p)) return kPathSimt;
  if (p.path == kPathSimt) return kPathSimt;
  if (p.path == kPathSmallM && p.M <= 128 && p.a_slabs <= 1) return kPathSmallM;
  if (p.path == kPathTiled) return kPathTiled;
  if (p.path == kPathPair) return pair_mode_ok(p) ? kPathPair : kPathTiled;
  if (p.path == kPathSkinny && p.M <= 65535 * kTileM) return kPathSkinny;
  if (p.path == kPathGemv && p.M <= 8 && p.K <= kGemvMaxK && p.a_slabs <= 1) return kPathGemv;
  // One to a few rows: the dp4a stream; from five rows on a large weight is
  // cheaper through the tensor cores.  (Back to back with itself the tensor-core stream is also 0.4 - 1.2 us
  // ahead at one to four rows of a weight of 32 MB or more, because consecutive launches overlap their
  // prologues; between the row kernels of a decoder step it is behind: 8 layers at batch 1 0.59 -> 0.67 ms.)
  const bool slabs = p.a_slabs > 1;  // read by the TMA paths (and the fallback) only
  if (!slabs && p.M <= 8 && p.K <= kGemvMaxK && (p.M <= 4 || p.N * p.K < (int64_t{1} << 25)))
    return kPathGemv;
  // Few rows: fine channel blocks over the full K, as long as one wave of CTAs
  // covers the output.
  const int64_t skinny_ctas = ((p.N + skinny_bn(p) - 1) / skinny_bn(p)) * ((p.M + kTileM - 1) / kTileM);
  if (p.M <= 128 || (p.M <= 1024 && skinny_ctas <= sm_count())) return kPathSkinny;
  // CTA pairs compute 256 x 256 tiles and move a third less data per operation
  // than single-CTA tiles, which are bound by the L2 feed for long K: they win
  // as soon as a quarter of the SM pairs have a tile.
  const int64_t pair_tiles = ((p.M + 255) / 256) * ((p.N + 255) / 256);
  return pair_tiles >= sm_count() / 4 && pair_mode_ok(p) ? kPathPair : kPathTiled;
}

int64_t qgemm_splitk_ws_bytes(int64_t M, int64_t N, int64_t K) {
  if (M > 128) return 0;
  const int64_t tiles_n = (N + kTileM - 1) / kTileM;
  const int64_t num_kb = (K + kTileKBytes - 1) / kTileKBytes;
  int64_t split = num_kb < 8 ? num_kb : 8;
  return (split * M * tiles_n * kTileM + kSplitCounterWords) * 4;
}

cudaError_t qgemm_launch(const QGemmParams& p, cudaStream_t stream, const char** err) {
  if (err) *err = nullptr;
  if (p.M <= 0 || p.N <= 0) return cudaSuccess;  // empty result
  if (p.K <= 0 || !p.a || !p.w || !p.out) {
    if (err) *err = "qgemm: null operand or K <= 0";
    return cudaErrorInvalidValue;
  }
  if (p.M > 0x7fffffff || p.N > 0x7fffffff || p.K > 0x7fffffff) {
    if (err) *err = "qgemm: extent exceeds 2^31-1";
    return cudaErrorInvalidValue;
  }
  if ((p.fold_out_scale || p.div_out_scale) && !p.out_scale) {
    if (err) *err = "qgemm: out_scale required";
    return cudaErrorInvalidValue;
  }
  if (p.div_out_scale && p.out_scale_kind == kScalePerCol) {
    if (err) *err = "qgemm: per-channel out_scale only in folded form";
    return cudaErrorInvalidValue;
  }
  if (p.a_slabs > 1 && (p.a_slab_cols <= 0 || p.lda <= 0 || p.a_slab_cols > p.lda ||
                        p.a_slabs * p.a_slab_cols != p.K)) {
    if (err) *err = "qgemm: K must equal a_slabs * a_slab_cols (and a_slab_cols <= lda)";
    return cudaErrorInvalidValue;
  }
  const int path = qgemm_choose_path(p);
  switch (p.out_dtype) {
    case kOutI8: return dispatch<int8_t>(p, path, stream, err);
    case kOutF16: return dispatch<__half>(p, path, stream, err);
    case kOutF32: return dispatch<float>(p, path, stream, err);
    case kOutI32: return dispatch<int32_t>(p, path, stream, err);
    default:
      if (err) *err = "qgemm: unknown out_dtype";
      return cudaErrorInvalidValue;
  }
}

// ------------------------------------------------ small-M without allocation
// Some hosts of this library cannot give the small-M path its split-K scratch:
// code running while a CUDA graph is being captured, a serving loop that has
// handed the whole device heap to its own pool, a callback on a thread where
// cudaMalloc would serialise against the rest of the process.  For them the
// scratch lives here, in the library's own image: every GPU that loads the
// library carries these bytes until the process exits.
constexpr int64_t kStaticScratchBytes = 8ll << 20;
static __device__ __align__(256) unsigned char g_static_splitk_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {};

// Device address of the array for the current device.  In host code the
// array's name is only a handle for the runtime, never a device pointer, so the
// address is asked for once per device (with that device current) and cached.
cudaError_t static_scratch_address(void** out, const char** err) {
  int dev = -1;
  cudaError_t st = cudaGetDevice(&dev);
  if (st != cudaSuccess) return st;
  if (dev < 0 || dev >= kMaxDevices) {
    if (err) *err = "no-alloc small-M qgemm: device ordinal out of range";
    return cudaErrorInvalidDevice;
  }
  std::lock_guard<std::mutex> l(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    st = cudaGetSymbolAddress(&p, g_static_splitk_scratch);
    if (st != cudaSuccess) {
      if (err) *err = "no-alloc small-M qgemm: cudaGetSymbolAddress failed";
      return st;
    }
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return cudaSuccess;
}
}  // namespace

int64_t qgemm_small_m_noalloc_capacity() { return kStaticScratchBytes; }

cudaError_t qgemm_small_m_noalloc_launch(const QGemmParams& in, cudaStream_t stream, const char** err) {
  if (err) *err = nullptr;
  if (in.M <= 0 || in.N <= 0) return cudaSuccess;
  if (in.K <= 0 || !in.a || !in.w || !in.out) {
    if (err) *err = "no-alloc small-M qgemm: null operand or K <= 0";
    return cudaErrorInvalidValue;
  }
  if (in.M > 128) {
    if (err) *err = "no-alloc small-M qgemm: more than 128 activation rows";
    return cudaErrorInvalidValue;
  }
  if (in.N > 0x7fffffff || in.K > 0x7fffffff) {
    if (err) *err = "no-alloc small-M qgemm: extent exceeds 2^31-1";
    return cudaErrorInvalidValue;
  }
  // The small-M kernel reads a plain row-major activation: the gathered slab
  // layout would be taken for overlapping rows, so it is refused here (the
  // regular entry point routes slabs to other kernels).
  if (in.a_slabs > 1) {
    if (err) *err = "no-alloc small-M qgemm: the gathered (slab) activation layout is not supported";
    return cudaErrorInvalidValue;
  }
  if (in.lda < in.K || in.ldw < in.K || in.ldo < in.N) {
    if (err) *err = "no-alloc small-M qgemm: a row stride is smaller than the row";
    return cudaErrorInvalidValue;
  }
  if (!tma_ok(in)) {
    if (err) *err = "no-alloc small-M qgemm: K and the row strides must be multiples of 16, bases 16-byte aligned";
    return cudaErrorInvalidValue;
  }
  if ((in.fold_out_scale || in.div_out_scale) && !in.out_scale) {
    if (err) *err = "no-alloc small-M qgemm: out_scale required";
    return cudaErrorInvalidValue;
  }
  if (in.div_out_scale && in.out_scale_kind == kScalePerCol) {
    if (err) *err = "no-alloc small-M qgemm: per-channel out_scale only in folded form";
    return cudaErrorInvalidValue;
  }
  QGemmParams p = in;
  p.path = kPathSmallM;
  const int split = small_split(p);
  const int64_t tiles_n = (p.N + kTileM - 1) / kTileM;
  const int64_t need = (static_cast<int64_t>(split) * p.M * tiles_n * kTileM + kSplitCounterWords) * 4;
  if (split > 1 && (need > kStaticScratchBytes || tiles_n > kSplitCounterWords)) {
    if (err) *err = "no-alloc small-M qgemm: problem needs more than the 8 MiB built-in scratch";
    return cudaErrorInvalidValue;
  }
  void* scratch = nullptr;
  cudaError_t st = static_scratch_address(&scratch, err);
  if (st != cudaSuccess) return st;
  // The arrival counters must start at zero; an earlier launch that was cut
  // short could have left them otherwise.  Stream-ordered, no allocation.
  st = cudaMemsetAsync(scratch, 0, kSplitCounterWords * sizeof(int32_t), stream);
  if (st != cudaSuccess) return st;
  p.splitk_ws = static_cast<int32_t*>(scratch);
  p.splitk_ws_bytes = kStaticScratchBytes;
  switch (p.out_dtype) {
    case kOutI8: return launch_smallm<int8_t>(p, stream, err);
    case kOutF16: return launch_smallm<__half>(p, stream, err);
    case kOutF32: return launch_smallm<float>(p, stream, err);
    case kOutI32: return launch_smallm<int32_t>(p, stream, err);
    default:
      if (err) *err = "no-alloc small-M qgemm: unknown out_dtype";
      return cudaErrorInvalidValue;
  }
}

// ------------------------------------------------------ wait-expiry self-test
// One warp waits, with the kernels' own bounded wait, on a barrier that nobody
// will ever arrive on: nothing is in flight (no copies, no TMEM), the wait runs
// out after `limit_ns`, records its code in the status word and the kernel
// returns.  It shows on a live GPU what a broken pipeline would do: give up and
// report, never spin on.
namespace {
__global__ void wait_expiry_selftest_kernel(uint64_t limit_ns, long long* waited_ns) {
  __shared__ __align__(8) uint64_t bar_storage;
  __shared__ int abort_flag_storage;
  const uint32_t bar = smem_u32(&bar_storage);
  volatile int* abort_flag = &abort_flag_storage;
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const uint64_t t0 = global_timer_ns();
  const bool ok = mbar_wait_limited(bar, 0, abort_flag, &g_kernel_status, kStatusTimeoutSelfTest, limit_ns);
  if (threadIdx.x == 0) waited_ns[0] = ok ? -1 : static_cast<long long>(global_timer_ns() - t0);
}
}  // namespace

cudaError_t wait_expiry_selftest(uint64_t limit_ns, long long* waited_ns_host, cudaStream_t stream, const char** err) {
  if (err) *err = nullptr;
  if (limit_ns == 0 || limit_ns > 100000000ull || !waited_ns_host) {   // at most 100 ms: this is a test, not a sleep
    if (err) *err = "wait self-test: limit must be 1 ns .. 100 ms and the result pointer set";
    return cudaErrorInvalidValue;
  }
  long long* d = nullptr;
  cudaError_t st = cudaMalloc(&d, sizeof(long long));
  if (st != cudaSuccess) return st;
  wait_expiry_selftest_kernel<<<1, 32, 0, stream>>>(limit_ns, d);
  st = cudaGetLastError();
  if (st == cudaSuccess) st = cudaStreamSynchronize(stream);
  if (st == cudaSuccess) st = cudaMemcpy(waited_ns_host, d, sizeof(long long), cudaMemcpyDeviceToHost);
  cudaFree(d);
  return st;
}

int kernel_status_fetch_and_clear() {
  int h = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&h, g_kernel_status, sizeof(int)) != cudaSuccess) return -1;
  if (h != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_kernel_status, &z, sizeof(int));
  }
  const int r = rowops_status_fetch_and_clear();
  const int a = attention_status_fetch_and_clear();
  const int w = woq_tc_status_fetch_and_clear();
  return h != 0 ? h : (r != 0 ? r : (a != 0 ? a : w));
}

}  // namespace disc_b200
