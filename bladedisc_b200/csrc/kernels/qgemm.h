// Host-side description of one quantized-linear launch.  Plain C types only so
// that the C-ABI layer can fill it in directly.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace disc_b200 {

enum QGemmOut : int { kOutI8 = 0, kOutF16 = 1, kOutF32 = 2, kOutI32 = 3 };
enum QGemmAct : int { kActNone = 0, kActGelu = 1, kActSilu = 2 };
enum QGemmBias : int { kBiasNone = 0, kBiasF32 = 1, kBiasI8 = 2 };
enum ScaleKind : int { kScaleNone = 0, kScaleScalar = 1, kScalePerCol = 2, kScalePerRow = 3 };
enum QGemmPath : int {
  kPathAuto = 0,
  kPathTiled = 1,   // one CTA per 128 x BN tile
  kPathSmallM = 2,  // operands swapped, optional split-K (M <= 128)
  kPathSimt = 3,    // shapes TMA cannot address
  kPathPair = 4,    // CTA pairs, 256 x 256 tiles
  kPathGemv = 5,    // M <= 8: dp4a matrix-vector stream
  kPathSkinny = 6   // few rows: BN = 16..256 channels per CTA over the full K, or K cut over a thread-block cluster
};

// out[m, n] = epilogue( sum_k a[m, k] * w[n, k] ), a and w int8, K-contiguous.
//
//   t  = float(acc) (* x_scale[m] when x_scale_kind == per-row)
//   cs = x_scale(n) * w_scale(n)            (x_scale omitted when per-row)
//   cs = cs / out_scale(n)                  when fold_out_scale (the reference's
//                                           host-side "kernel scale", computed here
//                                           on the device in the same order)
//   v  = fma(t, cs, bias[n]);  v = act(v)
//   v  = v / out_scale                      when div_out_scale (quantize-op form);
//                                           as v * (1 / out_scale) unless div_exact,
//                                           which differs from the quotient by at most
//                                           one int8 level, at rounding ties only
//   out = int8: sat(rne(v)) | f16 | f32 ; kOutI32 stores acc unchanged.
// Activation operand read straight from a channels-last int8 image (implicit GEMM of a convolution): row m of
// the product is the output pixel (n, oy, ox), its K index ((ky * k_w + kx) * in_ch + c).  The tiles are
// fetched by TMA in im2col mode, so the [pixels, k_h * k_w * in_ch] matrix never exists.  in_ch must be a
// multiple of 64: a K block is 128 channels of one window position, or 64 when in_ch is not a multiple of 128.
struct Im2colA {
  const int8_t* x;                        // element strides below; the channel stride is 1
  int64_t batch, in_h, in_w, in_ch;
  int64_t stride_n, stride_h, stride_w;   // of x, in elements (= bytes), multiples of 16
  int out_h, out_w, k_h, k_w;
  int conv_stride_h, conv_stride_w, dil_h, dil_w;
  int pad_top, pad_left, pad_bottom, pad_right;
};

struct QGemmParams {
  const int8_t* a;
  const int8_t* w;
  void* out;
  int64_t M, N, K;
  int64_t lda, ldw, ldo;  // row strides in elements
  const float* x_scale;
  const float* w_scale;
  const float* out_scale;
  const void* bias;
  int x_scale_kind;    // ScaleKind (scalar | per-col | per-row | none = 1.0)
  int w_scale_kind;    // scalar | per-col | none
  int out_scale_kind;  // scalar | per-col (fold only) | none
  int bias_kind;       // QGemmBias
  int fold_out_scale;
  int div_out_scale;
  int div_exact;  // with div_out_scale: the correctly rounded IEEE quotient instead of the reciprocal product
  int act;        // QGemmAct
  int out_dtype;  // QGemmOut
  int path;       // QGemmPath (tests force a path; callers leave kPathAuto)
  int split_k;    // small-M path: 0 = choose
  // Scratch for the small-M split-K reduction: 4096 int32 arrival counters
  // (zero on entry, left zero on exit), then int32 partial sums (need no
  // clearing).  Needed only when the launch splits K.
  int32_t* splitk_ws;
  int64_t splitk_ws_bytes;
  // Activation operand stored as `a_slabs` column slabs, the layout an
  // all-gather of column-parallel outputs leaves behind: element (m, k) lives at
  // a[(k / a_slab_cols) * a_slab_stride + m * lda + k % a_slab_cols], with
  // K = a_slabs * a_slab_cols.  a_slabs <= 1 means plain row-major.  Slabs need
  // a_slab_cols and lda multiples of 16 and a_slab_stride a multiple of lda.
  int a_slabs;
  int64_t a_slab_cols;
  int64_t a_slab_stride;
  // The weight (and nothing else) was final before the previous kernel on the
  // stream was launched, as inference weights are: the few-row paths then
  // start fetching it while that kernel still runs (programmatic dependent
  // launch) and wait for it only before they touch activations, scales or the
  // output.  0 = assume nothing.
  int weights_static;
  // Non-null: `a` is not read; the activation tiles come from this image (tiled kernel only; K must equal
  // k_h * k_w * in_ch and M batch * out_h * out_w).
  const Im2colA* im2col = nullptr;
};

// Bytes of zeroed scratch the small-M path may need for a given problem.
int64_t qgemm_splitk_ws_bytes(int64_t M, int64_t N, int64_t K);

// Launches on `stream`.  Returns cudaSuccess or the first error; `err` (if not
// null) receives a static description for argument errors.
cudaError_t qgemm_launch(const QGemmParams& p, cudaStream_t stream, const char** err);

// Small-M path with the split-K scratch taken from an array built into the
// library instead of from the caller (p.splitk_ws is ignored).  Allocates
// nothing; rejects M > 128, TMA-unfriendly shapes and problems whose partial
// sums exceed qgemm_small_m_noalloc_capacity() bytes.
cudaError_t qgemm_small_m_noalloc_launch(const QGemmParams& p, cudaStream_t stream, const char** err);
int64_t qgemm_small_m_noalloc_capacity();

// Which path kPathAuto resolves to (exposed for tests and the bench).
int qgemm_choose_path(const QGemmParams& p);

// Self-test of the bounded waits: launches one warp that waits `limit_ns` (at most 100 ms) on a barrier nobody
// arrives on, synchronises, and stores how long the wait lasted (-1 if it did not run out).  The status word
// then holds the self-test's code (9) until kernel_status_fetch_and_clear() reads it.
cudaError_t wait_expiry_selftest(uint64_t limit_ns, long long* waited_ns_host, cudaStream_t stream, const char** err);

// Reads and clears the device status word the kernels set when a bounded wait
// ran out (0 = ok).  Synchronises the device.
int kernel_status_fetch_and_clear();

}  // namespace disc_b200
