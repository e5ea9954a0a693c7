// Quantized convolution as gather + quantized linear (see qconv.h).
#include "qconv.h"

#include <cstring>

#include "qgemm.h"
#include "sm100_ptx.cuh"

namespace disc_b200 {
namespace {

constexpr int kChunk = 16;  // bytes of a matrix row one thread produces

__host__ __device__ inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// Row m = (n, oy, ox) of the gathered matrix, columns ordered (ky, kx, c); columns
// at or beyond k_h * k_w * in_ch are zero.  One thread writes 16 consecutive columns.
// `vec`: channels are contiguous in the input, a multiple of 16, and every pixel
// starts on a 16-byte boundary, so that the 16 columns are one aligned load.
__global__ void __launch_bounds__(256) qconv_gather_kernel(ConvGeometry g, const int8_t* __restrict__ x,
                                                           int8_t* __restrict__ a, int64_t rows, int64_t kp, int vec) {
  grid_dep_launch();
  grid_dep_wait();
  const int64_t chunks = kp / kChunk;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= rows * chunks) return;
  const int64_t m = t / chunks;
  const int64_t k0 = (t - m * chunks) * kChunk;
  const int64_t ox = m % g.out_w;
  const int64_t oy = (m / g.out_w) % g.out_h;
  const int64_t n = m / (g.out_w * g.out_h);
  const int64_t k_total = g.k_h * g.k_w * g.in_ch;
  const int8_t* xn = x + n * g.x_stride[0];
  uint4 packed = make_uint4(0u, 0u, 0u, 0u);
  if (vec) {
    if (k0 < k_total) {
      const int64_t c = k0 % g.in_ch;
      const int64_t kx = (k0 / g.in_ch) % g.k_w;
      const int64_t ky = k0 / (g.in_ch * g.k_w);
      const int64_t iy = oy * g.stride_h - g.pad_top + ky * g.dil_h;
      const int64_t ix = ox * g.stride_w - g.pad_left + kx * g.dil_w;
      if (iy >= 0 && iy < g.in_h && ix >= 0 && ix < g.in_w) {
        packed = __ldg(reinterpret_cast<const uint4*>(xn + iy * g.x_stride[2] + ix * g.x_stride[3] + c));
      }
    }
  } else {
    uint32_t words[4] = {0u, 0u, 0u, 0u};
    for (int j = 0; j < kChunk; ++j) {
      const int64_t k = k0 + j;
      if (k >= k_total) break;
      const int64_t c = k % g.in_ch;
      const int64_t kx = (k / g.in_ch) % g.k_w;
      const int64_t ky = k / (g.in_ch * g.k_w);
      const int64_t iy = oy * g.stride_h - g.pad_top + ky * g.dil_h;
      const int64_t ix = ox * g.stride_w - g.pad_left + kx * g.dil_w;
      if (iy >= 0 && iy < g.in_h && ix >= 0 && ix < g.in_w) {
        const uint32_t v = static_cast<uint8_t>(xn[c * g.x_stride[1] + iy * g.x_stride[2] + ix * g.x_stride[3]]);
        words[j >> 2] |= v << (8 * (j & 3));
      }
    }
    packed = make_uint4(words[0], words[1], words[2], words[3]);
  }
  *reinterpret_cast<uint4*>(a + m * kp + k0) = packed;
}

// Kernel [out_ch, (ky, kx, c)] with rows padded to kp, from any layout.
__global__ void __launch_bounds__(256) qconv_pack_weight_kernel(ConvGeometry g, const int8_t* __restrict__ w,
                                                                int8_t* __restrict__ wp, int64_t kp) {
  grid_dep_launch();
  grid_dep_wait();
  const int64_t chunks = kp / kChunk;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= g.out_ch * chunks) return;
  const int64_t o = t / chunks;
  const int64_t k0 = (t - o * chunks) * kChunk;
  const int64_t k_total = g.k_h * g.k_w * g.in_ch;
  uint32_t words[4] = {0u, 0u, 0u, 0u};
  for (int j = 0; j < kChunk; ++j) {
    const int64_t k = k0 + j;
    if (k >= k_total) break;
    const int64_t c = k % g.in_ch;
    const int64_t kx = (k / g.in_ch) % g.k_w;
    const int64_t ky = k / (g.in_ch * g.k_w);
    const uint32_t v =
        static_cast<uint8_t>(w[o * g.w_stride[0] + c * g.w_stride[1] + ky * g.w_stride[2] + kx * g.w_stride[3]]);
    words[j >> 2] |= v << (8 * (j & 3));
  }
  *reinterpret_cast<uint4*>(wp + o * kp + k0) = make_uint4(words[0], words[1], words[2], words[3]);
}

// Channels-last product [rows, out_ch] -> the output's own layout.  Threads run
// over the output in (n, o, y, x) order, the memory order of a channels-first result.
__global__ void __launch_bounds__(256) qconv_scatter_kernel(ConvGeometry g, const int8_t* __restrict__ d,
                                                            int8_t* __restrict__ out, int64_t total) {
  grid_dep_launch();
  grid_dep_wait();
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const int64_t ox = t % g.out_w;
  const int64_t oy = (t / g.out_w) % g.out_h;
  const int64_t o = (t / (g.out_w * g.out_h)) % g.out_ch;
  const int64_t n = t / (g.out_w * g.out_h * g.out_ch);
  const int64_t m = (n * g.out_h + oy) * g.out_w + ox;
  out[n * g.o_stride[0] + o * g.o_stride[1] + oy * g.o_stride[2] + ox * g.o_stride[3]] = d[m * g.out_ch + o];
}

struct Layout {
  int64_t rows, k, kp;
  bool pointwise;      // 1 x 1 window, unit strides, no padding, dense channels-last input: the input IS the
                       // [pixels, channels] matrix of the product, nothing is gathered
  bool implicit;       // channels-last input with a multiple of 64 channels and a ready kernel matrix: the product
                       // fetches its activation tiles from the image (TMA im2col mode), nothing is gathered
  bool weight_ready;   // the kernel already is [out_ch, kp] in (ky, kx, c) order
  bool out_direct;     // the output is dense channels-last
  int64_t a_bytes, w_bytes, d_bytes;
};

Layout layout_of(const ConvGeometry& g) {
  Layout l{};
  l.rows = g.batch * g.out_h * g.out_w;
  l.k = g.k_h * g.k_w * g.in_ch;
  l.kp = round_up(l.k, kChunk);
  l.weight_ready = l.kp == l.k && g.w_stride[1] == 1 && g.w_stride[3] == g.in_ch && g.w_stride[2] == g.k_w * g.in_ch &&
                   g.w_stride[0] == l.k;
  l.out_direct = g.o_stride[1] == 1 && g.o_stride[3] == g.out_ch && g.o_stride[2] == g.out_w * g.out_ch &&
                 g.o_stride[0] == g.out_h * g.out_w * g.out_ch;
  l.pointwise = g.k_h == 1 && g.k_w == 1 && g.stride_h == 1 && g.stride_w == 1 && g.pad_top == 0 && g.pad_bottom == 0 &&
                g.pad_left == 0 && g.pad_right == 0 && l.kp == l.k && g.x_stride[1] == 1 && g.x_stride[3] % kChunk == 0 &&
                g.x_stride[3] >= g.in_ch && g.x_stride[2] == g.in_w * g.x_stride[3] && g.x_stride[0] == g.in_h * g.x_stride[2];
  l.implicit = !l.pointwise && l.weight_ready && g.in_ch % 64 == 0 && g.x_stride[1] == 1 && g.x_stride[3] % kChunk == 0 &&
               g.x_stride[2] % kChunk == 0 && g.x_stride[0] % kChunk == 0 && g.stride_h >= 1 && g.stride_h <= 8 &&
               g.stride_w >= 1 && g.stride_w <= 8 && g.pad_top <= 64 && g.pad_left <= 64 && g.pad_bottom <= 64 &&
               g.pad_right <= 64 && (g.k_h - 1) * g.dil_h < 128 && (g.k_w - 1) * g.dil_w < 128 &&
               l.rows < (int64_t{1} << 31) && l.rows >= 128 && g.out_ch >= 16;
  l.a_bytes = round_up(l.rows * l.kp, 256);  // also for pointwise layers: an input that is not 16-byte aligned is gathered
  l.w_bytes = l.weight_ready ? 0 : round_up(g.out_ch * l.kp, 256);
  l.d_bytes = l.out_direct ? 0 : round_up(l.rows * g.out_ch, 256);
  return l;
}

unsigned blocks_for(int64_t threads) { return static_cast<unsigned>((threads + 255) / 256); }

}  // namespace

int64_t qconv_workspace_bytes(const ConvGeometry& g) {
  const Layout l = layout_of(g);
  return l.a_bytes + l.w_bytes + l.d_bytes;
}

cudaError_t qconv_launch(const QConvParams& p, cudaStream_t stream, const char** err) {
  static const char* none = "";
  const char** e = err ? err : &none;
  const ConvGeometry& g = p.g;
  const Layout l = layout_of(g);
  if (l.rows < 0 || g.out_ch < 0 || l.k < 0) {
    *e = "qconv: negative size";
    return cudaErrorInvalidValue;
  }
  if (l.rows == 0 || g.out_ch == 0) return cudaSuccess;
  if (!p.x || !p.w || !p.out || !p.x_scale || !p.w_scale || !p.out_scale) {
    *e = "qconv: null operand";
    return cudaErrorInvalidValue;
  }
  if (!p.workspace || p.workspace_bytes < l.a_bytes + l.w_bytes + l.d_bytes ||
      reinterpret_cast<uintptr_t>(p.workspace) % 256 != 0) {
    *e = "qconv: workspace missing, misaligned or smaller than qconv_workspace_bytes";
    return cudaErrorInvalidValue;
  }
  if (l.rows * (l.kp / kChunk) >= (int64_t{1} << 31) * 256 || l.rows * g.out_ch >= (int64_t{1} << 31) * 256) {
    *e = "qconv: problem too large for one launch";
    return cudaErrorInvalidValue;
  }
  int8_t* a = static_cast<int8_t*>(p.workspace);
  int8_t* wp = a + l.a_bytes;
  int8_t* d = wp + l.w_bytes;
  const int vec = g.x_stride[1] == 1 && g.in_ch % kChunk == 0 && g.x_stride[0] % kChunk == 0 &&
                  g.x_stride[2] % kChunk == 0 && g.x_stride[3] % kChunk == 0 &&
                  reinterpret_cast<uintptr_t>(p.x) % kChunk == 0;
  // a pointwise convolution over an input that is not 16-byte aligned still goes through the gather
  const bool direct = l.pointwise && reinterpret_cast<uintptr_t>(p.x) % kChunk == 0;
  const bool implicit = l.implicit && reinterpret_cast<uintptr_t>(p.x) % kChunk == 0;
  cudaError_t st = cudaSuccess;
  if (!direct && !implicit) {
    st = launch_dependent(qconv_gather_kernel, dim3(blocks_for(l.rows * (l.kp / kChunk))), dim3(256), 0, stream, g, p.x, a,
                          l.rows, l.kp, vec);
    if (st != cudaSuccess) return st;
  }
  const int8_t* wmat = p.w;
  if (!l.weight_ready) {
    st = launch_dependent(qconv_pack_weight_kernel, dim3(blocks_for(g.out_ch * (l.kp / kChunk))), dim3(256), 0, stream, g,
                          p.w, wp, l.kp);
    if (st != cudaSuccess) return st;
    wmat = wp;
  }
  QGemmParams q;
  std::memset(&q, 0, sizeof(q));
  q.a = (direct || implicit) ? p.x : a;
  q.w = wmat;
  Im2colA ic{};
  if (implicit) {
    ic.x = p.x;
    ic.batch = g.batch;
    ic.in_h = g.in_h;
    ic.in_w = g.in_w;
    ic.in_ch = g.in_ch;
    ic.stride_n = g.x_stride[0];
    ic.stride_h = g.x_stride[2];
    ic.stride_w = g.x_stride[3];
    ic.out_h = static_cast<int>(g.out_h);
    ic.out_w = static_cast<int>(g.out_w);
    ic.k_h = static_cast<int>(g.k_h);
    ic.k_w = static_cast<int>(g.k_w);
    ic.conv_stride_h = static_cast<int>(g.stride_h);
    ic.conv_stride_w = static_cast<int>(g.stride_w);
    ic.dil_h = static_cast<int>(g.dil_h);
    ic.dil_w = static_cast<int>(g.dil_w);
    ic.pad_top = static_cast<int>(g.pad_top);
    ic.pad_left = static_cast<int>(g.pad_left);
    ic.pad_bottom = static_cast<int>(g.pad_bottom);
    ic.pad_right = static_cast<int>(g.pad_right);
    q.im2col = &ic;
  }
  q.out = l.out_direct ? p.out : d;
  q.M = l.rows;
  q.N = g.out_ch;
  q.K = l.kp;
  q.lda = direct ? g.x_stride[3] : l.kp;
  q.ldw = l.kp;
  q.ldo = g.out_ch;
  q.x_scale = p.x_scale;
  q.x_scale_kind = kScaleScalar;
  q.w_scale = p.w_scale;
  q.w_scale_kind = p.w_scale_per_channel ? kScalePerCol : kScaleScalar;
  q.out_scale = p.out_scale;
  q.out_scale_kind = kScaleScalar;
  q.fold_out_scale = 1;
  q.out_dtype = kOutI8;
  // fewer than 16 output channels, or a product too small to fill a tensor-core tile
  // schedule: the plain kernel
  if (g.out_ch < 16 || l.rows * g.out_ch * l.kp < (int64_t{1} << 22)) q.path = kPathSimt;
  q.splitk_ws = p.splitk_ws;
  q.splitk_ws_bytes = p.splitk_ws_bytes;
  st = qgemm_launch(q, stream, e);
  if (st != cudaSuccess) return st;
  if (!l.out_direct) {
    st = launch_dependent(qconv_scatter_kernel, dim3(blocks_for(l.rows * g.out_ch)), dim3(256), 0, stream, g,
                          static_cast<const int8_t*>(d), p.out, l.rows * g.out_ch);
  }
  return st;
}

}  // namespace disc_b200
