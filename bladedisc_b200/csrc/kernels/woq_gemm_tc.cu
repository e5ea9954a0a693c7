// Weight-only quantized linear on the tensor cores (fp16 activations, 5 rows and more):
//   out[m, n] = (sum_k x[m, k] * (w[k, n] - zp[n])) * scale[n] + bias[n].
//
// The uint8 weights [K, N] stay in the layout the reference's pattern hands over
// (pytorch_blade/tests/disc/pdl/pdll_files/gpu/weight_only_qgemm.pdll:27: the
// transposed matrix, N contiguous).  A thread block owns 256 output channels and up to
// 128 rows:
//   * TMA streams the raw bytes (32 k rows x 256 channels per box) into a deep ring in
//     shared memory, so that the bytes in flight do not depend on how many blocks or
//     registers an SM holds;
//   * two groups of eight converter warps (alternating stages) turn every byte into the
//     exact fp16 value w - zp (the byte is dropped into the mantissa of 1024.0, then
//     1024 + zp is subtracted: both steps are exact for |zp| <= 1024) and transpose on
//     the way: a thread gathers 8 k x 4 channels with byte permutes and stores one
//     16-byte chunk (8 k) per channel into a second ring in the K-major, 64-byte-swizzled
//     form of the MMA's B operand.  Row j of the operand holds channel
//     4 * (j % 64) + j / 64 of the strip, which makes both the loads and the stores of
//     the transpose free of bank conflicts; the epilogue undoes the permutation;
//   * the activations are the A operand (K-major), brought in by TMA; only the rows that
//     exist are fetched, the other rows of the 128-row operand are whatever the shared
//     memory holds and reach accumulator rows nobody reads;
//   * one thread issues tcgen05.mma kind::f16 (M = 128 rows, N = 256 channels, K = 16),
//     fp32 accumulators in TMEM: D[row, channel].  The weights are the wide operand, so
//     that one MMA covers 4 KB of raw weights and the same block shape serves decode
//     (a few rows) and prefill (128 rows per block);
//   * the k range can be split over a thread-block cluster (few rows leave too few
//     channel strips to fill the GPU); the partial tiles meet in distributed shared
//     memory and every block finishes a slice, in rank order: no scratch, no atomics,
//     run-to-run identical results;
//   * scale and bias are applied to the fp32 sums, as the streaming kernel does.
// Products of two fp16 values are exact in fp32, so the result differs from the
// streaming kernel's only by the order of the fp32 additions.
//
// No TMA multicast; every barrier wait is bounded and reports through the status word.
#include "woq_gemm.h"

#include <cooperative_groups.h>
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>

#include "device_info.h"
#include "rowops.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

namespace cg = cooperative_groups;

namespace disc_b200 {
namespace {

constexpr int kStrip = 256;                  // channels per block = MMA N
constexpr int kRowsPerBlock = 128;           // activation rows per block = MMA M
constexpr int kKB = 64;                      // k per activation tile
constexpr int kWK = 32;                      // k per weight stage (two per activation tile)
constexpr int kMaxRawStages = 12;            // raw weight boxes in flight (8 KB each), as many as fit
constexpr int kWStages = 6;                  // converted fp16 tiles (16 KB each) between converters and MMA
constexpr int kMaxXStages = 8;               // activation tiles (rows x 128 bytes each)
constexpr int kRawBytes = kWK * kStrip;      // 32 k rows x 256 channels, one byte each
constexpr int kConvWarps = 8;                // warps that convert one stage together
constexpr int kConvGroups = 2;               // such groups; group g takes stages g, g + 2, ...: most of a warp's time
                                             // per stage is latency (waits, loads, stores, fence, arrival), so two
                                             // stages are converted at a time (45 -> 37 us on 16 x 4096 x 11008)
constexpr int kConvThreads = kConvWarps * 32;
constexpr int kThreads = (3 + kConvGroups * kConvWarps) * 32;  // weight copies, MMA issue, activation copies, converters
constexpr int kWBytes = kStrip * kWK * 2;    // converted tile: 256 channel rows x 32 k x 2 bytes (64-byte rows)
constexpr int kXTileBytes = kRowsPerBlock * 128;      // what the MMA reads of an activation tile
constexpr int kStatusTimeoutWoq = 17;        // a wait of this kernel ran out

__device__ int g_woq_tc_status = 0;

struct TcArgs {
  const __half* scale;
  const int32_t* zp;
  const __half* bias;
  __half* out;
  int M, N, K;
  int64_t ldo;
  int rows;          // activation rows fetched per row tile (multiple of 16, <= 128)
  int row_tiles;     // row tiles (128 rows, one accumulator each) per block: 1, or 2 for long inputs
  int x_stages;      // activation tiles in the ring
  int raw_stages;    // raw weight boxes in the ring
  int kb_per_rank;   // 64-row k blocks per block of the cluster
  int num_kb;        // k blocks in all
};

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// kind::f16, D = f32, A and B fp16, both K-major; N >> 3 at [17,23), M >> 4 at [24,29).
constexpr uint32_t kIdesc = (1u << 4) | (static_cast<uint32_t>(kStrip >> 3) << 17) |
                            (static_cast<uint32_t>(kRowsPerBlock >> 4) << 24);

// Two bytes (byte C of each word) -> the fp16 pair (1024 + a, 1024 + b) - zp2.
template <int C>
__device__ __forceinline__ uint32_t pair_to_half2(uint32_t wa, uint32_t wb, __half2 zp2) {
  uint32_t p = __byte_perm(wa, wb, C | ((4 + C) << 4));  // [wa.byteC, wb.byteC, ., .]
  uint32_t q = __byte_perm(p, 0x64646464u, 0x4140);     // each byte into the mantissa of an fp16 1024.0
  const __half2 r = __hsub2(*reinterpret_cast<__half2*>(&q), zp2);
  return *reinterpret_cast<const uint32_t*>(&r);
}
// Channel C of eight consecutive k (one word per k, four channels per word) -> the 16-byte chunk of its row.
// Rows are 64 bytes (32 k), 64-byte swizzle: chunk index ^= (row / 2) % 4.
template <int C>
__device__ __forceinline__ void store_channel(const uint32_t (&w)[8], __half2 zp2, uint32_t tile, int cg, int kg) {
  const uint32_t j = static_cast<uint32_t>(C * 64 + cg);  // row of the operand that holds this channel
  const uint32_t addr = tile + j * 64 + ((static_cast<uint32_t>(kg) ^ ((j >> 1) & 3)) << 4);
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pair_to_half2<C>(w[0], w[1], zp2)),
               "r"(pair_to_half2<C>(w[2], w[3], zp2)), "r"(pair_to_half2<C>(w[4], w[5], zp2)),
               "r"(pair_to_half2<C>(w[6], w[7], zp2))
               : "memory");
}

// Shared memory: [activation ring + slack][raw ring][fp16 ring][barriers].  The MMA reads 128 rows
// of an activation tile of which only `rows` were fetched: the slack keeps that read inside the
// allocation.  The partial tile of a split k range overlays the rings once the main loop is over.
struct Smem {
  // raw_full, raw_empty [kMaxRawStages]; w_full, w_empty [kWStages]; x_full, x_empty [kMaxXStages]; acc
  static constexpr int kNumBars = 2 * kMaxRawStages + 2 * kWStages + 2 * kMaxXStages + 1;
  // x_bytes = bytes of one activation stage (row tiles x rows x 128)
  static __host__ __device__ int w_off(int x_bytes, int row_tiles, int x_stages) {
    return ((x_stages - 1) * x_bytes + row_tiles * kXTileBytes + 1023) & ~1023;
  }
  static __host__ __device__ int raw_off(int x_bytes, int row_tiles, int x_stages) {
    return w_off(x_bytes, row_tiles, x_stages) + kWStages * kWBytes;
  }
  static int bars(int x_bytes, int row_tiles, int x_stages, int raw_stages) {
    return raw_off(x_bytes, row_tiles, x_stages) + raw_stages * kRawBytes;
  }
  static size_t total(int x_bytes, int row_tiles, int x_stages, int raw_stages) {
    return 1024 + bars(x_bytes, row_tiles, x_stages, raw_stages) + kNumBars * 8 + 16;
  }
};

__global__ void __launch_bounds__(kThreads)
woq_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, TcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  const int tile_bytes = a.row_tiles > 1 ? kXTileBytes : a.rows * 128;  // one row tile of an activation stage
  const int x_bytes = a.row_tiles * tile_bytes;
  const int w_off = Smem::w_off(x_bytes, a.row_tiles, a.x_stages);
  const int raw_off = w_off + kWStages * kWBytes;
  const int bars_off = raw_off + a.raw_stages * kRawBytes;
  const uint32_t bar_base = smem_base + bars_off;
  auto raw_full = [&](int s) { return bar_base + 8u * s; };
  auto raw_empty = [&](int s) { return bar_base + 8u * (kMaxRawStages + s); };
  auto w_full = [&](int s) { return bar_base + 8u * (2 * kMaxRawStages + s); };
  auto w_empty = [&](int s) { return bar_base + 8u * (2 * kMaxRawStages + kWStages + s); };
  auto x_full = [&](int s) { return bar_base + 8u * (2 * kMaxRawStages + 2 * kWStages + s); };
  auto x_empty = [&](int s) { return bar_base + 8u * (2 * kMaxRawStages + 2 * kWStages + kMaxXStages + s); };
  const uint32_t acc_bar = bar_base + 8u * (Smem::kNumBars - 1);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + bars_off + Smem::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  cg::cluster_group cluster = cg::this_cluster();
  const int rank = static_cast<int>(cluster.block_rank());  // the cluster spans blockIdx.y
  const int csize = static_cast<int>(cluster.num_blocks());
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * kRowsPerBlock * a.row_tiles;
  const int strip = blockIdx.z;
  const int kb_begin = rank * a.kb_per_rank;
  const int kb_count = max(0, min(a.num_kb, kb_begin + a.kb_per_rank) - kb_begin);

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.raw_stages; ++s) {
      mbar_init(raw_full(s), 1);
      mbar_init(raw_empty(s), kConvWarps);
    }
    for (int s = 0; s < kWStages; ++s) {
      mbar_init(w_full(s), kConvWarps);
      mbar_init(w_empty(s), 1);
    }
    for (int s = 0; s < a.x_stages; ++s) {
      mbar_init(x_full(s), 1);
      mbar_init(x_empty(s), 1);
    }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), static_cast<uint32_t>(kStrip * a.row_tiles));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int ws_count = 2 * kb_count;  // weight stages (32 k each) of this block

  // Position in a ring: stage index and the parity of its current round.  Kept by increments: the loops
  // below are a few dozen instructions per stage for a single thread, and a division by a ring size that
  // is only known at run time would double that.
  struct Ring {
    int stage = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void next(int size, int step = 1) {
      stage += step;
      if (stage >= size) {
        stage -= size;
        phase ^= 1;
      }
    }
  };

  if (warp == 0) {
    // ---- raw weights: constants of the model, no dependency wait
    if (lane == 0) {
      Ring raw;
      int k = kb_begin * kKB;
      for (int ws = 0; ws < ws_count; ++ws, k += kWK, raw.next(a.raw_stages)) {
        if (!mbar_wait(raw_empty(raw.stage), raw.phase ^ 1, abort_flag, &g_woq_tc_status, kStatusTimeoutWoq)) break;
        mbar_arrive_expect_tx(raw_full(raw.stage), kRawBytes);
        tma_load_2d(smem_base + raw_off + raw.stage * kRawBytes, &tmap_w, raw_full(raw.stage), strip * kStrip, k);
      }
    }
  } else if (warp == 2) {
    // ---- activations: one box of `rows` rows x 64 k per tile
    if (lane == 0) {
      grid_dep_wait();  // the activations may come from the kernel before this one
      Ring xr;
      int k = kb_begin * kKB;
      for (int kb = 0; kb < kb_count; ++kb, k += kKB, xr.next(a.x_stages)) {
        if (!mbar_wait(x_empty(xr.stage), xr.phase ^ 1, abort_flag, &g_woq_tc_status, kStatusTimeoutWoq)) break;
        mbar_arrive_expect_tx(x_full(xr.stage), static_cast<uint32_t>(x_bytes));
        for (int t = 0; t < a.row_tiles; ++t)  // rows past M read as zero and still count their bytes
          tma_load_2d(smem_base + xr.stage * x_bytes + t * tile_bytes, &tmap_x, x_full(xr.stage), k, m0 + t * kRowsPerBlock);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue: two weight stages per activation tile
    if (lane == 0) {
      Ring wr, xr;
      for (int kb = 0; kb < kb_count; ++kb, xr.next(a.x_stages)) {
        if (!mbar_wait(x_full(xr.stage), xr.phase, abort_flag, &g_woq_tc_status, kStatusTimeoutWoq)) break;
        const uint64_t a_desc = make_kmajor_sw128_desc(smem_base + xr.stage * x_bytes);
        bool ok = true;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf, wr.next(kWStages)) {
          if (!mbar_wait(w_full(wr.stage), wr.phase, abort_flag, &g_woq_tc_status, kStatusTimeoutWoq)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t b_desc = make_kmajor_sw64_desc(smem_base + w_off + wr.stage * kWBytes);
          for (int t = 0; t < a.row_tiles; ++t) {
#pragma unroll
            for (int kk = 0; kk < kWK / 16; ++kk) {
              // 16 k are 32 bytes further in both tiles; the second weight stage starts 32 k into the activation
              // tile; the second row tile is kXTileBytes further and has its own accumulator
              umma_f16(tmem_base + static_cast<uint32_t>(t * kStrip), a_desc + (t * kXTileBytes >> 4) + 4 * hf + 2 * kk,
                       b_desc + 2 * kk, kIdesc, (kb | hf | kk) != 0 ? 1u : 0u);
            }
          }
          umma_commit(w_empty(wr.stage));
        }
        if (!ok) break;
        umma_commit(x_empty(xr.stage));
      }
      umma_commit(acc_bar);
    }
  } else {
    // ---- raw bytes -> fp16 (w - zp), transposed into the K-major layout of the MMA's B operand
    const int group = (warp - 3) / kConvWarps;
    const int ct = (threadIdx.x - 96) % kConvThreads;
    const int cg = ct & 63;     // four channels: 4 * cg .. 4 * cg + 3 of the strip
    const int kg = ct >> 6;     // which 8 of the 32 k rows of a stage
    const int64_t n0 = static_cast<int64_t>(strip) * kStrip + cg * 4;
    const bool n_ok = n0 < a.N;  // N is a multiple of 16: a thread's channels are wholly inside or outside
    __half2 zp2[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float z = (n_ok && a.zp) ? static_cast<float>(__ldg(a.zp + n0 + c)) : 0.f;
      zp2[c] = __floats2half2_rn(1024.f + z, 1024.f + z);
    }
    const uint32_t src0 = smem_base + raw_off + cg * 4 + kg * 8 * kStrip;
    const uint32_t dst0 = smem_base + w_off;
    Ring raw, wr;  // both ring sizes are multiples of the number of groups
    raw.stage = wr.stage = group;
    for (int ws = group; ws < ws_count; ws += kConvGroups, raw.next(a.raw_stages, kConvGroups), wr.next(kWStages, kConvGroups)) {
      // one lane polls for the warp
      int go = 1;
      if (lane == 0) {
        go = mbar_wait(raw_full(raw.stage), raw.phase, abort_flag, &g_woq_tc_status, kStatusTimeoutWoq) &&
             mbar_wait(w_empty(wr.stage), wr.phase ^ 1, abort_flag, &g_woq_tc_status, kStatusTimeoutWoq);
      }
      go = __shfl_sync(0xffffffffu, go, 0);
      if (!go) break;
      const uint32_t src = src0 + raw.stage * kRawBytes;
      const uint32_t dst = dst0 + wr.stage * kWBytes;
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w[i]) : "r"(src + i * kStrip));
      }
      store_channel<0>(w, zp2[0], dst, cg, kg);
      store_channel<1>(w, zp2[1], dst, cg, kg);
      store_channel<2>(w, zp2[2], dst, cg, kg);
      store_channel<3>(w, zp2[3], dst, cg, kg);
      fence_proxy_async_smem();  // the stores above become visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(w_full(wr.stage));
        mbar_arrive(raw_empty(raw.stage));
      }
    }
  }
  grid_dep_launch();

  // ---- epilogue: the converter warps read D[row, channel]; warp w may touch TMEM lanes 32 * (w % 4) ...
  const bool split = csize > 1;
  float* tile = reinterpret_cast<float*>(smem);  // [rows][256] partial sums (the rings are free by now)
  if (warp >= 3 && warp < 3 + kConvWarps) {
    bool ok = true;
    if (kb_count > 0) ok = mbar_wait(acc_bar, 0, abort_flag, &g_woq_tc_status, kStatusTimeoutWoq);
    tc_fence_after();
    grid_dep_wait();  // the kernel before this one may still read the output buffer
    const int q = warp & 3;
    const int half = (warp - 3) >> 2;  // which 128 channels of the strip
    const int r_local = q * 32 + lane;
    for (int rt = 0; rt < a.row_tiles; ++rt) {
    const int m = m0 + rt * kRowsPerBlock + r_local;
    const uint32_t acc = tmem_base + static_cast<uint32_t>(rt * kStrip);
    if (q * 32 < a.rows && m0 + rt * kRowsPerBlock < a.M) {  // the same for the whole warp: rows of this quarter exist
      __half* orow = a.out + static_cast<int64_t>(m) * a.ldo;
      for (int it = 0; it < 2; ++it) {
        // column c * 64 + g of the accumulator is channel 4 * g + c: four loads of 16 columns (g0 .. g0 + 15,
        // c = 0 .. 3) are 64 consecutive channels
        const int g0 = half * 32 + it * 16;
        const int64_t nbase = static_cast<int64_t>(strip) * kStrip + 4 * g0;
        if (nbase >= a.N) break;
        uint32_t r[4][16];
        if (ok && kb_count > 0) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            tmem_ld_x16(acc + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(c * 64 + g0), r[c]);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int t = 0; t < 16; ++t) r[c][t] = 0u;
        }
        if (split) {
          if (r_local < a.rows) {
            float4* dst = reinterpret_cast<float4*>(tile + r_local * kStrip + 4 * g0);
#pragma unroll
            for (int t = 0; t < 16; ++t)
              dst[t] = make_float4(__uint_as_float(r[0][t]), __uint_as_float(r[1][t]), __uint_as_float(r[2][t]),
                                   __uint_as_float(r[3][t]));
          }
        } else if (m < a.M) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {  // 16 channels at a time: t = 4u .. 4u + 3
            const int64_t n = nbase + 16 * u;
            if (n >= a.N) break;  // N is a multiple of 16
            // scale and bias: the same addresses for every lane
            uint4 sv[2], bv[2], ov[2];
            sv[0] = __ldg(reinterpret_cast<const uint4*>(a.scale + n));
            sv[1] = __ldg(reinterpret_cast<const uint4*>(a.scale + n) + 1);
            if (a.bias) {
              bv[0] = __ldg(reinterpret_cast<const uint4*>(a.bias + n));
              bv[1] = __ldg(reinterpret_cast<const uint4*>(a.bias + n) + 1);
            } else {
              bv[0] = bv[1] = make_uint4(0, 0, 0, 0);
            }
            const __half2* s2 = reinterpret_cast<const __half2*>(sv);
            const __half2* b2 = reinterpret_cast<const __half2*>(bv);
            __half2* o2 = reinterpret_cast<__half2*>(ov);
#pragma unroll
            for (int tt = 0; tt < 4; ++tt) {
              const int t = 4 * u + tt;
              const float2 s01 = __half22float2(s2[2 * tt]), s23 = __half22float2(s2[2 * tt + 1]);
              const float2 b01 = __half22float2(b2[2 * tt]), b23 = __half22float2(b2[2 * tt + 1]);
              o2[2 * tt] = __floats2half2_rn(__uint_as_float(r[0][t]) * s01.x + b01.x, __uint_as_float(r[1][t]) * s01.y + b01.y);
              o2[2 * tt + 1] = __floats2half2_rn(__uint_as_float(r[2][t]) * s23.x + b23.x, __uint_as_float(r[3][t]) * s23.y + b23.y);
            }
            reinterpret_cast<uint4*>(orow + n)[0] = ov[0];
            reinterpret_cast<uint4*>(orow + n)[1] = ov[1];
          }
        }
      }
    }
    }  // row tiles
  }
  if (split) {
    // every block adds its slice of the tile over the cluster, in rank order
    cluster.sync();
    const int total = a.rows * kStrip;
    const int slice = (total + csize - 1) / csize;
    const int i_end = min(total, (rank + 1) * slice);
    for (int i = rank * slice + static_cast<int>(threadIdx.x); i < i_end; i += kThreads) {
      const int m = m0 + i / kStrip;
      const int64_t n = static_cast<int64_t>(strip) * kStrip + (i % kStrip);
      float v = 0.f;
      for (int j = 0; j < csize; ++j) v += cluster.map_shared_rank(tile, j)[i];
      if (m < a.M && n < a.N) {
        v = v * __half2float(a.scale[n]) + (a.bias ? __half2float(a.bias[n]) : 0.f);
        a.out[static_cast<int64_t>(m) * a.ldo + n] = __float2half_rn(v);
      }
    }
    cluster.sync();  // no block leaves while its tile may still be read
  }

  if (*abort_flag) {
    // a copy that was never seen to complete may still be landing
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(kStrip * a.row_tiles));
  }
}

}  // namespace

namespace {
// Clusters of `sp` blocks with `smem` bytes the current device holds at once; asked of the runtime once per
// (device, size, shared memory) and remembered (the query costs microseconds, a decode step has hundreds of calls).
int max_active_clusters(const cudaLaunchConfig_t& q, int sp, size_t smem) {
  static std::mutex mu;
  static std::map<std::tuple<int, int, size_t>, int> cache;
  const auto key = std::make_tuple(current_device_ordinal(), sp, smem);
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  int active = 0;
  if (cudaOccupancyMaxActiveClusters(&active, woq_tc_kernel, &q) != cudaSuccess || active < 1) {
    (void)cudaGetLastError();
    active = 0;
  }
  std::lock_guard<std::mutex> lock(mu);
  cache[key] = active;
  return active;
}
}  // namespace

bool woq_gemm_tc_usable(const WoqGemmParams& p) {
  return p.type == kF16 && p.K >= kKB && p.N % 16 == 0 && p.ldw % 16 == 0 && p.ldx % 8 == 0 && p.ldo % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(p.w) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.scale) & 15) == 0 &&
         (!p.bias || (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) && p.M <= 0x7fffffff && p.N <= 0x7fffffff &&
         p.K <= 0x7fffffff && (p.N + kStrip - 1) / kStrip <= 65535;
}

cudaError_t woq_gemm_tc_launch(const WoqGemmParams& p, cudaStream_t s, const char** err) {
  if (!woq_gemm_tc_usable(p)) {
    *err = "weight-only qgemm (tensor cores): needs f16, N a multiple of 16, 16-byte aligned operands and row pitches";
    return cudaErrorInvalidValue;
  }
  EncodeTiledFn fn = tensor_map_encode_fn();
  if (!fn) {
    *err = "cuTensorMapEncodeTiled unavailable";
    return cudaErrorInvalidValue;
  }
  const int sms = device_sm_count();
  TcArgs a;
  a.scale = static_cast<const __half*>(p.scale);
  a.zp = p.zp;
  a.bias = static_cast<const __half*>(p.bias);
  a.out = static_cast<__half*>(p.out);
  a.M = static_cast<int>(p.M);
  a.N = static_cast<int>(p.N);
  a.K = static_cast<int>(p.K);
  a.ldo = p.ldo;
  const int64_t strips = (p.N + kStrip - 1) / kStrip;
  // Long inputs: two row tiles per block share every converted weight tile (the conversion, not the tensor core,
  // bounds the kernel).  A block with two tiles takes about 1.5 times as long (measured at 2048 rows), so it
  // pays when it saves enough rounds of blocks over the SMs.
  {
    const int64_t rounds1 = (strips * ((p.M + kRowsPerBlock - 1) / kRowsPerBlock) + sms - 1) / sms;
    const int64_t rounds2 = (strips * ((p.M + 2 * kRowsPerBlock - 1) / (2 * kRowsPerBlock)) + sms - 1) / sms;
    a.row_tiles = (p.M > kRowsPerBlock && 3 * rounds2 <= 2 * rounds1) ? 2 : 1;
  }
  a.rows = a.row_tiles > 1 ? kRowsPerBlock : static_cast<int>((std::min<int64_t>(p.M, kRowsPerBlock) + 15) / 16 * 16);
  const int x_bytes = a.row_tiles * a.rows * 128;
  a.x_stages = std::max(2, std::min(kMaxXStages, 16384 / x_bytes));
  constexpr int kSmemBudget = 224 * 1024;
  a.raw_stages = std::max(2, std::min(kMaxRawStages, (kSmemBudget - Smem::raw_off(x_bytes, a.row_tiles, a.x_stages)) / kRawBytes));
  a.raw_stages -= a.raw_stages % kConvGroups;
  const int64_t m_groups = (p.M + kRowsPerBlock * a.row_tiles - 1) / (kRowsPerBlock * a.row_tiles);
  a.num_kb = static_cast<int>((p.K + kKB - 1) / kKB);
  const size_t smem = Smem::total(x_bytes, a.row_tiles, a.x_stages, a.raw_stages);
  cudaError_t st = cudaFuncSetAttribute(woq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (st != cudaSuccess) return st;
  st = cudaFuncSetAttribute(woq_tc_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 0);
  if (st != cudaSuccess) return st;
  // Few channel strips: the k range is cut over a cluster (any size up to 8).  How many clusters of a size
  // the GPU holds at once is asked of the runtime (large clusters pack badly into the GPCs); the size with
  // the smallest estimate of waves x (stages per block + fixed cost in stages) wins.
  int split = 1;
  {
    const int64_t base = strips * m_groups;
    double best = 1e30;
    for (int sp = 1; sp <= (a.row_tiles > 1 ? 1 : 8) && (sp == 1 || a.num_kb / sp >= 2); ++sp) {
      cudaLaunchConfig_t q{};
      q.gridDim = dim3(static_cast<unsigned>(m_groups), static_cast<unsigned>(sp), static_cast<unsigned>(strips));
      q.blockDim = dim3(kThreads);
      q.dynamicSmemBytes = smem;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 1;
      qa[0].val.clusterDim.y = sp;
      qa[0].val.clusterDim.z = 1;
      q.attrs = qa;
      q.numAttrs = 1;
      const int active_or_0 = max_active_clusters(q, sp, smem);
      int active = active_or_0;
      if (active < 1) {
        if (sp == 1) active = sms; else continue;
      }
      const int64_t waves = (base + active - 1) / active;
      const double stages = 2.0 * ((a.num_kb + sp - 1) / sp);
      // fixed cost of a block (launch, set-up, epilogue) about 16 stages; the exchange of partial tiles grows
      // with the rows of the tile
      const double cost = static_cast<double>(waves) * (stages + 16.0 + (sp > 1 ? 4.0 + a.rows / 8.0 : 0.0));
      if (cost < best * 0.97) {
        best = cost;
        split = sp;
      }
    }
  }
  a.kb_per_rank = (a.num_kb + split - 1) / split;
  if (m_groups > 0x7fffffff) {
    *err = "weight-only qgemm (tensor cores): too many rows";
    return cudaErrorInvalidValue;
  }

  CUtensorMap tw, tx;
  cuuint32_t estr[2] = {1, 1};
  {
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.N), static_cast<cuuint64_t>(p.K)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.ldw)};
    cuuint32_t box[2] = {kStrip, kWK};
    if (fn(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(p.w), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      *err = "cuTensorMapEncodeTiled failed (weights)";
      return cudaErrorInvalidValue;
    }
  }
  {
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.K), static_cast<cuuint64_t>(p.M)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.ldx * 2)};
    cuuint32_t box[2] = {kKB, static_cast<cuuint32_t>(a.rows)};
    if (fn(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(p.x), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      *err = "cuTensorMapEncodeTiled failed (activations)";
      return cudaErrorInvalidValue;
    }
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(m_groups), static_cast<unsigned>(split), static_cast<unsigned>(strips));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 1;
  attrs[0].val.clusterDim.y = split;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, woq_tc_kernel, tw, tx, a);
}

int woq_tc_status_fetch_and_clear() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_woq_tc_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_woq_tc_status, &zero, sizeof(int));
  }
  return v;
}

}  // namespace disc_b200
