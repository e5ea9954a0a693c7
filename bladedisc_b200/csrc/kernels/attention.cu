// Fused masked self-attention over packed sequences for sm_100a.
//
// In the reference's compiled encoder the two attention products are library
// GEMMs (ral_gemm, tao_compiler/mlir/ral/context/stream_executor_based_impl.cc:551-637)
// with a generated softmax kernel between them
// (tao_compiler/mlir/disc/transforms/lhlo_legalize_roots_to_loops.cc:1263-1289) and a
// quantize kernel after them: the [heads, L, L] scores cross HBM four times.
// Here one CTA owns 128 query rows of one head of one sequence and keeps the
// scores on chip:
//
//   S = Q K^T   tcgen05.mma kind::f16, Q [128 x 64] and up to four K blocks
//               [128 x 64] in 128B-swizzled shared memory (TMA), S in TMEM as
//               128 lanes x (128 columns per key block) fp32 -- all 512 columns.
//   softmax     eight warps, a thread per row and half of each key block: one
//               pass over TMEM for the row maximum, one for exp2 and the row
//               sum; P goes to shared memory as f16 in the K-major swizzled
//               layout the next product reads.
//   O = P V     tcgen05.mma kind::f16 with V [keys x 64] as the MN-major operand
//               straight from the TMA tile (no transpose); O reuses the TMEM
//               columns of the first score block, which is dead by then.
//   epilogue    O / rowsum, quantized to int8 at the consumer's scale (or f16),
//               written into [tokens, hidden] where the next linear reads it.
//
// Sequences are packed (no padding rows): K / V rows past the end of a sequence
// belong to the next one or are out of range (zero filled) and are masked.
#include "attention.h"

#include <cuda.h>
#include <cuda_fp16.h>

#include <mutex>

#include "device_info.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

namespace disc_b200 {

__device__ int g_attn_status = 0;

namespace {

constexpr int kRows = kAttnRowsPerBlock;      // query rows per CTA = MMA M
constexpr int kKeyBlock = 128;                // keys per score block = MMA N of the first product
constexpr int kMaxKeyBlocks = kAttnMaxKeys / kKeyBlock;
constexpr int kTileBytes = kRows * 128;       // 128 rows x 64 f16 = 16 KB
constexpr int kSoftmaxWarps = 8;
constexpr int kAttnThreads = (2 + kSoftmaxWarps) * 32;

struct AttnSmem {
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTileBytes;                       // 4 key blocks
  static constexpr int kV = kK + kMaxKeyBlocks * kTileBytes;       // 4 key blocks
  static constexpr int kP = kV + kMaxKeyBlocks * kTileBytes;       // 2 buffers x 2 sub-tiles of 64 keys
  static constexpr int kBars = kP + 4 * kTileBytes;
  // q_full, k_full[4], v_full[4], s_full[4], p_full[4], pv_done[4], o_full, q_free, o_read
  static constexpr int kNumBars = 1 + 5 * kMaxKeyBlocks + 3;
  static constexpr int kMisc = kBars + kNumBars * 8;               // tmem slot, abort flag
  static constexpr int kRed = ((kMisc + 16) + 15) & ~15;           // max[2][128], sum[2][128]
  static constexpr int kTotal = kRed + 4 * kRows * 4;
  static constexpr int kDynamic = kTotal + 1024;
};

// D (fp32, TMEM) (+)= A (f16, smem) * B (f16, smem), issued by one thread.
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

// Instruction descriptor for kind::f16: D = f32 (bits [4,6) = 1), A and B f16 (format 0), bit 16 set when B
// is MN-major (its N index contiguous in shared memory), N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t make_f16_idesc(int mma_m, int mma_n, bool b_mn_major) {
  return (1u << 4) | (b_mn_major ? (1u << 16) : 0u) | (static_cast<uint32_t>(mma_n >> 3) << 17) |
         (static_cast<uint32_t>(mma_m >> 4) << 24);
}

// Shared-memory descriptor of an MN-major operand tile with 128-byte swizzle: rows of the tile are K indices,
// each row holds 64 f16 along N (128 bytes); 8-row groups are 1024 bytes apart (stride byte offset); the
// leading byte offset would step to the next 64 columns of N and is unused for N = 64.
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(kTileBytes >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename OutT>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const AttnBlock* __restrict__ blocks, int hidden,
                 float scale_log2e, OutT* __restrict__ out, int64_t ld_out, const float* __restrict__ out_scale) {
  using L = AttnSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBars;
  const uint32_t q_full = bar_base;
  auto k_full = [&](int j) { return bar_base + 8u * (1 + j); };
  auto v_full = [&](int j) { return bar_base + 8u * (1 + kMaxKeyBlocks + j); };
  auto s_full = [&](int j) { return bar_base + 8u * (1 + 2 * kMaxKeyBlocks + j); };
  auto p_full = [&](int j) { return bar_base + 8u * (1 + 3 * kMaxKeyBlocks + j); };
  auto pv_done = [&](int j) { return bar_base + 8u * (1 + 4 * kMaxKeyBlocks + j); };
  const uint32_t o_full = bar_base + 8u * (1 + 5 * kMaxKeyBlocks);
  const uint32_t q_free = o_full + 8u;   // the score products of a query block are done: its Q tile may be replaced
  const uint32_t o_read = o_full + 16u;  // the epilogue has read O: the next query block's scores may overwrite it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMisc + 4);
  float* red_max = reinterpret_cast<float*>(smem + L::kRed);   // [2][128]
  float* red_sum = red_max + 2 * kRows;                          // [2][128]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.x;  // heads vary fastest: the heads of the longest items start first and read the same rows
  constexpr uint32_t kTmemCols = 512;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_qkv);
    for (int i = 0; i < L::kNumBars; ++i) mbar_init(bar_base + 8u * i, 1);
    for (int j = 0; j < kMaxKeyBlocks; ++j) mbar_init(p_full(j), kSoftmaxWarps);
    mbar_init(o_read, kSoftmaxWarps);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dep_launch();
  grid_dep_wait();  // qkv comes from the kernel before this one

  // A work item is `nq` consecutive blocks of 128 query rows of one sequence: K and V are fetched once and
  // stay in shared memory, the barriers that cycle per query block are waited on with the block's parity.
  const AttnBlock blk = blocks[blockIdx.y];
  const int len = blk.len;
  const int nkb = (len + kKeyBlock - 1) / kKeyBlock;   // 1 .. 4
  const int nq = blk.nq < 1 ? 1 : blk.nq;

  if (warp == 0) {
    if (lane == 0) {
      // every tile has its own place in shared memory: all loads go out at once
      mbar_arrive_expect_tx(q_full, kTileBytes);
      tma_load_2d(smem_base + L::kQ, &tmap_qkv, q_full, head * kAttnHeadDim, blk.tok0 + blk.q0);
      for (int j = 0; j < nkb; ++j) {
        mbar_arrive_expect_tx(k_full(j), kTileBytes);
        tma_load_2d(smem_base + L::kK + j * kTileBytes, &tmap_qkv, k_full(j), hidden + head * kAttnHeadDim,
                    blk.tok0 + j * kKeyBlock);
      }
      for (int j = 0; j < nkb; ++j) {
        mbar_arrive_expect_tx(v_full(j), kTileBytes);
        tma_load_2d(smem_base + L::kV + j * kTileBytes, &tmap_qkv, v_full(j), 2 * hidden + head * kAttnHeadDim,
                    blk.tok0 + j * kKeyBlock);
      }
      // the Q tiles of the following query blocks, each once the products that read the previous one are done
      for (int it = 1; it < nq; ++it) {
        if (!mbar_wait(q_free, (it - 1) & 1, abort_flag, &g_attn_status, 18)) break;
        mbar_arrive_expect_tx(q_full, kTileBytes);
        tma_load_2d(smem_base + L::kQ, &tmap_qkv, q_full, head * kAttnHeadDim, blk.tok0 + blk.q0 + it * kRows);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_f16_idesc(kRows, kKeyBlock, false);
      constexpr uint32_t idesc_o = make_f16_idesc(kRows, kAttnHeadDim, true);
      bool ok = true;
      for (int it = 0; it < nq && ok; ++it) {
        const uint32_t ph = it & 1;
        ok = mbar_wait(q_full, ph, abort_flag, &g_attn_status, 11);
        if (ok && it > 0) ok = mbar_wait(o_read, ph ^ 1, abort_flag, &g_attn_status, 19);   // O of the block before
        for (int j = 0; j < nkb && ok; ++j) {
          if (it == 0) ok = mbar_wait(k_full(j), 0, abort_flag, &g_attn_status, 12);
          if (!ok) break;
          tc_fence_after();
          const uint64_t a_desc = make_kmajor_sw128_desc(smem_base + L::kQ);
          const uint64_t b_desc = make_kmajor_sw128_desc(smem_base + L::kK + j * kTileBytes);
#pragma unroll
          for (int k = 0; k < kAttnHeadDim / 16; ++k) {   // 16 f16 = 32 bytes per MMA along the head dimension
            umma_f16(tmem_base + j * kKeyBlock, a_desc + 2 * k, b_desc + 2 * k, idesc_s, k != 0 ? 1u : 0u);
          }
          umma_commit(s_full(j));
        }
        if (ok) umma_commit(q_free);
        for (int j = 0; j < nkb && ok; ++j) {
          ok = mbar_wait(p_full(j), ph, abort_flag, &g_attn_status, 13);
          if (!ok) break;
          if (it == 0) ok = mbar_wait(v_full(j), 0, abort_flag, &g_attn_status, 14);
          if (!ok) break;
          tc_fence_after();
          const uint32_t p_addr = smem_base + L::kP + (j & 1) * 2 * kTileBytes;
          const uint32_t v_addr = smem_base + L::kV + j * kTileBytes;
#pragma unroll
          for (int kk = 0; kk < kKeyBlock / 16; ++kk) {   // 16 keys per MMA
            const uint64_t a_desc = make_kmajor_sw128_desc(p_addr + (kk >> 2) * kTileBytes) + 2 * (kk & 3);
            const uint64_t b_desc = make_mnmajor_sw128_desc(v_addr + kk * 16 * 128);
            umma_f16(tmem_base, a_desc, b_desc, idesc_o, (j | kk) != 0 ? 1u : 0u);
          }
          umma_commit(pv_done(j));
        }
        if (ok) umma_commit(o_full);
      }
    }
  } else {
    // softmax + epilogue: TMEM lane quadrant = warp % 4 (a hardware rule), `half` = which 64 keys of every
    // 128-key block (and, in the epilogue, which 32 output columns) this thread works on
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    bool ok = true;
    for (int it = 0; it < nq; ++it) {
    const uint32_t ph = it & 1;
    const int q_row0 = blk.q0 + it * kRows;

    // pass A: row maximum of the scaled scores over the valid keys
    float mx = -INFINITY;
    for (int j = 0; j < nkb && ok; ++j) {
      ok = mbar_wait(s_full(j), ph, abort_flag, &g_attn_status, 15);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t r[32];
        tmem_ld_x32(t_row + j * kKeyBlock + half * 64 + cc * 32, r);
        tmem_ld_wait();
        const int key0 = j * kKeyBlock + half * 64 + cc * 32;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = __uint_as_float(r[i]);
          if (key0 + i < len) mx = fmaxf(mx, s);
        }
      }
    }
    red_max[half * kRows + row] = mx;
    asm volatile("bar.sync 1, %0;" ::"r"(kSoftmaxWarps * 32) : "memory");
    mx = fmaxf(red_max[row], red_max[kRows + row]) * scale_log2e;   // the scale is positive: max commutes with it

    // pass B: p = exp2(s * scale * log2 e - max), row sums, P to shared memory as f16
    float sum = 0.f;
    for (int j = 0; j < nkb && ok; ++j) {
      if (j >= 2) {
        ok = mbar_wait(pv_done(j - 2), ph, abort_flag, &g_attn_status, 16);   // the P buffer is free again
        if (!ok) break;
      }
      uint8_t* p_tile = smem + L::kP + ((j & 1) * 2 + half) * kTileBytes + row * 128;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t r[32];
        tmem_ld_x32(t_row + j * kKeyBlock + half * 64 + cc * 32, r);
        tmem_ld_wait();
        const int key0 = j * kKeyBlock + half * 64 + cc * 32;
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = fast_exp2(__fmaf_rn(__uint_as_float(r[2 * i]), scale_log2e, -mx));
          float p1 = fast_exp2(__fmaf_rn(__uint_as_float(r[2 * i + 1]), scale_log2e, -mx));
          if (key0 + 2 * i >= len) p0 = 0.f;
          if (key0 + 2 * i + 1 >= len) p1 = 0.f;
          sum += p0 + p1;
          __half2 h = __floats2half2_rn(p0, p1);
          w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        // 32 keys = four 16-byte chunks of this row; chunk index xor (row & 7) is the 128-byte swizzle
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int chunk = cc * 4 + ch;
          *reinterpret_cast<uint4*>(p_tile + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(w[4 * ch], w[4 * ch + 1], w[4 * ch + 2], w[4 * ch + 3]);
        }
      }
      tc_fence_before();            // the TMEM reads of this block are done before the MMA warp is told
      fence_proxy_async_smem();     // and P is visible to the tensor core's reads of shared memory
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(j));
    }
    red_sum[half * kRows + row] = sum;
    asm volatile("bar.sync 1, %0;" ::"r"(kSoftmaxWarps * 32) : "memory");
    const float inv = 1.f / (red_sum[row] + red_sum[kRows + row]);

    // epilogue: this thread's 32 columns of its row
    if (ok) ok = mbar_wait(o_full, ph, abort_flag, &g_attn_status, 17);
    if (ok) {
      tc_fence_after();
      uint32_t r[32];
      tmem_ld_x32(t_row + half * 32, r);
      tmem_ld_wait();
      // O is in registers: the next query block's score products may overwrite its columns
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_read);
      if (q_row0 + row < len) {
        OutT* dst = out + static_cast<int64_t>(blk.tok0 + q_row0 + row) * ld_out + head * kAttnHeadDim + half * 32;
        if constexpr (sizeof(OutT) == 1) {
          const float k = inv * __frcp_rn(__ldg(out_scale));
          uint32_t w[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            uint32_t b[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float v = fminf(fmaxf(__uint_as_float(r[4 * i + e]) * k, -128.f), 127.f) + 12582912.f;
              b[e] = __float_as_uint(v);
            }
            w[i] = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
          }
          uint4* d4 = reinterpret_cast<uint4*>(dst);
          d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
          d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
          uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __half2 h = __floats2half2_rn(__uint_as_float(r[8 * i + 2 * e]) * inv,
                                            __uint_as_float(r[8 * i + 2 * e + 1]) * inv);
              w[e] = *reinterpret_cast<uint32_t*>(&h);
            }
            d4[i] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
    }   // query blocks
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
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

EncodeTiledFn encode_fn() { return tensor_map_encode_fn(); }

template <typename OutT>
cudaError_t launch_t(const AttentionParams& p, const CUtensorMap& tm, cudaStream_t stream) {
  auto kern = attention_kernel<OutT>;
  cudaError_t st = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem::kDynamic);
  if (st != cudaSuccess) return st;
  const float scale_log2e = p.scale * 1.4426950408889634f;
  return launch_dependent(kern, dim3(static_cast<unsigned>(p.heads), static_cast<unsigned>(p.num_blocks)),
                          dim3(kAttnThreads), AttnSmem::kDynamic, stream, tm, p.blocks, p.heads * kAttnHeadDim,
                          scale_log2e, static_cast<OutT*>(p.out), p.ld_out, p.out_scale);
}

}  // namespace

cudaError_t attention_launch(const AttentionParams& p, cudaStream_t stream, const char** err) {
  if (err) *err = nullptr;
  if (p.num_blocks <= 0 || p.tokens <= 0) return cudaSuccess;
  if (!p.qkv || !p.out || !p.blocks || p.heads <= 0) {
    if (err) *err = "attention: null operand or no heads";
    return cudaErrorInvalidValue;
  }
  const int64_t hidden = static_cast<int64_t>(p.heads) * kAttnHeadDim;
  if (p.ld_qkv < 3 * hidden || p.ld_qkv % 8 != 0 || (reinterpret_cast<uintptr_t>(p.qkv) & 15) != 0) {
    if (err) *err = "attention: qkv rows must hold 3 * hidden f16 values, 16-byte aligned";
    return cudaErrorInvalidValue;
  }
  const int out_bytes = p.out_scale ? 1 : 2;
  if (p.ld_out < hidden || (p.ld_out * out_bytes) % 16 != 0 || (reinterpret_cast<uintptr_t>(p.out) & 15) != 0) {
    if (err) *err = "attention: output rows must be 16-byte aligned";
    return cudaErrorInvalidValue;
  }
  if (p.scale <= 0.f) {
    if (err) *err = "attention: the score scale must be positive";
    return cudaErrorInvalidValue;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    if (err) *err = "cuTensorMapEncodeTiled unavailable";
    return cudaErrorInvalidValue;
  }
  CUtensorMap tm;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(3 * hidden), static_cast<cuuint64_t>(p.tokens)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.ld_qkv * 2)};
  cuuint32_t box[2] = {kAttnHeadDim, kRows};
  cuuint32_t estr[2] = {1, 1};
  if (fn(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(p.qkv), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    if (err) *err = "cuTensorMapEncodeTiled failed";
    return cudaErrorInvalidValue;
  }
  return p.out_scale ? launch_t<int8_t>(p, tm, stream) : launch_t<__half>(p, tm, stream);
}

int attention_status_fetch_and_clear() {
  int h = 0;
  if (cudaMemcpyFromSymbol(&h, g_attn_status, sizeof(int)) != cudaSuccess) return -1;
  if (h != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_attn_status, &z, sizeof(int));
  }
  return h;
}

}  // namespace disc_b200
