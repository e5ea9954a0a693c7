// LayerNorm / RMSNorm for fp16 rows of 2048 .. 8192 columns, the row staged in
// shared memory (included by rowops.cu).
//
// The register-resident kernel spends ~40 instructions per element on such
// rows and is bound by instruction issue at a third of the memory rate (a B200
// SM can afford about 16 per fp16 element at full HBM speed).  Most of that is
// code the row-in-registers design forces: every pass is unrolled over all
// vectors of the row, so the kernel is long, decides per element what a loop
// would decide once, and misses the instruction cache when made leaner.  Here
// a warp owns a row at a time:
//   * one lane asks for the row (and the residual row) with bulk async copies
//     into the warp's shared-memory buffers and the warp waits on its mbarrier;
//     activations stored as column slabs take one copy per slab;
//   * three short, rolled loops walk the row in shared memory 16 bytes per lane
//     at a time: sum (+ residual add, written back as fp16) and sum of squares;
//     normalise, round to fp16 in place, keep the largest magnitude on packed
//     halves; quantize;
//   * gamma / beta are copied to shared memory once per block;
//   * reductions are warp shuffles, there is no block-wide barrier.
// Measured on 16384 x 4096 (RMSNorm + per-token quantize): 105 -> 77 us; rows of
// 768 / 1024 columns are faster in the register-resident kernel and stay there.
// The arithmetic is that of norm_kernel: fp32 accumulation, x + residual and y
// rounded to fp16 where a separate kernel would have stored them, the int8
// output in the reciprocal form (quant_vec_recip: within one level of the
// divide-based formula).

constexpr int kStagedWarps = 4;  // warps (rows in flight) per block

__device__ int g_rowops_status = 0;  // a bounded wait of a row kernel ran out (code below)
constexpr int kRowStatusCopyTimeout = 16;

template <bool RMS>
__global__ void __launch_bounds__(kStagedWarps * 32)
norm_staged_f16_kernel(NormParams p) {
  constexpr int E = 8;
  extern __shared__ __align__(128) uint8_t staged_raw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cols = static_cast<int>(p.cols);
  const int nvec = cols / E;
  const uint32_t row_bytes = static_cast<uint32_t>(cols) * 2u;
  const bool has_res = p.residual != nullptr;
  // [gamma][beta] for the block, then per warp [x row][residual row if any], then one
  // mbarrier per warp and an abort flag
  const __half* gb = reinterpret_cast<const __half*>(p.gamma);
  const __half* bb = (!RMS && p.beta) ? reinterpret_cast<const __half*>(p.beta) : nullptr;
  const uint32_t warp_bytes = row_bytes * (has_res ? 2u : 1u);
  uint4* gs = reinterpret_cast<uint4*>(staged_raw);
  uint4* bs = reinterpret_cast<uint4*>(staged_raw + row_bytes);
  uint8_t* rows_base = staged_raw + 2 * static_cast<size_t>(row_bytes);
  uint8_t* my = rows_base + static_cast<size_t>(warp) * warp_bytes;
  uint4* xs = reinterpret_cast<uint4*>(my);
  const uint4* rs = reinterpret_cast<const uint4*>(my + row_bytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(rows_base + static_cast<size_t>(kStagedWarps) * warp_bytes);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kStagedWarps);
  const uint32_t bar = smem_u32(bars + warp);
  if (lane == 0) {
    mbar_init(bar, 1);
    if (warp == 0) *abort_flag = 0;
    fence_mbar_init();
  }
  // the per-column parameters are the same for every row: one copy per block
  for (int v = threadIdx.x; v < nvec; v += kStagedWarps * 32) {
    gs[v] = __ldg(reinterpret_cast<const uint4*>(gb) + v);
    if (bb) bs[v] = __ldg(reinterpret_cast<const uint4*>(bb) + v);
  }
  __syncthreads();

  const __half* xb = reinterpret_cast<const __half*>(p.x);
  const __half* rb = reinterpret_cast<const __half*>(p.residual);
  const int slabs = p.x_slab_cols > 0 ? static_cast<int>(p.cols / p.x_slab_cols) : 1;
  const int sc = p.x_slab_cols > 0 ? static_cast<int>(p.x_slab_cols) : cols;
  const float inv_n = 1.f / static_cast<float>(cols);
  const bool dyn = p.q_out && !p.q_scale;
  const float q_static = (p.q_out && p.q_scale) ? __ldg(p.q_scale) : 1.f;
  uint32_t parity = 0;

  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kStagedWarps + warp; row < p.rows;
       row += static_cast<int64_t>(gridDim.x) * kStagedWarps) {
    if (lane == 0) {
      // the buffers were last touched through ordinary loads and stores
      fence_proxy_async_smem();
      mbar_arrive_expect_tx(bar, row_bytes * (has_res ? 2u : 1u));
      for (int s = 0; s < slabs; ++s) {
        bulk_load_1d(smem_u32(my) + static_cast<uint32_t>(s) * sc * 2u, xb + s * p.x_slab_stride + row * sc,
                     static_cast<uint32_t>(sc) * 2u, bar);
      }
      if (has_res) bulk_load_1d(smem_u32(my) + row_bytes, rb + row * p.cols, row_bytes, bar);
    }
    if (!mbar_wait(bar, parity, abort_flag, &g_rowops_status, kRowStatusCopyTimeout)) break;
    parity ^= 1;

    // ---- pass 1: (x + residual, kept as fp16) and the sums
    float s1 = 0.f, ss = 0.f;
    __half* srow = (has_res && p.sum_out) ? reinterpret_cast<__half*>(p.sum_out) + row * p.cols : nullptr;
    if (has_res) {
#pragma unroll 2
      for (int v = lane; v < nvec; v += 32) {
        float a[E], b[E];
        VecT<__half>::unpack(xs[v], a);
        VecT<__half>::unpack(rs[v], b);
#pragma unroll
        for (int j = 0; j < E; ++j) a[j] += b[j];
        const uint4 packed = VecT<__half>::pack(a);
        xs[v] = packed;
        if (srow) *reinterpret_cast<uint4*>(srow + v * E) = packed;
        VecT<__half>::unpack(packed, a);
#pragma unroll
        for (int j = 0; j < E; ++j) {
          if (!RMS) s1 += a[j];
          else ss = __fmaf_rn(a[j], a[j], ss);
        }
      }
    } else {
#pragma unroll 2
      for (int v = lane; v < nvec; v += 32) {
        float a[E];
        VecT<__half>::unpack(xs[v], a);
#pragma unroll
        for (int j = 0; j < E; ++j) {
          if (!RMS) s1 += a[j];
          else ss = __fmaf_rn(a[j], a[j], ss);
        }
      }
    }
    float mean = 0.f;
    if (!RMS) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      mean = s1 * inv_n;
#pragma unroll 2
      for (int v = lane; v < nvec; v += 32) {
        float a[E];
        VecT<__half>::unpack(xs[v], a);
#pragma unroll
        for (int j = 0; j < E; ++j) {
          const float d = a[j] - mean;
          ss = __fmaf_rn(d, d, ss);
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = 1.f / sqrtf(ss * inv_n + p.eps);

    // ---- pass 2: y, rounded to fp16 in place; largest magnitude on packed halves
    __half* yrow = p.y ? reinterpret_cast<__half*>(p.y) + row * p.cols : nullptr;
    __half2 amax2 = __floats2half2_rn(0.f, 0.f);
#pragma unroll 2
    for (int v = lane; v < nvec; v += 32) {
      float a[E], g[E];
      VecT<__half>::unpack(xs[v], a);
      VecT<__half>::unpack(gs[v], g);
      if (bb) {
        float b[E];
        VecT<__half>::unpack(bs[v], b);
#pragma unroll
        for (int j = 0; j < E; ++j) a[j] = (a[j] - mean) * rstd * g[j] + b[j];
      } else {
#pragma unroll
        for (int j = 0; j < E; ++j) a[j] = (RMS ? a[j] : a[j] - mean) * rstd * g[j];
      }
      const uint4 packed = VecT<__half>::pack(a);
      if (yrow) *reinterpret_cast<uint4*>(yrow + v * E) = packed;
      if (p.q_out) {
        xs[v] = packed;
        const __half2* h = reinterpret_cast<const __half2*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) amax2 = __hmax2(amax2, __habs2(h[j]));
      }
    }
    if (p.q_out) {
      // ---- pass 3: int8
      float qs = q_static;
      if (dyn) {
        float m = fmaxf(__low2float(amax2), __high2float(amax2));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        qs = fmaxf(__fdiv_rn(m, 127.f), FLT_EPSILON);
        if (lane == 0 && p.q_row_scale) p.q_row_scale[row] = qs;
      }
      const RecipQuant d = make_recip_quant(qs);
      int8_t* qrow = p.q_out + row * p.cols;
#pragma unroll 2
      for (int v = lane; v < nvec; v += 32) {
        float y[E], q[E];
        VecT<__half>::unpack(xs[v], y);
        quant_vec_recip<E>(y, d, q);
        *reinterpret_cast<uint2*>(qrow + v * E) =
            make_uint2(pack4(q[0], q[1], q[2], q[3]), pack4(q[4], q[5], q[6], q[7]));
      }
    }
    __syncwarp();  // every lane is done with the buffers before the next row is requested
  }
  if (*abort_flag) {
    // a copy that was never seen to complete may still be landing: give it time before the
    // shared memory goes back to the SM
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
}
