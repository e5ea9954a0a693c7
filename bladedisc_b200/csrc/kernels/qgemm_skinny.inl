// Few-row path of the int8 quantized linear (included by qgemm_sm100.cu).
//
// For a handful up to a few hundred activation rows the weight is the whole
// traffic, so the job is to keep every SM streaming its share of W and to keep
// the latency chain around that stream short.  Instead of splitting K (partial
// sums through global scratch, a fence, an atomic and a second pass) the
// output channels are cut finer: a CTA owns BN channels, BN any multiple of 16
// chosen so that one wave of CTAs covers N, and walks the full K itself.
//
//   A operand (MMA M = 128): activation rows.  Only MT = 16/32/64/128 rows are
//     fetched per K block; the rows of the 128-row operand above MT are whatever
//     follows in shared memory.  They only feed accumulator rows nobody reads.
//   B operand (MMA N = BN): BN weight rows.
//   grid = (ceil(N / BN), ceil(M / 128)); CTAs of different row tiles read the
//     same weight slab at about the same time, so it crosses HBM once.
//
// Warp roles as in the small-M kernel: warp 0 TMA, warp 1 TMEM + MMA, warps
// 2..17 epilogue (TMEM lane quadrant = warp & 3 = 32 rows; the four warps of a
// quadrant interleave 16-column chunks).
//
// Long K and few tiles (the launcher's rule): gridDim.z
// blocks form a thread-block cluster along z and share a tile of 128 channels,
// each walking 1/z of the K blocks.  Every block writes its partial int32 tile
// from TMEM to its own shared memory (the stage ring is free by then), the
// cluster meets, and block r finishes the r-th slice of the tile: it adds the
// partial sums of all blocks in rank order through distributed shared memory,
// runs the epilogue on them and stores.  A second cluster barrier keeps every
// block's tile alive until all have read it.

constexpr int kSkinnyStageRegion = 184 * 1024;  // a short activation tile is read up to 16 KB past its end
constexpr int kSkinnyBarOffset = 200 * 1024;
constexpr int kSkinnyScaleOffset = kSkinnyBarOffset + 256;
constexpr int kSkinnyMaxBN = 256;  // widest channel block: above 128 only where N needs it to stay in one wave
constexpr int kSkinnyDynamic = kSkinnyScaleOffset + 2 * kSkinnyMaxBN * 4 + 1024;
constexpr int kSkinnyTilePad = 4;  // int32 words added to a row of the partial tile: 16-byte stores of a warp spread over the banks

template <typename OutT, int ACT, int DIV, bool RS>
__device__ __forceinline__ void skinny_epilogue_cols(uint32_t t_row, const float* cs, const float* cb,
                                                     const EpiCtx& ctx, OutT* out, int64_t m,
                                                     bool row_ok, int64_t col0, int64_t N,
                                                     int64_t ldo, int vec_ok, int g, int BN) {
#pragma unroll 1
  for (int c = g; c < BN / 16; c += 4) {
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

template <typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
qgemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_x,
                    const __grid_constant__ CUtensorMap tmap_w, EpiParams ep, int MT, int BN,
                    int stages, int kbs, int num_kb, int vec_ok, int k3d, SlabA slab, int early_w, int kb_per_rank) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + kSkinnyBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kSmallMaxStages + s); };
  const uint32_t tfull_bar = bar_base + 8u * (2 * kSmallMaxStages);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kSkinnyBarOffset + 8 * (2 * kSmallMaxStages + 1));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_cs = reinterpret_cast<float*>(smem + kSkinnyScaleOffset);
  float* s_cb = s_cs + kSkinnyMaxBN;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * BN;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kTileM;
  const uint32_t w_bytes = static_cast<uint32_t>(BN) * kTileKBytes;
  const uint32_t x_bytes = static_cast<uint32_t>(MT) * kTileKBytes;
  const uint32_t stage_bytes = kbs * (w_bytes + x_bytes);  // multiples of 1024
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(BN)) tmem_cols <<= 1;
  // K split over the thread-block cluster (gridDim.z blocks along z): rank r walks K blocks
  // [r * kb_per_rank, (r + 1) * kb_per_rank); the partial tiles meet in distributed shared memory below.
  const int ksplit = static_cast<int>(gridDim.z);
  const int rank = static_cast<int>(blockIdx.z);
  const int kb_lo = ksplit > 1 ? min(num_kb, rank * kb_per_rank) : 0;
  const int kb_hi = ksplit > 1 ? min(num_kb, kb_lo + kb_per_rank) : num_kb;

  // Loads of one stage (K blocks kb0 .. kb0 + nk - 1).  which: 1 = weight, 2 =
  // activation, 3 = both; the call that brings the weight arms the barrier.
  auto issue_stage = [&](int stage, int kb0, int which) {
    const uint32_t w_dst = smem_base + stage * stage_bytes;
    const uint32_t x_dst = w_dst + kbs * w_bytes;
    if (k3d) {
      // K blocks past the end of K read as zero and still count their bytes
      if (which & 1) {
        mbar_arrive_expect_tx(full_bar(stage), stage_bytes);
        tma_load_3d(w_dst, &tmap_w, full_bar(stage), 0, static_cast<int>(n0), kb0);
      }
      if (which & 2) tma_load_3d(x_dst, &tmap_x, full_bar(stage), 0, static_cast<int>(m0), kb0);
      return;
    }
    const int nk = kb_hi - kb0 < kbs ? kb_hi - kb0 : kbs;
    if (which & 1) mbar_arrive_expect_tx(full_bar(stage), nk * (w_bytes + x_bytes));
    for (int c = 0; c < nk; ++c) {
      const KCoord kc = k_coord(slab, kb0 + c);
      if (which & 1) tma_load_2d(w_dst + c * w_bytes, &tmap_w, full_bar(stage), kc.wx, static_cast<int>(n0));
      if (which & 2)
        tma_load_2d(x_dst + c * x_bytes, &tmap_x, full_bar(stage), kc.ax, kc.ay + static_cast<int>(m0));
    }
  };

  // The producer needs nothing but its own barriers, so the first ring of
  // stages is on its way before the accumulator columns are allocated and the
  // CTA meets at the barrier below.
  int first_kb = kb_lo;
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_w);
      tma_prefetch_desc(&tmap_x);
      for (int s = 0; s < stages; ++s) {
        mbar_init(full_bar(s), 1);
        mbar_init(empty_bar(s), 1);
      }
      mbar_init(tfull_bar, 1);
      *abort_flag = 0;
      fence_mbar_init();
      grid_dep_launch();  // the next kernel on the stream may begin its own prologue
      if (early_w) {
        // The weight does not depend on the kernel before this one: its first
        // ring of stages is requested while that kernel may still be running.
        int kb = kb_lo;
        for (int s = 0; s < stages && kb < kb_hi; ++s, kb += kbs) issue_stage(s, kb, 1);
        grid_dep_wait();
        for (int s = 0; s < stages && first_kb < kb_hi; ++s, first_kb += kbs) issue_stage(s, first_kb, 2);
      } else {
        grid_dep_wait();
        for (int s = 0; s < stages && first_kb < kb_hi; ++s, first_kb += kbs) issue_stage(s, first_kb, 3);
      }
    }
  } else if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // If anything is left the ring has been filled exactly once: stage 0 is
      // next, one phase later.
      int stage = 0;
      uint32_t phase = 1;
      for (int kb0 = first_kb; kb0 < kb_hi; kb0 += kbs) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, &g_kernel_status,
                       kStatusTimeoutEmpty))
          break;
        issue_stage(stage, kb0, 3);
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_i8_idesc(kTileM, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb0 = kb_lo; kb0 < kb_hi; kb0 += kbs) {
        const int nk = kb_hi - kb0 < kbs ? kb_hi - kb0 : kbs;
        ok = mbar_wait(full_bar(stage), phase, abort_flag, &g_kernel_status, kStatusTimeoutFull);
        if (!ok) break;
        tc_fence_after();
        const uint32_t w_addr = smem_base + stage * stage_bytes;
        const uint32_t x_addr = w_addr + kbs * w_bytes;
        for (int c = 0; c < nk; ++c) {
          const uint64_t a_desc = make_kmajor_sw128_desc(x_addr + c * x_bytes);
          const uint64_t b_desc = make_kmajor_sw128_desc(w_addr + c * w_bytes);
#pragma unroll
          for (int k = 0; k < kTileKBytes / kMmaK; ++k) {
            umma_i8(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb0 + c != kb_lo || k != 0) ? 1u : 0u);
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
    const int q = warp & 3;
    const int g = (warp - 2) >> 2;
    const int et = threadIdx.x - 64;
    grid_dep_wait();  // scales may come from the kernel before this one; the output may still be read by it
    // Column constants while the weight streams.
    EpiCtx ctx = make_epi_ctx(ep);
    for (int i = et; i < BN; i += kThreads - 64) {
      const int64_t n = n0 + i;
      float cs = 0.f, cb = 0.f;
      if (n < ep.N) col_consts(ep, ctx, n, cs, cb);
      s_cs[i] = cs;
      s_cb[i] = cb;
    }
    const int64_t m = m0 + q * 32 + lane;
    const bool row_ok = m < ep.M;
    if (ctx.has_rs && row_ok) ctx.rs = __ldg(ep.x_scale + m);
    asm volatile("bar.sync 1, %0;" ::"r"(kThreads - 64) : "memory");

    const bool ok = mbar_wait(tfull_bar, 0, abort_flag, &g_kernel_status, kStatusTimeoutTmemFull);
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    if (ksplit == 1) {
      if (ok && m0 + q * 32 < ep.M) {  // a quadrant without rows has nothing to read
        tc_fence_after();
        OutT* out = reinterpret_cast<OutT*>(ep.out);
        const int mode = epi_mode(ctx);
        DISC_EPI_SWITCH(mode, (skinny_epilogue_cols<OutT, ACT, DIV, RS>(
                                  t_row, s_cs, s_cb, ctx, out, m, row_ok, n0, ep.N, ep.ldo, vec_ok, g, BN)));
      }
    } else if (q * 32 < MT) {
      // partial sums of this block's K range -> its shared memory (the stages are free: every MMA has read them)
      tc_fence_after();
      int32_t* tile = reinterpret_cast<int32_t*>(smem);
      const int pitch = BN + kSkinnyTilePad;
      const int r_local = q * 32 + lane;
      const bool have = ok && kb_hi > kb_lo;
#pragma unroll 1
      for (int c = g; c < BN / 16; c += 4) {
        uint32_t r[16];
        if (have) {
          tmem_ld_x16(t_row + c * 16, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = 0u;
        }
        if (r_local < MT) {
          int4* dst = reinterpret_cast<int4*>(tile + r_local * pitch + c * 16);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            dst[j] = make_int4(static_cast<int>(r[4 * j]), static_cast<int>(r[4 * j + 1]), static_cast<int>(r[4 * j + 2]),
                               static_cast<int>(r[4 * j + 3]));
        }
      }
    }
  }

  if (ksplit > 1) {
    // Every block finishes a slice of the tile: the partial sums of all ranks, added in rank order (int32: exact
    // in any order), then the epilogue.  All threads of all blocks of the cluster meet at both barriers.
    cluster_sync_all();
    if (warp >= 2) {
      const int et = threadIdx.x - 64;
      const EpiCtx ctx0 = make_epi_ctx(ep);
      const int pitch = BN + kSkinnyTilePad;
      const int rows_valid = static_cast<int>(min(static_cast<int64_t>(MT), ep.M - m0));
      const int groups = BN / 4;
      const int items = rows_valid * groups;
      const int per = (items + ksplit - 1) / ksplit;
      const int i_end = min(items, (rank + 1) * per);
      const uint32_t tile_addr = smem_base;
      OutT* out = reinterpret_cast<OutT*>(ep.out);
      for (int i = rank * per + et; i < i_end; i += kThreads - 64) {
        const int row = i / groups;
        const int col = (i - row * groups) * 4;
        const uint32_t local = tile_addr + static_cast<uint32_t>(row * pitch + col) * 4u;
        int a0 = 0, a1 = 0, a2 = 0, a3 = 0;
        for (int j = 0; j < ksplit; ++j) {
          int v0, v1, v2, v3;
          asm volatile("ld.shared::cluster.v4.s32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
                       : "r"(map_to_cta(local, static_cast<uint32_t>(j))));
          a0 += v0;
          a1 += v1;
          a2 += v2;
          a3 += v3;
        }
        const int64_t mrow = m0 + row;
        EpiCtx ctx = ctx0;
        if (ctx.has_rs) ctx.rs = __ldg(ep.x_scale + mrow);
        const int acc[4] = {a0, a1, a2, a3};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int64_t n = n0 + col + e;
          if (n < ep.N)
            store_one_rt<OutT>(out + mrow * ep.ldo + n, epi_value(acc[e], s_cs[col + e], s_cb[col + e], ctx), acc[e], ctx);
        }
      }
    }
    cluster_sync_all();  // no block leaves while its tile may still be read
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
