// Included by qgemm_sm100.cu inside its anonymous namespace.
//
// qgemm_pair_kernel: the large-M path.  Two CTAs on neighbouring SMs (a
// cluster of 2, tcgen05 cta_group::2) compute one 256 x 256 output tile: CTA r
// of the pair owns rows [128 r, 128 r + 128) of the tile (its TMEM holds that
// half of the accumulator) and supplies half of the weight rows, so each CTA
// moves 32 KB per 128-byte K step for 128 x 256 x 128 multiply-adds, a third
// less L2 traffic per operation than two independent 128 x 256 tiles.  The
// leader CTA (rank 0) issues every MMA; mbarriers that both CTAs wait on are
// completed in both by tcgen05.commit with a CTA mask.  Loads are plain TMA
// tiles into the issuing CTA's own shared memory (no multicast).
//
// The epilogue leaves through shared memory: each epilogue warp stages a
// 32-row x 64-byte piece of the output (swizzled, conflict-free) and one lane
// hands it to a TMA store, which writes full 32-byte sectors and clips at the
// tensor edge; per-lane scattered 16-byte stores, one row per lane, were the
// bottleneck of the single-CTA kernel for short K.

constexpr int kPairStages = 5;
constexpr int kPairStageBytes = 2 * kTileM * kTileKBytes;  // A half + W half, 32 KB
constexpr int kPairBN = 256;
constexpr int kPairColsPerWarp = kPairBN / kEpiGroups;     // 64
constexpr int kPairStagingBytes = 32 * 64;                 // per epilogue warp: 32 rows x 64 B

struct PairSmem {
  static constexpr int kBarOffset = kPairStages * kPairStageBytes;
  static constexpr int kNumBars = 2 * kPairStages + 4;
  static constexpr int kMiscOffset = kBarOffset + kNumBars * 8;
  static constexpr int kScaleOffset = kMiscOffset + 16;
  static constexpr int kStagingOffset = ((kScaleOffset + kEpiWarps * 2 * kPairColsPerWarp * 4) + 1023) & ~1023;
  static constexpr int kTotal = kStagingOffset + kEpiWarps * kPairStagingBytes;
  static constexpr int kDynamic = kTotal + 1024;
};

// Where an epilogue warp reports that it has read its part of an accumulator
// buffer: the leader CTA's "accumulator empty" barrier.
struct PairRelease {
  uint32_t local_bar;   // this CTA's copy (used by the leader)
  uint32_t leader_bar;  // the leader's copy as a shared::cluster address
  bool is_leader;
};
__device__ __forceinline__ void pair_release(const PairRelease& rel, int lane) {
  tc_fence_before();
  __syncwarp();
  if (lane == 0) {
    // the accumulator left TMEM through registers, not through memory: no release of earlier writes is needed,
    // and a cluster-scope release made the peer CTA's epilogue 0.7 us per tile slower than the leader's
    if (rel.is_leader) mbar_arrive(rel.local_bar);
    else mbar_arrive_remote_relaxed(rel.leader_bar);
  }
}

// One epilogue warp's share of a pair tile: 64 columns of its 32 rows in four
// chunks of 16 columns.  The TMEM load of chunk c + 1 is in flight while chunk
// c is converted, and the accumulator buffer is handed back to the MMA warp as
// soon as the last load has landed in registers, before the arithmetic and the
// stores of the last chunk.  Results leave through a 32-row x 64-byte staging
// buffer (64-byte swizzle) and a TMA store per 64 bytes of row, or by direct
// stores when the output rows are not 16-byte aligned.
template <typename OutT, int ACT, int DIV, bool RS>
__device__ __forceinline__ void pair_epilogue_cols(uint32_t t_row, const float* cs, const float* cb,
                                                   const EpiCtx& ctx, OutT* out, int row0, int lane,
                                                   int col0, int M, int N, int64_t ldo,
                                                   uint8_t* stg, uint32_t stg_addr,
                                                   const CUtensorMap* tmap_out, int use_tma_store,
                                                   int vec_ok, const PairRelease& rel) {
  constexpr int CW = kPairColsPerWarp;
  constexpr int EB = static_cast<int>(sizeof(OutT));  // 16 columns = EB units of 16 bytes
  int nchunks = 0;
  if (row0 < M && col0 < N) {
    const int left = (N - col0 + 15) / 16;
    nchunks = left < CW / 16 ? left : CW / 16;
  }
  if (nchunks == 0) {  // uniform across the warp: nothing of this warp's share is inside the tensor
    pair_release(rel, lane);
    return;
  }

  auto process = [&](int c, uint32_t (&r)[16]) {
    const float4* cs4 = reinterpret_cast<const float4*>(cs + c * 16);
    const float4* cb4 = reinterpret_cast<const float4*>(cb + c * 16);
    if (!use_tma_store) {
      float v[16];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 s4 = cs4[i], b4 = cb4[i];
        v[4 * i + 0] = epi_value_t<ACT, DIV, RS, kUnitForm<OutT, DIV>>(static_cast<int32_t>(r[4 * i + 0]), s4.x, b4.x, ctx);
        v[4 * i + 1] = epi_value_t<ACT, DIV, RS, kUnitForm<OutT, DIV>>(static_cast<int32_t>(r[4 * i + 1]), s4.y, b4.y, ctx);
        v[4 * i + 2] = epi_value_t<ACT, DIV, RS, kUnitForm<OutT, DIV>>(static_cast<int32_t>(r[4 * i + 2]), s4.z, b4.z, ctx);
        v[4 * i + 3] = epi_value_t<ACT, DIV, RS, kUnitForm<OutT, DIV>>(static_cast<int32_t>(r[4 * i + 3]), s4.w, b4.w, ctx);
      }
      if (row0 + lane < M) {
        const int n0 = col0 + c * 16;
        OutT* dst = out + static_cast<int64_t>(row0 + lane) * ldo + n0;
        if (vec_ok && n0 + 16 <= N) {
          store_row16_vec<OutT, kUnitForm<OutT, DIV>>(dst, v, r);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (n0 + j < N) store_one<OutT, kUnitForm<OutT, DIV>>(dst + j, v[j], static_cast<int32_t>(r[j]));
          }
        }
      }
      return;
    }
    const int unit0 = (c * EB) & 3;  // first 16-byte unit of this chunk inside the 64-byte staging row
    if (unit0 == 0) {
      // a new 64-byte round: the previous round's store must have read the staging buffer
      if (lane == 0) tma_store_wait_read();
      __syncwarp();
    }
    // four values at a time, packed at once, so that few converted values are live together
    uint32_t w[4 * EB];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (std::is_same_v<OutT, int32_t>) {
        w[4 * i] = r[4 * i], w[4 * i + 1] = r[4 * i + 1], w[4 * i + 2] = r[4 * i + 2], w[4 * i + 3] = r[4 * i + 3];
      } else {
        const float4 s4 = cs4[i], b4 = cb4[i];
        const float v0 = epi_value_t<ACT, DIV, RS, kUnitForm<OutT, DIV>>(static_cast<int32_t>(r[4 * i + 0]), s4.x, b4.x, ctx);
        const float v1 = epi_value_t<ACT, DIV, RS, kUnitForm<OutT, DIV>>(static_cast<int32_t>(r[4 * i + 1]), s4.y, b4.y, ctx);
        const float v2 = epi_value_t<ACT, DIV, RS, kUnitForm<OutT, DIV>>(static_cast<int32_t>(r[4 * i + 2]), s4.z, b4.z, ctx);
        const float v3 = epi_value_t<ACT, DIV, RS, kUnitForm<OutT, DIV>>(static_cast<int32_t>(r[4 * i + 3]), s4.w, b4.w, ctx);
        if constexpr (EB == 1) {
          w[i] = pack4_s8<kUnitForm<OutT, DIV>>(v0, v1, v2, v3);
        } else if constexpr (EB == 2) {
          __half2 h0 = __floats2half2_rn(v0, v1), h1 = __floats2half2_rn(v2, v3);
          w[2 * i] = *reinterpret_cast<uint32_t*>(&h0);
          w[2 * i + 1] = *reinterpret_cast<uint32_t*>(&h1);
        } else {
          w[4 * i] = __float_as_uint(v0), w[4 * i + 1] = __float_as_uint(v1);
          w[4 * i + 2] = __float_as_uint(v2), w[4 * i + 3] = __float_as_uint(v3);
        }
      }
    }
    // unit index inside the 64-byte row is xor-ed with ((row >> 1) & 3): the 64-byte TMA swizzle
#pragma unroll
    for (int u = 0; u < EB; ++u) {
      const uint32_t off = lane * 64 + (((unit0 + u) ^ ((lane >> 1) & 3)) << 4);
      *reinterpret_cast<uint4*>(stg + off) = make_uint4(w[4 * u], w[4 * u + 1], w[4 * u + 2], w[4 * u + 3]);
    }
    const bool round_ends = ((unit0 + EB) & 3) == 0 || c + 1 == nchunks;
    if (round_ends) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int first_col = (c * 16 * EB / 64) * (64 / EB);  // first column of this round
        tma_store_2d(tmap_out, stg_addr, (col0 + first_col) * EB, row0);
        tma_store_commit();
      }
    }
  };

  uint32_t ra[16], rb[16];
  tmem_ld_x16(t_row, ra);
#pragma unroll 1
  for (int c = 0; c < nchunks; c += 2) {
    tmem_ld_wait_regs(ra);
    if (c + 1 < nchunks) tmem_ld_x16(t_row + (c + 1) * 16, rb);
    else pair_release(rel, lane);
    process(c, ra);
    if (c + 1 < nchunks) {
      tmem_ld_wait_regs(rb);
      if (c + 2 < nchunks) tmem_ld_x16(t_row + (c + 2) * 16, ra);
      else pair_release(rel, lane);
      process(c + 1, rb);
    }
  }
}

// The epilogue mode (activation, requantisation form, per-row scales) is a
// template parameter of the kernel, chosen by the host: with every mode inlined
// behind one switch the compiler kept the union of all modes' temporaries live
// and spilled in each of them.
template <typename OutT, int ACT, int DIV, bool RS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kTiledThreads, 1)
qgemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_w,
                  const __grid_constant__ CUtensorMap tmap_out, EpiParams ep, int num_kb, int tiles_m,
                  int tiles_n, int use_tma_store, int vec_ok, SlabA slab) {
  using L = PairSmem;
  constexpr int STAGES = kPairStages;
  constexpr int BN = kPairBN;
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
  float* s_scale = reinterpret_cast<float*>(smem + L::kScaleOffset);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  constexpr uint32_t kTmemCols = 2 * BN;
  constexpr int kProducerWarp = kEpiWarps;
  constexpr int kMmaWarp = kEpiWarps + 1;

  if (threadIdx.x == kProducerWarp * 32) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_out);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);   // the leader's own arrive; bytes of both CTAs are counted on it
      mbar_init(empty_bar(s), 1);  // one commit per use, delivered to both CTAs
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 2 * kEpiWarps);  // leader's copy is the one waited on: both CTAs' epilogue warps
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // set-up done while the kernel before this one may still have been finishing
  grid_dep_launch();
  grid_dep_wait();

  const int num_tiles = tiles_m * tiles_n;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (warp == kProducerWarp) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        const int m_blk = tile / tiles_n;
        const int n_blk = tile % tiles_n;
        const int a_row = m_blk * 2 * kTileM + static_cast<int>(rank) * kTileM;
        const int w_row = n_blk * BN + static_cast<int>(rank) * kTileM;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, &g_kernel_status,
                         kStatusTimeoutEmpty);
          if (!ok) break;
          if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * kPairStageBytes);
          const uint32_t a_dst = smem_base + stage * kPairStageBytes;
          const KCoord kc = k_coord(slab, kb);
          tma_load_2d_pair(a_dst, &tmap_a, full_bar(stage), kc.ax, kc.ay + a_row);
          tma_load_2d_pair(a_dst + kTileM * kTileKBytes, &tmap_w, full_bar(stage), kc.wx, w_row);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_i8_idesc(2 * kTileM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc_buf = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        ok = mbar_wait(tempty_bar(acc_buf), acc_phase ^ 1, abort_flag, &g_kernel_status,
                       kStatusTimeoutTmemEmpty);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc_buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(full_bar(stage), phase, abort_flag, &g_kernel_status, kStatusTimeoutFull);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * kPairStageBytes;
          const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
          const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + kTileM * kTileKBytes);
#pragma unroll
          for (int k = 0; k < kTileKBytes / kMmaK; ++k) {
            umma_i8_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(tfull_bar(acc_buf));
        acc_buf ^= 1;
        if (acc_buf == 0) acc_phase ^= 1;
      }
    }
  } else {
    constexpr int CW = kPairColsPerWarp;
    const int q = warp & 3;
    const int g = warp >> 2;
    float* cs = s_scale + warp * 2 * CW;
    float* cb = cs + CW;
    uint8_t* stg = smem + L::kStagingOffset + warp * kPairStagingBytes;
    const uint32_t stg_addr = smem_u32(stg);
    const uint32_t tempty_leader0 = map_to_cta(tempty_bar(0), 0);
    const uint32_t tempty_leader1 = map_to_cta(tempty_bar(1), 0);
    int acc_buf = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    EpiCtx ctx = make_epi_ctx(ep);
    OutT* out = reinterpret_cast<OutT*>(ep.out);
    // Column constants of the tile after the current one travel in registers:
    // their loads are issued before the current tile's arithmetic and finished
    // after it.  Fetched in line they were four dependent trips to L2 per tile
    // on the epilogue warps' critical path, more than a short-K main loop takes.
    constexpr int CPL = CW / 32;  // columns per lane
    ColRaw raw[CPL];
    auto request_consts = [&](int tile) {
      const int64_t c0 = static_cast<int64_t>(tile % tiles_n) * BN + g * CW;
#pragma unroll
      for (int i = 0; i < CPL; ++i) {
        const int64_t n = c0 + lane + 32 * i;
        raw[i] = col_raw_load(ep, n < ep.N ? n : ep.N - 1);
      }
    };
    if (cluster_id < num_tiles) request_consts(cluster_id);
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      const int m_blk = tile / tiles_n;
      const int n_blk = tile % tiles_n;
      const int col0 = n_blk * BN + g * CW;
      __syncwarp();
#pragma unroll
      for (int i = 0; i < CPL; ++i) {
        const int j = lane + 32 * i;
        col_raw_finish(ep, ctx, raw[i], col0 + j < ep.N, cs[j], cb[j]);
      }
      __syncwarp();
      if (tile + num_clusters < num_tiles) request_consts(tile + num_clusters);
      ok = mbar_wait(tfull_bar(acc_buf), acc_phase, abort_flag, &g_kernel_status,
                     kStatusTimeoutTmemFull);
      if (!ok) break;
      tc_fence_after();
      const int row0 = m_blk * 2 * kTileM + static_cast<int>(rank) * kTileM + q * 32;
      if (ctx.has_rs) ctx.rs = (row0 + lane < ep.M) ? __ldg(ep.x_scale + row0 + lane) : 1.f;
      const uint32_t t_row =
          tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc_buf * BN + g * CW;
      // the accumulator buffer is handed back inside, as soon as it has been read
      const PairRelease rel = {tempty_bar(acc_buf), acc_buf == 0 ? tempty_leader0 : tempty_leader1, rank == 0};
      pair_epilogue_cols<OutT, ACT, DIV, RS>(t_row, cs, cb, ctx, out, row0, lane, col0, static_cast<int>(ep.M),
                                             static_cast<int>(ep.N), ep.ldo, stg, stg_addr, &tmap_out,
                                             use_tma_store, vec_ok, rel);
      acc_buf ^= 1;
      if (acc_buf == 0) acc_phase ^= 1;
    }
    if (use_tma_store && lane == 0) tma_store_wait_all();
  }

  // Wind-down: nothing may leave while the other CTA can still touch its
  // shared memory or barriers, so both CTAs meet before TMEM is released.
  __syncwarp();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}
