// Included by qgemm_sm100.cu inside its anonymous namespace.
//
// qgemm_gemv_kernel: M <= 8 activation rows (decode steps of a generative
// model).  With so few rows the product is a matrix-vector stream: every
// weight byte is used M times and the tensor-core path's fixed latencies
// (TMEM allocation, TMA descriptor fetch, barrier hand-offs, split-K reduction)
// cost more than the arithmetic.  Here a warp owns two weight rows at a time,
// lanes walk K in 16-byte steps with four loads per row in flight, the
// activations sit in shared memory, the products are dp4a (int8 x int8 -> int32,
// exact), and one shuffle tree per activation row finishes the sum.  No
// scratch, no split.

constexpr int kGemvThreads = 256;
constexpr int kGemvRows = 2;     // weight rows a warp works on at once
constexpr int kGemvUnroll = 4;   // 16-byte steps per row in flight
constexpr int64_t kGemvMaxK = 16384;

template <typename OutT, int MR>
__global__ void __launch_bounds__(kGemvThreads, 2)
qgemm_gemv_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ w, int K, int64_t lda,
                  int64_t ldw, EpiParams ep) {
  extern __shared__ uint4 xs[];  // [MR][K / 16]
  const int kv = K >> 4;         // 16-byte vectors per row
  grid_dep_launch();  // the next kernel on the stream may start its prologue
  grid_dep_wait();    // everything read below may come from the kernel before this one
  const int M = static_cast<int>(ep.M);
  for (int i = threadIdx.x; i < MR * kv; i += kGemvThreads) {
    const int m = i / kv, v = i - m * kv;
    xs[i] = m < M ? *reinterpret_cast<const uint4*>(a + m * lda + v * 16) : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();

  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * (kGemvThreads / 32) + (threadIdx.x >> 5);
  const int warps_total = gridDim.x * (kGemvThreads / 32);
  const int64_t N = ep.N;
  const int64_t groups = (N + kGemvRows - 1) / kGemvRows;
  EpiCtx ctx = make_epi_ctx(ep);
  OutT* out = reinterpret_cast<OutT*>(ep.out);

  for (int64_t grp = warp_global; grp < groups; grp += warps_total) {
    const int64_t n0 = grp * kGemvRows;
    int32_t acc[kGemvRows][MR];
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r)
#pragma unroll
      for (int m = 0; m < MR; ++m) acc[r][m] = 0;
    const int8_t* wr[kGemvRows];
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) wr[r] = w + (n0 + r < N ? n0 + r : n0) * ldw;  // a padding row re-reads row n0

    for (int v0 = lane; v0 < kv; v0 += 32 * kGemvUnroll) {
      uint4 wv[kGemvRows][kGemvUnroll];
#pragma unroll
      for (int u = 0; u < kGemvUnroll; ++u) {
        const int v = v0 + u * 32;
#pragma unroll
        for (int r = 0; r < kGemvRows; ++r)
          wv[r][u] = v < kv ? __ldcs(reinterpret_cast<const uint4*>(wr[r]) + v) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < kGemvUnroll; ++u) {
        const int v = v0 + u * 32;
        if (v >= kv) break;
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          const uint4 xv = xs[m * kv + v];
#pragma unroll
          for (int r = 0; r < kGemvRows; ++r) {
            int32_t s = acc[r][m];
            s = __dp4a(static_cast<int>(wv[r][u].x), static_cast<int>(xv.x), s);
            s = __dp4a(static_cast<int>(wv[r][u].y), static_cast<int>(xv.y), s);
            s = __dp4a(static_cast<int>(wv[r][u].z), static_cast<int>(xv.z), s);
            s = __dp4a(static_cast<int>(wv[r][u].w), static_cast<int>(xv.w), s);
            acc[r][m] = s;
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r)
#pragma unroll
      for (int m = 0; m < MR; ++m) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[r][m] += __shfl_xor_sync(0xffffffffu, acc[r][m], o);
      }
    // lane m finishes activation row m
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) {
      const int64_t n = n0 + r;
      int32_t mine = 0;
#pragma unroll
      for (int m = 0; m < MR; ++m)
        if (lane == m) mine = acc[r][m];
      if (lane < M && n < N) {
        if (ctx.has_rs) ctx.rs = __ldg(ep.x_scale + lane);
        float cs, cb;
        col_consts(ep, ctx, n, cs, cb);
        const float v = epi_value(mine, cs, cb, ctx);
        store_one_rt<OutT>(out + static_cast<int64_t>(lane) * ep.ldo + n, v, mine, ctx);
      }
    }
  }
}

template <typename OutT, int MR>
cudaError_t launch_gemv_t(const QGemmParams& p, cudaStream_t stream) {
  auto kern = qgemm_gemv_kernel<OutT, MR>;
  const int smem = static_cast<int>(MR * p.K);
  cudaError_t st = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (st != cudaSuccess) return st;
  const int64_t groups = (p.N + kGemvRows - 1) / kGemvRows;
  int64_t blocks = (groups + kGemvThreads / 32 - 1) / (kGemvThreads / 32);
  const int64_t cap = 2 * static_cast<int64_t>(sm_count());
  if (blocks > cap) blocks = cap;
  return launch_dependent(kern, dim3(static_cast<unsigned>(blocks)), dim3(kGemvThreads), smem, stream, p.a, p.w,
                          static_cast<int>(p.K), p.lda, p.ldw, make_epi(p));
}

template <typename OutT>
cudaError_t launch_gemv(const QGemmParams& p, cudaStream_t stream, const char** err) {
  if (p.M > 8 || p.K > kGemvMaxK) {
    if (err) *err = "gemv qgemm path: M <= 8 and K <= 16384 only";
    return cudaErrorInvalidValue;
  }
  if (p.M <= 1) return launch_gemv_t<OutT, 1>(p, stream);
  if (p.M <= 2) return launch_gemv_t<OutT, 2>(p, stream);
  if (p.M <= 4) return launch_gemv_t<OutT, 4>(p, stream);
  return launch_gemv_t<OutT, 8>(p, stream);
}
