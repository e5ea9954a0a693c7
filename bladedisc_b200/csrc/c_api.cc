// Direct (non-dispatched) C entry points: plain pointers and sizes in, a
// status code out.  The custom calls of ral/calls.cc land on the same launch
// functions.
#include <dlfcn.h>

#include <algorithm>
#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "ral/context.h"
#include "ral/conv_plan.h"
#include "ral/cu_driver_dyn.h"
#include "ral/metadata.h"
#include "ral/nccl_dyn.h"
#include "../../include/disc_b200_ral.h"
#include "kernels/attention.h"
#include "kernels/observer.h"
#include "kernels/qconv.h"
#include "kernels/qgemm.h"
#include "kernels/rowops.h"
#include "kernels/woq_gemm.h"
#include "ral/pdl_attr.h"

namespace {

thread_local std::string g_last_error;

int32_t finish(cudaError_t st, const char* what, const char* detail) {
  if (st == cudaSuccess) {
    return 0;
  }
  g_last_error = std::string(what) + ": " + (detail ? detail : cudaGetErrorString(st));
  return static_cast<int32_t>(st);
}

void render(const disc_b200::ral::Attr& a, std::string& o) {
  using disc_b200::ral::Attr;
  switch (a.kind) {
    case Attr::kDict: {
      o += "{";
      bool first = true;
      for (const auto& kv : a.dict) {
        if (!first) o += ", ";
        first = false;
        o += kv.first + ": ";
        render(*kv.second, o);
      }
      o += "}";
      break;
    }
    case Attr::kStr: o += "\"" + a.str + "\""; break;
    case Attr::kBool: o += a.b ? "true" : "false"; break;
    case Attr::kInt: o += std::to_string(a.i); break;
    case Attr::kFloat: {
      char buf[64];
      snprintf(buf, sizeof(buf), "%.17g", a.f);
      o += buf;
      break;
    }
    case Attr::kIntArray: {
      o += "[";
      for (size_t i = 0; i < a.ints.size(); ++i) o += (i ? ", " : "") + std::to_string(a.ints[i]);
      o += "]";
      break;
    }
    case Attr::kArray: {
      o += "[";
      for (size_t i = 0; i < a.array.size(); ++i) {
        if (i) o += ", ";
        render(*a.array[i], o);
      }
      o += "]";
      break;
    }
    case Attr::kDense: {
      o += "dense<" + a.elem_type + std::to_string(a.elem_bits) + "[";
      for (size_t i = 0; i < a.shape.size(); ++i) o += (i ? "x" : "") + std::to_string(a.shape[i]);
      o += "]:" + std::to_string(a.raw.size()) + "B>";
      break;
    }
  }
}

disc_b200::QGemmParams to_params(const disc_b200_qgemm_args* a) {
  disc_b200::QGemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.a = a->a;
  p.w = a->w;
  p.out = a->out;
  p.M = a->M;
  p.N = a->N;
  p.K = a->K;
  p.lda = a->lda > 0 ? a->lda : a->K;
  p.ldw = a->ldw > 0 ? a->ldw : a->K;
  p.ldo = a->ldo > 0 ? a->ldo : a->N;
  p.x_scale = a->x_scale;
  p.w_scale = a->w_scale;
  p.out_scale = a->out_scale;
  p.bias = a->bias;
  p.x_scale_kind = a->x_scale ? a->x_scale_kind : disc_b200::kScaleNone;
  p.w_scale_kind = a->w_scale ? a->w_scale_kind : disc_b200::kScaleNone;
  p.out_scale_kind = a->out_scale ? a->out_scale_kind : disc_b200::kScaleNone;
  p.bias_kind = a->bias ? a->bias_kind : disc_b200::kBiasNone;
  p.fold_out_scale = a->fold_out_scale;
  p.div_out_scale = a->div_out_scale;
  p.div_exact = a->div_exact;
  p.act = a->act;
  p.out_dtype = a->out_dtype;
  p.path = a->path;
  p.split_k = a->split_k;
  p.splitk_ws = static_cast<int32_t*>(a->splitk_ws);
  p.splitk_ws_bytes = a->splitk_ws_bytes;
  p.a_slabs = a->a_slabs;
  p.a_slab_cols = a->a_slab_cols;
  p.a_slab_stride = a->a_slab_stride;
  p.weights_static = a->weights_static;
  return p;
}

}  // namespace

extern "C" {

int32_t disc_b200_qgemm(const disc_b200_qgemm_args* args, void* stream) {
  if (!args) {
    g_last_error = "qgemm: null args";
    return 1;
  }
  const char* detail = nullptr;
  cudaError_t st = disc_b200::qgemm_launch(to_params(args), static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "qgemm", detail);
}

int32_t disc_b200_qgemm_small_m_noalloc(const disc_b200_qgemm_args* args, void* stream) {
  if (!args) {
    g_last_error = "no-alloc small-M qgemm: null args";
    return 1;
  }
  const char* detail = nullptr;
  const cudaError_t st =
      disc_b200::qgemm_small_m_noalloc_launch(to_params(args), static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "qgemm_small_m_noalloc", detail);
}

int64_t disc_b200_qgemm_small_m_noalloc_capacity(void) { return disc_b200::qgemm_small_m_noalloc_capacity(); }

int64_t disc_b200_qgemm_scratch_bytes(int64_t M, int64_t N, int64_t K) {
  return disc_b200::qgemm_splitk_ws_bytes(M, N, K);
}

// ---- quantized linear on host buffers: rows streamed in, multiplied and streamed out in chunks
struct disc_b200_host_linear {
  int device = 0;
  int64_t chunk_rows = 0, K = 0, N = 0;
  int out_bytes = 1;
  int slots = 0;
  std::vector<int8_t*> a;       // device staging, one per slot
  std::vector<char*> o;
  cudaStream_t s_in = nullptr, s_mm = nullptr, s_out = nullptr;
  std::vector<cudaEvent_t> in_done, mm_done, out_done;
  cudaEvent_t start = nullptr, finished = nullptr;
};

void disc_b200_host_linear_destroy(disc_b200_host_linear* h) {
  if (!h) return;
  for (auto p : h->a) cudaFree(p);
  for (auto p : h->o) cudaFree(p);
  for (auto e : h->in_done) cudaEventDestroy(e);
  for (auto e : h->mm_done) cudaEventDestroy(e);
  for (auto e : h->out_done) cudaEventDestroy(e);
  if (h->start) cudaEventDestroy(h->start);
  if (h->finished) cudaEventDestroy(h->finished);
  if (h->s_in) cudaStreamDestroy(h->s_in);
  if (h->s_mm) cudaStreamDestroy(h->s_mm);
  if (h->s_out) cudaStreamDestroy(h->s_out);
  delete h;
}

disc_b200_host_linear* disc_b200_host_linear_create(int64_t chunk_rows, int64_t K, int64_t N, int32_t out_dtype,
                                                    int32_t slots) {
  if (chunk_rows <= 0 || K <= 0 || N <= 0 || slots < 2 || slots > 8 ||
      (out_dtype != DISC_B200_OUT_I8 && out_dtype != DISC_B200_OUT_F16)) {
    g_last_error = "host_linear_create: chunk_rows, K, N positive, 2..8 slots, int8 or f16 output";
    return nullptr;
  }
  auto* h = new disc_b200_host_linear;
  h->chunk_rows = chunk_rows;
  h->K = K;
  h->N = N;
  h->out_bytes = out_dtype == DISC_B200_OUT_I8 ? 1 : 2;
  h->slots = slots;
  bool ok = cudaGetDevice(&h->device) == cudaSuccess;
  ok = ok && cudaStreamCreateWithFlags(&h->s_in, cudaStreamNonBlocking) == cudaSuccess;
  ok = ok && cudaStreamCreateWithFlags(&h->s_mm, cudaStreamNonBlocking) == cudaSuccess;
  ok = ok && cudaStreamCreateWithFlags(&h->s_out, cudaStreamNonBlocking) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&h->start, cudaEventDisableTiming) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&h->finished, cudaEventDisableTiming) == cudaSuccess;
  for (int i = 0; ok && i < slots; ++i) {
    int8_t* a = nullptr;
    char* o = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr, e2 = nullptr;
    ok = cudaMalloc(&a, static_cast<size_t>(chunk_rows * K)) == cudaSuccess &&
         cudaMalloc(&o, static_cast<size_t>(chunk_rows * N * h->out_bytes)) == cudaSuccess &&
         cudaEventCreateWithFlags(&e0, cudaEventDisableTiming) == cudaSuccess &&
         cudaEventCreateWithFlags(&e1, cudaEventDisableTiming) == cudaSuccess &&
         cudaEventCreateWithFlags(&e2, cudaEventDisableTiming) == cudaSuccess;
    if (a) h->a.push_back(a);
    if (o) h->o.push_back(o);
    if (e0) h->in_done.push_back(e0);
    if (e1) h->mm_done.push_back(e1);
    if (e2) h->out_done.push_back(e2);
  }
  if (!ok) {
    g_last_error = std::string("host_linear_create: ") + cudaGetErrorString(cudaGetLastError());
    disc_b200_host_linear_destroy(h);
    return nullptr;
  }
  return h;
}

namespace {
// Row ranges of the chunks of a host-buffer linear.  The first copy in and the last copy out are not
// overlapped with anything, so long inputs start and end with quarter- and half-size chunks; in between
// full chunks, whose fixed cost per copy (some ten microseconds) is the smallest share.
std::vector<int64_t> host_linear_bounds(int64_t c, int64_t M) {
  std::vector<int64_t> bounds{0};
  const bool taper = M >= 4 * c && c >= 64;
  const int64_t head[3] = {c / 4, c / 4, c / 2};
  int64_t r = 0;
  if (taper)
    for (int64_t x : head) bounds.push_back(r += x);
  const int64_t tail_rows = taper ? c : 0;  // c / 2 + c / 4 + c / 4
  while (M - tail_rows - r > 0) bounds.push_back(r += std::min(c, M - tail_rows - r));
  if (taper)
    for (int i = 2; i >= 0; --i) bounds.push_back(r += head[i]);
  return bounds;
}
}  // namespace

int64_t disc_b200_host_linear_chunks(const disc_b200_host_linear* h, int64_t M) {
  if (!h || M <= 0) return 0;
  return static_cast<int64_t>(host_linear_bounds(h->chunk_rows, M).size()) - 1;
}

int32_t disc_b200_host_linear_run(disc_b200_host_linear* h, const disc_b200_qgemm_args* args, const int8_t* a_host,
                                  void* out_host, int64_t M, void* stream) {
  if (!h || !args || !a_host || !out_host || M < 0) {
    g_last_error = "host_linear_run: null argument";
    return 1;
  }
  if (args->K != h->K || args->N != h->N ||
      (args->out_dtype == DISC_B200_OUT_I8 ? 1 : 2) != h->out_bytes || args->a_slabs > 1) {
    g_last_error = "host_linear_run: the launch description does not match the pipeline (K, N, output type; no slabs)";
    return 1;
  }
  cudaStream_t cur = static_cast<cudaStream_t>(stream);
  cudaError_t st = cudaEventRecord(h->start, cur);
  for (cudaStream_t s : {h->s_in, h->s_mm, h->s_out}) {
    if (st == cudaSuccess) st = cudaStreamWaitEvent(s, h->start, 0);
  }
  const std::vector<int64_t> bounds = host_linear_bounds(h->chunk_rows, M);
  const int64_t chunks = static_cast<int64_t>(bounds.size()) - 1;
  const char* detail = nullptr;
  for (int64_t i = 0; st == cudaSuccess && i < chunks; ++i) {
    const int64_t r0 = bounds[i];
    const int64_t rows = bounds[i + 1] - r0;
    const int k = static_cast<int>(i % h->slots);
    // the slot's activation buffer is free once the product that read it is done
    if (i >= h->slots) st = cudaStreamWaitEvent(h->s_in, h->mm_done[k], 0);
    if (st == cudaSuccess)
      st = cudaMemcpyAsync(h->a[k], a_host + r0 * h->K, static_cast<size_t>(rows * h->K), cudaMemcpyHostToDevice, h->s_in);
    if (st == cudaSuccess) st = cudaEventRecord(h->in_done[k], h->s_in);
    if (st == cudaSuccess) st = cudaStreamWaitEvent(h->s_mm, h->in_done[k], 0);
    // and its result buffer once the copy that read it is done
    if (st == cudaSuccess && i >= h->slots) st = cudaStreamWaitEvent(h->s_mm, h->out_done[k], 0);
    if (st != cudaSuccess) break;
    disc_b200::QGemmParams p = to_params(args);
    p.a = h->a[k];
    p.out = h->o[k];
    p.M = rows;
    p.lda = h->K;
    p.ldo = h->N;
    st = disc_b200::qgemm_launch(p, h->s_mm, &detail);
    if (st == cudaSuccess) st = cudaEventRecord(h->mm_done[k], h->s_mm);
    if (st == cudaSuccess) st = cudaStreamWaitEvent(h->s_out, h->mm_done[k], 0);
    if (st == cudaSuccess)
      st = cudaMemcpyAsync(static_cast<char*>(out_host) + r0 * h->N * h->out_bytes, h->o[k],
                           static_cast<size_t>(rows * h->N * h->out_bytes), cudaMemcpyDeviceToHost, h->s_out);
    if (st == cudaSuccess) st = cudaEventRecord(h->out_done[k], h->s_out);
  }
  // the caller's stream continues when everything has left the pipeline
  for (cudaStream_t s : {h->s_in, h->s_mm, h->s_out}) {
    if (st == cudaSuccess) st = cudaEventRecord(h->finished, s);
    if (st == cudaSuccess) st = cudaStreamWaitEvent(cur, h->finished, 0);
  }
  return finish(st, "host_linear_run", detail);
}

int32_t disc_b200_qgemm_path(const disc_b200_qgemm_args* args) {
  if (!args) return -1;
  return disc_b200::qgemm_choose_path(to_params(args));
}

int32_t disc_b200_quantize(const void* x, int32_t in_type, int8_t* q, int64_t numel,
                           const float* scale, const int32_t* zero_point, int64_t channels,
                           int64_t inner, int32_t qmin, int32_t qmax, void* stream) {
  disc_b200::QuantizeParams p;
  p.x = x;
  p.q = q;
  p.numel = numel;
  p.in_type = in_type;
  p.scale = scale;
  p.zero_point = zero_point;
  p.channels = channels;
  p.inner = inner;
  p.qmin = qmin;
  p.qmax = qmax;
  const char* detail = nullptr;
  const cudaError_t st = disc_b200::quantize_launch(p, static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "quantize", detail);
}

int32_t disc_b200_dequantize(const int8_t* q, void* y, int32_t out_type, int64_t numel,
                             const float* scale, const int32_t* zero_point, int64_t channels,
                             int64_t inner, void* stream) {
  disc_b200::DequantizeParams p;
  p.q = q;
  p.y = y;
  p.numel = numel;
  p.out_type = out_type;
  p.scale = scale;
  p.zero_point = zero_point;
  p.channels = channels;
  p.inner = inner;
  const char* detail = nullptr;
  const cudaError_t st = disc_b200::dequantize_launch(p, static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "dequantize", detail);
}

int32_t disc_b200_dynamic_quantize(const void* x, int32_t in_type, int8_t* q, float* row_scale,
                                   int64_t rows, int64_t cols, void* stream) {
  disc_b200::DynQuantParams p;
  p.x = x;
  p.q = q;
  p.row_scale = row_scale;
  p.rows = rows;
  p.cols = cols;
  p.in_type = in_type;
  const char* detail = nullptr;
  const cudaError_t st = disc_b200::dynamic_quantize_launch(p, static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "dynamic_quantize", detail);
}

int32_t disc_b200_norm(const disc_b200_norm_args* a, void* stream) {
  if (!a) {
    g_last_error = "norm: null args";
    return 1;
  }
  disc_b200::NormParams p;
  p.x = a->x;
  p.residual = a->residual;
  p.gamma = a->gamma;
  p.beta = a->beta;
  p.y = a->y;
  p.sum_out = a->sum_out;
  p.q_out = a->q_out;
  p.q_scale = a->q_scale;
  p.q_row_scale = a->q_row_scale;
  p.rows = a->rows;
  p.cols = a->cols;
  p.eps = a->eps;
  p.type = a->type;
  p.rms = a->rms;
  p.x_slab_cols = a->x_slab_cols;
  p.x_slab_stride = a->x_slab_stride;
  const char* detail = nullptr;
  const cudaError_t st = disc_b200::norm_launch(p, static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "norm", detail);
}

int32_t disc_b200_softmax(const void* x, void* y, int32_t type, int64_t rows, int64_t cols,
                          int64_t rows_per_batch, const int32_t* lens, const void* mask,
                          float scale, int32_t log_softmax, void* stream) {
  disc_b200::SoftmaxParams p;
  p.x = x;
  p.y = y;
  p.rows = rows;
  p.cols = cols;
  p.rows_per_batch = rows_per_batch;
  p.lens = lens;
  p.mask = mask;
  p.scale = scale;
  p.type = type;
  p.log_softmax = log_softmax;
  const char* detail = nullptr;
  const cudaError_t st = disc_b200::softmax_launch(p, static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "softmax", detail);
}

int32_t disc_b200_observe_histogram(const void* x, int32_t type, int64_t n, float lo, float hi, int32_t bins,
                                    uint32_t* counts, void* stream) {
  disc_b200::HistogramParams p;
  p.x = x;
  p.type = type;
  p.n = n;
  p.lo = lo;
  p.hi = hi;
  p.bins = bins;
  p.counts = counts;
  const char* detail = nullptr;
  const cudaError_t st = disc_b200::histogram_observe_launch(p, static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "observe_histogram", detail);
}

int32_t disc_b200_attention(const disc_b200_attention_args* a, void* stream) {
  if (!a) {
    g_last_error = "attention: null args";
    return 1;
  }
  static_assert(sizeof(disc_b200::AttnBlock) == 4 * sizeof(int32_t), "block entries are four int32");
  disc_b200::AttentionParams p;
  p.qkv = a->qkv;
  p.tokens = a->tokens;
  p.ld_qkv = a->ld_qkv;
  p.heads = a->heads;
  p.blocks = reinterpret_cast<const disc_b200::AttnBlock*>(a->blocks);
  p.num_blocks = a->num_blocks;
  p.scale = a->scale;
  p.out = a->out;
  p.ld_out = a->ld_out;
  p.out_scale = a->out_scale;
  const char* detail = nullptr;
  const cudaError_t st = disc_b200::attention_launch(p, static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "attention", detail);
}

int32_t disc_b200_gated_quantize(const disc_b200_gated_quantize_args* a, void* stream) {
  if (!a) {
    g_last_error = "gated quantize: null args";
    return 1;
  }
  disc_b200::GatedQuantParams p;
  p.gate = a->gate;
  p.up = a->up;
  p.ld = a->ld;
  p.q = a->q;
  p.ldq = a->ldq;
  p.row_scale = a->row_scale;
  p.rows = a->rows;
  p.cols = a->cols;
  p.type = a->type;
  p.pass = a->pass;
  const char* detail = nullptr;
  const cudaError_t st = disc_b200::gated_quantize_launch(p, static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "gated_quantize", detail);
}

int32_t disc_b200_rope_kv_append(void* qkv, void* k_cache, void* v_cache, const float* cos_table,
                                 const float* sin_table, int64_t batch, int64_t seq, int64_t heads, int64_t dim,
                                 int64_t pos0, int64_t cache_len, void* stream) {
  disc_b200::RopeParams p;
  p.qkv = qkv;
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.cos = cos_table;
  p.sin = sin_table;
  p.batch = batch;
  p.seq = seq;
  p.heads = heads;
  p.dim = dim;
  p.pos0 = pos0;
  p.cache_len = cache_len;
  const char* detail = nullptr;
  const cudaError_t st = disc_b200::rope_kv_append_launch(p, static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "rope_kv_append", detail);
}

// ---- collectives of the column-parallel configuration
static int32_t nccl_fail(const char* what, int result) {
  const auto& api = disc_b200::ral::nccl_api();
  g_last_error = std::string(what) + ": " + (api.ok ? api.describe(result) : api.error);
  return 1;
}

int32_t disc_b200_nccl_available(void) {
  const auto& api = disc_b200::ral::nccl_api();
  if (!api.ok) g_last_error = "NCCL unavailable: " + api.error;
  return api.ok ? api.version : 0;
}

int32_t disc_b200_nccl_unique_id(void* id128) {
  const auto& api = disc_b200::ral::nccl_api();
  if (!api.ok || !id128) return nccl_fail("ncclGetUniqueId", 0);
  disc_b200::ral::NcclUniqueId id;
  const int st = api.GetUniqueId(&id);
  if (st != 0) return nccl_fail("ncclGetUniqueId", st);
  std::memcpy(id128, id.internal, sizeof(id.internal));
  return 0;
}

int32_t disc_b200_nccl_comm_create(const void* id128, int32_t nranks, int32_t rank, void** comm) {
  const auto& api = disc_b200::ral::nccl_api();
  if (!api.ok || !id128 || !comm || nranks <= 0 || rank < 0 || rank >= nranks) {
    return nccl_fail("ncclCommInitRank (arguments)", 0);
  }
  disc_b200::ral::NcclUniqueId id;
  std::memcpy(id.internal, id128, sizeof(id.internal));
  *comm = nullptr;
  const int st = api.CommInitRank(comm, nranks, id, rank);
  if (st != 0) return nccl_fail("ncclCommInitRank", st);
  return 0;
}

int32_t disc_b200_nccl_comm_destroy(void* comm) {
  const auto& api = disc_b200::ral::nccl_api();
  if (!api.ok || !comm) return 0;
  const int st = api.CommDestroy(comm);
  return st == 0 ? 0 : nccl_fail("ncclCommDestroy", st);
}

int32_t disc_b200_all_gather(void* comm, const void* send, void* recv, int64_t bytes_per_rank,
                             void* stream) {
  const auto& api = disc_b200::ral::nccl_api();
  if (!api.ok || !comm) return nccl_fail("ncclAllGather (no communicator)", 0);
  if (bytes_per_rank <= 0) return 0;
  const int st = api.AllGather(send, recv, static_cast<size_t>(bytes_per_rank), disc_b200::ral::kNcclInt8,
                               comm, static_cast<cudaStream_t>(stream));
  return st == 0 ? 0 : nccl_fail("ncclAllGather", st);
}

int32_t disc_b200_all_gather_rows(void* comm, void* buf, int32_t nranks, int64_t slot_bytes,
                                  int64_t offset_bytes, int64_t bytes, void* stream) {
  const auto& api = disc_b200::ral::nccl_api();
  if (!api.ok || !comm) return nccl_fail("ncclBroadcast (no communicator)", 0);
  if (bytes <= 0 || nranks <= 1) return 0;
  if (!buf || offset_bytes < 0 || offset_bytes + bytes > slot_bytes) return nccl_fail("all_gather_rows (range)", 0);
  // one broadcast per slot, root = the slot's rank, grouped so that they run as one operation
  int st = api.GroupStart();
  for (int r = 0; r < nranks && st == 0; ++r) {
    char* p = static_cast<char*>(buf) + static_cast<int64_t>(r) * slot_bytes + offset_bytes;
    st = api.Broadcast(p, p, static_cast<size_t>(bytes), disc_b200::ral::kNcclInt8, r, comm,
                       static_cast<cudaStream_t>(stream));
  }
  const int end = api.GroupEnd();
  if (st == 0) st = end;
  return st == 0 ? 0 : nccl_fail("ncclBroadcast (grouped gather of a row range)", st);
}

int32_t disc_b200_all_reduce_f32(void* comm, const float* send, float* recv, int64_t count,
                                 int32_t op, void* stream) {
  const auto& api = disc_b200::ral::nccl_api();
  if (!api.ok || !comm) return nccl_fail("ncclAllReduce (no communicator)", 0);
  if (count <= 0) return 0;
  if (op < 0 || op > 3) return nccl_fail("ncclAllReduce (op)", 0);
  const int st = api.AllReduce(send, recv, static_cast<size_t>(count), disc_b200::ral::kNcclFloat32, op,
                               comm, static_cast<cudaStream_t>(stream));
  return st == 0 ? 0 : nccl_fail("ncclAllReduce", st);
}

struct disc_b200_executable {
  void* lib = nullptr;
  void (*entry)(void**) = nullptr;
  disc_b200_context* ctx = nullptr;
};

disc_b200_executable* disc_b200_executable_open(const char* so_path, const char* metadata_path,
                                                const disc_b200_context_options* opts) {
  if (!so_path) {
    g_last_error = "executable_open: null path";
    return nullptr;
  }
  void* lib = dlopen(so_path, RTLD_NOW | RTLD_LOCAL);
  if (!lib) {
    const char* why = dlerror();
    g_last_error = std::string("executable_open: ") + (why ? why : so_path);
    return nullptr;
  }
  void* entry = dlsym(lib, kMlirLoweredEntry);
  if (!entry) {
    g_last_error = std::string("executable_open: no entry point \"") + kMlirLoweredEntry + "\" in " + so_path;
    dlclose(lib);
    return nullptr;
  }
  disc_b200_context* ctx = disc_b200_context_create(opts);
  if (metadata_path && disc_b200_context_load_metadata(ctx, metadata_path) != 0) {
    disc_b200_context_destroy(ctx);
    dlclose(lib);
    return nullptr;
  }
  auto* exe = new disc_b200_executable;
  exe->lib = lib;
  exe->entry = reinterpret_cast<void (*)(void**)>(entry);
  exe->ctx = ctx;
  return exe;
}

disc_b200_context* disc_b200_executable_context(disc_b200_executable* exe) { return exe ? exe->ctx : nullptr; }

disc_b200_exec* disc_b200_executable_run(disc_b200_executable* exe, int32_t n_inputs,
                                         const disc_b200_buffer_ref* inputs) {
  if (!exe || n_inputs < 0 || (n_inputs > 0 && !inputs)) {
    g_last_error = "executable_run: null argument";
    return nullptr;
  }
  disc_b200_exec* exec = disc_b200_exec_create(exe->ctx);
  for (int32_t i = 0; i < n_inputs; ++i) {
    if (disc_b200_exec_bind_input(exec, i, inputs[i].data, inputs[i].rank, inputs[i].sizes) != 0) {
      g_last_error = "executable_run: bad input " + std::to_string(i);
      disc_b200_exec_destroy(exec);
      return nullptr;
    }
  }
  // what the generated disc_ral_call stub expects: { execution context, dispatcher }
  void* ctx_struct[2] = {exec, reinterpret_cast<void*>(&tao_ral_call_impl)};
  exe->entry(ctx_struct);
  const char* msg = nullptr;
  if (tao_ral_last_error(exe->ctx, &msg) != 0) {
    g_last_error = msg ? msg : "executable_run: a custom call failed";
    disc_b200_exec_destroy(exec);
    return nullptr;
  }
  return exec;
}

void disc_b200_executable_close(disc_b200_executable* exe) {
  if (!exe) return;
  disc_b200_context_destroy(exe->ctx);
  dlclose(exe->lib);
  delete exe;
}

int32_t disc_b200_context_load_metadata(disc_b200_context* handle, const char* path) {
  auto* ctx = reinterpret_cast<disc_b200::ral::Context*>(handle);
  if (!ctx || !path) {
    g_last_error = "load_metadata: null context or path";
    return 1;
  }
  // the reference's switch for the process-level store (common_context_impl.cc:57-64)
  const char* env = std::getenv("DISC_USE_GLOBAL_CONST_STORE");
  std::string flag = env ? env : "";
  for (char& c : flag) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
  if (flag == "true" || flag == "1") return disc_b200_context_share_metadata(handle, path);
  std::string why;
  auto file = disc_b200::ral::MetadataFile::load(path, &why);
  if (!file) {
    g_last_error = why;
    return 1;
  }
  auto store = std::make_shared<disc_b200::ral::ConstStore>();
  store->metadata = std::move(file);
  std::lock_guard<std::mutex> l(ctx->mu);
  ctx->consts = std::move(store);
  return 0;
}

int32_t disc_b200_context_share_metadata(disc_b200_context* handle, const char* path) {
  auto* ctx = reinterpret_cast<disc_b200::ral::Context*>(handle);
  if (!ctx || !path) {
    g_last_error = "share_metadata: null context or path";
    return 1;
  }
  std::string why;
  auto store = disc_b200::ral::shared_const_store(path, ctx->device, &why);
  if (!store) {
    g_last_error = why;
    return 1;
  }
  std::lock_guard<std::mutex> l(ctx->mu);
  ctx->consts = std::move(store);
  return 0;
}

int32_t disc_b200_metadata_write(const char* path, int32_t n, const char* const* names, const int32_t* is_host,
                                 const void* const* data, const int64_t* bytes) {
  if (!path || n < 0 || (n > 0 && (!names || !is_host || !data || !bytes))) {
    g_last_error = "metadata_write: null argument";
    return 1;
  }
  disc_b200::ral::MetadataWriter w(path);
  if (!w.ok()) {
    g_last_error = std::string("metadata_write: cannot create ") + path;
    return 1;
  }
  for (int32_t i = 0; i < n; ++i) {
    if (!names[i] || bytes[i] < 0 || !w.add(names[i], is_host[i] != 0, data[i], static_cast<size_t>(bytes[i]))) {
      g_last_error = std::string("metadata_write: duplicated key or write error at ") + (names[i] ? names[i] : "?");
      return 1;
    }
  }
  if (!w.finish()) {
    g_last_error = "metadata_write: write error";
    return 1;
  }
  return 0;
}

int32_t disc_b200_const_name_info(const char* unique_name, int32_t* rank, int64_t* sizes8, int64_t* elem_bytes) {
  std::vector<int64_t> shape;
  int64_t width = 0;
  if (!unique_name || !disc_b200::ral::parse_const_name(unique_name, &shape, &width) || shape.size() > 8) return 1;
  if (rank) *rank = static_cast<int32_t>(shape.size());
  if (sizes8) {
    for (size_t i = 0; i < shape.size(); ++i) sizes8[i] = shape[i];
  }
  if (elem_bytes) *elem_bytes = width;
  return 0;
}

int32_t disc_b200_weight_only_qgemm_plan(int64_t m, int64_t n, int64_t k, int32_t align, int32_t sm_count,
                                         int64_t* out7) {
  if (!out7) return 1;
  return disc_b200::woq_gemm_plan_describe(m, n, k, align, sm_count, out7);
}

int32_t disc_b200_weight_only_qgemm(const disc_b200_weight_only_qgemm_args* a, void* stream) {
  if (!a) {
    g_last_error = "weight-only qgemm: null args";
    return 1;
  }
  disc_b200::WoqGemmParams p;
  p.x = a->x;
  p.w = a->w;
  p.scale = a->scale;
  p.zp = a->zero_point;
  p.bias = a->bias;
  p.out = a->out;
  p.M = a->m;
  p.N = a->n;
  p.K = a->k;
  p.ldx = a->ldx;
  p.ldw = a->ldw;
  p.ldo = a->ldo;
  p.type = a->type;
  p.path = a->path;
  const char* detail = nullptr;
  const cudaError_t st = disc_b200::woq_gemm_launch(p, static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "weight_only_qgemm", detail);
}

namespace {
// geometry of a direct call; fills g or returns the reason it cannot
std::string geometry_of(const disc_b200_qconv2d_args* a, disc_b200::ConvGeometry* g) {
  return disc_b200::ral::conv2d_geometry(a->input_sizes, a->kernel_sizes, a->output_sizes, a->padding, a->metadata, 16,
                                         g);
}
}  // namespace

int32_t disc_b200_qconv2d_plan(const char* data_format, const int64_t* strides, int32_t n_strides,
                               const int64_t* dilations, int32_t n_dilations, const char* padding,
                               const int64_t* explicit_paddings, int32_t n_explicit, int32_t weight_is_const,
                               const int64_t* input_sizes4, const int64_t* weight_sizes4, int32_t* padding_out4,
                               int64_t* result_sizes4, int32_t* metadata_out17) {
  if (!data_format || !padding || !input_sizes4 || !weight_sizes4 || !padding_out4 || !result_sizes4 ||
      !metadata_out17 || n_strides < 0 || n_dilations < 0 || n_explicit < 0 || (n_strides > 0 && !strides) ||
      (n_dilations > 0 && !dilations) || (n_explicit > 0 && !explicit_paddings)) {
    g_last_error = "qconv2d_plan: null argument";
    return 1;
  }
  const std::string why = disc_b200::ral::plan_conv2d_from_attrs(
      data_format, std::vector<int64_t>(strides, strides + n_strides),
      std::vector<int64_t>(dilations, dilations + n_dilations), padding,
      std::vector<int64_t>(explicit_paddings, explicit_paddings + n_explicit), weight_is_const != 0, input_sizes4,
      weight_sizes4, padding_out4, result_sizes4, metadata_out17);
  if (!why.empty()) {
    g_last_error = why;
    return 1;
  }
  return 0;
}

int64_t disc_b200_qconv2d_workspace_bytes(const disc_b200_qconv2d_args* a) {
  disc_b200::ConvGeometry g;
  if (!a || !geometry_of(a, &g).empty()) return -1;
  return disc_b200::qconv_workspace_bytes(g);
}

int32_t disc_b200_qconv2d(const disc_b200_qconv2d_args* a, void* stream) {
  if (!a) {
    g_last_error = "qconv2d: null args";
    return 1;
  }
  disc_b200::QConvParams p;
  const std::string why = geometry_of(a, &p.g);
  if (!why.empty()) {
    g_last_error = "qconv2d: " + why;
    return 1;
  }
  p.x = a->x;
  p.w = a->w;
  p.out = a->out;
  p.x_scale = a->x_scale;
  p.w_scale = a->w_scale;
  p.w_scale_per_channel = a->w_scale_per_channel;
  p.out_scale = a->out_scale;
  p.workspace = a->workspace;
  p.workspace_bytes = a->workspace_bytes;
  p.splitk_ws = static_cast<int32_t*>(a->splitk_ws);
  p.splitk_ws_bytes = a->splitk_ws_bytes;
  const char* detail = nullptr;
  const cudaError_t st = disc_b200::qconv_launch(p, static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "qconv2d", detail);
}

int64_t disc_b200_observe_minmax_scratch_floats(int64_t outer, int64_t channels, int64_t inner) {
  return disc_b200::minmax_scratch_floats(outer, channels, inner);
}

int32_t disc_b200_observe_minmax(const void* x, int32_t type, int64_t outer, int64_t channels, int64_t inner,
                                 float* min_val, float* max_val, float* scratch, int64_t scratch_floats,
                                 void* stream) {
  disc_b200::MinMaxParams p;
  p.x = x;
  p.type = type;
  p.outer = outer;
  p.channels = channels;
  p.inner = inner;
  p.min_val = min_val;
  p.max_val = max_val;
  p.scratch = scratch;
  p.scratch_floats = scratch_floats;
  const char* detail = nullptr;
  const cudaError_t st = disc_b200::minmax_observe_launch(p, static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "observe_minmax", detail);
}

int32_t disc_b200_minmax_qparams(const float* min_val, const float* max_val, int64_t n, int32_t qmin, int32_t qmax,
                                 int32_t symmetric, int32_t symmetric_zero_point, float* scale, int32_t* zero_point,
                                 void* stream) {
  disc_b200::QParamsParams p;
  p.min_val = min_val;
  p.max_val = max_val;
  p.n = n;
  p.qmin = qmin;
  p.qmax = qmax;
  p.symmetric = symmetric;
  p.symmetric_zero_point = symmetric_zero_point;
  p.scale = scale;
  p.zero_point = zero_point;
  const char* detail = nullptr;
  const cudaError_t st = disc_b200::minmax_qparams_launch(p, static_cast<cudaStream_t>(stream), &detail);
  return finish(st, "minmax_qparams", detail);
}

int32_t disc_b200_select_device_image(int64_t num_images, int32_t cc_major, int32_t cc_minor) {
  return num_images < 0 ? -1 : disc_b200::ral::select_blob(static_cast<size_t>(num_images), cc_major, cc_minor);
}

const char* disc_b200_last_error_string(void) { return g_last_error.c_str(); }

int32_t disc_b200_selftest_wait_expiry(uint64_t limit_ns, int64_t* waited_ns, void* stream) {
  const char* detail = nullptr;
  long long waited = 0;
  const cudaError_t st = disc_b200::wait_expiry_selftest(limit_ns, waited_ns ? &waited : nullptr,
                                                         static_cast<cudaStream_t>(stream), &detail);
  if (waited_ns) *waited_ns = waited;
  return finish(st, "selftest_wait_expiry", detail);
}

int32_t disc_b200_kernel_status(void) { return disc_b200::kernel_status_fetch_and_clear(); }

const char* disc_b200_version(void) { return "disc-b200-ral 0.1 (sm_100a)"; }

int32_t disc_b200_attrs_describe(const void* blob, char* out, int32_t capacity) {
  return disc_b200_attrs_describe_bounded(blob, int64_t{1} << 30, out, capacity);
}

int32_t disc_b200_attrs_describe_bounded(const void* blob, int64_t blob_bytes, char* out, int32_t capacity) {
  if (!blob || !out || capacity <= 0 || blob_bytes < 0) return -1;
  const uint8_t* cur = static_cast<const uint8_t*>(blob);
  auto a = disc_b200::ral::parse_attr(&cur, blob_bytes);
  if (!a) return -1;
  std::string text;
  render(*a, text);
  const int32_t n = static_cast<int32_t>(text.size()) < capacity - 1 ? static_cast<int32_t>(text.size()) : capacity - 1;
  std::memcpy(out, text.data(), n);
  out[n] = 0;
  return n;
}

}  // extern "C"
