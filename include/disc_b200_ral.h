/* C ABI of libdisc_b200_ral.so: a B200 (sm_100a) implementation of the
 * quantized-inference custom calls of BladeDISC's RAL (runtime abstraction
 * layer).  Plain C types only.  All device pointers refer to the CUDA device
 * that is current on the calling thread; work is enqueued on the given
 * stream and the calls do not synchronise unless they say so.
 *
 * Citations name files of the reference project (alibaba/BladeDISC).
 */
#ifndef DISC_B200_RAL_H_
#define DISC_B200_RAL_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------
 * 1. The RAL dispatcher.  A DISC-compiled executable receives
 *    ctx_struct = { execution context, pointer to this function } and calls
 *    every runtime service through it with a mangled name
 *    "<api>___<device>___<arg types>___<ret type>" and type-erased arguments.
 *    Replaces tao_compiler/mlir/ral/ral_api.h:59-67 (declared there without
 *    these exact parameter names; the symbols and meaning are the same).
 * ---------------------------------------------------------------------- */

/* Entry symbol of a compiled executable (tao_compiler/mlir/ral/ral_api.cc:29). */
extern const char* const kMlirLoweredEntry;

typedef void* tao_ral_context_t;
typedef int32_t tao_ral_status_t;

/* `ctx` is an execution context made by disc_b200_exec_create.  `name` is a
 * NUL-terminated mangled api name, `args[i]` points at the i-th flattened
 * argument; a rank-N memref occupies 3 + 2N slots (base pointer, aligned
 * pointer, offset, sizes, strides); the slot after the last argument points at
 * storage for the returned value (tao_compiler/mlir/ral/ral_helper.h:160-236).
 * Unknown names and kernel failures put the context into an error state that
 * tao_ral_last_error reports; nothing aborts and nothing throws. */
void tao_ral_call_impl(tao_ral_context_t ctx, void* name, void** args);

/* 0 when healthy.  Accepts a context or an execution context handle.  The
 * message pointer stays valid until the error is cleared. */
tao_ral_status_t tao_ral_last_error(tao_ral_context_t ctx, const char** err_msg);
void tao_ral_clear_error(tao_ral_context_t ctx);

/* ------------------------------------------------------------------------
 * 2. Contexts.  What torch_blade's RalContext builds with
 *    MakeBaseCudaContext / MakeExecutionContext
 *    (pytorch_blade/pytorch_blade/compiler/mlir/runtime/ral_context.cpp:243-321,
 *    tao_compiler/mlir/ral/context/base/cuda/cuda_context_impl.h:50-58).
 *    One context per (device, stream); one execution context per inference.
 * ---------------------------------------------------------------------- */

typedef void* (*disc_b200_alloc_fn)(void* user, size_t bytes);
typedef void (*disc_b200_free_fn)(void* user, void* ptr);

typedef struct disc_b200_context_options {
  int32_t device;        /* CUDA device ordinal */
  void* stream;          /* cudaStream_t all work of this context runs on */
  disc_b200_alloc_fn gpu_alloc; /* device allocator; NULL = cudaMalloc / cudaFree */
  disc_b200_free_fn gpu_free;
  void* alloc_user;
  void* nccl_comm;       /* ncclComm_t for ral_all_gather; NULL = collectives unavailable */
  void* comm_stream;     /* cudaStream_t for asynchronous collectives; NULL = `stream` */
} disc_b200_context_options;

typedef struct disc_b200_context disc_b200_context;
typedef struct disc_b200_exec disc_b200_exec;

disc_b200_context* disc_b200_context_create(const disc_b200_context_options* opts);
void disc_b200_context_destroy(disc_b200_context* ctx);

disc_b200_exec* disc_b200_exec_create(disc_b200_context* ctx);
/* Frees buffers of this execution that were neither deallocated nor handed
 * out as outputs. */
void disc_b200_exec_destroy(disc_b200_exec* exec);

/* Input idx of the executable: a borrowed buffer and its shape
 * (ExecutionContext::bindInput, tao_compiler/mlir/ral/ral_context.h:164-170). */
int32_t disc_b200_exec_bind_input(disc_b200_exec* exec, int32_t idx, const void* data, int32_t rank,
                                  const int64_t* sizes);
/* Output idx after the executable ran.  *owned = 1 when the buffer is a device
 * buffer allocated by this execution and now the caller's to free with
 * disc_b200_exec_free_output, 2 when it is a host buffer of this execution
 * (disc_b200_exec_free_host_output), 0 when it aliases an input, a constant or
 * an earlier output (ExecutionContext::bindOutput). */
int32_t disc_b200_exec_get_output(disc_b200_exec* exec, int32_t idx, void** data, int32_t* rank,
                                  int64_t* sizes8, int32_t* owned);
void disc_b200_exec_free_output(disc_b200_context* ctx, void* data);
void disc_b200_exec_free_host_output(void* data);

/* ---- A compiled executable: the shared object DISC emits plus its metadata
 * file.  Replaces RalContext's constructor, LoadEngine and Execute
 * (pytorch_blade/pytorch_blade/compiler/mlir/runtime/ral_context.cpp:104-166,
 * 293-321): dlopen, entry point "main" (kMlirLoweredEntry), one context, and per
 * run an execution context whose address travels to the entry together with
 * this library's dispatcher (tao_compiler/mlir/disc/disc_compiler.cc:95-131). */
typedef struct disc_b200_executable disc_b200_executable;
typedef struct disc_b200_buffer_ref {
  const void* data;
  int32_t rank;
  const int64_t* sizes;
} disc_b200_buffer_ref;

/* NULL on failure (disc_b200_last_error_string says why).  metadata_path may be
 * NULL for an executable without constants. */
disc_b200_executable* disc_b200_executable_open(const char* so_path, const char* metadata_path,
                                                const disc_b200_context_options* opts);
disc_b200_context* disc_b200_executable_context(disc_b200_executable* exe);
/* One inference: binds the inputs, calls the entry.  Returns the execution
 * context to read the outputs from (disc_b200_exec_get_output; the caller
 * destroys it) or NULL when a custom call failed; the error then stays on the
 * context until tao_ral_clear_error. */
disc_b200_exec* disc_b200_executable_run(disc_b200_executable* exe, int32_t n_inputs,
                                         const disc_b200_buffer_ref* inputs);
void disc_b200_executable_close(disc_b200_executable* exe);

/* Registry inspection (the reference keeps its registry private:
 * tao_compiler/mlir/ral/ral_helper.h:254-269). */
int32_t disc_b200_registry_size(void);
const char* disc_b200_registry_name(int32_t i);
int32_t disc_b200_registry_has(const char* mangled_name);

/* ------------------------------------------------------------------------
 * 3. Kernels by direct call.  The custom calls above unpack their memrefs and
 *    land here; a host that is not a DISC executable can call these itself.
 *    Every function returns 0 on success or a non-zero code with a message
 *    available from disc_b200_last_error_string (thread local).
 * ---------------------------------------------------------------------- */

enum { DISC_B200_OUT_I8 = 0, DISC_B200_OUT_F16 = 1, DISC_B200_OUT_F32 = 2, DISC_B200_OUT_I32 = 3 };
enum { DISC_B200_ACT_NONE = 0, DISC_B200_ACT_GELU = 1, DISC_B200_ACT_SILU = 2 };
enum { DISC_B200_BIAS_NONE = 0, DISC_B200_BIAS_F32 = 1, DISC_B200_BIAS_I8 = 2 };
enum { DISC_B200_SCALE_NONE = 0, DISC_B200_SCALE_SCALAR = 1, DISC_B200_SCALE_PER_COL = 2,
       DISC_B200_SCALE_PER_ROW = 3 };
enum { DISC_B200_PATH_AUTO = 0, DISC_B200_PATH_TILED = 1, DISC_B200_PATH_SMALL_M = 2,
       DISC_B200_PATH_SIMT = 3, DISC_B200_PATH_PAIR = 4, DISC_B200_PATH_GEMV = 5,
       DISC_B200_PATH_SKINNY = 6 };
enum { DISC_B200_F32 = 0, DISC_B200_F16 = 1 };

/* out[m, n] = epilogue(sum_k a[m, k] * w[n, k]); a int8 [M, K], w int8 [N, K],
 * both row-major.  All scale / bias pointers are DEVICE pointers: nothing is
 * copied to the host, unlike the reference which reads the three scales back
 * on first use (tao_compiler/mlir/ral/context/quantized_gpu_kernel_impl.cc:356-386).
 *
 *   t  = float(acc) [* x_scale[m] if x_scale_kind == PER_ROW]
 *   cs = x_scale(n) * w_scale(n)                 [x_scale left out if PER_ROW]
 *   cs = cs / out_scale(n)                       if fold_out_scale
 *   v  = fma(t, cs, bias[n]);  v = act(v)
 *   v  = v / out_scale                           if div_out_scale (see div_exact)
 *   out = sat_s8(rne(v)) | f16(v) | f32(v) ; OUT_I32 stores acc itself.
 *
 * The reference's ral_pdll_qgemm (quantized_gpu_kernel_impl.cc:328-422) is
 * { fold_out_scale = 1, act = NONE, out = I8, bias F32 or I8 }.
 * splitk_ws: device scratch of at least disc_b200_qgemm_scratch_bytes(M, N, K)
 * bytes, needed when M <= 128 takes the small-M path; its first 16 KiB (the
 * arrival counters of the split-K reduction) must be zero before the first use
 * and are left zero; launches that share it must not overlap on the GPU. */
typedef struct disc_b200_qgemm_args {
  const int8_t* a;
  const int8_t* w;
  void* out;
  int64_t M, N, K;
  int64_t lda, ldw, ldo;
  const float* x_scale;
  const float* w_scale;
  const float* out_scale;
  const void* bias;
  int32_t x_scale_kind, w_scale_kind, out_scale_kind, bias_kind;
  int32_t fold_out_scale, div_out_scale;
  int32_t act, out_dtype;
  int32_t path, split_k;
  void* splitk_ws;
  int64_t splitk_ws_bytes;
  /* Activation stored as a_slabs column slabs (what an all-gather of
   * column-parallel outputs leaves, see disc_b200_qgemm_all_gather): element
   * (m, k) is a[(k / a_slab_cols) * a_slab_stride + m * lda + k % a_slab_cols],
   * K = a_slabs * a_slab_cols.  0 or 1 = plain row-major. */
  int32_t a_slabs;
  int64_t a_slab_cols;
  int64_t a_slab_stride;
  /* Non-zero: `w` was final before the previous kernel on the stream was
   * launched (inference weights).  The few-row paths then fetch it while that
   * kernel still runs and wait for it only before touching anything else
   * (the reference's ral_qgemm carries the same promise as weight_is_const,
   * stream_executor_based_impl.cc:427-433). */
  int32_t weights_static;
  /* With div_out_scale.  0: v * (1 / out_scale) with the correctly rounded
   * reciprocal (folded into the column scale and bias when there is no
   * activation): the int8 result equals the divide-based one except for values
   * within a few ulp of a rounding tie, where it may land on the neighbouring
   * level (at most 1 LSB, the tolerance of requantized outputs; out_scale and
   * its reciprocal must be normal floats, 2^-126 <= |out_scale| <= 2^126).  Non-zero: the
   * correctly rounded IEEE quotient, bit for bit the divide-based quantize of
   * disc_lower_quantize_and_dequantize.cc:77-93, at about twice the epilogue
   * arithmetic. */
  int32_t div_exact;
} disc_b200_qgemm_args;

int32_t disc_b200_qgemm(const disc_b200_qgemm_args* args, void* stream);
int64_t disc_b200_qgemm_scratch_bytes(int64_t M, int64_t N, int64_t K);
/* Path (DISC_B200_PATH_*) the launch would take. */
int32_t disc_b200_qgemm_path(const disc_b200_qgemm_args* args);

/* The quantized linear on HOST buffers, for a serving process whose activations arrive in host memory: the
 * rows are streamed host -> device, multiplied and the result streamed back in chunks of `chunk_rows` over three
 * streams of the pipeline, so that both copy directions and the tensor-core work overlap (pin the host buffers,
 * or the copies serialise).  The weight, scales and bias of `args` stay resident on the device, as the constants
 * of a compiled graph do (tao_compiler/mlir/ral/context/common_context_impl_cuda.cc:61-132); `args->a`, `out`, `M`,
 * `lda`, `ldo` are ignored in favour of the host buffers.  create allocates the staging buffers (slots x
 * chunk_rows x (K + N * element size) bytes on the current device); run orders itself after `stream` and makes
 * `stream` wait for its completion; it does not synchronise the host. */
typedef struct disc_b200_host_linear disc_b200_host_linear;
disc_b200_host_linear* disc_b200_host_linear_create(int64_t chunk_rows, int64_t K, int64_t N, int32_t out_dtype,
                                                    int32_t slots);
int32_t disc_b200_host_linear_run(disc_b200_host_linear* h, const disc_b200_qgemm_args* args, const int8_t* a_host,
                                  void* out_host, int64_t M, void* stream);
/* Chunks (= kernel launches) a call with M rows is cut into.  Host only. */
int64_t disc_b200_host_linear_chunks(const disc_b200_host_linear* h, int64_t M);
void disc_b200_host_linear_destroy(disc_b200_host_linear* h);

/* The small-M path (M <= 128) of disc_b200_qgemm for callers that cannot
 * allocate device memory at the point of the call and so have no scratch to
 * pass: code that runs while a stream is being captured, servers that gave
 * the whole device heap to their own pool, threads on which a cudaMalloc
 * would stall the rest of the process.  This entry point has no counterpart
 * in the reference.  It allocates nothing (no cudaMalloc / cudaFree, no
 * allocating library routine): the split-K scratch is an 8 MiB array built
 * into the library, resident on every GPU that loads it until the process
 * exits.  `splitk_ws` / `splitk_ws_bytes` / `path` of `args` are ignored; the
 * caller still provides inputs and outputs.
 *   - Limits: M <= 128, K and row strides multiples of 16 with 16-byte aligned
 *     bases (the TMA rules), and split * M * round_up(N, 128) * 4 + 16 KiB must
 *     fit the array (disc_b200_qgemm_small_m_noalloc_capacity() bytes); the
 *     activation must be plain row-major (a_slabs <= 1), every row stride at
 *     least its row, and a per-channel out_scale only in folded form;
 *     anything else is refused with a message, never silently redirected.
 *   - The first call on each device looks up the array's device address; make
 *     that first call before starting any stream capture.
 *   - All calls on a device share the one array, which keeps what the previous
 *     call left; the part that must start at zero is cleared on the stream by
 *     every call.  Two calls that overlap on the GPU (different streams, no
 *     ordering between them) race on it: order them. */
int32_t disc_b200_qgemm_small_m_noalloc(const disc_b200_qgemm_args* args, void* stream);
int64_t disc_b200_qgemm_small_m_noalloc_capacity(void);

/* q = clamp(rne(x / scale + zero_point), qmin, qmax): the arithmetic of
 * QuantizeOpConverter with RoundHalfToEven
 * (tao_compiler/mlir/disc/transforms/disc_lower_quantize_and_dequantize.cc:36-97).
 * channels == 1: per-tensor; otherwise the tensor is viewed as
 * [outer, channels, inner] and scale / zero_point have `channels` entries.
 * zero_point may be NULL. */
int32_t disc_b200_quantize(const void* x, int32_t in_type, int8_t* q, int64_t numel,
                           const float* scale, const int32_t* zero_point, int64_t channels,
                           int64_t inner, int32_t qmin, int32_t qmax, void* stream);

/* y = float(q - zero_point) * scale: DequantizeOpConverter
 * (disc_lower_quantize_and_dequantize.cc:99-139). */
int32_t disc_b200_dequantize(const int8_t* q, void* y, int32_t out_type, int64_t numel,
                             const float* scale, const int32_t* zero_point, int64_t channels,
                             int64_t inner, void* stream);

/* Per-row symmetric quantize, row_scale[r] = max(max|x[r, :]| / 127, FLT_EPSILON).
 * No counterpart in the reference, whose quantize op rejects use_dynamic
 * (disc_lower_quantize_and_dequantize.cc:41-43). */
int32_t disc_b200_dynamic_quantize(const void* x, int32_t in_type, int8_t* q, float* row_scale,
                                   int64_t rows, int64_t cols, void* stream);

/* LayerNorm / RMSNorm over the last axis with optional fused residual add and
 * optional int8 second output; stands in for the kStitch fusion DISC generates
 * for aten.layer_norm (tao_compiler/mlir/disc/transforms/
 * lhlo_legalize_roots_to_loops.cc:3091-3330).  Pointers may be NULL where the
 * comment of the field in rowops.h says so: residual, beta, y, sum_out, q_out,
 * q_scale, q_row_scale. */
typedef struct disc_b200_norm_args {
  const void* x;
  const void* residual;
  const void* gamma;
  const void* beta;
  void* y;
  void* sum_out;
  int8_t* q_out;
  const float* q_scale;
  float* q_row_scale;
  int64_t rows, cols;
  float eps;
  int32_t type;
  int32_t rms;
  /* x stored as column slabs (the buffer disc_b200_qgemm_all_gather returns):
   * element (r, c) at x[(c / x_slab_cols) * x_slab_stride + r * x_slab_cols +
   * c % x_slab_cols]; 0 = plain row-major. */
  int64_t x_slab_cols;
  int64_t x_slab_stride;
} disc_b200_norm_args;
int32_t disc_b200_norm(const disc_b200_norm_args* args, void* stream);

/* Per-row symmetric int8 quantization of h = up ? silu(gate) * up : gate in
 * two passes, for rows whose columns are spread over the GPUs of a
 * column-parallel split: pass 0 writes row_scale[r] = max(max|h[r, :]| / 127,
 * FLT_EPSILON) over the local columns; the caller takes the maximum over the
 * ranks (disc_b200_all_reduce_f32, op 2); pass 1 writes
 * q = sat(rne(h / row_scale[r])); pass 2 does both at once for rows that are
 * whole on this GPU.  gate / up have row stride ld, q row stride
 * ldq (elements).  No counterpart in the reference (dynamic quantization is
 * rejected there, disc_lower_quantize_and_dequantize.cc:41-43). */
typedef struct disc_b200_gated_quantize_args {
  const void* gate;
  const void* up; /* may be NULL */
  int64_t ld;
  int8_t* q; /* pass 1 */
  int64_t ldq;
  float* row_scale;
  int64_t rows, cols;
  int32_t type;
  int32_t pass;
} disc_b200_gated_quantize_args;
int32_t disc_b200_gated_quantize(const disc_b200_gated_quantize_args* args, void* stream);

/* Rotary position embedding of q and k inside a fused QKV output
 * fp16 [batch * seq, 3, heads, dim] (q in place) and the append of the rotated
 * k and of v to the caches fp16 [batch, heads, cache_len, dim] at positions
 * pos0 .. pos0 + seq - 1; cos / sin are fp32 [>= pos0 + seq, dim / 2]; pairs
 * (i, i + dim / 2).  Decoder glue around the quantized linears of the 7B-shaped
 * configuration; the reference compiles this as generated elementwise kernels. */
int32_t disc_b200_rope_kv_append(void* qkv, void* k_cache, void* v_cache, const float* cos_table,
                                 const float* sin_table, int64_t batch, int64_t seq, int64_t heads, int64_t dim,
                                 int64_t pos0, int64_t cache_len, void* stream);

/* Weight-only quantized linear: out[m, n] = sum_k x[m, k] * (w[k, n] - zp[n]) * scale[n]
 * + bias[n]; x / scale / bias / out all f32 or all f16 (`type`), w uint8 [K, N]
 * row-major exactly as the pattern of the reference leaves it (weight_only_qgemm.pdll:2-106;
 * custom call ral_pdll_weight_only_qgemm, for which the reference has no open kernel),
 * zero_point int32 [N] or NULL.  Sums are fp32.  Two kernels: a streaming one (any
 * type and alignment; up to 16 rows stream the weights once, more rows re-read them per
 * group of 16) and, for f16 with 4 rows and more, one on the tensor cores (weights
 * dequantized to fp16 on the way into shared memory, up to 256 rows per pass over the
 * weights; needs n a multiple of 16, w and x 16-byte aligned with ldw a multiple of 16
 * and ldx of 8, zero points within [-1024, 1024]).  `path`: 0 = chosen by shape,
 * 1 = streaming, 2 = tensor cores (refused with a message when the operands do not
 * qualify).  No scratch memory.  w holds constants of the model: the kernel may read it
 * before the preceding kernel on the stream has finished. */
typedef struct disc_b200_weight_only_qgemm_args {
  const void* x;
  const uint8_t* w;
  const void* scale;
  const int32_t* zero_point;
  const void* bias; /* may be NULL */
  void* out;
  int64_t m, n, k;
  int64_t ldx, ldw, ldo;
  int32_t type; /* DISC_B200_F32 / DISC_B200_F16 */
  int32_t path; /* 0 = by shape, 1 = streaming kernel, 2 = tensor cores */
} disc_b200_weight_only_qgemm_args;
int32_t disc_b200_weight_only_qgemm(const disc_b200_weight_only_qgemm_args* args, void* stream);
/* Host only: the launch plan for a problem on a GPU with sm_count SMs and weights aligned to
 * `align` (4, 8 or 16) bytes: out7 = {rows per pass, rows padded to 1/2/4/8/16, weight bytes per
 * lane and load, blocks along N, cluster size along K, k rows per block, dynamic shared memory
 * bytes}.  0 = ok, 1 = bad argument, 2 = K too large for the shared-memory staging. */
int32_t disc_b200_weight_only_qgemm_plan(int64_t m, int64_t n, int64_t k, int32_t align, int32_t sm_count,
                                         int64_t* out7);

/* Quantized 2-D convolution, int8 x int8 -> int8, symmetric:
 *   out = sat_s8(rne( conv(x, w) * (x_scale * w_scale(o) / out_scale) ))
 * (ral_qconv on "gpu": tao_compiler/mlir/ral/context/stream_executor_based_impl.cc:1832-1950;
 * ral_pdll_qconv2d: common_context_impl_quantization.cc:363-607).  Operands are dense
 * row-major tensors of rank 4 whose dimension roles come from `metadata`, in the
 * reference's order (stream_executor_based_impl.cc:1127-1152): input (batch, channel,
 * y, x dims), kernel (in-feature, out-feature, y, x dims), output (batch, channel, y,
 * x dims), strides (y, x), dilations (y, x); `padding` = (top, bottom, left, right).
 * One group.  Scales are device pointers.  The product runs on the int8 tensor cores as
 * the quantized linear.  Channels-last inputs with a multiple of 64 channels (and a kernel
 * already [out, y, x, in]) are read in place: the linear fetches its activation tiles from
 * the image with TMA in im2col mode; 1 x 1 windows with unit strides over dense
 * channels-last inputs are the linear itself.  Otherwise the receptive fields are gathered
 * into `workspace` first.  `workspace` (device, 256-byte aligned, at least
 * disc_b200_qconv2d_workspace_bytes) is required in every case; splitk_ws is the linear's
 * scratch (see disc_b200_qgemm_args), needed when batch * out_h * out_w <= 128. */
typedef struct disc_b200_qconv2d_args {
  const int8_t* x;
  const int8_t* w;
  int8_t* out;
  int64_t input_sizes[4];
  int64_t kernel_sizes[4];
  int64_t output_sizes[4];
  int32_t padding[4];
  int32_t metadata[16];
  const float* x_scale;
  const float* w_scale;
  int32_t w_scale_per_channel; /* 0: one value, 1: one per output channel */
  const float* out_scale;
  void* workspace;
  int64_t workspace_bytes;
  void* splitk_ws;
  int64_t splitk_ws_bytes;
} disc_b200_qconv2d_args;
/* -1 if the shapes, padding and metadata do not describe a convolution. */
int64_t disc_b200_qconv2d_workspace_bytes(const disc_b200_qconv2d_args* args);
int32_t disc_b200_qconv2d(const disc_b200_qconv2d_args* args, void* stream);
/* Host only: padding (top, bottom, left, right), result sizes (in the data format)
 * and metadata (17 entries: the 16 above + weight_is_const) from the attributes of
 * ral_pdll_qconv2d, by the reference's rules (common_context_impl_quantization.h:45-215):
 * data_format "NHWC" | "NCHW"; strides / dilations of 1, 2 or 4 entries; padding
 * "SAME" | "VALID" | "EXPLICIT" (explicit_paddings of 4 or 8 entries); kernel
 * [out, y, x, in]. */
int32_t disc_b200_qconv2d_plan(const char* data_format, const int64_t* strides, int32_t n_strides,
                               const int64_t* dilations, int32_t n_dilations, const char* padding,
                               const int64_t* explicit_paddings, int32_t n_explicit, int32_t weight_is_const,
                               const int64_t* input_sizes4, const int64_t* weight_sizes4, int32_t* padding_out4,
                               int64_t* result_sizes4, int32_t* metadata_out17);

/* Calibration observers on the device (the reference runs them as eager torch ops:
 * MinMaxObserver, PerChannelMinMaxObserver and Observer._calculate_qparams,
 * tools/torch_quant/torch_quant/observer.py:134-165, 230-297).
 * observe: min_val[c] = min(min_val[c], min x[:, c, :]), max_val likewise, x f32 / f16
 * viewed as [outer, channels, inner]; the caller starts the state at +inf / -inf;
 * scratch: at least disc_b200_observe_minmax_scratch_floats floats.
 * qparams: lo = min(min_val, 0), hi = max(max_val, 0);
 *   symmetric: scale = max(max(-lo, hi) / ((qmax - qmin) / 2), eps), zero point as given
 *              (0 for signed, 128 for unsigned 8-bit);
 *   affine:    scale = max((hi - lo) / (qmax - qmin), eps),
 *              zero point = clamp(qmin - rne(lo / scale), qmin, qmax);
 *   a range never observed (min > max) gives scale 1, zero point 0. */
int64_t disc_b200_observe_minmax_scratch_floats(int64_t outer, int64_t channels, int64_t inner);
int32_t disc_b200_observe_minmax(const void* x, int32_t type, int64_t outer, int64_t channels, int64_t inner,
                                 float* min_val, float* max_val, float* scratch, int64_t scratch_floats,
                                 void* stream);
int32_t disc_b200_minmax_qparams(const float* min_val, const float* max_val, int64_t n, int32_t qmin, int32_t qmax,
                                 int32_t symmetric, int32_t symmetric_zero_point, float* scale, int32_t* zero_point,
                                 void* stream);

/* counts[b] += number of x in bin b of `bins` equal bins over [lo, hi], the binning of torch.histc, which the
 * reference's HistogramObserver runs once per calibration batch
 * (tools/torch_quant/torch_quant/observer.py:674-724): bin (int)((x - lo) * bins / (hi - lo)) in float32, the
 * last bin includes hi, values outside [lo, hi] and NaN are skipped.  counts (uint32, device) is accumulated into. */
int32_t disc_b200_observe_histogram(const void* x, int32_t type, int64_t n, float lo, float hi, int32_t bins,
                                    uint32_t* counts, void* stream);

/* softmax(x * scale + mask) over the last axis; lens / mask may be NULL
 * (kStitch softmax; same reference files as above). */
int32_t disc_b200_softmax(const void* x, void* y, int32_t type, int64_t rows, int64_t cols,
                          int64_t rows_per_batch, const int32_t* lens, const void* mask,
                          float scale, int32_t log_softmax, void* stream);

/* Masked self-attention over packed sequences in one kernel:
 * out = quantize(softmax(Q K^T * scale) V) per head, the scores never leaving the
 * SM.  It stands for the chain the reference's compiled encoder runs there:
 * two library GEMMs (ral_gemm,
 * tao_compiler/mlir/ral/context/stream_executor_based_impl.cc:551-637), the
 * generated softmax between them and the quantize after them.
 * qkv: f16 [tokens, 3 * heads * 64] (q | k | v, head h in columns h * 64 .. of
 * each third), sequences stored one after the other without padding rows.
 * blocks: device array with one entry per work item = one or more consecutive
 * blocks of 128 query rows of one sequence ({first token of the sequence, its
 * length 1..512, first query row of the item inside the sequence, number of
 * 128-row blocks of the item}); the items of a sequence cover its rows once.
 * out: [tokens, heads * 64], int8 quantized at *out_scale (reciprocal form,
 * at most one level from the divide-based quantize) or f16 when out_scale is NULL. */
typedef struct disc_b200_attention_args {
  const void* qkv;
  int64_t tokens;
  int64_t ld_qkv;
  int32_t heads;
  const int32_t* blocks;
  int32_t num_blocks;
  float scale;
  void* out;
  int64_t ld_out;
  const float* out_scale;
} disc_b200_attention_args;
int32_t disc_b200_attention(const disc_b200_attention_args* args, void* stream);

/* ---- Collectives of the column-parallel (N-split) configuration.
 * One process per GPU.  NCCL is reached through dlopen (the copy already
 * mapped into the process, else the system's libnccl.so.2), so the library
 * loads without it.  The communicator made here (or any ncclComm_t of the same
 * NCCL) goes into disc_b200_context_options.nccl_comm for the custom calls
 * ral_all_gather / ral_all_reduce / ral_async_collective_done
 * (tao_compiler/mlir/ral/collective.cu.cc:60-309,398-504 in the reference, which
 * takes its communicator from the execution context the same way) and
 * disc_b200_qgemm_all_gather. */

/* NCCL version code (e.g. 22809) when NCCL could be bound, 0 otherwise. */
int32_t disc_b200_nccl_available(void);
/* Rank 0 makes the 128-byte id and hands it to the other ranks (any host
 * channel); every rank then creates its communicator with it. */
int32_t disc_b200_nccl_unique_id(void* id128);
int32_t disc_b200_nccl_comm_create(const void* id128, int32_t nranks, int32_t rank, void** comm);
int32_t disc_b200_nccl_comm_destroy(void* comm);
/* recv[r * bytes_per_rank ...] = rank r's send buffer; in place when
 * send == recv + rank * bytes_per_rank. */
int32_t disc_b200_all_gather(void* comm, const void* send, void* recv, int64_t bytes_per_rank,
                             void* stream);
/* The same for a byte range of every slot of a [nranks][slot_bytes] buffer:
 * bytes [offset_bytes, offset_bytes + bytes) of slot r come from rank r.  Lets a
 * host gather a block of rows while the kernel computing the next block of
 * rows still runs (the slots of a column-parallel result are row-major, so a
 * block of rows is one contiguous range per slot). */
int32_t disc_b200_all_gather_rows(void* comm, void* buf, int32_t nranks, int64_t slot_bytes,
                                  int64_t offset_bytes, int64_t bytes, void* stream);
/* op: 0 sum, 1 prod, 2 max, 3 min (per-token activation scales of a row that
 * is spread over the ranks are agreed on with max). */
int32_t disc_b200_all_reduce_f32(void* comm, const float* send, float* recv, int64_t count,
                                 int32_t op, void* stream);

/* ---- Constants of a compiled executable.
 * A DISC executable asks for its constants (the int8 weights, scale vectors and
 * biases of the quantized path among them) through the custom call ral_const
 * (ctx, stream handle, unique name, module-unique index) -> memref, on "cpu" for
 * host constants and "gpu" for device ones
 * (tao_compiler/mlir/ral/context/common_context_impl.cc:279-420,
 * common_context_impl_cuda.cc:61-200).  The values live in the metadata file
 * written next to the executable (tao_compiler/mlir/ral/ral_metadata.cc:65-167:
 * magic, {is_host, key, hexadecimal value} entries, count); a unique name is
 * "<id>_<type tag>_<d0xd1x...>".  The host loads the file into the context once;
 * constants are decoded on first use, device constants uploaded once and kept
 * until the context is destroyed. */
int32_t disc_b200_context_load_metadata(disc_b200_context* ctx, const char* path);
/* The same, with the constants shared by every context of this process that attaches the
 * same file on the same device: each constant is decoded and uploaded once per process and
 * lives until the last such context is destroyed (the reference's process-level store,
 * common_context_impl.cc:152-185).  disc_b200_context_load_metadata does this too when the
 * environment has DISC_USE_GLOBAL_CONST_STORE=true|1, the reference's switch. */
int32_t disc_b200_context_share_metadata(disc_b200_context* ctx, const char* path);
/* Writes a metadata file in the reference's format (tools, tests). */
int32_t disc_b200_metadata_write(const char* path, int32_t n, const char* const* names, const int32_t* is_host,
                                 const void* const* data, const int64_t* bytes);
/* Shape (up to 8 dims) and element width encoded in a constant's unique name. */
int32_t disc_b200_const_name_info(const char* unique_name, int32_t* rank, int64_t* sizes8, int64_t* elem_bytes);

/* ---- Compiler-generated kernels.  ral_kernel_launch (blobs, num_blobs, kernel
 * name, grid, block, shared memory, stream, params) loads one of the device
 * images the executable embeds and launches the named kernel
 * (tao_compiler/mlir/ral/context/base/cuda/cuda_context_impl.cc:348-445).  This is
 * the reference's choice of image for a device (common_context_impl.cc:209-215:
 * image 0 carries PTX, images 1..4 are sm_70 / 75 / 80 / 86 code): a B200 gets
 * image 0 and the driver compiles its PTX.  -1 if there is no image. */
int32_t disc_b200_select_device_image(int64_t num_images, int32_t cc_major, int32_t cc_minor);

/* ------------------------------------------------------------------------
 * 4. Diagnostics.
 * ---------------------------------------------------------------------- */

/* Message of the last failing section-3 call on this thread ("" if none). */
const char* disc_b200_last_error_string(void);
/* Synchronises the device, returns and clears the status word kernels set when
 * one of their bounded waits ran out (0 = none did). */
int32_t disc_b200_kernel_status(void);
/* Self-test of that mechanism on a live GPU: one warp waits, with the kernels' own bounded wait, on a
 * barrier that nobody arrives on.  Nothing is in flight and nothing faults: after limit_ns (1 ns .. 100 ms) the
 * wait gives up, the kernel returns and the status word holds code 9 until disc_b200_kernel_status() reads it.
 * *waited_ns (host) receives the time the wait lasted.  Synchronises the stream.  No counterpart in the
 * reference, whose runtime has no device-side waits of its own. */
int32_t disc_b200_selftest_wait_expiry(uint64_t limit_ns, int64_t* waited_ns, void* stream);
const char* disc_b200_version(void);
/* Parses a serialized custom_attrs blob (wire format of tao_compiler/mlir/ral/
 * context/pdll_util.cc:20-170) and writes a canonical text rendering such as
 * {a: true, b: 127, c: "s", d: [1, 2], e: dense<int64[2]>} into `out`.
 * Returns the length written, or -1 if the blob does not parse. */
int32_t disc_b200_attrs_describe(const void* blob, char* out, int32_t capacity);
/* The same for a blob whose size is known: nothing past blob_bytes is read. */
int32_t disc_b200_attrs_describe_bounded(const void* blob, int64_t blob_bytes, char* out, int32_t capacity);

#ifdef __cplusplus
}
#endif

#endif /* DISC_B200_RAL_H_ */
