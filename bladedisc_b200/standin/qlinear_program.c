/* A stand-in for the shared object the DISC compiler would emit for one quantized linear with the
 * fused epilogue, written by hand the way generated code behaves: an entry point "main" that receives
 * { execution context, dispatcher } and reaches every runtime service through the dispatcher with a
 * mangled name and a type-erased argument array (tao_compiler/mlir/disc/disc_compiler.cc:95-131,
 * tao_compiler/mlir/disc/transforms/disc_to_llvm.cc:302-365).  No DISC compiler exists outside the
 * reference's build, so the benchmark drives the boundary with this program:
 *
 *   x      = ral_recv_input(0)                      int8 [M, K] on the GPU (torch_blade hands engines CUDA tensors)
 *   w, b, s_x, s_w, s_out = ral_const(...)          from the metadata file; uploaded once per context
 *   q      = disc_b200_qgemm(x, w, b, s_x, s_w, s_out, attrs)   int8 [M, N]
 *   ral_send_output(0, q)
 *
 * The names of the constants carry the shapes (Nx K etc.) and are passed in at compile time:
 *   -DCONST_W='"0_i8_4096x4096"' -DCONST_B='"1_f32_4096"' -DCONST_SW='"3_f32_4096"'
 * ATTRS_BLOB_H names a generated header with `static const unsigned char attrs_blob[]`, the serialized
 * attribute dictionary of the call ({"activation": "none"}). */
#include <stdint.h>
#include <string.h>

#include ATTRS_BLOB_H

typedef void (*dispatch_fn)(void* ctx, const char* name, void** args);

static void disc_ral_call(void** ctx_struct, const char* name, void** args) {
  void* real_ctx = ctx_struct[0];
  dispatch_fn fn = (dispatch_fn)ctx_struct[1];
  *(void**)args[0] = real_ctx;
  fn(real_ctx, name, args);
}

typedef struct { void* base; void* data; int64_t offset; } memref0;
typedef struct { void* base; void* data; int64_t offset; int64_t sizes[1]; int64_t strides[1]; } memref1;
typedef struct { void* base; void* data; int64_t offset; int64_t sizes[2]; int64_t strides[2]; } memref2;

static int put0(void** a, int i, memref0* m) { a[i++] = &m->base; a[i++] = &m->data; a[i++] = &m->offset; return i; }
static int put1(void** a, int i, memref1* m) {
  a[i++] = &m->base; a[i++] = &m->data; a[i++] = &m->offset; a[i++] = &m->sizes[0]; a[i++] = &m->strides[0];
  return i;
}
static int put2(void** a, int i, memref2* m) {
  a[i++] = &m->base; a[i++] = &m->data; a[i++] = &m->offset;
  a[i++] = &m->sizes[0]; a[i++] = &m->sizes[1]; a[i++] = &m->strides[0]; a[i++] = &m->strides[1];
  return i;
}

static void get_const(void** cs, const char* api, const char* name, int32_t index, void* result) {
  void* ctx = 0;
  void* stream = 0;
  const char* n = name;
  void* args[5] = {&ctx, &stream, &n, &index, result};
  disc_ral_call(cs, api, args);
}

void main(void** cs) {
  void* ctx = 0;
  void* stream = 0;
  const void* attrs = attrs_blob;
  int64_t idx = 0;
  memref2 x, w, q;
  memref1 bias, sw;
  memref0 sx, so;
  memset(&x, 0, sizeof(x));
  memset(&w, 0, sizeof(w));
  memset(&q, 0, sizeof(q));
  memset(&bias, 0, sizeof(bias));
  memset(&sw, 0, sizeof(sw));
  memset(&sx, 0, sizeof(sx));
  memset(&so, 0, sizeof(so));
  { void* args[3] = {&ctx, &idx, &x}; disc_ral_call(cs, "ral_recv_input___cpu___pvoid_i64___m2di8", args); }
  get_const(cs, "ral_const___gpu___pvoid_pvoid_pvoid_i32___m2di8", CONST_W, 0, &w);
  get_const(cs, "ral_const___gpu___pvoid_pvoid_pvoid_i32___m1df32", CONST_B, 1, &bias);
  get_const(cs, "ral_const___gpu___pvoid_pvoid_pvoid_i32___m0df32", "2_f32_", 2, &sx);
  get_const(cs, "ral_const___gpu___pvoid_pvoid_pvoid_i32___m1df32", CONST_SW, 3, &sw);
  get_const(cs, "ral_const___gpu___pvoid_pvoid_pvoid_i32___m0df32", "4_f32_", 4, &so);
  if (!x.data || !w.data) return;   /* a failed call left the context in its error state */
  void* args[40];
  int i = 0;
  args[i++] = &ctx;
  args[i++] = &stream;
  i = put2(args, i, &x);
  i = put2(args, i, &w);
  i = put1(args, i, &bias);
  i = put0(args, i, &sx);
  i = put1(args, i, &sw);
  i = put0(args, i, &so);
  args[i++] = &attrs;
  args[i++] = &q;
  disc_ral_call(cs, "disc_b200_qgemm___gpu___pvoid_pvoid_m2di8_m2di8_m1df32_m0df32_m1df32_m0df32_pvoid___m2di8", args);
  int64_t o = 0;
  args[0] = &ctx; args[1] = &o; put2(args, 2, &q);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m2di8___void", args);
}
