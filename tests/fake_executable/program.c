/* TEST INFRASTRUCTURE.  A stand-in for the shared object the DISC compiler emits,
 * written by hand the way generated code behaves: an entry point "main" that
 * receives { execution context, dispatcher }, and a local disc_ral_call stub that
 * stores the real context into the first argument slot and calls the dispatcher
 * with a mangled name and a type-erased argument array
 * (tao_compiler/mlir/disc/disc_compiler.cc:95-131,
 * tao_compiler/mlir/disc/transforms/disc_to_llvm.cc:302-365).
 *
 * It links against nothing: every runtime service comes through the dispatcher.
 *   -DHOST_PROGRAM: out0 = in0 + const "0_f32_8" computed on the host in a buffer
 *     from "alloc" on "cpu"; out1 = the constant; out2 = in0 itself; out3 = out0's
 *     buffer under a second name ([1, n], made by "inc_ref") after the first name
 *     was released with "dealloc".
 *   -DHOST_PROGRAM2: rank-3 and rank-0 inputs, a persistent buffer, a reshape of an input
 *     and a second name for a scalar (see the comment at that entry point).
 *   -DHOST_PROGRAM3: the reference's two custom_call_v2 test kernels, attributes and a tuple result.
 *   default: a quantized linear on the GPU; weight, bias and scales from ral_const,
 *     the product from ral_pdll_qgemm; out0 = the int8 result, out1 = a host
 *     constant, out2 = a host buffer holding the result's shape. */
#include <stdint.h>
#include <string.h>

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

/* flattens a memref into argument slots; returns the next free slot */
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

static void* host_alloc(void** cs, uint64_t bytes) {
  void* ctx = 0;
  void* p = 0;
  void* args[3] = {&ctx, &bytes, &p};
  disc_ral_call(cs, "alloc___cpu___pvoid_i64___pvoid", args);
  return p;
}

#ifdef HOST_PROGRAM
void main(void** cs) {
  void* ctx = 0;
  int64_t idx = 0;
  memref1 x, c, y;
  memset(&x, 0, sizeof(x));
  memset(&c, 0, sizeof(c));
  { void* args[3] = {&ctx, &idx, &x}; disc_ral_call(cs, "ral_recv_input___cpu___pvoid_i64___m1df32", args); }
  get_const(cs, "ral_const___cpu___pvoid_pvoid_pvoid_i32___m1df32", "0_f32_8", 0, &c);
  if (!x.data || !c.data) return;   /* a failed call left the context in its error state */
  int64_t n = x.sizes[0] < c.sizes[0] ? x.sizes[0] : c.sizes[0];
  float* out = (float*)host_alloc(cs, (uint64_t)n * sizeof(float));
  void* scratch = host_alloc(cs, 256);      /* a temporary the program frees itself */
  for (int64_t i = 0; i < n; ++i) out[i] = ((float*)x.data)[i] + ((float*)c.data)[i];
  { void* args[2] = {&ctx, &scratch}; disc_ral_call(cs, "dealloc___cpu___pvoid_pvoid___void", args); }
  (void)host_alloc(cs, 64);                 /* and one it forgets: freed with the execution */
  y.base = y.data = out; y.offset = 0; y.sizes[0] = n; y.strides[0] = 1;
  void* args[16];
  int64_t o;
  /* a second name for the result, [1, n], by the reshape call; the first name is then released */
  memref2 view;
  memset(&view, 0, sizeof(view));
  {
    int64_t dims[2] = {1, n};
    memref1 shape;
    void* stream = 0;
    shape.base = shape.data = dims; shape.offset = 0; shape.sizes[0] = 2; shape.strides[0] = 1;
    int i = 0;
    args[i++] = &ctx; args[i++] = &stream;
    i = put1(args, i, &y);
    i = put1(args, i, &shape);
    args[i++] = &view;
    disc_ral_call(cs, "inc_ref___cpu___pvoid_pvoid_m1df32_m1di64___m2df32", args);
    void* first_name = out;
    void* dargs[2] = {&ctx, &first_name};
    disc_ral_call(cs, "dealloc___cpu___pvoid_pvoid___void", dargs);
  }
  o = 0; args[0] = &ctx; args[1] = &o; put1(args, 2, &y);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m1df32___void", args);
  o = 1; args[0] = &ctx; args[1] = &o; put1(args, 2, &c);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m1df32___void", args);
  o = 2; args[0] = &ctx; args[1] = &o; put1(args, 2, &x);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m1df32___void", args);
  o = 3; args[0] = &ctx; args[1] = &o; put2(args, 2, &view);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m2df32___void", args);
}
#elif defined(HOST_PROGRAM3)
/* in0, in1: f32 [r, c].  Calls the two custom_call_v2 test kernels with an attribute blob that is
 * part of the executable's constant data (ATTRS_BLOB_H defines `static const unsigned char
 * attrs_blob[]`, generated by the test): out0 = (in0 + in1)^2 from the single-result call,
 * out1 = in0 + in1 and out2 = (in0 + in1)^2 from the call that returns a tuple: one result slot
 * per element of the tuple. */
#include ATTRS_BLOB_H
void main(void** cs) {
  void* ctx = 0;
  void* stream = 0;
  const void* attrs = attrs_blob;
  int64_t idx;
  memref2 a, b, sq, sum2, sq2;
  memset(&a, 0, sizeof(a));
  memset(&b, 0, sizeof(b));
  memset(&sq, 0, sizeof(sq));
  memset(&sum2, 0, sizeof(sum2));
  memset(&sq2, 0, sizeof(sq2));
  idx = 0;
  { void* args[3] = {&ctx, &idx, &a}; disc_ral_call(cs, "ral_recv_input___cpu___pvoid_i64___m2df32", args); }
  idx = 1;
  { void* args[3] = {&ctx, &idx, &b}; disc_ral_call(cs, "ral_recv_input___cpu___pvoid_i64___m2df32", args); }
  void* args[24];
  int i = 0;
  args[i++] = &ctx; args[i++] = &stream;
  i = put2(args, i, &a);
  i = put2(args, i, &b);
  args[i++] = &attrs;
  args[i++] = &sq;
  disc_ral_call(cs, "disc.custom_call.test.tf_fused_add_mul___cpu___pvoid_pvoid_m2df32_m2df32_pvoid___m2df32", args);
  i = 0;
  args[i++] = &ctx; args[i++] = &stream;
  i = put2(args, i, &a);
  i = put2(args, i, &b);
  args[i++] = &attrs;
  args[i++] = &sum2;   /* first element of the tuple */
  args[i++] = &sq2;    /* second element */
  disc_ral_call(cs,
                "disc.custom_call.test.tf_fused_add_mul_multi_results___cpu___pvoid_pvoid_m2df32_m2df32_pvoid___"
                "m2df32_m2df32",
                args);
  int64_t o;
  o = 0; args[0] = &ctx; args[1] = &o; put2(args, 2, &sq);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m2df32___void", args);
  o = 1; args[0] = &ctx; args[1] = &o; put2(args, 2, &sum2);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m2df32___void", args);
  o = 2; args[0] = &ctx; args[1] = &o; put2(args, 2, &sq2);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m2df32___void", args);
}
#elif defined(HOST_PROGRAM2)
/* in0: f32 [a, b, c], in1: i64 scalar.
 * out0: i64 [3] = in0's shape, in a buffer from "ral_cpu_alloc_persistent";
 * out1: i64 scalar = in1 + 1, in a buffer from "alloc";
 * out2: f32 [a * b, c] = in0 itself under a new shape ("inc_ref" with a shape operand);
 * out3: i64 scalar = out1's buffer under a second name ("inc_ref" without a shape operand). */
typedef struct { void* base; void* data; int64_t offset; int64_t sizes[3]; int64_t strides[3]; } memref3;
void main(void** cs) {
  void* ctx = 0;
  void* stream = 0;
  int64_t idx;
  memref3 x;
  memref0 s;
  memset(&x, 0, sizeof(x));
  memset(&s, 0, sizeof(s));
  idx = 0;
  { void* args[3] = {&ctx, &idx, &x}; disc_ral_call(cs, "ral_recv_input___cpu___pvoid_i64___m3df32", args); }
  idx = 1;
  { void* args[3] = {&ctx, &idx, &s}; disc_ral_call(cs, "ral_recv_input___cpu___pvoid_i64___m0di64", args); }
  if (!s.data) return;
  uint64_t bytes = 3 * sizeof(int64_t);
  int64_t* dims = 0;
  { void* args[3] = {&ctx, &bytes, &dims}; disc_ral_call(cs, "ral_cpu_alloc_persistent___cpu___pvoid_i64___pvoid", args); }
  int64_t* next = (int64_t*)host_alloc(cs, sizeof(int64_t));
  if (!dims || !next) return;
  dims[0] = x.sizes[0]; dims[1] = x.sizes[1]; dims[2] = x.sizes[2];
  *next = *(int64_t*)s.data + 1;
  memref1 d;
  d.base = d.data = dims; d.offset = 0; d.sizes[0] = 3; d.strides[0] = 1;
  memref0 n0;
  n0.base = n0.data = next; n0.offset = 0;
  /* in0 as [a * b, c] */
  int64_t flat[2];
  flat[0] = x.sizes[0] * x.sizes[1]; flat[1] = x.sizes[2];
  memref1 shape;
  shape.base = shape.data = flat; shape.offset = 0; shape.sizes[0] = 2; shape.strides[0] = 1;
  memref2 x2;
  memset(&x2, 0, sizeof(x2));
  void* args[24];
  int i = 0;
  args[i++] = &ctx; args[i++] = &stream;
  args[i++] = &x.base; args[i++] = &x.data; args[i++] = &x.offset;
  args[i++] = &x.sizes[0]; args[i++] = &x.sizes[1]; args[i++] = &x.sizes[2];
  args[i++] = &x.strides[0]; args[i++] = &x.strides[1]; args[i++] = &x.strides[2];
  i = put1(args, i, &shape);
  args[i++] = &x2;
  disc_ral_call(cs, "inc_ref___cpu___pvoid_pvoid_m3df32_m1di64___m2df32", args);
  /* a second name for the scalar */
  memref0 n1;
  memset(&n1, 0, sizeof(n1));
  i = 0;
  args[i++] = &ctx; args[i++] = &stream;
  i = put0(args, i, &n0);
  args[i++] = &n1;
  disc_ral_call(cs, "inc_ref___cpu___pvoid_pvoid_m0di64___m0di64", args);
  int64_t o;
  o = 0; args[0] = &ctx; args[1] = &o; put1(args, 2, &d);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m1di64___void", args);
  o = 1; args[0] = &ctx; args[1] = &o; put0(args, 2, &n0);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m0di64___void", args);
  o = 2; args[0] = &ctx; args[1] = &o; put2(args, 2, &x2);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m2df32___void", args);
  o = 3; args[0] = &ctx; args[1] = &o; put0(args, 2, &n1);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m0di64___void", args);
}
#else
void main(void** cs) {
  void* ctx = 0;
  void* stream = 0;
  void* attrs = 0;
  int64_t idx = 0;
  memref2 x, w, q;
  memref1 bias, dims;
  memref0 sx, sw, so, zp;
  memset(&x, 0, sizeof(x));
  memset(&w, 0, sizeof(w));
  memset(&q, 0, sizeof(q));
  memset(&bias, 0, sizeof(bias));
  memset(&dims, 0, sizeof(dims));
  memset(&sx, 0, sizeof(sx));
  memset(&sw, 0, sizeof(sw));
  memset(&so, 0, sizeof(so));
  memset(&zp, 0, sizeof(zp));
  { void* args[3] = {&ctx, &idx, &x}; disc_ral_call(cs, "ral_recv_input___cpu___pvoid_i64___m2di8", args); }
  get_const(cs, "ral_const___gpu___pvoid_pvoid_pvoid_i32___m2di8", "0_i8_192x256", 0, &w);
  get_const(cs, "ral_const___gpu___pvoid_pvoid_pvoid_i32___m1df32", "1_f32_192", 1, &bias);
  get_const(cs, "ral_const___gpu___pvoid_pvoid_pvoid_i32___m0df32", "2_f32_", 2, &sx);
  get_const(cs, "ral_const___gpu___pvoid_pvoid_pvoid_i32___m0df32", "3_f32_", 3, &sw);
  get_const(cs, "ral_const___gpu___pvoid_pvoid_pvoid_i32___m0df32", "4_f32_", 4, &so);
  get_const(cs, "ral_const___gpu___pvoid_pvoid_pvoid_i32___m0di32", "5_i32_", 5, &zp);
  get_const(cs, "ral_const___cpu___pvoid_pvoid_pvoid_i32___m1di64", "6_i64_2", 6, &dims);
  void* args[48];
  int i = 0;
  args[i++] = &ctx;
  args[i++] = &stream;
  i = put2(args, i, &x);
  i = put2(args, i, &w);
  i = put1(args, i, &bias);
  i = put0(args, i, &sx);
  i = put0(args, i, &zp);
  i = put0(args, i, &sw);
  i = put0(args, i, &zp);
  i = put0(args, i, &so);
  i = put0(args, i, &zp);
  args[i++] = &attrs;
  args[i++] = &q;
  disc_ral_call(cs,
                "ral_pdll_qgemm___gpu___pvoid_pvoid_m2di8_m2di8_m1df32_m0df32_m0di32_m0df32_m0di32_m0df32_m0di32_"
                "pvoid___m2di8",
                args);
  int64_t* shape = (int64_t*)host_alloc(cs, 2 * sizeof(int64_t));
  if (!shape) return;
  shape[0] = q.sizes[0];
  shape[1] = q.sizes[1];
  memref1 sh;
  sh.base = sh.data = shape; sh.offset = 0; sh.sizes[0] = 2; sh.strides[0] = 1;
  int64_t o;
  o = 0; args[0] = &ctx; args[1] = &o; put2(args, 2, &q);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m2di8___void", args);
  o = 1; args[0] = &ctx; args[1] = &o; put1(args, 2, &dims);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m1di64___void", args);
  o = 2; args[0] = &ctx; args[1] = &o; put1(args, 2, &sh);
  disc_ral_call(cs, "ral_send_output___cpu___pvoid_i64_m1di64___void", args);
}
#endif
