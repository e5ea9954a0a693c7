// The two host custom calls the reference ships for testing the custom_call_v2
// mechanism itself: "disc.custom_call.test.tf_fused_add_mul" ((A + B)^2) and
// "..._multi_results" ((A + B), (A + B)^2), f32 rank 2 on "cpu", operands
// (A, B, custom_attrs) (tao_compiler/mlir/ral/context/common_context_impl_pdll.cc:30-360).
// With them a compiled executable that exercises attributes and tuple results runs
// on this runtime exactly as on the reference's, which is how the tests pin the
// result-slot convention of multi-result calls.  Host code only.
#include <cstring>
#include <string>
#include <tuple>

#include "abi.h"
#include "context.h"
#include "pdl_attr.h"

namespace disc_b200 {
namespace ral {
namespace {

bool attrs_parse(ExecContext* ctx, void* blob) {
  if (!blob) return true;
  const uint8_t* cur = static_cast<const uint8_t*>(blob);
  auto a = parse_attr(&cur);
  if (!a || a->kind != Attr::kDict) {
    ctx->signal_error("fail to parse custom_attrs");
    return false;
  }
  return true;
}

MemRef<float, 2> like(ExecContext* ctx, const MemRef<float, 2>& a) {
  const int64_t n = a.sizes[0] * a.sizes[1];
  float* data = static_cast<float*>(ctx->host_alloc(static_cast<size_t>(n) * sizeof(float)));
  return make_memref<float, 2>(data, a.sizes);
}

MemRef<float, 2> fused_add_mul(ExecContext* ctx, void* stream_handle, MemRef<float, 2> a, MemRef<float, 2> b,
                               void* custom_attrs) {
  MemRef<float, 2> out = like(ctx, a);
  if (!attrs_parse(ctx, custom_attrs) || !out.data) return out;
  const int64_t n = a.sizes[0] * a.sizes[1];
  for (int64_t i = 0; i < n; ++i) out.data[i] = (a.data[i] + b.data[i]) * (a.data[i] + b.data[i]);
  return out;
}

std::tuple<MemRef<float, 2>, MemRef<float, 2>> fused_add_mul_multi(ExecContext* ctx, void* stream_handle,
                                                                   MemRef<float, 2> a, MemRef<float, 2> b,
                                                                   void* custom_attrs) {
  MemRef<float, 2> sum = like(ctx, a);
  MemRef<float, 2> sq = like(ctx, a);
  if (!attrs_parse(ctx, custom_attrs) || !sum.data || !sq.data) return std::make_tuple(sum, sq);
  const int64_t n = a.sizes[0] * a.sizes[1];
  for (int64_t i = 0; i < n; ++i) {
    sum.data[i] = a.data[i] + b.data[i];
    sq.data[i] = sum.data[i] * sum.data[i];
  }
  return std::make_tuple(sum, sq);
}

DISC_B200_RAL_API("disc.custom_call.test.tf_fused_add_mul", "cpu", fused_add_mul);
DISC_B200_RAL_API("disc.custom_call.test.tf_fused_add_mul_multi_results", "cpu", fused_add_mul_multi);

}  // namespace
}  // namespace ral
}  // namespace disc_b200
