#include "pdl_attr.h"

#include <cstring>

namespace disc_b200 {
namespace ral {
namespace {

struct Reader {
  const uint8_t* p;
  int64_t budget;
  bool bad = false;

  template <typename T>
  T pod() {
    T v{};
    if (bad || budget < static_cast<int64_t>(sizeof(T))) {
      bad = true;
      return v;
    }
    std::memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    budget -= sizeof(T);
    return v;
  }
  // A blob comes as a bare pointer: its true length is unknown, so every length field is
  // also held against what such a field can sensibly be, before anything is read through it.
  std::string str(int64_t limit) {
    const int64_t n = pod<int64_t>();
    if (bad || n < 0 || n > budget || n > limit) {
      bad = true;
      return std::string();
    }
    std::string s(reinterpret_cast<const char*>(p), static_cast<size_t>(n));
    p += n;
    budget -= n;
    return s;
  }
};

constexpr int64_t kMaxTypeName = 32;        // "denseElementsAttr" is the longest
constexpr int64_t kMaxKey = 4096;
constexpr int64_t kMaxString = 1 << 20;
constexpr int64_t kMaxCount = 1 << 20;      // entries of a dict / array / intArray
constexpr int64_t kMaxDenseBytes = 1 << 28;

std::unique_ptr<Attr> parse_value(Reader& r, int depth) {
  if (depth > 64) {
    r.bad = true;
    return nullptr;
  }
  const std::string type = r.str(kMaxTypeName);
  if (r.bad) return nullptr;
  auto a = std::make_unique<Attr>();
  if (type == "dict") {
    a->kind = Attr::kDict;
    const int64_t n = r.pod<int64_t>();
    if (r.bad || n < 0 || n > kMaxCount) return nullptr;
    for (int64_t i = 0; i < n; ++i) {
      std::string key = r.str(kMaxKey);
      auto v = parse_value(r, depth + 1);
      if (!v) return nullptr;
      a->dict[key] = std::move(v);
    }
  } else if (type == "str") {
    a->kind = Attr::kStr;
    a->str = r.str(kMaxString);
  } else if (type == "bool") {
    a->kind = Attr::kBool;
    a->b = r.pod<uint8_t>() != 0;
  } else if (type == "int") {
    a->kind = Attr::kInt;
    a->i = r.pod<int64_t>();
  } else if (type == "float") {
    a->kind = Attr::kFloat;
    a->f = r.pod<double>();
  } else if (type == "intArray") {
    a->kind = Attr::kIntArray;
    const int64_t n = r.pod<int64_t>();
    if (r.bad || n < 0 || n > kMaxCount || n * 8 > r.budget) return nullptr;
    a->ints.reserve(static_cast<size_t>(n));
    for (int64_t i = 0; i < n; ++i) a->ints.push_back(r.pod<int64_t>());
  } else if (type == "array") {
    a->kind = Attr::kArray;
    const int64_t n = r.pod<int64_t>();
    if (r.bad || n < 0 || n > kMaxCount) return nullptr;
    for (int64_t i = 0; i < n; ++i) {
      auto v = parse_value(r, depth + 1);
      if (!v) return nullptr;
      a->array.push_back(std::move(v));
    }
  } else if (type == "denseElementsAttr") {
    a->kind = Attr::kDense;
    a->elem_type = r.str(kMaxTypeName);
    a->elem_bits = r.pod<uint32_t>();
    const int64_t rank = r.pod<int64_t>();
    if (r.bad || rank < 0 || rank > 64 || a->elem_bits > 1024) return nullptr;
    int64_t numel = 1;
    for (int64_t i = 0; i < rank; ++i) {
      const int64_t d = r.pod<int64_t>();
      if (r.bad || d < 0 || (d != 0 && numel > kMaxDenseBytes / d)) return nullptr;
      a->shape.push_back(d);
      numel *= d;
    }
    const bool splat = r.pod<uint8_t>() != 0;
    const std::string data = r.str(kMaxDenseBytes);
    if (r.bad) return nullptr;
    if (splat) {
      const size_t eb = a->elem_bits / 8;
      if (eb == 0 || data.size() != eb || numel > kMaxDenseBytes / static_cast<int64_t>(eb)) return nullptr;
      a->raw.resize(static_cast<size_t>(numel) * eb);
      for (size_t i = 0; i < a->raw.size(); ++i) a->raw[i] = static_cast<uint8_t>(data[i % eb]);
    } else {
      a->raw.assign(data.begin(), data.end());
    }
  } else {
    return nullptr;
  }
  if (r.bad) return nullptr;
  return a;
}

}  // namespace

std::unique_ptr<Attr> parse_attr(const uint8_t** cursor, int64_t max_bytes) {
  if (!cursor || !*cursor) return nullptr;
  Reader r{*cursor, max_bytes};
  auto a = parse_value(r, 0);
  if (a) *cursor = r.p;
  return a;
}

}  // namespace ral
}  // namespace disc_b200
