// Reader (and writer, for tests and hosts that build calls by hand) of the
// serialized `custom_attrs` blob a custom_call_v2 carries as its last pvoid
// argument.  Wire format (writer: tao_compiler/mlir/disc/transforms/
// disc_lower_to_library_call.cc:693-848; reader: tao_compiler/mlir/ral/context/
// pdll_util.cc:20-170):
//   str   := int64 length, bytes
//   value := str(type) payload
//   dict  : int64 n, n x (str key, value)      bool : 1 byte
//   str   : str                                int  : int64
//   float : double                             intArray : int64 n, n x int64
//   array : int64 n, n x value
//   denseElementsAttr : str elem type, uint32 bits, int64 rank, rank x int64,
//                       bool splat, str raw bytes (one element when splat)
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace disc_b200 {
namespace ral {

struct Attr {
  enum Kind { kDict, kStr, kBool, kInt, kFloat, kIntArray, kArray, kDense } kind = kInt;
  std::map<std::string, std::unique_ptr<Attr>> dict;
  std::string str;
  bool b = false;
  int64_t i = 0;
  double f = 0.0;
  std::vector<int64_t> ints;
  std::vector<std::unique_ptr<Attr>> array;
  // dense elements
  std::string elem_type;
  uint32_t elem_bits = 0;
  std::vector<int64_t> shape;
  std::vector<uint8_t> raw;  // expanded when the blob stored a splat

  const Attr* find(const std::string& key) const {
    auto it = dict.find(key);
    return it == dict.end() ? nullptr : it->second.get();
  }
  bool get_bool(const std::string& key, bool dflt) const {
    const Attr* a = find(key);
    return a && a->kind == kBool ? a->b : dflt;
  }
  int64_t get_int(const std::string& key, int64_t dflt) const {
    const Attr* a = find(key);
    return a && a->kind == kInt ? a->i : dflt;
  }
  double get_float(const std::string& key, double dflt) const {
    const Attr* a = find(key);
    return a && a->kind == kFloat ? a->f : dflt;
  }
  std::string get_str(const std::string& key, const std::string& dflt) const {
    const Attr* a = find(key);
    return a && a->kind == kStr ? a->str : dflt;
  }
};

// Parses one value starting at `*cursor` and advances it.  Returns nullptr on
// an unknown type tag or an implausible length (the blob carries no total
// size, so lengths are sanity-checked against `max_bytes`).
std::unique_ptr<Attr> parse_attr(const uint8_t** cursor, int64_t max_bytes = (int64_t)1 << 30);

// Serializer producing the same wire format.
class AttrWriter {
 public:
  void begin_dict(int64_t n) { tag("dict"); i64(n); }
  void key(const std::string& k) { str_raw(k); }
  void put_str(const std::string& v) { tag("str"); str_raw(v); }
  void put_bool(bool v) { tag("bool"); buf_.push_back(v ? 1 : 0); }
  void put_int(int64_t v) { tag("int"); i64(v); }
  void put_float(double v) { tag("float"); raw(&v, sizeof(v)); }
  void put_int_array(const std::vector<int64_t>& v) {
    tag("intArray");
    i64(static_cast<int64_t>(v.size()));
    for (int64_t x : v) i64(x);
  }
  void begin_array(int64_t n) { tag("array"); i64(n); }
  void put_dense(const std::string& elem_type, uint32_t bits, const std::vector<int64_t>& shape,
                 bool splat, const void* data, size_t bytes) {
    tag("denseElementsAttr");
    str_raw(elem_type);
    raw(&bits, sizeof(bits));
    i64(static_cast<int64_t>(shape.size()));
    for (int64_t d : shape) i64(d);
    buf_.push_back(splat ? 1 : 0);
    i64(static_cast<int64_t>(bytes));
    raw(data, bytes);
  }
  const std::vector<uint8_t>& bytes() const { return buf_; }

 private:
  void tag(const char* t) { str_raw(t); }
  void str_raw(const std::string& s) {
    i64(static_cast<int64_t>(s.size()));
    raw(s.data(), s.size());
  }
  void i64(int64_t v) { raw(&v, sizeof(v)); }
  void raw(const void* p, size_t n) {
    const uint8_t* b = static_cast<const uint8_t*>(p);
    buf_.insert(buf_.end(), b, b + n);
  }
  std::vector<uint8_t> buf_;
};

}  // namespace ral
}  // namespace disc_b200
