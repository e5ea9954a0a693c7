// The metadata file that travels with a compiled DISC executable: the (possibly
// large) constants of the graph -- for the quantized path the int8 weights, the
// scale vectors and the biases -- keyed by their unique names.
//
// File format (writer: tao_compiler/mlir/ral/ral_metadata.cc:123-167; reader
// :65-91): u64 magic 0x1234567890ABCDEF, then per constant { bool is_host;
// size_t key length, key bytes; size_t value length, value bytes } and at the
// very end a size_t count.  A value is the constant's bytes as a hexadecimal
// string (common_context_impl.cc:264-277); a unique name is
// "<id>_<type tag>_<d0xd1x...>" whose tag gives the element width and whose
// last field the shape (:217-237); a value shorter than the tensor is a splat.
//
// Own design: the file is mapped, not copied into maps of strings (7B int8
// weights are gigabytes of hex text); the index holds views into the mapping;
// releasing a constant drops its pages.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <string_view>
#include <unordered_map>
#include <vector>

namespace disc_b200 {
namespace ral {

constexpr uint64_t kMetadataMagic = 0x1234567890ABCDEFull;

class MetadataFile {
 public:
  // nullptr (and `error` filled) if the file is missing, truncated or not a metadata file.
  static std::unique_ptr<MetadataFile> load(const std::string& path, std::string* error);
  ~MetadataFile();

  // Hex text of a constant, empty view if there is none (or it was released).
  std::string_view host_constant(const std::string& name) const;
  std::string_view device_constant(const std::string& name) const;
  // Forgets the constant and gives its pages back; false if there is none.
  bool release_host(const std::string& name);
  bool release_device(const std::string& name);
  size_t host_count() const { return host_.size(); }
  size_t device_count() const { return device_.size(); }

 private:
  MetadataFile() = default;
  MetadataFile(const MetadataFile&) = delete;
  MetadataFile& operator=(const MetadataFile&) = delete;
  bool release(std::unordered_map<std::string, std::string_view>* map, const std::string& name);

  void* map_ = nullptr;
  size_t bytes_ = 0;
  std::unordered_map<std::string, std::string_view> host_;
  std::unordered_map<std::string, std::string_view> device_;
};

// Writes the same format (tools and tests; the compiler side in the reference).
class MetadataWriter {
 public:
  explicit MetadataWriter(const std::string& path);
  ~MetadataWriter();
  bool ok() const { return file_ != nullptr; }
  // false on a duplicated key or a write error
  bool add(const std::string& name, bool is_host, const void* data, size_t bytes);
  bool finish();

 private:
  void* file_ = nullptr;  // FILE*
  std::unordered_map<std::string, bool> seen_;
  size_t count_ = 0;
};

// Bytes of a hexadecimal string; an odd length means a leading half byte
// (common_context_impl.cc:264-277).  false on a character that is not a hex digit.
bool decode_hex(std::string_view hex, std::vector<uint8_t>* out);

// Shape and element width of a constant from its unique name
// "<id>_<tag>_<d0xd1x...>": width = digits of the tag / 8, at least 1; an empty
// last field is rank 0.  false if the name does not have three fields.
bool parse_const_name(const std::string& name, std::vector<int64_t>* shape, int64_t* elem_bytes);

}  // namespace ral
}  // namespace disc_b200
