#include "metadata.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>

namespace disc_b200 {
namespace ral {
namespace {

// Bounded cursor over the mapping: every read checks what is left.
struct Cursor {
  const char* p;
  size_t left;
  template <typename T>
  bool read(T* v) {
    if (left < sizeof(T)) return false;
    std::memcpy(v, p, sizeof(T));
    p += sizeof(T);
    left -= sizeof(T);
    return true;
  }
  bool read_view(std::string_view* v) {
    size_t n = 0;
    if (!read(&n) || n > left) return false;
    *v = std::string_view(p, n);
    p += n;
    left -= n;
    return true;
  }
};

int hex_digit(char c) {
  if (c >= '0' && c <= '9') return c - '0';
  if (c >= 'a' && c <= 'f') return c - 'a' + 10;
  if (c >= 'A' && c <= 'F') return c - 'A' + 10;
  return -1;
}

}  // namespace

std::unique_ptr<MetadataFile> MetadataFile::load(const std::string& path, std::string* error) {
  auto fail = [&](const std::string& why) -> std::unique_ptr<MetadataFile> {
    if (error) *error = "metadata file " + path + ": " + why;
    return nullptr;
  };
  const int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) return fail("cannot open");
  struct stat st;
  if (::fstat(fd, &st) != 0 || st.st_size < static_cast<off_t>(sizeof(uint64_t) + sizeof(size_t))) {
    ::close(fd);
    return fail("too short");
  }
  void* map = ::mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (map == MAP_FAILED) return fail("mmap failed");
  std::unique_ptr<MetadataFile> f(new MetadataFile);
  f->map_ = map;
  f->bytes_ = static_cast<size_t>(st.st_size);
  const char* base = static_cast<const char*>(map);
  uint64_t magic = 0;
  std::memcpy(&magic, base, sizeof(magic));
  if (magic != kMetadataMagic) return fail("bad magic number");
  size_t count = 0;
  std::memcpy(&count, base + f->bytes_ - sizeof(size_t), sizeof(size_t));
  Cursor cur{base + sizeof(uint64_t), f->bytes_ - sizeof(uint64_t) - sizeof(size_t)};
  for (size_t i = 0; i < count; ++i) {
    bool is_host = false;
    std::string_view key, value;
    if (!cur.read(&is_host) || !cur.read_view(&key) || !cur.read_view(&value)) return fail("truncated entry");
    (is_host ? f->host_ : f->device_).emplace(std::string(key), value);
  }
  return f;
}

MetadataFile::~MetadataFile() {
  if (map_) ::munmap(map_, bytes_);
}

std::string_view MetadataFile::host_constant(const std::string& name) const {
  auto it = host_.find(name);
  return it == host_.end() ? std::string_view() : it->second;
}

std::string_view MetadataFile::device_constant(const std::string& name) const {
  auto it = device_.find(name);
  return it == device_.end() ? std::string_view() : it->second;
}

bool MetadataFile::release(std::unordered_map<std::string, std::string_view>* map, const std::string& name) {
  auto it = map->find(name);
  if (it == map->end()) return false;
  // whole pages inside the value go back to the system; the mapping itself stays
  const long page = ::sysconf(_SC_PAGESIZE);
  if (page > 0 && it->second.size() >= static_cast<size_t>(2 * page)) {
    const uintptr_t b = reinterpret_cast<uintptr_t>(it->second.data());
    const uintptr_t lo = (b + page - 1) / page * page;
    const uintptr_t hi = (b + it->second.size()) / page * page;
    if (hi > lo) ::madvise(reinterpret_cast<void*>(lo), hi - lo, MADV_DONTNEED);
  }
  map->erase(it);
  return true;
}

bool MetadataFile::release_host(const std::string& name) { return release(&host_, name); }
bool MetadataFile::release_device(const std::string& name) { return release(&device_, name); }

MetadataWriter::MetadataWriter(const std::string& path) {
  FILE* f = std::fopen(path.c_str(), "wb");
  if (f && std::fwrite(&kMetadataMagic, sizeof(kMetadataMagic), 1, f) != 1) {
    std::fclose(f);
    f = nullptr;
  }
  file_ = f;
}

MetadataWriter::~MetadataWriter() {
  if (file_) std::fclose(static_cast<FILE*>(file_));
}

bool MetadataWriter::add(const std::string& name, bool is_host, const void* data, size_t bytes) {
  FILE* f = static_cast<FILE*>(file_);
  if (!f || !seen_.emplace(name + (is_host ? "#h" : "#d"), true).second) return false;
  static const char kDigits[] = "0123456789ABCDEF";
  std::string hex(bytes * 2, '0');
  const uint8_t* b = static_cast<const uint8_t*>(data);
  for (size_t i = 0; i < bytes; ++i) {
    hex[2 * i] = kDigits[b[i] >> 4];
    hex[2 * i + 1] = kDigits[b[i] & 15];
  }
  const size_t klen = name.size(), vlen = hex.size();
  const bool ok = std::fwrite(&is_host, sizeof(bool), 1, f) == 1 && std::fwrite(&klen, sizeof(klen), 1, f) == 1 &&
                  std::fwrite(name.data(), 1, klen, f) == klen && std::fwrite(&vlen, sizeof(vlen), 1, f) == 1 &&
                  std::fwrite(hex.data(), 1, vlen, f) == vlen;
  if (ok) ++count_;
  return ok;
}

bool MetadataWriter::finish() {
  FILE* f = static_cast<FILE*>(file_);
  if (!f) return false;
  const bool ok = std::fwrite(&count_, sizeof(count_), 1, f) == 1;
  const bool closed = std::fclose(f) == 0;
  file_ = nullptr;
  return ok && closed;
}

bool decode_hex(std::string_view hex, std::vector<uint8_t>* out) {
  out->clear();
  out->reserve((hex.size() + 1) / 2);
  size_t i = 0;
  if (hex.size() % 2 == 1) {
    const int d = hex_digit(hex[0]);
    if (d < 0) return false;
    out->push_back(static_cast<uint8_t>(d));
    i = 1;
  }
  for (; i < hex.size(); i += 2) {  // an even number of digits is left
    const int hi = hex_digit(hex[i]), lo = hex_digit(hex[i + 1]);
    if (hi < 0 || lo < 0) return false;
    out->push_back(static_cast<uint8_t>((hi << 4) | lo));
  }
  return true;
}

bool parse_const_name(const std::string& name, std::vector<int64_t>* shape, int64_t* elem_bytes) {
  const size_t a = name.find('_');
  if (a == std::string::npos) return false;
  const size_t b = name.find('_', a + 1);
  if (b == std::string::npos || name.find('_', b + 1) != std::string::npos) return false;
  const std::string tag = name.substr(a + 1, b - a - 1);
  const std::string dims = name.substr(b + 1);
  if (tag.size() < 2) return false;
  int64_t bits = 0;
  size_t first = 1;  // the width follows the letter(s) of the tag: i8, f32, ui8, bf16
  while (first < tag.size() && (tag[first] < '0' || tag[first] > '9')) ++first;
  if (first == tag.size()) return false;
  for (size_t i = first; i < tag.size(); ++i) {
    if (tag[i] < '0' || tag[i] > '9') return false;
    bits = bits * 10 + (tag[i] - '0');
    if (bits > 1024) return false;
  }
  *elem_bytes = bits / 8 < 1 ? 1 : bits / 8;
  shape->clear();
  size_t pos = 0;
  while (pos < dims.size()) {
    size_t x = dims.find('x', pos);
    if (x == std::string::npos) x = dims.size();
    if (x == pos) return false;
    int64_t d = 0;
    for (size_t i = pos; i < x; ++i) {
      if (dims[i] < '0' || dims[i] > '9') return false;
      d = d * 10 + (dims[i] - '0');
      if (d > (int64_t{1} << 40)) return false;
    }
    shape->push_back(d);
    pos = x + 1;
    if (x + 1 == dims.size()) return false;  // trailing 'x'
  }
  return true;
}

}  // namespace ral
}  // namespace disc_b200
