#include "safetensors.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <stdexcept>

#include "json_min.h"

namespace kvcm {

int safetensors_dtype_size(const std::string& d) {
  if (d == "F64" || d == "I64" || d == "U64") return 8;
  if (d == "F32" || d == "I32" || d == "U32") return 4;
  if (d == "BF16" || d == "F16" || d == "I16" || d == "U16") return 2;
  if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
  return 0;
}

namespace {

struct Fd {
  int fd = -1;
  ~Fd() { if (fd >= 0) ::close(fd); }
};

std::string shape_text(const std::vector<long long>& shape) {
  std::string s = "[";
  for (size_t i = 0; i < shape.size(); ++i) s += (i ? ", " : "") + std::to_string(shape[i]);
  return s + "]";
}

}  // namespace

SafetensorsReader::SafetensorsReader(const std::string& path) : path_(path) {
  Fd f;
  f.fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
  if (f.fd < 0) throw std::runtime_error("cannot open '" + path + "': " + std::strerror(errno));
  struct stat st;
  if (::fstat(f.fd, &st) != 0) throw std::runtime_error("cannot stat '" + path + "': " + std::strerror(errno));
  const long long size = static_cast<long long>(st.st_size);
  if (size < 8) throw std::runtime_error(path + ": truncated (no header length)");
  unsigned char head[8];
  if (::pread(f.fd, head, 8, 0) != 8) throw std::runtime_error(path + ": truncated (no header length)");
  unsigned long long n = 0;
  for (int i = 7; i >= 0; --i) n = (n << 8) | head[i];
  if (n > static_cast<unsigned long long>(size - 8) || n > (100ull << 20))
    throw std::runtime_error(path + ": header length " + std::to_string(n) + " does not fit the file (" +
                             std::to_string(size) + " bytes)");
  map_len_ = static_cast<size_t>(size);
  void* m = ::mmap(nullptr, map_len_, PROT_READ, MAP_PRIVATE, f.fd, 0);
  if (m == MAP_FAILED) {
    map_len_ = 0;
    throw std::runtime_error("cannot map '" + path + "': " + std::strerror(errno));
  }
  map_ = static_cast<unsigned char*>(m);
  data_start_ = 8 + static_cast<long long>(n);
  data_len_ = size - data_start_;

  json::Value header;
  try {
    header = json::Parser(reinterpret_cast<const char*>(map_ + 8), static_cast<size_t>(n)).parse_document();
  } catch (const std::runtime_error& e) {
    throw std::runtime_error(path + ": header is not valid JSON (" + e.what() + ")");
  }
  if (header.kind != json::Value::Object) throw std::runtime_error(path + ": header must be a JSON object");
  for (const auto& member : header.members) {
    const std::string& name = member.first;
    const json::Value& e = member.second;
    if (name == "__metadata__") {
      if (e.kind == json::Value::Object)
        for (const auto& kv : e.members)
          if (kv.second.kind == json::Value::String) metadata_.emplace_back(kv.first, kv.second.text);
      continue;
    }
    SafetensorsEntry out;
    const json::Value* dt = e.kind == json::Value::Object ? e.find("dtype") : nullptr;
    const json::Value* sh = e.kind == json::Value::Object ? e.find("shape") : nullptr;
    const json::Value* off = e.kind == json::Value::Object ? e.find("data_offsets") : nullptr;
    bool ok = dt && dt->kind == json::Value::String && sh && sh->kind == json::Value::Array && off &&
              off->kind == json::Value::Array && off->items.size() == 2;
    const int isz = ok ? safetensors_dtype_size(dt->text) : 0;
    ok = ok && isz > 0;
    if (ok) {
      out.dtype = dt->text;
      for (const auto& d : sh->items) {
        if (d.kind != json::Value::Number || !d.is_integer || d.integer < 0) { ok = false; break; }
        out.shape.push_back(d.integer);
      }
      for (const auto& d : off->items)
        if (d.kind != json::Value::Number || !d.is_integer) ok = false;
    }
    if (!ok) throw std::runtime_error(path + ": bad header entry for '" + name + "'");
    out.begin = off->items[0].integer;
    out.end = off->items[1].integer;
    // Products are checked: a header like [2^32, 2^32, k] must not wrap round to a size that fits.
    long long numel = 1;
    bool overflow = false;
    for (long long d : out.shape) {
      if (d < 0 || __builtin_mul_overflow(numel, d, &numel)) overflow = true;
    }
    long long need = 0;
    if (!overflow && __builtin_mul_overflow(numel, static_cast<long long>(isz), &need)) overflow = true;
    if (overflow)
      throw std::runtime_error(path + ": tensor '" + name + "' has a shape " + shape_text(out.shape) +
                               " whose size does not fit 63 bits");
    if (out.begin < 0 || out.end < out.begin || out.end > data_len_)
      throw std::runtime_error(path + ": tensor '" + name + "' data_offsets [" + std::to_string(out.begin) + ", " +
                               std::to_string(out.end) + ") lie outside the data section of " +
                               std::to_string(data_len_) + " bytes (file truncated?)");
    if (out.end - out.begin != need)
      throw std::runtime_error(path + ": tensor '" + name + "' has " + std::to_string(out.end - out.begin) +
                               " bytes but shape " + shape_text(out.shape) + " of " + out.dtype + " needs " +
                               std::to_string(need));
    if (entries_.count(name))
      throw std::runtime_error(path + ": tensor name '" + name + "' appears twice in the header");
    names_.push_back(name);
    entries_[name] = std::move(out);
  }
}

SafetensorsReader::~SafetensorsReader() {
  if (map_ && map_len_) ::munmap(map_, map_len_);
}

const SafetensorsEntry& SafetensorsReader::entry(const std::string& name) const {
  auto it = entries_.find(name);
  if (it == entries_.end()) throw std::out_of_range(path_ + ": no tensor '" + name + "'");
  return it->second;
}

std::uintptr_t SafetensorsReader::address(const std::string& name) const {
  const SafetensorsEntry& e = entry(name);
  return reinterpret_cast<std::uintptr_t>(map_ + data_start_ + e.begin);
}

}  // namespace kvcm
