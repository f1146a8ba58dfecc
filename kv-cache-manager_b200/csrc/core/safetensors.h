// Reader of the safetensors container, against the file format itself:
//     8 bytes  little-endian u64  N = length of the JSON header
//     N bytes  JSON {"name": {"dtype": "BF16", "shape": [..], "data_offsets": [begin, end]}, ...,
//                    "__metadata__": {...}}
//     rest     raw little-endian tensor bytes; offsets count from the end of the header
// The file is memory-mapped read-only; a tensor is an address inside the map.  The reference
// reads a private flat binary in C++ (src/model/weights.cpp:24-83); reading the public container
// by tensor name replaces its Python export step (tools/export_weights.py:58-85).
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

namespace kvcm {

struct SafetensorsEntry {
  std::string dtype;                 // "F32", "BF16", ...
  std::vector<long long> shape;
  long long begin = 0, end = 0;      // byte range in the data section
};

// Bytes of one element of a dtype name; 0 = unknown.
int safetensors_dtype_size(const std::string& dtype);

class SafetensorsReader {
 public:
  explicit SafetensorsReader(const std::string& path);     // throws std::runtime_error with the file's fault
  ~SafetensorsReader();
  SafetensorsReader(const SafetensorsReader&) = delete;
  SafetensorsReader& operator=(const SafetensorsReader&) = delete;

  const std::string& path() const { return path_; }
  const std::vector<std::string>& names() const { return names_; }          // in header order
  const SafetensorsEntry& entry(const std::string& name) const;             // throws std::out_of_range
  bool has(const std::string& name) const { return entries_.count(name) != 0; }
  const std::vector<std::pair<std::string, std::string>>& metadata() const { return metadata_; }
  // Address of the tensor's first byte inside the map (valid while this object lives).
  std::uintptr_t address(const std::string& name) const;
  long long data_bytes() const { return data_len_; }

 private:
  std::string path_;
  std::vector<std::string> names_;
  std::map<std::string, SafetensorsEntry> entries_;
  std::vector<std::pair<std::string, std::string>> metadata_;
  unsigned char* map_ = nullptr;
  size_t map_len_ = 0;
  long long data_start_ = 0, data_len_ = 0;
};

}  // namespace kvcm
