// 64-bit xxHash (the public XXH64 algorithm) over a byte range, and the chained page hash
// built on it:  h_i = XXH64(bytes of page i's int32 token ids, seed = h_{i-1}),  h_{-1} = 0.
// Same chain as the reference (src/core/hash.h:29-73) so that page identities agree with it.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>

namespace kvcm {

class XXH64 {
 public:
  static uint64_t digest(const void* data, size_t len, uint64_t seed) {
    const unsigned char* cur = static_cast<const unsigned char*>(data);
    const unsigned char* const stop = cur + len;
    uint64_t acc;
    if (len >= 32) {
      uint64_t lane[4] = {seed + kA + kB, seed + kB, seed, seed - kA};
      for (; stop - cur >= 32; cur += 32)
        for (int i = 0; i < 4; ++i) lane[i] = mix(lane[i], load64(cur + 8 * i));
      acc = rot(lane[0], 1) + rot(lane[1], 7) + rot(lane[2], 12) + rot(lane[3], 18);
      for (int i = 0; i < 4; ++i) acc = (acc ^ mix(0, lane[i])) * kA + kD;
    } else {
      acc = seed + kE;
    }
    acc += static_cast<uint64_t>(len);
    for (; stop - cur >= 8; cur += 8) acc = rot(acc ^ mix(0, load64(cur)), 27) * kA + kD;
    if (stop - cur >= 4) {
      acc = rot(acc ^ (static_cast<uint64_t>(load32(cur)) * kA), 23) * kB + kC;
      cur += 4;
    }
    for (; cur < stop; ++cur) acc = rot(acc ^ (static_cast<uint64_t>(*cur) * kE), 11) * kA;
    acc = (acc ^ (acc >> 33)) * kB;
    acc = (acc ^ (acc >> 29)) * kC;
    return acc ^ (acc >> 32);
  }

 private:
  static constexpr uint64_t kA = 0x9E3779B185EBCA87ULL, kB = 0xC2B2AE3D27D4EB4FULL,
                            kC = 0x165667B19E3779F9ULL, kD = 0x85EBCA77C2B2AE63ULL,
                            kE = 0x27D4EB2F165667C5ULL;
  static uint64_t rot(uint64_t v, int s) { return (v << s) | (v >> (64 - s)); }
  static uint64_t mix(uint64_t acc, uint64_t word) { return rot(acc + word * kB, 31) * kA; }
  static uint64_t load64(const unsigned char* p) { uint64_t v; std::memcpy(&v, p, 8); return v; }
  static uint32_t load32(const unsigned char* p) { uint32_t v; std::memcpy(&v, p, 4); return v; }
};

inline uint64_t page_hash(uint64_t parent, const int32_t* tokens, int count) {
  return XXH64::digest(tokens, sizeof(int32_t) * static_cast<size_t>(count), parent);
}

}  // namespace kvcm
