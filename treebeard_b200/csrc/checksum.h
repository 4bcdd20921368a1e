// Checksum of the compiled-model file and of the packed image: catches truncated or edited
// files, not an integrity guarantee.  Large buffers (a packed forest is hundreds of megabytes)
// are hashed in 1 MiB blocks, word by word in four independent lanes, the blocks in parallel;
// the block hashes are then folded in order, so the result does not depend on the thread count.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <vector>

namespace tb {

constexpr uint64_t kHashSeed = 14695981039346656037ull;
constexpr uint64_t kHashPrime = 1099511628211ull;

inline uint64_t hash_small(uint64_t h, const unsigned char *p, size_t n) { // FNV-1a
  for (size_t i = 0; i < n; ++i) {
    h ^= p[i];
    h *= kHashPrime;
  }
  return h;
}

inline uint64_t hash_block(const unsigned char *p, size_t n) {
  uint64_t lane[4] = {kHashSeed, kHashSeed ^ 0x9e3779b97f4a7c15ull, kHashSeed ^ 0xc2b2ae3d27d4eb4full, kHashSeed ^ 0x165667b19e3779f9ull};
  size_t i = 0;
  for (; i + 32 <= n; i += 32) {
    uint64_t w[4];
    std::memcpy(w, p + i, 32);
    for (int k = 0; k < 4; ++k) lane[k] = (lane[k] ^ w[k]) * 0x9e3779b97f4a7c15ull;
  }
  uint64_t h = kHashSeed;
  for (int k = 0; k < 4; ++k) h = (h ^ lane[k] ^ (lane[k] >> 29)) * kHashPrime;
  return hash_small(h, p + i, n - i);
}

inline uint64_t hash_bytes(uint64_t h, const void *data, size_t n) {
  const unsigned char *p = static_cast<const unsigned char *>(data);
  constexpr size_t kBlock = 1u << 20;
  if (n < 4096) return hash_small(h, p, n);
  const size_t blocks = (n + kBlock - 1) / kBlock;
  std::vector<uint64_t> part(blocks);
#pragma omp parallel for schedule(static)
  for (long long b = 0; b < (long long)blocks; ++b) {
    const size_t at = (size_t)b * kBlock;
    part[b] = hash_block(p + at, n - at < kBlock ? n - at : kBlock);
  }
  for (size_t b = 0; b < blocks; ++b) h = (h ^ part[b]) * kHashPrime;
  return h;
}

} // namespace tb
