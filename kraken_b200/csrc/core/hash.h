// 64-bit mixers shared by host and device code.
//
// Mix64 reproduces the reference's utils::Hash bit for bit
// (kraken/common/utils.h:30-48); checkpoints written by either side place a
// row on the ring by Mix64(table_id) ^ Mix64(sparse_id), so the constants are
// frozen.  SlotHash is this framework's own second mixer: it decorrelates the
// hash-table slot from the owner choice, which uses Mix64 directly.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define KB_HD __host__ __device__ __forceinline__
#else
#define KB_HD inline
#endif

namespace kb {

KB_HD uint64_t Mix64(uint64_t v) {
  v = v * 3935559000370003845ull + 2691343689449507681ull;
  v ^= v >> 21;
  v ^= v << 37;
  v ^= v >> 4;
  v *= 4768777513237032717ull;
  v ^= v << 20;
  v ^= v >> 41;
  v ^= v << 5;
  return v;
}

KB_HD uint64_t Mix64(uint64_t a, uint64_t b) { return Mix64(a) ^ Mix64(b); }

// Owner rank of (table, id) among `world` GPU shards.
KB_HD uint32_t OwnerOf(uint64_t table_salt, uint64_t id, uint32_t world) {
  return static_cast<uint32_t>((table_salt ^ Mix64(id)) % world);
}

// Multiplicative (Fibonacci) slot hash into a table of 2^bits slots.
KB_HD uint64_t SlotHash(uint64_t key, uint32_t bits) {
  uint64_t h = (key ^ (key >> 32)) * 0x9E3779B97F4A7C15ull;
  h ^= h >> 29;
  h *= 0xBF58476D1CE4E5B9ull;
  return h >> (64 - bits);
}

// Philox key for the initial values of a table's rows.
KB_HD uint64_t SeedKey(uint64_t seed, uint64_t table_id) {
  return Mix64(seed * 0x9E3779B97F4A7C15ull + table_id + 1);
}

// Salt mixed into OwnerOf so different tables spread the same id differently.
KB_HD uint64_t TableSalt(uint64_t table_id) { return Mix64(table_id); }

constexpr uint64_t kEmptyKey = 0xFFFFFFFFFFFFFFFFull;  // reserved: never a valid row id

}  // namespace kb
