// Pieces shared by the single-table exchange kernels (sparse.cu) and the multi-table ones
// (sparse_group.cu): geometry of row-parallel loops, 16-byte / 4-byte vector accessors, the views
// built from host-side descriptors, and the entry format of the dedup scratch set.
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace kb {
namespace cu {
namespace sparse_detail {

constexpr int kThreads = 256;
constexpr uint64_t kDedupSalt = 0x5bd1e9955bd1e995ull;

inline Sym to_sym(const SymHost& h) {
  Sym s;
  for (int i = 0; i < kMaxWorld; ++i) s.base[i] = static_cast<char*>(h.base[i]);
  s.rank = h.rank;
  s.world = h.world;
  return s;
}

inline TableView to_view(const TableHost& h) {
  TableView t;
  t.keys = static_cast<unsigned long long*>(h.keys);
  t.val = h.val;
  for (int i = 0; i < 3; ++i) t.s[i] = h.s[i];
  t.steps = h.steps;
  t.lead = static_cast<unsigned long long*>(h.lead);
  t.size = h.size;
  t.status = h.status;
  t.bits = h.bits;
  t.dim = h.dim;
  t.init = h.init;
  t.seed_key = h.seed_key;
  return t;
}

inline int grid_for(long long work_items, int per_block = kThreads, int cap = 148 * 8) {
  long long g = (work_items + per_block - 1) / per_block;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return static_cast<int>(g);
}

// Row-parallel geometry: a row of `dim` floats is handled by `lpr` adjacent
// lanes (a power of two <= 32), each moving VEC floats per chunk.
struct RowGeom {
  int vec;     // 4 or 1
  int chunks;  // dim / vec
  int lpr;     // lanes per row
};

inline RowGeom row_geom(int dim) {
  RowGeom g;
  g.vec = (dim % 4 == 0) ? 4 : 1;
  g.chunks = dim / g.vec;
  int l = 1;
  while (l < g.chunks && l < 32) l <<= 1;
  g.lpr = l;
  return g;
}

template <int VEC>
struct Vec;
template <>
struct Vec<4> {
  using T = float4;
  static __device__ __forceinline__ T ldcg(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
  static __device__ __forceinline__ T ld(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void st(float* p, T v) { *reinterpret_cast<float4*>(p) = v; }
  static __device__ __forceinline__ void red(float* p, T v) { red_add_v4(p, v); }
  static __device__ __forceinline__ T zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  static __device__ __forceinline__ T fill(float x) { return make_float4(x, x, x, x); }
  static __device__ __forceinline__ void fma(T& a, float w, T b) {
    a.x += w * b.x;
    a.y += w * b.y;
    a.z += w * b.z;
    a.w += w * b.w;
  }
  static __device__ __forceinline__ T scale(T a, float w) { return make_float4(a.x * w, a.y * w, a.z * w, a.w * w); }
};
template <>
struct Vec<1> {
  using T = float;
  static __device__ __forceinline__ T ldcg(const float* p) { return __ldcg(p); }
  static __device__ __forceinline__ T ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, T v) { *p = v; }
  static __device__ __forceinline__ void red(float* p, T v) { atomicAdd(p, v); }
  static __device__ __forceinline__ T zero() { return 0.f; }
  static __device__ __forceinline__ T fill(float x) { return x; }
  static __device__ __forceinline__ void fma(T& a, float w, T b) { a += w * b; }
  static __device__ __forceinline__ T scale(T a, float w) { return a * w; }
};


// The scratch hash set of the dedup is an array of 16-byte entries {key, pos | win << 32}: the key that the probe
// compares, and - in the same 32-byte sector - the rank of the unique id inside its owner group and
// the index of the occurrence that inserted it.  An insert and the later finalize therefore touch one
// random sector per id each instead of three separate arrays.
struct DedupEntry {
  unsigned long long key;
  unsigned long long pos_win;
};

// Owner of unique entry u given the exclusive scan of the per-owner counts.
__device__ __forceinline__ int owner_of_index(const int* s_off, int world, int u) {
  int o = 0;
  while (o + 1 < world && u >= s_off[o + 1]) ++o;
  return o;
}

}  // namespace sparse_detail
}  // namespace cu
}  // namespace kb
