// Maintenance kernels of a hash-table shard: clear, bulk import (checkpoint
// load, rehash, resharding receive), lookup without insert, and filtered
// export (checkpoint save, rehash, resharding send, eviction).
//
// The reference walks its skip lists on the host for all of these
// (kraken/ps/ps.cc:60-118,236-333; kraken/checkpoint/checkpoint.cc:494-507,628-646);
// here a full-table scan is one pass over the key array at HBM speed.
#include "common.cuh"
#include "kernels.h"

namespace kb {
namespace cu {

namespace {

constexpr int kThreads = 256;

TableView to_view(const TableHost& h) {
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

__global__ void table_clear_kernel(TableView t) {
  const uint64_t cap = 1ull << t.bits;
  for (uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; i < cap;
       i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
    t.keys[i] = kEmptyKey;
    if (t.steps) t.steps[i] = 0;
    if (t.lead) t.lead[i] = 0;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) *t.size = 0;
}

__global__ void table_import_kernel(TableView t, const int64_t* __restrict__ ids, const float* __restrict__ vals,
                                    const float* __restrict__ s0, const float* __restrict__ s1,
                                    const float* __restrict__ s2, const int* __restrict__ steps, int n) {
  for (int base = blockIdx.x * blockDim.x; base < n; base += gridDim.x * blockDim.x) {
    const int i = base + threadIdx.x;
    bool created = false;
    if (i < n) {
      const uint64_t id = static_cast<uint64_t>(ids[i]);
      // find-or-claim without running the initializer: the row is overwritten below
      const uint64_t mask = (1ull << t.bits) - 1;
      uint64_t slot = SlotHash(id, t.bits);
      int found = -1;
      const uint32_t max_probe = t.bits >= 13 ? 8192u : (1u << t.bits);
      for (uint32_t p = 0; p < max_probe && found < 0; ++p) {
        const unsigned long long k = __ldcg(&t.keys[slot]);
        if (k == id) {
          found = static_cast<int>(slot);
        } else if (k == kEmptyKey) {
          const unsigned long long old = atomicCAS(&t.keys[slot], kEmptyKey, static_cast<unsigned long long>(id));
          if (old == kEmptyKey) {
            created = true;
            found = static_cast<int>(slot);
          } else if (old == id) {
            found = static_cast<int>(slot);
          }
        }
        if (found < 0) slot = (slot + 1) & mask;
      }
      if (found < 0) {
        set_status(t.status, err::kTableFull);
      } else {
        const size_t dst = static_cast<size_t>(found) * t.dim, src = static_cast<size_t>(i) * t.dim;
        for (int j = 0; j < t.dim; ++j) {
          t.val[dst + j] = vals[src + j];
          if (t.s[0] && s0) t.s[0][dst + j] = s0[src + j];
          if (t.s[1] && s1) t.s[1][dst + j] = s1[src + j];
          if (t.s[2] && s2) t.s[2][dst + j] = s2[src + j];
        }
        if (t.steps && steps) t.steps[found] = steps[i];
      }
    }
    count_created(t, created);
  }
}

__global__ void table_lookup_kernel(TableView t, const int64_t* __restrict__ ids, int n, float* rows, uint8_t* found) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  bool created;
  const int slot = table_find_or_insert(t, static_cast<uint64_t>(ids[i]), false, &created);
  found[i] = slot >= 0;
  for (int j = 0; j < t.dim; ++j)
    rows[static_cast<size_t>(i) * t.dim + j] = slot >= 0 ? t.val[static_cast<size_t>(slot) * t.dim + j] : 0.f;
}

__global__ void table_export_kernel(TableView t, int filter_mode, uint64_t salt, int world, int rank, int min_steps,
                                    int64_t* out_ids, float* out_vals, float* out_s0, float* out_s1, float* out_s2,
                                    int* out_steps, int* out_count, int out_cap) {
  const uint64_t cap = 1ull << t.bits;
  for (uint64_t base = blockIdx.x * static_cast<uint64_t>(blockDim.x); base < cap;
       base += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
    const uint64_t slot = base + threadIdx.x;
    bool take = false;
    unsigned long long k = kEmptyKey;
    if (slot < cap) {
      k = t.keys[slot];
      if (k != kEmptyKey) {
        switch (filter_mode) {
          case 1: take = static_cast<int>(OwnerOf(salt, k, world)) == rank; break;
          case 2: take = static_cast<int>(OwnerOf(salt, k, world)) != rank; break;
          case 3: take = t.steps ? t.steps[slot] >= min_steps : true; break;
          case 4: take = static_cast<int>(k % static_cast<unsigned long long>(world)) == rank; break;  // id % world == rank
          default: take = true;
        }
      }
    }
    // one atomic per warp, then lane-ranked positions
    const unsigned m = __ballot_sync(0xffffffffu, take);
    int warp_base = 0;
    const int lane = threadIdx.x & 31;
    if (m != 0 && lane == __ffs(m) - 1) warp_base = atomicAdd(out_count, __popc(m));
    warp_base = __shfl_sync(0xffffffffu, warp_base, m ? __ffs(m) - 1 : 0);
    if (take) {
      const int pos = warp_base + __popc(m & ((1u << lane) - 1));
      if (pos < out_cap) {
        out_ids[pos] = static_cast<int64_t>(k);
        const size_t src = slot * t.dim, dst = static_cast<size_t>(pos) * t.dim;
        for (int j = 0; j < t.dim; ++j) {
          out_vals[dst + j] = t.val[src + j];
          if (out_s0 && t.s[0]) out_s0[dst + j] = t.s[0][src + j];
          if (out_s1 && t.s[1]) out_s1[dst + j] = t.s[1][src + j];
          if (out_s2 && t.s[2]) out_s2[dst + j] = t.s[2][src + j];
        }
        if (out_steps) out_steps[pos] = t.steps ? t.steps[slot] : 0;
      }
    }
  }
}

__global__ void owner_of_kernel(const int64_t* __restrict__ ids, int n, uint64_t salt, int world, int* owners) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) owners[i] = static_cast<int>(OwnerOf(salt, static_cast<uint64_t>(ids[i]), world));
}

}  // namespace

void owner_of(const int64_t* ids, int n, uint64_t salt, int world, int* owners, cudaStream_t stream) {
  if (n <= 0) return;
  owner_of_kernel<<<(n + kThreads - 1) / kThreads, kThreads, 0, stream>>>(ids, n, salt, world, owners);
}

void table_clear(TableHost table, cudaStream_t stream) {
  table_clear_kernel<<<148 * 4, kThreads, 0, stream>>>(to_view(table));
}

void table_import(TableHost table, const int64_t* ids, const float* vals, const float* s0, const float* s1,
                  const float* s2, const int* steps, int n, cudaStream_t stream) {
  if (n <= 0) return;
  int grid = (n + kThreads - 1) / kThreads;
  if (grid > 148 * 8) grid = 148 * 8;
  table_import_kernel<<<grid, kThreads, 0, stream>>>(to_view(table), ids, vals, s0, s1, s2, steps, n);
}

void table_lookup(TableHost table, const int64_t* ids, int n, float* rows, uint8_t* found, cudaStream_t stream) {
  if (n <= 0) return;
  table_lookup_kernel<<<(n + kThreads - 1) / kThreads, kThreads, 0, stream>>>(to_view(table), ids, n, rows, found);
}

void table_export(TableHost table, int filter_mode, uint64_t salt, int world, int rank, int min_steps,
                  int64_t* out_ids, float* out_vals, float* out_s0, float* out_s1, float* out_s2, int* out_steps,
                  int* out_count, int out_cap, cudaStream_t stream) {
  cudaMemsetAsync(out_count, 0, sizeof(int), stream);
  table_export_kernel<<<148 * 8, kThreads, 0, stream>>>(to_view(table), filter_mode, salt, world, rank, min_steps,
                                                        out_ids, out_vals, out_s0, out_s1, out_s2, out_steps, out_count,
                                                        out_cap);
}

}  // namespace cu
}  // namespace kb
