// Device-side building blocks shared by the sm_100a kernels: system-scope
// signalling between GPUs, bounded waits, vector reductions, and the views of
// the symmetric (peer-mapped) heap and of a hash-table shard.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <utility>

#include "../core/hash.h"
#include "../core/optim_math.h"
#include "../core/types.h"

namespace kb {
namespace cu {

constexpr int kMaxWorld = 16;

// Every rank allocates a heap with the same layout and maps all peers' heaps;
// a buffer is named by its byte offset, so `base[p] + off` is rank p's copy.
struct Sym {
  char* base[kMaxWorld];
  int rank;
  int world;
  template <typename T>
  __device__ __forceinline__ T* at(int peer, size_t off) const {
    return reinterpret_cast<T*>(base[peer] + off);
  }
};

// One hash-table shard (open addressing, linear probing, no tombstones: rows
// are never deleted on the training path; eviction rebuilds the table).
struct TableView {
  unsigned long long* keys;  // [cap], kEmptyKey = free
  float* val;                // [cap, dim]
  float* s[3];               // optimizer state slabs [cap, dim] or nullptr
  int* steps;                // [cap] or nullptr
  unsigned long long* lead;  // [cap] (push epoch << 32 | entry) or nullptr when world == 1
  int* size;                 // number of occupied slots
  int* status;               // first error code wins
  uint32_t bits;             // cap = 1 << bits
  int dim;
  InitPOD init;
  uint64_t seed_key;
};

__device__ __forceinline__ void set_status(int* status, int code) { atomicCAS(status, 0, code); }

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Spins until *flag >= want or `limit` polls have passed; false on give-up.
// Never an unbounded wait: a peer that does not show up costs `limit` polls,
// after which the caller records kTimeout and returns.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t want, uint32_t limit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - want) >= 0) return true;
    __nanosleep(it < 64 ? 32 : 256);
  }
  return false;
}

// Programmatic dependent launch.  A kernel launched through launch_pdl() may become resident while the
// kernel in front of it in the stream is still running: its blocks are scheduled once every block of that
// kernel has executed pdl_trigger(), and they run their prologue (barrier set-up, tensor-memory allocation,
// loads of data the predecessor does not write) until pdl_wait(), which returns when the predecessor has
// completed and its writes are visible.  Rule kept by every kernel here: pdl_trigger() comes AFTER the
// kernel's own pdl_wait(), so "predecessor complete" stays transitive along the stream.  Launched without
// the attribute both instructions do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
  pdl_wait();
  pdl_trigger();
}

// Vector float reduction into global memory (sm_90+): one 16-byte L2 atomic.
__device__ __forceinline__ void red_add_v4(float* addr, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

// Marks the calling block as finished; returns true in exactly one block: the
// last one of the grid to arrive.  All of the grid's earlier global / peer
// stores are then visible system-wide to whoever observes a later release store.
// One thread per block fences, after the block barrier: the barrier orders the
// block's stores before that thread, and its fence is cumulative over them.
__device__ __forceinline__ bool last_block_done(uint32_t* counter) {
  __shared__ bool is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t prev = atomicAdd(counter, 1u);
    is_last = (prev == gridDim.x - 1);
    if (is_last) {
      *counter = 0;
      __threadfence_system();
    }
  }
  __syncthreads();
  return is_last;
}

// Finds `id`; with insert=true claims a free slot (created = true: the caller must have
// the value row initialised before anyone reads it).  Returns the slot or -1 (absent / table full).
__device__ __forceinline__ int table_find_or_insert(const TableView& t, uint64_t id, bool insert, bool* created) {
  const uint64_t mask = (1ull << t.bits) - 1;
  uint64_t slot = SlotHash(id, t.bits);
  const uint32_t max_probe = t.bits >= 13 ? 8192u : (1u << t.bits);
  *created = false;
  for (uint32_t probe = 0; probe < max_probe; ++probe) {
    unsigned long long k = __ldcg(&t.keys[slot]);
    if (k == id) return static_cast<int>(slot);
    if (k == kEmptyKey) {
      if (!insert) return -1;
      const unsigned long long old = atomicCAS(&t.keys[slot], kEmptyKey, static_cast<unsigned long long>(id));
      if (old == kEmptyKey) {
        *created = true;
        return static_cast<int>(slot);
      }
      if (old == id) return static_cast<int>(slot);
    }
    slot = (slot + 1) & mask;
  }
  set_status(t.status, err::kTableFull);
  return -1;
}

// Adds `created` flags of the warp into the size counter with one atomic.
__device__ __forceinline__ void count_created(const TableView& t, bool created) {
  const unsigned m = __ballot_sync(__activemask(), created);
  if (created && (__ffs(m) - 1) == static_cast<int>(threadIdx.x & 31)) atomicAdd(t.size, __popc(m));
}

// Host side: launch with the programmatic-stream-serialization attribute (see pdl_wait above).  KRAKEN_PDL=0 in
// the environment turns it off (plain stream order), for comparison.
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("KRAKEN_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <typename... P, typename... A>
inline cudaError_t launch_pdl(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<A>(args)...);
}

}  // namespace cu
}  // namespace kb
