// Implementation of the allocation-free dedup entry point (see dedup_noalloc.h).
// The two kernels are the hash-set dedup of sparse.cu restated over one scratch
// block whose sub-buffers are carved out by offset.
#include "dedup_noalloc.h"

#include <cstdio>
#include <mutex>

#include "../core/hash.h"
#include "../core/types.h"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxWorld = 16;
constexpr int kMaxDevices = 64;
constexpr uint32_t kMaxSlots = 2u * KRAKEN_NOALLOC_MAX_IDS;  // 131072 hash slots
constexpr uint64_t kSalt = 0x5bd1e9955bd1e995ull;

// Layout inside the scratch block (all offsets multiples of 256 bytes).
constexpr size_t kOffKeys = 0;                                      // u64 [kMaxSlots]   1 MiB
constexpr size_t kOffPos = kOffKeys + sizeof(uint64_t) * kMaxSlots;  // i32 [kMaxSlots]   512 KiB
constexpr size_t kOffWin = kOffPos + sizeof(int) * kMaxSlots;        // i32 [kMaxSlots]   512 KiB
constexpr size_t kOffSlotOf = kOffWin + sizeof(int) * kMaxSlots;     // i32 [MAX_IDS]     256 KiB
constexpr size_t kOffCnt = kOffSlotOf + sizeof(int) * KRAKEN_NOALLOC_MAX_IDS;  // i32 [16]
constexpr size_t kUsed = kOffCnt + 256;
static_assert(kUsed <= KRAKEN_NOALLOC_SCRATCH_BYTES, "scratch block too small for its layout");

// The scratch itself.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is never passed to a kernel.
static __device__ __align__(256) unsigned char g_scratch[KRAKEN_NOALLOC_SCRATCH_BYTES];

__global__ void __launch_bounds__(kThreads)
noalloc_insert_kernel(const int64_t* __restrict__ ids, int n, int world, uint64_t salt, unsigned char* scratch,
                      uint32_t hbits, int* status) {
  unsigned long long* hkeys = reinterpret_cast<unsigned long long*>(scratch + kOffKeys);
  int* hpos = reinterpret_cast<int*>(scratch + kOffPos);
  int* hwin = reinterpret_cast<int*>(scratch + kOffWin);
  int* slot_of = reinterpret_cast<int*>(scratch + kOffSlotOf);
  int* cnt = reinterpret_cast<int*>(scratch + kOffCnt);
  __shared__ int s_cnt[kMaxWorld];
  __shared__ int s_base[kMaxWorld];
  if (threadIdx.x < kMaxWorld) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  bool won = false;
  int owner = 0, lpos = 0;
  uint64_t slot = 0;
  if (i < n) {
    uint64_t id = static_cast<uint64_t>(ids[i]);
    if (id == kb::kEmptyKey) {
      if (status) atomicCAS(status, 0, kb::err::kBadArgument);
      id = kb::kEmptyKey - 1;
    }
    const uint64_t mask = (1ull << hbits) - 1;
    slot = kb::SlotHash(id ^ kSalt, hbits);
    for (uint64_t probe = 0; probe <= mask; ++probe) {
      const unsigned long long k = __ldcg(&hkeys[slot]);
      if (k == id) break;
      if (k == kb::kEmptyKey) {
        const unsigned long long old = atomicCAS(&hkeys[slot], kb::kEmptyKey, static_cast<unsigned long long>(id));
        if (old == kb::kEmptyKey) {
          won = true;
          break;
        }
        if (old == id) break;
      }
      slot = (slot + 1) & mask;
    }
    slot_of[i] = static_cast<int>(slot);
    if (won) {
      owner = static_cast<int>(kb::OwnerOf(salt, id, world));
      lpos = atomicAdd(&s_cnt[owner], 1);
    }
  }
  __syncthreads();
  if (threadIdx.x < world && s_cnt[threadIdx.x] > 0)
    s_base[threadIdx.x] = atomicAdd(&cnt[threadIdx.x], s_cnt[threadIdx.x]);
  __syncthreads();
  if (won) {
    hpos[slot] = s_base[owner] + lpos;
    hwin[slot] = i;
  }
}

__global__ void __launch_bounds__(kThreads)
noalloc_finalize_kernel(const int64_t* __restrict__ ids, int n, int world, uint64_t salt,
                        const unsigned char* __restrict__ scratch, int* off, int64_t* uniq, int* inv) {
  const int* hpos = reinterpret_cast<const int*>(scratch + kOffPos);
  const int* hwin = reinterpret_cast<const int*>(scratch + kOffWin);
  const int* slot_of = reinterpret_cast<const int*>(scratch + kOffSlotOf);
  const int* cnt = reinterpret_cast<const int*>(scratch + kOffCnt);
  __shared__ int s_off[kMaxWorld + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int o = 0; o < world; ++o) {
      s_off[o] = acc;
      acc += cnt[o];
    }
    s_off[world] = acc;
    if (blockIdx.x == 0)
      for (int o = 0; o <= world; ++o) off[o] = s_off[o];
  }
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint64_t id = static_cast<uint64_t>(ids[i]);
  if (id == kb::kEmptyKey) id = kb::kEmptyKey - 1;
  const int slot = slot_of[i];
  const int u = s_off[kb::OwnerOf(salt, id, world)] + hpos[slot];
  inv[i] = u;
  if (hwin[slot] == i) uniq[u] = static_cast<int64_t>(id);
}

// Device address of g_scratch per device, resolved on the first call there.
std::mutex g_mu;
unsigned char* g_ptr[kMaxDevices] = {nullptr};

int fail(char* err, size_t err_len, int code, const char* msg, const char* detail = "") {
  if (err && err_len > 0) std::snprintf(err, err_len, "kraken_dedup_bucketize_noalloc: %s%s", msg, detail);
  return code;
}

}  // namespace

extern "C" int kraken_dedup_bucketize_noalloc(const int64_t* ids, int n, int world, uint64_t salt, int32_t* off,
                                              int64_t* uniq, int32_t* inv, int32_t* status, cudaStream_t stream,
                                              char* err, size_t err_len) {
  if (n < 0 || n > KRAKEN_NOALLOC_MAX_IDS) {
    char detail[96];
    std::snprintf(detail, sizeof(detail), " (n = %d, built-in scratch holds at most %d ids)", n, KRAKEN_NOALLOC_MAX_IDS);
    return fail(err, err_len, -1, "too many ids for the built-in scratch", detail);
  }
  if (world < 1 || world > kMaxWorld) return fail(err, err_len, -2, "world must be between 1 and 16");
  if (off == nullptr || (n > 0 && (ids == nullptr || uniq == nullptr || inv == nullptr)))
    return fail(err, err_len, -3, "null input or output pointer");

  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(err, err_len, -4, "cannot identify the current device: ", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) {
    char detail[64];
    std::snprintf(detail, sizeof(detail), " (ordinal %d, supported 0..%d)", dev, kMaxDevices - 1);
    return fail(err, err_len, -4, "device ordinal out of the supported range", detail);
  }
  unsigned char* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_ptr[dev] == nullptr) {
      // once per device, with that device current: the symbol's address on THIS device
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_scratch);
      if (e != cudaSuccess || p == nullptr)
        return fail(err, err_len, -4, "cudaGetSymbolAddress failed: ", cudaGetErrorString(e));
      g_ptr[dev] = static_cast<unsigned char*>(p);
    }
    scratch = g_ptr[dev];
  }

  // The array still holds the previous call's contents: empty the part of the hash set this
  // call will probe (all-ones = free) and zero the per-owner counters, in stream order.
  uint32_t hbits = 4;
  while ((1u << hbits) < 2u * static_cast<uint32_t>(n > 0 ? n : 1)) ++hbits;
  e = cudaMemsetAsync(scratch + kOffKeys, 0xFF, sizeof(uint64_t) << hbits, stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(scratch + kOffCnt, 0, sizeof(int) * kMaxWorld, stream);
  if (e != cudaSuccess) return fail(err, err_len, -4, "cudaMemsetAsync failed: ", cudaGetErrorString(e));
  if (n == 0) {
    e = cudaMemsetAsync(off, 0, sizeof(int32_t) * (world + 1), stream);
    return e == cudaSuccess ? 0 : fail(err, err_len, -4, "cudaMemsetAsync failed: ", cudaGetErrorString(e));
  }
  const int blocks = (n + kThreads - 1) / kThreads;
  // cudaPeekAtLastError right after each launch reports that launch's configuration errors; a sticky
  // error left by earlier, unrelated asynchronous work shows up here too, hence the wording.
  noalloc_insert_kernel<<<blocks, kThreads, 0, stream>>>(ids, n, world, salt, scratch, hbits, status);
  e = cudaPeekAtLastError();
  if (e == cudaSuccess) {
    noalloc_finalize_kernel<<<blocks, kThreads, 0, stream>>>(ids, n, world, salt, scratch, off, uniq, inv);
    e = cudaPeekAtLastError();
  }
  if (e != cudaSuccess)
    return fail(err, err_len, -4, "CUDA reported an error at kernel launch (this launch, or earlier work on the context): ",
                cudaGetErrorString(e));
  return 0;
}
