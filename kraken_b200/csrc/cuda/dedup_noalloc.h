// Allocation-free entry point for id dedup + bucketing by owner.
//
// This entry point has no counterpart in the reference (its client dedups ids
// on the host with an unordered_map, kraken/worker/emitter.cc:139-149).  It
// exists for callers that may not allocate device memory at the point where
// they need the operation: code that runs while a memory pool is frozen or its
// budget is fully committed (an inference server that hands all HBM to its
// tables and activations up front), and plain-C or ctypes hosts that drive the
// library without torch's allocator.  Every other launcher in this library
// receives its scratch from the caller; this one keeps its scratch inside the
// library image instead.
//
// What it computes is exactly dedup_bucketize of kernels.h: the unique ids of
// `ids`, grouped by owner rank (OwnerOf(salt, id, world)), with the map from
// every occurrence to its unique id.
//
// Scratch: a file-scope static __device__ array of KRAKEN_NOALLOC_SCRATCH_BYTES
// bytes (hash set for 2 * KRAKEN_NOALLOC_MAX_IDS keys, slot bookkeeping,
// per-owner counters).  Every GPU that loads the library's device code holds that
// array until the process exits.  With CUDA's default lazy module loading the
// device code, and with it the array, is placed on a GPU at the library's first
// use there, not at dlopen time: a caller that hands out all remaining device
// memory afterwards must make its first call on each GPU BEFORE it commits that
// memory, or the load itself can fail for lack of room.
//
// Rules for callers:
//   * n must be <= KRAKEN_NOALLOC_MAX_IDS and 1 <= world <= 16; anything else is
//     refused with a negative return code and a message, nothing is launched.
//   * The FIRST call on a device resolves the array's device address
//     (cudaGetSymbolAddress, with that device current).  Make that first call
//     outside of any stream capture, and before the memory budget is committed
//     (see above).
//   * `stream` must belong to the device that is current when the call is made:
//     the scratch address that the kernels receive is that device's.
//   * All calls on a device share the one array and it keeps whatever the last
//     call left there; each call clears the parts it needs on `stream` before
//     its kernels run.  Two calls whose work overlaps on the GPU (different
//     streams without an ordering between them) race on the array: order them.
//   * No cudaMalloc / cudaFree / allocating library routine is called, on any path.
#pragma once

#include <cuda_runtime.h>

#include <stddef.h>
#include <stdint.h>

#define KRAKEN_NOALLOC_MAX_IDS 65536
#define KRAKEN_NOALLOC_SCRATCH_BYTES (2u * 1024u * 1024u + 512u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

// ids[n] (device, int64)           in
// off[world + 1] (device, int32)   out: exclusive scan of the per-owner unique counts
// uniq[n] (device, int64)          out: unique ids, grouped by owner (off[o] .. off[o + 1])
// inv[n] (device, int32)           out: occurrence -> position in uniq
// status (device, int32, may be 0) out: err::kBadArgument if an id equals the reserved value -1
// err / err_len                    out: message when the call is refused (may be null / 0)
// Returns 0 when the work was enqueued on `stream`, a negative code otherwise:
//   -1 n out of range, -2 world out of range, -3 null argument, -4 CUDA error during set-up or launch.
int kraken_dedup_bucketize_noalloc(const int64_t* ids, int n, int world, uint64_t salt, int32_t* off, int64_t* uniq,
                                   int32_t* inv, int32_t* status, cudaStream_t stream, char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
