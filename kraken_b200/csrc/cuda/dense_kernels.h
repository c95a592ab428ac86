// Launchers of the dense-parameter path: the fused reduce-scatter + optimizer +
// all-gather step over peer memory, and the DCT (top-k threshold with error
// feedback) kernels.  Same conventions as kernels.h.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../core/optim_math.h"
#include "kernels.h"

namespace kb {
namespace cu {

constexpr int kDenseChunk = 256;  // elements; tables start on chunk boundaries

// Byte offsets inside every rank's symmetric heap.
struct DenseLayout {
  size_t grad;       // f32 [n_pad]  this rank's local gradient (summed by the owners)
  size_t param;      // f32 [n_pad]  this rank's full copy of the parameters
  size_t flag_grad;  // u32 [world]  "rank s finished its backward" (written by s)
  size_t flag_done;  // u32 [world]  "owner o finished writing its slice" (written by o)
  size_t coo_cnt;    // i32 [world]  DCT: pairs this rank emitted for owner o
  size_t coo_idx;    // i32 [n_pad]  DCT: element offsets inside the owner's slice, grouped by owner slice
  size_t coo_val;    // f32 [n_pad]  DCT: values, same order
};

struct DenseCtrl {
  uint32_t epoch;
  uint32_t done[2];
  int status;
  int abort;  // raised by a rendezvous that ran out of polls: the step then changes no parameter
  int pad[3];
};
constexpr int kDenseCtrlInts = static_cast<int>(sizeof(DenseCtrl) / sizeof(int));

// One optimizer step over all dense tables, all ranks together:
//   owner(slice) sums every rank's gradient slice straight out of peer memory,
//   runs the optimizer on its slice (state slabs are local, slice-sized) and
//   stores the new values into every rank's parameter copy.
// chunk_table[n_pad / 256] maps a chunk to its table; table_active[t] == 0
// leaves table t untouched; table_steps[t] is bumped for active tables.
// use_coo != 0: gradients arrive as the (idx, val) lists written by dct_compact.
// The local gradient buffer is zero again when the call's last kernel ends.
// Between GPUs the call is a short sequence in stream order - a one-warp rendezvous ("my gradient is
// complete" to every peer, wait for theirs), the update grid, a one-warp wait for every owner's
// "slice written", the zeroing grid - so that no block of a large grid ever spins on a peer.
void dense_step(SymHost sym, DenseLayout lay, DenseCtrl* ctrl, long long n_pad, float* s0, float* s1, float* s2,
                float* acc, const int* chunk_table, int* table_steps, const uint8_t* table_active, int n_tables,
                OptimPOD optim, const float* lr, float grad_scale, int use_coo, uint32_t spin_limit,
                cudaStream_t stream);

// ---- DCT ----
// f = g + e written over g (in place); returns nothing.  Part of every DCT step.
void dct_accumulate(float* grad, const float* residual, long long n, cudaStream_t stream);
// k-th largest |x| over x[0..n) by 4-pass radix select on the float bits.
// hist is scratch of 4 * 256 uint32 (zeroed here); *tau receives the result.
void dct_select_tau(const float* x, long long n, long long k, uint32_t* hist, uint32_t* prefix_state, float* tau,
                    cudaStream_t stream);
// Single pass over f (held in `grad`): entries with |f| >= tau_table[table of the entry] are
// appended to the list of the slice owner (idx relative to the slice, val) and zeroed in
// `residual`; the others stay in `residual`; `grad` itself is zeroed (the lists carry the
// gradient).  slice = n_pad / world.  A table with tau 0 (fewer than 256 elements) travels whole.
void dct_compact(SymHost sym, DenseLayout lay, long long n_pad, float* residual, const float* tau_table,
                 const int* chunk_table, cudaStream_t stream);
// Same thresholding without compaction: grad = |f| >= tau ? f : 0, residual = the rest.
void dct_threshold_dense(float* grad, float* residual, long long n, const float* tau_table, const int* chunk_table,
                         cudaStream_t stream);

}  // namespace cu
}  // namespace kb
