// Host-callable launchers of the sm_100a kernels.  Plain pointers and a
// stream: nothing here depends on torch, so the kernels can be driven from
// C, C++ or ctypes.  Every launcher is asynchronous on `stream`, allocates
// nothing and never synchronises; errors are reported through the `status`
// words the kernels write (codes of core/types.h).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../core/optim_math.h"

namespace kb {
namespace cu {

constexpr int kMaxWorldHost = 16;

struct SymHost {
  void* base[kMaxWorldHost];
  int rank;
  int world;
};

// Byte offsets of one exchange channel inside every rank's symmetric heap.
struct ChanLayout {
  size_t inbox_ids;   // u64  [world][capS]   ids sent by each source
  size_t inbox_meta;  // int2 [world]         {count, base offset in the source's receive buffer}
  size_t rows_recv;   // f32  [capU][dim]     rows returned for this rank's unique ids
  size_t inbox_grad;  // f32  [world][capS][dim]
  size_t flag_req;    // u32  [world]
  size_t flag_rsp;    // u32  [world]
  size_t flag_push;   // u32  [world]
  size_t inbox_tcnt;  // int  [world][T + 1]  multi-table channels only: per source, prefix of its ids per table
  int capS;           // ids one source may send to one owner
  int capU;           // unique ids one rank may request
};

// Per-channel device control block (local memory, not peer-mapped).
// `snap` is this rank's private copy of {count, base} of every source for the exchange in flight:
// peers overwrite inbox_meta as soon as THEY start their next lookup, which can be while this rank's
// push kernels of the previous exchange still run, so every owner-side kernel reads the copy.
// `abort` is raised by a wait that ran out of polls; the kernels of that exchange then move no data.
struct Ctrl {
  uint32_t pull_epoch;
  uint32_t push_epoch;
  uint32_t done[2];
  int status;
  int abort;
  int pad[2];
  int2 snap[kMaxWorldHost];
};
constexpr int kCtrlInts = static_cast<int>(sizeof(Ctrl) / sizeof(int));

struct TableHost {
  void* keys;
  float* val;
  float* s[3];
  int* steps;
  void* lead;
  int* size;
  int* status;
  uint32_t bits;
  int dim;
  InitPOD init;
  uint64_t seed_key;
};

// Scratch of the dedup kernels: an open-addressing set of 1 << hbits slots
// (hbits chosen so that it holds at least 2 n ids), all keys kEmptyKey between calls.
struct DedupScratch {
  void* table;   // [1 << hbits] entries of 16 bytes: u64 key, then u32 rank of the unique id inside its owner
                 // group and u32 index of the occurrence that inserted it (one 32-byte sector holds two entries)
  int* slot_of;  // int [n]
  uint32_t hbits;
};

// ---- dedup + bucketise by owner (unique ids grouped by owner rank) ----
// cnt[world] is scratch (zeroed here).  Outputs: off[world + 1] (exclusive scan of
// the per-owner unique counts), uniq[off[world]], inv[n] (occurrence -> unique).  cap_u is the
// capacity of uniq and of the buffers later indexed by inv: beyond it the call reports
// kInboxOverflow and clamps its outputs into range.
// owner_world <= world: rows are owned by ranks 0 .. owner_world - 1 only (OwnerOf(salt, id, owner_world)); the other
// ranks still look rows up and push gradients.  Normally equal to world; smaller after a live reshard.
void dedup_bucketize(const int64_t* ids, int n, int world, int owner_world, uint64_t salt, DedupScratch sc, int* cnt,
                     int* off, int64_t* uniq, int* inv, int cap_u, int* status, cudaStream_t stream);
// The same, with the pull's id dispatch (pull_dispatch below) done by the second kernel of the dedup:
// unique ids go straight into their owners' inboxes and the channel's pull epoch advances.
void dedup_bucketize_dispatch(const int64_t* ids, int n, int world, int owner_world, uint64_t salt, DedupScratch sc,
                              int* cnt, int* off, int64_t* uniq, int* inv, int cap_u, int* status, SymHost sym,
                              ChanLayout lay, Ctrl* ctrl, cudaStream_t stream);

// ---- sparse pull ----
// Cross-GPU waits never run inside the big grids: each is a one-warp kernel in stream order
// (exchange_wait), so a block that spins never holds registers or shared memory that a producer on
// another stream of the same GPU could need.  pull_probe, pull_combine / pull_wait and push_apply
// launch the wait they depend on themselves when world > 1.
void pull_dispatch(SymHost sym, ChanLayout lay, Ctrl* ctrl, const int64_t* uniq, const int* off, int max_n,
                   cudaStream_t stream);
void pull_probe(SymHost sym, ChanLayout lay, Ctrl* ctrl, TableHost table, int* slot_cache, bool insert,
                uint32_t spin_limit, cudaStream_t stream);
void pull_gather(SymHost sym, ChanLayout lay, Ctrl* ctrl, TableHost table, const int* slot_cache, cudaStream_t stream);
// out[n, dim] (bag_offsets == nullptr) or pooled out[k, dim].
void pull_combine(SymHost sym, ChanLayout lay, Ctrl* ctrl, const int* inv, int n, int dim, const int64_t* bag_offsets,
                  int k, const float* weights, bool mean, const uint8_t* bag_mean, float patch_value, float* out,
                  uint32_t spin_limit, cudaStream_t stream);

// ---- sparse push ----
// ugrad[capU, dim] must be zero on entry (push_dispatch re-zeroes what it sends).
void push_scatter(const float* grads, const int* inv, int n, int dim, const int64_t* bag_offsets, int k,
                  const float* weights, bool mean, const uint8_t* bag_mean, float* ugrad, cudaStream_t stream);
void push_dispatch(SymHost sym, ChanLayout lay, Ctrl* ctrl, float* ugrad, const int* off, int max_n, int dim,
                   cudaStream_t stream);
void push_apply(SymHost sym, ChanLayout lay, Ctrl* ctrl, TableHost table, const int* slot_cache, OptimPOD optim,
                const float* lr, uint32_t spin_limit, cudaStream_t stream);

// One of the channel's rendezvous points as a launch of its own: kind 0 = every source's request has
// arrived (also snapshots the counts), 1 = every owner has answered the pull, 2 = every source's gradient
// rows have arrived.  Nothing is launched when world == 1.
void exchange_wait(SymHost sym, ChanLayout lay, Ctrl* ctrl, int kind, uint32_t spin_limit, cudaStream_t stream);

// ---- one exchange for several tables of the same row width (sparse_group.cu) ----
// The ids of the group's tables are one concatenated list; occ_start[T + 1] gives each table's part.
// The dedup scratch set is split into one region per table (region_base / region_bits, in entries),
// so equal ids of different tables stay distinct; unique ids come out grouped by (owner, table).
// All arrays are device memory, rewritten by the host only when the shapes of a call change.
struct GroupDesc {
  int T;
  int owner_world;                     // rows are owned by ranks 0 .. owner_world - 1
  const int* occ_start;                // [T + 1]
  const int* region_base;              // [T]
  const int* region_bits;              // [T]
  const unsigned long long* salt;      // [T] owner salt of every table
};
// Fills out_host[T * group_table_view_bytes()] with the device-side descriptors of the tables; the caller
// copies the block to device memory and passes that pointer as `table_views` below (again after a table
// was reallocated).
void group_table_views(const TableHost* tables, int T, void* out_host);
size_t group_table_view_bytes();
// dedup + dispatch of the whole group (cnt: scratch of world * T ints).
void group_dedup_dispatch(const int64_t* ids, int n, const GroupDesc& d, int world, DedupScratch sc, int* cnt,
                          int* off, int64_t* uniq, int* inv, int cap_u, int* status, SymHost sym, ChanLayout lay,
                          Ctrl* ctrl, cudaStream_t stream);
// Owner side: request rendezvous (always launched: it also copies the per-table prefixes into snap_t
// [world * (T + 1)]), then find-or-insert of every received id in its table; records slot and table per entry.
void group_probe(SymHost sym, ChanLayout lay, Ctrl* ctrl, const void* table_views, int T, int dim, int* snap_t,
                 int* slot_cache, int16_t* ttab, bool insert, uint32_t spin_limit, cudaStream_t stream);
void group_gather(SymHost sym, ChanLayout lay, Ctrl* ctrl, const void* table_views, int dim, const int* slot_cache,
                  const int16_t* ttab, cudaStream_t stream);
void group_push_apply(SymHost sym, ChanLayout lay, Ctrl* ctrl, const void* table_views, int dim, const int* slot_cache,
                      const int16_t* ttab, OptimPOD optim, const float* lr, uint32_t spin_limit, cudaStream_t stream);

// Owner rank of every id under the modulo placement (OwnerOf of core/hash.h).
void owner_of(const int64_t* ids, int n, uint64_t salt, int world, int* owners, cudaStream_t stream);

// ---- table maintenance ----
void table_clear(TableHost table, cudaStream_t stream);
// Inserts rows with given values and states (any of s0..s2 / steps may be null).
void table_import(TableHost table, const int64_t* ids, const float* vals, const float* s0, const float* s1,
                  const float* s2, const int* steps, int n, cudaStream_t stream);
// Finds ids (no insert); rows[n, dim] gets the values, found[n] 1/0.
void table_lookup(TableHost table, const int64_t* ids, int n, float* rows, uint8_t* found, cudaStream_t stream);
// Compacts the occupied slots that pass the filter into the out_* arrays; *out_count receives how many.
// filter_mode 0: all; 1: OwnerOf(salt, id, world) == rank; 2: OwnerOf(...) != rank; 3: steps >= min_steps;
// 4: id % world == rank (a checkpoint file's slot: world = 8, rank = slot).
void table_export(TableHost table, int filter_mode, uint64_t salt, int world, int rank, int min_steps,
                  int64_t* out_ids, float* out_vals, float* out_s0, float* out_s1, float* out_s2, int* out_steps,
                  int* out_count, int out_cap, cudaStream_t stream);

// ---- model kernels ----
void jagged_forward(const float* values, const float* weights, const int64_t* offsets, int k, int dim, bool mean,
                    float patch_value, float* out, cudaStream_t stream);
void jagged_backward(const float* grads, const float* weights, const int64_t* offsets, int k, int dim, bool mean,
                     float* out, cudaStream_t stream);
// FM second-order interaction over emb[B, F, D]: out[b] = 0.5 * sum_k((sum_f e)^2 - sum_f e^2).
void fm_forward(const float* emb, int B, int F, int D, float* out, cudaStream_t stream);
void fm_backward(const float* emb, const float* gout, int B, int F, int D, float* gemb, cudaStream_t stream);
// Binary cross entropy with logits, mean reduction: loss[0] += sum / n (loss must be zero on entry);
// grad (optional) = (sigmoid(x) - y) / n.
void bce_forward_backward(const float* logits, const float* labels, int n, float* loss, float* grad,
                          cudaStream_t stream);

// ---- DeepFM front end fused around the sparse exchange (deepfm_fused.cu) ----
// Waits (bounded) until every owner has answered the channel's current pull.
void pull_wait(SymHost sym, ChanLayout lay, Ctrl* ctrl, uint32_t spin_limit, cudaStream_t stream);
// x[B, ldx] bf16 = [emb rows of F fields x D | ND dense features | zeros], fm_logit[B] fp32.
// rows2 [*, RD] / rows1 [*, 1] are unique rows, inv2 / inv1 [B * F] map occurrences to them.  D % 4 == 0,
// RD % 4 == 0, D / 4 a power of two <= 32.  rows1 == nullptr: the first-order weight is column D of rows2
// (RD >= D + 1).  ssum [B, D] (nullable in the forward) receives sum_f e_f per sample; the backward reads it.
// slots2 / slots1 (nullable): rows2 / rows1 are then the tables' value slabs and unique entry u lives in
// row slots[u] (the in-place path of single-GPU jobs).
void deepfm_pack_forward(const float* rows2, const int* inv2, const int* slots2, const float* rows1, const int* inv1,
                         const int* slots1, const float* dense, int B, int F, int D, int RD, int ND, __nv_bfloat16* x,
                         int ldx, float* fm_logit, float* ssum, cudaStream_t stream);
// Adds each occurrence's gradient into ugrad2 [*, RD] / ugrad1 [*, 1] (per unique id).  dx may be null;
// ugrad1 == nullptr: the first-order gradient goes to column D of ugrad2.
void deepfm_pack_backward(const float* rows2, const int* inv2, const int* slots2, const int* inv1,
                          const __nv_bfloat16* dx, int lddx, const float* dlogit, const float* ssum, int B, int F, int D,
                          int RD, float* ugrad2, float* ugrad1, cudaStream_t stream);

// bf16 copy [N, K] and bf16 transpose [K, N] of an fp32 weight matrix [N, K], one pass.
void cast_w_wt(const float* w, int N, int K, __nv_bfloat16* w16, __nv_bfloat16* wt16, cudaStream_t stream);

// Linear layer with one output over bf16 rows x[M, K] (pitch ldx):
// y[m] = x[m, :] . w + bias[0] + addend[m]   (bias and addend optional).
void rowdot_forward(const __nv_bfloat16* x, int ldx, const float* w, const float* bias, const float* addend, int M,
                    int K, float* y, cudaStream_t stream);
// Its backward: dx (optional, bf16, optionally masked by x > 0), dw[K] += ..., db[0] += sum(dy).
void rowdot_backward(const __nv_bfloat16* x, int ldx, const float* w, const float* dy, int M, int K, bool relu_mask,
                     __nv_bfloat16* dx, int lddx, float* dw, float* db, cudaStream_t stream);

}  // namespace cu
}  // namespace kb
