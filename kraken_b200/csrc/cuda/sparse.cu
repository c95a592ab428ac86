// Sparse pull / push for GPU-resident hash-table shards, exchanged over peer
// memory (NVLink / NVSwitch) from inside the kernels.
//
// One step of a table ("channel") on every rank, all ranks running the same
// sequence (the calls are collective):
//
//   dedup_bucketize   unique ids of the local batch, grouped by owner rank
//   pull_dispatch     store each owner's id list into that owner's inbox (peer st), raise flag_req
//   pull_probe        owner: wait for a source's flag, find-or-insert its ids, remember the slots
//   pull_gather       owner: copy the rows straight into the requester's receive buffer (peer st),
//                     raise flag_rsp
//   pull_combine      requester: wait for the owners, expand unique rows to occurrences or pool bags
//   ... model forward / backward ...
//   push_scatter      segment-sum of occurrence (or bag) gradients per unique id (vector red)
//   push_dispatch     store summed gradient rows into the owners' gradient inboxes, raise flag_push
//   push_apply        owner: merge rows that several sources sent for one slot, then run the
//                     optimizer in place on value + state slabs (slots remembered from the pull)
//
// This replaces the reference's client-side dedup / routing / scatter-gather
// RPC (kraken/worker/emitter.cc:123-183, :491-550) and the server's per-slot
// locked skip-list loops (kraken/ps/sparse_table.cc:33-108).  Flags carry a
// per-channel epoch; every wait is bounded (common.cuh: wait_flag) and ends in
// a status code instead of a hang.  Peer memory is only touched with plain
// loads / stores / release stores, never with TMA.
//
// Waiting is done by exchange_wait_kernel, ONE warp launched in stream order ahead of the grid that
// needs the data: the request wait (before pull_probe) also copies the peer-writable
// {count, base} words into the channel's control block, which is what every later owner-side
// kernel of the exchange reads - a peer may already be writing the next exchange's words while this
// rank still applies the previous push.  No block of a large grid ever spins, so two streams of
// one GPU cannot starve each other's producers.
#include "sparse_common.cuh"

namespace kb {
namespace cu {

using namespace sparse_detail;

namespace {

// The channel's three rendezvous points.  One warp; lane s polls source s.
//   kWaitRequest   owner: every source's ids of the current pull have arrived; snapshots their counts
//   kWaitResponse  requester: every owner has written the rows of the current pull
//   kWaitPush      owner: every source's gradient rows of the current push have arrived
// A wait that runs out of polls records kTimeout and raises `abort`; the request wait of the next
// exchange lowers it again.
enum WaitKind { kWaitRequest = 0, kWaitResponse = 1, kWaitPush = 2 };

__global__ void exchange_wait_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, int kind, uint32_t spin_limit) {
  pdl_enter();
  const int s = threadIdx.x;
  const size_t flag_off = kind == kWaitRequest ? lay.flag_req : kind == kWaitResponse ? lay.flag_rsp : lay.flag_push;
  const uint32_t want = kind == kWaitPush ? ctrl->push_epoch : ctrl->pull_epoch;
  bool ok = true;
  if (s < sym.world) ok = wait_flag(sym.at<uint32_t>(sym.rank, flag_off) + s, want, spin_limit);
  const bool all_ok = __all_sync(0xffffffffu, ok);
  if (kind == kWaitRequest && all_ok && s < sym.world) ctrl->snap[s] = __ldcg(sym.at<int2>(sym.rank, lay.inbox_meta) + s);
  if (s == 0) {
    if (!all_ok) {
      set_status(&ctrl->status, err::kTimeout);
      ctrl->abort = 1;
    } else if (kind == kWaitRequest) {
      ctrl->abort = 0;
    }
  }
}

void launch_wait(const Sym& s, const ChanLayout& lay, Ctrl* ctrl, int kind, uint32_t spin_limit, cudaStream_t stream) {
  if (s.world > 1) launch_pdl(exchange_wait_kernel, dim3(1), dim3(32), 0, stream, s, lay, ctrl, kind, spin_limit);
}

// ------------------------------------------------------------------ dedup
__global__ void __launch_bounds__(kThreads)
dedup_insert_kernel(const int64_t* __restrict__ ids, int n, int world, int owner_world, uint64_t salt, DedupEntry* table,
                    uint32_t hbits, int* slot_of, int* cnt, int* status) {
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
    if (id == kEmptyKey) {  // reserved value: reported, then treated as its neighbour
      set_status(status, err::kBadArgument);
      id = kEmptyKey - 1;
    }
    const uint64_t mask = (1ull << hbits) - 1;
    slot = SlotHash(id ^ kDedupSalt, hbits);
    for (uint64_t probe = 0; probe <= mask; ++probe) {
      const unsigned long long k = __ldcg(&table[slot].key);
      if (k == id) break;
      if (k == kEmptyKey) {
        const unsigned long long old = atomicCAS(&table[slot].key, kEmptyKey, static_cast<unsigned long long>(id));
        if (old == kEmptyKey) {
          won = true;
          break;
        }
        if (old == id) break;
      }
      slot = (slot + 1) & mask;
    }
    slot_of[i] = static_cast<int>(slot);
    if (won) {
      owner = static_cast<int>(OwnerOf(salt, id, owner_world));
      lpos = atomicAdd(&s_cnt[owner], 1);
    }
  }
  __syncthreads();
  if (threadIdx.x < world && s_cnt[threadIdx.x] > 0) s_base[threadIdx.x] = atomicAdd(&cnt[threadIdx.x], s_cnt[threadIdx.x]);
  __syncthreads();
  if (won)
    table[slot].pos_win = static_cast<unsigned long long>(static_cast<uint32_t>(s_base[owner] + lpos)) |
                          (static_cast<unsigned long long>(static_cast<uint32_t>(i)) << 32);
}

// DISPATCH: the pull's id dispatch is done here as well - every unique id goes straight into its
// owner's inbox (a peer store for other ranks), block 0 writes the per-owner counts, and the last
// block to finish raises the request flags and advances the channel's pull epoch - so a lookup needs
// no separate dispatch launch.
template <bool DISPATCH>
__global__ void __launch_bounds__(kThreads)
dedup_finalize_kernel(const int64_t* __restrict__ ids, int n, int world, int owner_world, uint64_t salt, DedupEntry* table,
                      const int* __restrict__ slot_of, const int* __restrict__ cnt, int* off, int64_t* uniq, int* inv,
                      int cap_u, int* status, Sym sym, ChanLayout lay, Ctrl* ctrl) {
  pdl_enter();
  __shared__ int s_off[kMaxWorld + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int o = 0; o < world; ++o) {
      s_off[o] = acc;
      acc += cnt[o];
    }
    s_off[world] = acc;
    if (blockIdx.x == 0) {
      // more unique ids than the exchange buffers hold: report it and clamp, so that no
      // later kernel indexes past a buffer (the step's result is then invalid, not its memory)
      if (acc > cap_u) set_status(status, err::kInboxOverflow);
      for (int o = 0; o <= world; ++o) off[o] = min(s_off[o], cap_u);
      if (DISPATCH && acc > lay.capU) set_status(&ctrl->status, err::kInboxOverflow);
    }
  }
  __syncthreads();
  if (DISPATCH && blockIdx.x == 0 && threadIdx.x < world) {
    const int o = threadIdx.x;
    const int lo = min(s_off[o], cap_u), hi = min(s_off[o + 1], cap_u);
    const int2 m = make_int2(min(hi - lo, lay.capS), lo);
    sym.at<int2>(o, lay.inbox_meta)[sym.rank] = m;
    if (o == sym.rank) ctrl->snap[o] = m;  // single-GPU jobs launch no request wait
  }
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    uint64_t id = static_cast<uint64_t>(ids[i]);
    if (id == kEmptyKey) id = kEmptyKey - 1;
    const int slot = slot_of[i];
    const int o = static_cast<int>(OwnerOf(salt, id, owner_world));
    const unsigned long long pw = __ldcg(&table[slot].pos_win);
    const int j = static_cast<int>(static_cast<uint32_t>(pw));  // position among the ids of owner o
    const int u = s_off[o] + j;
    inv[i] = u < cap_u ? u : 0;
    if (static_cast<int>(pw >> 32) == i) {
      if (u < cap_u) {
        uniq[u] = static_cast<int64_t>(id);
        if (DISPATCH) {
          if (j < lay.capS)
            sym.at<unsigned long long>(o, lay.inbox_ids)[static_cast<size_t>(sym.rank) * lay.capS + j] = id;
          else
            set_status(&ctrl->status, err::kInboxOverflow);
        }
      }
      table[slot].key = kEmptyKey;  // leave the set empty for the next call
    }
  }
  if (DISPATCH) {
    if (last_block_done(&ctrl->done[0])) {
      const uint32_t e = ctrl->pull_epoch + 1;
      __syncthreads();
      if (threadIdx.x < world) st_release_sys(sym.at<uint32_t>(threadIdx.x, lay.flag_req) + sym.rank, e);
      if (threadIdx.x == 0) ctrl->pull_epoch = e;
    }
  }
}

// ------------------------------------------------------------------ pull
__global__ void __launch_bounds__(kThreads)
pull_dispatch_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, const int64_t* __restrict__ uniq,
                     const int* __restrict__ off) {
  __shared__ int s_off[kMaxWorld + 1];
  if (threadIdx.x <= sym.world) s_off[threadIdx.x] = off[threadIdx.x];
  __syncthreads();
  const int U = s_off[sym.world];
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int gsize = gridDim.x * blockDim.x;
  for (int u = gtid; u < U; u += gsize) {
    const int o = owner_of_index(s_off, sym.world, u);
    const int j = u - s_off[o];
    if (j < lay.capS) {
      sym.at<unsigned long long>(o, lay.inbox_ids)[static_cast<size_t>(sym.rank) * lay.capS + j] =
          static_cast<unsigned long long>(uniq[u]);
    } else {
      set_status(&ctrl->status, err::kInboxOverflow);
    }
  }
  if (U > lay.capU && gtid == 0) set_status(&ctrl->status, err::kInboxOverflow);
  if (gtid < sym.world) {
    const int o = gtid;
    int c = s_off[o + 1] - s_off[o];
    if (c > lay.capS) c = lay.capS;
    sym.at<int2>(o, lay.inbox_meta)[sym.rank] = make_int2(c, s_off[o]);
    if (o == sym.rank) ctrl->snap[o] = make_int2(c, s_off[o]);
  }
  if (last_block_done(&ctrl->done[0])) {
    const uint32_t e = ctrl->pull_epoch + 1;
    __syncthreads();
    if (threadIdx.x < sym.world) st_release_sys(sym.at<uint32_t>(threadIdx.x, lay.flag_req) + sym.rank, e);
    if (threadIdx.x == 0) ctrl->pull_epoch = e;
  }
}

// Owner side of a lookup: one thread per received id finds (or, with `insert`, claims) its slot and
// records it in slot_cache; the rows that the warp's threads have just created are then initialised
// by the whole warp together, `lpr` lanes per row, so that the Philox draws and the stores of a row
// are spread over lanes.  Readers of the rows (pull_gather, a fused consumer) are later launches.
template <int VEC>
__global__ void __launch_bounds__(kThreads)
pull_probe_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, TableView t, int* slot_cache, int insert, int chunks, int lpr) {
  pdl_enter();
  if (ctrl->abort) return;
  const unsigned long long* inbox = sym.at<unsigned long long>(sym.rank, lay.inbox_ids);
  const int lane = threadIdx.x & 31;
  const int rows_per_pass = 32 / lpr;
  for (int k = 0; k < sym.world; ++k) {
    const int s = (sym.rank + k) % sym.world;
    const int cnt = ctrl->snap[s].x;
    for (int base = blockIdx.x * blockDim.x; base < cnt; base += gridDim.x * blockDim.x) {
      const int j = base + threadIdx.x;
      bool created = false;
      int slot = -1;
      uint64_t id = 0;
      if (j < cnt) {
        const size_t e = static_cast<size_t>(s) * lay.capS + j;
        id = __ldcg(&inbox[e]);
        slot = table_find_or_insert(t, id, insert != 0, &created);
        if (slot < 0 && !insert) set_status(&ctrl->status, err::kSparseIdNotExist);
        slot_cache[e] = slot;
      }
      count_created(t, created);
      unsigned todo = __ballot_sync(0xffffffffu, created);
      while (todo) {
        // the next rows_per_pass creators of the warp, one per lane group
        int src = -1;
        unsigned rest = todo;
        for (int g = 0; g < rows_per_pass && rest; ++g) {
          const int l = __ffs(rest) - 1;
          rest &= rest - 1;
          if (g == lane / lpr) src = l;
        }
        todo = rest;
        const int r_slot = __shfl_sync(0xffffffffu, slot, src < 0 ? 0 : src);
        const uint64_t r_id = __shfl_sync(0xffffffffu, id, src < 0 ? 0 : src);
        if (src >= 0) {
          float* row = t.val + static_cast<size_t>(r_slot) * t.dim;
          for (int c = lane % lpr; c < chunks; c += lpr) {
            float q[4];
            if (VEC == 4) {
              InitQuad(t.init, t.seed_key, r_id, c, t.dim, q);
              *reinterpret_cast<float4*>(row + c * 4) = make_float4(q[0], q[1], q[2], q[3]);
            } else {
              InitQuad(t.init, t.seed_key, r_id, c >> 2, t.dim, q);
              row[c] = q[c & 3];
            }
          }
        }
      }
    }
  }
}

template <int VEC>
__global__ void __launch_bounds__(kThreads)
pull_gather_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, TableView t, const int* __restrict__ slot_cache, int chunks,
                   int lpr) {
  pdl_enter();
  using V = Vec<VEC>;
  const int2* meta = ctrl->snap;
  const bool aborted = ctrl->abort != 0;  // the answer flags still go up, so the peers do not time out in turn
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int row0 = gtid / lpr;
  const int row_stride = (gridDim.x * blockDim.x) / lpr;
  // Four rows per thread and iteration: the four slot lookups, then the four row loads, are all in
  // flight before the first store, which is what it takes to keep HBM busy with 16-byte requests.
  constexpr int kUnroll = 4;
  for (int k = 0; k < sym.world; ++k) {
    const int s = (sym.rank + k) % sym.world;
    int2 m = meta[s];
    if (aborted) m.x = 0;
    float* dst_base = sym.at<float>(s, lay.rows_recv) + static_cast<size_t>(m.y) * t.dim;
    const int* slots = slot_cache + static_cast<size_t>(s) * lay.capS;
    for (int r = row0; r < m.x; r += row_stride * kUnroll) {
      int slot[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int ru = r + u * row_stride;
        slot[u] = ru < m.x ? slots[ru] : -1;
      }
      for (int c = lane; c < chunks; c += lpr) {
        typename V::T v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          v[u] = slot[u] < 0 ? V::zero() : V::ld(t.val + static_cast<size_t>(slot[u]) * t.dim + c * VEC);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int ru = r + u * row_stride;
          if (ru < m.x) V::st(dst_base + static_cast<size_t>(ru) * t.dim + c * VEC, v[u]);
        }
      }
    }
  }
  if (last_block_done(&ctrl->done[0])) {
    if (threadIdx.x < sym.world)
      st_release_sys(sym.at<uint32_t>(threadIdx.x, lay.flag_rsp) + sym.rank, ctrl->pull_epoch);
  }
}

template <int VEC>
__global__ void __launch_bounds__(kThreads)
pull_combine_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, const int* __restrict__ inv, int n, int dim, int chunks,
                    int lpr, const int64_t* __restrict__ bag_offsets, int nbags, const float* __restrict__ weights,
                    int mean, const uint8_t* __restrict__ bag_mean, float patch_value, float* __restrict__ out) {
  pdl_enter();
  using V = Vec<VEC>;
  const float* rows = sym.at<float>(sym.rank, lay.rows_recv);
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int row0 = gtid / lpr;
  const int row_stride = (gridDim.x * blockDim.x) / lpr;
  if (bag_offsets == nullptr) {
    constexpr int kUnroll = 4;  // four occurrences per thread in flight, as in the gather
    for (int i = row0; i < n; i += row_stride * kUnroll) {
      int u_of[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int iu = i + u * row_stride;
        u_of[u] = iu < n ? inv[iu] : -1;
      }
      for (int c = lane; c < chunks; c += lpr) {
        typename V::T v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          v[u] = u_of[u] < 0 ? V::zero() : V::ldcg(rows + static_cast<size_t>(u_of[u]) * dim + c * VEC);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int iu = i + u * row_stride;
          if (iu < n) V::st(out + static_cast<size_t>(iu) * dim + c * VEC, v[u]);
        }
      }
    }
  } else {
    for (int b = row0; b < nbags; b += row_stride) {
      const int64_t lo = bag_offsets[b], hi = bag_offsets[b + 1];
      float* dst = out + static_cast<size_t>(b) * dim;
      const bool is_mean = bag_mean ? bag_mean[b] != 0 : mean != 0;
      for (int c = lane; c < chunks; c += lpr) {
        typename V::T acc = V::zero();
        for (int64_t r = lo; r < hi; ++r)
          V::fma(acc, weights ? weights[r] : 1.f, V::ldcg(rows + static_cast<size_t>(inv[r]) * dim + c * VEC));
        if (hi <= lo)
          acc = V::fill(patch_value);
        else if (is_mean)
          acc = V::scale(acc, 1.f / static_cast<float>(hi - lo));
        V::st(dst + c * VEC, acc);
      }
    }
  }
}

// ------------------------------------------------------------------ push
template <int VEC>
__global__ void __launch_bounds__(kThreads)
push_scatter_kernel(const float* __restrict__ grads, const int* __restrict__ inv, int n, int dim, int chunks, int lpr,
                    const int64_t* __restrict__ bag_offsets, int nbags, const float* __restrict__ weights, int mean,
                    const uint8_t* __restrict__ bag_mean, float* ugrad) {
  pdl_enter();
  using V = Vec<VEC>;
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int row0 = gtid / lpr;
  const int row_stride = (gridDim.x * blockDim.x) / lpr;
  if (bag_offsets == nullptr) {
    for (int i = row0; i < n; i += row_stride) {
      const float* src = grads + static_cast<size_t>(i) * dim;
      float* dst = ugrad + static_cast<size_t>(inv[i]) * dim;
      for (int c = lane; c < chunks; c += lpr) V::red(dst + c * VEC, V::ld(src + c * VEC));
    }
  } else {
    for (int b = row0; b < nbags; b += row_stride) {
      const int64_t lo = bag_offsets[b], hi = bag_offsets[b + 1];
      if (hi <= lo) continue;
      const bool is_mean = bag_mean ? bag_mean[b] != 0 : mean != 0;
      const float scale = is_mean ? 1.f / static_cast<float>(hi - lo) : 1.f;
      const float* src = grads + static_cast<size_t>(b) * dim;
      for (int c = lane; c < chunks; c += lpr) {
        const typename V::T g = V::scale(V::ld(src + c * VEC), scale);
        for (int64_t r = lo; r < hi; ++r)
          V::red(ugrad + static_cast<size_t>(inv[r]) * dim + c * VEC, weights ? V::scale(g, weights[r]) : g);
      }
    }
  }
}

template <int VEC>
__global__ void __launch_bounds__(kThreads)
push_dispatch_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, float* ugrad, const int* __restrict__ off, int dim,
                     int chunks, int lpr) {
  pdl_enter();
  using V = Vec<VEC>;
  __shared__ int s_off[kMaxWorld + 1];
  if (threadIdx.x <= sym.world) s_off[threadIdx.x] = off[threadIdx.x];
  __syncthreads();
  const int U = s_off[sym.world];
  const bool aborted = ctrl->abort != 0;
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int row_stride = (gridDim.x * blockDim.x) / lpr;
  for (int u = gtid / lpr; u < U; u += row_stride) {
    const int o = owner_of_index(s_off, sym.world, u);
    const int j = u - s_off[o];
    float* src = ugrad + static_cast<size_t>(u) * dim;
    float* dst = sym.at<float>(o, lay.inbox_grad) + (static_cast<size_t>(sym.rank) * lay.capS + j) * dim;
    for (int c = lane; c < chunks; c += lpr) {
      // after a failed pull the rows (and so the gradients) mean nothing: zeros keep the owners' tables intact
      if (j < lay.capS) V::st(dst + c * VEC, aborted ? V::zero() : V::ld(src + c * VEC));
      V::st(src + c * VEC, V::zero());  // ready for the next step's segment-sum
    }
  }
  if (last_block_done(&ctrl->done[1])) {
    const uint32_t e = ctrl->push_epoch + 1;
    __syncthreads();
    if (threadIdx.x < sym.world) st_release_sys(sym.at<uint32_t>(threadIdx.x, lay.flag_push) + sym.rank, e);
    if (threadIdx.x == 0) ctrl->push_epoch = e;
  }
}

// Owner side, world > 1: several sources may have sent a row for the same
// slot.  The first entry to claim the slot this epoch becomes its leader and
// the others add their row into the leader's inbox row.
template <int VEC>
__global__ void __launch_bounds__(kThreads)
push_merge_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, TableView t, const int* __restrict__ slot_cache, int chunks,
                  int lpr) {
  pdl_enter();
  using V = Vec<VEC>;
  if (ctrl->abort) return;
  const uint32_t epoch = ctrl->push_epoch;
  const int2* meta = ctrl->snap;
  float* inbox = sym.at<float>(sym.rank, lay.inbox_grad);
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int row_stride = (gridDim.x * blockDim.x) / lpr;
  const unsigned group_mask = (lpr == 32 ? 0xffffffffu : ((1u << lpr) - 1u)) << ((threadIdx.x & 31) / lpr * lpr);
  for (int s = 0; s < sym.world; ++s) {
    const int cnt = meta[s].x;
    const int rounds = (cnt + row_stride - 1) / row_stride;
    for (int it = 0; it < rounds; ++it) {
      const int r = gtid / lpr + it * row_stride;
      unsigned leader = 0xffffffffu;
      unsigned entry = 0;
      if (r < cnt) {
        entry = static_cast<unsigned>(s) * lay.capS + r;
        const int slot = slot_cache[entry];
        if (lane == 0 && slot >= 0) {
          const unsigned long long mine = (static_cast<unsigned long long>(epoch) << 32) | entry;
          unsigned long long old = t.lead[slot];
          while (static_cast<uint32_t>(old >> 32) != epoch) {
            const unsigned long long prev = atomicCAS(&t.lead[slot], old, mine);
            if (prev == old) {
              old = mine;
              break;
            }
            old = prev;
          }
          leader = static_cast<unsigned>(old);
        }
      }
      leader = __shfl_sync(group_mask, leader, (threadIdx.x & 31) / lpr * lpr);
      if (r < cnt && leader != 0xffffffffu && leader != entry) {
        const float* src = inbox + static_cast<size_t>(entry) * t.dim;
        float* dst = inbox + static_cast<size_t>(leader) * t.dim;
        for (int c = lane; c < chunks; c += lpr) V::red(dst + c * VEC, V::ldcg(src + c * VEC));
      }
    }
  }
}

// OPT is the optimizer type as a compile-time constant: the update switch folds away, Adam's bias
// terms exist only where they are used, and the kernel fits four blocks per SM.
template <int VEC, int OPT>
__global__ void __launch_bounds__(kThreads, 4)
push_update_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, TableView t, const int* __restrict__ slot_cache,
                   OptimPOD optim_in, const float* __restrict__ lr_ptr, int chunks, int lpr) {
  pdl_enter();
  using V = Vec<VEC>;
  OptimPOD optim = optim_in;
  optim.type = OPT;
  if (ctrl->abort) return;
  const uint32_t epoch = ctrl->push_epoch;
  const int2* meta = ctrl->snap;
  const float* inbox = sym.at<float>(sym.rank, lay.inbox_grad);
  const float lr = *lr_ptr;
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int row_stride = (gridDim.x * blockDim.x) / lpr;
  const unsigned group_mask = (lpr == 32 ? 0xffffffffu : ((1u << lpr) - 1u)) << ((threadIdx.x & 31) / lpr * lpr);
  for (int s = 0; s < sym.world; ++s) {
    const int cnt = meta[s].x;
    for (int r = gtid / lpr; r < cnt; r += row_stride) {
      const unsigned entry = static_cast<unsigned>(s) * lay.capS + r;
      const int slot = slot_cache[entry];
      if (slot < 0) continue;
      if (sym.world > 1 && t.lead[slot] != ((static_cast<unsigned long long>(epoch) << 32) | entry)) continue;
      // Lane 0 of the row owns the step counter: it reads, bumps and shares it.
      int step_i = 1;
      if (t.steps) {
        if (lane == 0) {
          step_i = t.steps[slot] + 1;
          t.steps[slot] = step_i;
        }
        step_i = __shfl_sync(group_mask, step_i, (threadIdx.x & 31) / lpr * lpr);
      }
      const int64_t step = step_i;
      const AdamBias ab = optim.type == 1 ? AdamBiasAt(optim, step) : AdamBias{1.f, 1.f};
      const size_t row = static_cast<size_t>(slot) * t.dim;
      for (int c = lane; c < chunks; c += lpr) {
        float g[VEC], w[VEC], a0[VEC], a1[VEC], a2[VEC];
        *reinterpret_cast<typename V::T*>(g) = V::ldcg(inbox + static_cast<size_t>(entry) * t.dim + c * VEC);
        *reinterpret_cast<typename V::T*>(w) = V::ld(t.val + row + c * VEC);
        *reinterpret_cast<typename V::T*>(a0) = t.s[0] ? V::ld(t.s[0] + row + c * VEC) : V::zero();
        *reinterpret_cast<typename V::T*>(a1) = t.s[1] ? V::ld(t.s[1] + row + c * VEC) : V::zero();
        *reinterpret_cast<typename V::T*>(a2) = t.s[2] ? V::ld(t.s[2] + row + c * VEC) : V::zero();
#pragma unroll
        for (int e = 0; e < VEC; ++e) UpdateElem(optim, lr, g[e], step, ab, w[e], a0[e], a1[e], a2[e]);
        V::st(t.val + row + c * VEC, *reinterpret_cast<typename V::T*>(w));
        if (t.s[0]) V::st(t.s[0] + row + c * VEC, *reinterpret_cast<typename V::T*>(a0));
        if (t.s[1]) V::st(t.s[1] + row + c * VEC, *reinterpret_cast<typename V::T*>(a1));
        if (t.s[2]) V::st(t.s[2] + row + c * VEC, *reinterpret_cast<typename V::T*>(a2));
      }
    }
  }
}

}  // namespace

// ------------------------------------------------------------------ launchers
void dedup_bucketize(const int64_t* ids, int n, int world, int owner_world, uint64_t salt, DedupScratch sc, int* cnt,
                     int* off, int64_t* uniq, int* inv, int cap_u, int* status, cudaStream_t stream) {
  const int blocks = (n + kThreads - 1) / kThreads;
  cudaMemsetAsync(cnt, 0, sizeof(int) * world, stream);
  if (n <= 0) {
    cudaMemsetAsync(off, 0, sizeof(int) * (world + 1), stream);
    return;
  }
  dedup_insert_kernel<<<blocks, kThreads, 0, stream>>>(ids, n, world, owner_world, salt, static_cast<DedupEntry*>(sc.table), sc.hbits,
                                                       sc.slot_of, cnt, status);
  launch_pdl(dedup_finalize_kernel<false>, dim3(blocks), dim3(kThreads), 0, stream, ids, n, world, owner_world, salt, static_cast<DedupEntry*>(sc.table),
                                                                sc.slot_of, cnt, off, uniq, inv, cap_u, status, Sym{},
                                                                ChanLayout{}, nullptr);
}

void dedup_bucketize_dispatch(const int64_t* ids, int n, int world, int owner_world, uint64_t salt, DedupScratch sc,
                              int* cnt, int* off, int64_t* uniq, int* inv, int cap_u, int* status, SymHost sym,
                              ChanLayout lay, Ctrl* ctrl, cudaStream_t stream) {
  if (n <= 0) {  // nothing to deduplicate: the plain dispatch still has to publish empty counts and the epoch
    dedup_bucketize(ids, n, world, owner_world, salt, sc, cnt, off, uniq, inv, cap_u, status, stream);
    pull_dispatch_kernel<<<1, kThreads, 0, stream>>>(to_sym(sym), lay, ctrl, uniq, off);
    return;
  }
  const int blocks = (n + kThreads - 1) / kThreads;
  cudaMemsetAsync(cnt, 0, sizeof(int) * world, stream);
  dedup_insert_kernel<<<blocks, kThreads, 0, stream>>>(ids, n, world, owner_world, salt, static_cast<DedupEntry*>(sc.table), sc.hbits,
                                                       sc.slot_of, cnt, status);
  launch_pdl(dedup_finalize_kernel<true>, dim3(blocks), dim3(kThreads), 0, stream, ids, n, world, owner_world, salt, static_cast<DedupEntry*>(sc.table),
                                                               sc.slot_of, cnt, off, uniq, inv, cap_u, status,
                                                               to_sym(sym), lay, ctrl);
}

void pull_dispatch(SymHost sym, ChanLayout lay, Ctrl* ctrl, const int64_t* uniq, const int* off, int max_n,
                   cudaStream_t stream) {
  pull_dispatch_kernel<<<grid_for(max_n), kThreads, 0, stream>>>(to_sym(sym), lay, ctrl, uniq, off);
}

void pull_probe(SymHost sym, ChanLayout lay, Ctrl* ctrl, TableHost table, int* slot_cache, bool insert,
                uint32_t spin_limit, cudaStream_t stream) {
  const Sym s = to_sym(sym);
  launch_wait(s, lay, ctrl, kWaitRequest, spin_limit, stream);
  const RowGeom g = row_geom(table.dim);
  const int grid = grid_for(static_cast<long long>(lay.capS));
  if (g.vec == 4)
    launch_pdl(pull_probe_kernel<4>, dim3(grid), dim3(kThreads), 0, stream, s, lay, ctrl, to_view(table), slot_cache, insert ? 1 : 0,
                                                        g.chunks, g.lpr);
  else
    launch_pdl(pull_probe_kernel<1>, dim3(grid), dim3(kThreads), 0, stream, s, lay, ctrl, to_view(table), slot_cache, insert ? 1 : 0,
                                                        g.chunks, g.lpr);
}

void exchange_wait(SymHost sym, ChanLayout lay, Ctrl* ctrl, int kind, uint32_t spin_limit, cudaStream_t stream) {
  launch_wait(to_sym(sym), lay, ctrl, kind, spin_limit, stream);
}

void pull_wait(SymHost sym, ChanLayout lay, Ctrl* ctrl, uint32_t spin_limit, cudaStream_t stream) {
  launch_wait(to_sym(sym), lay, ctrl, kWaitResponse, spin_limit, stream);
}

void pull_gather(SymHost sym, ChanLayout lay, Ctrl* ctrl, TableHost table, const int* slot_cache,
                 cudaStream_t stream) {
  const RowGeom g = row_geom(table.dim);
  const int grid = grid_for(static_cast<long long>(lay.capS) * g.lpr);
  if (g.vec == 4)
    launch_pdl(pull_gather_kernel<4>, dim3(grid), dim3(kThreads), 0, stream, to_sym(sym), lay, ctrl, to_view(table), slot_cache, g.chunks,
                                                         g.lpr);
  else
    launch_pdl(pull_gather_kernel<1>, dim3(grid), dim3(kThreads), 0, stream, to_sym(sym), lay, ctrl, to_view(table), slot_cache, g.chunks,
                                                         g.lpr);
}

void pull_combine(SymHost sym, ChanLayout lay, Ctrl* ctrl, const int* inv, int n, int dim, const int64_t* bag_offsets,
                  int k, const float* weights, bool mean, const uint8_t* bag_mean, float patch_value, float* out,
                  uint32_t spin_limit, cudaStream_t stream) {
  const RowGeom g = row_geom(dim);
  const long long rows = bag_offsets ? k : n;
  const int grid = grid_for(rows * g.lpr);
  launch_wait(to_sym(sym), lay, ctrl, kWaitResponse, spin_limit, stream);
  if (g.vec == 4)
    launch_pdl(pull_combine_kernel<4>, dim3(grid), dim3(kThreads), 0, stream, to_sym(sym), lay, ctrl, inv, n, dim, g.chunks, g.lpr,
                                                          bag_offsets, k, weights, mean ? 1 : 0, bag_mean, patch_value,
                                                          out);
  else
    launch_pdl(pull_combine_kernel<1>, dim3(grid), dim3(kThreads), 0, stream, to_sym(sym), lay, ctrl, inv, n, dim, g.chunks, g.lpr,
                                                          bag_offsets, k, weights, mean ? 1 : 0, bag_mean, patch_value,
                                                          out);
}

void push_scatter(const float* grads, const int* inv, int n, int dim, const int64_t* bag_offsets, int k,
                  const float* weights, bool mean, const uint8_t* bag_mean, float* ugrad, cudaStream_t stream) {
  const RowGeom g = row_geom(dim);
  const long long rows = bag_offsets ? k : n;
  if (rows <= 0) return;
  const int grid = grid_for(rows * g.lpr, kThreads, 148 * 16);
  if (g.vec == 4)
    launch_pdl(push_scatter_kernel<4>, dim3(grid), dim3(kThreads), 0, stream, grads, inv, n, dim, g.chunks, g.lpr, bag_offsets, k, weights,
                                                          mean ? 1 : 0, bag_mean, ugrad);
  else
    launch_pdl(push_scatter_kernel<1>, dim3(grid), dim3(kThreads), 0, stream, grads, inv, n, dim, g.chunks, g.lpr, bag_offsets, k, weights,
                                                          mean ? 1 : 0, bag_mean, ugrad);
}

void push_dispatch(SymHost sym, ChanLayout lay, Ctrl* ctrl, float* ugrad, const int* off, int max_n, int dim,
                   cudaStream_t stream) {
  const RowGeom g = row_geom(dim);
  const int grid = grid_for(static_cast<long long>(max_n) * g.lpr);
  if (g.vec == 4)
    launch_pdl(push_dispatch_kernel<4>, dim3(grid), dim3(kThreads), 0, stream, to_sym(sym), lay, ctrl, ugrad, off, dim, g.chunks, g.lpr);
  else
    launch_pdl(push_dispatch_kernel<1>, dim3(grid), dim3(kThreads), 0, stream, to_sym(sym), lay, ctrl, ugrad, off, dim, g.chunks, g.lpr);
}

namespace {
template <int VEC>
void launch_update(int grid, cudaStream_t stream, const Sym& s, const ChanLayout& lay, Ctrl* ctrl, const TableView& t,
                   const int* slot_cache, const OptimPOD& optim, const float* lr, int chunks, int lpr) {
  switch (optim.type) {
    case 0: launch_pdl(push_update_kernel<VEC, 0>, dim3(grid), dim3(kThreads), 0, stream, s, lay, ctrl, t, slot_cache, optim, lr, chunks, lpr); break;
    case 1: launch_pdl(push_update_kernel<VEC, 1>, dim3(grid), dim3(kThreads), 0, stream, s, lay, ctrl, t, slot_cache, optim, lr, chunks, lpr); break;
    case 2: launch_pdl(push_update_kernel<VEC, 2>, dim3(grid), dim3(kThreads), 0, stream, s, lay, ctrl, t, slot_cache, optim, lr, chunks, lpr); break;
    default: launch_pdl(push_update_kernel<VEC, 3>, dim3(grid), dim3(kThreads), 0, stream, s, lay, ctrl, t, slot_cache, optim, lr, chunks, lpr); break;
  }
}
}  // namespace

void push_apply(SymHost sym, ChanLayout lay, Ctrl* ctrl, TableHost table, const int* slot_cache, OptimPOD optim,
                const float* lr, uint32_t spin_limit, cudaStream_t stream) {
  const RowGeom g = row_geom(table.dim);
  const int grid = grid_for(static_cast<long long>(lay.capS) * g.lpr);
  const Sym s = to_sym(sym);
  const TableView t = to_view(table);
  launch_wait(s, lay, ctrl, kWaitPush, spin_limit, stream);
  if (g.vec == 4) {
    if (sym.world > 1) launch_pdl(push_merge_kernel<4>, dim3(grid), dim3(kThreads), 0, stream, s, lay, ctrl, t, slot_cache, g.chunks, g.lpr);
    launch_update<4>(grid, stream, s, lay, ctrl, t, slot_cache, optim, lr, g.chunks, g.lpr);
  } else {
    if (sym.world > 1) launch_pdl(push_merge_kernel<1>, dim3(grid), dim3(kThreads), 0, stream, s, lay, ctrl, t, slot_cache, g.chunks, g.lpr);
    launch_update<1>(grid, stream, s, lay, ctrl, t, slot_cache, optim, lr, g.chunks, g.lpr);
  }
}

}  // namespace cu
}  // namespace kb
