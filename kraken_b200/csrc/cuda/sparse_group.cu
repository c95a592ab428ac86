// One exchange for SEVERAL sparse tables of the same row width.
//
// The reference sends map<table, ids> to every server in one request round and the server walks
// the tables one after the other (kraken/worker/emitter.cc:185-278 pull, :552-632 push;
// kraken/ps/ps_op.cc:370-387, :456-469).  Here the ids of all tables of a group are one
// concatenated list: one dedup keyed by (table, id), one dispatch into the owners' inboxes, one
// owner-side probe, one gather, and one push sequence serve the whole group, so a model built from
// dozens of small tables (the reference's DeepFM example has 39 + 39) pays for one exchange per
// row width instead of one per table.
//
// How (table, id) stays exact with 64-bit keys: the dedup scratch set is split into one region per
// table, and unique ids are grouped by (owner, table) - so the position of an entry inside a
// source's segment tells the owner which table it belongs to (a per-source prefix table travels with
// the counts).  The owner's probe records that table index per entry; gather, merge and update read it.
#include "sparse_common.cuh"

namespace kb {
namespace cu {

using namespace sparse_detail;

namespace {

// Largest t with prefix[t] <= i (prefix has T + 1 ascending entries, prefix[0] == 0).
__device__ __forceinline__ int segment_of(const int* prefix, int T, int i) {
  int lo = 0, hi = T;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= i) lo = mid; else hi = mid;
  }
  return lo;
}

extern __shared__ int g_smem[];

__global__ void __launch_bounds__(kThreads)
group_dedup_insert_kernel(const int64_t* __restrict__ ids, int n, GroupDesc d, int world, DedupEntry* table,
                          int* slot_of, int* cnt, int* status) {
  int* s_occ = g_smem;                    // [T + 1]
  int* s_cnt = s_occ + d.T + 1;           // [world * T]
  int* s_base = s_cnt + world * d.T;      // [world * T]
  for (int k = threadIdx.x; k <= d.T; k += blockDim.x) s_occ[k] = d.occ_start[k];
  for (int k = threadIdx.x; k < world * d.T; k += blockDim.x) s_cnt[k] = 0;
  __syncthreads();

  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  bool won = false;
  int cell = 0, lpos = 0;
  uint64_t slot = 0;
  if (i < n) {
    uint64_t id = static_cast<uint64_t>(ids[i]);
    if (id == kEmptyKey) {
      set_status(status, err::kBadArgument);
      id = kEmptyKey - 1;
    }
    const int t = segment_of(s_occ, d.T, i);
    const uint32_t bits = static_cast<uint32_t>(d.region_bits[t]);
    const uint64_t mask = (1ull << bits) - 1;
    DedupEntry* region = table + d.region_base[t];
    uint64_t p = SlotHash(id ^ kDedupSalt, bits);
    for (uint64_t probe = 0; probe <= mask; ++probe) {
      const unsigned long long k = __ldcg(&region[p].key);
      if (k == id) break;
      if (k == kEmptyKey) {
        const unsigned long long old = atomicCAS(&region[p].key, kEmptyKey, static_cast<unsigned long long>(id));
        if (old == kEmptyKey) {
          won = true;
          break;
        }
        if (old == id) break;
      }
      p = (p + 1) & mask;
    }
    slot = static_cast<uint64_t>(d.region_base[t]) + p;
    slot_of[i] = static_cast<int>(slot);
    if (won) {
      cell = static_cast<int>(OwnerOf(d.salt[t], id, d.owner_world)) * d.T + t;
      lpos = atomicAdd(&s_cnt[cell], 1);
    }
  }
  __syncthreads();
  for (int k = threadIdx.x; k < world * d.T; k += blockDim.x)
    if (s_cnt[k] > 0) s_base[k] = atomicAdd(&cnt[k], s_cnt[k]);
  __syncthreads();
  if (won)
    table[slot].pos_win = static_cast<unsigned long long>(static_cast<uint32_t>(s_base[cell] + lpos)) |
                          (static_cast<unsigned long long>(static_cast<uint32_t>(i)) << 32);
}

// Exclusive scan of cnt[0 .. W) into s_off[0 .. W], by the whole block (W up to a few thousand).
__device__ void block_exclusive_scan(const int* __restrict__ cnt, int W, int* s_off, int* s_part) {
  const int per = (W + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * per, hi = min(lo + per, W);
  int sum = 0;
  for (int k = lo; k < hi; ++k) sum += cnt[k];
  s_part[threadIdx.x] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int k = 0; k < blockDim.x; ++k) {
      const int v = s_part[k];
      s_part[k] = acc;
      acc += v;
    }
    s_off[W] = acc;
  }
  __syncthreads();
  int acc = s_part[threadIdx.x];
  for (int k = lo; k < hi; ++k) {
    s_off[k] = acc;
    acc += cnt[k];
  }
  __syncthreads();
}

template <bool DISPATCH>
__global__ void __launch_bounds__(kThreads)
group_dedup_finalize_kernel(const int64_t* __restrict__ ids, int n, GroupDesc d, int world, DedupEntry* table,
                            const int* __restrict__ slot_of, const int* __restrict__ cnt, int* off, int64_t* uniq,
                            int* inv, int cap_u, int* status, Sym sym, ChanLayout lay, Ctrl* ctrl) {
  int* s_occ = g_smem;                     // [T + 1]
  int* s_off = s_occ + d.T + 1;            // [world * T + 1]  exclusive scan over (owner, table) cells
  int* s_part = s_off + world * d.T + 1;   // [blockDim.x]
  const int W = world * d.T;
  for (int k = threadIdx.x; k <= d.T; k += blockDim.x) s_occ[k] = d.occ_start[k];
  block_exclusive_scan(cnt, W, s_off, s_part);
  const int total = s_off[W];
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) {
      if (total > cap_u) set_status(status, err::kInboxOverflow);
      if (DISPATCH && total > lay.capU) set_status(&ctrl->status, err::kInboxOverflow);
    }
    for (int o = threadIdx.x; o <= world; o += blockDim.x) off[o] = min(o < world ? s_off[o * d.T] : total, cap_u);
    if (DISPATCH) {
      // to every owner: how many ids this rank sends, where their rows go, and the per-table prefix
      for (int o = threadIdx.x; o < world; o += blockDim.x) {
        const int lo = min(s_off[o * d.T], cap_u), hi = min(s_off[(o + 1) * d.T], cap_u);
        const int2 m = make_int2(min(hi - lo, lay.capS), lo);
        sym.at<int2>(o, lay.inbox_meta)[sym.rank] = m;
        if (o == sym.rank) ctrl->snap[o] = m;
      }
      for (int k = threadIdx.x; k < world * (d.T + 1); k += blockDim.x) {
        const int o = k / (d.T + 1), t = k % (d.T + 1);
        const int lo = min(s_off[o * d.T], cap_u), at = min(s_off[o * d.T + t], cap_u);
        sym.at<int>(o, lay.inbox_tcnt)[static_cast<size_t>(sym.rank) * (d.T + 1) + t] = min(at - lo, lay.capS);
      }
    }
  }
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    uint64_t id = static_cast<uint64_t>(ids[i]);
    if (id == kEmptyKey) id = kEmptyKey - 1;
    const int t = segment_of(s_occ, d.T, i);
    const int slot = slot_of[i];
    const int o = static_cast<int>(OwnerOf(d.salt[t], id, d.owner_world));
    const unsigned long long pw = __ldcg(&table[slot].pos_win);
    const int u = s_off[o * d.T + t] + static_cast<int>(static_cast<uint32_t>(pw));
    inv[i] = u < cap_u ? u : 0;
    if (static_cast<int>(pw >> 32) == i) {
      if (u < cap_u) {
        uniq[u] = static_cast<int64_t>(id);
        if (DISPATCH) {
          const int j = u - s_off[o * d.T];  // position inside the segment this rank sends to owner o
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

// Request rendezvous of a group: waits (bounded) for every source's ids, then copies the peer-writable
// counts and per-table prefixes into local memory, which is what the owner-side kernels read.
__global__ void __launch_bounds__(kThreads)
group_wait_request_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, int T, int* snap_t, uint32_t spin_limit) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (sym.world > 1 && threadIdx.x < sym.world &&
      !wait_flag(sym.at<uint32_t>(sym.rank, lay.flag_req) + threadIdx.x, ctrl->pull_epoch, spin_limit))
    s_ok = 0;
  __syncthreads();
  const bool ok = s_ok != 0;
  if (ok) {
    if (threadIdx.x < sym.world) ctrl->snap[threadIdx.x] = __ldcg(sym.at<int2>(sym.rank, lay.inbox_meta) + threadIdx.x);
    const int* src = sym.at<int>(sym.rank, lay.inbox_tcnt);
    for (int k = threadIdx.x; k < sym.world * (T + 1); k += blockDim.x) snap_t[k] = __ldcg(src + k);
  }
  if (threadIdx.x == 0) {
    ctrl->abort = ok ? 0 : 1;
    if (!ok) set_status(&ctrl->status, err::kTimeout);
  }
}

template <int VEC>
__global__ void __launch_bounds__(kThreads)
group_probe_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, const TableView* __restrict__ tv, int T,
                   const int* __restrict__ snap_t, int* slot_cache, int16_t* ttab, int insert, int chunks, int lpr) {
  if (ctrl->abort) return;
  int* s_pre = g_smem;  // [T + 1] prefix of the source being served
  const unsigned long long* inbox = sym.at<unsigned long long>(sym.rank, lay.inbox_ids);
  const int lane = threadIdx.x & 31;
  const int rows_per_pass = 32 / lpr;
  for (int k = 0; k < sym.world; ++k) {
    const int s = (sym.rank + k) % sym.world;
    const int cnt = ctrl->snap[s].x;
    __syncthreads();
    for (int q = threadIdx.x; q <= T; q += blockDim.x) s_pre[q] = snap_t[s * (T + 1) + q];
    __syncthreads();
    for (int base = blockIdx.x * blockDim.x; base < cnt; base += gridDim.x * blockDim.x) {
      const int j = base + threadIdx.x;
      bool created = false;
      int slot = -1, t = 0;
      uint64_t id = 0;
      if (j < cnt) {
        const size_t e = static_cast<size_t>(s) * lay.capS + j;
        id = __ldcg(&inbox[e]);
        t = segment_of(s_pre, T, j);
        slot = table_find_or_insert(tv[t], id, insert != 0, &created);
        if (slot < 0 && !insert) set_status(&ctrl->status, err::kSparseIdNotExist);
        slot_cache[e] = slot;
        ttab[e] = static_cast<int16_t>(t);
      }
      // rows created by this warp: counted per table, then initialised by the whole warp, lpr lanes per row
      unsigned todo = __ballot_sync(0xffffffffu, created);
      if (created) atomicAdd(tv[t].size, 1);
      while (todo) {
        int src = -1;
        unsigned rest = todo;
        for (int g = 0; g < rows_per_pass && rest; ++g) {
          const int l = __ffs(rest) - 1;
          rest &= rest - 1;
          if (g == lane / lpr) src = l;
        }
        todo = rest;
        const int r_slot = __shfl_sync(0xffffffffu, slot, src < 0 ? 0 : src);
        const int r_t = __shfl_sync(0xffffffffu, t, src < 0 ? 0 : src);
        const uint64_t r_id = __shfl_sync(0xffffffffu, id, src < 0 ? 0 : src);
        if (src >= 0) {
          const TableView& tb = tv[r_t];
          float* row = tb.val + static_cast<size_t>(r_slot) * tb.dim;
          for (int c = lane % lpr; c < chunks; c += lpr) {
            float q[4];
            if (VEC == 4) {
              InitQuad(tb.init, tb.seed_key, r_id, c, tb.dim, q);
              *reinterpret_cast<float4*>(row + c * 4) = make_float4(q[0], q[1], q[2], q[3]);
            } else {
              InitQuad(tb.init, tb.seed_key, r_id, c >> 2, tb.dim, q);
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
group_gather_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, const TableView* __restrict__ tv,
                    const int* __restrict__ slot_cache, const int16_t* __restrict__ ttab, int dim, int chunks, int lpr) {
  using V = Vec<VEC>;
  const bool aborted = ctrl->abort != 0;
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int row0 = gtid / lpr;
  const int row_stride = (gridDim.x * blockDim.x) / lpr;
  constexpr int kUnroll = 4;
  for (int k = 0; k < sym.world; ++k) {
    const int s = (sym.rank + k) % sym.world;
    int2 m = ctrl->snap[s];
    if (aborted) m.x = 0;
    float* dst_base = sym.at<float>(s, lay.rows_recv) + static_cast<size_t>(m.y) * dim;
    const size_t e0 = static_cast<size_t>(s) * lay.capS;
    for (int r = row0; r < m.x; r += row_stride * kUnroll) {
      const float* src[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int ru = r + u * row_stride;
        src[u] = nullptr;
        if (ru < m.x) {
          const int slot = slot_cache[e0 + ru];
          if (slot >= 0) src[u] = tv[ttab[e0 + ru]].val + static_cast<size_t>(slot) * dim;
        }
      }
      for (int c = lane; c < chunks; c += lpr) {
        typename V::T v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) v[u] = src[u] ? V::ld(src[u] + c * VEC) : V::zero();
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int ru = r + u * row_stride;
          if (ru < m.x) V::st(dst_base + static_cast<size_t>(ru) * dim + c * VEC, v[u]);
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
group_push_merge_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, const TableView* __restrict__ tv,
                        const int* __restrict__ slot_cache, const int16_t* __restrict__ ttab, int dim, int chunks,
                        int lpr) {
  using V = Vec<VEC>;
  if (ctrl->abort) return;
  const uint32_t epoch = ctrl->push_epoch;
  float* inbox = sym.at<float>(sym.rank, lay.inbox_grad);
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int row_stride = (gridDim.x * blockDim.x) / lpr;
  const unsigned group_mask = (lpr == 32 ? 0xffffffffu : ((1u << lpr) - 1u)) << ((threadIdx.x & 31) / lpr * lpr);
  for (int s = 0; s < sym.world; ++s) {
    const int cnt = ctrl->snap[s].x;
    const int rounds = (cnt + row_stride - 1) / row_stride;
    for (int it = 0; it < rounds; ++it) {
      const int r = gtid / lpr + it * row_stride;
      unsigned leader = 0xffffffffu;
      unsigned entry = 0;
      if (r < cnt) {
        entry = static_cast<unsigned>(s) * lay.capS + r;
        const int slot = slot_cache[entry];
        if (lane == 0 && slot >= 0) {
          unsigned long long* lead = tv[ttab[entry]].lead;
          const unsigned long long mine = (static_cast<unsigned long long>(epoch) << 32) | entry;
          unsigned long long old = lead[slot];
          while (static_cast<uint32_t>(old >> 32) != epoch) {
            const unsigned long long prev = atomicCAS(&lead[slot], old, mine);
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
        const float* src = inbox + static_cast<size_t>(entry) * dim;
        float* dst = inbox + static_cast<size_t>(leader) * dim;
        for (int c = lane; c < chunks; c += lpr) V::red(dst + c * VEC, V::ldcg(src + c * VEC));
      }
    }
  }
}

template <int VEC, int OPT>
__global__ void __launch_bounds__(kThreads, 4)
group_push_update_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, const TableView* __restrict__ tv,
                         const int* __restrict__ slot_cache, const int16_t* __restrict__ ttab, OptimPOD optim_in,
                         const float* __restrict__ lr_ptr, int dim, int chunks, int lpr) {
  using V = Vec<VEC>;
  if (ctrl->abort) return;
  OptimPOD optim = optim_in;
  optim.type = OPT;
  const uint32_t epoch = ctrl->push_epoch;
  const float* inbox = sym.at<float>(sym.rank, lay.inbox_grad);
  const float lr = *lr_ptr;
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int row_stride = (gridDim.x * blockDim.x) / lpr;
  const unsigned group_mask = (lpr == 32 ? 0xffffffffu : ((1u << lpr) - 1u)) << ((threadIdx.x & 31) / lpr * lpr);
  for (int s = 0; s < sym.world; ++s) {
    const int cnt = ctrl->snap[s].x;
    for (int r = gtid / lpr; r < cnt; r += row_stride) {
      const unsigned entry = static_cast<unsigned>(s) * lay.capS + r;
      const int slot = slot_cache[entry];
      if (slot < 0) continue;
      const TableView& t = tv[ttab[entry]];
      if (sym.world > 1 && t.lead[slot] != ((static_cast<unsigned long long>(epoch) << 32) | entry)) continue;
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
      const size_t row = static_cast<size_t>(slot) * dim;
      for (int c = lane; c < chunks; c += lpr) {
        float g[VEC], w[VEC], a0[VEC], a1[VEC], a2[VEC];
        *reinterpret_cast<typename V::T*>(g) = V::ldcg(inbox + static_cast<size_t>(entry) * dim + c * VEC);
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

template <int VEC>
void launch_group_update(int grid, cudaStream_t stream, const Sym& s, const ChanLayout& lay, Ctrl* ctrl,
                         const TableView* tv, const int* slot_cache, const int16_t* ttab, const OptimPOD& optim,
                         const float* lr, int dim, int chunks, int lpr) {
  switch (optim.type) {
    case 0: group_push_update_kernel<VEC, 0><<<grid, kThreads, 0, stream>>>(s, lay, ctrl, tv, slot_cache, ttab, optim, lr, dim, chunks, lpr); break;
    case 1: group_push_update_kernel<VEC, 1><<<grid, kThreads, 0, stream>>>(s, lay, ctrl, tv, slot_cache, ttab, optim, lr, dim, chunks, lpr); break;
    case 2: group_push_update_kernel<VEC, 2><<<grid, kThreads, 0, stream>>>(s, lay, ctrl, tv, slot_cache, ttab, optim, lr, dim, chunks, lpr); break;
    default: group_push_update_kernel<VEC, 3><<<grid, kThreads, 0, stream>>>(s, lay, ctrl, tv, slot_cache, ttab, optim, lr, dim, chunks, lpr); break;
  }
}

}  // namespace

// ------------------------------------------------------------------ launchers
void group_table_views(const TableHost* tables, int T, void* out_host) {
  TableView* tv = static_cast<TableView*>(out_host);
  for (int t = 0; t < T; ++t) tv[t] = to_view(tables[t]);
}

size_t group_table_view_bytes() { return sizeof(TableView); }

void group_dedup_dispatch(const int64_t* ids, int n, const GroupDesc& d, int world, DedupScratch sc, int* cnt,
                          int* off, int64_t* uniq, int* inv, int cap_u, int* status, SymHost sym, ChanLayout lay,
                          Ctrl* ctrl, cudaStream_t stream) {
  const int W = world * d.T;
  cudaMemsetAsync(cnt, 0, sizeof(int) * W, stream);
  const int blocks = n > 0 ? (n + kThreads - 1) / kThreads : 1;
  const size_t sm1 = sizeof(int) * (d.T + 1 + 2 * W);
  const size_t sm2 = sizeof(int) * (d.T + 1 + W + 1 + kThreads);
  if (n > 0)
    group_dedup_insert_kernel<<<blocks, kThreads, sm1, stream>>>(ids, n, d, world, static_cast<DedupEntry*>(sc.table),
                                                                 sc.slot_of, cnt, status);
  group_dedup_finalize_kernel<true><<<blocks, kThreads, sm2, stream>>>(ids, n, d, world,
                                                                       static_cast<DedupEntry*>(sc.table), sc.slot_of,
                                                                       cnt, off, uniq, inv, cap_u, status, to_sym(sym),
                                                                       lay, ctrl);
}

void group_probe(SymHost sym, ChanLayout lay, Ctrl* ctrl, const void* table_views, int T, int dim, int* snap_t,
                 int* slot_cache, int16_t* ttab, bool insert, uint32_t spin_limit, cudaStream_t stream) {
  const Sym s = to_sym(sym);
  const TableView* tv = static_cast<const TableView*>(table_views);
  group_wait_request_kernel<<<1, kThreads, 0, stream>>>(s, lay, ctrl, T, snap_t, spin_limit);
  const RowGeom g = row_geom(dim);
  const int grid = grid_for(static_cast<long long>(lay.capS));
  const size_t sm = sizeof(int) * (T + 1);
  if (g.vec == 4)
    group_probe_kernel<4><<<grid, kThreads, sm, stream>>>(s, lay, ctrl, tv, T, snap_t, slot_cache, ttab, insert ? 1 : 0,
                                                          g.chunks, g.lpr);
  else
    group_probe_kernel<1><<<grid, kThreads, sm, stream>>>(s, lay, ctrl, tv, T, snap_t, slot_cache, ttab, insert ? 1 : 0,
                                                          g.chunks, g.lpr);
}

void group_gather(SymHost sym, ChanLayout lay, Ctrl* ctrl, const void* table_views, int dim, const int* slot_cache,
                  const int16_t* ttab, cudaStream_t stream) {
  const TableView* tv = static_cast<const TableView*>(table_views);
  const RowGeom g = row_geom(dim);
  const int grid = grid_for(static_cast<long long>(lay.capS) * g.lpr);
  if (g.vec == 4)
    group_gather_kernel<4><<<grid, kThreads, 0, stream>>>(to_sym(sym), lay, ctrl, tv, slot_cache, ttab, dim, g.chunks, g.lpr);
  else
    group_gather_kernel<1><<<grid, kThreads, 0, stream>>>(to_sym(sym), lay, ctrl, tv, slot_cache, ttab, dim, g.chunks, g.lpr);
}

void group_push_apply(SymHost sym, ChanLayout lay, Ctrl* ctrl, const void* table_views, int dim, const int* slot_cache,
                      const int16_t* ttab, OptimPOD optim, const float* lr, uint32_t spin_limit, cudaStream_t stream) {
  const TableView* tv = static_cast<const TableView*>(table_views);
  const RowGeom g = row_geom(dim);
  const int grid = grid_for(static_cast<long long>(lay.capS) * g.lpr);
  const Sym s = to_sym(sym);
  if (sym.world > 1) exchange_wait(sym, lay, ctrl, 2, spin_limit, stream);
  if (g.vec == 4) {
    if (sym.world > 1)
      group_push_merge_kernel<4><<<grid, kThreads, 0, stream>>>(s, lay, ctrl, tv, slot_cache, ttab, dim, g.chunks, g.lpr);
    launch_group_update<4>(grid, stream, s, lay, ctrl, tv, slot_cache, ttab, optim, lr, dim, g.chunks, g.lpr);
  } else {
    if (sym.world > 1)
      group_push_merge_kernel<1><<<grid, kThreads, 0, stream>>>(s, lay, ctrl, tv, slot_cache, ttab, dim, g.chunks, g.lpr);
    launch_group_update<1>(grid, stream, s, lay, ctrl, tv, slot_cache, ttab, optim, lr, dim, g.chunks, g.lpr);
  }
}

}  // namespace cu
}  // namespace kb
