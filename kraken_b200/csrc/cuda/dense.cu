// Dense-parameter step fused with its collective, and the DCT kernels.
//
// dense_step is one short launch sequence per rank that does what the reference does with a
// push RPC per table, a server-side optimizer and a pull RPC per step
// (kraken/worker/emitter.cc:377-447, kraken/ps/dense_table.cc:31-43,
// kraken/pytorch/optimizer.py:151-173):
//
//   1. one warp raises "my gradient is complete" on every peer (release store) and
//      waits (bounded) for the same flag from every rank;
//   2. the update grid, for the slice this rank owns: sums the slice of every
//      rank's gradient buffer directly out of peer memory (reduce-scatter by
//      loads), runs the optimizer on value + slice-local state, stores the new
//      values into every rank's parameter copy (all-gather by stores);
//   3. one warp raises "slice done" on every peer, counts the step, and waits for
//      "slice done" of all owners, after which a grid zeroes the local gradient
//      buffer for the next backward.
// The waits and signals are separate one-warp launches so that no block of a large
// grid spins, or ends on a fence that waits for the switch, while holding registers
// another stream's kernels need; on a single GPU the call is the update grid alone
// (which then also clears the gradient it has just read).
//
// With DCT the gradients do not travel dense: dct_compact turns the local
// f = g + e into per-owner (index, value) lists and the owner scatter-adds the
// lists of all ranks (dense_gather_coo) before step 3 reads its accumulator.
// DCT here is Dynamic Communication Thresholding, kraken/worker/dct_emitter.cc:16-43.
#include <algorithm>
#include <stdexcept>
#include <string>

#include "common.cuh"
#include "dense_kernels.h"

namespace kb {
namespace cu {

namespace {

constexpr int kThreads = 256;

Sym to_sym(const SymHost& h) {
  Sym s;
  for (int i = 0; i < kMaxWorld; ++i) s.base[i] = static_cast<char*>(h.base[i]);
  s.rank = h.rank;
  s.world = h.world;
  return s;
}

// phase 0: announce this rank's gradient and wait for every rank's.
// phase 1 (launched behind the update grid): tell every rank that this rank's slice is written, count the
// step of the tables that took part, then wait until every owner has written its slice.  The update grid
// itself signals nothing: its stores into peer memory are complete when it has ended, which stream order
// puts before this kernel, so no block of it has to end on a fence that waits for the switch.
// One warp, lane p talks to peer p.
__global__ void dense_rendezvous_kernel(Sym sym, DenseLayout lay, DenseCtrl* ctrl, int phase, uint32_t spin_limit,
                                        int* table_steps, const uint8_t* __restrict__ table_active, int n_tables) {
  const int p = threadIdx.x;
  const uint32_t epoch = ctrl->epoch + 1;
  bool ok = true;
  if (phase == 1) __threadfence_system();
  if (p < sym.world) {
    st_release_sys(sym.at<uint32_t>(p, phase == 0 ? lay.flag_grad : lay.flag_done) + sym.rank, epoch);
    ok = wait_flag(sym.at<uint32_t>(sym.rank, phase == 0 ? lay.flag_grad : lay.flag_done) + p, epoch, spin_limit);
  }
  const bool all_ok = __all_sync(0xffffffffu, ok);
  if (phase == 1) {
    const bool aborted = ctrl->abort != 0;
    for (int t = p; t < n_tables && !aborted; t += 32)
      if (table_active[t]) table_steps[t] += 1;
    __syncwarp();
  }
  if (p == 0) {
    if (!all_ok) {
      set_status(&ctrl->status, err::kTimeout);
      ctrl->abort = 1;
    } else if (phase == 0) {
      ctrl->abort = 0;
    }
    if (phase == 1) ctrl->epoch = epoch;
  }
}

__global__ void __launch_bounds__(kThreads)
dense_zero_kernel(Sym sym, DenseLayout lay, long long n_pad, int use_coo) {
  const long long gtid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long gsize = static_cast<long long>(gridDim.x) * blockDim.x;
  float4* gz = reinterpret_cast<float4*>(sym.at<float>(sym.rank, lay.grad));
  for (long long q = gtid; q * 4 < n_pad; q += gsize) gz[q] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (use_coo && gtid < sym.world) sym.at<int>(sym.rank, lay.coo_cnt)[gtid] = 0;
}

// Owner side of the DCT exchange: scatter-add every rank's list into acc[slice].
__global__ void __launch_bounds__(kThreads)
dense_gather_coo_kernel(Sym sym, DenseLayout lay, DenseCtrl* ctrl, long long slice, float* acc) {
  if (ctrl->abort) return;
  const long long gtid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long gsize = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int k = 0; k < sym.world; ++k) {
    const int p = (sym.rank + k) % sym.world;
    const int cnt = __ldcg(sym.at<int>(p, lay.coo_cnt) + sym.rank);
    const int* idx = sym.at<int>(p, lay.coo_idx) + static_cast<size_t>(sym.rank) * slice;
    const float* val = sym.at<float>(p, lay.coo_val) + static_cast<size_t>(sym.rank) * slice;
    for (long long j = gtid; j < cnt; j += gsize) {
      const int i = __ldcg(idx + j);
      if (i >= 0 && i < slice) atomicAdd(acc + i, __ldcg(val + j));
    }
  }
}

// The update grid.  OPT fixes the optimizer type at compile time (-1: read it from the descriptor) and
// SLABS is the bit mask of state slabs that exist, so that an SGD-momentum step carries 12 registers of
// payload per float4 group instead of 20 and the switch in UpdateElem folds away.  A block handles kIlp
// consecutive runs of 256 float4 groups and every load of a thread is issued before the first is used:
// HBM needs ~45 KB of reads in flight per SM all the time, and a thread alternates between a load and a
// store phase, so the SM must hold several times that in resident threads x bytes per thread.
template <int OPT, int SLABS, bool MULTI>
__global__ void __launch_bounds__(kThreads)
dense_step_kernel(Sym sym, DenseLayout lay, DenseCtrl* ctrl, long long n_pad, float* __restrict__ s0,
                  float* __restrict__ s1, float* __restrict__ s2, float* acc, const int* __restrict__ chunk_table,
                  int* table_steps, const uint8_t* __restrict__ table_active, int n_tables, OptimPOD optim,
                  const float* __restrict__ lr_ptr, float grad_scale, int use_coo) {
  constexpr int kIlp = MULTI ? 2 : 4;  // with peers every group also has world - 1 loads from peer memory in flight
  constexpr bool kS0 = (SLABS & 1) != 0, kS1 = (SLABS & 2) != 0, kS2 = (SLABS & 4) != 0;
  if (OPT >= 0) optim.type = static_cast<uint8_t>(OPT);
  const uint32_t epoch = ctrl->epoch + 1;
  const int world = MULTI ? sym.world : 1;
  const long long slice = n_pad / world;
  const long long base = slice * (MULTI ? sym.rank : 0);
  const float lr = *lr_ptr;
  const bool aborted = ctrl->abort != 0;  // a peer's gradient never arrived: change nothing, keep the flags moving
  float* const param = sym.at<float>(sym.rank, lay.param);
  float* const grad = sym.at<float>(sym.rank, lay.grad);

  const long long groups = slice / 4;
  const long long per_block = static_cast<long long>(kThreads) * kIlp;
  for (long long b0 = blockIdx.x * per_block; b0 < groups && !aborted; b0 += gridDim.x * per_block) {
    long long li[kIlp];
    int tab[kIlp];
    bool inside[kIlp];
    float4 g[kIlp], w[kIlp], a0[kIlp], a1[kIlp], a2[kIlp];
#pragma unroll
    for (int u = 0; u < kIlp; ++u) {
      const long long q = b0 + u * kThreads + threadIdx.x;
      li[u] = q * 4;  // offset inside the slice; base + li is the offset inside the flat buffer
      inside[u] = q < groups;
      tab[u] = inside[u] ? chunk_table[(base + li[u]) / kDenseChunk] : -1;
      g[u] = a0[u] = a1[u] = a2[u] = w[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      // none of the loads below waits for the table lookup above: a chunk that takes no update is read all the same
      if (!inside[u]) continue;
      w[u] = *reinterpret_cast<const float4*>(param + base + li[u]);
      if (kS0) a0[u] = *reinterpret_cast<const float4*>(s0 + li[u]);
      if (kS1) a1[u] = *reinterpret_cast<const float4*>(s1 + li[u]);
      if (kS2) a2[u] = *reinterpret_cast<const float4*>(s2 + li[u]);
      if (use_coo) {
        g[u] = *reinterpret_cast<const float4*>(acc + li[u]);
      } else if (!MULTI) {
        g[u] = __ldcs(reinterpret_cast<const float4*>(grad + li[u]));
      } else {
        // four peers' slices requested before the first is added (a peer load is a round trip over the switch)
        for (int k0 = 0; k0 < world; k0 += 4) {
          float4 v[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k0 + j < world) {
              const int p = (sym.rank + k0 + j) % world;
              v[j] = __ldcg(reinterpret_cast<const float4*>(sym.at<float>(p, lay.grad) + base + li[u]));
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) g[u].x += v[j].x, g[u].y += v[j].y, g[u].z += v[j].z, g[u].w += v[j].w;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kIlp; ++u) {
      if (!inside[u]) continue;
      if (use_coo) *reinterpret_cast<float4*>(acc + li[u]) = make_float4(0.f, 0.f, 0.f, 0.f);
      // single GPU: nobody else reads this gradient, so it is cleared for the next backward here
      if (!MULTI) __stcs(reinterpret_cast<float4*>(grad + li[u]), make_float4(0.f, 0.f, 0.f, 0.f));
      if (tab[u] < 0 || !table_active[tab[u]]) continue;
      const int64_t step = static_cast<int64_t>(table_steps[tab[u]]) + 1;
      const AdamBias ab = optim.type == 1 ? AdamBiasAt(optim, step) : AdamBias{1.f, 1.f};
      UpdateElem(optim, lr, g[u].x * grad_scale, step, ab, w[u].x, a0[u].x, a1[u].x, a2[u].x);
      UpdateElem(optim, lr, g[u].y * grad_scale, step, ab, w[u].y, a0[u].y, a1[u].y, a2[u].y);
      UpdateElem(optim, lr, g[u].z * grad_scale, step, ab, w[u].z, a0[u].z, a1[u].z, a2[u].z);
      UpdateElem(optim, lr, g[u].w * grad_scale, step, ab, w[u].w, a0[u].w, a1[u].w, a2[u].w);
      if (kS0) *reinterpret_cast<float4*>(s0 + li[u]) = a0[u];
      if (kS1) *reinterpret_cast<float4*>(s1 + li[u]) = a1[u];
      if (kS2) *reinterpret_cast<float4*>(s2 + li[u]) = a2[u];
      if (!MULTI) {
        *reinterpret_cast<float4*>(param + li[u]) = w[u];
      } else {
        for (int k = 0; k < world; ++k) {
          const int p = (sym.rank + k) % world;
          *reinterpret_cast<float4*>(sym.at<float>(p, lay.param) + base + li[u]) = w[u];
        }
      }
    }
  }

  if (MULTI) return;  // the one-warp launch behind this grid publishes the slice and counts the step
  if (last_block_done(&ctrl->done[0])) {
    for (int t = threadIdx.x; t < n_tables; t += blockDim.x)
      if (table_active[t]) table_steps[t] += 1;
    if (threadIdx.x == 0) ctrl->epoch = epoch;
  }
  if (use_coo && blockIdx.x == 0 && threadIdx.x == 0) sym.at<int>(sym.rank, lay.coo_cnt)[0] = 0;
}

template <int OPT, int SLABS>
void launch_dense_step(bool multi, int grid, cudaStream_t stream, Sym s, DenseLayout lay, DenseCtrl* ctrl,
                       long long n_pad, float* s0, float* s1, float* s2, float* acc, const int* chunk_table,
                       int* table_steps, const uint8_t* table_active, int n_tables, OptimPOD optim, const float* lr,
                       float grad_scale, int use_coo) {
  if (multi)
    dense_step_kernel<OPT, SLABS, true><<<grid, kThreads, 0, stream>>>(
        s, lay, ctrl, n_pad, s0, s1, s2, acc, chunk_table, table_steps, table_active, n_tables, optim, lr, grad_scale,
        use_coo);
  else
    dense_step_kernel<OPT, SLABS, false><<<grid, kThreads, 0, stream>>>(
        s, lay, ctrl, n_pad, s0, s1, s2, acc, chunk_table, table_steps, table_active, n_tables, optim, lr, grad_scale,
        use_coo);
}

// ------------------------------------------------------------------ DCT
__global__ void dct_accumulate_kernel(float* __restrict__ grad, const float* __restrict__ residual, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    grad[i] += residual[i];
}

// prefix_state[0] = bits fixed so far, prefix_state[1] = k still to skip from the top.
__global__ void __launch_bounds__(kThreads)
radix_hist_kernel(const float* __restrict__ x, long long n, int pass, const uint32_t* __restrict__ prefix_state,
                  uint32_t* hist) {
  __shared__ uint32_t sh[256];
  sh[threadIdx.x] = 0;
  __syncthreads();
  const int shift = 24 - 8 * pass;
  const uint32_t prefix = prefix_state[0];
  const uint32_t hi_mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint32_t b = __float_as_uint(x[i]) & 0x7FFFFFFFu;
    if ((b & hi_mask) == prefix) atomicAdd(&sh[(b >> shift) & 0xFFu], 1u);
  }
  __syncthreads();
  if (sh[threadIdx.x]) atomicAdd(&hist[pass * 256 + threadIdx.x], sh[threadIdx.x]);
}

__global__ void radix_pick_kernel(int pass, uint32_t* prefix_state, const uint32_t* __restrict__ hist, float* tau) {
  if (threadIdx.x != 0) return;
  const int shift = 24 - 8 * pass;
  uint32_t k = prefix_state[1];
  int d = 255;
  for (; d > 0; --d) {
    const uint32_t c = hist[pass * 256 + d];
    if (c >= k) break;
    k -= c;
  }
  prefix_state[0] |= static_cast<uint32_t>(d) << shift;
  prefix_state[1] = k;
  if (pass == 3) *tau = __uint_as_float(prefix_state[0]);
}

__global__ void radix_init_kernel(uint32_t* prefix_state, uint32_t* hist, uint32_t k) {
  for (int i = threadIdx.x; i < 4 * 256; i += blockDim.x) hist[i] = 0;
  if (threadIdx.x == 0) {
    prefix_state[0] = 0;
    prefix_state[1] = k;
  }
}

__global__ void __launch_bounds__(kThreads)
dct_compact_kernel(Sym sym, DenseLayout lay, long long n_pad, float* __restrict__ residual,
                   const float* __restrict__ tau_table, const int* __restrict__ chunk_table) {
  const long long slice = n_pad / sym.world;
  float* grad = sym.at<float>(sym.rank, lay.grad);
  int* cnt = sym.at<int>(sym.rank, lay.coo_cnt);
  int* idx = sym.at<int>(sym.rank, lay.coo_idx);
  float* val = sym.at<float>(sym.rank, lay.coo_val);
  const int lane = threadIdx.x & 31;
  for (long long base = blockIdx.x * static_cast<long long>(blockDim.x); base < n_pad;
       base += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long i = base + threadIdx.x;  // n_pad is a multiple of 256: always in range
    const float f = grad[i];
    const int t = chunk_table[i / kDenseChunk];
    const bool keep = t >= 0 && fabsf(f) >= tau_table[t];
    // a warp's 32 elements share an owner: slices are multiples of 256 elements
    const int owner = static_cast<int>(i / slice);
    const unsigned m = __ballot_sync(0xffffffffu, keep);
    int wbase = 0;
    if (m != 0 && lane == __ffs(m) - 1) wbase = atomicAdd(&cnt[owner], __popc(m));
    wbase = __shfl_sync(0xffffffffu, wbase, m ? __ffs(m) - 1 : 0);
    if (keep) {
      const long long pos = static_cast<long long>(owner) * slice + wbase + __popc(m & ((1u << lane) - 1));
      idx[pos] = static_cast<int>(i - static_cast<long long>(owner) * slice);
      val[pos] = f;
    }
    residual[i] = keep ? 0.f : f;
    grad[i] = 0.f;
  }
}

__global__ void dct_threshold_dense_kernel(float* __restrict__ grad, float* __restrict__ residual, long long n,
                                           const float* __restrict__ tau_table, const int* __restrict__ chunk_table) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float f = grad[i];
    const int t = chunk_table[i / kDenseChunk];
    const bool keep = t >= 0 && fabsf(f) >= tau_table[t];
    grad[i] = keep ? f : 0.f;
    residual[i] = keep ? 0.f : f;
  }
}

int grid_for(long long items, int cap = 148 * 4) {
  long long g = (items + kThreads - 1) / kThreads;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return static_cast<int>(g);
}

}  // namespace

void dense_step(SymHost sym, DenseLayout lay, DenseCtrl* ctrl, long long n_pad, float* s0, float* s1, float* s2,
                float* acc, const int* chunk_table, int* table_steps, const uint8_t* table_active, int n_tables,
                OptimPOD optim, const float* lr, float grad_scale, int use_coo, uint32_t spin_limit,
                cudaStream_t stream) {
  const long long slice = n_pad / sym.world;
  const Sym s = to_sym(sym);
  const bool multi = sym.world > 1;
  // one pass per block: short-lived blocks keep the loads of some blocks and the stores of others in flight
  // at the same time; the kernel strides where the grid would exceed 2^20 blocks
  const int per_block = kThreads * (multi ? 2 : 4);
  const int grid = static_cast<int>(std::min<long long>((slice / 4 + per_block - 1) / per_block, 1 << 20));
  if (multi)
    dense_rendezvous_kernel<<<1, 32, 0, stream>>>(s, lay, ctrl, 0, spin_limit, table_steps, table_active, n_tables);
  if (use_coo) dense_gather_coo_kernel<<<grid_for(slice / 4, 148 * 8), kThreads, 0, stream>>>(s, lay, ctrl, slice, acc);
  const int slabs = (s0 ? 1 : 0) | (s1 ? 2 : 0) | (s2 ? 4 : 0);
#define KB_DENSE_STEP(OPT, SLABS)                                                                                    \
  launch_dense_step<OPT, SLABS>(multi, grid, stream, s, lay, ctrl, n_pad, s0, s1, s2, acc, chunk_table, table_steps, \
                                table_active, n_tables, optim, lr, grad_scale, use_coo)
  const int key = optim.type * 8 + slabs;
  switch (key) {
    case 0 * 8 + 1: KB_DENSE_STEP(0, 1); break;  // Adagrad
    case 1 * 8 + 3: KB_DENSE_STEP(1, 3); break;  // Adam
    case 1 * 8 + 7: KB_DENSE_STEP(1, 7); break;  // Adam, amsgrad
    case 2 * 8 + 1: KB_DENSE_STEP(2, 1); break;  // RMSprop
    case 2 * 8 + 3: KB_DENSE_STEP(2, 3); break;  //   centered
    case 2 * 8 + 5: KB_DENSE_STEP(2, 5); break;  //   momentum
    case 2 * 8 + 7: KB_DENSE_STEP(2, 7); break;  //   centered, momentum
    case 3 * 8 + 0: KB_DENSE_STEP(3, 0); break;  // SGD
    case 3 * 8 + 1: KB_DENSE_STEP(3, 1); break;  // SGD, momentum
    default:
      throw std::invalid_argument("dense_step: optimizer type " + std::to_string(int(optim.type)) +
                                  " does not go with state slab mask " + std::to_string(slabs));
  }
#undef KB_DENSE_STEP
  if (multi) {
    dense_rendezvous_kernel<<<1, 32, 0, stream>>>(s, lay, ctrl, 1, spin_limit, table_steps, table_active, n_tables);
    dense_zero_kernel<<<grid_for(n_pad / 4, 148 * 8), kThreads, 0, stream>>>(s, lay, n_pad, use_coo);
  }
}

void dct_accumulate(float* grad, const float* residual, long long n, cudaStream_t stream) {
  dct_accumulate_kernel<<<grid_for(n), kThreads, 0, stream>>>(grad, residual, n);
}

void dct_select_tau(const float* x, long long n, long long k, uint32_t* hist, uint32_t* prefix_state, float* tau,
                    cudaStream_t stream) {
  radix_init_kernel<<<1, kThreads, 0, stream>>>(prefix_state, hist, static_cast<uint32_t>(k));
  for (int pass = 0; pass < 4; ++pass) {
    radix_hist_kernel<<<grid_for(n), kThreads, 0, stream>>>(x, n, pass, prefix_state, hist);
    radix_pick_kernel<<<1, 32, 0, stream>>>(pass, prefix_state, hist, tau);
  }
}

void dct_compact(SymHost sym, DenseLayout lay, long long n_pad, float* residual, const float* tau_table,
                 const int* chunk_table, cudaStream_t stream) {
  dct_compact_kernel<<<grid_for(n_pad), kThreads, 0, stream>>>(to_sym(sym), lay, n_pad, residual, tau_table,
                                                               chunk_table);
}

void dct_threshold_dense(float* grad, float* residual, long long n, const float* tau_table, const int* chunk_table,
                         cudaStream_t stream) {
  dct_threshold_dense_kernel<<<grid_for(n), kThreads, 0, stream>>>(grad, residual, n, tau_table, chunk_table);
}

}  // namespace cu
}  // namespace kb
