// tcgen05 GEMM kernels behind linear_forward / linear_dgrad / linear_wgrad.
//
// All three kernels share one warp-specialised structure per CTA (320 threads):
//   warp 0 (one lane)  TMA producer: fills a ring of shared-memory stages with 128-byte-swizzled
//                      tiles of 64 k-elements, one mbarrier per stage counting bytes;
//   warp 1 (one lane)  MMA issuer: four tcgen05.mma (K = 16 each) per stage into a TMEM
//                      accumulator, tcgen05.commit frees the stage and finally signals the epilogue;
//   warps 2-9          epilogue: two warps per TMEM lane quarter, each taking half of the tile's
//                      columns; tcgen05.ld the accumulator (one row per thread) and fuse bias + ReLU
//                      (+ a one-bit ReLU mask) in the forward pass, the ReLU mask in the input
//                      gradient, or a split-K vector red.add into the fp32 gradient buffer.
// gemm_kernel computes one 128 x BN tile per CTA; gemm_bres_kernel and gemm_pair_kernel are
// persistent, keep their slice of the weights in shared memory and stream activation tiles past it
// with two TMEM accumulators (the pair variant runs tcgen05.mma.cta_group::2 on two CTAs).
// Operands are K-major except in the weight gradient, which contracts over the batch and
// therefore reads both activations MN-major, as they sit in memory.
// Every mbarrier wait is bounded; on a give-up the CTA records kTimeout, lets its outstanding
// TMA copies land, frees its tensor memory and returns.  No TMA load uses cluster multicast.
#include <cuda_bf16.h>

#include <mutex>

#include "../core/types.h"
#include "common.cuh"
#include "mlp_gemm.h"
#include "tcgen05.cuh"

namespace kb {
namespace cu {

namespace {

constexpr int kBM = 128;         // rows of the output tile = TMEM lanes
constexpr int kBK = 64;          // k-elements per stage = one 128-byte swizzle atom of bf16
constexpr int kEpiWarps = 8;     // two warps per TMEM lane quarter, each taking half of the tile's columns
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr int kMaxStages = 8;

enum { EPI_BIAS_ACT = 0, EPI_RELU_MASK = 1, EPI_RED_F32 = 2 };

struct GemmArgs {
  int M, N, K;            // output is M x N, contraction length K
  int BN;                 // tile width (multiple of 16; of 64 when B is MN-major)
  int stages;
  int kb_per_split;       // k-blocks per blockIdx.z
  int relu;
  const float* bias;      // [N]            (EPI_BIAS_ACT)
  const __nv_bfloat16* H; // [M, ldh]       (EPI_RELU_MASK, when no bit mask is given)
  int ldh;
  const uint16_t* mask;   // [chunks, ldm] one bit per element: word (c, r) = columns [16c, 16c + 16) of row r
  uint16_t* mask_out;     // same layout, written by EPI_BIAS_ACT with relu: bit = output > 0
  int ldm;                // row pitch of the mask in words (>= M): a warp's 32 rows are 64 contiguous bytes
  int mask_chunks;        // number of 16-column words per row that the mask holds
  int out_v8;             // bf16 output rows and tile columns are 32-byte aligned: one 256-bit store per chunk
  __nv_bfloat16* out;     // [M, ldo] bf16  (EPI_BIAS_ACT, EPI_RELU_MASK)
  int ldo;
  float* out32;           // [M, ldo32] f32 (EPI_RED_F32)
  int ldo32;
  int* status;
};

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}


// ------------------------------------------------------------------ epilogue
// Slow path for a 16-column chunk that straddles N: the whole warp calls it (the decision depends
// on the column only); it reads the chunk from tensor memory itself and writes element-wise with
// bounds checks, so the fast path never needs its registers in addressable memory.
template <int EPI>
__device__ __noinline__ void epilogue_tail(const GemmArgs& g, const float* s_bias, uint32_t taddr, int row, int col,
                                           int c) {
  uint32_t r[16];
  tc::tmem_ld16(taddr, r);
  tc::tmem_ld_wait();
  if (row >= g.M) return;
  uint32_t bits_out = 0;
  const uint32_t bits_in =
      (EPI == EPI_RELU_MASK && g.mask != nullptr) ? g.mask[static_cast<size_t>(col >> 4) * g.ldm + row] : 0xFFFFu;
  for (int j = 0; j < 16 && col + j < g.N; ++j) {
    float v = __uint_as_float(r[j]);
    if (EPI == EPI_BIAS_ACT) {
      v += s_bias[c + j];
      if (g.relu) v = fmaxf(v, 0.f);
      if (v > 0.f) bits_out |= 1u << j;
    }
    if (EPI == EPI_RELU_MASK && g.mask != nullptr && !((bits_in >> j) & 1u)) v = 0.f;
    if (EPI == EPI_RELU_MASK && g.mask == nullptr && g.H != nullptr &&
        !(__bfloat162float(g.H[static_cast<size_t>(row) * g.ldh + col + j]) > 0.f))
      v = 0.f;
    if (EPI == EPI_RED_F32)
      atomicAdd(g.out32 + static_cast<size_t>(row) * g.ldo32 + col + j, v);
    else
      g.out[static_cast<size_t>(row) * g.ldo + col + j] = __float2bfloat16(v);
  }
  if (EPI == EPI_BIAS_ACT && g.mask_out != nullptr)
    g.mask_out[static_cast<size_t>(col >> 4) * g.ldm + row] = static_cast<uint16_t>(bits_out);
}

// Fast path: all 16 columns valid.  Everything is unrolled with constant indices so the
// accumulator chunk stays in registers.
template <int EPI>
__device__ __forceinline__ void epilogue_full(const GemmArgs& g, const float* s_bias, int row, int col, int c,
                                              const uint32_t (&r)[16], uint32_t keep_bits) {
  float v[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
  if (EPI == EPI_BIAS_ACT) {
    uint32_t bits = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      v[j] += s_bias[c + j];
      if (g.relu) v[j] = fmaxf(v[j], 0.f);
      bits |= (v[j] > 0.f ? 1u : 0u) << j;
    }
    if (g.mask_out != nullptr) g.mask_out[static_cast<size_t>(col >> 4) * g.ldm + row] = static_cast<uint16_t>(bits);
  }
  if (EPI == EPI_RELU_MASK) {
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (!((keep_bits >> j) & 1u)) v[j] = 0.f;
  }
  if (EPI == EPI_RED_F32) {
    float* o = g.out32 + static_cast<size_t>(row) * g.ldo32 + col;
#pragma unroll
    for (int j = 0; j < 16; j += 4)
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + j), "f"(v[j]), "f"(v[j + 1]),
                   "f"(v[j + 2]), "f"(v[j + 3])
                   : "memory");
  } else {
    __nv_bfloat16* o = g.out + static_cast<size_t>(row) * g.ldo + col;
    uint4 w0, w1;
    w0.x = pack_bf16(v[0], v[1]);   w0.y = pack_bf16(v[2], v[3]);
    w0.z = pack_bf16(v[4], v[5]);   w0.w = pack_bf16(v[6], v[7]);
    w1.x = pack_bf16(v[8], v[9]);   w1.y = pack_bf16(v[10], v[11]);
    w1.z = pack_bf16(v[12], v[13]); w1.w = pack_bf16(v[14], v[15]);
    if (g.out_v8) {
      // one 32-byte sector per request: the L2 write-request rate, not bytes, bounds this epilogue
      asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(o), "r"(w0.x), "r"(w0.y), "r"(w0.z),
                   "r"(w0.w), "r"(w1.x), "r"(w1.y), "r"(w1.z), "r"(w1.w)
                   : "memory");
    } else {
      *reinterpret_cast<uint4*>(o) = w0;
      *reinterpret_cast<uint4*>(o + 8) = w1;
    }
  }
}

// 16 keep-bits from 16 bf16 activations: bf16 > 0  <=>  sign bit clear and not zero.
__device__ __forceinline__ uint32_t keep_bits_of(const uint4& h0, const uint4& h1) {
  const uint32_t hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
  uint32_t bits = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t lo = hw[j] & 0xFFFFu, hi = hw[j] >> 16;
    bits |= ((lo != 0u && !(lo & 0x8000u)) ? 1u : 0u) << (2 * j);
    bits |= ((hi != 0u && !(hi & 0x8000u)) ? 1u : 0u) << (2 * j + 1);
  }
  return bits;
}

// The mask words of one row for up to eight 16-column chunks starting at chunk `cb`, packed into
// 128 bits.  Issued before the accumulator wait, so the loads fly while the MMAs run.
struct RowMask {
  unsigned long long lo, hi;
  __device__ __forceinline__ uint32_t chunk(int i) const {
    return static_cast<uint32_t>((i < 4 ? lo >> (16 * i) : hi >> (16 * (i - 4))) & 0xFFFFull);
  }
};

__device__ __forceinline__ RowMask load_row_mask(const GemmArgs& g, int row, int cb, int nchunks) {
  RowMask m{~0ull, ~0ull};
  if (g.mask == nullptr || row >= g.M) return m;
  const uint16_t* p = g.mask + row;
  unsigned long long lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const unsigned long long w =
        (i < nchunks && cb + i < g.mask_chunks) ? __ldg(p + static_cast<size_t>(cb + i) * g.ldm) : 0xFFFFull;
    if (i < 4) lo |= w << (16 * i); else hi |= w << (16 * (i - 4));
  }
  m.lo = lo, m.hi = hi;
  return m;
}

// One epilogue warp's share of a 128 x BN accumulator: TMEM lanes of its quarter (one row per
// thread) and the column range [c_begin, c_end).  Two 16-column chunks are in flight per wait.
template <int EPI>
__device__ __forceinline__ void epilogue_rows(const GemmArgs& g, const float* s_bias, uint32_t t_row, int row, int n0,
                                              int c_begin, int c_end, const RowMask& rm) {
  const bool in_rows = row < g.M;
  // ReLU keep-bits come from the bit mask when there is one (already in registers), else from H
  const bool from_h = EPI == EPI_RELU_MASK && g.mask == nullptr && g.H != nullptr;
  int c = c_begin;
  // pairs of full chunks: both loads are issued before the single wait
  for (; c + 32 <= c_end && n0 + c + 32 <= g.N; c += 32) {
    const int col = n0 + c;
    uint32_t r0[16], r1[16];
    tc::tmem_ld16(t_row + c, r0);
    tc::tmem_ld16(t_row + c + 16, r1);
    uint32_t k0 = rm.chunk((c - c_begin) >> 4), k1 = rm.chunk(((c - c_begin) >> 4) + 1);
    if (from_h && in_rows) {
      const __nv_bfloat16* h = g.H + static_cast<size_t>(row) * g.ldh + col;
      k0 = keep_bits_of(*reinterpret_cast<const uint4*>(h), *reinterpret_cast<const uint4*>(h + 8));
      k1 = keep_bits_of(*reinterpret_cast<const uint4*>(h + 16), *reinterpret_cast<const uint4*>(h + 24));
    }
    tc::tmem_ld_wait();
    if (in_rows) {
      epilogue_full<EPI>(g, s_bias, row, col, c, r0, k0);
      epilogue_full<EPI>(g, s_bias, row, col + 16, c + 16, r1, k1);
    }
  }
  // what is left: single chunks, full or straddling N (all conditions are warp-uniform)
  for (; c < c_end && n0 + c < g.N; c += 16) {
    const int col = n0 + c;
    if (col + 16 <= g.N) {
      uint32_t r0[16];
      tc::tmem_ld16(t_row + c, r0);
      uint32_t k0 = rm.chunk((c - c_begin) >> 4);
      if (from_h && in_rows) {
        const __nv_bfloat16* h = g.H + static_cast<size_t>(row) * g.ldh + col;
        k0 = keep_bits_of(*reinterpret_cast<const uint4*>(h), *reinterpret_cast<const uint4*>(h + 8));
      }
      tc::tmem_ld_wait();
      if (in_rows) epilogue_full<EPI>(g, s_bias, row, col, c, r0, k0);
    } else {
      epilogue_tail<EPI>(g, s_bias, t_row + c, row, col, c);
    }
  }
}

// Column range of epilogue warp `ew` (0 .. kEpiWarps - 1): the tile's 16-column chunks are split
// between the two warps that share a TMEM lane quarter.
__device__ __forceinline__ void epi_cols(int bn, int ew, int* c_begin, int* c_end) {
  const int chunks = bn / 16;
  const int first = (chunks + 1) / 2;
  if (ew < 4) {
    *c_begin = 0;
    *c_end = first * 16;
  } else {
    *c_begin = first * 16;
    *c_end = bn;
  }
}

// Bias of the tile's columns into shared memory (zeros where there is none).
__device__ __forceinline__ void stage_bias(const GemmArgs& g, float* s_bias, int n0, int tid, int nthreads) {
  for (int j = tid; j < 256; j += nthreads) s_bias[j] = (g.bias && j < g.BN && n0 + j < g.N) ? g.bias[n0 + j] : 0.f;
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(kThreads)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t a_bytes = kBM * 128;
  const uint32_t b_bytes = static_cast<uint32_t>(g.BN) * 128;
  const uint32_t stage_bytes = a_bytes + b_bytes;

  __shared__ uint64_t full_bar[kMaxStages];
  __shared__ uint64_t empty_bar[kMaxStages];
  __shared__ uint64_t acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float s_bias[256];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * kBM;
  const int n0 = blockIdx.y * g.BN;
  const int total_kb = (g.K + kBK - 1) / kBK;
  const int kb_begin = blockIdx.z * g.kb_per_split;
  const int kb_end = min(total_kb, kb_begin + g.kb_per_split);
  const int num_kb = max(0, kb_end - kb_begin);
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(g.BN)) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < g.stages; ++s) {
      tc::mbar_init(&full_bar[s], 1);
      tc::mbar_init(&empty_bar[s], 1);
    }
    tc::mbar_init(&acc_bar, 1);
    abort_flag = 0;
    tc::fence_barrier_init();
    tc::prefetch_tmap(&tmA);
    tc::prefetch_tmap(&tmB);
  }
  if (warp == 1) tc::tmem_alloc(&tmem_slot, tmem_cols);
  if (EPI == EPI_BIAS_ACT) stage_bias(g, s_bias, n0, threadIdx.x, blockDim.x);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  pdl_enter();  // everything above touches nothing the kernel in front of this one writes
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer
    bool ok = true;
    for (int i = 0; i < num_kb && ok; ++i) {
      const int s = i % g.stages;
      const uint32_t round = static_cast<uint32_t>(i / g.stages);
      if (round > 0) ok = tc::mbar_wait(&empty_bar[s], (round - 1) & 1, kWaitLimit);
      if (!ok) break;
      uint8_t* a_dst = smem + static_cast<size_t>(s) * stage_bytes;
      uint8_t* b_dst = a_dst + a_bytes;
      const int k0 = (kb_begin + i) * kBK;
      tc::mbar_expect_tx(&full_bar[s], stage_bytes);
      if (A_MN) {
        for (int j = 0; j < kBM / 64; ++j) tc::tma_load_2d(a_dst + j * 8192, &tmA, &full_bar[s], m0 + 64 * j, k0);
      } else {
        tc::tma_load_2d(a_dst, &tmA, &full_bar[s], k0, m0);
      }
      if (B_MN) {
        for (int j = 0; j < g.BN / 64; ++j) tc::tma_load_2d(b_dst + j * 8192, &tmB, &full_bar[s], n0 + 64 * j, k0);
      } else {
        tc::tma_load_2d(b_dst, &tmB, &full_bar[s], k0, n0);
      }
    }
    if (!ok) {
      atomicCAS(g.status, 0, err::kTimeout);
      abort_flag = 1;
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer
    const uint32_t idesc = tc::instr_desc_bf16(kBM, g.BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
    bool ok = true;
    for (int i = 0; i < num_kb && ok; ++i) {
      const int s = i % g.stages;
      ok = tc::mbar_wait(&full_bar[s], static_cast<uint32_t>(i / g.stages) & 1, kWaitLimit);
      if (!ok) break;
      tc::fence_after_sync();
      const uint32_t a_addr = tc::smem_u32(smem + static_cast<size_t>(s) * stage_bytes);
      const uint32_t b_addr = a_addr + a_bytes;
#pragma unroll
      for (int k = 0; k < kBK / 16; ++k) {
        const uint64_t ad = A_MN ? tc::smem_desc(a_addr + k * 2048, 8192, 1024) : tc::smem_desc(a_addr + k * 32, 16, 1024);
        const uint64_t bd = B_MN ? tc::smem_desc(b_addr + k * 2048, 8192, 1024) : tc::smem_desc(b_addr + k * 32, 16, 1024);
        tc::mma_bf16(tmem_base, ad, bd, idesc, (i > 0 || k > 0) ? 1u : 0u);
      }
      tc::mma_commit(&empty_bar[s]);  // the stage is free again once these MMAs have read it
    }
    if (ok) {
      tc::mma_commit(&acc_bar);
    } else {
      atomicCAS(g.status, 0, err::kTimeout);
      abort_flag = 1;
      tc::mbar_arrive(&acc_bar);  // release the epilogue warps; they see abort_flag and skip
    }
  } else if (warp >= 2) {
    // ---------------- epilogue: thread = one accumulator row, warp = one column half
    const int quarter = warp & 3;  // a warp may only read TMEM lanes [32 * (warp % 4), +32)
    const int row = m0 + quarter * 32 + lane;
    int c_begin, c_end;
    epi_cols(g.BN, warp - 2, &c_begin, &c_end);
    RowMask rm{~0ull, ~0ull};
    if (EPI == EPI_RELU_MASK) rm = load_row_mask(g, row, (n0 + c_begin) >> 4, (c_end - c_begin + 15) >> 4);
    const bool ok = tc::mbar_wait(&acc_bar, 0, kWaitLimit);
    tc::fence_after_sync();
    if (!ok && lane == 0) atomicCAS(g.status, 0, err::kTimeout);
    if (ok && abort_flag == 0 && num_kb > 0)
      epilogue_rows<EPI>(g, s_bias, tmem_base + (static_cast<uint32_t>(quarter * 32) << 16), row, n0, c_begin, c_end, rm);
  }

  // ---------------- teardown: let the copies that were issued land, then free tensor memory
  if (warp == 0 && lane == 0) {
    const int first = max(0, num_kb - g.stages);
    for (int i = first; i < num_kb; ++i)
      tc::mbar_wait(&full_bar[i % g.stages], static_cast<uint32_t>(i / g.stages) & 1, kWaitLimit);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) tc::tmem_dealloc(tmem_base, tmem_cols);
}

// ------------------------------------------------------------------ weight-resident persistent variant
// Forward and input-gradient GEMMs of an MLP are tall and skinny: M = batch (tens of thousands),
// N and K a few hundred.  With one output tile per CTA every CTA re-reads its 128 x K slice of the
// weights from L2, and that traffic, not the tensor cores, sets the time.  Here a CTA (one per SM)
// loads its BN x K slice of the weight matrix ONCE, keeps it in shared memory, and then streams
// activation tiles for many 128-row tiles through a small ring, with two TMEM accumulators so the
// epilogue of tile j overlaps the MMAs of tile j + 1.
template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bres_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int total_kb = (g.K + kBK - 1) / kBK;
  const uint32_t a_bytes = kBM * 128;
  const uint32_t b_bytes = static_cast<uint32_t>(g.BN) * 128;  // one k-block of the resident weights
  uint8_t* b_res = smem;
  uint8_t* a_ring = smem + static_cast<size_t>(total_kb) * b_bytes;

  __shared__ uint64_t b_full, a_full[kMaxStages], a_empty[kMaxStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float s_bias[256];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n0 = blockIdx.y * g.BN;
  const int m_tiles = (g.M + kBM - 1) / kBM;
  const int my_tiles = (m_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  constexpr uint32_t kAccCols = 256;  // column stride between the two accumulators

  if (threadIdx.x == 0) {
    tc::mbar_init(&b_full, 1);
    for (int s = 0; s < g.stages; ++s) {
      tc::mbar_init(&a_full[s], 1);
      tc::mbar_init(&a_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&acc_full[b], 1);
      tc::mbar_init(&acc_empty[b], kEpiWarps);  // one arrival per epilogue warp
    }
    abort_flag = 0;
    tc::fence_barrier_init();
    tc::prefetch_tmap(&tmA);
    tc::prefetch_tmap(&tmB);
  }
  if (warp == 1) tc::tmem_alloc(&tmem_slot, 512);
  if (EPI == EPI_BIAS_ACT) stage_bias(g, s_bias, n0, threadIdx.x, blockDim.x);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  pdl_enter();  // everything above touches nothing the kernel in front of this one writes
  const uint32_t tmem_base = tmem_slot;
  const int total_it = my_tiles * total_kb;

  if (warp == 0 && lane == 0) {
    // ---------------- producer: the weights once, then the activation stream
    tc::mbar_expect_tx(&b_full, static_cast<uint32_t>(total_kb) * b_bytes);
    for (int kb = 0; kb < total_kb; ++kb)
      tc::tma_load_2d(b_res + static_cast<size_t>(kb) * b_bytes, &tmB, &b_full, kb * kBK, n0);
    bool ok = true;
    for (int it = 0; it < total_it && ok; ++it) {
      const int s = it % g.stages;
      const uint32_t round = static_cast<uint32_t>(it / g.stages);
      if (round > 0) ok = tc::mbar_wait(&a_empty[s], (round - 1) & 1, kWaitLimit);
      if (!ok) break;
      const int tile = blockIdx.x + (it / total_kb) * gridDim.x;
      const int kb = it % total_kb;
      tc::mbar_expect_tx(&a_full[s], a_bytes);
      tc::tma_load_2d(a_ring + static_cast<size_t>(s) * a_bytes, &tmA, &a_full[s], kb * kBK, tile * kBM);
    }
    if (!ok) {
      atomicCAS(g.status, 0, err::kTimeout);
      abort_flag = 1;
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer
    const uint32_t idesc = tc::instr_desc_bf16(kBM, g.BN, 0, 0);
    bool ok = tc::mbar_wait(&b_full, 0, kWaitLimit);
    tc::fence_after_sync();
    const uint32_t b_addr0 = tc::smem_u32(b_res);
    const uint32_t a_addr0 = tc::smem_u32(a_ring);
    int it = 0;
    for (int j = 0; j < my_tiles && ok; ++j) {
      const int buf = j & 1;
      const uint32_t use = static_cast<uint32_t>(j >> 1);
      if (use > 0) {
        ok = tc::mbar_wait(&acc_empty[buf], (use - 1) & 1, kWaitLimit);  // epilogue has drained this buffer
        if (!ok) break;
        tc::fence_after_sync();
      }
      const uint32_t d_tmem = tmem_base + buf * kAccCols;
      for (int kb = 0; kb < total_kb && ok; ++kb, ++it) {
        const int s = it % g.stages;
        ok = tc::mbar_wait(&a_full[s], static_cast<uint32_t>(it / g.stages) & 1, kWaitLimit);
        if (!ok) break;
        tc::fence_after_sync();
        const uint32_t a_addr = a_addr0 + s * a_bytes;
        const uint32_t b_addr = b_addr0 + kb * b_bytes;
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k)
          tc::mma_bf16(d_tmem, tc::smem_desc(a_addr + k * 32, 16, 1024), tc::smem_desc(b_addr + k * 32, 16, 1024), idesc,
                       (kb > 0 || k > 0) ? 1u : 0u);
        tc::mma_commit(&a_empty[s]);
      }
      if (ok) tc::mma_commit(&acc_full[buf]);
    }
    if (!ok) {
      atomicCAS(g.status, 0, err::kTimeout);
      abort_flag = 1;
      tc::mbar_arrive(&acc_full[0]);
      tc::mbar_arrive(&acc_full[1]);
    }
  } else if (warp >= 2) {
    // ---------------- epilogue
    const int quarter = warp & 3;
    int c_begin, c_end;
    epi_cols(g.BN, warp - 2, &c_begin, &c_end);
    bool ok = true;
    for (int j = 0; j < my_tiles && ok; ++j) {
      const int buf = j & 1;
      const int tile = blockIdx.x + j * gridDim.x;
      const int row = tile * kBM + quarter * 32 + lane;
      RowMask rm{~0ull, ~0ull};
      if (EPI == EPI_RELU_MASK) rm = load_row_mask(g, row, (n0 + c_begin) >> 4, (c_end - c_begin + 15) >> 4);
      ok = tc::mbar_wait(&acc_full[buf], static_cast<uint32_t>(j >> 1) & 1, kWaitLimit);
      tc::fence_after_sync();
      if (!ok || abort_flag != 0) {
        if (!ok && lane == 0) atomicCAS(g.status, 0, err::kTimeout);
        ok = false;
        break;
      }
      epilogue_rows<EPI>(g, s_bias, tmem_base + buf * kAccCols + (static_cast<uint32_t>(quarter * 32) << 16), row, n0,
                         c_begin, c_end, rm);
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
    }
  }

  // ---------------- teardown
  if (warp == 0 && lane == 0) {
    tc::mbar_wait(&b_full, 0, kWaitLimit);
    const int first = max(0, total_it - g.stages);
    for (int it = first; it < total_it; ++it)
      tc::mbar_wait(&a_full[it % g.stages], static_cast<uint32_t>(it / g.stages) & 1, kWaitLimit);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) tc::tmem_dealloc(tmem_base, 512);
}

// ------------------------------------------------------------------ weight-resident CTA-pair variant
// The single-CTA resident kernel above is bound by what one SM can take in: every MMA reads
// (128 + BN) x 32 bytes of operands from shared memory, which keeps the shared-memory port busy
// for most of the MMA's duration and stalls the TMA stream that shares it, and a column tile
// narrow enough to leave room for a deep activation ring makes every activation tile cross the
// L2-to-SM fabric once per column tile.  A pair of CTAs on one TPC running tcgen05.mma with
// cta_group::2 fixes both: each CTA keeps only half of the column tile's weights (so the same
// shared memory holds a wider tile AND a deeper ring) and reads only half of the B bytes per MMA.
//
//   cluster = 2 CTAs; pair tile = 256 rows x BN columns; CTA r loads rows [r * 128, +128) of A and
//   weight rows [n0 + r * BN / 2, +BN / 2); the even CTA's warp 1 issues every MMA; the byte
//   counts of both CTAs' loads complete on the even CTA's barriers; tcgen05.commit with a CTA
//   mask frees ring stages and publishes accumulators in both CTAs; epilogue warps of both CTAs
//   release an accumulator buffer by arriving on the even CTA's barrier.
template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int total_kb = (g.K + kBK - 1) / kBK;
  const int half_bn = g.BN / 2;
  const uint32_t a_bytes = kBM * 128;
  const uint32_t b_bytes = static_cast<uint32_t>(half_bn) * 128;  // one k-block of this CTA's half of the weights
  uint8_t* b_res = smem;
  uint8_t* a_ring = smem + static_cast<size_t>(total_kb) * b_bytes;

  __shared__ uint64_t b_full, a_full[kMaxStages], a_empty[kMaxStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float s_bias[256];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = tc::cluster_ctarank();  // 0 = the CTA that issues the MMAs
  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;
  const int n0 = blockIdx.y * g.BN;
  const int m_tiles = (g.M + 2 * kBM - 1) / (2 * kBM);  // pair tiles of 256 rows
  const int my_tiles = (m_tiles - pair + pairs - 1) / pairs;
  constexpr uint32_t kAccCols = 256;

  if (threadIdx.x == 0) {
    tc::mbar_init(&b_full, 1);
    for (int s = 0; s < g.stages; ++s) {
      tc::mbar_init(&a_full[s], 1);
      tc::mbar_init(&a_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&acc_full[b], 1);
      tc::mbar_init(&acc_empty[b], 2 * kEpiWarps);  // every epilogue warp of both CTAs
    }
    abort_flag = 0;
    tc::fence_barrier_init();
    tc::prefetch_tmap(&tmA);
    tc::prefetch_tmap(&tmB);
  }
  if (warp == 1) tc::tmem_alloc_pair(&tmem_slot, 512);
  if (EPI == EPI_BIAS_ACT) stage_bias(g, s_bias, n0, threadIdx.x, blockDim.x);
  tc::fence_before_sync();
  __syncthreads();
  tc::cluster_sync_all();  // the other CTA's barriers exist before anything arrives on them
  tc::fence_after_sync();
  pdl_enter();  // everything above touches nothing the kernel in front of this one writes
  const uint32_t tmem_base = tmem_slot;
  const int total_it = my_tiles * total_kb;

  if (warp == 0 && lane == 0) {
    // ---------------- producer (both CTAs): own half of the weights once, then own rows of the stream
    const uint32_t lead_b_full = tc::map_to_cta(tc::smem_u32(&b_full), 0);
    if (rank == 0) tc::mbar_expect_tx(&b_full, 2u * static_cast<uint32_t>(total_kb) * b_bytes);
    for (int kb = 0; kb < total_kb; ++kb)
      tc::tma_load_2d_pair(b_res + static_cast<size_t>(kb) * b_bytes, &tmB, lead_b_full, kb * kBK,
                           n0 + static_cast<int>(rank) * half_bn);
    bool ok = true;
    for (int it = 0; it < total_it && ok; ++it) {
      const int s = it % g.stages;
      const uint32_t round = static_cast<uint32_t>(it / g.stages);
      if (round > 0) ok = tc::mbar_wait(&a_empty[s], (round - 1) & 1, kWaitLimit);
      if (!ok) break;
      const int tile = pair + (it / total_kb) * pairs;
      const int kb = it % total_kb;
      if (rank == 0) tc::mbar_expect_tx(&a_full[s], 2u * a_bytes);
      tc::tma_load_2d_pair(a_ring + static_cast<size_t>(s) * a_bytes, &tmA, tc::map_to_cta(tc::smem_u32(&a_full[s]), 0),
                           kb * kBK, tile * 2 * kBM + static_cast<int>(rank) * kBM);
    }
    if (!ok) {
      atomicCAS(g.status, 0, err::kTimeout);
      abort_flag = 1;
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---------------- MMA issuer (even CTA only)
    const uint32_t idesc = tc::instr_desc_bf16(2 * kBM, g.BN, 0, 0);
    bool ok = tc::mbar_wait(&b_full, 0, kWaitLimit);
    tc::fence_after_sync();
    const uint32_t b_addr0 = tc::smem_u32(b_res);
    const uint32_t a_addr0 = tc::smem_u32(a_ring);
    int it = 0;
    for (int j = 0; j < my_tiles && ok; ++j) {
      const int buf = j & 1;
      const uint32_t use = static_cast<uint32_t>(j >> 1);
      if (use > 0) {
        ok = tc::mbar_wait(&acc_empty[buf], (use - 1) & 1, kWaitLimit);
        if (!ok) break;
        tc::fence_after_sync();
      }
      const uint32_t d_tmem = tmem_base + buf * kAccCols;
      for (int kb = 0; kb < total_kb && ok; ++kb, ++it) {
        const int s = it % g.stages;
        ok = tc::mbar_wait(&a_full[s], static_cast<uint32_t>(it / g.stages) & 1, kWaitLimit);
        if (!ok) break;
        tc::fence_after_sync();
        const uint32_t a_addr = a_addr0 + s * a_bytes;
        const uint32_t b_addr = b_addr0 + kb * b_bytes;
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k)
          tc::mma_bf16_pair(d_tmem, tc::smem_desc(a_addr + k * 32, 16, 1024), tc::smem_desc(b_addr + k * 32, 16, 1024),
                            idesc, (kb > 0 || k > 0) ? 1u : 0u);
        tc::mma_commit_pair(&a_empty[s], 3);  // the stage is free in both CTAs
      }
      if (ok) tc::mma_commit_pair(&acc_full[buf], 3);
    }
    if (!ok) {
      atomicCAS(g.status, 0, err::kTimeout);
      abort_flag = 1;
    }
  } else if (warp >= 2) {
    // ---------------- epilogue (both CTAs, each on its own 128 rows)
    const int quarter = warp & 3;
    const uint32_t lead_acc_empty[2] = {tc::map_to_cta(tc::smem_u32(&acc_empty[0]), 0),
                                        tc::map_to_cta(tc::smem_u32(&acc_empty[1]), 0)};
    int c_begin, c_end;
    epi_cols(g.BN, warp - 2, &c_begin, &c_end);
    bool ok = true;
    for (int j = 0; j < my_tiles && ok; ++j) {
      const int buf = j & 1;
      const int tile = pair + j * pairs;
      const int row = tile * 2 * kBM + static_cast<int>(rank) * kBM + quarter * 32 + lane;
      RowMask rm{~0ull, ~0ull};
      if (EPI == EPI_RELU_MASK) rm = load_row_mask(g, row, (n0 + c_begin) >> 4, (c_end - c_begin + 15) >> 4);
      ok = tc::mbar_wait(&acc_full[buf], static_cast<uint32_t>(j >> 1) & 1, kWaitLimit);
      tc::fence_after_sync();
      if (!ok) {
        if (lane == 0) atomicCAS(g.status, 0, err::kTimeout);
        break;
      }
      epilogue_rows<EPI>(g, s_bias, tmem_base + buf * kAccCols + (static_cast<uint32_t>(quarter * 32) << 16), row, n0,
                         c_begin, c_end, rm);
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive_cluster(lead_acc_empty[buf]);
    }
  }

  // ---------------- teardown: the even CTA's barriers count both CTAs' copies
  if (warp == 0 && lane == 0 && rank == 0) {
    tc::mbar_wait(&b_full, 0, kWaitLimit);
    const int first = max(0, total_it - g.stages);
    for (int it = first; it < total_it; ++it)
      tc::mbar_wait(&a_full[it % g.stages], static_cast<uint32_t>(it / g.stages) & 1, kWaitLimit);
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::cluster_sync_all();  // neither CTA leaves while the other may still touch its memory or barriers
  if (warp == 1) tc::tmem_dealloc_pair(tmem_base, 512);
}

// ------------------------------------------------------------------ column sums
__global__ void __launch_bounds__(256)
colsum_bf16_kernel(const __nv_bfloat16* __restrict__ x, int ld, int M, int N, int rows_per_block, float* out) {
  pdl_enter();
  // block = 256 threads: 32 column pairs x 8 row lanes over a 64-column strip
  const int cpair = threadIdx.x & 31;
  const int rlane = threadIdx.x >> 5;
  const int col = blockIdx.x * 64 + cpair * 2;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(M, r0 + rows_per_block);
  float s0 = 0.f, s1 = 0.f;
  if (col < N) {
    for (int r = r0 + rlane; r < r1; r += 8) {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(x + static_cast<size_t>(r) * ld + col);
      s0 += __bfloat162float(v.x);
      s1 += __bfloat162float(v.y);
    }
  }
  __shared__ float sh[8][64];
  sh[rlane][cpair * 2] = s0;
  sh[rlane][cpair * 2 + 1] = s1;
  __syncthreads();
  if (threadIdx.x < 64) {
    float t = 0.f;
    for (int k = 0; k < 8; ++k) t += sh[k][threadIdx.x];
    const int c = blockIdx.x * 64 + threadIdx.x;
    if (c < N) atomicAdd(out + c, t);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D bf16 row-major tensor [rows, cols] with pitch ld (elements); box = box_cols x box_rows,
// 128-byte swizzle, out-of-range elements read as zero.
bool make_tmap(CUtensorMap* m, const __nv_bfloat16* base, int rows, int cols, int ld, int box_cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld % 8) != 0 || box_cols != 64 || box_rows > 256) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int pick_bn(int n, int granule) {
  // fewest tiles first, then the narrowest tile that still covers n with that many tiles
  const int tiles = (n + 255) / 256;
  int bn = (n + tiles - 1) / tiles;
  bn = (bn + granule - 1) / granule * granule;
  return bn < granule ? granule : bn;
}

// With at most one CTA per SM there is no second CTA to hide a short pipeline behind: go to 4
// stages when the whole grid fits in one wave, else 2 stages and two CTAs per SM.
int one_wave_stages(int m, int n, int bn) {
  const int tiles = ((m + kBM - 1) / kBM) * ((n + bn - 1) / bn);
  return tiles <= 148 ? 4 : 2;
}

template <bool A_MN, bool B_MN, int EPI>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs g, int splits, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(g.stages) * (kBM + g.BN) * 128 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemm_kernel<A_MN, B_MN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    attr_set = true;
  }
  dim3 grid((g.M + kBM - 1) / kBM, (g.N + g.BN - 1) / g.BN, splits);
  launch_pdl(gemm_kernel<A_MN, B_MN, EPI>, grid, dim3(kThreads), smem, stream, ta, tb, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int g_variant = 0;           // 0 = choose; 1 = CTA pair; 2 = single-CTA resident; 3 = one tile per CTA
int g_resident_n_tiles = 0;  // 0 = choose; otherwise the number of column tiles of the resident variant

// Plan of the resident-weight variant for an M x N output contracting over K: tile width and depth
// of the activation ring.  The ring's depth decides how many bytes a CTA keeps in flight from L2,
// and that, not the tensor cores, bounds these tall-and-skinny products; so the plan takes the
// fewest column tiles whose weight slice leaves room for at least four 16 KB activation stages
// (more column tiles re-read the activations from L2 once more each, which costs less than a
// starved ring).  Returns false when the variant does not apply.
bool plan_resident(int M, int N, int K, int* bn_out, int* stages_out) {
  const int total_kb = (K + kBK - 1) / kBK;
  const int m_tiles = (M + kBM - 1) / kBM;
  const size_t budget = 225 * 1024 - 1024;
  int best_bn = 0, best_stages = 0;
  for (int n_tiles = (N + 255) / 256; n_tiles <= 8; ++n_tiles) {
    if (g_resident_n_tiles > 0 && n_tiles != g_resident_n_tiles) continue;
    int bn = (N + n_tiles - 1) / n_tiles;
    bn = (bn + 15) / 16 * 16;
    if (bn < 16) bn = 16;
    const size_t weights = static_cast<size_t>(total_kb) * bn * 128;
    if (weights + 2 * kBM * 128 > budget) continue;
    int stages = static_cast<int>((budget - weights) / (kBM * 128));
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages > best_stages) best_bn = bn, best_stages = stages;
    if (stages >= 4) break;
  }
  if (best_bn == 0) return false;
  const int n_tiles = (N + best_bn - 1) / best_bn;
  if (n_tiles > 148 || m_tiles * n_tiles < 2 * 148) return false;
  *bn_out = best_bn;
  *stages_out = best_stages;
  return true;
}

// Plan of the CTA-pair variant: the widest column tile (fewest activation re-reads) whose half
// slice of the weights leaves at least four ring stages.
bool plan_pair(int M, int N, int K, int* bn_out, int* stages_out) {
  const int total_kb = (K + kBK - 1) / kBK;
  const int m_tiles = (M + 2 * kBM - 1) / (2 * kBM);
  const size_t budget = 225 * 1024 - 1024;
  for (int n_tiles = (N + 255) / 256; n_tiles <= 4; ++n_tiles) {
    if (g_resident_n_tiles > 0 && n_tiles != g_resident_n_tiles) continue;
    int bn = (N + n_tiles - 1) / n_tiles;
    bn = (bn + 15) / 16 * 16;  // the MMA's N is a multiple of 16; each half is then whole 8-row swizzle groups
    const size_t weights = static_cast<size_t>(total_kb) * (bn / 2) * 128;
    if (weights + 4 * kBM * 128 > budget) continue;
    int stages = static_cast<int>((budget - weights) / (kBM * 128));
    if (stages > kMaxStages) stages = kMaxStages;
    if (m_tiles * n_tiles < 2 * 74) return false;  // too few tiles to amortise loading the weights
    *bn_out = bn;
    *stages_out = stages;
    return true;
  }
  return false;
}

template <int EPI>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs g, cudaStream_t stream) {
  const int total_kb = (g.K + kBK - 1) / kBK;
  const int n_tiles = (g.N + g.BN - 1) / g.BN;
  const int m_tiles = (g.M + 2 * kBM - 1) / (2 * kBM);
  const size_t smem = static_cast<size_t>(total_kb) * (g.BN / 2) * 128 + static_cast<size_t>(g.stages) * kBM * 128 + 1024;
  static size_t attr_smem = 0;
  if (smem > attr_smem) {
    if (cudaFuncSetAttribute(gemm_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess) {
      cudaGetLastError();
      return -2;
    }
    attr_smem = smem;
  }
  int pairs = 74 / n_tiles;
  if (pairs > m_tiles) pairs = m_tiles;
  launch_pdl(gemm_pair_kernel<EPI>, dim3(2 * pairs, n_tiles), dim3(kThreads), smem, stream, ta, tb, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

template <int EPI>
int launch_resident(const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs g, cudaStream_t stream) {
  const int total_kb = (g.K + kBK - 1) / kBK;
  const int n_tiles = (g.N + g.BN - 1) / g.BN;
  const int m_tiles = (g.M + kBM - 1) / kBM;
  const size_t smem = static_cast<size_t>(total_kb) * g.BN * 128 + static_cast<size_t>(g.stages) * kBM * 128 + 1024;
  static size_t attr_smem = 0;  // static + dynamic shared memory share the 227 KB limit: ask for what is needed
  if (smem > attr_smem) {
    if (cudaFuncSetAttribute(gemm_bres_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess) {
      cudaGetLastError();
      return -2;
    }
    attr_smem = smem;
  }
  int per_n = 148 / n_tiles;
  if (per_n > m_tiles) per_n = m_tiles;
  launch_pdl(gemm_bres_kernel<EPI>, dim3(per_n, n_tiles), dim3(kThreads), smem, stream, ta, tb, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace

// 256-bit stores need 32-byte aligned rows; tile columns are multiples of 16 elements already.
static int can_store_v8(const void* out, int ld) {
  return (reinterpret_cast<uintptr_t>(out) % 32 == 0 && ld % 16 == 0) ? 1 : 0;
}

int linear_forward(const __nv_bfloat16* X, int ldx, const __nv_bfloat16* W, int ldw, const float* bias,
                   __nv_bfloat16* Y, int ldy, int M, int N, int K, bool relu, uint16_t* mask_out, int ldm, int* status,
                   cudaStream_t stream) {
  GemmArgs g{};
  g.M = M, g.N = N, g.K = K;
  g.BN = pick_bn(N, 16);
  g.stages = 2;
  g.kb_per_split = (K + kBK - 1) / kBK;
  g.relu = relu ? 1 : 0;
  g.bias = bias;
  g.out = Y, g.ldo = ldy;
  g.mask_out = mask_out, g.ldm = ldm, g.mask_chunks = (N + 15) / 16;
  g.out_v8 = can_store_v8(Y, ldy);
  if (mask_out != nullptr && ldm < M) return -1;
  g.status = status;
  CUtensorMap ta, tb;
  const bool pair = (g_variant == 0 || g_variant == 1) && plan_pair(M, N, K, &g.BN, &g.stages);
  const bool resident = !pair && (g_variant == 0 || g_variant == 2) && plan_resident(M, N, K, &g.BN, &g.stages);
  if ((ldy % 8) != 0 || !make_tmap(&ta, X, M, K, ldx, 64, kBM) ||
      !make_tmap(&tb, W, N, K, ldw, 64, pair ? g.BN / 2 : g.BN))
    return -1;
  if (pair) return launch_pair<EPI_BIAS_ACT>(ta, tb, g, stream);
  if (resident) return launch_resident<EPI_BIAS_ACT>(ta, tb, g, stream);
  g.stages = one_wave_stages(M, N, g.BN);
  return launch<false, false, EPI_BIAS_ACT>(ta, tb, g, 1, stream);
}

int linear_dgrad(const __nv_bfloat16* dY, int lddy, const __nv_bfloat16* Wt, int ldwt, const __nv_bfloat16* H,
                 int ldh, const uint16_t* mask, int ldm, __nv_bfloat16* dX, int lddx, int M, int N, int K, int* status,
                 cudaStream_t stream) {
  // out dX is [M, K]; the contraction runs over the layer's N outputs
  GemmArgs g{};
  g.M = M, g.N = K, g.K = N;
  g.BN = pick_bn(K, 16);
  g.stages = 2;
  g.kb_per_split = (N + kBK - 1) / kBK;
  g.H = H, g.ldh = ldh;
  g.mask = mask, g.ldm = ldm, g.mask_chunks = (K + 15) / 16;
  g.out_v8 = can_store_v8(dX, lddx);
  if (mask != nullptr && ldm < M) return -1;
  g.out = dX, g.ldo = lddx;
  g.status = status;
  CUtensorMap ta, tb;
  const bool pair = (g_variant == 0 || g_variant == 1) && plan_pair(M, K, N, &g.BN, &g.stages);
  const bool resident = !pair && (g_variant == 0 || g_variant == 2) && plan_resident(M, K, N, &g.BN, &g.stages);
  if ((lddx % 8) != 0 || (H && (ldh % 8) != 0) || !make_tmap(&ta, dY, M, N, lddy, 64, kBM) ||
      !make_tmap(&tb, Wt, K, N, ldwt, 64, pair ? g.BN / 2 : g.BN))
    return -1;
  if (pair) return launch_pair<EPI_RELU_MASK>(ta, tb, g, stream);
  if (resident) return launch_resident<EPI_RELU_MASK>(ta, tb, g, stream);
  g.stages = one_wave_stages(M, K, g.BN);
  return launch<false, false, EPI_RELU_MASK>(ta, tb, g, 1, stream);
}

int linear_wgrad(const __nv_bfloat16* dY, int lddy, const __nv_bfloat16* X, int ldx, float* dW, int lddw, int M,
                 int N, int K, int* status, cudaStream_t stream) {
  // out dW is [N, K]; the contraction runs over the M batch rows, split across blockIdx.z
  GemmArgs g{};
  g.M = N, g.N = K, g.K = M;
  g.BN = pick_bn(K, 64);
  g.stages = 4;
  const int total_kb = (M + kBK - 1) / kBK;
  const int tiles = ((N + kBM - 1) / kBM) * ((K + g.BN - 1) / g.BN);
  int splits = 148 / (tiles > 0 ? tiles : 1);
  if (splits < 1) splits = 1;
  if (splits > total_kb) splits = total_kb;
  g.kb_per_split = (total_kb + splits - 1) / splits;
  splits = (total_kb + g.kb_per_split - 1) / g.kb_per_split;  // no empty split
  g.out32 = dW, g.ldo32 = lddw;
  g.status = status;
  CUtensorMap ta, tb;
  if ((lddw % 4) != 0 || (reinterpret_cast<uintptr_t>(dW) & 15) != 0 || !make_tmap(&ta, dY, M, N, lddy, 64, 64) ||
      !make_tmap(&tb, X, M, K, ldx, 64, 64))
    return -1;
  return launch<true, true, EPI_RED_F32>(ta, tb, g, splits, stream);
}

void gemm_set_tuning(int variant, int n_tiles) {
  g_variant = variant;
  g_resident_n_tiles = n_tiles;
}

void colsum_bf16(const __nv_bfloat16* dY, int lddy, int M, int N, float* db, cudaStream_t stream) {
  const int strips = (N + 63) / 64;
  int row_blocks = (148 * 4 + strips - 1) / strips;
  int rows_per_block = (M + row_blocks - 1) / row_blocks;
  if (rows_per_block < 64) rows_per_block = 64;
  row_blocks = (M + rows_per_block - 1) / rows_per_block;
  launch_pdl(colsum_bf16_kernel, dim3(strips, row_blocks), dim3(256), 0, stream, dY, lddy, M, N, rows_per_block, db);
}

}  // namespace cu
}  // namespace kb
