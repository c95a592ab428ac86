// DeepFM front end fused around the sparse exchange.
//
// Two table layouts are accepted: a dim-D embedding table plus a separate dim-1 first-order
// table, or ONE table whose rows are RD >= D + 1 floats wide with the first-order weight in
// column D (rows1 / ugrad1 null): the second costs one exchange per step instead of two.
//
// Forward: reads the UNIQUE rows that the pull left in the receive buffers (second-order
// table [U2, D] and first-order table [U1, 1]) through the occurrence -> unique maps and, in
// one pass per sample, writes the bf16 MLP input [emb | dense | 0-pad] and the fp32 FM logit
//   sum_f w_f + 0.5 * sum_d ((sum_f e_fd)^2 - sum_f e_fd^2).
// Backward: from d(MLP input) and d(logit) forms each occurrence's embedding gradient
//   dlogit * (S_d - e_fd) + dX[f, d]   and   dlogit (first order)
// and red-adds it straight into the per-unique gradient buffers that push_dispatch sends, so
// the expanded [B, F, D] tensors of the unfused path never exist.
// Reference model math: examples/DeepFM/model/DeepFM.py:87-125 (torch CPU ops).
#include <cuda_bf16.h>

#include "common.cuh"
#include "kernels.h"

namespace kb {
namespace cu {

namespace {

constexpr int kThreads = 256;

// Row index of unique entry `u`: the entry itself when the rows were gathered into a receive
// buffer, or the table slot the owner resolved for it when the kernel reads the table in place
// (single-GPU jobs: no copy of the rows is made).  A failed lookup (slot < 0) reads row 0; the
// status word already carries the error.
__device__ __forceinline__ size_t row_of(const int* __restrict__ slots, int u) {
  if (slots == nullptr) return static_cast<size_t>(u);
  const int s = __ldg(slots + u);
  return static_cast<size_t>(s < 0 ? 0 : s);
}

// Lanes per sample = (D / 4) x G: lane (g, c) owns dims [4c, 4c + 4) of the fields g, g + G, ...
// Splitting the fields over G lane groups (a power of two) multiplies the number of independent
// row loads in flight; the per-sample sums are combined with shuffles and the forward pass leaves
// S[b, :] = sum_f e_f for the backward pass, whose lanes then need nothing from each other.
__global__ void __launch_bounds__(kThreads)
deepfm_pack_forward_kernel(const float* __restrict__ rows2, const int* __restrict__ inv2,
                           const int* __restrict__ slots2, const float* __restrict__ rows1,
                           const int* __restrict__ inv1, const int* __restrict__ slots1,
                           const float* __restrict__ dense, int B, int F, int D, int RD, int ND, int lpr, int G,
                           __nv_bfloat16* __restrict__ x, int ldx, float* __restrict__ fm_logit,
                           float* __restrict__ ssum) {
  pdl_enter();
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int stride = (gridDim.x * blockDim.x) / lpr;
  const unsigned group_mask = (lpr == 32 ? 0xffffffffu : ((1u << lpr) - 1u)) << ((threadIdx.x & 31) / lpr * lpr);
  const int chunks = D / 4;
  const int c = lane % chunks;   // chunks * G == lpr
  const int fg = lane / chunks;
  const int rounds = (B + stride - 1) / stride;
  for (int it = 0; it < rounds; ++it) {
    const int b = gtid / lpr + it * stride;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f), q = s;
    float part = 0.f;
    if (b < B) {
      const int* i2 = inv2 + static_cast<size_t>(b) * F;
      __nv_bfloat16* xr = x + static_cast<size_t>(b) * ldx;
#pragma unroll 4
      for (int f = fg; f < F; f += G) {
        const float4 e = __ldcg(reinterpret_cast<const float4*>(rows2 + row_of(slots2, i2[f]) * RD) + c);
        s.x += e.x, s.y += e.y, s.z += e.z, s.w += e.w;
        q.x += e.x * e.x, q.y += e.y * e.y, q.z += e.z * e.z, q.w += e.w * e.w;
        __nv_bfloat162 lo = __floats2bfloat162_rn(e.x, e.y), hi = __floats2bfloat162_rn(e.z, e.w);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(xr + f * D + c * 4) = packed;
      }
      // first-order weights, dense features and the zero pad, spread over the sample's lanes
      if (rows1 != nullptr) {
        const int* i1 = inv1 + static_cast<size_t>(b) * F;
        for (int f = lane; f < F; f += lpr) part += __ldcg(rows1 + row_of(slots1, i1[f]));
      } else {
        // folded layout: column D of the same row is the field's first-order weight
        for (int f = lane; f < F; f += lpr) part += __ldcg(rows2 + row_of(slots2, i2[f]) * RD + D);
      }
      const int base = F * D;
      for (int j = lane; base + j < ldx; j += lpr)
        xr[base + j] = __float2bfloat16(j < ND ? dense[static_cast<size_t>(b) * ND + j] : 0.f);
    }
    // sums over the field groups of the same chunk (lanes c, c + chunks, c + 2 chunks, ...)
    for (int o = chunks; o < lpr; o <<= 1) {
      s.x += __shfl_xor_sync(group_mask, s.x, o), s.y += __shfl_xor_sync(group_mask, s.y, o);
      s.z += __shfl_xor_sync(group_mask, s.z, o), s.w += __shfl_xor_sync(group_mask, s.w, o);
      q.x += __shfl_xor_sync(group_mask, q.x, o), q.y += __shfl_xor_sync(group_mask, q.y, o);
      q.z += __shfl_xor_sync(group_mask, q.z, o), q.w += __shfl_xor_sync(group_mask, q.w, o);
    }
    if (b < B && fg == 0) {
      part += 0.5f * (s.x * s.x - q.x + s.y * s.y - q.y + s.z * s.z - q.z + s.w * s.w - q.w);
      if (ssum != nullptr) *reinterpret_cast<float4*>(ssum + static_cast<size_t>(b) * D + c * 4) = s;
    }
    for (int o = lpr >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(group_mask, part, o);
    if (b < B && lane == 0) fm_logit[b] = part;
  }
}

__global__ void __launch_bounds__(kThreads)
deepfm_pack_backward_kernel(const float* __restrict__ rows2, const int* __restrict__ inv2,
                            const int* __restrict__ slots2, const int* __restrict__ inv1,
                            const __nv_bfloat16* __restrict__ dx, int lddx, const float* __restrict__ dlogit,
                            const float* __restrict__ ssum, int B, int F, int D, int RD, int lpr, int G,
                            float* ugrad2, float* ugrad1) {
  pdl_enter();
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int stride = (gridDim.x * blockDim.x) / lpr;
  const int chunks = D / 4;
  const int c = lane % chunks;
  const int fg = lane / chunks;
  for (int b = gtid / lpr; b < B; b += stride) {
    const int* i2 = inv2 + static_cast<size_t>(b) * F;
    const float g = dlogit[b];
    const __nv_bfloat16* dxr = dx ? dx + static_cast<size_t>(b) * lddx : nullptr;
    const float4 s = *reinterpret_cast<const float4*>(ssum + static_cast<size_t>(b) * D + c * 4);
#pragma unroll 4
    for (int f = fg; f < F; f += G) {
      const int u = i2[f];
      const float4 e = __ldcg(reinterpret_cast<const float4*>(rows2 + row_of(slots2, u) * RD) + c);
      float4 d = make_float4(g * (s.x - e.x), g * (s.y - e.y), g * (s.z - e.z), g * (s.w - e.w));
      if (dxr) {
        const uint2 p = *reinterpret_cast<const uint2*>(dxr + f * D + c * 4);
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&p.x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&p.y);
        d.x += __bfloat162float(lo.x), d.y += __bfloat162float(lo.y);
        d.z += __bfloat162float(hi.x), d.w += __bfloat162float(hi.y);
      }
      red_add_v4(ugrad2 + static_cast<size_t>(u) * RD + c * 4, d);
    }
    if (ugrad1 != nullptr) {
      const int* i1 = inv1 + static_cast<size_t>(b) * F;
      for (int f = lane; f < F; f += lpr) atomicAdd(ugrad1 + i1[f], g);
    } else {
      for (int f = lane; f < F; f += lpr) atomicAdd(ugrad2 + static_cast<size_t>(i2[f]) * RD + D, g);
    }
  }
}

Sym to_sym(const SymHost& h) {
  Sym s;
  for (int i = 0; i < kMaxWorld; ++i) s.base[i] = static_cast<char*>(h.base[i]);
  s.rank = h.rank;
  s.world = h.world;
  return s;
}

// Field groups per sample: as many as keep (D / 4) x G lanes within a quarter warp.
int field_groups(int chunks) {
  int g = 1;
  while (chunks * g * 2 <= 16) g <<= 1;
  return g;
}

int grid_for(long long rows, int lpr) {
  long long g = (rows * lpr + kThreads - 1) / kThreads;
  if (g < 1) g = 1;
  if (g > 148 * 16) g = 148 * 16;
  return static_cast<int>(g);
}

}  // namespace

void deepfm_pack_forward(const float* rows2, const int* inv2, const int* slots2, const float* rows1, const int* inv1,
                         const int* slots1, const float* dense, int B, int F, int D, int RD, int ND, __nv_bfloat16* x,
                         int ldx, float* fm_logit, float* ssum, cudaStream_t stream) {
  if (B <= 0) return;
  const int chunks = D / 4;
  const int G = field_groups(chunks);
  const int lpr = chunks * G;
  launch_pdl(deepfm_pack_forward_kernel, dim3(grid_for(B, lpr)), dim3(kThreads), 0, stream, rows2, inv2, slots2, rows1, inv1, slots1, dense,
                                                                        B, F, D, RD, ND, lpr, G, x, ldx, fm_logit, ssum);
}

void deepfm_pack_backward(const float* rows2, const int* inv2, const int* slots2, const int* inv1,
                          const __nv_bfloat16* dx, int lddx,
                          const float* dlogit, const float* ssum, int B, int F, int D, int RD, float* ugrad2,
                          float* ugrad1, cudaStream_t stream) {
  if (B <= 0) return;
  const int chunks = D / 4;
  const int G = field_groups(chunks);
  const int lpr = chunks * G;
  launch_pdl(deepfm_pack_backward_kernel, dim3(grid_for(B, lpr)), dim3(kThreads), 0, stream, rows2, inv2, slots2, inv1, dx, lddx, dlogit,
                                                                         ssum, B, F, D, RD, lpr, G, ugrad2, ugrad1);
}

}  // namespace cu
}  // namespace kb
