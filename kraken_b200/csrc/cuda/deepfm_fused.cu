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

// One-block kernel that only waits for the owners' answers of the current pull.
__global__ void pull_wait_kernel(Sym sym, ChanLayout lay, Ctrl* ctrl, uint32_t spin_limit) {
  if (sym.world <= 1) return;
  if (threadIdx.x < sym.world &&
      !wait_flag(sym.at<uint32_t>(sym.rank, lay.flag_rsp) + threadIdx.x, ctrl->pull_epoch, spin_limit))
    set_status(&ctrl->status, err::kTimeout);
}

// Row index of unique entry `u`: the entry itself when the rows were gathered into a receive
// buffer, or the table slot the owner resolved for it when the kernel reads the table in place
// (single-GPU jobs: no copy of the rows is made).  A failed lookup (slot < 0) reads row 0; the
// status word already carries the error.
__device__ __forceinline__ size_t row_of(const int* __restrict__ slots, int u) {
  if (slots == nullptr) return static_cast<size_t>(u);
  const int s = __ldg(slots + u);
  return static_cast<size_t>(s < 0 ? 0 : s);
}

// lanes per sample = D / 4; lane l owns dims [4l, 4l + 4) of every field.
__global__ void __launch_bounds__(kThreads)
deepfm_pack_forward_kernel(const float* __restrict__ rows2, const int* __restrict__ inv2,
                           const int* __restrict__ slots2, const float* __restrict__ rows1,
                           const int* __restrict__ inv1, const int* __restrict__ slots1,
                           const float* __restrict__ dense, int B, int F, int D, int RD, int ND, int lpr,
                           __nv_bfloat16* __restrict__ x, int ldx, float* __restrict__ fm_logit) {
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int stride = (gridDim.x * blockDim.x) / lpr;
  const unsigned group_mask = (lpr == 32 ? 0xffffffffu : ((1u << lpr) - 1u)) << ((threadIdx.x & 31) / lpr * lpr);
  const int chunks = D / 4;
  const int rounds = (B + stride - 1) / stride;
  for (int it = 0; it < rounds; ++it) {
    const int b = gtid / lpr + it * stride;
    float part = 0.f;
    if (b < B) {
      const int* i2 = inv2 + static_cast<size_t>(b) * F;
      __nv_bfloat16* xr = x + static_cast<size_t>(b) * ldx;
      for (int c = lane; c < chunks; c += lpr) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f), q = s;
#pragma unroll 4
        for (int f = 0; f < F; ++f) {
          const float4 e = __ldcg(reinterpret_cast<const float4*>(rows2 + row_of(slots2, i2[f]) * RD) + c);
          s.x += e.x, s.y += e.y, s.z += e.z, s.w += e.w;
          q.x += e.x * e.x, q.y += e.y * e.y, q.z += e.z * e.z, q.w += e.w * e.w;
          __nv_bfloat162 lo = __floats2bfloat162_rn(e.x, e.y), hi = __floats2bfloat162_rn(e.z, e.w);
          uint2 packed;
          packed.x = *reinterpret_cast<uint32_t*>(&lo);
          packed.y = *reinterpret_cast<uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(xr + f * D + c * 4) = packed;
        }
        part += 0.5f * (s.x * s.x - q.x + s.y * s.y - q.y + s.z * s.z - q.z + s.w * s.w - q.w);
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
    for (int o = lpr >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(group_mask, part, o);
    if (b < B && lane == 0) fm_logit[b] = part;
  }
}

__global__ void __launch_bounds__(kThreads)
deepfm_pack_backward_kernel(const float* __restrict__ rows2, const int* __restrict__ inv2,
                            const int* __restrict__ slots2, const int* __restrict__ inv1, const __nv_bfloat16* __restrict__ dx, int lddx,
                            const float* __restrict__ dlogit, int B, int F, int D, int RD, int lpr, float* ugrad2,
                            float* ugrad1) {
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int stride = (gridDim.x * blockDim.x) / lpr;
  const int chunks = D / 4;
  for (int b = gtid / lpr; b < B; b += stride) {
    const int* i2 = inv2 + static_cast<size_t>(b) * F;
    const float g = dlogit[b];
    const __nv_bfloat16* dxr = dx ? dx + static_cast<size_t>(b) * lddx : nullptr;
    for (int c = lane; c < chunks; c += lpr) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
      for (int f = 0; f < F; ++f) {
        const float4 e = __ldcg(reinterpret_cast<const float4*>(rows2 + row_of(slots2, i2[f]) * RD) + c);
        s.x += e.x, s.y += e.y, s.z += e.z, s.w += e.w;
      }
#pragma unroll 4
      for (int f = 0; f < F; ++f) {
        const float4 e = __ldcg(reinterpret_cast<const float4*>(rows2 + row_of(slots2, i2[f]) * RD) + c);
        float4 d = make_float4(g * (s.x - e.x), g * (s.y - e.y), g * (s.z - e.z), g * (s.w - e.w));
        if (dxr) {
          const uint2 p = *reinterpret_cast<const uint2*>(dxr + f * D + c * 4);
          const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&p.x);
          const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&p.y);
          d.x += __bfloat162float(lo.x), d.y += __bfloat162float(lo.y);
          d.z += __bfloat162float(hi.x), d.w += __bfloat162float(hi.y);
        }
        red_add_v4(ugrad2 + static_cast<size_t>(i2[f]) * RD + c * 4, d);
      }
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

int lanes_for_chunks(int chunks) {
  int l = 1;
  while (l < chunks && l < 32) l <<= 1;
  return l;
}

int grid_for(long long rows, int lpr) {
  long long g = (rows * lpr + kThreads - 1) / kThreads;
  if (g < 1) g = 1;
  if (g > 148 * 16) g = 148 * 16;
  return static_cast<int>(g);
}

}  // namespace

void pull_wait(SymHost sym, ChanLayout lay, Ctrl* ctrl, uint32_t spin_limit, cudaStream_t stream) {
  pull_wait_kernel<<<1, 32, 0, stream>>>(to_sym(sym), lay, ctrl, spin_limit);
}

void deepfm_pack_forward(const float* rows2, const int* inv2, const int* slots2, const float* rows1, const int* inv1,
                         const int* slots1, const float* dense, int B, int F, int D, int RD, int ND, __nv_bfloat16* x,
                         int ldx, float* fm_logit, cudaStream_t stream) {
  if (B <= 0) return;
  const int lpr = lanes_for_chunks(D / 4);
  deepfm_pack_forward_kernel<<<grid_for(B, lpr), kThreads, 0, stream>>>(rows2, inv2, slots2, rows1, inv1, slots1, dense,
                                                                        B, F, D, RD, ND, lpr, x, ldx, fm_logit);
}

void deepfm_pack_backward(const float* rows2, const int* inv2, const int* slots2, const int* inv1,
                          const __nv_bfloat16* dx, int lddx,
                          const float* dlogit, int B, int F, int D, int RD, float* ugrad2, float* ugrad1,
                          cudaStream_t stream) {
  if (B <= 0) return;
  const int lpr = lanes_for_chunks(D / 4);
  deepfm_pack_backward_kernel<<<grid_for(B, lpr), kThreads, 0, stream>>>(rows2, inv2, slots2, inv1, dx, lddx, dlogit, B,
                                                                         F, D, RD, lpr, ugrad2, ugrad1);
}

}  // namespace cu
}  // namespace kb
