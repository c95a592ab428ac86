// Memory-bound model kernels: jagged (bag) pooling, FM second-order
// interaction and binary cross entropy with logits.  Each makes one pass over
// its input at HBM speed with the reduction done in registers / shuffles.
//
// Counterparts in the reference: kraken/pytorch/py/jagged_ops.cc:14-420 (CPU,
// OpenMP), examples/DeepFM/model/DeepFM.py:96-107 (FM as torch expressions)
// and :140 (BCEWithLogits).
#include <cuda_bf16.h>

#include "common.cuh"
#include "kernels.h"

namespace kb {
namespace cu {

namespace {

constexpr int kThreads = 256;

int lanes_for(int dim) {
  int l = 1;
  while (l < dim && l < 32) l <<= 1;
  return l;
}

int grid_rows(long long rows, int lpr, int cap = 148 * 16) {
  long long g = (rows * lpr + kThreads - 1) / kThreads;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return static_cast<int>(g);
}

__global__ void __launch_bounds__(kThreads)
jagged_forward_kernel(const float* __restrict__ values, const float* __restrict__ weights,
                      const int64_t* __restrict__ offsets, int k, int dim, int lpr, int mean, float patch_value,
                      float* __restrict__ out) {
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int stride = (gridDim.x * blockDim.x) / lpr;
  for (int b = gtid / lpr; b < k; b += stride) {
    const int64_t lo = offsets[b], hi = offsets[b + 1];
    for (int j = lane; j < dim; j += lpr) {
      float acc = 0.f;
      for (int64_t r = lo; r < hi; ++r) acc += (weights ? weights[r] : 1.f) * values[r * dim + j];
      if (hi <= lo)
        acc = patch_value;
      else if (mean)
        acc /= static_cast<float>(hi - lo);
      out[static_cast<size_t>(b) * dim + j] = acc;
    }
  }
}

__global__ void __launch_bounds__(kThreads)
jagged_backward_kernel(const float* __restrict__ grads, const float* __restrict__ weights,
                       const int64_t* __restrict__ offsets, int k, int dim, int lpr, int mean,
                       float* __restrict__ out) {
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int stride = (gridDim.x * blockDim.x) / lpr;
  for (int b = gtid / lpr; b < k; b += stride) {
    const int64_t lo = offsets[b], hi = offsets[b + 1];
    if (hi <= lo) continue;
    const float scale = mean ? 1.f / static_cast<float>(hi - lo) : 1.f;
    for (int j = lane; j < dim; j += lpr) {
      const float g = grads[static_cast<size_t>(b) * dim + j] * scale;
      for (int64_t r = lo; r < hi; ++r) out[r * dim + j] = weights ? g * weights[r] : g;
    }
  }
}

__global__ void __launch_bounds__(kThreads)
fm_forward_kernel(const float* __restrict__ emb, int B, int F, int D, int lpr, float* __restrict__ out) {
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int stride = (gridDim.x * blockDim.x) / lpr;
  const unsigned group_mask = (lpr == 32 ? 0xffffffffu : ((1u << lpr) - 1u)) << ((threadIdx.x & 31) / lpr * lpr);
  const int rounds = (B + stride - 1) / stride;
  for (int it = 0; it < rounds; ++it) {
    const int b = gtid / lpr + it * stride;
    float part = 0.f;
    if (b < B) {
      const float* e = emb + static_cast<size_t>(b) * F * D;
      for (int j = lane; j < D; j += lpr) {
        float s = 0.f, q = 0.f;
        for (int f = 0; f < F; ++f) {
          const float v = e[f * D + j];
          s += v;
          q += v * v;
        }
        part += 0.5f * (s * s - q);
      }
    }
    for (int o = lpr >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(group_mask, part, o);
    if (b < B && lane == 0) out[b] = part;
  }
}

__global__ void __launch_bounds__(kThreads)
fm_backward_kernel(const float* __restrict__ emb, const float* __restrict__ gout, int B, int F, int D, int lpr,
                   float* __restrict__ gemb) {
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = gtid % lpr;
  const int stride = (gridDim.x * blockDim.x) / lpr;
  for (int b = gtid / lpr; b < B; b += stride) {
    const float* e = emb + static_cast<size_t>(b) * F * D;
    float* g = gemb + static_cast<size_t>(b) * F * D;
    const float go = gout[b];
    for (int j = lane; j < D; j += lpr) {
      float s = 0.f;
      for (int f = 0; f < F; ++f) s += e[f * D + j];
      for (int f = 0; f < F; ++f) g[f * D + j] = go * (s - e[f * D + j]);
    }
  }
}

__global__ void __launch_bounds__(kThreads)
bce_kernel(const float* __restrict__ logits, const float* __restrict__ labels, int n, float inv_n, float* loss,
           float* __restrict__ grad) {
  pdl_enter();
  float acc = 0.f;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const float x = logits[i], y = labels[i];
    const float ax = fabsf(x);
    const float t = expf(-ax);
    acc += fmaxf(x, 0.f) - x * y + log1pf(t);
    if (grad) {
      const float sig = x >= 0.f ? 1.f / (1.f + t) : t / (1.f + t);
      grad[i] = (sig - y) * inv_n;
    }
  }
  __shared__ float warp_sum[kThreads / 32];
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kThreads / 32 ? warp_sum[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) atomicAdd(loss, v * inv_n);
  }
}

// ---- Linear layer with a single output (the MLP's logit head): y[m] = x[m, :] . w + b
__global__ void __launch_bounds__(kThreads)
rowdot_forward_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const float* __restrict__ w,
                      const float* __restrict__ bias, const float* __restrict__ addend, int M, int K,
                      float* __restrict__ y) {
  pdl_enter();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int m = warp; m < M; m += nwarps) {
    const __nv_bfloat16* row = x + static_cast<size_t>(m) * ldx;
    float acc = 0.f;
    for (int k = lane * 2; k < K; k += 64) {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(row + k);
      acc += __bfloat162float(v.x) * w[k];
      if (k + 1 < K) acc += __bfloat162float(v.y) * w[k + 1];
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[m] = acc + (bias ? bias[0] : 0.f) + (addend ? addend[m] : 0.f);
  }
}

// dx[m, k] = dy[m] * w[k] * (x[m, k] > 0 if relu_mask), dw[k] += sum_m dy[m] x[m, k], db += sum_m dy[m]
__global__ void __launch_bounds__(kThreads)
rowdot_backward_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const float* __restrict__ w,
                       const float* __restrict__ dy, int M, int K, int rows_per_block, int relu_mask,
                       __nv_bfloat16* __restrict__ dx, int lddx, float* dw, float* db) {
  pdl_enter();
  const int r0 = blockIdx.x * rows_per_block;
  const int r1 = min(M, r0 + rows_per_block);
  for (int k = threadIdx.x * 2; k < K; k += 2 * blockDim.x) {
    const float w0 = w[k], w1 = (k + 1 < K) ? w[k + 1] : 0.f;
    float a0 = 0.f, a1 = 0.f;
    for (int m = r0; m < r1; ++m) {
      const float g = dy[m];
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(x + static_cast<size_t>(m) * ldx + k);
      const float x0 = __bfloat162float(v.x), x1 = __bfloat162float(v.y);
      a0 += g * x0;
      a1 += g * x1;
      if (dx) {
        const float d0 = (!relu_mask || x0 > 0.f) ? g * w0 : 0.f;
        const float d1 = (!relu_mask || x1 > 0.f) ? g * w1 : 0.f;
        *reinterpret_cast<__nv_bfloat162*>(dx + static_cast<size_t>(m) * lddx + k) = __floats2bfloat162_rn(d0, d1);
      }
    }
    atomicAdd(dw + k, a0);
    if (k + 1 < K) atomicAdd(dw + k + 1, a1);
  }
  if (db && threadIdx.x == 0) {
    float s = 0.f;
    for (int m = r0; m < r1; ++m) s += dy[m];
    atomicAdd(db, s);
  }
}

// Same contract, for K % 8 == 0 and 16-byte aligned rows: a thread owns 8 columns (one 16-byte
// load and store per row), the block's threads are split into row lanes, and every thread keeps
// two rows in flight, so the kernel streams x and dx at memory speed instead of waiting on one
// 4-byte load at a time.
__global__ void __launch_bounds__(kThreads)
rowdot_backward_wide_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const float* __restrict__ w,
                            const float* __restrict__ dy, int M, int K, int rows_per_block, int relu_mask,
                            __nv_bfloat16* __restrict__ dx, int lddx, float* dw, float* db) {
  pdl_enter();
  extern __shared__ float s_dw[];  // [K] partial sums of this block
  const int groups = K / 8;                       // 16-byte column groups per row
  const int lanes = blockDim.x / groups;          // row lanes (>= 1: the launcher guarantees groups <= blockDim.x)
  const int cg = threadIdx.x % groups;
  const int rl = threadIdx.x / groups;
  const int r0 = blockIdx.x * rows_per_block;
  const int r1 = min(M, r0 + rows_per_block);
  for (int k = threadIdx.x; k < K; k += blockDim.x) s_dw[k] = 0.f;
  __syncthreads();
  if (rl < lanes) {
    float wk[8], acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) wk[j] = w[cg * 8 + j], acc[j] = 0.f;
    for (int m = r0 + rl; m < r1; m += 2 * lanes) {
      const int m2 = m + lanes;
      const bool two = m2 < r1;
      const uint4 va = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(m) * ldx + cg * 8);
      const uint4 vb = two ? *reinterpret_cast<const uint4*>(x + static_cast<size_t>(m2) * ldx + cg * 8) : va;
      const float ga = dy[m], gb = two ? dy[m2] : 0.f;
      const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
      uint32_t oa[4], ob[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 pa = *reinterpret_cast<const __nv_bfloat162*>(&wa[j]);
        const __nv_bfloat162 pb = *reinterpret_cast<const __nv_bfloat162*>(&wb[j]);
        const float a0 = __bfloat162float(pa.x), a1 = __bfloat162float(pa.y);
        const float b0 = __bfloat162float(pb.x), b1 = __bfloat162float(pb.y);
        acc[2 * j] += ga * a0 + gb * b0;
        acc[2 * j + 1] += ga * a1 + gb * b1;
        const __nv_bfloat162 da = __floats2bfloat162_rn((!relu_mask || a0 > 0.f) ? ga * wk[2 * j] : 0.f,
                                                        (!relu_mask || a1 > 0.f) ? ga * wk[2 * j + 1] : 0.f);
        const __nv_bfloat162 dbv = __floats2bfloat162_rn((!relu_mask || b0 > 0.f) ? gb * wk[2 * j] : 0.f,
                                                         (!relu_mask || b1 > 0.f) ? gb * wk[2 * j + 1] : 0.f);
        oa[j] = *reinterpret_cast<const uint32_t*>(&da);
        ob[j] = *reinterpret_cast<const uint32_t*>(&dbv);
      }
      if (dx) {
        *reinterpret_cast<uint4*>(dx + static_cast<size_t>(m) * lddx + cg * 8) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
        if (two)
          *reinterpret_cast<uint4*>(dx + static_cast<size_t>(m2) * lddx + cg * 8) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(&s_dw[cg * 8 + j], acc[j]);
  }
  __syncthreads();
  for (int k = threadIdx.x; k < K; k += blockDim.x) atomicAdd(dw + k, s_dw[k]);
  if (db && threadIdx.x == 0) {
    float sum = 0.f;
    for (int m = r0; m < r1; ++m) sum += dy[m];
    atomicAdd(db, sum);
  }
}

// fp32 weight [N, K] -> bf16 copy [N, K] and bf16 transpose [K, N] in one pass (the forward and
// the input-gradient GEMMs want the two layouts).
__global__ void __launch_bounds__(256)
cast_w_wt_kernel(const float* __restrict__ w, int N, int K, __nv_bfloat16* __restrict__ w16,
                 __nv_bfloat16* __restrict__ wt16) {
  pdl_enter();
  __shared__ float tile[32][33];
  const int n0 = blockIdx.y * 32, k0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int r = ty; r < 32; r += 8) {
    const int n = n0 + r, k = k0 + tx;
    const float v = (n < N && k < K) ? w[static_cast<size_t>(n) * K + k] : 0.f;
    tile[r][tx] = v;
    if (n < N && k < K) w16[static_cast<size_t>(n) * K + k] = __float2bfloat16(v);
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int k = k0 + r, n = n0 + tx;
    if (k < K && n < N) wt16[static_cast<size_t>(k) * N + n] = __float2bfloat16(tile[tx][r]);
  }
}

}  // namespace

void jagged_forward(const float* values, const float* weights, const int64_t* offsets, int k, int dim, bool mean,
                    float patch_value, float* out, cudaStream_t stream) {
  if (k <= 0) return;
  const int lpr = lanes_for(dim);
  jagged_forward_kernel<<<grid_rows(k, lpr), kThreads, 0, stream>>>(values, weights, offsets, k, dim, lpr, mean ? 1 : 0,
                                                                    patch_value, out);
}

void jagged_backward(const float* grads, const float* weights, const int64_t* offsets, int k, int dim, bool mean,
                     float* out, cudaStream_t stream) {
  if (k <= 0) return;
  const int lpr = lanes_for(dim);
  jagged_backward_kernel<<<grid_rows(k, lpr), kThreads, 0, stream>>>(grads, weights, offsets, k, dim, lpr, mean ? 1 : 0,
                                                                     out);
}

void fm_forward(const float* emb, int B, int F, int D, float* out, cudaStream_t stream) {
  if (B <= 0) return;
  const int lpr = lanes_for(D);
  fm_forward_kernel<<<grid_rows(B, lpr), kThreads, 0, stream>>>(emb, B, F, D, lpr, out);
}

void fm_backward(const float* emb, const float* gout, int B, int F, int D, float* gemb, cudaStream_t stream) {
  if (B <= 0) return;
  const int lpr = lanes_for(D);
  fm_backward_kernel<<<grid_rows(B, lpr), kThreads, 0, stream>>>(emb, gout, B, F, D, lpr, gemb);
}

void bce_forward_backward(const float* logits, const float* labels, int n, float* loss, float* grad,
                          cudaStream_t stream) {
  if (n <= 0) return;
  int grid = (n + kThreads - 1) / kThreads;
  if (grid > 148 * 4) grid = 148 * 4;
  launch_pdl(bce_kernel, dim3(grid), dim3(kThreads), 0, stream, logits, labels, n, 1.f / static_cast<float>(n), loss, grad);
}

void rowdot_forward(const __nv_bfloat16* x, int ldx, const float* w, const float* bias, const float* addend, int M,
                    int K, float* y, cudaStream_t stream) {
  if (M <= 0) return;
  int grid = (M * 32 + kThreads - 1) / kThreads;
  if (grid > 148 * 8) grid = 148 * 8;
  launch_pdl(rowdot_forward_kernel, dim3(grid), dim3(kThreads), 0, stream, x, ldx, w, bias, addend, M, K, y);
}

void rowdot_backward(const __nv_bfloat16* x, int ldx, const float* w, const float* dy, int M, int K, bool relu_mask,
                     __nv_bfloat16* dx, int lddx, float* dw, float* db, cudaStream_t stream) {
  if (M <= 0) return;
  int blocks = 148 * 4;
  int rows_per_block = (M + blocks - 1) / blocks;
  if (rows_per_block < 16) rows_per_block = 16;
  blocks = (M + rows_per_block - 1) / rows_per_block;
  const bool wide = K % 8 == 0 && K / 8 <= kThreads && ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                    (dx == nullptr || (lddx % 8 == 0 && (reinterpret_cast<uintptr_t>(dx) & 15) == 0));
  if (wide) {
    launch_pdl(rowdot_backward_wide_kernel, dim3(blocks), dim3(kThreads), K * sizeof(float), stream, x, ldx, w, dy, M, K,
               rows_per_block, relu_mask ? 1 : 0, dx, lddx, dw, db);
    return;
  }
  launch_pdl(rowdot_backward_kernel, dim3(blocks), dim3(kThreads), 0, stream, x, ldx, w, dy, M, K, rows_per_block,
             relu_mask ? 1 : 0, dx, lddx, dw, db);
}

void cast_w_wt(const float* w, int N, int K, __nv_bfloat16* w16, __nv_bfloat16* wt16, cudaStream_t stream) {
  if (N <= 0 || K <= 0) return;
  launch_pdl(cast_w_wt_kernel, dim3((K + 31) / 32, (N + 31) / 32), dim3(256), 0, stream, w, N, K, w16, wt16);
}

}  // namespace cu
}  // namespace kb
