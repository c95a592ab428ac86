// bf16 GEMMs of the MLP head on the 5th-generation tensor cores (tcgen05),
// operands staged by TMA into 128-byte-swizzled shared memory, fp32 accumulators
// in tensor memory, epilogue fused.  Three entry points cover a Linear layer's
// forward, input gradient and weight gradient:
//
//   linear_forward   Y[M,N]  = act(X[M,K] * W[N,K]^T + bias)         bf16 out
//   linear_dgrad     dX[M,K] = (dY[M,N] * Wt[K,N]^T) .* (H > 0)       bf16 out, Wt = W^T stored [K,N]
//   linear_wgrad     dW[N,K] += dY[M,N]^T * X[M,K]                    fp32 red-add, split over M
//
// All matrices are row-major with leading dimensions (in elements) that are
// multiples of 8, so every TMA row pitch is a multiple of 16 bytes.
// The reference runs these layers as torch.nn.Linear on the CPU
// (examples/DeepFM/model/DeepFM.py:113-116, examples/WideAndDeep/model.py:114-125).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace kb {
namespace cu {

// Each returns 0 on success or a negative code when a tensor map cannot be encoded
// (bad alignment / driver entry point missing).  `status` (device int) receives
// err::kTimeout if a pipeline wait inside the kernel gives up.
//
// ReLU mask: the forward pass can leave one bit per output element (output > 0) in
// mask_out[ceil(N / 16), ldm] (uint16 word (c, r) = columns [16c, 16c + 16) of row r, ldm >= M, so the
// 32 rows of a warp write 64 contiguous bytes); the input gradient of the next layer then takes that
// bit mask instead of re-reading the bf16 activations H, which cuts its extra read traffic
// sixteen-fold.  Either may be null; with both null no mask is applied.
int linear_forward(const __nv_bfloat16* X, int ldx, const __nv_bfloat16* W, int ldw, const float* bias,
                   __nv_bfloat16* Y, int ldy, int M, int N, int K, bool relu, uint16_t* mask_out, int ldm, int* status,
                   cudaStream_t stream);

int linear_dgrad(const __nv_bfloat16* dY, int lddy, const __nv_bfloat16* Wt, int ldwt, const __nv_bfloat16* H,
                 int ldh, const uint16_t* mask, int ldm, __nv_bfloat16* dX, int lddx, int M, int N, int K, int* status,
                 cudaStream_t stream);

int linear_wgrad(const __nv_bfloat16* dY, int lddy, const __nv_bfloat16* X, int ldx, float* dW, int lddw, int M,
                 int N, int K, int* status, cudaStream_t stream);

// Knobs for measurements.  variant: 0 = chosen from the shape, 1 = weight-resident CTA pair
// (cta_group::2), 2 = weight-resident single CTA, 3 = one output tile per CTA.  n_tiles: column
// tiles of the resident variants (0 = chosen from the shape).
void gemm_set_tuning(int variant, int n_tiles);

// Column sums of a bf16 matrix added into an fp32 vector: db[n] += sum_m dY[m, n].
void colsum_bf16(const __nv_bfloat16* dY, int lddy, int M, int N, float* db, cudaStream_t stream);

}  // namespace cu
}  // namespace kb
