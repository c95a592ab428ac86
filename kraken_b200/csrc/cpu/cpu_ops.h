// CPU kernels of the client ("emitter") side: id dedup with duplicate-gradient
// summation, jagged (bag) pooling, and DCT = Dynamic Communication
// Thresholding (top-k magnitude sparsification with error feedback).
// They are the CPU backend's hot loops and the oracle for the CUDA kernels.
#pragma once

#include <cstdint>
#include <vector>

namespace kb {
namespace cpu {

// uniq: first-occurrence order; inverse[i] = position of ids[i] in uniq
// (the dedup of kraken/worker/emitter.cc:139-149).
void Dedup(const uint64_t* ids, int64_t n, std::vector<uint64_t>* uniq, std::vector<int64_t>* inverse);

// out[u] = sum of grads[i] over inverse[i] == u  (kraken/worker/emitter.cc:516-531).
void SegmentSum(const float* grads, const int64_t* inverse, int64_t n, int64_t dim, int64_t num_uniq, float* out);

// Bag pooling over values [R, dim] with offsets [k+1].  Empty bags produce
// patch_value.  mean=true divides by the bag length.  Optional per-row weights.
// API of kraken/pytorch/py/jagged_ops.cc:14-145,205-308.
void JaggedForward(const float* values, const float* weights, const int64_t* offsets, int64_t k, int64_t dim,
                   bool mean, float patch_value, float* out);
// Gradient w.r.t. values: every row of a bag receives the bag's gradient
// (scaled by 1/len for mean, by its weight if given).  The reference's
// SumBackward writes only the first row of each bag
// (kraken/pytorch/py/jagged_ops.cc:152-157); this one fills all rows.
void JaggedBackward(const float* grads, const float* weights, const int64_t* offsets, int64_t k, int64_t dim,
                    bool mean, float* out);

// k-th largest |x| (k >= 1).
float KthLargestAbs(const float* x, int64_t n, int64_t k);

// One DCT step on a flat gradient (kraken/worker/dct_emitter.cc:16-43):
//   f = g + e;  every life_span steps tau = k-th largest |f| with k = (int64)(n * (1 - eta));
//   emit (i, f[i]) for |f[i]| >= tau in ascending i;  e = |f| < tau ? f : 0.
// Returns false (nothing touched) when n < 256: the caller sends g dense.
struct DctState {
  std::vector<float> e;
  float tau = 0.f;
  int64_t step = 0;
};
bool DctCompress(const float* g, int64_t n, int64_t life_span, float eta, DctState* st, std::vector<int64_t>* idx,
                 std::vector<float>* vals);

}  // namespace cpu
}  // namespace kb
