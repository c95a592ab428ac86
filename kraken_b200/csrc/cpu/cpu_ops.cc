#include "cpu_ops.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <unordered_map>

#include "../core/hash.h"
#include "../core/types.h"

namespace kb {
namespace cpu {

void Dedup(const uint64_t* ids, int64_t n, std::vector<uint64_t>* uniq, std::vector<int64_t>* inverse) {
  // Flat open-addressing set (linear probing, at most half full): unique ids keep the order of
  // their first occurrence.  About four times faster than std::unordered_map at a few 10^4 ids.
  uniq->clear();
  inverse->resize(static_cast<size_t>(n));
  size_t cap = 16;
  while (cap < static_cast<size_t>(2 * n)) cap <<= 1;
  const size_t mask = cap - 1;
  std::vector<uint64_t> keys(cap);
  std::vector<int64_t> pos(cap, -1);
  for (int64_t i = 0; i < n; ++i) {
    const uint64_t id = ids[i];
    size_t h = static_cast<size_t>(Mix64(id)) & mask;
    while (pos[h] >= 0 && keys[h] != id) h = (h + 1) & mask;
    if (pos[h] < 0) {
      keys[h] = id;
      pos[h] = static_cast<int64_t>(uniq->size());
      uniq->push_back(id);
    }
    (*inverse)[static_cast<size_t>(i)] = pos[h];
  }
}

void SegmentSum(const float* grads, const int64_t* inverse, int64_t n, int64_t dim, int64_t num_uniq, float* out) {
  std::memset(out, 0, sizeof(float) * num_uniq * dim);
  for (int64_t i = 0; i < n; ++i) {
    float* dst = out + inverse[i] * dim;
    const float* src = grads + i * dim;
    for (int64_t j = 0; j < dim; ++j) dst[j] += src[j];
  }
}

void JaggedForward(const float* values, const float* weights, const int64_t* offsets, int64_t k, int64_t dim,
                   bool mean, float patch_value, float* out) {
  for (int64_t b = 0; b < k; ++b) {
    float* dst = out + b * dim;
    const int64_t lo = offsets[b], hi = offsets[b + 1];
    if (hi <= lo) {
      for (int64_t j = 0; j < dim; ++j) dst[j] = patch_value;
      continue;
    }
    for (int64_t j = 0; j < dim; ++j) dst[j] = 0.f;
    for (int64_t r = lo; r < hi; ++r) {
      const float w = weights ? weights[r] : 1.f;
      const float* src = values + r * dim;
      for (int64_t j = 0; j < dim; ++j) dst[j] += w * src[j];
    }
    if (mean) {
      const float inv = 1.f / static_cast<float>(hi - lo);
      for (int64_t j = 0; j < dim; ++j) dst[j] *= inv;
    }
  }
}

void JaggedBackward(const float* grads, const float* weights, const int64_t* offsets, int64_t k, int64_t dim,
                    bool mean, float* out) {
  for (int64_t b = 0; b < k; ++b) {
    const int64_t lo = offsets[b], hi = offsets[b + 1];
    if (hi <= lo) continue;
    const float scale = mean ? 1.f / static_cast<float>(hi - lo) : 1.f;
    const float* src = grads + b * dim;
    for (int64_t r = lo; r < hi; ++r) {
      const float w = scale * (weights ? weights[r] : 1.f);
      float* dst = out + r * dim;
      for (int64_t j = 0; j < dim; ++j) dst[j] = w * src[j];
    }
  }
}

float KthLargestAbs(const float* x, int64_t n, int64_t k) {
  KB_CHECK(k >= 1 && k <= n, err::kBadArgument, "k-th largest: k out of range");
  std::vector<float> a(n);
  for (int64_t i = 0; i < n; ++i) a[i] = std::fabs(x[i]);
  std::nth_element(a.begin(), a.begin() + (k - 1), a.end(), std::greater<float>());
  return a[k - 1];
}

bool DctCompress(const float* g, int64_t n, int64_t life_span, float eta, DctState* st, std::vector<int64_t>* idx,
                 std::vector<float>* vals) {
  if (n < 256) return false;
  if (st->e.size() != static_cast<size_t>(n)) st->e.assign(n, 0.f);
  std::vector<float> f(n);
  for (int64_t i = 0; i < n; ++i) f[i] = g[i] + st->e[i];
  if (st->step % life_span == 0) {
    const int64_t k = static_cast<int64_t>(static_cast<double>(n) * (1.0 - static_cast<double>(eta)));
    KB_CHECK(k >= 1, err::kBadArgument, "DCT keeps no element: eta too close to 1");
    st->tau = KthLargestAbs(f.data(), n, k);
  }
  idx->clear();
  vals->clear();
  const float tau = st->tau;
  for (int64_t i = 0; i < n; ++i) {
    if (std::fabs(f[i]) >= tau) {
      idx->push_back(i);
      vals->push_back(f[i]);
      st->e[i] = 0.f;
    } else {
      st->e[i] = f[i];
    }
  }
  st->step += 1;
  return true;
}

}  // namespace cpu
}  // namespace kb
