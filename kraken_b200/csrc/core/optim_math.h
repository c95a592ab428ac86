// Server-side optimizer and initializer math, one element at a time, shared by
// the CPU shard and the CUDA row/dense-slice kernels so both run the same
// arithmetic.
//
// Update rules follow the reference's server optimizers
// (kraken/ps/optim/sgd.cc:25-63, adagrad.cc:18-48, adam.cc:23-81,
// rmsprop.cc:23-78) including their quirks: SGD's first momentum step copies
// the gradient, Adam keeps a step counter per row / per dense table and its
// amsgrad maximum is taken over the bias-corrected second moment.  One
// addition: Adagrad's `initial_accumulator_value` (default 0, which is the
// reference's behaviour).
//
// State slab assignment (slab index -> checkpoint StateType):
//   SGD      s0 = MomentumBuffer
//   Adagrad  s0 = StateSum
//   Adam     s0 = FirstMoment  s1 = SecondMoment  s2 = SecondMomentMax (amsgrad)
//   RMSprop  s0 = SquareAverage  s1 = GAve (centered)  s2 = MomentumBuffer (momentum)
#pragma once

#include <cmath>
#include <cstdint>

#include "hash.h"
#include "types.h"

namespace kb {

struct OptimPOD {
  uint8_t type = 3;  // OptimType
  bool has_weight_decay = false;
  bool has_momentum = false;
  bool has_dampening = false;
  bool nesterov = false;
  bool amsgrad = false;
  bool centered = false;
  float weight_decay = 0.f;
  float momentum = 0.f;
  float dampening = 0.f;
  float beta1 = 0.9f;
  float beta2 = 0.999f;
  float alpha = 0.99f;
  float eps = 1e-8f;
  float initial_accumulator_value = 0.f;

  // Whether state slab `slab` (0..2) is allocated for this optimizer.
  KB_HD bool SlabUsed(int slab) const {
    switch (type) {
      case 0: return slab == 0;
      case 1: return slab < 2 || amsgrad;
      case 2: return slab == 0 || (slab == 1 && centered) || (slab == 2 && has_momentum);
      default: return slab == 0 && has_momentum;
    }
  }
  KB_HD bool NeedsSteps() const { return type == 1 || (type == 3 && has_momentum); }
};

struct InitPOD {
  uint8_t type = 0;  // InitializerType
  float a = 0.f;     // constant: value | uniform: lower | normal: mean | xavier: gain
  float b = 1.f;     // uniform: upper | normal: stddev
};

// Per-step scalars of Adam that depend only on the step count.
struct AdamBias {
  float inv_bc1;
  float inv_bc2;
};

KB_HD AdamBias AdamBiasAt(const OptimPOD& o, int64_t step) {
  AdamBias b;
  b.inv_bc1 = 1.f / (1.f - powf(o.beta1, static_cast<float>(step)));
  b.inv_bc2 = 1.f / (1.f - powf(o.beta2, static_cast<float>(step)));
  return b;
}

// Applies one update to a single element.  `step` is the counter AFTER the
// increment (1 on the first update).  Unused state references may alias a dummy.
KB_HD void UpdateElem(const OptimPOD& o, float lr, float g, int64_t step, const AdamBias& ab, float& w, float& s0,
                      float& s1, float& s2) {
  if (o.has_weight_decay) g += o.weight_decay * w;
  switch (o.type) {
    case 0: {  // Adagrad
      s0 += g * g;
      w -= lr * g / (sqrtf(s0) + o.eps);
      break;
    }
    case 1: {  // Adam
      s0 = o.beta1 * s0 + (1.f - o.beta1) * g;
      s1 = o.beta2 * s1 + (1.f - o.beta2) * g * g;
      const float mhat = s0 * ab.inv_bc1;
      float vhat = s1 * ab.inv_bc2;
      if (o.amsgrad) {
        s2 = fmaxf(s2, vhat);
        vhat = s2;
      }
      w -= lr * mhat / (sqrtf(vhat) + o.eps);
      break;
    }
    case 2: {  // RMSprop
      s0 = o.alpha * s0 + (1.f - o.alpha) * g * g;
      float avg = s0;
      if (o.centered) {
        s1 = o.alpha * s1 + (1.f - o.alpha) * g;
        avg = s0 - s1 * s1;
      }
      if (o.has_momentum) {
        s2 = o.momentum * s2 + g / (sqrtf(avg) + o.eps);
        w -= lr * s2;
      } else {
        w -= lr * g / (sqrtf(avg) + o.eps);
      }
      break;
    }
    default: {  // SGD
      if (o.has_momentum) {
        s0 = (step <= 1) ? g : o.momentum * s0 + (1.f - (o.has_dampening ? o.dampening : 0.f)) * g;
        g = o.nesterov ? g + o.momentum * s0 : s0;
      }
      w -= lr * g;
      break;
    }
  }
}

// ---------------------------------------------------------------- counter RNG
// Philox-4x32-10 keyed by (seed, table) with counter (row id, lane): a new row
// gets the same initial value no matter which rank or kernel creates it.
struct Philox4 {
  uint32_t v[4];
};

KB_HD void MulHiLo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
  const uint64_t p = static_cast<uint64_t>(a) * b;
  hi = static_cast<uint32_t>(p >> 32);
  lo = static_cast<uint32_t>(p);
}

KB_HD Philox4 Philox(uint64_t key, uint64_t ctr_lo, uint64_t ctr_hi) {
  uint32_t c0 = static_cast<uint32_t>(ctr_lo), c1 = static_cast<uint32_t>(ctr_lo >> 32);
  uint32_t c2 = static_cast<uint32_t>(ctr_hi), c3 = static_cast<uint32_t>(ctr_hi >> 32);
  uint32_t k0 = static_cast<uint32_t>(key), k1 = static_cast<uint32_t>(key >> 32);
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (int r = 0; r < 10; ++r) {
    uint32_t h0, l0, h1, l1;
    MulHiLo(0xD2511F53u, c0, h0, l0);
    MulHiLo(0xCD9E8D57u, c2, h1, l1);
    c0 = h1 ^ c1 ^ k0;
    c1 = l1;
    c2 = h0 ^ c3 ^ k1;
    c3 = l0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  Philox4 out;
  out.v[0] = c0;
  out.v[1] = c1;
  out.v[2] = c2;
  out.v[3] = c3;
  return out;
}

KB_HD float U01(uint32_t x) { return (static_cast<float>(x >> 8) + 0.5f) * (1.0f / 16777216.0f); }  // (0,1)

// Initial values of elements 4q .. 4q+3 of the row `id` of a `dim`-wide table
// (one Philox call yields four values).
// Xavier on a [dim] row uses fan_out = dim, fan_in = 1 (kraken/t/math.cc:24-50,476-517).
KB_HD void InitQuad(const InitPOD& ip, uint64_t seed_key, uint64_t id, uint32_t q, uint32_t dim, float out[4]) {
  if (ip.type == 0) {
    out[0] = out[1] = out[2] = out[3] = ip.a;
    return;
  }
  const Philox4 r = Philox(seed_key, id, static_cast<uint64_t>(q));
  const float u0 = U01(r.v[0]), u1 = U01(r.v[1]), u2 = U01(r.v[2]), u3 = U01(r.v[3]);
  const float xavier_std = ip.a * sqrtf(2.f / (static_cast<float>(dim) + 1.f));
  if (ip.type == 1 || ip.type == 3) {
    const float lo = ip.type == 1 ? ip.a : -1.7320508075688772f * xavier_std;
    const float hi = ip.type == 1 ? ip.b : 1.7320508075688772f * xavier_std;
    out[0] = lo + (hi - lo) * u0;
    out[1] = lo + (hi - lo) * u1;
    out[2] = lo + (hi - lo) * u2;
    out[3] = lo + (hi - lo) * u3;
  } else {
    const float mean = ip.type == 2 ? ip.a : 0.f;
    const float stdv = ip.type == 2 ? ip.b : xavier_std;
    const float r0 = stdv * sqrtf(-2.f * logf(u0)), r1 = stdv * sqrtf(-2.f * logf(u2));
    const float t0 = 6.283185307179586f * u1, t1 = 6.283185307179586f * u3;
    out[0] = mean + r0 * cosf(t0);
    out[1] = mean + r0 * sinf(t0);
    out[2] = mean + r1 * cosf(t1);
    out[3] = mean + r1 * sinf(t1);
  }
}

// Writes the initial values of a whole row.
KB_HD void InitRow(const InitPOD& ip, uint64_t seed_key, uint64_t id, uint32_t dim, float* row) {
  for (uint32_t q = 0; q * 4 < dim; ++q) {
    float v[4];
    InitQuad(ip, seed_key, id, q, dim, v);
    for (uint32_t k = 0; k < 4 && q * 4 + k < dim; ++k) row[q * 4 + k] = v[k];
  }
}

}  // namespace kb
