// Regularised split gain and leaf weight in the reference's arithmetic
// (src/core/gain.cu:8-238), for sums held in double.  The histograms of this
// build are exact fixed-point integers; they are converted to double (exactly)
// and then follow the reference's `double` / `double2` overloads operation by
// operation: weights and the three gain terms are rounded to float where the
// reference rounds them, the inner expression is evaluated in double.
#pragma once
#include <cuda_runtime.h>

namespace arb {

struct GainParams {  // GainFunctionParameters, gain.cuh:11-30
  unsigned min_leaf_size;
  float hess;  // tree.min_child_weight (garden.cu:90-92)
  float gamma_absolute;
  float gamma_relative;
  float lambda;
  float alpha;
  float max_leaf_weight;
};

__host__ __device__ inline int sgn(double v) { return (0.0 < v) - (v < 0.0); }

__host__ __device__ inline double grad_regularized(double grad, float alpha) {  // gain.cu:19-23
  const double grad_abs = fabs(grad);
  return sgn(grad) * fmax(0.0, grad_abs - alpha);
}

__host__ __device__ inline float threshold_weight(float w, float mlw) {  // gain.cu:25-32
  if (mlw != 0.0f) {
    if (w > mlw) return mlw;
    if (w < -mlw) return -mlw;
  }
  return w;
}

// PAIR = true : (sum g, sum h) statistics  -> Weight(double2, ...) gain.cu:67-76
// PAIR = false: sum g with hessian == count -> Weight(double, ...)  gain.cu:45-54
template <bool PAIR>
__host__ __device__ inline float leaf_weight(double g, double h, unsigned c, float mcw,
                                             unsigned mls, float lambda, float alpha,
                                             float mlw) {
  float w = 0.0f;
  if (PAIR) {
    if (c >= mls && h >= mcw) w = float(grad_regularized(g, alpha) / (h + lambda));
  } else {
    if (c >= mls && c >= mcw) w = float(grad_regularized(g, alpha) / (c + lambda));
  }
  return threshold_weight(w, mlw);
}

template <bool PAIR>
__host__ __device__ inline float gain_term(double g, double h, unsigned long long c, float w,
                                           float lambda, float alpha) {  // gain.cu:13-17
  if (PAIR) return float(-2 * (g * (-w) + 0.5 * (h + lambda) * w * w + alpha * fabsf(w)));
  return float(-2 * (g * (-w) + 0.5 * (c + lambda) * w * w + alpha * fabsf(w)));
}

// gain.cu:125-152 (double2) and :212-238 (double).  `lc`, `tc` are row counts; for
// PAIR statistics the caller may pass any value that is >= min_leaf_size exactly
// when the true count is (this build passes 0/1 for empty/non-empty when
// min_leaf_size <= 1).
template <bool PAIR>
__host__ __device__ inline float split_gain(double lg, double lh, double tg, double th,
                                            unsigned long long lc, unsigned long long tc,
                                            const GainParams &p) {
  const double rg = tg - lg, rh = th - lh;
  const unsigned long long rc = tc - lc;
  bool ok = lc >= p.min_leaf_size && rc >= p.min_leaf_size;
  if (PAIR) ok = ok && fabs(lh) >= p.hess && fabs(rh) >= p.hess;
  if (!ok) return 0.0f;
  const float wl = leaf_weight<PAIR>(lg, lh, unsigned(lc), p.hess, p.min_leaf_size, p.lambda,
                                     p.alpha, p.max_leaf_weight);
  const float wr = leaf_weight<PAIR>(rg, rh, unsigned(rc), p.hess, p.min_leaf_size, p.lambda,
                                     p.alpha, p.max_leaf_weight);
  const float wp = leaf_weight<PAIR>(tg, th, unsigned(tc), p.hess, p.min_leaf_size, p.lambda,
                                     p.alpha, p.max_leaf_weight);
  const float l = gain_term<PAIR>(lg, lh, lc, wl, p.lambda, p.alpha);
  const float r = gain_term<PAIR>(rg, rh, rc, wr, p.lambda, p.alpha);
  const float q = gain_term<PAIR>(tg, th, tc, wp, p.lambda, p.alpha);
  const float diff = l + r - q;
  return (diff > p.gamma_absolute && diff > p.gamma_relative * q) * diff;
}

}  // namespace arb
