// C wrappers around the reference's own gain_func / Weight (src/core/gain.cu),
// compiled as host code from the reference tree where it lies.  Test
// infrastructure: used to validate oracle.cpp's restatement of those functions.
#include "gain.cuh"

using arboretum::core::GainFunctionParameters;
using arboretum::core::gain_func;
using arboretum::core::Weight;

namespace arboretum {
namespace core {
// declared in gain.cu but not in gain.cuh
__host__ __device__ float Weight(const float s, const unsigned int c,
                                 const GainFunctionParameters &param);
__host__ __device__ float Weight(const double s, const unsigned int c,
                                 const GainFunctionParameters &param);
__host__ __device__ float Weight(const float2 s, const unsigned int c,
                                 const GainFunctionParameters &param);
__host__ __device__ float Weight(const double2 s, const unsigned int c,
                                 const GainFunctionParameters &param);
}  // namespace core
}  // namespace arboretum

struct P {
  unsigned min_leaf_size;
  float hess, gamma_absolute, gamma_relative, lambda, alpha, max_leaf_weight;
};
static GainFunctionParameters mk(const P *p) {
  return GainFunctionParameters(p->min_leaf_size, p->hess, p->gamma_absolute,
                                p->gamma_relative, p->lambda, p->alpha,
                                p->max_leaf_weight);
}

extern "C" {
float ref_gain_f(float l, float t, unsigned long long lc, unsigned long long tc, const P *p) {
  return gain_func(l, t, size_t(lc), size_t(tc), mk(p));
}
float ref_gain_d(double l, double t, unsigned long long lc, unsigned long long tc, const P *p) {
  return gain_func(l, t, size_t(lc), size_t(tc), mk(p));
}
float ref_gain_f2(float lx, float ly, float tx, float ty, unsigned long long lc,
                  unsigned long long tc, const P *p) {
  return gain_func(make_float2(lx, ly), make_float2(tx, ty), size_t(lc), size_t(tc), mk(p));
}
float ref_gain_d2(double lx, double ly, double tx, double ty, unsigned long long lc,
                  unsigned long long tc, const P *p) {
  return gain_func(make_double2(lx, ly), make_double2(tx, ty), size_t(lc), size_t(tc), mk(p));
}
float ref_weight_f(float s, unsigned c, const P *p) { return Weight(s, c, mk(p)); }
float ref_weight_d(double s, unsigned c, const P *p) { return Weight(s, c, mk(p)); }
float ref_weight_f2(float x, float y, unsigned c, const P *p) {
  return Weight(make_float2(x, y), c, mk(p));
}
float ref_weight_d2(double x, double y, unsigned c, const P *p) {
  return Weight(make_double2(x, y), c, mk(p));
}
}
