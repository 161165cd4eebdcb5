// Pre-included when compiling the reference's src/core/gain.cu for the host
// (oracle/Makefile target `ref`).  The reference's cuda_helpers.h does not
// compile with CUDA 12.9 (its `void atomicAdd(float2*, float2)` collides with the
// toolkit's overload), and gain.cu needs only the vector subtraction operators
// from it, so the header is replaced by these two operators.
#ifndef SRC_CORE_CUDA_HELPERS_H
#define SRC_CORE_CUDA_HELPERS_H
#include <cuda_runtime.h>
#include <cmath>
inline __host__ __device__ float2 operator-(const float2 a, const float2 b) {
  return make_float2(a.x - b.x, a.y - b.y);
}
inline __host__ __device__ double2 operator-(const double2 a, const double2 b) {
  return make_double2(a.x - b.x, a.y - b.y);
}
#endif
