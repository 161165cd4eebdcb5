// Sums of the mixed (float2, double2-derived) pairs that the toolkit's CUB forms when the
// reference reduces float2 gradients into its double-precision pair type (garden.cu:432-435,
// builder.h:226).  Component-wise double additions, like the reference's own operators.
#pragma once

inline __host__ __device__ mydouble2 operator+(const mydouble2 a, const float2 b) {
  return mydouble2(make_double2(a.x + b.x, a.y + b.y));
}
inline __host__ __device__ mydouble2 operator+(const float2 a, const mydouble2 b) {
  return mydouble2(make_double2(a.x + b.x, a.y + b.y));
}
inline __host__ __device__ mydouble2 operator+(const mydouble2 a, const mydouble2 b) {
  return mydouble2(make_double2(a.x + b.x, a.y + b.y));
}
