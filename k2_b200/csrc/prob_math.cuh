// Mantissa/exponent arithmetic for log-semiring recursions carried out in the
// probability domain: a value is m * 2^e with m in [1,2) (or m == 0), so sums over
// arcs need only multiplies, adds and integer operations on the exponent.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace k2b {

constexpr int32_t kZeroExp = -(1 << 30);

__device__ __forceinline__ void ExpToMantExp(float score, double *f, int32_t *k) {
  if (score == -INFINITY) {
    *f = 0.0;
    *k = kZeroExp;
    return;
  }
  // exp(x) = 2^(x / ln 2): split x / ln 2 into integer and fraction in double
  double y = (double)score * 1.4426950408889634074;  // log2(e)
  double fl = floor(y);
  double frac = y - fl;                 // [0,1)
  *f = exp2(frac);                      // [1,2)
  double kk = fmax(fmin(fl, 268435456.0), -268435456.0);
  *k = (int32_t)kk;
}

// 2^d for d <= 0 (0 when the result would be subnormal).
__device__ __forceinline__ double Pow2NonPos(int32_t d) {
  return d < -1000 ? 0.0 : __longlong_as_double((long long)(1023 + d) << 52);
}

// x * 2^d for d <= 0 and x == 0 or 1 <= x < 2^20: an integer add on the exponent field.
__device__ __forceinline__ double ScaleDown(double x, int32_t d) {
  const int32_t hi = __double2hiint(x) + (d << 20);
  return (d < -1000 || x == 0.0) ? 0.0 : __hiloint2double(hi, __double2loint(x));
}

// One state's score in shared memory: mantissa and exponent side by side.
struct __align__(16) ProbState {
  double m;
  int32_t e;
  int32_t pad;
};

// Normalise s >= 0 (a sum of a few numbers in [1,4) scaled by powers of two <= 1)
// to m in [1,2) and add its exponent to *e.
__device__ __forceinline__ double Renorm(double s, int32_t *e) {
  if (s == 0.0) {
    *e = kZeroExp;
    return 0.0;
  }
  const int32_t hi = __double2hiint(s);
  const int32_t ex = (hi >> 20) - 1023;  // s > 0 and normal
  *e += ex;
  return __hiloint2double(hi - (ex << 20), __double2loint(s));
}

}  // namespace k2b
