// expf with the results of the host C library, for device code.
//
// The reference's softmax and SiLU call f32::exp (crates/aot-kernels/src/ops.rs:
// 98-120), which resolves to the platform libm. glibc's expf is the published
// table-driven algorithm exp(x) = 2^(k/32) * 2^(r/32), k = round(x*32/ln2), with
// a degree-3 polynomial for 2^(r/32) evaluated in double precision and one final
// rounding to f32. Restated here in fp64 device arithmetic, with the reduction
// r = fma(32/ln2, x, -k) that the FMA build of the library performs, it returns
// the same bits as the library on every one of the 2^32 inputs (checked
// exhaustively on the CPU by tests/test_expf.py through a host copy of this
// function).
//
// The table holds bits(2^(i/32)) - (i << 47) for i in 0..31, each 2^(i/32)
// correctly rounded to double (generated with 80-digit decimal arithmetic; the
// test recomputes it).
#pragma once
#include "blockmath.cuh"

namespace aot {

#if defined(__CUDACC__)
#define AOT_EXP_TAB_QUAL __device__ __constant__
#else
#define AOT_EXP_TAB_QUAL static const
#endif

#define AOT_EXP2_TABLE_VALUES                                                                          \
  0x3ff0000000000000ULL, 0x3fefd9b0d3158574ULL, 0x3fefb5586cf9890fULL, 0x3fef9301d0125b51ULL,          \
      0x3fef72b83c7d517bULL, 0x3fef54873168b9aaULL, 0x3fef387a6e756238ULL, 0x3fef1e9df51fdee1ULL,      \
      0x3fef06fe0a31b715ULL, 0x3feef1a7373aa9cbULL, 0x3feedea64c123422ULL, 0x3feece086061892dULL,      \
      0x3feebfdad5362a27ULL, 0x3feeb42b569d4f82ULL, 0x3feeab07dd485429ULL, 0x3feea47eb03a5585ULL,      \
      0x3feea09e667f3bcdULL, 0x3fee9f75e8ec5f74ULL, 0x3feea11473eb0187ULL, 0x3feea589994cce13ULL,      \
      0x3feeace5422aa0dbULL, 0x3feeb737b0cdc5e5ULL, 0x3feec49182a3f090ULL, 0x3feed503b23e255dULL,      \
      0x3feee89f995ad3adULL, 0x3feeff76f2fb5e47ULL, 0x3fef199bdd85529cULL, 0x3fef3720dcef9069ULL,      \
      0x3fef5818dcfba487ULL, 0x3fef7c97337b9b5fULL, 0x3fefa4afa2a490daULL, 0x3fefd0765b6e4540ULL

#if defined(__CUDACC__)
static __device__ __constant__ uint64_t c_exp2_tab[32] = {AOT_EXP2_TABLE_VALUES};
#endif
static const uint64_t h_exp2_tab[32] = {AOT_EXP2_TABLE_VALUES};

AOT_HD double dfma(double a, double b, double c) {
#if AOT_DEVICE_CODE
  return __fma_rn(a, b, c);
#else
  return fma(a, b, c);
#endif
}
AOT_HD double dmul(double a, double b) {
#if AOT_DEVICE_CODE
  return __dmul_rn(a, b);
#else
  volatile double r = a * b;
  return r;
#endif
}
AOT_HD double dadd(double a, double b) {
#if AOT_DEVICE_CODE
  return __dadd_rn(a, b);
#else
  volatile double r = a + b;
  return r;
#endif
}
AOT_HD uint64_t d2u(double d) {
#if AOT_DEVICE_CODE
  return (uint64_t)__double_as_longlong(d);
#else
  uint64_t u;
  memcpy(&u, &d, 8);
  return u;
#endif
}
AOT_HD double u2d(uint64_t u) {
#if AOT_DEVICE_CODE
  return __longlong_as_double((long long)u);
#else
  double d;
  memcpy(&d, &u, 8);
  return d;
#endif
}

AOT_HD float expf_exact(float x) {
  const double kInvLn2N = 0x1.71547652b82fep+0 * 32.0;
  const double kShift = 0x1.8p+52;
  const double kC0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
  const double kC1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
  const double kC2 = 0x1.62e42ff0c52d6p-1 / 32.0;
  uint32_t ux = f2u(x);
  uint32_t abstop = (ux >> 20) & 0x7ffu;
  if (abstop >= 0x42bu) {  // |x| >= 88 or NaN
    if (ux == 0xff800000u) return 0.0f;
    if (abstop >= 0x7f8u) return fadd(x, x);
    if (x > 0x1.62e42ep6f) return u2f(0x7f800000u);  // overflow
    if (x < -0x1.9fe368p6f) return 0.0f;             // underflow
  }
  double xd = (double)x;
  double z = dmul(kInvLn2N, xd);
  double kd = dadd(z, kShift);
  uint64_t ki = d2u(kd);
  kd = dadd(kd, -kShift);
  double r = dfma(kInvLn2N, xd, -kd);
#if AOT_DEVICE_CODE
  uint64_t t = c_exp2_tab[ki & 31u];
#else
  uint64_t t = h_exp2_tab[ki & 31u];
#endif
  t += ki << 47;
  double s = u2d(t);
  double p = dfma(kC0, r, kC1);
  double r2 = dmul(r, r);
  double y = dfma(kC2, r, 1.0);
  y = dfma(p, r2, y);
  y = dmul(y, s);
  return (float)y;
}

}  // namespace aot
