// Math-library mapping per work type, mirroring the CPU mapping of the
// reference (solid/include/solid/core/cpu/unary_ops_cpu.h:24-156) so that the
// same formula is evaluated with the same precision:
//   - float functions are the single-precision ones, double the double ones;
//   - the DOUBLE pow is single precision there (SOLID_DOUBLE_POW = powf, line 87),
//     so double `power`, complex-double cbrt and norm(p) on doubles are only
//     float-accurate on the oracle and therefore here;
//   - exp10(x) is exp(ln10 * x) with ln10 rounded to the work type (lines 48,93);
//   - FLOAT fmod calls the double fmod, which is exact, so fmodf is equivalent.
#pragma once
#include "dtypes.cuh"

namespace sd {

template <class W> struct mf;

#define SD_MF1(NAME, FN32, FN64)                                   \
   template <class W> SD_D W m_##NAME(W x)                         \
   {  if constexpr (std::is_same<W, float>::value) return FN32(x); \
      else return FN64(x); }

SD_MF1(sin, sinf, ::sin)       SD_MF1(cos, cosf, ::cos)       SD_MF1(tan, tanf, ::tan)
SD_MF1(sinh, sinhf, ::sinh)    SD_MF1(cosh, coshf, ::cosh)    SD_MF1(tanh, tanhf, ::tanh)
SD_MF1(asin, asinf, ::asin)    SD_MF1(acos, acosf, ::acos)    SD_MF1(atan, atanf, ::atan)
SD_MF1(asinh, asinhf, ::asinh) SD_MF1(acosh, acoshf, ::acosh) SD_MF1(atanh, atanhf, ::atanh)
SD_MF1(sqrt, sqrtf, ::sqrt)    SD_MF1(cbrt, cbrtf, ::cbrt)
SD_MF1(exp, expf, ::exp)       SD_MF1(exp2, exp2f, ::exp2)    SD_MF1(expm1, expm1f, ::expm1)
SD_MF1(log, logf, ::log)       SD_MF1(log2, log2f, ::log2)    SD_MF1(log10, log10f, ::log10)
SD_MF1(log1p, log1pf, ::log1p) SD_MF1(fabs, fabsf, ::fabs)
SD_MF1(ceil, ceilf, ::ceil)    SD_MF1(floor, floorf, ::floor) SD_MF1(trunc, truncf, ::trunc)
SD_MF1(round, roundf, ::round)
#undef SD_MF1

template <class W> SD_D W m_ln2()  { return (W)0.69314718055994529; }
template <class W> SD_D W m_ln10() { return (W)2.3025850929940459; }
template <class W> SD_D W m_inf()  { return (W)(1. / 0.); }
template <class W> SD_D W m_exp10(W x) { return m_exp<W>(m_ln10<W>() * x); }

template <class W> SD_D W m_atan2(W y, W x)
{  if constexpr (std::is_same<W, float>::value) return atan2f(y, x); else return ::atan2(y, x); }
// Single precision hypot goes through double (products exact, one rounding in the
// sum, one in the root, one in the narrowing), which is how current glibc
// evaluates hypotf; the double version is the CUDA library function.
template <class W> SD_D W m_hypot(W x, W y)
{
   if constexpr (std::is_same<W, float>::value) {
      if (fabsf(x) == (float)(1. / 0.) || fabsf(y) == (float)(1. / 0.)) return (float)(1. / 0.);
      return (float)::sqrt((double)x * (double)x + (double)y * (double)y);
   } else return ::hypot(x, y);
}
template <class W> SD_D W m_fmod(W x, W y)
{  if constexpr (std::is_same<W, float>::value) return fmodf(x, y); else return ::fmod(x, y); }
template <class W> SD_D W m_copysign(W x, W y)
{  if constexpr (std::is_same<W, float>::value) return copysignf(x, y); else return ::copysign(x, y); }
// pow in the oracle is ALWAYS powf
template <class W> SD_D W m_pow(W x, W y) { return (W)powf((float)x, (float)y); }

template <class W> SD_D bool m_isnan(W x)    { return x != x; }
template <class W> SD_D bool m_isinf(W x)    { return m_fabs<W>(x) == m_inf<W>(); }
template <class W> SD_D bool m_isfinite(W x) { return m_fabs<W>(x) < m_inf<W>(); }

} // namespace sd
