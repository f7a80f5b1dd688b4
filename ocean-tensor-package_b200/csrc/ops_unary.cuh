// Unary element operations, one functor per table name.
//
// Scalar semantics are those of solid/include/solid/core/generic/unary_ops.h:203-673
// as instantiated for the CPU by solid/src/core/cpu/template_unary.c (the parity
// oracle): bool and integers at lines 212-277, real floating point 279-325,
// complex 327-621.  Integer transcendental functions evaluate in double and cast
// back; half computes in float; complex sqrt is Friedland's Algorithm 312 (the
// CPU choice, template_unary.c:109), not the polar form of the reference's GPU file.
//
// Each functor has   template <class T> using out = ...;   (result element type)
//                    template <class T> static out<T> f(T x);
#pragma once
#include "mathfn.cuh"

namespace sd {

// ----- helpers --------------------------------------------------------------
// integer op evaluated in double and cast back with the oracle's cast
#define SD_INT_VIA_DOUBLE(T, EXPR_ON_D) float_to_int<T, double>(EXPR_ON_D)

template <class T> struct same_out { using type = T; };

// Generic real-function functor: ints through double, reals through the work
// type, complex through a component formula supplied by CPLX(xr, xi, &yr, &yi).
#define SD_UNARY_REALFN(NAME, FN, ...)                                           \
   struct u_##NAME {                                                                   \
      template <class T> using out = T;                                                \
      template <class T> static SD_D T f(T x)                                          \
      {                                                                                \
         if constexpr (is_int<T>) {                                                    \
            return float_to_int<T, double>(FN<double>((double)x));                     \
         } else if constexpr (is_real<T>) {                                            \
            using W = work_t<T>;                                                       \
            return from_work<T>(FN<W>(to_work<T>(x)));                                 \
         } else {                                                                      \
            using E = elem_t<T>; using W = work_t<E>;                                  \
            W xr = ew<E>(x.re), xi = ew<E>(x.im), yr, yi;                              \
            __VA_ARGS__                                                                 \
            T y; y.re = few<E>(yr); y.im = few<E>(yi); return y;                       \
         }                                                                             \
      }                                                                                \
   };

SD_UNARY_REALFN(sin, m_sin,   { yr = m_sin<W>(xr) * m_cosh<W>(xi); yi = m_cos<W>(xr) * m_sinh<W>(xi); })
SD_UNARY_REALFN(cos, m_cos,   { yr = m_cos<W>(xr) * m_cosh<W>(xi); yi = m_sin<W>(xr) * m_sinh<W>(xi) * -1; })
SD_UNARY_REALFN(tan, m_tan,   { W a = 2 * xr, b = 2 * xi; W r = m_cos<W>(a) + m_cosh<W>(b);
                                yr = m_sin<W>(a) / r; yi = m_sinh<W>(b) / r; })
SD_UNARY_REALFN(sinh, m_sinh, { yr = m_sinh<W>(xr) * m_cos<W>(xi); yi = m_cosh<W>(xr) * m_sin<W>(xi); })
SD_UNARY_REALFN(cosh, m_cosh, { yr = m_cosh<W>(xr) * m_cos<W>(xi); yi = m_sinh<W>(xr) * m_sin<W>(xi); })
SD_UNARY_REALFN(tanh, m_tanh, { W a = 2 * xr, b = 2 * xi; W r = (W)(1. / (double)(m_cosh<W>(a) + m_cos<W>(b)));
                                yr = m_sinh<W>(a) * r; yi = m_sin<W>(b) * r; })
SD_UNARY_REALFN(arcsin, m_asin, {
      W v1 = 1 - (xr * xr) + (xi * xi); W v2 = -2 * xr * xi;
      W gamma = m_sqrt<W>(m_hypot<W>(v1, v2)); W theta = m_atan2<W>(v2, v1) / 2;
      v1 = -xi + gamma * m_cos<W>(theta); v2 = xr + gamma * m_sin<W>(theta);
      yr = m_atan2<W>(v2, v1); yi = m_log<W>(v1 * v1 + v2 * v2) / -2; })
SD_UNARY_REALFN(arccos, m_acos, {
      W v1 = 1 - (xr * xr) + (xi * xi); W v2 = -2 * xr * xi;
      W gamma = m_sqrt<W>(m_hypot<W>(v1, v2)); W theta = m_atan2<W>(v2, v1) / 2;
      v1 = xr - gamma * m_sin<W>(theta); v2 = xi + gamma * m_cos<W>(theta);
      yr = m_atan2<W>(v2, v1); yi = m_log<W>(v1 * v1 + v2 * v2) / -2; })
SD_UNARY_REALFN(arctan, m_atan, {
      W v1 = xr * xr; W v2 = xi * xi;
      yr = m_atan2<W>(2 * xr, 1 - v1 - v2) / 2;
      v2 = 1 + xi;
      yi = m_log<W>(1 - 4 * xi / (v2 * v2 + v1)) / -4; })
SD_UNARY_REALFN(arcsinh, m_asinh, {
      W v1 = 1 + (xr * xr) - (xi * xi); W v2 = 2 * xr * xi;
      W gamma = m_sqrt<W>(m_hypot<W>(v1, v2)); W theta = m_atan2<W>(v2, v1) / 2;
      v1 = xr + gamma * m_cos<W>(theta); v2 = xi + gamma * m_sin<W>(theta);
      yr = m_log<W>(v1 * v1 + v2 * v2) / 2; yi = m_atan2<W>(v2, v1); })
SD_UNARY_REALFN(arccosh, m_acosh, {
      W v1 = (xr * xr) - (xi * xi) - 1; W v2 = 2 * xr * xi;
      W gamma = m_sqrt<W>(m_hypot<W>(v1, v2)); W theta = m_atan2<W>(v2, v1) / 2;
      v1 = xr + gamma * m_cos<W>(theta); v2 = xi + gamma * m_sin<W>(theta);
      yr = m_log<W>(v1 * v1 + v2 * v2) / 2; yi = m_atan2<W>(v2, v1); })
// The oracle's complex arctanh stores both results into the imaginary part and
// never writes the real part (unary_ops.h:472-474); what follows is the formula
// that code states in its comment, so complex arctanh is outside bit parity.
SD_UNARY_REALFN(arctanh, m_atanh, {
      W v1 = xr * xr; W v2 = xi * xi;
      yi = m_atan2<W>(2 * xi, 1 - v1 - v2) / 2;
      v1 = 1 - xr;
      yr = m_log<W>(1 + 4 * xr / (v1 * v1 + v2)) / 4; })
SD_UNARY_REALFN(cbrt, m_cbrt, {
      W scale = (xr * xr) + (xi * xi);
      if (scale > 0) { scale = m_pow<W>(scale, (W)(1. / 6)); W angle = m_atan2<W>(xi, xr) / 3;
                       yr = scale * m_cos<W>(angle); yi = scale * m_sin<W>(angle); }
      else { yr = 0; yi = 0; } })
SD_UNARY_REALFN(exp, m_exp,     { W s = m_exp<W>(xr); yr = s * m_cos<W>(xi); yi = s * m_sin<W>(xi); })
SD_UNARY_REALFN(exp2, m_exp2,   { W b = xi * m_ln2<W>(); W s = m_exp2<W>(xr); yr = s * m_cos<W>(b); yi = s * m_sin<W>(b); })
SD_UNARY_REALFN(exp10, m_exp10, { W b = xi * m_ln10<W>(); W s = m_exp10<W>(xr); yr = s * m_cos<W>(b); yi = s * m_sin<W>(b); })
SD_UNARY_REALFN(expm1, m_expm1, { W s = m_exp<W>(xr); yr = s * m_cos<W>(xi) - 1; yi = s * m_sin<W>(xi); })
#undef SD_UNARY_REALFN

// sqrt / log family: signed integers return 0 for arguments outside the domain
// (unary_ops.h:250-259); log1p tests x <= -1.
#define SD_UNARY_DOMAINFN(NAME, FN, LIMIT_EXPR, ...)                             \
   struct u_##NAME {                                                                   \
      template <class T> using out = T;                                                \
      template <class T> static SD_D T f(T x)                                          \
      {                                                                                \
         if constexpr (is_sint<T>) {                                                   \
            return (LIMIT_EXPR) ? (T)0 : float_to_int<T, double>(FN<double>((double)x)); \
         } else if constexpr (is_uint<T>) {                                            \
            return float_to_int<T, double>(FN<double>((double)x));                     \
         } else if constexpr (is_real<T>) {                                            \
            using W = work_t<T>;                                                       \
            return from_work<T>(FN<W>(to_work<T>(x)));                                 \
         } else {                                                                      \
            using E = elem_t<T>; using W = work_t<E>;                                  \
            W xr = ew<E>(x.re), xi = ew<E>(x.im), yr, yi;                              \
            T y;                                                                       \
            __VA_ARGS__                                                                 \
            return y;                                                                  \
         }                                                                             \
      }                                                                                \
   };

#define SD_CPLX_STORE  y.re = few<E>(yr); y.im = few<E>(yi);
SD_UNARY_DOMAINFN(log, m_log, x <= 0,
   { W s = xr * xr + xi * xi; yr = (W)((double)m_log<W>(s) * 0.5); yi = m_atan2<W>(xi, xr); SD_CPLX_STORE })
SD_UNARY_DOMAINFN(log2, m_log2, x <= 0,
   { W s = xr * xr + xi * xi; yr = (W)((double)m_log2<W>(s) * 0.5); yi = m_atan2<W>(xi, xr) / m_ln2<W>(); SD_CPLX_STORE })
SD_UNARY_DOMAINFN(log10, m_log10, x <= 0,
   { W s = xr * xr + xi * xi; yr = (W)((double)m_log10<W>(s) * 0.5); yi = m_atan2<W>(xi, xr) / m_ln10<W>(); SD_CPLX_STORE })
SD_UNARY_DOMAINFN(log1p, m_log1p, (double)x <= -1,
   { xr = xr + 1; W s = xr * xr + xi * xi; yr = (W)((double)m_log<W>(s) * 0.5); yi = m_atan2<W>(xi, xr); SD_CPLX_STORE })
// Complex square root: Algorithm 312 (unary_ops.h:493-524)
SD_UNARY_DOMAINFN(sqrt, m_sqrt, x <= 0,
   {  W v = m_hypot<W>(xr, xi);
      if (!(v > 0)) { y.re = few<E>(v); y.im = y.re; }
      else if (m_isinf<W>(xi)) {
         if constexpr (is_half<E>) y.re.v = 0xFC00; else y.re = m_inf<W>();
         y.im = x.im; }
      else if (m_isinf<W>(xr)) {
         y.re = few<E>((xr > 0) ? xr : (W)0);
         y.im = few<E>(m_copysign<W>((xr < 0) ? xr : (W)0, xi)); }
      else if (xr >= 0) {
         v = m_sqrt<W>((W)((double)(xr + v) * 0.5));
         y.re = few<E>(v); y.im = few<E>(xi / (2 * v)); }
      else {
         v = m_sqrt<W>((W)((double)(-xr + v) * 0.5));
         y.re = few<E>(((xi >= 0) ? xi : -xi) / (2 * v));
         y.im = few<E>(m_copysign<W>(v, xi)); }
      (void)yr; (void)yi; })
#undef SD_UNARY_DOMAINFN
#undef SD_CPLX_STORE

struct u_negative {
   template <class T> using out = T;
   template <class T> static SD_D T f(T x)
   {
      if constexpr (is_bool<T>) { Bool r; r.v = x.v ^ 0x01; return r; }          // alias of logical_not
      else if constexpr (is_int<T>) return (T)(-1 * x);
      else if constexpr (is_real<T>) return from_work<T>(-1 * to_work<T>(x));
      else { using E = elem_t<T>; T y; y.re = few<E>(-1 * ew<E>(x.re)); y.im = few<E>(-1 * ew<E>(x.im)); return y; }
   }
};
struct u_conj {
   template <class T> using out = T;
   template <class T> static SD_D T f(T x)
   {  using E = elem_t<T>; T y; y.re = x.re; y.im = few<E>(-1 * ew<E>(x.im)); return y; }
};
struct u_reciprocal {
   template <class T> using out = T;
   template <class T> static SD_D T f(T x)
   {
      if constexpr (is_int<T>) return (x == 0) ? (T)0 : (T)(1 / x);
      else if constexpr (is_real<T>) { using W = work_t<T>; return from_work<T>((W)(1. / (double)to_work<T>(x))); }
      else {
         using E = elem_t<T>; using W = work_t<E>;
         W xr = ew<E>(x.re), xi = ew<E>(x.im);
         W scale = (W)(1. / (double)((xr * xr) + (xi * xi)));
         T y; y.re = few<E>(xr * scale); y.im = few<E>(xi * scale * -1); return y;
      }
   }
};
struct u_bitwise_not {
   template <class T> using out = T;
   template <class T> static SD_D T f(T x)
   {  if constexpr (is_bool<T>) { Bool r; r.v = x.v ^ 0x01; return r; } else return (T)(~x); }
};
using u_logical_not = u_bitwise_not;

struct u_square {
   template <class T> using out = T;
   template <class T> static SD_D T f(T x)
   {
      if constexpr (is_int<T>) return (T)(x * x);
      else if constexpr (is_real<T>) { auto w = to_work<T>(x); return from_work<T>(w * w); }
      else { using E = elem_t<T>; using W = work_t<E>; W xr = ew<E>(x.re), xi = ew<E>(x.im);
             T y; y.re = few<E>(xr * xr - xi * xi); y.im = few<E>(2 * xr * xi); return y; }
   }
};
struct u_fabs {
   template <class T> using out = T;
   template <class T> static SD_D T f(T x)
   {
      if constexpr (is_bool<T> || is_uint<T>) return x;
      else if constexpr (is_sint<T>) return (T)(((x >= 0) - (x < 0)) * x);
      else if constexpr (is_real<T>) { using W = work_t<T>; return from_work<T>(m_fabs<W>(to_work<T>(x))); }
      else { using E = elem_t<T>; using W = work_t<E>;
             T y; y.re = few<E>(m_hypot<W>(ew<E>(x.re), ew<E>(x.im)));
             if constexpr (is_half<E>) y.im.v = 0; else y.im = 0;
             return y; }
   }
};
struct u_absolute {                       // complex -> real component type
   template <class T> using out = elem_t<T>;
   template <class T> static SD_D elem_t<T> f(T x)
   {
      if constexpr (is_cplx<T>) { using E = elem_t<T>; using W = work_t<E>;
                                  return few<E>(m_hypot<W>(ew<E>(x.re), ew<E>(x.im))); }
      else return u_fabs::f<T>(x);
   }
};
struct u_sign {
   template <class T> using out = T;
   template <class T> static SD_D T f(T x)
   {
      if constexpr (is_bool<T>) return x;
      else if constexpr (is_uint<T>) return (T)(x > 0);
      else if constexpr (is_sint<T>) return (T)((x > 0) - (x < 0));
      else if constexpr (is_real<T>) { using W = work_t<T>; W w = to_work<T>(x);
                                       return m_isnan<W>(w) ? x : from_work<T>((W)((w > 0) - (w < 0))); }
      else {
         using E = elem_t<T>; using W = work_t<E>; W xr = ew<E>(x.re), xi = ew<E>(x.im);
         T y;
         if (m_isnan<W>(xr) || m_isnan<W>(xi)) y.re = few<E>(xr + xi);
         else y.re = few<E>((W)(((xr > 0) - (xr < 0)) + (xr == 0) * ((xi > 0) - (xi < 0))));
         if constexpr (is_half<E>) y.im.v = 0; else y.im = 0;
         return y;
      }
   }
};

#define SD_UNARY_ROUNDFN(NAME, FN)                                                     \
   struct u_##NAME {                                                                   \
      template <class T> using out = T;                                                \
      template <class T> static SD_D T f(T x)                                          \
      {                                                                                \
         if constexpr (is_real<T>) { using W = work_t<T>; return from_work<T>(FN<W>(to_work<T>(x))); } \
         else { using E = elem_t<T>; using W = work_t<E>;                              \
                T y; y.re = few<E>(FN<W>(ew<E>(x.re))); y.im = few<E>(FN<W>(ew<E>(x.im))); return y; } \
      }                                                                                \
   };
SD_UNARY_ROUNDFN(ceil, m_ceil) SD_UNARY_ROUNDFN(floor, m_floor)
SD_UNARY_ROUNDFN(trunc, m_trunc) SD_UNARY_ROUNDFN(round, m_round)
#undef SD_UNARY_ROUNDFN

// Classification: bool output.  Complex isnan tests isinf on the imaginary part,
// as the oracle does (unary_ops.h:660).
#define SD_UNARY_QUERY(NAME, INTVAL, REAL_EXPR, CPLX_EXPR)                             \
   struct u_##NAME {                                                                   \
      template <class T> using out = Bool;                                             \
      template <class T> static SD_D Bool f(T x)                                       \
      {                                                                                \
         Bool r;                                                                       \
         if constexpr (is_bool<T> || is_int<T>) { (void)x; r.v = INTVAL; }             \
         else if constexpr (is_real<T>) { using W = work_t<T>; W w = to_work<T>(x); r.v = (REAL_EXPR) ? 1 : 0; } \
         else { using E = elem_t<T>; using W = work_t<E>; W xr = ew<E>(x.re), xi = ew<E>(x.im); \
                (void)xr; (void)xi; r.v = (CPLX_EXPR) ? 1 : 0; }                       \
         return r;                                                                     \
      }                                                                                \
   };
SD_UNARY_QUERY(isinf,    0, m_isinf<W>(w),            m_isinf<W>(xr) || m_isinf<W>(xi))
SD_UNARY_QUERY(isnan,    0, m_isnan<W>(w),            m_isnan<W>(xr) || m_isinf<W>(xi))
SD_UNARY_QUERY(isfinite, 1, m_isfinite<W>(w),         m_isfinite<W>(xr) && m_isfinite<W>(xi))
SD_UNARY_QUERY(isposinf, 0, (w > 0) && m_isinf<W>(w), false)
SD_UNARY_QUERY(isneginf, 0, (w < 0) && m_isinf<W>(w), false)
#undef SD_UNARY_QUERY

} // namespace sd
