// Binary element operations, one functor per table name.
//
// Scalar semantics: solid/include/solid/core/generic/binary_ops.h:112-520, with the
// per-type aliases of solid/src/core/cpu/template_binary.c (bool min/max are
// and/or, unsigned divide/floor_divide are true_divide, unsigned fmod is mod,
// integer fmin/fmax are min/max).  Integer arithmetic goes through C integer
// promotion exactly as the C macros do; floating point runs in the work type
// with one rounding per operation (the library is built without FMA contraction).
//
// Each functor has   template <class T> using in2 = ...;  type of the second operand
//                    template <class T> using out = ...;  type of the result
//                    template <class T> static out<T> f(T x, in2<T> y);
#pragma once
#include "mathfn.cuh"

namespace sd {

#define SD_BIN_SAME  template <class T> using in2 = T; template <class T> using out = T;

// ---- helpers on the three arithmetic kinds ---------------------------------
template <class T> SD_D Bool mkbool(bool b) { Bool r; r.v = b ? 1 : 0; return r; }

#define SD_BIN_ARITH(NAME, BOOL_EXPR, INT_EXPR, REAL_EXPR, ...)                        \
   struct b_##NAME {                                                                   \
      SD_BIN_SAME                                                                      \
      template <class T> static SD_D T f(T x, T y)                                     \
      {                                                                                \
         if constexpr (is_bool<T>) { Bool r; uint8_t a = x.v, b = y.v; (void)a; (void)b; r.v = (uint8_t)(BOOL_EXPR); return r; } \
         else if constexpr (is_int<T>) { T a = x, b = y; (void)a; (void)b; return (T)(INT_EXPR); } \
         else if constexpr (is_real<T>) { using W = work_t<T>; W a = to_work<T>(x), b = to_work<T>(y); \
                                          (void)a; (void)b; return from_work<T>((W)(REAL_EXPR)); } \
         else { using E = elem_t<T>; using W = work_t<E>;                              \
                W xr = ew<E>(x.re), xi = ew<E>(x.im), yr = ew<E>(y.re), yi = ew<E>(y.im), zr, zi; \
                __VA_ARGS__                                                            \
                T z; z.re = few<E>(zr); z.im = few<E>(zi); return z; }                 \
      }                                                                                \
   };

SD_BIN_ARITH(add,      a | b,   a + b, a + b, { zr = xr + yr; zi = xi + yi; })
SD_BIN_ARITH(subtract, a & ~b,  a - b, a - b, { zr = xr - yr; zi = xi - yi; })
SD_BIN_ARITH(multiply, a & b,   a * b, a * b, { zr = xr * yr - xi * yi; zi = xr * yi + yr * xi; })
SD_BIN_ARITH(true_divide, a & b, (b == 0) ? 0 : (a / b), a / b,
             { W r = yr * yr + yi * yi; zr = (xr * yr + xi * yi) / r; zi = (xi * yr - xr * yi) / r; })
#undef SD_BIN_ARITH

// Signed floor division by the branch-free correction of binary_ops.h:154-203.
// `divide` evaluates the whole expression in the promoted type; `floor_divide`
// stores the corrected numerator back into the element type first (lines 196-197),
// which wraps for the extreme values of the 8- and 16-bit types.
template <class T, bool STORE_BACK> SD_D T int_floor_div(T x, T y)
{
   if (y == 0) return 0;
   auto xx = +x; auto yy = +y;                       // integer promotion
   auto num = xx - ((xx * yy) < 0) * (yy + ((yy < 0) - (yy > 0)));
   if constexpr (STORE_BACK) return (T)((T)num / yy);
   else                      return (T)(num / yy);
}

struct b_divide {
   SD_BIN_SAME
   template <class T> static SD_D T f(T x, T y)
   {  if constexpr (is_sint<T>) return int_floor_div<T, false>(x, y); else return b_true_divide::f<T>(x, y); }
};
struct b_floor_divide {
   SD_BIN_SAME
   template <class T> static SD_D T f(T x, T y)
   {
      if constexpr (is_sint<T>) return int_floor_div<T, true>(x, y);
      else if constexpr (is_real<T>) { using W = work_t<T>; W a = to_work<T>(x), b = to_work<T>(y);
                                       return from_work<T>(m_floor<W>(a / b)); }
      else return b_true_divide::f<T>(x, y);
   }
};
struct b_mod {
   SD_BIN_SAME
   template <class T> static SD_D T f(T x, T y)
   {
      if constexpr (is_bool<T>) { Bool r; r.v = 0; return r; }
      else if constexpr (is_uint<T>) return (y == 0) ? (T)0 : (T)(x % y);
      else if constexpr (is_sint<T>) {
         if (y == 0) return 0;
         auto xx = +x; auto yy = +y; auto zz = xx % yy;
         return (T)(zz + ((xx * yy < 0) && (zz != 0)) * yy);
      } else { using W = work_t<T>; W a = to_work<T>(x), b = to_work<T>(y);
               W z = m_floor<W>(a / b); return from_work<T>(a - z * b); }
   }
};
struct b_fmod {
   SD_BIN_SAME
   template <class T> static SD_D T f(T x, T y)
   {
      if constexpr (is_bool<T>) { Bool r; r.v = 0; return r; }
      else if constexpr (is_uint<T>) return (y == 0) ? (T)0 : (T)(x % y);       // alias of mod
      else if constexpr (is_sint<T>) return (y == 0) ? (T)0 : (T)(x % y);
      else { using W = work_t<T>; return from_work<T>(m_fmod<W>(to_work<T>(x), to_work<T>(y))); }
   }
};

#define SD_BIN_BITOP(NAME, OP)                                                         \
   struct b_##NAME {                                                                   \
      SD_BIN_SAME                                                                      \
      template <class T> static SD_D T f(T x, T y)                                     \
      {  if constexpr (is_bool<T>) { Bool r; r.v = (uint8_t)(x.v OP y.v); return r; }  \
         else return (T)(x OP y); }                                                    \
   };
SD_BIN_BITOP(bitwise_and, &) SD_BIN_BITOP(bitwise_or, |) SD_BIN_BITOP(bitwise_xor, ^)
#undef SD_BIN_BITOP
using b_logical_and = b_bitwise_and;
using b_logical_or  = b_bitwise_or;
using b_logical_xor = b_bitwise_xor;

// Comparisons: complex orders lexicographically on (real, imag); note that the
// complex "le"/"ge" decide on the real parts with a strict test (binary_ops.h:425-444).
#define SD_BIN_COMPARE(NAME, OP, CPLX_EXPR)                                            \
   struct b_##NAME {                                                                   \
      template <class T> using in2 = T; template <class T> using out = Bool;           \
      template <class T> static SD_D Bool f(T x, T y)                                  \
      {                                                                                \
         Bool r;                                                                       \
         if constexpr (is_bool<T>) r.v = (x.v OP y.v) ? 1 : 0;                         \
         else if constexpr (is_int<T>) r.v = (x OP y) ? 1 : 0;                         \
         else if constexpr (is_real<T>) r.v = (to_work<T>(x) OP to_work<T>(y)) ? 1 : 0; \
         else { using E = elem_t<T>; using W = work_t<E>;                              \
                W xr = ew<E>(x.re), xi = ew<E>(x.im), yr = ew<E>(y.re), yi = ew<E>(y.im); \
                r.v = (CPLX_EXPR) ? 1 : 0; }                                           \
         return r;                                                                     \
      }                                                                                \
   };
SD_BIN_COMPARE(lt, <,  (xr != yr) ? (xr < yr) : (xi <  yi))
SD_BIN_COMPARE(le, <=, (xr != yr) ? (xr < yr) : (xi <= yi))
SD_BIN_COMPARE(ge, >=, (xr != yr) ? (xr > yr) : (xi >= yi))
SD_BIN_COMPARE(gt, >,  (xr != yr) ? (xr > yr) : (xi >  yi))
SD_BIN_COMPARE(eq, ==, (xr == yr) && (xi == yi))
SD_BIN_COMPARE(ne, !=, (xr != yr) || (xi != yi))
#undef SD_BIN_COMPARE

// min / max propagate a NaN of the SECOND operand; fmin / fmax prefer the
// non-NaN operand (binary_ops.h:316-342, complex 462-520).
#define SD_BIN_MINMAX(NAME, BOOLOP, INT_CMP, REAL_COND, CPLX_COND)                     \
   struct b_##NAME {                                                                   \
      SD_BIN_SAME                                                                      \
      template <class T> static SD_D T f(T x, T y)                                     \
      {                                                                                \
         if constexpr (is_bool<T>) { Bool r; r.v = (uint8_t)(x.v BOOLOP y.v); return r; } \
         else if constexpr (is_int<T>) return (x INT_CMP y) ? x : y;                   \
         else if constexpr (is_real<T>) { using W = work_t<T>; W a = to_work<T>(x), b = to_work<T>(y); \
                                          if (REAL_COND) a = b; return from_work<T>(a); } \
         else { using E = elem_t<T>; using W = work_t<E>;                              \
                W xr = ew<E>(x.re), xi = ew<E>(x.im), yr = ew<E>(y.re), yi = ew<E>(y.im); \
                T z;                                                                   \
                if (CPLX_COND) { z.re = few<E>(yr); z.im = few<E>(yi); }               \
                else           { z.re = few<E>(xr); z.im = few<E>(xi); }               \
                return z; }                                                            \
      }                                                                                \
   };
SD_BIN_MINMAX(min,  &, <=, m_isnan<W>(b) || (b < a),
              (m_isnan<W>(yr) || m_isnan<W>(yi)) || (yr < xr) || ((yr == xr) && (yi < xi)))
SD_BIN_MINMAX(max,  |, >=, m_isnan<W>(b) || (b > a),
              (m_isnan<W>(yr) || m_isnan<W>(yi)) || (yr > xr) || ((yr == xr) && (yi > xi)))
SD_BIN_MINMAX(fmin, &, <=, m_isnan<W>(a) || (b <= a),
              ((yr < xr) || m_isnan<W>(xr)) || ((xr == yr) && ((yi < xi) || m_isnan<W>(xi))))
SD_BIN_MINMAX(fmax, |, >=, m_isnan<W>(a) || (b >= a),
              ((yr > xr) || m_isnan<W>(xr)) || ((xr == yr) && ((yi > xi) || m_isnan<W>(xi))))
#undef SD_BIN_MINMAX

// Shifts: the count is a signed 8-bit tensor; a negative count shifts the other
// way (binary_ops.h:253-254).  The value operand is promoted to int first.
template <bool LEFT> struct b_bitshift {
   template <class T> using in2 = int8_t; template <class T> using out = T;
   template <class T> static SD_D T f(T x, int8_t s)
   {
      if constexpr (is_bool<T>) { Bool r; r.v = (s == 0) ? (x.v & 0x01) : 0; return r; }
      else {
         auto xx = +x;
         int n = (s < 0) ? -(int)s : (int)s;
         bool left = LEFT ? (s >= 0) : (s < 0);
         return (T)(left ? (xx << n) : (xx >> n));
      }
   }
};
using b_bitshift_left  = b_bitshift<true>;
using b_bitshift_right = b_bitshift<false>;

// power: integers by repeated squaring with an int16 exponent tensor (negative
// exponent gives 0), reals through pow (single precision in the oracle), complex
// through exp(y*log(x)) with 0^0 = 1 (binary_ops.h:238-248,309-313,386-414).
struct b_power {
   template <class T> using in2 = typename std::conditional<is_bool<T> || is_int<T>, int16_t, T>::type;
   template <class T> using out = T;
   template <class T> static SD_D T f(T x, in2<T> y)
   {
      if constexpr (is_bool<T>) { Bool r; r.v = ((x.v != 0) | (y == 0)) ? 1 : 0; return r; }
      else if constexpr (is_int<T>) {
         T b = x; T z; int64_t e = y;
         z = (T)(e >= 0);
         while (e > 0) { if (e & 1) z = (T)(z * b); e >>= 1; b = (T)(b * b); }
         return z;
      } else if constexpr (is_real<T>) {
         using W = work_t<T>; return from_work<T>(m_pow<W>(to_work<T>(x), to_work<T>(y)));
      } else {
         using E = elem_t<T>; using W = work_t<E>;
         W xr = ew<E>(x.re), xi = ew<E>(x.im), yr = ew<E>(y.re), yi = ew<E>(y.im);
         W scale = xr * xr + xi * xi;
         T z;
         if (scale == 0) {
            z.re = few<E>((W)((yr == 0) && (yi == 0)));
            if constexpr (is_half<E>) z.im.v = 0; else z.im = 0;
         } else {
            W zi = m_atan2<W>(xi, xr);
            W zr = (W)((double)m_log<W>(scale) * 0.5);
            xr = yr * zr - yi * zi;
            xi = yr * zi + yi * zr;
            scale = m_exp<W>(xr);
            xr = scale * m_cos<W>(xi);
            xi = scale * m_sin<W>(xi);
            z.re = few<E>(xr); z.im = few<E>(xi);
         }
         return z;
      }
   }
};

} // namespace sd
