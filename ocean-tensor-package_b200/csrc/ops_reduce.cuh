// Reduction operations (global and per axis), one class template per table name.
//
// Semantics: solid/include/solid/core/generic/reduce_ops.h:141-1287 (init /
// accumulate / combine / finalize of every reduction and its result type):
//   - accumulation runs in the WORK type of the RESULT type: bool/unsigned sums
//     in uint64, signed in int64, half in float, complex component-wise;
//   - any/all/nnz test "!(x == 0)", so a NaN counts as non-zero;
//   - maximum/minimum start from the FIRST element and afterwards ignore NaN
//     ("!isnan(t) && !(acc >= t)", lines 900-911), so an all-NaN tensor returns
//     its first element and the result never depends on an identity value;
//   - norm2 = sqrt(sum x*x) unscaled; norm(p) = (sum (x*x)^(p/2))^(1/p) with the
//     oracle's single-precision pow; integer norms accumulate in double.
//
// A reduction object R<T> carries its parameters (bounds, p) and provides
//     acc_t, out_t, static constexpr bool seeded
//     acc_t  init()            identity                       (when !seeded)
//     acc_t  seed(T first)     accumulator made from element 0 (when seeded)
//     void   accum(acc_t&, T)  fold one element
//     void   combine(acc_t&, acc_t)  fold a partial result; partials are folded
//                              in a fixed order, so results are reproducible
//     out_t  finalize(acc_t)
#pragma once
#include "mathfn.cuh"
#include "word_accum.cuh"

namespace sd {

template <class T> using sum_out_t =
   typename std::conditional<is_bool<T> || is_uint<T>, uint64_t,
   typename std::conditional<is_sint<T>, int64_t, T>::type>::type;
template <class T> using abs_out_t =            // SDTYPE_ABSTYPE: signed -> unsigned, complex -> component
   typename std::conditional<is_sint<T>, typename std::make_unsigned<
      typename std::conditional<is_sint<T>, T, int>::type>::type,
   typename std::conditional<is_cplx<T>, elem_t<T>, T>::type>::type;

template <class T> SD_D bool nonzero(T x)
{
   if constexpr (is_cplx<T>) { using E = elem_t<T>; return (!(ew<E>(x.re) == 0)) || (!(ew<E>(x.im) == 0)); }
   else return !(to_work<T>(x) == 0);
}
template <class T> SD_D bool has_nan(T x)
{
   if constexpr (is_cplx<T>) { using E = elem_t<T>; using W = work_t<E>; return m_isnan<W>(ew<E>(x.re)) || m_isnan<W>(ew<E>(x.im)); }
   else if constexpr (is_real<T>) { using W = work_t<T>; return m_isnan<W>(to_work<T>(x)); }
   else return false;
}

// ---- bool-valued reductions -------------------------------------------------
template <class T, bool ANY, class PRED> struct r_logical {
   using acc_t = uint8_t; using out_t = Bool; static constexpr bool seeded = false;
   PRED pred;
   SD_D acc_t init() const { return ANY ? 0 : 1; }
   SD_D void accum(acc_t &a, T x) const { if (ANY) { if (pred(x)) a = 1; } else { if (!pred(x)) a = 0; } }
   SD_D void combine(acc_t &a, acc_t b) const { if (ANY) a |= b; else a &= b; }
   SD_D out_t finalize(acc_t a) const { Bool r; r.v = a; return r; }
};
template <class T> struct p_nonzero { SD_D bool operator()(T x) const { return nonzero<T>(x); } };
template <class T> struct p_finite {
   SD_D bool operator()(T x) const {
      if constexpr (is_cplx<T>) { using E = elem_t<T>; using W = work_t<E>; return m_isfinite<W>(ew<E>(x.re)) && m_isfinite<W>(ew<E>(x.im)); }
      else { using W = work_t<T>; return m_isfinite<W>(to_work<T>(x)); } } };
template <class T> struct p_inf {
   SD_D bool operator()(T x) const {
      if constexpr (is_cplx<T>) { using E = elem_t<T>; using W = work_t<E>; return m_isinf<W>(ew<E>(x.re)) || m_isinf<W>(ew<E>(x.im)); }
      else { using W = work_t<T>; return m_isinf<W>(to_work<T>(x)); } } };
template <class T> struct p_nan { SD_D bool operator()(T x) const { return has_nan<T>(x); } };

template <class T> using r_any        = r_logical<T, true,  p_nonzero<T>>;
template <class T> using r_all        = r_logical<T, false, p_nonzero<T>>;
template <class T> using r_all_finite = r_logical<T, false, p_finite<T>>;
template <class T> using r_any_inf    = r_logical<T, true,  p_inf<T>>;
template <class T> using r_any_nan    = r_logical<T, true,  p_nan<T>>;

// Range tests (reduce_ops.h:350-600).  LO/HI: 0 = no bound, 1 = strict, 2 = inclusive.
// Complex values order lexicographically; the one-sided complex "lt"/"le" tests
// reject on real > bound (lines 360-364, 386-390), mirrored here.
template <class T, int LO, int HI> struct p_range {
   work_t<T> lower, upper;
   SD_D bool operator()(T x) const
   {
      if constexpr (!is_cplx<T>) {
         auto w = to_work<T>(x);
         if constexpr (LO == 1) { if (w <= lower) return false; }
         if constexpr (LO == 2) { if (w <  lower) return false; }
         if constexpr (HI == 1) { if (w >= upper) return false; }
         if constexpr (HI == 2) { if (w >  upper) return false; }
         return true;
      } else {
         using E = elem_t<T>;
         auto re = ew<E>(x.re); auto im = ew<E>(x.im);
         if constexpr (LO != 0 && HI != 0) {
            if ((re < lower.re) || (re > upper.re)) return false;
            if constexpr (LO == 1) { if ((re == lower.re) && (im <= lower.im)) return false; }
            else                   { if ((re == lower.re) && (im <  lower.im)) return false; }
            if constexpr (HI == 1) { if ((re == upper.re) && (im >= upper.im)) return false; }
            else                   { if ((re == upper.re) && (im >  upper.im)) return false; }
            return true;
         } else if constexpr (HI != 0) {
            if (re > upper.re) return false;
            if constexpr (HI == 1) { if ((re == upper.re) && (im >= upper.im)) return false; }
            else                   { if ((re == upper.re) && (im >  upper.im)) return false; }
            return true;
         } else {
            if (re < lower.re) return false;
            if constexpr (LO == 1) { if ((re == lower.re) && (im <= lower.im)) return false; }
            else                   { if ((re == lower.re) && (im <  lower.im)) return false; }
            return true;
         }
      }
   }
};
template <class T, int LO, int HI> using r_range = r_logical<T, false, p_range<T, LO, HI>>;

// ---- counting ----------------------------------------------------------------
template <class T, bool SKIP_NAN> struct r_count {
   using acc_t = uint64_t; using out_t = uint64_t; static constexpr bool seeded = false;
   SD_D acc_t init() const { return 0; }
   SD_D void accum(acc_t &a, T x) const
   {  if constexpr (SKIP_NAN) { if (!has_nan<T>(x) && nonzero<T>(x)) a++; } else { if (nonzero<T>(x)) a++; } }
   SD_D void combine(acc_t &a, acc_t b) const { a += b; }
   SD_D out_t finalize(acc_t a) const { return a; }
};
template <class T> using r_nnz     = r_count<T, false>;
template <class T> using r_nnz_nan = r_count<T, (is_real<T> || is_cplx<T>)>;

// ---- sum / prod --------------------------------------------------------------
template <class T, bool SKIP_NAN> struct r_sum_ {
   using out_t = sum_out_t<T>; using acc_t = work_t<out_t>; static constexpr bool seeded = false;
   SD_D acc_t init() const { if constexpr (is_cplx<T>) { acc_t a; a.re = 0; a.im = 0; return a; } else return 0; }
   SD_D void accum(acc_t &a, T x) const
   {
      if constexpr (is_cplx<T>) { auto w = to_work<T>(x);
         if constexpr (SKIP_NAN) { if (has_nan<T>(x)) return; }
         a.re += w.re; a.im += w.im; }
      else { auto w = to_work<T>(x);
         if constexpr (SKIP_NAN) { if (has_nan<T>(x)) return; }
         a += w; }
   }
   SD_D void combine(acc_t &a, acc_t b) const { if constexpr (is_cplx<T>) { a.re += b.re; a.im += b.im; } else a += b; }
   SD_D out_t finalize(acc_t a) const { return from_work<out_t>(a); }
};
template <class T> using r_sum     = r_sum_<T, false>;
template <class T> using r_sum_nan = r_sum_<T, (is_real<T> || is_cplx<T>)>;

// The NaN-skipping complex product of the oracle accumulates the imaginary part
// with a minus sign (reduce_ops.h:779); partial results are then combined with
// the regular complex product.  Reproduced as is.
template <class T, bool SKIP_NAN> struct r_prod_ {
   using out_t = sum_out_t<T>; using acc_t = work_t<out_t>; static constexpr bool seeded = false;
   SD_D acc_t init() const { if constexpr (is_cplx<T>) { acc_t a; a.re = 1; a.im = 0; return a; } else return 1; }
   SD_D void accum(acc_t &a, T x) const
   {
      if constexpr (is_cplx<T>) { auto w = to_work<T>(x);
         if constexpr (SKIP_NAN) {
            if (has_nan<T>(x)) return;
            auto t = a.re; a.re = t * w.re - a.im * w.im; a.im = t * w.im - a.im * w.re;
         } else {
            auto t = a.re; a.re = t * w.re - a.im * w.im; a.im = t * w.im + a.im * w.re;
         } }
      else { auto w = to_work<T>(x);
         if constexpr (SKIP_NAN) { if (has_nan<T>(x)) return; }
         a *= w; }
   }
   SD_D void combine(acc_t &a, acc_t b) const
   {  if constexpr (is_cplx<T>) { auto t = a.re; a.re = t * b.re - a.im * b.im; a.im = t * b.im + a.im * b.re; } else a *= b; }
   SD_D out_t finalize(acc_t a) const { return from_work<out_t>(a); }
};
template <class T> using r_prod     = r_prod_<T, false>;
template <class T> using r_prod_nan = r_prod_<T, (is_real<T> || is_cplx<T>)>;

// ---- sum of magnitudes ---------------------------------------------------------
template <class T, bool SKIP_NAN> struct r_sum_abs_ {
   using out_t = typename std::conditional<is_bool<T> || is_int<T>, uint64_t, abs_out_t<T>>::type;
   using acc_t = work_t<out_t>; static constexpr bool seeded = false;
   SD_D acc_t init() const { return 0; }
   SD_D void accum(acc_t &a, T x) const
   {
      if constexpr (is_bool<T> || is_uint<T>) a += to_work<T>(x);
      else if constexpr (is_sint<T>) { if (x < 0) a -= (uint64_t)(int64_t)x; else a += (uint64_t)(int64_t)x; }
      else if constexpr (is_real<T>) { using W = work_t<T>; W w = to_work<T>(x);
         if constexpr (SKIP_NAN) { if (m_isnan<W>(w)) return; }
         a += m_fabs<W>(w); }
      else { using E = elem_t<T>; using W = work_t<E>; W re = ew<E>(x.re), im = ew<E>(x.im);
         if constexpr (SKIP_NAN) { if (m_isnan<W>(re) || m_isnan<W>(im)) return; }
         a += m_hypot<W>(re, im); }
   }
   SD_D void combine(acc_t &a, acc_t b) const { a += b; }
   SD_D out_t finalize(acc_t a) const { return from_work<out_t>(a); }
};
template <class T> using r_sum_abs     = r_sum_abs_<T, false>;
template <class T> using r_sum_abs_nan = r_sum_abs_<T, (is_real<T> || is_cplx<T>)>;

// ---- extrema -------------------------------------------------------------------
template <class T, bool MAX> struct r_extremum {
   using out_t = T; using acc_t = work_t<T>; static constexpr bool seeded = true;
   SD_D acc_t seed(T first) const { return to_work<T>(first); }
   SD_D static bool better_real(acc_t acc, acc_t t)      // true when t must replace acc
   {
      if constexpr (is_bool<T> || is_int<T>) return MAX ? (acc < t) : (acc > t);
      else { return (!m_isnan<acc_t>(t)) && (MAX ? !(acc >= t) : !(acc <= t)); }
   }
   SD_D void fold(acc_t &a, acc_t t) const
   {
      if constexpr (is_cplx<T>) {
         using W = ework_t<T>;
         bool first = MAX ? !(a.re >= t.re) : !(a.re <= t.re);
         bool tie   = (!(a.re < t.re)) && (!(a.re > t.re)) && (MAX ? !(a.im >= t.im) : !(a.im <= t.im));
         if ((!m_isnan<W>(t.re)) && (!m_isnan<W>(t.im)) && (first || tie || m_isnan<W>(a.im))) a = t;
      } else { if (better_real(a, t)) a = t; }
   }
   SD_D void accum(acc_t &a, T x) const { fold(a, to_work<T>(x)); }
   SD_D void combine(acc_t &a, acc_t b) const { fold(a, b); }
   SD_D out_t finalize(acc_t a) const { return from_work<T>(a); }
};
template <class T> using r_maximum = r_extremum<T, true>;
template <class T> using r_minimum = r_extremum<T, false>;

template <class T, bool MAX> struct r_extremum_abs {
   using out_t = abs_out_t<T>; using acc_t = work_t<out_t>; static constexpr bool seeded = true;
   SD_D static acc_t mag(T x)
   {
      if constexpr (is_bool<T> || is_uint<T>) return to_work<T>(x);
      else if constexpr (is_sint<T>) return (x < 0) ? (acc_t)((acc_t)0 - (acc_t)x) : (acc_t)x;
      else if constexpr (is_real<T>) return m_fabs<acc_t>(to_work<T>(x));
      else { using E = elem_t<T>; return m_hypot<acc_t>(ew<E>(x.re), ew<E>(x.im)); }
   }
   SD_D acc_t seed(T first) const { return mag(first); }
   SD_D void fold(acc_t &a, acc_t t) const
   {
      if constexpr (is_bool<T> || is_int<T>) { if (MAX ? (a < t) : (a > t)) a = t; }
      else { if ((!m_isnan<acc_t>(t)) && (MAX ? !(a >= t) : !(a <= t))) a = t; }
   }
   SD_D void accum(acc_t &a, T x) const { fold(a, mag(x)); }
   SD_D void combine(acc_t &a, acc_t b) const { fold(a, b); }
   SD_D out_t finalize(acc_t a) const { return from_work<out_t>(a); }
};
template <class T> using r_maximum_abs = r_extremum_abs<T, true>;
template <class T> using r_minimum_abs = r_extremum_abs<T, false>;

// ---- norms ---------------------------------------------------------------------
template <class T> using norm_out_t =
   typename std::conditional<is_bool<T> || is_int<T>, double, abs_out_t<T>>::type;

template <class T, bool SKIP_NAN> struct r_norm2_ {
   using out_t = norm_out_t<T>; using acc_t = work_t<out_t>; static constexpr bool seeded = false;
   SD_D acc_t init() const { return 0; }
   SD_D void accum(acc_t &a, T x) const
   {
      if constexpr (is_bool<T> || is_int<T>) { double t = (double)to_work<T>(x); a += t * t; }
      else if constexpr (is_real<T>) { acc_t t = to_work<T>(x);
         if constexpr (SKIP_NAN) { if (m_isnan<acc_t>(t)) return; }
         a += t * t; }
      else { auto w = to_work<T>(x); acc_t t = (w.re * w.re) + (w.im * w.im);
         if constexpr (SKIP_NAN) { if (m_isnan<acc_t>(t)) return; }
         a += t; }
   }
   SD_D void combine(acc_t &a, acc_t b) const { a += b; }
   SD_D out_t finalize(acc_t a) const { return from_work<out_t>(m_sqrt<acc_t>(a)); }
};
template <class T> using r_norm2     = r_norm2_<T, false>;
template <class T> using r_norm2_nan = r_norm2_<T, (is_real<T> || is_cplx<T>)>;

template <class T, bool SKIP_NAN> struct r_norm_ {
   using out_t = norm_out_t<T>; using acc_t = work_t<out_t>; static constexpr bool seeded = false;
   acc_t phalf, pinv;
   SD_D acc_t init() const { return 0; }
   SD_D void accum(acc_t &a, T x) const
   {
      if constexpr (is_bool<T> || is_int<T>) { double t = (double)to_work<T>(x); t *= t; a += m_pow<double>(t, phalf); }
      else if constexpr (is_real<T>) { acc_t t = to_work<T>(x);
         if constexpr (SKIP_NAN) { if (m_isnan<acc_t>(t)) return; }
         t *= t; a += m_pow<acc_t>(t, phalf); }
      else { auto w = to_work<T>(x); acc_t t = (w.re * w.re) + (w.im * w.im);
         if constexpr (SKIP_NAN) { if (m_isnan<acc_t>(t)) return; }
         a += m_pow<acc_t>(t, phalf); }
   }
   SD_D void combine(acc_t &a, acc_t b) const { a += b; }
   SD_D out_t finalize(acc_t a) const { return from_work<out_t>(m_pow<acc_t>(a, pinv)); }
};
template <class T> using r_norm     = r_norm_<T, false>;
template <class T> using r_norm_nan = r_norm_<T, (is_real<T> || is_cplx<T>)>;

// ---------------------------------------------------------------------------
// Four 1-byte elements at a time.  For the reductions below a 32-bit word of packed
// bool / uint8 / int8 elements can be folded with one or two SIMD-in-register
// instructions instead of four extract-test-accumulate sequences; the kernels use
// this when word_accum<R, T>::ok.
// ---------------------------------------------------------------------------

template <class T> struct word_accum<r_count<T, false>, T> {               // nnz: bytes that are not zero
   static constexpr bool ok = sizeof(T) == 1;
   SD_D static void apply(const r_count<T, false> &, uint64_t &a, uint32_t w) { a += __popc(__vcmpne4(w, 0u)) >> 3; }
};
template <class T> struct word_accum<r_logical<T, true, p_nonzero<T>>, T> {  // any
   static constexpr bool ok = sizeof(T) == 1;
   SD_D static void apply(const r_logical<T, true, p_nonzero<T>> &, uint8_t &a, uint32_t w) { if (w) a = 1; }
};
template <class T> struct word_accum<r_logical<T, false, p_nonzero<T>>, T> { // all
   static constexpr bool ok = sizeof(T) == 1;
   SD_D static void apply(const r_logical<T, false, p_nonzero<T>> &, uint8_t &a, uint32_t w) { if (__vcmpeq4(w, 0u)) a = 0; }
};
template <class T> struct word_accum<r_sum_<T, false>, T> {                  // sum of bytes
   static constexpr bool ok = sizeof(T) == 1;
   SD_D static void apply(const r_sum_<T, false> &, typename r_sum_<T, false>::acc_t &a, uint32_t w)
   {
      if constexpr (is_sint<T>) a += (int64_t)__dp4a((int)w, 0x01010101, 0);
      else                      a += (uint64_t)__dp4a(w, 0x01010101u, 0u);
   }
};

} // namespace sd
