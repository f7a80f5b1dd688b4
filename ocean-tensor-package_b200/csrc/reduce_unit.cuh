// Shared by reduce_all.cu and reduce_axis.cu: maps each table name to the
// reduction class of ops_reduce.cuh for the unit's element type T, following the
// per-type aliases of solid/src/core/gpu/template_reduce_all.cu:240-437 (unsigned
// and bool sum_abs is sum, their maximum_abs/minimum_abs are maximum/minimum; the
// *_nan forms of integer types are the plain forms).
#pragma once
#include "unit.cuh"
#include "reduce.cuh"
#include "ops_reduce.cuh"

namespace sdu {
using namespace sd;
constexpr bool unsigned_like = is_bool<T> || is_uint<T>;
using R_any = r_any<T>;                 using R_all = r_all<T>;
using R_all_finite = r_all_finite<T>;   using R_any_inf = r_any_inf<T>;   using R_any_nan = r_any_nan<T>;
using R_nnz = r_nnz<T>;                 using R_nnz_nan = r_nnz_nan<T>;
using R_sum = r_sum<T>;                 using R_sum_nan = r_sum_nan<T>;
using R_prod = r_prod<T>;               using R_prod_nan = r_prod_nan<T>;
using R_sum_abs     = std::conditional<unsigned_like, r_sum<T>, r_sum_abs<T>>::type;
using R_sum_abs_nan = std::conditional<unsigned_like, r_sum<T>, r_sum_abs_nan<T>>::type;
using R_maximum = r_maximum<T>;         using R_minimum = r_minimum<T>;
using R_maximum_abs = std::conditional<unsigned_like, r_maximum<T>, r_maximum_abs<T>>::type;
using R_minimum_abs = std::conditional<unsigned_like, r_minimum<T>, r_minimum_abs<T>>::type;
using R_norm2 = r_norm2<T>;             using R_norm2_nan = r_norm2_nan<T>;
using R_norm = r_norm<T>;               using R_norm_nan = r_norm_nan<T>;

template <class R> inline R make_norm(double p)
{
   R r; double phalf = p / 2, pinv = 1 / p;
   r.phalf = (typename R::acc_t)phalf; r.pinv = (typename R::acc_t)pinv;
   return r;
}
// bound scalar (element type T on the host) -> work type
template <class U> inline work_t<U> bound_value_(const solid_scalar *s)
{
   U v; memcpy(&v, s, sizeof(U));
   if constexpr (is_bool<U>) return v.v;
   else if constexpr (is_half<U>) return half_to_float(v);
   else if constexpr (std::is_same<U, CHalf>::value) { CFloat r; r.re = half_to_float(v.re); r.im = half_to_float(v.im); return r; }
   else return v;
}
inline work_t<T> bound_value(const solid_scalar *s) { return bound_value_<T>(s); }
} // namespace sdu
