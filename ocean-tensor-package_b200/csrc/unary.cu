// solid_gpu_<unary op>_<SDX> for one element type (list: SOLID_GPU_UNARY_OPS).
// Replaces solid/src/core/gpu/template_unary.cu:52-246 for that type.
#include "unit.cuh"
#include "elemwise.cuh"
#include "ops_unary.cuh"

#define SD_DEFINE_UNARY(NAME, GROUP) SD_WHEN(GROUP)(                                              \
   extern "C" int SD_PASTE(solid_gpu_##NAME##_, SDX)(SOLID_GPU_ARGS_UNARY)                         \
   {  return sd::launch_unary<sd::u_##NAME, T>(ndims, size, strides1, ptr1, strides2, ptr2, stream); })

SOLID_GPU_UNARY_OPS(SD_DEFINE_UNARY)

// The functions with a domain, fused with the domain test (list: SOLID_GPU_CHECKED_OPS): the element function is the
// one above; a vector of elements sets the caller's flag with one store when any of them fails the test.
namespace sd {
// "outside" is what makes the reference's reductions fail (solid/include/solid/core/generic/reduce_ops.h:434-441,
// 572-580: x < bound, x > bound), so a NaN is not outside, exactly as there.
struct dom_ge_zero  { template <class W> static SD_D bool outside(W x) { return x < (W)0; } };
struct dom_ge_neg1  { template <class W> static SD_D bool outside(W x) { return x < (W)-1; } };
struct dom_ge_one   { template <class W> static SD_D bool outside(W x) { return x < (W)1; } };
struct dom_unit     { template <class W> static SD_D bool outside(W x) { return (x < (W)-1) || (x > (W)1); } };
struct dom_nonzero  { template <class W> static SD_D bool outside(W x) { return x == (W)0; } };

template <class Op, class Dom, class T> struct CheckedApply {
   static constexpr int NIN = 1;
   static constexpr bool VECTOR = true;
   using in1_t = T; using in2_t = Nothing; using out_t = T;
   int *flag;
   SD_D T operator()(T x, Nothing) const
   {
      if (Dom::outside(to_work<T>(x))) *flag = 1;
      return Op::template f<T>(x);
   }
   template <int N> SD_D Vec<T, N> vec(const Vec<T, N> &x, const Vec<Nothing, N> &) const
   {
      Vec<T, N> o; bool bad = false;
#pragma unroll
      for (int j = 0; j < N; j++) { bad = bad || Dom::outside(to_work<T>(x.v[j])); o.v[j] = Op::template f<T>(x.v[j]); }
      if (bad) *flag = 1;                                  // every writer stores the same value
      return o;
   }
};
template <class Op, class Dom, class T>
int launch_checked(int ndims, const size_t *size, const ptrdiff_t *strides1, void *ptr1,
                   const ptrdiff_t *strides2, void *ptr2, int *outside, cudaStream_t stream)
{
   if (outside == nullptr) SD_ERROR("The checked functions need the address of the flag");
   if (strides2 == nullptr && ptr2 == nullptr) { strides2 = strides1; ptr2 = ptr1; }   // in place
   const ptrdiff_t *st[2] = { strides1, strides2 }; void *pt[2] = { ptr1, ptr2 };
   Layout<2> L;
   if (make_layout<2>(L, ndims, size, st, pt, 1) != 0) return -1;
   CheckedApply<Op, Dom, T> ap; ap.flag = outside;
   return ew_launch(ap, L, stream);
}
} // namespace sd
#define SD_DEFINE_CHECKED(NAME, DOM) SD_WHEN(real)(                                               \
   extern "C" int SD_PASTE(solid_gpu_##NAME##_checked_, SDX)(SOLID_GPU_ARGS_UNARY_CHECKED)          \
   {  return sd::launch_checked<sd::u_##NAME, sd::DOM, T>(ndims, size, strides1, ptr1, strides2, ptr2, outside, stream); })
SD_DEFINE_CHECKED(sqrt, dom_ge_zero) SD_DEFINE_CHECKED(log, dom_ge_zero) SD_DEFINE_CHECKED(log2, dom_ge_zero)
SD_DEFINE_CHECKED(log10, dom_ge_zero) SD_DEFINE_CHECKED(log1p, dom_ge_neg1) SD_DEFINE_CHECKED(arccosh, dom_ge_one)
SD_DEFINE_CHECKED(arcsin, dom_unit) SD_DEFINE_CHECKED(arccos, dom_unit) SD_DEFINE_CHECKED(arctanh, dom_unit)
SD_DEFINE_CHECKED(reciprocal, dom_nonzero)
