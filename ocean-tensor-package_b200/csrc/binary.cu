// solid_gpu_<binary op>_<SDX> for one element type (list: SOLID_GPU_BINARY_OPS).
// Replaces solid/src/core/gpu/template_binary.cu:35-270 for that type.
#include "unit.cuh"
#include "elemwise.cuh"
#include "ops_binary.cuh"

#define SD_DEFINE_BINARY(NAME, GROUP) SD_WHEN(GROUP)(                                             \
   extern "C" int SD_PASTE(solid_gpu_##NAME##_, SDX)(SOLID_GPU_ARGS_BINARY)                        \
   {  return sd::launch_binary<sd::b_##NAME, T>(ndims, size, strides1, ptr1, strides2, ptr2,       \
                                                strides3, ptr3, stream); })

SOLID_GPU_BINARY_OPS(SD_DEFINE_BINARY)

// z = a*x + y with the product rounded to the element type first: what Ocean's
// multiplyScalar followed by add produces (src/core/interface/tensor_itf.c:4221-4251),
// in one pass.  Real floating-point types.
namespace sd {
template <class T> struct AxpyApply {
   static constexpr int NIN = 2;
   using in1_t = T; using in2_t = T; using out_t = T;
   T a;
   SD_D T operator()(T x, T y) const
   {
      using W = work_t<T>;
      if constexpr (is_half<T>) {
         // Same values as the generic form below with fewer instructions.  (1) The inputs are
         // decoded by the hardware conversion alone: its only difference from half.c, -0 instead
         // of +0, cannot reach the result, because a zero product is re-encoded as +0 before the
         // addition and a zero sum is encoded as +0 at the end.  (2) Rounding the product to half
         // and decoding it again is done on the float bits: for the normal half range that is
         // "add half a unit of the 13 dropped bits, clear them".
         const float xf = __half2float(__ushort_as_half(x.v)), yf = __half2float(__ushort_as_half(y.v));
         const float af = __half2float(__ushort_as_half(a.v));
         const float p = af * xf;
         const uint32_t raw = __float_as_uint(p);
         float pr;
         if (((raw >> 23) & 0xFFu) - 113u < 29u) pr = __uint_as_float((raw + 0x1000u) & 0xFFFFE000u);
         else pr = half_to_float(float_to_half(p));
         return float_to_half(pr + yf);
      } else {
         T prod = from_work<T>(to_work<T>(a) * to_work<T>(x));
         return from_work<T>((W)(to_work<T>(prod) + to_work<T>(y)));
      }
   }
};
} // namespace sd
SD_WHEN(real)(
extern "C" int SD_PASTE(solid_gpu_axpy_, SDX)(SOLID_GPU_ARGS_AXPY)
{
   const ptrdiff_t *st[3] = { strides1, strides2, strides3 }; void *pt[3] = { ptr1, ptr2, ptr3 };
   sd::Layout<3> L;
   if (sd::make_layout<3>(L, ndims, size, st, pt, 2) != 0) return -1;
   sd::AxpyApply<T> ap; memcpy(&ap.a, &a, sizeof(T));
   return sd::ew_launch(ap, L, stream);
})
