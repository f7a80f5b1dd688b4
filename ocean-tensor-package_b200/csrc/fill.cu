// solid_gpu_fill_<SDX>, fill_nan, masked_fill and byteswap for one element type.
// Replaces solid/src/core/gpu/template_fill.cu:35-109.  fill_nan really replaces
// NaN elements (the reference's GPU wrapper launches the plain fill kernel,
// template_fill.cu:72-79; the CPU semantics of unary_ops.h:320-322,666-669 apply).
#include "unit.cuh"
#include "elemwise.cuh"
#include "mathfn.cuh"

namespace sd {
template <class T> struct FillApply {
   static constexpr int NIN = 0;
   using in1_t = Nothing; using in2_t = Nothing; using out_t = T;
   T value;
   SD_D T operator()(Nothing, Nothing) const { return value; }
};
template <class T> struct FillNanApply {          // in place: dst = isnan(dst) ? value : dst
   static constexpr int NIN = 1;
   using in1_t = T; using in2_t = Nothing; using out_t = T;
   T value;
   SD_D T operator()(T x, Nothing) const
   {
      if constexpr (is_cplx<T>) { using E = elem_t<T>; using W = work_t<E>;
         return (m_isnan<W>(ew<E>(x.re)) || m_isinf<W>(ew<E>(x.im))) ? value : x; }   // sic: isinf on imag
      else { using W = work_t<T>; return m_isnan<W>(to_work<T>(x)) ? value : x; }
   }
};
template <class T> struct MaskedFillApply {       // dst = mask ? value : dst
   static constexpr int NIN = 2;
   using in1_t = T; using in2_t = Bool; using out_t = T;
   T value;
   SD_D T operator()(T x, Bool m) const { return m.v ? value : x; }
};
template <class T> struct ByteswapApply {
   static constexpr int NIN = 1;
   using in1_t = T; using in2_t = Nothing; using out_t = T;
   SD_D T operator()(T x, Nothing) const { return bswap<T>(x); }
};
} // namespace sd

static inline T scalar_value(const solid_scalar &s) { T v; memcpy(&v, &s, sizeof(T)); return v; }

extern "C" int SD_PASTE(solid_gpu_fill_, SDX)(SOLID_GPU_ARGS_FILL)
{
   const ptrdiff_t *st[1] = { strides }; void *pt[1] = { ptr };
   sd::Layout<1> L;
   if (sd::make_layout<1>(L, ndims, size, st, pt, 0) != 0) return -1;
   sd::FillApply<T> a; a.value = scalar_value(value);
   return sd::ew_launch(a, L, stream);
}

SD_WHEN(float)(
extern "C" int SD_PASTE(solid_gpu_fill_nan_, SDX)(SOLID_GPU_ARGS_FILL)
{
   const ptrdiff_t *st[2] = { strides, strides }; void *pt[2] = { ptr, ptr };
   sd::Layout<2> L;
   if (sd::make_layout<2>(L, ndims, size, st, pt, 1) != 0) return -1;
   sd::FillNanApply<T> a; a.value = scalar_value(value);
   return sd::ew_launch(a, L, stream);
})

extern "C" int SD_PASTE(solid_gpu_masked_fill_, SDX)(SOLID_GPU_ARGS_MASKED_FILL)
{
   const ptrdiff_t *st[3] = { strides1, strides2, strides1 }; void *pt[3] = { ptr1, ptr2, ptr1 };
   sd::Layout<3> L;
   if (sd::make_layout<3>(L, ndims, size, st, pt, 2) != 0) return -1;
   sd::MaskedFillApply<T> a; a.value = scalar_value(value);
   return sd::ew_launch(a, L, stream);
}

extern "C" int SD_PASTE(solid_gpu_byteswap_, SDX)(SOLID_GPU_ARGS_BYTESWAP)
{
   const ptrdiff_t *st[2] = { strides, strides }; void *pt[2] = { ptr, ptr };
   sd::Layout<2> L;
   if (sd::make_layout<2>(L, ndims, size, st, pt, 1) != 0) return -1;
   return sd::ew_launch(sd::ByteswapApply<T>(), L, stream);
}
