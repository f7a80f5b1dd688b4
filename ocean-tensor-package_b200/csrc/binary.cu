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

// dst = op(src, value) with the scalar in the launch arguments (list: SOLID_GPU_SCALAR_OPS); the same
// functors as the tensor operations, so the results are those of a broadcast second operand.
namespace sd {
template <class Op, class T> struct ScalarApply {
   static constexpr int NIN = 1;
   using in1_t = T; using in2_t = Nothing; using out_t = typename Op::template out<T>;
   T s;
   SD_D out_t operator()(T x, Nothing) const { return Op::template f<T>(x, s); }
};
template <class Op, class T>
int launch_scalar(int ndims, const size_t *size, const ptrdiff_t *strides1, void *ptr1, const solid_scalar &value,
                  const ptrdiff_t *strides2, void *ptr2, cudaStream_t stream)
{
   if (strides2 == nullptr && ptr2 == nullptr) { strides2 = strides1; ptr2 = ptr1; }   // in place
   const ptrdiff_t *st[2] = { strides1, strides2 }; void *pt[2] = { ptr1, ptr2 };
   Layout<2> L;
   if (make_layout<2>(L, ndims, size, st, pt, 1) != 0) return -1;
   ScalarApply<Op, T> ap; memcpy(&ap.s, &value, sizeof(T));
   return ew_launch(ap, L, stream);
}
} // namespace sd
#define SD_DEFINE_SCALAR(NAME, OP, GROUP) SD_WHEN(GROUP)(                                          \
   extern "C" int SD_PASTE(solid_gpu_##NAME##_, SDX)(SOLID_GPU_ARGS_SCALAR_OP)                      \
   {  return sd::launch_scalar<sd::b_##OP, T>(ndims, size, strides1, ptr1, value, strides2, ptr2, stream); })
SD_DEFINE_SCALAR(add_scalar, add, all) SD_DEFINE_SCALAR(subtract_scalar, subtract, all)
SD_DEFINE_SCALAR(multiply_scalar, multiply, all)
SD_DEFINE_SCALAR(bitwise_and_scalar, bitwise_and, integer_bool) SD_DEFINE_SCALAR(bitwise_or_scalar, bitwise_or, integer_bool)
SD_DEFINE_SCALAR(bitwise_xor_scalar, bitwise_xor, integer_bool)

// z = a*x + y with the product rounded to the element type first: what Ocean's
// multiplyScalar followed by add produces (src/core/interface/tensor_itf.c:4221-4251),
// in one pass.  Real floating-point types.
namespace sd {
template <class T> struct AxpyApply {
   static constexpr int NIN = 2;
   static constexpr bool VECTOR = is_half<T>;
   static constexpr int MIN_BLOCKS = is_half<T> ? 4 : 0;
   using in1_t = T; using in2_t = T; using out_t = T;
   T a;
   SD_D T operator()(T x, T y) const
   {
      using W = work_t<T>;
      T prod = from_work<T>(to_work<T>(a) * to_work<T>(x));
      return from_work<T>((W)(to_work<T>(prod) + to_work<T>(y)));
   }
   // Half, a whole vector at a time.  While the product and the sum of every element stay inside the normal half
   // range, the two roundings of the reference (half.c rounds half away from zero) are done on the float bits:
   // "add half a unit of the 13 dropped bits, clear them".  The inputs then need the hardware conversion only
   // (its one difference from half.c, -0 for +0, cannot survive a non-zero product or sum), and the result is
   // exactly representable, so the hardware conversion back is exact.  One out-of-range element (zero, subnormal,
   // overflow, inf, nan) sends the whole vector through the per-element form above, out of line.
   template <int N> SD_D Vec<T, N> vec(const Vec<T, N> &x, const Vec<T, N> &y) const
   {
      if constexpr (is_half<T> && (N % 2 == 0)) {
         // Two halves per 32-bit word, converted by the PACKED instructions (cvt.f32.f16 issues on the
         // special-function pipe, a few lanes per cycle: with one conversion per element this kernel ran at
         // 4.2 TB/s bound by that pipe, with one per pair it runs at the HBM rate).
         const float af = __half2float(__ushort_as_half(a.v));
         uint32_t xw[N / 2], yw[N / 2];
         memcpy(xw, &x, sizeof(xw)); memcpy(yw, &y, sizeof(yw));
         float w[N];
         // magnitude bits of every product and of every sum: smallest and largest over the vector
         uint32_t plo = 0x7FFFFFFFu, phi = 0u, slo = 0x7FFFFFFFu, shi = 0u;
#pragma unroll
         for (int k = 0; k < N / 2; k++) {
            const float2 xf = __half22float2(*reinterpret_cast<const __half2 *>(&xw[k]));
            const float2 yf = __half22float2(*reinterpret_cast<const __half2 *>(&yw[k]));
            const float xs[2] = { xf.x, xf.y }, ys[2] = { yf.x, yf.y };
            uint32_t pm[2], sm[2];
#pragma unroll
            for (int e = 0; e < 2; e++) {
               const uint32_t praw = __float_as_uint(af * xs[e]);
               pm[e] = praw & 0x7FFFFFFFu;
               const uint32_t sraw = __float_as_uint(__uint_as_float((praw + 0x1000u) & 0xFFFFE000u) + ys[e]);
               sm[e] = sraw & 0x7FFFFFFFu;
               w[2 * k + e] = __uint_as_float((sraw + 0x1000u) & 0xFFFFE000u);
            }
            plo = __vimin3_u32(plo, pm[0], pm[1]); phi = __vimax3_u32(phi, pm[0], pm[1]);
            slo = __vimin3_u32(slo, sm[0], sm[1]); shi = __vimax3_u32(shi, sm[0], sm[1]);
         }
         // 2^-14 <= |product| < 2^15 and 2^-14 <= |sum| < 2^16 (nan and inf have the largest magnitude bits)
         const bool plain = plo >= 0x38800000u && phi < 0x47000000u && slo >= 0x38800000u && shi < 0x47800000u;
         if (!plain) return rare<N>(x, y);
         uint32_t ow[N / 2];
#pragma unroll
         for (int k = 0; k < N / 2; k++) {
            const __half2 h = __floats2half2_rn(w[2 * k], w[2 * k + 1]);
            memcpy(&ow[k], &h, 4);
         }
         Vec<T, N> o;
         memcpy(&o, ow, sizeof(ow));
         return o;
      } else {
         Vec<T, N> o;
#pragma unroll
         for (int j = 0; j < N; j++) o.v[j] = (*this)(x.v[j], y.v[j]);
         return o;
      }
   }
   template <int N> __device__ __noinline__ Vec<T, N> rare(Vec<T, N> x, Vec<T, N> y) const      // by value: stays in registers
   {
      Vec<T, N> o;
#pragma unroll
      for (int j = 0; j < N; j++) o.v[j] = (*this)(x.v[j], y.v[j]);
      return o;
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
