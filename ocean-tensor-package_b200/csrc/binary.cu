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
// z = half(half(a * x) + y) element by element with the general conversions, for eight halves in four words
__device__ __noinline__ inline uint4 axpy_half_rare8(uint32_t abits, uint4 x, uint4 y)
{
   Half a; a.v = (uint16_t)abits;
   const uint32_t xs[4] = { x.x, x.y, x.z, x.w }, ys[4] = { y.x, y.y, y.z, y.w };
   uint32_t o[4];
   const float af = half_to_float(a);
#pragma unroll
   for (int k = 0; k < 4; k++) {
      uint32_t r = 0;
#pragma unroll
      for (int e = 0; e < 2; e++) {
         Half xh, yh; xh.v = (uint16_t)(xs[k] >> (16 * e)); yh.v = (uint16_t)(ys[k] >> (16 * e));
         const Half prod = float_to_half(af * half_to_float(xh));
         const Half z = float_to_half(half_to_float(prod) + half_to_float(yh));
         r |= (uint32_t)z.v << (16 * e);
      }
      o[k] = r;
   }
   return make_uint4(o[0], o[1], o[2], o[3]);
}

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
   // overflow, inf, nan) sends the whole vector through the per-element form, out of line.
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
         if (!plain) {
            if constexpr (N == 8) {
               // out of line, operands BY VALUE in registers: a call that takes them by reference (or as a member
               // function of this object) makes the compiler keep a copy of x, y and the object in local memory
               // for every vector, rare or not -- measured as 1.5 million local stores per launch and a third of
               // the run time
               const uint4 r = axpy_half_rare8(a.v, make_uint4(xw[0], xw[1], xw[2], xw[3]), make_uint4(yw[0], yw[1], yw[2], yw[3]));
               Vec<T, N> o; memcpy(&o, &r, 16); return o;
            } else {
               Vec<T, N> o;
#pragma unroll
               for (int j = 0; j < N; j++) o.v[j] = (*this)(x.v[j], y.v[j]);
               return o;
            }
         }
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
};
// Dense half tensors: eight halves per 16-byte access, four accesses per operand in flight, one chunk per block,
// and nothing else in the kernel (no broadcast, alignment or stride cases): the general engine runs the same
// arithmetic at 4.2-4.7 TB/s, this form at the HBM rate (6.2 TB/s on 2^26 elements).
constexpr int AXH_U = 4;
template <int AXH_UNROLL>          // a template so that the per-type units of this file share one definition
__global__ void __launch_bounds__(EW_THREADS) axpy_half_dense(const AxpyApply<Half> apply, const uint4 *__restrict__ x,
                                                              const uint4 *__restrict__ y, uint4 *__restrict__ z, uint64_t nvec)
{
   const uint64_t base = (uint64_t)blockIdx.x * (EW_THREADS * AXH_UNROLL) + threadIdx.x;
   uint4 vx[AXH_UNROLL], vy[AXH_UNROLL];
#pragma unroll
   for (int u = 0; u < AXH_UNROLL; u++) {
      const uint64_t i = base + (uint64_t)u * EW_THREADS;
      if (i < nvec) { vx[u] = __ldcs(x + i); vy[u] = __ldcs(y + i); }
   }
#pragma unroll
   for (int u = 0; u < AXH_UNROLL; u++) {
      const uint64_t i = base + (uint64_t)u * EW_THREADS;
      if (i < nvec) {
         Vec<Half, 8> a, b; memcpy(&a, &vx[u], 16); memcpy(&b, &vy[u], 16);
         const Vec<Half, 8> o = apply.template vec<8>(a, b);
         uint4 r; memcpy(&r, &o, 16);
         __stcs(z + i, r);
      }
   }
}
// Runs the dedicated kernel on the whole vectors of one dense, 16-byte aligned run of halves and shortens the
// layout to what is left (possibly nothing); other types and layouts are left untouched for the engine.
template <class T> int axpy_dense_part(const AxpyApply<T> &ap, Layout<3> &L, cudaStream_t stream)
{
   if constexpr (is_half<T>) {
      if (L.ndims == 1 && L.nelem >= 8 && L.stride[0][0] == 2 && L.stride[1][0] == 2 && L.stride[2][0] == 2 &&
          aligned_to(L.ptr[0], 16) && aligned_to(L.ptr[1], 16) && aligned_to(L.ptr[2], 16)) {
         const uint64_t nvec = (uint64_t)L.nelem / 8;
         const uint64_t blocks = (nvec + EW_THREADS * AXH_U - 1) / (EW_THREADS * AXH_U);
         if (blocks <= 0x7FFFFFFFull) {
            axpy_half_dense<AXH_U><<<(unsigned)blocks, EW_THREADS, 0, stream>>>(
               ap, (const uint4 *)L.ptr[0], (const uint4 *)L.ptr[1], (uint4 *)L.ptr[2], nvec);
            SD_LAUNCH_CHECK();
            const int64_t done = (int64_t)(nvec * 8);
            for (int k = 0; k < 3; k++) L.ptr[k] += done * 2;
            L.size[0] -= done; L.nelem -= done;
         }
      }
   }
   return 0;
}
} // namespace sd
SD_WHEN(real)(
extern "C" int SD_PASTE(solid_gpu_axpy_, SDX)(SOLID_GPU_ARGS_AXPY)
{
   const ptrdiff_t *st[3] = { strides1, strides2, strides3 }; void *pt[3] = { ptr1, ptr2, ptr3 };
   sd::Layout<3> L;
   if (sd::make_layout<3>(L, ndims, size, st, pt, 2) != 0) return -1;
   sd::AxpyApply<T> ap; memcpy(&ap.a, &a, sizeof(T));
   if (sd::axpy_dense_part<T>(ap, L, stream) != 0) return -1;
   if (L.nelem == 0) return 0;
   return sd::ew_launch(ap, L, stream);
})
