// solid_gpu_steps_{int64,double,cdouble}_<SDX>: tensor[i] = offset + i * step, with i the position of the
// element in the column-major order of the tensor's own dimensions (Ocean's range / linspace).
// Replaces solid/src/core/gpu/template_steps.cu:30-122 for one element type; the values follow the CPU file
// solid/src/core/cpu/template_steps.c:27-92 (the parity oracle): the position is a size_t there, so the int64
// form evaluates offset + i * step in unsigned 64-bit arithmetic before the cast to the element's work type,
// and the double form multiplies and adds in double without contraction.
#include "unit.cuh"
#include "layout.h"

namespace sd {

struct StepsInt64   { int64_t offset, step; };
struct StepsDouble  { double offset, step; };
struct StepsCDouble { double offset_re, offset_im, step_re, step_im; };

struct StepsParams {
   char    *dst;
   int64_t  index0;                    // position of the element at dst (not 0 once reversed dimensions were flipped)
   int      ndims;
   int64_t  size[MAXD], dstride[MAXD], istride[MAXD];
   uint64_t total;                     // threads: elements, or vectors along dimension 0
};

template <class E> SD_D E steps_zero() { if constexpr (is_half<E>) { Half h; h.v = 0; return h; } else return (E)0; }

// (element type)(work type)(unsigned 64-bit value)
template <class E> SD_D E steps_cast(uint64_t u)
{
   if constexpr (is_bool<E>) { Bool r; r.v = (uint8_t)u; return r; }
   else if constexpr (is_half<E>) return float_to_half((float)u);
   else return (E)u;
}
// (element type)(work type)(double value); integers convert as the x86 truncating instructions do
template <class E> SD_D E steps_cast(double d)
{
   if constexpr (is_bool<E>) { Bool r; r.v = float_to_int<uint8_t, double>(d); return r; }
   else if constexpr (is_half<E>) return float_to_half((float)d);
   else if constexpr (std::is_integral<E>::value) return float_to_int<E, double>(d);
   else return (E)d;
}

template <class T> SD_D T steps_value(uint64_t i, const StepsInt64 &s)
{
   const uint64_t u = (uint64_t)s.offset + i * (uint64_t)s.step;
   if constexpr (is_cplx<T>) { T r; r.re = steps_cast<elem_t<T>>(u); r.im = steps_zero<elem_t<T>>(); return r; }
   else return steps_cast<T>(u);
}
template <class T> SD_D T steps_value(uint64_t i, const StepsDouble &s)
{
   const double p = (double)i * s.step;
   const double d = s.offset + p;
   if constexpr (is_cplx<T>) { T r; r.re = steps_cast<elem_t<T>>(d); r.im = steps_zero<elem_t<T>>(); return r; }
   else return steps_cast<T>(d);
}
template <class T> SD_D T steps_value(uint64_t i, const StepsCDouble &s)
{
   const double pr = (double)i * s.step_re, pi = (double)i * s.step_im;
   if constexpr (is_cplx<T>) { T r; r.re = steps_cast<elem_t<T>>(s.offset_re + pr); r.im = steps_cast<elem_t<T>>(s.offset_im + pi); return r; }
   else return steps_cast<T>(s.offset_re + pr);
}

template <class T, class P, int VEC>
__global__ void __launch_bounds__(256) steps_kernel(const StepsParams p, const P param)
{
   const uint64_t t = (uint64_t)blockIdx.x * 256 + threadIdx.x;
   if (t >= p.total) return;
   uint64_t r = t;
   int64_t doff = 0, ioff = p.index0;
   for (int d = 0; d < p.ndims - 1; d++) {
      const uint64_t n = (uint64_t)(d == 0 ? p.size[0] / VEC : p.size[d]);
      const uint64_t q = udiv64(r, n), c = r - q * n; r = q;
      doff += (int64_t)c * (d == 0 ? p.dstride[0] * VEC : p.dstride[d]);
      ioff += (int64_t)c * (d == 0 ? p.istride[0] * VEC : p.istride[d]);
   }
   {  const int d = p.ndims - 1;
      doff += (int64_t)r * (d == 0 ? p.dstride[0] * VEC : p.dstride[d]);
      ioff += (int64_t)r * (d == 0 ? p.istride[0] * VEC : p.istride[d]);
   }
   Vec<T, VEC> v;
#pragma unroll
   for (int j = 0; j < VEC; j++) v.v[j] = steps_value<T>((uint64_t)(ioff + (int64_t)j * p.istride[0]), param);
   st_vec<T, VEC>(p.dst + doff, v);
}

template <class T, class P>
int launch_steps(int ndims, const size_t *size, const ptrdiff_t *strides, void *ptr, const P &param, cudaStream_t stream)
{
   constexpr int VEC = 16 / (int)sizeof(T) > 0 ? 16 / (int)sizeof(T) : 1;
   if (ndims < 0 || ndims > MAXD) SD_ERROR("Number of dimensions (%d) exceeds the maximum of %d", ndims, MAXD);
   // The position is carried through the layout normalisation as a second operand whose "address" is the
   // position itself: stride of dimension d = product of the sizes before it, base 0.
   ptrdiff_t pos[MAXD]; ptrdiff_t run = 1;
   for (int d = 0; d < ndims; d++) { pos[d] = run; run *= (ptrdiff_t)size[d]; }
   const ptrdiff_t *st[2] = { pos, strides }; void *pt[2] = { nullptr, ptr };
   Layout<2> L;
   if (make_layout<2>(L, ndims, size, st, pt, 1) != 0) return -1;
   if (L.nelem == 0) return 0;
   if (!aligned_to(L.ptr[1], sizeof(T))) SD_ERROR("Tensor data must be aligned to the element size");
   StepsParams p; memset(&p, 0, sizeof(p));
   p.dst = L.ptr[1]; p.index0 = (int64_t)(intptr_t)L.ptr[0]; p.ndims = L.ndims;
   bool vec = VEC > 1 && L.stride[1][0] == (int64_t)sizeof(T) && L.size[0] % VEC == 0 && aligned_to(L.ptr[1], 16);
   for (int d = 0; d < L.ndims; d++) {
      p.size[d] = L.size[d]; p.istride[d] = L.stride[0][d]; p.dstride[d] = L.stride[1][d];
      if (d > 0 && L.stride[1][d] % 16 != 0) vec = false;
   }
   p.total = (uint64_t)L.nelem / (vec ? VEC : 1);
   const uint64_t blocks = (p.total + 255) / 256;
   if (blocks > 0x7FFFFFFFull) SD_ERROR("steps: tensor too large for one launch");
   if (vec) steps_kernel<T, P, VEC><<<(unsigned)blocks, 256, 0, stream>>>(p, param);
   else     steps_kernel<T, P, 1><<<(unsigned)blocks, 256, 0, stream>>>(p, param);
   SD_LAUNCH_CHECK();
   return 0;
}

} // namespace sd

extern "C" int SD_PASTE(solid_gpu_steps_int64_, SDX)(SOLID_GPU_ARGS_STEPS_INT64)
{  sd::StepsInt64 s = { offset, step };
   return sd::launch_steps<T>(ndims, size, strides, ptr, s, stream); }
extern "C" int SD_PASTE(solid_gpu_steps_double_, SDX)(SOLID_GPU_ARGS_STEPS_DOUBLE)
{  sd::StepsDouble s = { offset, step };
   return sd::launch_steps<T>(ndims, size, strides, ptr, s, stream); }
SD_WHEN(complex)(
extern "C" int SD_PASTE(solid_gpu_steps_cdouble_, SDX)(SOLID_GPU_ARGS_STEPS_CDOUBLE)
{  sd::StepsCDouble s = { offset.real, offset.imag, step.real, step.imag };
   return sd::launch_steps<T>(ndims, size, strides, ptr, s, stream); })
