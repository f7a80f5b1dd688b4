// Type-converting copies FROM one element type (SDX) to each of the fifteen:
// solid_gpu_copy_<SDX>_<dst>, solid_gpu_copy_regular_<SDX>_<dst> and the
// byte-order variants.  Replaces solid/src/core/gpu/template_copy.cu:31-86 (which
// has neither byte reversal nor unaligned access; those follow the CPU file
// solid/src/core/cpu/template_copy.c:79-89 and dtype_assign.h:297-371).
//
// Conversion and byte reversal happen in registers between the load and the
// store, so a converting copy moves sizeof(src)+sizeof(dst) bytes per element.
#include "unit.cuh"
#include "elemwise.cuh"

namespace sd {

template <class S, class D> struct ConvertApply {
   static constexpr int NIN = 1;
   using in1_t = S; using in2_t = Nothing; using out_t = D;
   int swap_src, swap_dst;
   SD_D D operator()(S x, Nothing) const
   {
      if (swap_src) x = bswap<S>(x);
      D y = convert<D, S>(x);
      if (swap_dst) y = bswap<D>(y);
      return y;
   }
};

// Copy between tensors of different shape and equal element count: element i of
// the source (column-major order of ITS shape) goes to element i of the
// destination (column-major order of its own shape).
struct ReshapeParams {
   char    *src, *dst;
   int      nd1, nd2;
   int64_t  size1[MAXD], stride1[MAXD], size2[MAXD], stride2[MAXD];
   uint64_t nelem;
   uint32_t unal;
};

template <class A, bool UNAL>
__global__ void __launch_bounds__(EW_THREADS) ew_reshape(const A apply, const ReshapeParams p)
{
   using S = typename A::in1_t; using D = typename A::out_t;
   for (uint64_t idx = (uint64_t)blockIdx.x * EW_THREADS + threadIdx.x; idx < p.nelem;
        idx += (uint64_t)gridDim.x * EW_THREADS) {
      int64_t o1 = 0, o2 = 0;
      uint64_t r = idx;
      for (int d = 0; d < p.nd1 - 1; d++) { uint64_t q = udiv64(r, (uint64_t)p.size1[d]); o1 += (int64_t)(r - q * p.size1[d]) * p.stride1[d]; r = q; }
      o1 += (int64_t)r * p.stride1[p.nd1 - 1];
      r = idx;
      for (int d = 0; d < p.nd2 - 1; d++) { uint64_t q = udiv64(r, (uint64_t)p.size2[d]); o2 += (int64_t)(r - q * p.size2[d]) * p.stride2[d]; r = q; }
      o2 += (int64_t)r * p.stride2[p.nd2 - 1];
      Vec<S, 1> a = ew_load<S, 1, UNAL>(p.src + o1, false, p.unal & 1u);
      Vec<D, 1> o; o.v[0] = apply(a.v[0], Nothing());
      ew_store<D, 1, UNAL>(p.dst + o2, o, p.unal & 2u);
   }
}

// drop unit dimensions and merge neighbours that are jointly contiguous (order kept)
static int squeeze(int ndims, const size_t *size, const ptrdiff_t *strides, int64_t *osize, int64_t *ostride, uint64_t *nelem)
{
   int n = 0; uint64_t ne = 1;
   for (int i = 0; i < ndims; i++) {
      ne *= size[i];
      if (size[i] == 1) continue;
      if (n > 0 && strides[i] == ostride[n - 1] * osize[n - 1]) { osize[n - 1] *= (int64_t)size[i]; continue; }
      osize[n] = (int64_t)size[i]; ostride[n] = strides[i]; n++;
   }
   if (n == 0) { osize[0] = 1; ostride[0] = 0; n = 1; }
   *nelem = ne;
   return n;
}

template <class S, class D>
int copy_regular(int flags, int ndims, const size_t *size, const ptrdiff_t *strides1, void *ptr1,
                 const ptrdiff_t *strides2, void *ptr2, cudaStream_t stream)
{
   const ptrdiff_t *st[2] = { strides1, strides2 }; void *pt[2] = { ptr1, ptr2 };
   Layout<2> L;
   if (make_layout<2>(L, ndims, size, st, pt, 1) != 0) return -1;
   ConvertApply<S, D> a; a.swap_src = (flags & SOLID_GPU_COPY_SRC_SWAPPED) ? 1 : 0;
   a.swap_dst = (flags & SOLID_GPU_COPY_DST_SWAPPED) ? 1 : 0;
   return ew_launch<ConvertApply<S, D>, true>(a, L, stream);
}

template <class S, class D>
int copy_general(int flags, int ndims1, const size_t *size1, const ptrdiff_t *strides1, void *ptr1,
                 int ndims2, const size_t *size2, const ptrdiff_t *strides2, void *ptr2, cudaStream_t stream)
{
   if (ndims1 > MAXD || ndims2 > MAXD || ndims1 < 0 || ndims2 < 0)
      SD_ERROR("Number of dimensions exceeds the maximum of %d", MAXD);
   // same shape (or a scalar on either side with the other holding one element): regular copy
   bool regular = (ndims1 == ndims2);
   if (regular) for (int i = 0; i < ndims1; i++) if (size1[i] != size2[i]) { regular = false; break; }
   if (regular) return copy_regular<S, D>(flags, ndims1, size1, strides1, ptr1, strides2, ptr2, stream);

   ReshapeParams p; memset(&p, 0, sizeof(p));
   uint64_t n1, n2;
   p.nd1 = squeeze(ndims1, size1, strides1, p.size1, p.stride1, &n1);
   p.nd2 = squeeze(ndims2, size2, strides2, p.size2, p.stride2, &n2);
   if (n1 != n2) SD_ERROR("Mismatch in the number of elements in tensor copy (%llu vs %llu)",
                          (unsigned long long)n1, (unsigned long long)n2);
   if (n1 == 0) return 0;
   if (p.nd1 == 1 && p.nd2 == 1) {                      // both sides are single runs: reuse the fast path
      size_t sz = (size_t)n1; ptrdiff_t s1 = p.stride1[0], s2 = p.stride2[0];
      return copy_regular<S, D>(flags, 1, &sz, &s1, ptr1, &s2, ptr2, stream);
   }
   p.src = (char *)ptr1; p.dst = (char *)ptr2; p.nelem = n1;
   auto misaligned = [](const void *ptr, const int64_t *stride, int nd, int es) {
      if (!aligned_to(ptr, (size_t)es)) return true;
      for (int d = 0; d < nd; d++) if (stride[d] % es != 0) return true;
      return false;
   };
   if (misaligned(ptr1, p.stride1, p.nd1, (int)sizeof(S))) p.unal |= 1u;
   if (misaligned(ptr2, p.stride2, p.nd2, (int)sizeof(D))) p.unal |= 2u;
   ConvertApply<S, D> a; a.swap_src = (flags & SOLID_GPU_COPY_SRC_SWAPPED) ? 1 : 0;
   a.swap_dst = (flags & SOLID_GPU_COPY_DST_SWAPPED) ? 1 : 0;
   DeviceInfo dev;
   if (current_device_info(&dev) != 0) return -1;
   int grid = ew_grid(n1, EW_THREADS, dev);
   if (p.unal) ew_reshape<ConvertApply<S, D>, true><<<grid, EW_THREADS, 0, stream>>>(a, p);
   else        ew_reshape<ConvertApply<S, D>, false><<<grid, EW_THREADS, 0, stream>>>(a, p);
   SD_LAUNCH_CHECK();
   return 0;
}

} // namespace sd

#define SD_SRCDST(PREFIX, DST) SD_PASTE(SD_PASTE(SD_PASTE(PREFIX, SDX), _), DST)

#define SD_DEFINE_COPY(UNUSED, DST)                                                              \
   extern "C" int SD_SRCDST(solid_gpu_copy_regular_, DST)(SOLID_GPU_ARGS_UNARY)                   \
   {  return sd::copy_regular<T, SD_T(DST)>(0, ndims, size, strides1, ptr1, strides2, ptr2, stream); } \
   extern "C" int SD_SRCDST(solid_gpu_copy_, DST)(SOLID_GPU_ARGS_COPY)                            \
   {  return sd::copy_general<T, SD_T(DST)>(0, ndims1, size1, strides1, ptr1,                     \
                                            ndims2, size2, strides2, ptr2, stream); }             \
   extern "C" int SD_SRCDST(solid_gpu_byteswap_copy_, DST)(SOLID_GPU_ARGS_COPY)                   \
   {  return sd::copy_general<T, SD_T(DST)>(SOLID_GPU_COPY_SRC_SWAPPED, ndims1, size1, strides1, ptr1, \
                                            ndims2, size2, strides2, ptr2, stream); }
SOLID_TYPES2_all(SD_DEFINE_COPY, unused)

// row SDX of the table behind solid_gpu_copy_ex
#define SD_COPY_EX_CASE(UNUSED, DST)                                                             \
   case sd::traits<SD_T(DST)>::index:                                                            \
      return sd::copy_general<T, SD_T(DST)>(flags, ndims1, size1, strides1, ptr1,                \
                                            ndims2, size2, strides2, ptr2, stream);
extern "C" int SD_PASTE(solid_gpu_copy_ex_from_, SDX)(int dsttype, int flags, SOLID_GPU_ARGS_COPY)
{
   switch (dsttype) {
      SOLID_TYPES2_all(SD_COPY_EX_CASE, unused)
      default: SD_ERROR("Invalid destination type index %d", dsttype);
   }
}
