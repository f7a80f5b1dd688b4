// Host-side tensor layout normalisation and launch helpers shared by all kernels.
//
// Ocean normally simplifies layouts before calling Solid (drop unit dimensions,
// flip negative destination strides, sort by destination stride, merge jointly
// contiguous dimensions: src/external/ocean-solid/ocean_solid.c:260-329 and
// src/base/shape.c:292-325,380-412).  The same steps are repeated here because
// they cost microseconds and let a direct caller of the C-ABI reach the
// vectorised kernels with any equivalent description of the same memory.
#pragma once
#include <cstdint>
#include <cstddef>
#include <cstdio>
#include <cstring>
#include <algorithm>
#include <cuda_runtime.h>
#include "solid_gpu_types.h"

extern "C" char *solid_errmsg;

#define SD_ERROR(...) \
   do { snprintf(solid_errmsg, SOLID_ERRMSG_SIZE, __VA_ARGS__); return -1; } while (0)

#define SD_CUDA_CHECK(EXPR) \
   do { cudaError_t e__ = (EXPR); \
        if (e__ != cudaSuccess) SD_ERROR("Cuda error: %s", cudaGetErrorString(e__)); } while (0)

// Every launch is followed by this (the reference checks cudaGetLastError after
// each kernel, solid/include/solid/core/gpu/apply_elemwise1.h:219-222).
#define SD_LAUNCH_CHECK() \
   do { cudaError_t e__ = cudaGetLastError(); \
        if (e__ != cudaSuccess) SD_ERROR("Cuda error: %s", cudaGetErrorString(e__)); } while (0)

namespace sd {

constexpr int MAXD = SOLID_MAX_TENSOR_DIMS;

// Unsigned 32-bit division by an invariant divisor: q = (n * m) >> (32 + s)
// for all n < 2^32 (Granlund-Montgomery, round-up variant with a 33-bit
// multiplier folded into an add-shift).
struct FastDiv {
   uint32_t d, m, s;
};
inline FastDiv make_fastdiv(uint32_t d)
{
   FastDiv f; f.d = d ? d : 1;
   uint32_t l = 0; while ((1ull << l) < f.d) l++;
   f.s = l;
   f.m = (uint32_t)((((1ull << l) - f.d) << 32) / f.d + 1);
   return f;
}
#ifdef __CUDACC__
__device__ __forceinline__ uint32_t fastdiv(uint32_t n, const FastDiv &f)
{
   uint32_t t = __umulhi(n, f.m);
   return (uint32_t)((((uint64_t)t + n)) >> f.s);   // (t + n) can carry into bit 32
}
#endif

// A group of NOPS operands over one shared shape.  dim 0 is the innermost
// (smallest destination stride) after normalisation.
template <int NOPS> struct Layout {
   int      ndims;
   int64_t  size[MAXD];
   int64_t  stride[NOPS][MAXD];      // bytes
   char    *ptr[NOPS];
   int64_t  nelem;
};

// Build and simplify.  `dst` is the index of the operand that is written (its
// strides are made positive and drive the ordering), or -1 for read-only groups.
template <int NOPS>
inline int make_layout(Layout<NOPS> &L, int ndims, const size_t *size,
                       const ptrdiff_t *const strides[NOPS], void *const ptr[NOPS], int dst)
{
   if (ndims < 0 || ndims > MAXD) SD_ERROR("Number of dimensions (%d) exceeds the maximum of %d", ndims, MAXD);
   L.nelem = 1; L.ndims = 0;
   for (int k = 0; k < NOPS; k++) L.ptr[k] = (char *)ptr[k];
   for (int i = 0; i < ndims; i++) {
      L.nelem *= (int64_t)size[i];
      if (size[i] == 1) continue;                      // unit dimensions carry no information
      L.size[L.ndims] = (int64_t)size[i];
      for (int k = 0; k < NOPS; k++) L.stride[k][L.ndims] = strides[k][i];
      L.ndims++;
   }
   if (L.nelem == 0) { L.ndims = 0; return 0; }
   // positive destination strides
   int ref = dst >= 0 ? dst : 0;
   for (int i = 0; i < L.ndims; i++) {
      if (L.stride[ref][i] < 0) {
         for (int k = 0; k < NOPS; k++) {
            L.ptr[k] += (L.size[i] - 1) * L.stride[k][i];
            L.stride[k][i] = -L.stride[k][i];
         }
      }
   }
   // sort ascending by the reference operand, ties by the others (insertion sort, <= 8 dims)
   auto less = [&](int a, int b) {
      if (L.stride[ref][a] != L.stride[ref][b]) return L.stride[ref][a] < L.stride[ref][b];
      for (int k = NOPS - 1; k >= 0; k--) {
         int64_t sa = L.stride[k][a] < 0 ? -L.stride[k][a] : L.stride[k][a];
         int64_t sb = L.stride[k][b] < 0 ? -L.stride[k][b] : L.stride[k][b];
         if (sa != sb) return sa < sb;
      }
      return false;
   };
   for (int i = 1; i < L.ndims; i++) {
      for (int j = i; j > 0 && less(j, j - 1); j--) {
         std::swap(L.size[j], L.size[j - 1]);
         for (int k = 0; k < NOPS; k++) std::swap(L.stride[k][j], L.stride[k][j - 1]);
      }
   }
   // merge dimension i+1 into i when every operand steps contiguously across the boundary
   int n = 0;
   for (int i = 0; i < L.ndims; i++) {
      bool merge = n > 0;
      if (merge) for (int k = 0; k < NOPS; k++)
         if (L.stride[k][i] != L.stride[k][n - 1] * L.size[n - 1]) { merge = false; break; }
      if (merge) { L.size[n - 1] *= L.size[i]; }
      else {
         L.size[n] = L.size[i];
         for (int k = 0; k < NOPS; k++) L.stride[k][n] = L.stride[k][i];
         n++;
      }
   }
   L.ndims = n;
   if (L.ndims == 0) {                                  // a single element
      L.ndims = 1; L.size[0] = 1;
      for (int k = 0; k < NOPS; k++) L.stride[k][0] = 0;
   }
   return 0;
}

// Largest byte offset magnitude any operand reaches (decides 32- vs 64-bit index math)
template <int NOPS> inline int64_t max_extent(const Layout<NOPS> &L)
{
   int64_t m = 0;
   for (int k = 0; k < NOPS; k++) {
      int64_t e = 0;
      for (int i = 0; i < L.ndims; i++) {
         int64_t s = L.stride[k][i] < 0 ? -L.stride[k][i] : L.stride[k][i];
         e += (L.size[i] - 1) * s;
      }
      m = std::max(m, e);
   }
   return m;
}

// Device properties of the current device, cached per device.
struct DeviceInfo { int device; int sms; int max_threads_per_sm; };
int current_device_info(DeviceInfo *info);    // defined in base.cu; returns -1 with solid_errmsg set

inline bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

} // namespace sd
