// Element types of the Solid tables, their work types and the conversions
// between them, as device code.
//
// Semantics follow the CPU side of the reference (the parity oracle):
//   work types        solid/include/solid/base/cpu/dtype_cpu.h:61-63   (bool->bool, half->float, chalf->cfloat)
//   conversions       solid/include/solid/base/generic/dtype_assign.h:99-163
//   half <-> float    solid/src/base/generic/half.c:26-149  (NOT IEEE round-to-nearest-even, see below)
//   byte reversal     solid/include/solid/base/generic/dtype_assign.h:55-83,171-214
#pragma once
#include <cstdint>
#include <cstddef>
#include <type_traits>
#include <cuda_runtime.h>
#include <cuda_fp16.h>

namespace sd {

#define SD_HD __host__ __device__ __forceinline__
#define SD_D  __device__ __forceinline__

// 64-bit unsigned division is a long emulated sequence on the GPU; nearly every quotient the
// kernels need has both operands below 2^32, where a single 32-bit division does.
SD_D uint64_t udiv64(uint64_t a, uint64_t b)
{
   if (((a | b) >> 32) == 0) return (uint32_t)a / (uint32_t)b;
   return a / b;
}

// Distinct C++ types for the fifteen table indices.  bool and half share a
// representation with uint8/uint16 but not their semantics, so they are wrapped.
struct Bool { uint8_t v; };
struct Half { uint16_t v; };
template <class R> struct Cplx { R re, im; };
using CHalf   = Cplx<Half>;
using CFloat  = Cplx<float>;
using CDouble = Cplx<double>;

using t_bool = Bool;        using t_uint8 = uint8_t;   using t_uint16 = uint16_t;
using t_uint32 = uint32_t;  using t_uint64 = uint64_t; using t_int8 = int8_t;
using t_int16 = int16_t;    using t_int32 = int32_t;   using t_int64 = int64_t;
using t_half = Half;        using t_float = float;     using t_double = double;
using t_chalf = CHalf;      using t_cfloat = CFloat;   using t_cdouble = CDouble;

enum Kind { K_BOOL = 0, K_UINT = 1, K_SINT = 2, K_REAL = 3, K_CPLX = 4 };

template <class T> struct traits;
#define SD_TRAITS(T, IDX, KIND, WORK, ELEM)                                            \
   template <> struct traits<T> {                                                      \
      static constexpr int index = IDX; static constexpr Kind kind = KIND;             \
      using work = WORK; using elem = ELEM; };
SD_TRAITS(Bool,     0,  K_BOOL, uint8_t,  Bool)
SD_TRAITS(uint8_t,  1,  K_UINT, uint8_t,  uint8_t)
SD_TRAITS(uint16_t, 2,  K_UINT, uint16_t, uint16_t)
SD_TRAITS(uint32_t, 3,  K_UINT, uint32_t, uint32_t)
SD_TRAITS(uint64_t, 4,  K_UINT, uint64_t, uint64_t)
SD_TRAITS(int8_t,   5,  K_SINT, int8_t,   int8_t)
SD_TRAITS(int16_t,  6,  K_SINT, int16_t,  int16_t)
SD_TRAITS(int32_t,  7,  K_SINT, int32_t,  int32_t)
SD_TRAITS(int64_t,  8,  K_SINT, int64_t,  int64_t)
SD_TRAITS(Half,     9,  K_REAL, float,    Half)
SD_TRAITS(float,    10, K_REAL, float,    float)
SD_TRAITS(double,   11, K_REAL, double,   double)
SD_TRAITS(CHalf,    12, K_CPLX, CFloat,   Half)
SD_TRAITS(CFloat,   13, K_CPLX, CFloat,   float)
SD_TRAITS(CDouble,  14, K_CPLX, CDouble,  double)
#undef SD_TRAITS

template <class T> constexpr bool is_bool   = traits<T>::kind == K_BOOL;
template <class T> constexpr bool is_uint   = traits<T>::kind == K_UINT;
template <class T> constexpr bool is_sint   = traits<T>::kind == K_SINT;
template <class T> constexpr bool is_int    = is_uint<T> || is_sint<T>;
template <class T> constexpr bool is_real   = traits<T>::kind == K_REAL;
template <class T> constexpr bool is_cplx   = traits<T>::kind == K_CPLX;
template <class T> constexpr bool is_half   = std::is_same<T, Half>::value;
template <class T> using work_t = typename traits<T>::work;
template <class T> using elem_t = typename traits<T>::elem;       // component type of a complex
template <class T> using ework_t = work_t<elem_t<T>>;              // its work type

// ---------------------------------------------------------------------------
// half <-> float, bit for bit as solid/src/base/generic/half.c
// ---------------------------------------------------------------------------
// half -> float is exact, except that -0 becomes +0 (half.c:37-39 tests the
// magnitude for zero after the sign was stripped and returns a literal 0).
SD_HD float half_to_float(Half hh)
{
#ifdef __CUDA_ARCH__
   // the hardware conversion is exact for zero, subnormal and normal inputs; only the
   // two deviations of half.c are patched in: +-0 -> +0, and inf/nan rebuilt from the bits
   const uint32_t h = hh.v;
   float f = __half2float(__ushort_as_half(hh.v)) + 0.0f;              // -0 + +0 = +0, every other value unchanged
   if ((h & 0x7C00u) == 0x7C00u) f = __uint_as_float(((h & 0x8000u) << 16) | 0x7F800000u | ((h & 0x03FFu) << 13));
   return f;
#else
   uint32_t h = hh.v;
   uint32_t s = (h & 0x8000u) << 16;
   h &= 0x7FFFu;
   if (h == 0) return 0.0f;
   uint32_t e = h & 0x7C00u, d;
   if (e == 0) {                       // subnormal: normalise
      uint32_t shift = 1; h <<= 1;
      while (!(h & 0x0400u)) { shift++; h <<= 1; }
      d = ((h & 0xFFFFu) << 13) + ((112u - shift) << 23);
   } else if (e == 0x7C00u) {          // inf / nan keep their payload
      d = (h << 13) | 0x7F800000u;
   } else {
      d = (h << 13) + 0x38000000u;
   }
   d |= s;
   float f; __builtin_memcpy(&f, &d, 4); return f;
#endif
}

// float -> half as half.c:101-149: magnitudes below 2^-15 (biased exponent < 112)
// give +0 with the sign dropped; exponents 112..143 are re-biased by a plain
// subtraction (so 2^-15..2^-14 and 65536..131072 are encoded "as is", the
// latter running into the inf/nan patterns); the 13 dropped mantissa bits round
// half AWAY from zero (>= 0x1000 adds one); exponent >= 144 gives +-inf; NaN
// gives 0x7F00.
// general form, branch free: the regular encoding (16-bit wrap-around included), then the overrides
SD_HD uint32_t float_to_half_bits(uint32_t raw)
{
   const uint32_t d = raw & 0x007FFFFFu;
   const uint32_t e = (raw >> 23) & 0xFFu;
   const uint32_t s = (raw >> 16) & 0x8000u;
   uint32_t x = ((((e - 112u) << 10) | (d >> 13) | s) + ((d & 0x1FFFu) >= 0x1000u ? 1u : 0u)) & 0xFFFFu;
   const uint32_t special = (e == 255u && d != 0) ? 0x7F00u : (s | 0x7C00u);
   x = (e > 143u) ? special : x;
   x = (e < 112u) ? 0u : x;
   return x;
}
#ifdef __CUDACC__
// Out of line on the device: values outside the normal half range are rare, and keeping this code out of the
// unrolled element loops keeps those loops inside the instruction cache.
__device__ __noinline__ inline uint32_t float_to_half_bits_rare(uint32_t raw) { return float_to_half_bits(raw); }
#endif

SD_HD Half float_to_half(float f)
{
   uint32_t raw;
#ifdef __CUDA_ARCH__
   raw = __float_as_uint(f);
   // Normal half range (biased float exponent 113..142): half.c rounds the 13 dropped mantissa bits half away
   // from zero, which on the float bits is "add half a unit, clear the bits"; the value is then exactly
   // representable and the hardware conversion only re-biases it.  A carry out of the mantissa into the
   // exponent behaves the same in both encodings.
   const uint32_t e = (raw >> 23) & 0xFFu;
   Half r;
   if (e - 113u < 30u)        r.v = __half_as_ushort(__float2half_rn(__uint_as_float((raw + 0x1000u) & 0xFFFFE000u)));
   else if ((raw << 1) == 0u) r.v = 0;                                // +-0 -> +0 (zeros are common, keep them inline)
   else                       r.v = (uint16_t)float_to_half_bits_rare(raw);
   return r;
#else
   __builtin_memcpy(&raw, &f, 4);
   Half r; r.v = (uint16_t)float_to_half_bits(raw);
   return r;
#endif
}

// ---------------------------------------------------------------------------
// float/double -> integer with the results the oracle's x86-64 build gives.
// Out-of-range casts are undefined in C; gcc emits cvttss2si/cvttsd2si, whose
// out-of-range answer is the "integer indefinite" 0x80..0, on a 32-bit
// register for targets up to 32 bits signed and on a 64-bit register for
// uint32 and the 64-bit targets, then keeps the low bytes.
// ---------------------------------------------------------------------------
template <class F> SD_D int32_t x86_cvtt32(F x)
{  return (x >= (F)-2147483648.0 && x < (F)2147483648.0) ? (int32_t)x : (int32_t)0x80000000; }
template <class F> SD_D int64_t x86_cvtt64(F x)
{  return (x >= (F)-9223372036854775808.0 && x < (F)9223372036854775808.0) ? (int64_t)x
                                                                          : (int64_t)0x8000000000000000ull; }
template <class I, class F> SD_D I float_to_int(F x)
{
   if constexpr (std::is_same<I, uint64_t>::value) {
      if (x >= (F)9223372036854775808.0)
         return (uint64_t)x86_cvtt64<F>(x - (F)9223372036854775808.0) ^ 0x8000000000000000ull;
      return (uint64_t)x86_cvtt64<F>(x);
   } else if constexpr (std::is_same<I, int64_t>::value || std::is_same<I, uint32_t>::value) {
      return (I)x86_cvtt64<F>(x);
   } else {
      return (I)x86_cvtt32<F>(x);
   }
}

// ---------------------------------------------------------------------------
// convert<D>(S): one element, solid/include/solid/base/generic/dtype_assign.h:109-163,222-288
// ---------------------------------------------------------------------------
template <class D, class S> SD_D D convert(S x);

// real -> real
template <class D, class S> SD_D D convert_real(S x)
{
   if constexpr (std::is_same<D, S>::value) {
      return x;                                              // raw copy, bool bytes included
   } else if constexpr (is_bool<D>) {
      Bool r;
      if constexpr (is_half<S>) r.v = ((x.v & 0x7FFFu) == 0) ? 0 : 1;
      else                      r.v = (x == 0) ? 0 : 1;      // NaN -> 1
      return r;
   } else if constexpr (is_bool<S>) {
      if constexpr (is_half<D>) return float_to_half((float)x.v);
      else                      return (D)x.v;
   } else if constexpr (is_half<D>) {
      return float_to_half((float)x);                        // double -> float rounds first
   } else if constexpr (is_half<S>) {
      return convert_real<D, float>(half_to_float(x));
   } else if constexpr (std::is_floating_point<S>::value && std::is_integral<D>::value) {
      return float_to_int<D, S>(x);
   } else {
      return (D)x;
   }
}

template <class D, class S> SD_D D convert(S x)
{
   if constexpr (std::is_same<D, S>::value) {
      return x;
   } else if constexpr (is_cplx<S> && is_cplx<D>) {
      D r; r.re = convert_real<elem_t<D>>(x.re); r.im = convert_real<elem_t<D>>(x.im); return r;
   } else if constexpr (is_cplx<S> && is_bool<D>) {
      Bool r; r.v = (convert_real<Bool>(x.re).v || convert_real<Bool>(x.im).v) ? 1 : 0; return r;
   } else if constexpr (is_cplx<S>) {
      return convert_real<D>(x.re);                          // imaginary part discarded
   } else if constexpr (is_cplx<D>) {
      D r; r.re = convert_real<elem_t<D>>(x);
      if constexpr (is_half<elem_t<D>>) r.im.v = 0; else r.im = 0;
      return r;
   } else {
      return convert_real<D>(x);
   }
}

// work type <-> storage type
template <class T> SD_D work_t<T> to_work(T x)
{
   if constexpr (is_bool<T>) return x.v;
   else if constexpr (is_half<T>) return half_to_float(x);
   else if constexpr (std::is_same<T, CHalf>::value) { CFloat r; r.re = half_to_float(x.re); r.im = half_to_float(x.im); return r; }
   else return x;
}
template <class T> SD_D T from_work(work_t<T> w)
{
   if constexpr (is_bool<T>) { Bool r; r.v = w; return r; }
   else if constexpr (is_half<T>) return float_to_half(w);
   else if constexpr (std::is_same<T, CHalf>::value) { CHalf r; r.re = float_to_half(w.re); r.im = float_to_half(w.im); return r; }
   else return w;
}
// one real component (used by the complex operations)
template <class E> SD_D work_t<E> ew(E x) { return to_work<E>(x); }
template <class E> SD_D E few(work_t<E> w) { return from_work<E>(w); }

// ---------------------------------------------------------------------------
// Byte reversal of each real component
// ---------------------------------------------------------------------------
SD_D uint16_t bswap16(uint16_t x) { return (uint16_t)((x << 8) | (x >> 8)); }
SD_D uint32_t bswap32(uint32_t x) { return __byte_perm(x, 0, 0x0123); }
SD_D uint64_t bswap64(uint64_t x)
{  return ((uint64_t)bswap32((uint32_t)x) << 32) | bswap32((uint32_t)(x >> 32)); }

template <int N> struct raw_of;
template <> struct raw_of<1> { using type = uint8_t; };
template <> struct raw_of<2> { using type = uint16_t; };
template <> struct raw_of<4> { using type = uint32_t; };
template <> struct raw_of<8> { using type = uint64_t; };

template <class R> SD_D R bswap_real(R x)
{
   if constexpr (sizeof(R) == 1) return x;
   else {
      typename raw_of<sizeof(R)>::type u;
      memcpy(&u, &x, sizeof(R));
      if constexpr (sizeof(R) == 2) u = bswap16(u);
      else if constexpr (sizeof(R) == 4) u = bswap32(u);
      else u = bswap64(u);
      memcpy(&x, &u, sizeof(R));
      return x;
   }
}
template <class T> SD_D T bswap(T x)
{
   if constexpr (is_cplx<T>) { x.re = bswap_real(x.re); x.im = bswap_real(x.im); return x; }
   else return bswap_real(x);
}

// ---------------------------------------------------------------------------
// N consecutive elements moved with the widest global accesses available
// (128-bit where N*sizeof(T) >= 16).  Streaming hints (ld.global.cs /
// st.global.cs) mark the data evict-first: every tensor here is read or written
// once per call, so it should not displace anything from L2.
// ---------------------------------------------------------------------------
template <class T, int N> struct Vec { T v[N]; };

template <int B> struct chunk_of;
template <> struct chunk_of<16> { using type = uint4; };
template <> struct chunk_of<8>  { using type = uint2; };
template <> struct chunk_of<4>  { using type = uint32_t; };
template <> struct chunk_of<2>  { using type = uint16_t; };
template <> struct chunk_of<1>  { using type = uint8_t; };

template <class T, int N> SD_D Vec<T, N> ld_vec(const void *p)
{
   constexpr int B = (int)sizeof(T) * N;
   constexpr int C = B >= 16 ? 16 : B;
   static_assert(B % C == 0 && (C & (C - 1)) == 0, "vector bytes must be a power of two or a multiple of 16");
   using chunk = typename chunk_of<C>::type;
   Vec<T, N> o;
#pragma unroll
   for (int i = 0; i < B / C; i++) {
      chunk r = __ldcs(reinterpret_cast<const chunk *>(p) + i);
      memcpy(reinterpret_cast<char *>(&o) + i * C, &r, C);
   }
   return o;
}
template <class T, int N> SD_D void st_vec(void *p, const Vec<T, N> &x)
{
   constexpr int B = (int)sizeof(T) * N;
   constexpr int C = B >= 16 ? 16 : B;
   using chunk = typename chunk_of<C>::type;
#pragma unroll
   for (int i = 0; i < B / C; i++) {
      chunk r;
      memcpy(&r, reinterpret_cast<const char *>(&x) + i * C, C);
      __stcs(reinterpret_cast<chunk *>(p) + i, r);
   }
}
template <class T> SD_D T ld_one(const void *p) { return ld_vec<T, 1>(p).v[0]; }
template <class T> SD_D void st_one(void *p, T x) { Vec<T, 1> v; v.v[0] = x; st_vec<T, 1>(p, v); }

} // namespace sd
