// Elementwise engine: one kernel family for fill (0 inputs), unary, copy/convert
// (1 input) and binary (2 inputs) operations over up to 8 strided dimensions.
//
// It replaces the reference's four macro kernel generators
// (solid/include/solid/core/gpu/apply_elemwise{1,2,2b,3}.h, variant selection in
// solid/src/core/gpu/op/apply_elemwise{1,2,3}.c), which issue one scalar access
// per element and decompose the index with % and / per element.  Here:
//
//   ew_contig   every operand is dense along one merged dimension (or a broadcast
//               scalar): each thread moves VEC elements per operand with 128-bit
//               ld.global.cs / st.global.cs, UNROLL independent vectors in flight,
//               64-bit element counts (2^32 elements and beyond);
//   ew_tiled    a source is dense along another dimension than the destination
//               (transposed views): 32 x 32 tiles staged through shared memory, so
//               both sides are accessed along their dense dimension;
//   ew_strided  general case: the innermost dimension is vectorised when every
//               operand is dense or broadcast along it and rows start on 16-byte
//               boundaries (VEC > 1), otherwise one element per access (VEC == 1);
//               outer dimensions are decomposed with multiply-shift division.
//
// The operation is an "apply" object A with
//     A::out_t, A::in1_t, A::in2_t, A::NIN (0, 1 or 2)
//     out_t A::operator()(in1_t, in2_t) const
// passed by value, so scalar parameters travel in the kernel arguments.
//
// HBM traffic per element = sizeof(out) + sum sizeof(in): every byte is moved once.
#pragma once
#include "dtypes.cuh"
#include "layout.h"

namespace sd {

struct Nothing {};

constexpr int EW_THREADS = 256;
#ifndef EW_CONTIG_THREADS
#define EW_CONTIG_THREADS 256
#endif
constexpr int EWC_THREADS = EW_CONTIG_THREADS;     // block size of the contiguous kernel

template <int NOPS> struct EwParams {
   char    *ptr[NOPS];
   int64_t  stride[NOPS][MAXD];     // bytes; [k][0] is the innermost dimension
   uint32_t size[MAXD];             // size[0] counts VECTORS in the vectorised variant
   FastDiv  div[MAXD];
   int64_t  size64[MAXD];
   int      ndims;
   int      wide;                   // 1: total index count needs 64 bits
   uint64_t total;                  // number of (vector) indices
   uint64_t nelem;                  // number of elements (ew_contig)
   uint32_t bcast;                  // bit k: operand k is constant along dimension 0
   uint32_t unal;                   // bit k: operand k is not aligned to its element size
};

template <class A> struct ew_traits {
   static constexpr int NIN = A::NIN;
   static constexpr int NOPS = NIN + 1;
   using out_t = typename A::out_t;
   using in1_t = typename A::in1_t;
   using in2_t = typename A::in2_t;
   static constexpr int s_out = (int)sizeof(out_t);
   static constexpr int s_in1 = NIN >= 1 ? (int)sizeof(in1_t) : s_out;
   static constexpr int s_in2 = NIN >= 2 ? (int)sizeof(in2_t) : s_out;
   static constexpr int s_min = s_out < s_in1 ? (s_out < s_in2 ? s_out : s_in2) : (s_in1 < s_in2 ? s_in1 : s_in2);
   static constexpr int s_max = s_out > s_in1 ? (s_out > s_in2 ? s_out : s_in2) : (s_in1 > s_in2 ? s_in1 : s_in2);
   // elements per thread-iteration: 16 bytes of the narrowest operand, at most 64 of the widest
   static constexpr int VEC0 = 16 / s_min > 0 ? 16 / s_min : 1;
   static constexpr int VEC = (VEC0 * s_max > 64) ? (64 / s_max > 0 ? 64 / s_max : 1) : VEC0;
   // Independent iterations in flight, as bytes of the widest operand per thread.  Measured on B200 with arrays of
   // 1-3 GB (256 threads, one chunk per block), 64 / 32 / 16 bytes: 4-byte elements 7.0 / 7.0 / 7.2 TB/s on add and
   // 6.8 / 6.2 / 5.4 on sin, so 64; 8- and 16-byte elements 6.2 / 7.0 / 7.1 on add and 6.2 / 6.7 / 5.8 on fabs
   // (the wide forms need 58-64 registers, four blocks per multiprocessor), so 32; 2-byte elements 4.0 / 6.0 / 7.2 on
   // add and 5.6 / 6.5 / 6.0 on negative, 1-byte elements 2.0 / 3.2 / 4.8 and 3.5 / 4.6 / 4.9 (unpacking makes them
   // instruction-bound, more warps hide it), so 16, except 32 for one-source operations on 2-byte elements.
#ifdef EW_FLIGHT_BYTES_FORCED
   static constexpr int FLIGHT = EW_FLIGHT_BYTES_FORCED;
#else
   static constexpr int FLIGHT = s_max >= 8 ? 32 : (s_max == 4 ? 64 : ((s_max == 1 || NIN == 2) ? 16 : 32));
#endif
   static constexpr int UNROLL = (FLIGHT / (VEC * s_max)) > 0 ? (FLIGHT / (VEC * s_max)) : 1;
};

// An apply object may provide   template <int N> Vec<out_t, N> vec(const Vec<in1_t, N> &, const Vec<in2_t, N> &) const
// next to its per-element operator() (announced by  static constexpr bool VECTOR = true): it then sees the
// whole vector of a thread-iteration and can take shortcuts that depend on all of its elements.
// An apply object may also ask for a number of resident blocks per multiprocessor (static constexpr int MIN_BLOCKS).
template <class A, class = void> struct ew_min_blocks { static constexpr int value = 0; };   // 0: no request
template <class A> struct ew_min_blocks<A, std::enable_if_t<(A::MIN_BLOCKS > 0)>> { static constexpr int value = A::MIN_BLOCKS; };
template <class A, class = void> struct has_vector_apply : std::false_type {};
template <class A> struct has_vector_apply<A, std::enable_if_t<A::VECTOR>> : std::true_type {};

// Access to elements that do not start on a multiple of their size (only the copy
// family accepts such tensors).  Loads fetch the aligned 32-bit words that cover
// the bytes and realign them with a funnel shift; the word after the last one is
// touched only when the data really extends into it.  Stores go byte by byte.
template <int NW> SD_D void ld_words_aligned16(const uint4 *q, uint32_t (&w)[NW])
{
#pragma unroll
   for (int i = 0; i < NW / 4; i++) {
      uint4 r = __ldg(q + i);
      w[4 * i] = r.x; w[4 * i + 1] = r.y; w[4 * i + 2] = r.z; w[4 * i + 3] = r.w;
   }
}
template <class T, int N> SD_D Vec<T, N> ld_unaligned(const char *p)
{
   constexpr int B = (int)sizeof(T) * N;
   Vec<T, N> o;
   if constexpr (B % 16 == 0) {
      // B bytes starting anywhere: fetch the B + 16 bytes of the enclosing 16-byte lines with
      // 128-bit loads (the extra line is the next thread's first one, so it comes from cache),
      // then realign.  The word offset 0..3 is the same for every thread of a contiguous copy,
      // so the switch does not diverge.
      const uintptr_t a = reinterpret_cast<uintptr_t>(p);
      const uint4 *q = reinterpret_cast<const uint4 *>(a & ~(uintptr_t)15);
      const uint32_t wo = (uint32_t)(a & 15) >> 2, sh = (uint32_t)(a & 3) * 8;
      constexpr int NW = B / 4;
      uint32_t w[NW + 4];
      if ((a & 15) == 0) { uint32_t t[NW]; ld_words_aligned16<NW>(q, t);
#pragma unroll
         for (int i = 0; i < NW; i++) w[i] = t[i];
         w[NW] = w[NW + 1] = w[NW + 2] = w[NW + 3] = 0; }
      else ld_words_aligned16<NW + 4>(q, w);
      uint32_t r[NW];
      switch (wo) {
         case 0:
#pragma unroll
            for (int i = 0; i < NW; i++) r[i] = __funnelshift_r(w[i], w[i + 1], sh);
            break;
         case 1:
#pragma unroll
            for (int i = 0; i < NW; i++) r[i] = __funnelshift_r(w[i + 1], w[i + 2], sh);
            break;
         case 2:
#pragma unroll
            for (int i = 0; i < NW; i++) r[i] = __funnelshift_r(w[i + 2], w[i + 3], sh);
            break;
         default:
#pragma unroll
            for (int i = 0; i < NW; i++) r[i] = __funnelshift_r(w[i + 3], (i + 4 < NW + 4) ? w[i + 4] : 0u, sh);
            break;
      }
      memcpy(&o, r, B);
   } else if constexpr (B % 4 == 0) {
      const uintptr_t a = reinterpret_cast<uintptr_t>(p);
      const uint32_t *q = reinterpret_cast<const uint32_t *>(a & ~(uintptr_t)3);
      const uint32_t sh = (uint32_t)(a & 3) * 8;
      uint32_t w[B / 4 + 1];
#pragma unroll
      for (int i = 0; i < B / 4; i++) w[i] = __ldg(q + i);
      w[B / 4] = sh ? __ldg(q + B / 4) : 0u;
      uint32_t r[B / 4];
#pragma unroll
      for (int i = 0; i < B / 4; i++) r[i] = __funnelshift_r(w[i], w[i + 1], sh);
      memcpy(&o, r, B);
   } else {
      uint8_t r[B];
#pragma unroll
      for (int i = 0; i < B; i++) r[i] = __ldg(reinterpret_cast<const uint8_t *>(p) + i);
      memcpy(&o, r, B);
   }
   return o;
}
template <class T, int N> SD_D void st_unaligned(char *p, const Vec<T, N> &x)
{
   constexpr int B = (int)sizeof(T) * N;
   uint8_t r[B];
   memcpy(r, &x, B);
#pragma unroll
   for (int i = 0; i < B; i++) reinterpret_cast<uint8_t *>(p)[i] = r[i];
}

template <class T, int VEC, bool UNAL> SD_D Vec<T, VEC> ew_load(const char *p, bool bcast, bool unal)
{
   if (bcast) {
      T x;
      if (UNAL && unal) x = ld_unaligned<T, 1>(p).v[0]; else x = ld_one<T>(p);
      Vec<T, VEC> v;
#pragma unroll
      for (int j = 0; j < VEC; j++) v.v[j] = x;
      return v;
   }
   if (UNAL && unal) return ld_unaligned<T, VEC>(p);
   return ld_vec<T, VEC>(p);
}
template <class T, int VEC, bool UNAL> SD_D void ew_store(char *p, const Vec<T, VEC> &x, bool unal)
{
   if (UNAL && unal) st_unaligned<T, VEC>(p, x); else st_vec<T, VEC>(p, x);
}

// ---------------------------------------------------------------------------
template <class A, bool UNAL>
__global__ void __launch_bounds__(EWC_THREADS, ew_min_blocks<A>::value) ew_contig(const A apply, const EwParams<A::NIN + 1> p)
{
   using X = ew_traits<A>;
   constexpr int VEC = X::VEC, U = X::UNROLL, NIN = X::NIN;
   using out_t = typename X::out_t; using in1_t = typename X::in1_t; using in2_t = typename X::in2_t;
   const uint64_t nvec = p.nelem / VEC;
   const uint64_t chunk = (uint64_t)EWC_THREADS * U;
   const bool b1 = p.bcast & 1u, b2 = p.bcast & 2u;
   const bool u1 = p.unal & 1u, u2 = p.unal & 2u, uo = p.unal & (1u << NIN);
   char *const po = p.ptr[NIN];

   for (uint64_t base = (uint64_t)blockIdx.x * chunk; base < nvec; base += (uint64_t)gridDim.x * chunk) {
      Vec<in1_t, VEC> a[U]; Vec<in2_t, VEC> b[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
         uint64_t i = base + (uint64_t)u * EWC_THREADS + threadIdx.x;
         if (i < nvec) {
            if constexpr (NIN >= 1) a[u] = ew_load<in1_t, VEC, UNAL>(p.ptr[0] + (b1 ? 0 : i * (VEC * sizeof(in1_t))), b1, u1);
            if constexpr (NIN >= 2) b[u] = ew_load<in2_t, VEC, UNAL>(p.ptr[1] + (b2 ? 0 : i * (VEC * sizeof(in2_t))), b2, u2);
         }
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
         uint64_t i = base + (uint64_t)u * EWC_THREADS + threadIdx.x;
         if (i < nvec) {
            Vec<out_t, VEC> o;
            if constexpr (has_vector_apply<A>::value && (VEC > 1)) o = apply.template vec<VEC>(a[u], b[u]);
            else {
#pragma unroll
               for (int j = 0; j < VEC; j++) o.v[j] = apply(a[u].v[j], b[u].v[j]);
            }
            ew_store<out_t, VEC, UNAL>(po + i * (VEC * sizeof(out_t)), o, uo);
         }
      }
   }
   // ragged tail (fewer than VEC elements), one thread each
   if (VEC > 1 && blockIdx.x == 0) {
      uint64_t i = nvec * VEC + threadIdx.x;
      if (i < p.nelem) {
         in1_t x{}; in2_t y{};
         if constexpr (NIN >= 1) x = ew_load<in1_t, 1, UNAL>(p.ptr[0] + (b1 ? 0 : i * sizeof(in1_t)), false, u1).v[0];
         if constexpr (NIN >= 2) y = ew_load<in2_t, 1, UNAL>(p.ptr[1] + (b2 ? 0 : i * sizeof(in2_t)), false, u2).v[0];
         Vec<out_t, 1> o; o.v[0] = apply(x, y);
         ew_store<out_t, 1, UNAL>(po + i * sizeof(out_t), o, uo);
      }
   }
}

// ---------------------------------------------------------------------------
// One position (a run of K vectors of VEC elements along dimension 0) per thread and loop pass; the grid has one
// block per EW_THREADS positions.  K > 1 spreads the index decomposition over K vectors: with 16-byte vectors of
// doubles (VEC = 2) one vector per thread left the kernel bound by the decomposition, not by memory (a double add
// with a row broadcast along dimension 0 took the time of a three-operand add).  Measured on 4096^2 (B200), K = 1 / 2 /
// 4: double add with a broadcast row 67.8 / 49.4 / 53.0 us, double add on padded rows 67.7 / 59.7 / 69.8 us, float
// add on padded rows 35.7 / 34.8 / 42.0 us: two vectors it is (64 contiguous bytes per thread cost coalescing).
// Measured and rejected: several POSITIONS per thread with all loads issued first (2 and 4 positions: 15 % and 35 %
// slower on padded rows).
#ifndef EW_STRIDED_K
#define EW_STRIDED_K 2
#endif
template <class A, int VEC, int K, bool UNAL>
__global__ void __launch_bounds__(EW_THREADS) ew_strided(const A apply, const EwParams<A::NIN + 1> p)
{
   using X = ew_traits<A>;
   constexpr int NIN = X::NIN, NOPS = NIN + 1;
   using out_t = typename X::out_t; using in1_t = typename X::in1_t; using in2_t = typename X::in2_t;
   const bool b1 = p.bcast & 1u, b2 = p.bcast & 2u;
   const bool u1 = p.unal & 1u, u2 = p.unal & 2u, uo = p.unal & (1u << NIN);

   for (uint64_t idx = (uint64_t)blockIdx.x * EW_THREADS + threadIdx.x; idx < p.total;
        idx += (uint64_t)gridDim.x * EW_THREADS) {
      int64_t off[NOPS];
#pragma unroll
      for (int k = 0; k < NOPS; k++) off[k] = 0;
      if (!p.wide) {
         uint32_t r = (uint32_t)idx;
         for (int d = 0; d < p.ndims - 1; d++) {
            uint32_t q = fastdiv(r, p.div[d]);
            uint32_t c = r - q * p.size[d];
            r = q;
#pragma unroll
            for (int k = 0; k < NOPS; k++) off[k] += (int64_t)c * p.stride[k][d];
         }
#pragma unroll
         for (int k = 0; k < NOPS; k++) off[k] += (int64_t)r * p.stride[k][p.ndims - 1];
      } else {
         uint64_t r = idx;
         for (int d = 0; d < p.ndims - 1; d++) {
            uint64_t q = udiv64(r, (uint64_t)p.size64[d]);
            uint64_t c = r - q * (uint64_t)p.size64[d];
            r = q;
#pragma unroll
            for (int k = 0; k < NOPS; k++) off[k] += (int64_t)c * p.stride[k][d];
         }
#pragma unroll
         for (int k = 0; k < NOPS; k++) off[k] += (int64_t)r * p.stride[k][p.ndims - 1];
      }
      // K > 1 only with VEC > 1: every operand is then dense (or broadcast) along dimension 0
      Vec<in1_t, VEC> a[K]; Vec<in2_t, VEC> b[K];
#pragma unroll
      for (int j = 0; j < K; j++) {
         if constexpr (NIN >= 1) { if (j == 0 || !b1) a[j] = ew_load<in1_t, VEC, UNAL>(p.ptr[0] + off[0] + (b1 ? 0 : j * VEC * (int)sizeof(in1_t)), VEC > 1 && b1, u1); else a[j] = a[0]; }
         if constexpr (NIN >= 2) { if (j == 0 || !b2) b[j] = ew_load<in2_t, VEC, UNAL>(p.ptr[1] + off[1] + (b2 ? 0 : j * VEC * (int)sizeof(in2_t)), VEC > 1 && b2, u2); else b[j] = b[0]; }
      }
#pragma unroll
      for (int j = 0; j < K; j++) {
         Vec<out_t, VEC> o;
         if constexpr (has_vector_apply<A>::value && (VEC > 1)) o = apply.template vec<VEC>(a[j], b[j]);
         else {
#pragma unroll
            for (int e = 0; e < VEC; e++) o.v[e] = apply(a[j].v[e], b[j].v[e]);
         }
         ew_store<out_t, VEC, UNAL>(p.ptr[NIN] + off[NIN] + j * VEC * (int)sizeof(out_t), o, uo);
      }
   }
}


// ---------------------------------------------------------------------------
// ew_tiled: some source is dense along ANOTHER dimension T than the destination (a transposed view, the classic
// B = A^T or C = A^T + B).  Read along the destination's dense dimension, such a source touches one element per
// 32-byte sector, which is what ew_strided<VEC = 1> (and the reference's kernels) do.  Here a block owns a
// 32 x 32 (or 32 x 64) tile over (dimension 0, dimension T): sources dense along T are read row by row along T
// (coalesced), parked in shared memory (odd row pitch, so the transposed read is free of bank conflicts for
// 4-byte elements and two-way at most for wider ones), and the block then walks the tile along dimension 0,
// taking those sources from shared memory and everything else (destination, sources dense or broadcast along
// dimension 0) straight from global memory.  Every byte still moves once.  Remaining dimensions are decomposed
// once per block.  Measured on 4096^2 (B200): double transposing copy 44.5 us (6.0 TB/s, the rate of a plain
// device copy), float 24.7 us, float add with one transposed operand 35 us.
// ---------------------------------------------------------------------------
constexpr int EW_TILE = 32;              // tile extent along dimension 0
constexpr int EW_TILE_T_WIDE = 64;       // tile extent along T for one-source operations on elements of at most 4 bytes

template <int NOPS> struct EwTiledParams {
   char    *ptr[NOPS];
   int64_t  stride[NOPS][MAXD];
   uint32_t size[MAXD];
   FastDiv  div[MAXD];
   FastDiv  div_tiles0, div_tilesT;
   uint32_t tiles0, tilesT;
   int      ndims, tdim;
   uint32_t staged;                  // bit k: source k goes through shared memory
};

// One tile.  STAGED (which sources go through shared memory), the tile extent along T and FULL (no element of the
// tile lies outside the tensor) are compile-time, so the inner loops carry no case distinctions; every access
// walks a pointer that is set up once per thread.
//   phase 1  TST lanes along T, 256 / TST rows of dimension 0 per pass: the staged sources, coalesced along T
//   phase 2  32 lanes along dimension 0, 8 rows of T per pass: shared memory, direct sources, destination
// The direct sources are fetched BEFORE phase 1, so that all global loads of the tile are in flight together.
template <class A, int STAGED, int TST, bool FULL>
SD_D void ew_tile_body(const A &apply, const EwTiledParams<A::NIN + 1> &p, const int64_t (&off)[A::NIN + 1],
                       uint32_t base0, uint32_t baseT,
                       typename A::in1_t (*tile1)[TST + 1], typename A::in2_t (*tile2)[TST + 1])
{
   using X = ew_traits<A>;
   constexpr int NIN = X::NIN, TS = EW_TILE, R1 = EW_THREADS / TST, R2 = EW_THREADS / TS, PER = TS / R1;
   static_assert(TS / R1 == TST / R2, "both phases must move the same number of elements per thread");
   using out_t = typename X::out_t; using in1_t = typename X::in1_t; using in2_t = typename X::in2_t;
   const int T = p.tdim;
   const uint32_t size0 = p.size[0], sizeT = p.size[T];
   const uint32_t tx1 = threadIdx.x % TST, ty1 = threadIdx.x / TST;
   const uint32_t tx2 = threadIdx.x % TS,  ty2 = threadIdx.x / TS;
   bool ok1[PER], ok2[PER];
#pragma unroll
   for (int j = 0; j < PER; j++) {
      ok1[j] = FULL || ((base0 + ty1 + R1 * j < size0) && (baseT + tx1 < sizeT));
      ok2[j] = FULL || ((base0 + tx2 < size0) && (baseT + ty2 + R2 * j < sizeT));
   }
   in1_t a[PER]; in2_t b[PER];
   // direct sources, phase-2 mapping
   if constexpr (NIN >= 1 && !(STAGED & 1)) {
      const char *q = p.ptr[0] + off[0] + (int64_t)(base0 + tx2) * p.stride[0][0] + (int64_t)(baseT + ty2) * p.stride[0][T];
      const int64_t step = R2 * p.stride[0][T];
#pragma unroll
      for (int j = 0; j < PER; j++, q += step) if (ok2[j]) a[j] = ld_one<in1_t>(q);
   }
   if constexpr (NIN >= 2 && !(STAGED & 2)) {
      const char *q = p.ptr[1] + off[1] + (int64_t)(base0 + tx2) * p.stride[1][0] + (int64_t)(baseT + ty2) * p.stride[1][T];
      const int64_t step = R2 * p.stride[1][T];
#pragma unroll
      for (int j = 0; j < PER; j++, q += step) if (ok2[j]) b[j] = ld_one<in2_t>(q);
   }
   // staged sources, phase-1 mapping
   if constexpr (NIN >= 1 && (STAGED & 1)) {
      const char *q = p.ptr[0] + off[0] + (int64_t)(base0 + ty1) * p.stride[0][0] + (int64_t)(baseT + tx1) * p.stride[0][T];
      const int64_t step = R1 * p.stride[0][0];
      in1_t r[PER];
#pragma unroll
      for (int j = 0; j < PER; j++, q += step) if (ok1[j]) r[j] = ld_one<in1_t>(q);
#pragma unroll
      for (int j = 0; j < PER; j++) tile1[ty1 + R1 * j][tx1] = r[j];
   }
   if constexpr (NIN >= 2 && (STAGED & 2)) {
      const char *q = p.ptr[1] + off[1] + (int64_t)(base0 + ty1) * p.stride[1][0] + (int64_t)(baseT + tx1) * p.stride[1][T];
      const int64_t step = R1 * p.stride[1][0];
      in2_t r[PER];
#pragma unroll
      for (int j = 0; j < PER; j++, q += step) if (ok1[j]) r[j] = ld_one<in2_t>(q);
#pragma unroll
      for (int j = 0; j < PER; j++) tile2[ty1 + R1 * j][tx1] = r[j];
   }
   __syncthreads();
   if constexpr (NIN >= 1 && (STAGED & 1)) {
#pragma unroll
      for (int j = 0; j < PER; j++) a[j] = tile1[tx2][ty2 + R2 * j];
   }
   if constexpr (NIN >= 2 && (STAGED & 2)) {
#pragma unroll
      for (int j = 0; j < PER; j++) b[j] = tile2[tx2][ty2 + R2 * j];
   }
   char *qo = p.ptr[NIN] + off[NIN] + (int64_t)(base0 + tx2) * p.stride[NIN][0] + (int64_t)(baseT + ty2) * p.stride[NIN][T];
   const int64_t ostep = R2 * p.stride[NIN][T];
#pragma unroll
   for (int j = 0; j < PER; j++, qo += ostep) if (ok2[j]) st_one<out_t>(qo, apply(a[j], b[j]));
}

template <class A, int STAGED, int TST>
__global__ void __launch_bounds__(EW_THREADS) ew_tiled(const A apply, const EwTiledParams<A::NIN + 1> p)
{
   using X = ew_traits<A>;
   constexpr int NIN = X::NIN, NOPS = NIN + 1, TS = EW_TILE;
   using in1_t = typename X::in1_t; using in2_t = typename X::in2_t;
   __shared__ in1_t tile1[(STAGED & 1) ? TS : 1][TST + 1];
   __shared__ in2_t tile2[(STAGED & 2) ? TS : 1][TST + 1];

   // block -> (tile along 0, tile along T, position in the remaining dimensions)
   uint32_t q = blockIdx.x;
   uint32_t qq = fastdiv(q, p.div_tiles0);
   const uint32_t base0 = (q - qq * p.tiles0) * TS; q = qq;
   qq = fastdiv(q, p.div_tilesT);
   const uint32_t baseT = (q - qq * p.tilesT) * TST; q = qq;
   int64_t off[NOPS];
#pragma unroll
   for (int k = 0; k < NOPS; k++) off[k] = 0;
   for (int d = 1; d < p.ndims; d++) {
      if (d == p.tdim) continue;
      qq = fastdiv(q, p.div[d]);
      const uint32_t c = q - qq * p.size[d]; q = qq;
#pragma unroll
      for (int k = 0; k < NOPS; k++) off[k] += (int64_t)c * p.stride[k][d];
   }
   if (base0 + TS <= p.size[0] && baseT + TST <= p.size[p.tdim]) ew_tile_body<A, STAGED, TST, true>(apply, p, off, base0, baseT, tile1, tile2);
   else                                                         ew_tile_body<A, STAGED, TST, false>(apply, p, off, base0, baseT, tile1, tile2);
}

// Extent of the tile along T for an operation: one-source operations on narrow elements move eight elements per
// thread (measured on 4096^2 floats: 24.7 us against 30.9 us with four), everything else four.
template <class A> constexpr int ew_tile_t()
{  return (A::NIN == 1 && ew_traits<A>::s_max <= 4) ? EW_TILE_T_WIDE : EW_TILE; }

template <class A, int STAGED>
void ew_tiled_launch(const A &apply, const EwTiledParams<A::NIN + 1> &p, unsigned blocks, cudaStream_t stream)
{  ew_tiled<A, STAGED, ew_tile_t<A>()><<<blocks, EW_THREADS, 0, stream>>>(apply, p); }

// Can the operation run as ew_tiled?  Requires aligned elements, a destination dense along dimension 0, at least
// one source that is neither dense nor constant along dimension 0 but dense along some other dimension, that
// dimension being the same for all such sources, and tiles worth the trouble.  Fills the parameters if so.
template <class A>
bool ew_plan_tiled(const Layout<A::NIN + 1> &L, EwTiledParams<A::NIN + 1> &p)
{
   using X = ew_traits<A>;
   constexpr int NIN = X::NIN, NOPS = NIN + 1;
   const int esize[3] = { NIN >= 1 ? X::s_in1 : X::s_out, NIN >= 2 ? X::s_in2 : X::s_out, X::s_out };
   auto es = [&](int k) { return k == NIN ? X::s_out : esize[k]; };
   if (NIN == 0 || L.ndims < 2 || L.stride[NIN][0] != es(NIN)) return false;
   int tdim = -1; uint32_t staged = 0;
   for (int k = 0; k < NIN; k++) {
      if (L.stride[k][0] == es(k) || L.stride[k][0] == 0) continue;
      int mine = -1;
      for (int d = 1; d < L.ndims; d++) if (L.stride[k][d] == es(k)) { mine = d; break; }
      if (mine < 0 || (tdim >= 0 && mine != tdim)) return false;
      tdim = mine; staged |= (1u << k);
   }
   if (tdim < 0 || L.size[0] < 8 || L.size[tdim] < 8) return false;
   uint64_t blocks = 1;
   memset(&p, 0, sizeof(p));
   for (int d = 0; d < L.ndims; d++) {
      if (L.size[d] > 0x7FFFFFFFll) return false;
      p.size[d] = (uint32_t)L.size[d];
      p.div[d] = make_fastdiv(p.size[d]);
      for (int k = 0; k < NOPS; k++) p.stride[k][d] = L.stride[k][d];
      const int64_t ext = (d == tdim) ? ew_tile_t<A>() : EW_TILE;
      blocks *= (d == 0 || d == tdim) ? (uint64_t)((L.size[d] + ext - 1) / ext) : (uint64_t)L.size[d];
   }
   if (blocks > 0x7FFFFFFFull) return false;
   for (int k = 0; k < NOPS; k++) p.ptr[k] = L.ptr[k];
   p.ndims = L.ndims; p.tdim = tdim; p.staged = staged;
   p.tiles0 = (uint32_t)((L.size[0] + EW_TILE - 1) / EW_TILE);
   p.tilesT = (uint32_t)((L.size[tdim] + ew_tile_t<A>() - 1) / ew_tile_t<A>());
   p.div_tiles0 = make_fastdiv(p.tiles0); p.div_tilesT = make_fastdiv(p.tilesT);
   return true;
}

// ---------------------------------------------------------------------------
// Host side: pick the variant and launch.
// ---------------------------------------------------------------------------
inline int ew_grid(uint64_t work_items, uint64_t items_per_block, const DeviceInfo &dev)
{
   uint64_t blocks = (work_items + items_per_block - 1) / items_per_block;
   // One chunk per block: on B200 a streaming kernel launched this way measured 7.1 TB/s against 6.4-6.6 TB/s
   // for a grid of one to four waves whose blocks stride through the arrays.  The loops in the kernels remain for
   // tensors beyond the grid limit.
   (void)dev;
   const uint64_t cap = 0x7FFFFFFFull;
   if (blocks > cap) blocks = cap;
   if (blocks < 1) blocks = 1;
   return (int)blocks;
}

template <class A, bool ALLOW_UNALIGNED = false>
int ew_launch(const A &apply, Layout<A::NIN + 1> &L, cudaStream_t stream)
{
   using X = ew_traits<A>;
   constexpr int NIN = X::NIN, NOPS = NIN + 1, VEC = X::VEC;
   const int esize[3] = { NIN >= 1 ? X::s_in1 : X::s_out, NIN >= 2 ? X::s_in2 : X::s_out, X::s_out };
   auto es = [&](int k) { return k == NIN ? X::s_out : esize[k]; };
   if (L.nelem == 0) return 0;
   DeviceInfo dev;
   if (current_device_info(&dev) != 0) return -1;

   EwParams<NOPS> p;
   memset(&p, 0, sizeof(p));
   for (int k = 0; k < NOPS; k++) p.ptr[k] = L.ptr[k];
   p.nelem = (uint64_t)L.nelem;

   // dense (or broadcast) along dimension 0 for every operand?
   bool dense0 = true; uint32_t bcast = 0;
   for (int k = 0; k < NOPS; k++) {
      if (L.stride[k][0] == es(k) || L.size[0] == 1) continue;
      if (L.stride[k][0] == 0 && k != NIN) { bcast |= (1u << k); continue; }
      dense0 = false;
   }
   // vector accesses need 16-byte aligned addresses (or the natural alignment of a narrower vector)
   auto vec_align = [&](int k) { int b = es(k) * VEC; return (size_t)(b >= 16 ? 16 : b); };
   // operands whose addresses are not multiples of the element size
   uint32_t unal = 0;
   for (int k = 0; k < NOPS; k++) {
      bool bad = !aligned_to(L.ptr[k], (size_t)es(k));
      for (int d = 0; d < L.ndims && !bad; d++) if (L.stride[k][d] % es(k) != 0) bad = true;
      if (bad) unal |= (1u << k);
   }
   if (unal && !ALLOW_UNALIGNED) SD_ERROR("Tensor data must be aligned to the element size");
   p.unal = unal;
   bool aligned = true;
   for (int k = 0; k < NOPS; k++) {
      if ((bcast | unal) & (1u << k)) continue;
      if (!aligned_to(L.ptr[k], vec_align(k))) aligned = false;
   }

   if (L.ndims == 1 && dense0 && (aligned || VEC == 1)) {
      p.bcast = bcast;
      uint64_t nvec = p.nelem / VEC;
      int grid = ew_grid(nvec ? nvec : 1, (uint64_t)EWC_THREADS * X::UNROLL, dev);
      if (ALLOW_UNALIGNED && unal) ew_contig<A, ALLOW_UNALIGNED><<<grid, EWC_THREADS, 0, stream>>>(apply, p);
      else                         ew_contig<A, false><<<grid, EWC_THREADS, 0, stream>>>(apply, p);
      SD_LAUNCH_CHECK();
      return 0;
   }

   // a source dense along another dimension than the destination: shared-memory tiles
   if constexpr (NIN >= 1) {
      if (!dense0 && !unal) {
         EwTiledParams<NOPS> tp;
         if (ew_plan_tiled<A>(L, tp)) {
            uint64_t blocks = (uint64_t)tp.tiles0 * tp.tilesT;
            for (int d = 1; d < L.ndims; d++) if (d != tp.tdim) blocks *= (uint64_t)L.size[d];
            if constexpr (NIN == 1) ew_tiled_launch<A, 1>(apply, tp, (unsigned)blocks, stream);
            else {
               if (tp.staged == 1u)      ew_tiled_launch<A, 1>(apply, tp, (unsigned)blocks, stream);
               else if (tp.staged == 2u) ew_tiled_launch<A, 2>(apply, tp, (unsigned)blocks, stream);
               else                      ew_tiled_launch<A, 3>(apply, tp, (unsigned)blocks, stream);
            }
            SD_LAUNCH_CHECK();
            return 0;
         }
      }
   }

   // strided: can the innermost dimension be vectorised?
   bool vec_ok = dense0 && aligned && VEC > 1 && (L.size[0] % VEC == 0);
   if (vec_ok) for (int k = 0; k < NOPS && vec_ok; k++) {
      if ((bcast | unal) & (1u << k)) continue;
      for (int d = 1; d < L.ndims; d++) if (L.stride[k][d] % (int64_t)vec_align(k) != 0) { vec_ok = false; break; }
   }
   // K consecutive vectors per thread when rows divide evenly and are long enough to keep a warp on one row
   constexpr int K = (VEC > 1 && VEC * X::s_max * EW_STRIDED_K <= 64) ? EW_STRIDED_K : ((VEC > 1 && VEC * X::s_max * 2 <= 64) ? 2 : 1);
   const bool run_ok = vec_ok && K > 1 && (L.size[0] % (VEC * K) == 0) && (L.size[0] / (VEC * K) >= 32);
   const int vec = vec_ok ? (run_ok ? VEC * K : VEC) : 1;
   p.ndims = L.ndims;
   p.bcast = vec_ok ? bcast : 0;
   uint64_t total = 1; bool fits32 = true;
   for (int d = 0; d < L.ndims; d++) {
      int64_t sz = (d == 0) ? L.size[0] / vec : L.size[d];
      p.size64[d] = sz;
      if (sz > 0x7FFFFFFFll) fits32 = false;
      p.size[d] = (uint32_t)sz;
      p.div[d] = make_fastdiv((uint32_t)sz);
      total *= (uint64_t)sz;
      for (int k = 0; k < NOPS; k++) p.stride[k][d] = (d == 0) ? L.stride[k][0] * vec : L.stride[k][d];
   }
   p.total = total;
   p.wide = (total > 0xFFFFFFFFull || !fits32) ? 1 : 0;
   int grid = ew_grid(total, EW_THREADS, dev);
   if (ALLOW_UNALIGNED && unal) {
      if (run_ok)      ew_strided<A, VEC, K, ALLOW_UNALIGNED><<<grid, EW_THREADS, 0, stream>>>(apply, p);
      else if (vec_ok) ew_strided<A, VEC, 1, ALLOW_UNALIGNED><<<grid, EW_THREADS, 0, stream>>>(apply, p);
      else             ew_strided<A, 1, 1, ALLOW_UNALIGNED><<<grid, EW_THREADS, 0, stream>>>(apply, p);
   } else {
      if (run_ok)      ew_strided<A, VEC, K, false><<<grid, EW_THREADS, 0, stream>>>(apply, p);
      else if (vec_ok) ew_strided<A, VEC, 1, false><<<grid, EW_THREADS, 0, stream>>>(apply, p);
      else             ew_strided<A, 1, 1, false><<<grid, EW_THREADS, 0, stream>>>(apply, p);
   }
   SD_LAUNCH_CHECK();
   return 0;
}

// ---------------------------------------------------------------------------
// Apply adaptors for the functors of ops_unary.cuh / ops_binary.cuh
// ---------------------------------------------------------------------------
// Operations on 8- and 16-bit integers and on bool bytes that act on each byte (or half word) independently are
// run on whole 32-bit words whenever every operand is dense along dimension 0 with word-aligned rows: the tensors
// are re-described as tensors of uint32 and go through the same engine (contiguous, strided, runs) as any 4-byte
// type.  A vector of sixteen separate bytes costs the compiler some fifty registers and a pack / unpack sequence:
// the per-element form of a contiguous uint8 and ran at 2.0-4.6 TB/s (64 to 16 bytes in flight) where a 4-byte add
// runs at 7.0.  word_op<Op, T>::f is the operation on four packed bytes / two packed half words.
struct b_bitwise_and; struct b_bitwise_or; struct b_bitwise_xor; struct b_add; struct b_subtract; struct b_multiply;
struct u_negative; struct u_bitwise_not;                   // defined in ops_binary.cuh / ops_unary.cuh
template <class Op, class T, class = void> struct word_op { static constexpr bool value = false; };
template <class T> constexpr bool is_narrow_int = is_int<T> && sizeof(T) <= 2;
template <class T> constexpr bool is_narrow = (is_int<T> && sizeof(T) <= 2) || is_bool<T>;
#define SD_WORD_OP(OP, COND, EXPR)                                                                   \
   template <class T> struct word_op<OP, T, std::enable_if_t<(COND)>> {                               \
      static constexpr bool value = true;                                                            \
      static SD_D uint32_t f(uint32_t a, uint32_t b) { (void)b; return (EXPR); } };
SD_WORD_OP(b_bitwise_and, is_narrow<T>, a & b)
SD_WORD_OP(b_bitwise_or,  is_narrow<T>, a | b)
SD_WORD_OP(b_bitwise_xor, is_narrow<T>, a ^ b)
SD_WORD_OP(b_add,      is_narrow_int<T>, sizeof(T) == 1 ? __vadd4(a, b) : __vadd2(a, b))      // wrap-around per element
SD_WORD_OP(b_subtract, is_narrow_int<T>, sizeof(T) == 1 ? __vsub4(a, b) : __vsub2(a, b))
SD_WORD_OP(b_add,      is_bool<T>, a | b)                                                      // the bool aliases
SD_WORD_OP(b_subtract, is_bool<T>, a & ~b)
SD_WORD_OP(b_multiply, is_bool<T>, a & b)
SD_WORD_OP(u_negative,    is_narrow_int<T>, sizeof(T) == 1 ? __vneg4(a) : __vneg2(a))
SD_WORD_OP(u_negative,    is_bool<T>, a ^ 0x01010101u)
SD_WORD_OP(u_bitwise_not, is_narrow_int<T>, ~a)
SD_WORD_OP(u_bitwise_not, is_bool<T>, a ^ 0x01010101u)
#undef SD_WORD_OP
template <class Op, class T> struct WordUnaryApply {
   static constexpr int NIN = 1;
   using in1_t = uint32_t; using in2_t = Nothing; using out_t = uint32_t;
   SD_D uint32_t operator()(uint32_t x, Nothing) const { return word_op<Op, T>::f(x, x); }
};
template <class Op, class T> struct WordBinaryApply {
   static constexpr int NIN = 2;
   using in1_t = uint32_t; using in2_t = uint32_t; using out_t = uint32_t;
   SD_D uint32_t operator()(uint32_t x, uint32_t y) const { return word_op<Op, T>::f(x, y); }
};
// Re-describe operands of `es`-byte elements as words; false (layout untouched) when some operand is not made of
// whole aligned words along dimension 0.
template <int NOPS> inline bool layout_as_words(Layout<NOPS> &L, int es)
{
   const int per = 4 / es;
   if (L.nelem == 0 || L.ndims < 1 || L.size[0] % per != 0) return false;
   for (int k = 0; k < NOPS; k++) {
      if (L.stride[k][0] != es || !aligned_to(L.ptr[k], 4)) return false;
      for (int d = 1; d < L.ndims; d++) if (L.stride[k][d] % 4 != 0) return false;
   }
   L.size[0] /= per; L.nelem /= per;
   for (int k = 0; k < NOPS; k++) L.stride[k][0] = 4;
   return true;
}

template <class Op, class T> struct UnaryApply {
   static constexpr int NIN = 1;
   using in1_t = T; using in2_t = Nothing; using out_t = typename Op::template out<T>;
   SD_D out_t operator()(T x, Nothing) const { return Op::template f<T>(x); }
};
template <class Op, class T> struct BinaryApply {
   static constexpr int NIN = 2;
   using in1_t = T; using in2_t = typename Op::template in2<T>; using out_t = typename Op::template out<T>;
   SD_D out_t operator()(in1_t x, in2_t y) const { return Op::template f<T>(x, y); }
};

template <class Op, class T>
int launch_unary(int ndims, const size_t *size, const ptrdiff_t *strides1, void *ptr1,
                 const ptrdiff_t *strides2, void *ptr2, cudaStream_t stream)
{
   if (strides2 == nullptr && ptr2 == nullptr) { strides2 = strides1; ptr2 = ptr1; }   // in place
   const ptrdiff_t *st[2] = { strides1, strides2 }; void *pt[2] = { ptr1, ptr2 };
   Layout<2> L;
   if (make_layout<2>(L, ndims, size, st, pt, 1) != 0) return -1;
   if constexpr (word_op<Op, T>::value) { if (layout_as_words<2>(L, (int)sizeof(T))) return ew_launch(WordUnaryApply<Op, T>(), L, stream); }
   return ew_launch(UnaryApply<Op, T>(), L, stream);
}

template <class Op, class T>
int launch_binary(int ndims, const size_t *size, const ptrdiff_t *strides1, void *ptr1,
                  const ptrdiff_t *strides2, void *ptr2, const ptrdiff_t *strides3, void *ptr3,
                  cudaStream_t stream)
{
   if (strides3 == nullptr && ptr3 == nullptr) { strides3 = strides1; ptr3 = ptr1; }   // into operand 1
   const ptrdiff_t *st[3] = { strides1, strides2, strides3 }; void *pt[3] = { ptr1, ptr2, ptr3 };
   Layout<3> L;
   if (make_layout<3>(L, ndims, size, st, pt, 2) != 0) return -1;
   if constexpr (word_op<Op, T>::value) { if (layout_as_words<3>(L, (int)sizeof(T))) return ew_launch(WordBinaryApply<Op, T>(), L, stream); }
   return ew_launch(BinaryApply<Op, T>(), L, stream);
}

} // namespace sd
