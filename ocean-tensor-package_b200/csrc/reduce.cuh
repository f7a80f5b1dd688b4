// Reduction engine: global and per-axis reductions share three kernels plus a
// finalize pass.  A global reduction is the per-axis problem with one output.
//
// Replaces solid/include/solid/core/gpu/reduce_all.h:136-274 (512-entry volatile
// shared-memory tree, one scalar load per thread-iteration, 1-warp finalize) and
// reduce_axis.h:142-519 (thread / warp / block modes, all with per-element
// index decomposition and scalar loads).
//
//   red_row   the first reduced dimension is dense in memory: a group of 32 or 256
//             threads sweeps each output's data with 128-bit loads, four vectors in
//             flight per thread; warp-shuffle tree, then a fixed-order fold of the
//             warp results through shared memory;
//   red_col   the first kept dimension is dense: each thread owns VEC adjacent
//             outputs and walks the reduced range, so a warp still reads whole
//             128-byte lines; blockDim.y slices the range and is folded in order;
//   red_gen   anything else: one thread per output, full index decomposition;
//   red_fin   when the reduced range of an output was split over several blocks
//             (few outputs, e.g. the global case) the blocks write partial
//             accumulators to scratch memory and this second pass folds them in
//             index order and applies the finalize step.  With a SINGLE output the
//             second pass rides in red_row itself: every block counts its arrival on
//             the stream's counter (one atomicAdd, nothing waits on it) and the block
//             that arrives last does the same ordered fold.  The atomic only decides
//             WHICH block folds, never the order, so results are bit-reproducible for a
//             given device and shape.
//
// HBM traffic: every input element is read once; partials are a few KB.
#pragma once
#include "dtypes.cuh"
#include "layout.h"
#include "word_accum.cuh"

namespace sd {

constexpr int RED_THREADS = 256;
// Blocks per multiprocessor that a reduction aims for when it splits outputs over blocks: one resident
// wave.  Measured on B200 (global and 8192^2 axis reductions), 16 or 32 per multiprocessor were slower.
constexpr int RED_WANT_PER_SM = 8;
// Resident blocks per multiprocessor asked of the compiler for the streaming kernels (64 registers per
// thread: red_row always four); the 1- and 2-byte forms of red_col keep 16 or 8 accumulators per thread
// and are left alone.
#define RED_MIN_BLOCKS(T) (sizeof(T) >= 4 ? 4 : 1)

struct RedParams {
   char    *src, *dst, *buf;
   int      ndims, rdims;
   int64_t  size[MAXD], stride1[MAXD], stride2[MAXD];
   int64_t  rsize[MAXD], rstride[MAXD];
   uint64_t nout, relem;
   uint32_t split;          // blocks (or groups) that share one output
   uint32_t group;          // red_row: threads per output chunk (32 or 256)
   uint64_t tiles0;         // red_col: tiles along outer dimension 0
   unsigned int *ticket;    // single output split over blocks: arrival counter of the stream (the last block folds), or null
   uint32_t *flag;          // host-returning form: word the finishing thread sets to flag_value after the result, or null
   uint32_t flag_value;
};

// Arrival counter for single-pass folds on `stream` of the current device (reduce_plan.cu): one word
// of a zero-initialised device array per stream, which the last block of a launch sets back to zero.
// Null when no counter can be given (per-thread default stream, table full); callers then use red_fin.
unsigned int *red_ticket_for_stream(cudaStream_t stream);

// offset of output `o` in source (outer part) and destination
SD_D void outer_offsets(const RedParams &p, uint64_t o, int64_t &off1, int64_t &off2)
{
   off1 = 0; off2 = 0;
   for (int d = 0; d < p.ndims - 1; d++) {
      uint64_t q = udiv64(o, (uint64_t)p.size[d]); uint64_t c = o - q * (uint64_t)p.size[d]; o = q;
      off1 += (int64_t)c * p.stride1[d]; off2 += (int64_t)c * p.stride2[d];
   }
   if (p.ndims > 0) { off1 += (int64_t)o * p.stride1[p.ndims - 1]; off2 += (int64_t)o * p.stride2[p.ndims - 1]; }
}
// offset of reduced index r, decomposed over reduced dimensions first..rdims-1
SD_D int64_t reduced_offset(const RedParams &p, uint64_t r, int first)
{
   int64_t off = 0;
   for (int d = first; d < p.rdims - 1; d++) {
      uint64_t q = udiv64(r, (uint64_t)p.rsize[d]); uint64_t c = r - q * (uint64_t)p.rsize[d]; r = q;
      off += (int64_t)c * p.rstride[d];
   }
   if (p.rdims > first) off += (int64_t)r * p.rstride[p.rdims - 1];
   return off;
}

template <class V> SD_D V shfl_down_any(const V &x, int delta)
{
   constexpr int W = (sizeof(V) + 3) / 4;
   uint32_t w[W] = {0};
   memcpy(w, &x, sizeof(V));
#pragma unroll
   for (int i = 0; i < W; i++) w[i] = __shfl_down_sync(0xFFFFFFFFu, w[i], delta);
   V y; memcpy(&y, w, sizeof(V));
   return y;
}

// Fold the accumulators of `width` consecutive lanes into the first lane.
template <class R, class A> SD_D void warp_fold(const R &r, A &acc, int width = 32)
{
#pragma unroll
   for (int d = 16; d >= 1; d >>= 1) {
      A other = shfl_down_any<A>(acc, d);
      if (d < width) r.combine(acc, other);
   }
}

// Fold one accumulator per thread of the block into thread 0 (fixed order).
template <class R, class A> SD_D void block_fold(const R &r, A &acc, A *smem)
{
   warp_fold(r, acc);
   const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x * blockDim.y) >> 5;
   if (lane == 0) smem[warp] = acc;
   __syncthreads();
   if (threadIdx.x == 0) for (int w = 1; w < nwarps; w++) r.combine(acc, smem[w]);
}

template <class R, class T> SD_D typename R::acc_t red_start(const R &r, const char *first_elem)
{
   if constexpr (R::seeded) return r.seed(ld_one<T>(first_elem));
   else { (void)first_elem; return r.init(); }
}

// Tell a polling host that the result is in place (the result itself lives in mapped host memory).
SD_D void red_signal(const RedParams &p)
{
   if (p.flag) { __threadfence_system(); *reinterpret_cast<volatile uint32_t *>(p.flag) = p.flag_value; }
}

template <class R> SD_D void red_emit(const R &r, const RedParams &p, uint64_t out, uint32_t s,
                                      int64_t off2, const typename R::acc_t &acc)
{
   using A = typename R::acc_t; using O = typename R::out_t;
   if (p.split > 1) reinterpret_cast<A *>(p.buf)[out * p.split + s] = acc;
   else { *reinterpret_cast<O *>(p.dst + off2) = r.finalize(acc); red_signal(p); }
}

// Fold all VEC elements of one vector into the accumulator (packed-word form for 1-byte types
// where the reduction has one).
template <class R, class T, int VEC> SD_D void accum_vec(const R &r, typename R::acc_t &acc, const Vec<T, VEC> &v)
{
   if constexpr (word_accum<R, T>::ok && VEC % 4 == 0) {
      uint32_t w[VEC / 4];
      memcpy(w, &v, VEC);
#pragma unroll
      for (int i = 0; i < VEC / 4; i++) word_accum<R, T>::apply(r, acc, w[i]);
   } else {
#pragma unroll
      for (int e = 0; e < VEC; e++) r.accum(acc, v.v[e]);
   }
}

// Second pass: a group of GROUP threads (one warp, or the whole block when an output has many
// partials) folds the `split` partials of one output.  Thread l of the group takes partials
// l, l+GROUP, ... in order; the threads are then joined by the shuffle tree and, for the block
// form, by a fixed-order pass over the warps.  Threads without a partial are skipped, because
// an extra copy of a partial is harmless only for idempotent folds.
template <class R, class A> SD_D void fold_have(const R &r, A &acc, bool &have, uint32_t lane)
{
#pragma unroll
   for (int d = 16; d >= 1; d >>= 1) {
      A other = shfl_down_any<A>(acc, d);
      bool other_has = __shfl_down_sync(0xFFFFFFFFu, (int)have, d) != 0 && (lane + d < 32);
      if (other_has) { if (have) r.combine(acc, other); else { acc = other; have = true; } }
   }
}

// Partials come from other multiprocessors: read them past the L1.
template <class A> SD_D A load_partial(const A *q)
{
   if constexpr (sizeof(A) % 4 == 0) {
      uint32_t w[sizeof(A) / 4];
#pragma unroll
      for (int i = 0; i < (int)(sizeof(A) / 4); i++) w[i] = __ldcg(reinterpret_cast<const uint32_t *>(q) + i);
      A a; memcpy(&a, w, sizeof(A)); return a;
   } else if constexpr (std::is_arithmetic<A>::value) {
      return *reinterpret_cast<const volatile A *>(q);
   } else {
      return *q;
   }
}

template <class R, int GROUP>
SD_D void red_fin_body(const R &r, const RedParams &p, uint64_t out, bool live, typename R::acc_t *smem, int *shave)
{
   using A = typename R::acc_t; using O = typename R::out_t;
   const uint32_t t = threadIdx.x % GROUP, lane = threadIdx.x & 31;
   const A *part = reinterpret_cast<const A *>(p.buf) + (live ? out : 0) * p.split;
   bool have = t < p.split;
   A acc = load_partial(part + (have ? t : 0));
   for (uint32_t i = t + GROUP; i < p.split; i += GROUP) r.combine(acc, load_partial(part + i));
   fold_have(r, acc, have, lane);
   if (GROUP > 32) {
      const int warp = threadIdx.x >> 5;
      if (lane == 0) { smem[warp] = acc; shave[warp] = have; }
      __syncthreads();
      if (threadIdx.x == 0)
         for (int w = 1; w < RED_THREADS / 32; w++) if (shave[w]) r.combine(acc, smem[w]);   // warp 0 always has data
   }
   if (t == 0 && live) {
      int64_t off1, off2;
      outer_offsets(p, out, off1, off2);
      *reinterpret_cast<O *>(p.dst + off2) = r.finalize(acc);
      red_signal(p);
   }
}

// ---------------------------------------------------------------------------
template <class R, class T, int VEC>
__global__ void __launch_bounds__(RED_THREADS, 4) red_row(const R r, const RedParams p)
{
   using A = typename R::acc_t;
   __shared__ A smem[RED_THREADS / 32];
   __shared__ int shave[RED_THREADS / 32];
   __shared__ int last_block;
   const uint32_t group = p.group;
   const uint32_t gpb = RED_THREADS / group;
   const uint64_t gid = (uint64_t)blockIdx.x * gpb + threadIdx.x / group;
   const uint32_t lane = threadIdx.x % group;
   const uint64_t out = udiv64(gid, p.split);
   const uint32_t s = (uint32_t)(gid - out * p.split);
   const bool live = out < p.nout;

   int64_t off1 = 0, off2 = 0;
   if (live) outer_offsets(p, out, off1, off2);
   const char *base = p.src + off1;
   A acc = red_start<R, T>(r, live ? base : p.src);

   if (live) {
      const uint64_t rowlen = (uint64_t)p.rsize[0];
      const uint64_t nslot = (rowlen + VEC - 1) / VEC;              // vector slots per row (last may be ragged)
      const uint64_t rows = udiv64(p.relem, rowlen);
      const uint64_t total = rows * nslot;
      constexpr int U = sizeof(T) >= 4 ? 8 : 4;         // vectors in flight per thread (measured: 8 is slower for 1-byte types)
      // slots per split, rounded up to whole passes of the group (trailing splits may be empty).  Rounding to whole
      // iterations of the unrolled loop instead left 80 of 592 blocks without work on 2^24 floats (2048 iterations of
      // 32 KB over 592 blocks: four each for 512 of them), 17.6 us where an even split takes 15.
      uint64_t chunk = udiv64(total + p.split - 1, p.split);
      chunk = udiv64(chunk + (uint64_t)group - 1, (uint64_t)group) * (uint64_t)group;
      const uint64_t begin = (uint64_t)s * chunk < total ? (uint64_t)s * chunk : total;
      const uint64_t end = begin + chunk < total ? begin + chunk : total;
      uint64_t slot0 = begin + lane;
      if (rows == 1) {
         // One dense row: whole vectors by pointer increment, nothing predicated per element.
         const uint64_t nfull = rowlen / VEC;
         const uint64_t fend = end < nfull ? end : nfull;
         const char *q = base + slot0 * (VEC * sizeof(T));
         const uint64_t gstep = (uint64_t)group * (VEC * sizeof(T));
         for (; slot0 + (uint64_t)(U - 1) * group < fend; slot0 += (uint64_t)group * U, q += gstep * U) {
            Vec<T, VEC> v[U];
#pragma unroll
            for (int u = 0; u < U; u++) v[u] = ld_vec<T, VEC>(q + u * gstep);
#pragma unroll
            for (int u = 0; u < U; u++) accum_vec<R, T, VEC>(r, acc, v[u]);
         }
         if (U >= 8 && slot0 + (uint64_t)3 * group < fend) {        // the remainder in halves of the unroll factor
            Vec<T, VEC> v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) v[u] = ld_vec<T, VEC>(q + u * gstep);
#pragma unroll
            for (int u = 0; u < 4; u++) accum_vec<R, T, VEC>(r, acc, v[u]);
            slot0 += (uint64_t)group * 4; q += gstep * 4;
         }
         if (slot0 + (uint64_t)group < fend) {
            Vec<T, VEC> v[2];
#pragma unroll
            for (int u = 0; u < 2; u++) v[u] = ld_vec<T, VEC>(q + u * gstep);
#pragma unroll
            for (int u = 0; u < 2; u++) accum_vec<R, T, VEC>(r, acc, v[u]);
            slot0 += (uint64_t)group * 2; q += gstep * 2;
         }
         for (; slot0 < fend; slot0 += group, q += gstep) accum_vec<R, T, VEC>(r, acc, ld_vec<T, VEC>(q));
         // the ragged last slot (fewer than VEC elements) is left to the general loop below
      }
      constexpr int UG = 2;                             // general form: index arithmetic per slot, few vectors in flight
      for (; slot0 < end; slot0 += (uint64_t)group * UG) {
         Vec<T, VEC> v[UG]; int cnt[UG];
#pragma unroll
         for (int u = 0; u < UG; u++) {
            uint64_t slot = slot0 + (uint64_t)u * group;
            cnt[u] = 0;
            if (slot < end) {
               uint64_t row = 0, j = slot;
               if (rows > 1) { row = udiv64(slot, nslot); j = slot - row * nslot; }
               const char *q = base + (rows > 1 ? reduced_offset(p, row, 1) : 0) + (int64_t)(j * VEC * sizeof(T));
               uint64_t left = rowlen - j * VEC;
               if (VEC == 1 || left >= (uint64_t)VEC) { v[u] = ld_vec<T, VEC>(q); cnt[u] = VEC; }
               else { cnt[u] = (int)left;
#pragma unroll
                  for (int e = 0; e < VEC; e++) if (e < (int)left) v[u].v[e] = ld_one<T>(q + e * sizeof(T)); }
            }
         }
#pragma unroll
         for (int u = 0; u < UG; u++) {
#pragma unroll
            for (int e = 0; e < VEC; e++) if (e < cnt[u]) r.accum(acc, v[u].v[e]);
         }
      }
   }
   // fold the group
   if (group == 32) {
      warp_fold(r, acc);
      if (lane == 0 && live) red_emit(r, p, out, s, off2, acc);
   } else {
      block_fold(r, acc, smem);
      if (threadIdx.x == 0 && live) red_emit(r, p, out, s, off2, acc);
      if (p.ticket != nullptr) {
         // One output shared by the `split` blocks of this grid: each block announces its partial on the
         // stream's counter, and the block that arrives last folds all partials (in index order, so the
         // result does not depend on which block that is) and leaves the counter at zero for the next launch.
         if (threadIdx.x == 0) { __threadfence(); last_block = (atomicAdd(p.ticket, 1u) == p.split - 1u); }
         __syncthreads();
         if (last_block) {
            __threadfence();
            red_fin_body<R, RED_THREADS>(r, p, 0, true, smem, shave);
            if (threadIdx.x == 0) *p.ticket = 0u;
         }
      }
   }
}

// ---------------------------------------------------------------------------
// blockDim = (bx, 256 / bx): x owns VEC adjacent outputs along outer dimension 0, y slices
// the reduced range.
template <class R, class T, int VEC>
__global__ void __launch_bounds__(RED_THREADS, RED_MIN_BLOCKS(T)) red_col(const R r, const RedParams p)
{
   using A = typename R::acc_t;
   __shared__ A smem[RED_THREADS][VEC];                                  // [y * blockDim.x + x]
   uint64_t bid = blockIdx.x;
   const uint64_t bq = udiv64(bid, p.split);
   const uint32_t s = (uint32_t)(bid - bq * p.split); bid = bq;
   const uint64_t rest = udiv64(bid, p.tiles0); const uint64_t tile = bid - rest * p.tiles0;
   const uint64_t o0 = (tile * blockDim.x + threadIdx.x) * VEC;         // first of my outputs along dim 0
   const bool live = o0 < (uint64_t)p.size[0];
   const int nmine = live ? (int)(((uint64_t)p.size[0] - o0) < (uint64_t)VEC ? ((uint64_t)p.size[0] - o0) : VEC) : 0;

   // offsets of the outer dimensions 1.. (dimension 0 is dense)
   int64_t off1 = 0, off2 = 0;
   {  uint64_t o = rest;
      for (int d = 1; d < p.ndims - 1; d++) {
         uint64_t q = udiv64(o, (uint64_t)p.size[d]); uint64_t c = o - q * (uint64_t)p.size[d]; o = q;
         off1 += (int64_t)c * p.stride1[d]; off2 += (int64_t)c * p.stride2[d]; }
      if (p.ndims > 1) { off1 += (int64_t)o * p.stride1[p.ndims - 1]; off2 += (int64_t)o * p.stride2[p.ndims - 1]; }
   }
   const char *base = p.src + off1 + (int64_t)(o0 * sizeof(T));
   A acc[VEC];
#pragma unroll
   for (int e = 0; e < VEC; e++) acc[e] = red_start<R, T>(r, (e < nmine) ? base + e * sizeof(T) : p.src);

   const uint64_t chunk = udiv64(p.relem + p.split - 1, p.split);
   const uint64_t begin = (uint64_t)s * chunk;
   const uint64_t end = begin + chunk < p.relem ? begin + chunk : p.relem;
   if (live) {
      constexpr int U = (sizeof(T) * VEC >= 16) ? 8 : 4;
      uint64_t r0 = begin + threadIdx.y;
      if (nmine == VEC && p.rdims == 1) {
         // full vector of outputs, one reduced dimension: pointer increments only
         const int64_t rs = p.rstride[0];
         const char *q = base + (int64_t)r0 * rs;
         const int64_t ystep = (int64_t)blockDim.y * rs;
         for (; r0 + (uint64_t)(U - 1) * blockDim.y < end; r0 += (uint64_t)blockDim.y * U, q += ystep * U) {
            Vec<T, VEC> v[U];
#pragma unroll
            for (int u = 0; u < U; u++) v[u] = ld_vec<T, VEC>(q + u * ystep);
#pragma unroll
            for (int u = 0; u < U; u++) {
#pragma unroll
               for (int e = 0; e < VEC; e++) r.accum(acc[e], v[u].v[e]);
            }
         }
         // the rows left over (fewer than U per y slice) in one more round, all loads issued together
         if (r0 < end) {
            Vec<T, VEC> v[U]; bool ok[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
               ok[u] = r0 + (uint64_t)u * blockDim.y < end;
               if (ok[u]) v[u] = ld_vec<T, VEC>(q + u * ystep);
            }
#pragma unroll
            for (int u = 0; u < U; u++) if (ok[u]) {
#pragma unroll
               for (int e = 0; e < VEC; e++) r.accum(acc[e], v[u].v[e]);
            }
            r0 = end;
         }
      }
      constexpr int UG = 2;
      for (; r0 < end; r0 += (uint64_t)blockDim.y * UG) {
         Vec<T, VEC> v[UG]; bool ok[UG];
#pragma unroll
         for (int u = 0; u < UG; u++) {
            uint64_t rr = r0 + (uint64_t)u * blockDim.y;
            ok[u] = rr < end;
            if (ok[u]) {
               const char *q = base + (p.rdims == 1 ? (int64_t)rr * p.rstride[0] : reduced_offset(p, rr, 0));
               if (nmine == VEC) v[u] = ld_vec<T, VEC>(q);
               else {
#pragma unroll
                  for (int e = 0; e < VEC; e++) if (e < nmine) v[u].v[e] = ld_one<T>(q + e * sizeof(T)); }
            }
         }
#pragma unroll
         for (int u = 0; u < UG; u++) if (ok[u]) {
#pragma unroll
            for (int e = 0; e < VEC; e++) if (e < nmine) r.accum(acc[e], v[u].v[e]);
         }
      }
   }
#pragma unroll
   for (int e = 0; e < VEC; e++) smem[threadIdx.y * blockDim.x + threadIdx.x][e] = acc[e];
   __syncthreads();
   if (threadIdx.y == 0 && live) {
      for (int y = 1; y < (int)blockDim.y; y++) {
#pragma unroll
         for (int e = 0; e < VEC; e++) r.combine(acc[e], smem[y * blockDim.x + threadIdx.x][e]);
      }
      const uint64_t outbase = rest * (uint64_t)p.size[0] + o0;
#pragma unroll
      for (int e = 0; e < VEC; e++) if (e < nmine)
         red_emit(r, p, outbase + e, s, off2 + (int64_t)(o0 + e) * p.stride2[0], acc[e]);
   }
}

// ---------------------------------------------------------------------------
template <class R, class T>
__global__ void __launch_bounds__(RED_THREADS) red_gen(const R r, const RedParams p)
{
   using A = typename R::acc_t;
   const uint64_t gid = (uint64_t)blockIdx.x * RED_THREADS + threadIdx.x;
   const uint64_t out = udiv64(gid, p.split);
   const uint32_t s = (uint32_t)(gid - out * p.split);
   if (out >= p.nout) return;
   int64_t off1, off2;
   outer_offsets(p, out, off1, off2);
   const char *base = p.src + off1;
   A acc = red_start<R, T>(r, base);
   const uint64_t chunk = udiv64(p.relem + p.split - 1, p.split);
   const uint64_t begin = (uint64_t)s * chunk;
   const uint64_t end = begin + chunk < p.relem ? begin + chunk : p.relem;
   for (uint64_t rr = begin; rr < end; rr++) r.accum(acc, ld_one<T>(base + reduced_offset(p, rr, 0)));
   red_emit(r, p, out, s, off2, acc);
}

// ---------------------------------------------------------------------------
template <class R, int GROUP>
__global__ void __launch_bounds__(RED_THREADS) red_fin(const R r, const RedParams p)
{
   using A = typename R::acc_t;
   __shared__ A smem[RED_THREADS / 32];
   __shared__ int shave[RED_THREADS / 32];
   const uint64_t out = (uint64_t)blockIdx.x * (RED_THREADS / GROUP) + threadIdx.x / GROUP;
   red_fin_body<R, GROUP>(r, p, out, out < p.nout, smem, shave);
}

// ---------------------------------------------------------------------------
// Planning (host)
// ---------------------------------------------------------------------------
struct RedPlan {
   RedParams p;
   uint32_t  split_cap;     // upper bound on split used to size the scratch buffer
};

// Largest number of blocks that may share one output, from the shape alone.
inline uint32_t red_split_cap(uint64_t nout, uint64_t relem, int sms)
{
   uint64_t by_work = relem / 256; if (by_work < 1) by_work = 1;     // a split covers at least 256 reduced positions
                                                                     // (measured on 8192^2 floats, dense columns: 32 splits
                                                                     // of 256 rows ran at 47 us, 74 splits of 111 at 58 us)
   uint64_t tiles = nout / 512; if (tiles < 1) tiles = 1;
   uint64_t by_fill = ((uint64_t)sms * RED_WANT_PER_SM + tiles - 1) / tiles;
   uint64_t cap = by_work < by_fill ? by_work : by_fill;
   if (cap < 1) cap = 1;
   if (cap > 65535) cap = 65535;
   return (uint32_t)cap;
}

// Normalise outer and reduced dimensions (sizes, strides in bytes).
inline int red_make_params(RedParams &p, int ndims, const size_t *size, const ptrdiff_t *strides1, void *ptr1,
                           const ptrdiff_t *strides2, void *ptr2, int rdims, const size_t *rsize,
                           const ptrdiff_t *rstrides)
{
   memset(&p, 0, sizeof(p));
   Layout<2> LO; Layout<1> LR;
   const ptrdiff_t zero[MAXD] = {0};
   {  const ptrdiff_t *st[2] = { strides1, strides2 ? strides2 : zero }; void *pt[2] = { ptr1, ptr2 };
      if (make_layout<2>(LO, ndims, size, st, pt, -1) != 0) return -1; }
   char *src = LO.ptr[0];
   {  const ptrdiff_t *st[1] = { rstrides }; void *pt[1] = { src };
      if (make_layout<1>(LR, rdims, rsize, st, pt, 0) != 0) return -1; }
   p.src = LR.ptr[0]; p.dst = LO.ptr[1];
   p.nout = (uint64_t)LO.nelem; p.relem = (uint64_t)LR.nelem;
   p.ndims = LO.nelem ? LO.ndims : 0; p.rdims = LR.nelem ? LR.ndims : 0;
   for (int d = 0; d < p.ndims; d++) { p.size[d] = LO.size[d]; p.stride1[d] = LO.stride[0][d]; p.stride2[d] = LO.stride[1][d]; }
   for (int d = 0; d < p.rdims; d++) { p.rsize[d] = LR.size[d]; p.rstride[d] = LR.stride[0][d]; }
   return 0;
}

template <class R, class T>
int red_launch(const R &r, RedParams p, uint32_t split_cap, cudaStream_t stream)
{
   using A = typename R::acc_t;
   constexpr int VEC = 16 / (int)sizeof(T) > 0 ? 16 / (int)sizeof(T) : 1;
   if (p.nout == 0 || p.relem == 0) return 0;
   DeviceInfo dev;
   if (current_device_info(&dev) != 0) return -1;
   if (!aligned_to(p.src, sizeof(T))) SD_ERROR("Tensor data must be aligned to the element size");
   // Splitting aims at one resident wave: blocks per multiprocessor that the chosen kernel can hold (asked of
   // the runtime once per kernel), never more than the RED_WANT_PER_SM that sized the scratch buffer.
   uint64_t want = (uint64_t)dev.sms * RED_WANT_PER_SM;
   // (cached per kernel AND per device: a host may hold different GPUs; a racing first call stores the same value)
   auto resident = [&](auto kernel, int (&cache)[64]) {
      int &slot = cache[(dev.device >= 0 && dev.device < 64) ? dev.device : 0];
      if (slot == 0) {
         int n = 0;
         if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, RED_THREADS, 0) != cudaSuccess) { (void)cudaGetLastError(); n = 0; }
         slot = n < 1 ? 1 : (n > RED_WANT_PER_SM ? RED_WANT_PER_SM : n);
      }
      want = (uint64_t)dev.sms * slot; };
   static int occ_row_v[64] = { 0 }, occ_row_s[64] = { 0 }, occ_col_v[64] = { 0 }, occ_col_s[64] = { 0 };
   auto pick_split = [&](uint64_t units) {                       // units: blocks the launch has without splitting
      uint64_t s = (want + units / 2) / units; if (s < 1) s = 1;
      if (s > split_cap) s = split_cap; return (uint32_t)s; };
   if (!p.buf) split_cap = 1;

   const bool row_dense = p.rdims >= 1 && p.rstride[0] == (int64_t)sizeof(T) && p.rsize[0] >= 16;
   const bool col_dense = p.ndims >= 1 && p.stride1[0] == (int64_t)sizeof(T) && p.size[0] >= 16;
   int fin_needed = 0;

   if (row_dense && (p.rsize[0] >= 128 || !col_dense)) {
      // can whole vectors be loaded?  every row start must sit on a 16-byte boundary
      bool vec = VEC > 1 && aligned_to(p.src, 16);
      for (int d = 0; d < p.ndims && vec; d++) if (p.stride1[d] % 16 != 0) vec = false;
      for (int d = 1; d < p.rdims && vec; d++) if (p.rstride[d] % 16 != 0) vec = false;
      // a warp per output when there are enough outputs to fill the machine with warps (no block
      // barrier, 32 lanes x 4 vectors in flight each), a block per output otherwise
      if (vec) resident(red_row<R, T, VEC>, occ_row_v); else resident(red_row<R, T, 1>, occ_row_s);
      p.group = (p.relem < 2048 || p.nout >= (uint64_t)dev.sms * 32) ? 32 : 256;
      p.split = pick_split((p.nout * p.group + RED_THREADS - 1) / RED_THREADS);
      {  // no more splits than whole iterations of the dense loop (the kernel rounds a split's share up to one)
         const uint64_t v = vec ? VEC : 1, per_iter = (uint64_t)p.group * (sizeof(T) >= 4 ? 8 : 4);
         const uint64_t slots = (p.relem / (uint64_t)p.rsize[0]) * (((uint64_t)p.rsize[0] + v - 1) / v);
         const uint64_t most = slots / per_iter < 1 ? 1 : slots / per_iter;
         if (p.split > most) p.split = (uint32_t)most;
      }
      uint64_t groups = p.nout * p.split;
      uint64_t gpb = RED_THREADS / p.group;
      uint64_t blocks = (groups + gpb - 1) / gpb;
      if (blocks > 0x7FFFFFFFull) SD_ERROR("Reduction grid too large");
      p.ticket = (p.nout == 1 && p.group == (uint32_t)RED_THREADS && p.split > 1) ? red_ticket_for_stream(stream) : nullptr;
      fin_needed = p.split > 1 && p.ticket == nullptr;
      if (vec) red_row<R, T, VEC><<<(unsigned)blocks, RED_THREADS, 0, stream>>>(r, p);
      else     red_row<R, T, 1><<<(unsigned)blocks, RED_THREADS, 0, stream>>>(r, p);
   } else if (col_dense) {
      bool vec = VEC > 1 && aligned_to(p.src, 16);
      for (int d = 1; d < p.ndims && vec; d++) if (p.stride1[d] % 16 != 0) vec = false;
      for (int d = 0; d < p.rdims && vec; d++) if (p.rstride[d] % 16 != 0) vec = false;
      const int v = vec ? VEC : 1;
      if (vec) resident(red_col<R, T, VEC>, occ_col_v); else resident(red_col<R, T, 1>, occ_col_s);
      // Block shape (bx, 256 / bx): x runs over adjacent outputs, y slices the reduced range.  A wide x makes every
      // row access of the block one contiguous span (4 KB at bx = 256), which keeps DRAM pages open; narrow output
      // dimensions get a narrower x so that no thread idles.
      unsigned bx = 256;
      while (bx > 32 && (uint64_t)(bx / 2) * v >= (uint64_t)p.size[0]) bx /= 2;
      p.tiles0 = ((uint64_t)p.size[0] + (uint64_t)bx * v - 1) / ((uint64_t)bx * v);
      uint64_t rest = p.nout / (uint64_t)p.size[0];
      p.split = pick_split(p.tiles0 * rest);
      uint64_t blocks = p.tiles0 * rest * p.split;
      if (blocks > 0x7FFFFFFFull) SD_ERROR("Reduction grid too large");
      dim3 bd(bx, RED_THREADS / bx);
      if (vec) red_col<R, T, VEC><<<(unsigned)blocks, bd, 0, stream>>>(r, p);
      else     red_col<R, T, 1><<<(unsigned)blocks, bd, 0, stream>>>(r, p);
      fin_needed = p.split > 1;
   } else {
      p.split = pick_split(p.nout / RED_THREADS + 1);
      uint64_t threads = p.nout * p.split;
      uint64_t blocks = (threads + RED_THREADS - 1) / RED_THREADS;
      if (blocks > 0x7FFFFFFFull) SD_ERROR("Reduction grid too large");
      red_gen<R, T><<<(unsigned)blocks, RED_THREADS, 0, stream>>>(r, p);
      fin_needed = p.split > 1;
   }
   SD_LAUNCH_CHECK();
   if (fin_needed) {
      if (p.split > 64) {
         if (p.nout > 0x7FFFFFFFull) SD_ERROR("Reduction grid too large");
         red_fin<R, RED_THREADS><<<(unsigned)p.nout, RED_THREADS, 0, stream>>>(r, p);
      } else {
         uint64_t blocks = (p.nout + (RED_THREADS / 32) - 1) / (RED_THREADS / 32);
         red_fin<R, 32><<<(unsigned)blocks, RED_THREADS, 0, stream>>>(r, p);
      }
      SD_LAUNCH_CHECK();
   }
   (void)sizeof(A);
   return 0;
}

// Launch one axis reduction from the caller's configuration (filled by
// solid_gpu_reduce_axis_prepare, scratch pointer in data.ptrBuffer).
template <class R, class T>
int reduce_axis(const R &r, solid_gpu_reduce_axis_config *config)
{
   const solid_gpu_reduce_axis_data &d = config->data;
   RedParams p;
   if (red_make_params(p, d.ndims, d.size, d.strides1, d.ptr1, d.strides2, d.ptr2,
                       d.rdims, d.rsize, d.rstrides) != 0) return -1;
   if (p.nout == 0) return 0;
   if (p.relem == 0) SD_ERROR("Axis reduction over an empty range");
   p.buf = d.ptrBuffer;
   uint32_t cap = (uint32_t)config->sharedMem;                 // split bound chosen by prepare()
   if (cap < 1 || p.buf == nullptr) cap = 1;
   if (cap > 1 && (uint64_t)sizeof(typename R::acc_t) * p.nout * cap > config->bufferSize)
      cap = (uint32_t)(config->bufferSize / (sizeof(typename R::acc_t) * p.nout));
   if (cap < 1) cap = 1;
   return red_launch<R, T>(r, p, cap, config->stream);
}

} // namespace sd
