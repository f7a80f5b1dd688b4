// Indexed access: solid_gpu_{get,set,fill}_index_<T>, solid_gpu_add_if_negative_<T>, solid_gpu_index_to_offset_<T>.
// Replaces solid/src/core/gpu/template_index.cu:30-185 with the kernel generators of
// solid/include/solid/core/gpu/index1.h and index2.h.
//
// get/set/fill move whole elements, so there is one kernel per element LAYOUT (component size x component count:
// complex elements are only aligned to their components), not per type.  A dimension either has a table of
// int64 BYTE offsets in device memory (offsets[d] != NULL: element i of that dimension lies offsets[d][i] bytes
// into the indexed tensor) or is addressed by its stride.  Positions are decomposed with 32-bit divisions
// whenever they fit; four elements per thread are in flight, their accesses a block apart.
#include "solid_core_gpu.h"
#include "dtypes.cuh"
#include "layout.h"
#include "elemwise.cuh"

namespace sd {

struct IndexParams {
   int            ndims;
   uint64_t       nelem;
   int64_t        size[MAXD];
   const int64_t *offsets[MAXD];      // device pointers, or null
   int64_t        stride1[MAXD], stride2[MAXD];
   char          *ptr1, *ptr2;        // indexed tensor; dense-strided tensor (unused by fill)
};

template <int CS> struct raw_comp;
template <> struct raw_comp<1> { using type = uint8_t; };
template <> struct raw_comp<2> { using type = uint16_t; };
template <> struct raw_comp<4> { using type = uint32_t; };
template <> struct raw_comp<8> { using type = uint64_t; };
template <int CS, int NC> struct RawElem { typename raw_comp<CS>::type c[NC]; };

constexpr int IX_THREADS = 256, IX_U = 4;
enum { IX_GET = 0, IX_SET = 1, IX_FILL = 2 };

// A thread moves IX_U groups of V consecutive positions of dimension 0.  V > 1 is used when the dense-strided
// tensor (ptr2) is contiguous and 16-byte aligned along dimension 0: its side is then one 16-byte access per
// group, and the position is decomposed once per group.  The indexed side (ptr1) is always accessed element by
// element, because the alignment of table entries (device data) is not known when the kernel is chosen.
template <int CS, int NC, int MODE, int V>
__global__ void __launch_bounds__(IX_THREADS) index_kernel(const IndexParams p, const RawElem<CS, NC> value)
{
   using C = typename raw_comp<CS>::type;
   using E = RawElem<CS, NC>;
   const uint64_t ngroups = p.nelem / V;
   const uint64_t base = (uint64_t)blockIdx.x * (IX_THREADS * IX_U) + threadIdx.x;
   const uint64_t size0 = (uint64_t)p.size[0] / V;
   const int64_t *tab0 = p.ndims > 0 ? p.offsets[0] : nullptr;
   int64_t o1[IX_U], o2[IX_U]; uint64_t c0[IX_U]; bool ok[IX_U];
#pragma unroll
   for (int u = 0; u < IX_U; u++) {
      uint64_t r = base + (uint64_t)u * IX_THREADS;
      ok[u] = r < ngroups;
      o1[u] = 0; o2[u] = 0; c0[u] = 0;
      if (ok[u] && p.ndims > 0) {
         {  const uint64_t q = udiv64(r, size0); c0[u] = (r - q * size0) * V; r = q; }
         if (MODE != IX_FILL) o2[u] = (int64_t)c0[u] * p.stride2[0];
         for (int d = 1; d < p.ndims; d++) {
            const uint64_t q = udiv64(r, (uint64_t)p.size[d]), c = r - q * (uint64_t)p.size[d]; r = q;
            const int64_t *tab = p.offsets[d];
            o1[u] += tab ? __ldg(tab + c) : (int64_t)c * p.stride1[d];
            if (MODE != IX_FILL) o2[u] += (int64_t)c * p.stride2[d];
         }
      }
   }
   // offsets of the V positions along dimension 0 on the indexed side
   int64_t d1[IX_U][V];
#pragma unroll
   for (int u = 0; u < IX_U; u++) {
#pragma unroll
      for (int j = 0; j < V; j++)
         d1[u][j] = !ok[u] ? 0 : (tab0 ? __ldg(tab0 + c0[u] + j) : (int64_t)(c0[u] + j) * p.stride1[0]);
   }
   Vec<E, V> e[IX_U];
   if (MODE == IX_FILL) {
#pragma unroll
      for (int u = 0; u < IX_U; u++) {
#pragma unroll
         for (int j = 0; j < V; j++) e[u].v[j] = value;
      }
   } else if (MODE == IX_GET) {
#pragma unroll
      for (int u = 0; u < IX_U; u++) if (ok[u]) {
#pragma unroll
         for (int j = 0; j < V; j++) {
            const C *q = reinterpret_cast<const C *>(p.ptr1 + o1[u] + d1[u][j]);
#pragma unroll
            for (int k = 0; k < NC; k++) e[u].v[j].c[k] = q[k];
         }
      }
   } else {
#pragma unroll
      for (int u = 0; u < IX_U; u++) if (ok[u]) {
         if (V > 1) e[u] = ld_vec<E, V>(p.ptr2 + o2[u]);
         else {
            const C *q = reinterpret_cast<const C *>(p.ptr2 + o2[u]);
#pragma unroll
            for (int k = 0; k < NC; k++) e[u].v[0].c[k] = q[k];
         }
      }
   }
#pragma unroll
   for (int u = 0; u < IX_U; u++) if (ok[u]) {
      if (MODE == IX_GET) {
         if (V > 1) st_vec<E, V>(p.ptr2 + o2[u], e[u]);
         else {
            C *q = reinterpret_cast<C *>(p.ptr2 + o2[u]);
#pragma unroll
            for (int k = 0; k < NC; k++) q[k] = e[u].v[0].c[k];
         }
      } else {
#pragma unroll
         for (int j = 0; j < V; j++) {
            C *q = reinterpret_cast<C *>(p.ptr1 + o1[u] + d1[u][j]);
#pragma unroll
            for (int k = 0; k < NC; k++) q[k] = e[u].v[j].c[k];
         }
      }
   }
}

// Whole runs along dimension 0 (A[:, perm], A[:, :, idx], ...): dimension 0 carries no table and both tensors are
// contiguous along it, so each position of the other dimensions is a run of size[0] elements that is copied as
// bytes.  A block owns one piece of one run: the run's two offsets (table look-ups included) are computed once per
// block instead of once per group of four elements, and the piece moves as 16-byte accesses when both of its ends are
// 16-byte aligned (a property of table entries, so it is tested on the device, uniformly for the block), else element
// by element.  The element-wise kernel above spends some fifty instructions per element on such selections (a
// gather of 32 KB runs ran at 3.5 TB/s).
constexpr int IXR_U = 4;                                       // 16-byte pieces per thread
template <int CS, int NC, int MODE>
__global__ void __launch_bounds__(IX_THREADS) index_runs_kernel(const IndexParams p, const uint4 value16, const uint32_t pieces)
{
   constexpr int ES = CS * NC;
   // block -> (run, piece)
   const uint32_t run = blockIdx.x / pieces, piece = blockIdx.x - run * pieces;
   int64_t o1 = 0, o2 = 0;
   {  uint64_t r = run;
      for (int d = 1; d < p.ndims; d++) {
         const uint64_t q = udiv64(r, (uint64_t)p.size[d]), c = r - q * (uint64_t)p.size[d]; r = q;
         const int64_t *tab = p.offsets[d];
         o1 += tab ? __ldg(tab + c) : (int64_t)c * p.stride1[d];
         if (MODE != IX_FILL) o2 += (int64_t)c * p.stride2[d];
      }
   }
   const uint64_t bytes = (uint64_t)p.size[0] * ES;
   const uint64_t span = (uint64_t)IX_THREADS * IXR_U * 16;    // bytes per piece
   const uint64_t first = (uint64_t)piece * span;
   const uint64_t len = bytes - first < span ? bytes - first : span;
   char *q1 = p.ptr1 + o1 + first;
   char *q2 = (MODE != IX_FILL) ? p.ptr2 + o2 + first : nullptr;
   const bool wide = ((reinterpret_cast<uintptr_t>(q1) | (MODE != IX_FILL ? reinterpret_cast<uintptr_t>(q2) : 0)) & 15u) == 0;
   if (wide) {
      const uint64_t nvec = len / 16;
      uint4 v[IXR_U];
#pragma unroll
      for (int u = 0; u < IXR_U; u++) {
         const uint64_t i = (uint64_t)u * IX_THREADS + threadIdx.x;
         if (MODE == IX_FILL) v[u] = value16;
         else if (i < nvec) v[u] = __ldcs(reinterpret_cast<const uint4 *>(MODE == IX_GET ? q1 : q2) + i);
      }
#pragma unroll
      for (int u = 0; u < IXR_U; u++) {
         const uint64_t i = (uint64_t)u * IX_THREADS + threadIdx.x;
         if (i < nvec) __stcs(reinterpret_cast<uint4 *>(MODE == IX_GET ? q2 : q1) + i, v[u]);
      }
      // the last bytes of the run (fewer than 16), byte by byte
      const uint64_t done = nvec * 16;
      if (done + threadIdx.x < len) {
         const uint64_t i = done + threadIdx.x;
         if (MODE == IX_FILL) q1[i] = reinterpret_cast<const char *>(&value16)[i % ES];
         else if (MODE == IX_GET) q2[i] = q1[i];
         else q1[i] = q2[i];
      }
   } else {
      // component by component (the tensors and the table entries are aligned to the components)
      using C = typename raw_comp<CS>::type;
      const uint64_t n = len / CS;
      for (uint64_t i = threadIdx.x; i < n; i += IX_THREADS) {
         if (MODE == IX_FILL) reinterpret_cast<C *>(q1)[i] = reinterpret_cast<const C *>(&value16)[i % (16 / CS)];
         else if (MODE == IX_GET) reinterpret_cast<C *>(q2)[i] = reinterpret_cast<const C *>(q1)[i];
         else reinterpret_cast<C *>(q1)[i] = reinterpret_cast<const C *>(q2)[i];
      }
   }
}

// Gather ALONG dimension 0 (A[perm, :]: a table on dimension 0, the destination contiguous there).  Element
// gathers from global memory are bound by the load unit (up to 32 sectors per warp instruction: the general kernel
// ran 4-byte gathers at 2.9 TB/s).  Here a block owns up to IXG_ROWS positions of dimension 0 for an even share of
// the runs of the destination (the grid is one resident wave, or fewer blocks with at least IXG_RUNS runs each).  It reads its slice of the table to find the span of source bytes the slice
// addresses; when that span fits the shared-memory window (a permutation of a column, a sort, a shuffle within a
// block of rows) the slice is kept in registers as 32-bit offsets from its lowest entry and, run by run, the span
// is fetched with coalesced 16-byte loads and the gather runs on shared memory; otherwise the block gathers from
// global memory directly.  The table (8 bytes per 4-byte element of ONE run) is so read twice per block
// instead of twice per run, which was what bounded the one-run form (80 us on 4-byte gathers within 32 KB columns).
// Measured on that case (8192 x 4096 floats): 256 threads with 4 / 8 / 16 runs per block 69.8 / 68.3 / 65.9 us (16 runs
// leave fewer blocks than the GPU holds), 512 threads 80-83 us, 1024 threads 101-106 us, three resident blocks by a
// register cap (80 registers, spills; also with the offsets packed two per register) 78-82 us; the copy of the next
// run's span overlapping the gather of this one (two buffers of 32 KB) 72 -> 70 us.
#ifndef IXG_THREADS_N
#define IXG_THREADS_N 256
#endif
#ifndef IXG_RUNS_N
#define IXG_RUNS_N 8
#endif
constexpr int IXG_T = IXG_THREADS_N;                           // threads of a block
constexpr int IXG_ROWS = 8192;                                 // positions of dimension 0 per block
constexpr int IXG_PER = IXG_ROWS / IXG_T;                      // ... per thread: their table entries stay in registers
constexpr int IXG_RUNS = IXG_RUNS_N;                           // fewest runs (positions of the other dimensions) a block serves with them
constexpr int IXG_WINDOW = 64 * 1024;                          // bytes of the source a block may stage per run
#ifndef IXG_MINB
#define IXG_MINB 2             // two resident blocks (128 registers): without the request the compiler takes more and one block fits
#endif
template <int CS, int NC>
__global__ void __launch_bounds__(IXG_T, IXG_MINB) index_gather0_kernel(const IndexParams p, const uint32_t chunks, const uint64_t runs,
                                                                        const uint32_t shares)
{
   constexpr int ES = CS * NC;
   constexpr int GU = IXG_PER < 8 ? IXG_PER : 8;                                      // loads a thread has in flight
   using C = typename raw_comp<CS>::type;
   extern __shared__ __align__(16) unsigned char ixg_smem[];
   __shared__ long long red_lo[IXG_T / 32], red_hi[IXG_T / 32];
   // block -> (share of the runs, chunk of dimension 0); share k of `shares` covers runs [k * runs / shares, (k + 1) * runs / shares)
   const uint32_t share = blockIdx.x / chunks, chunk = blockIdx.x - share * chunks;
   const uint64_t run_begin = (uint64_t)share * runs / shares, run_end = (uint64_t)(share + 1) * runs / shares;
   const uint64_t r0 = (uint64_t)chunk * IXG_ROWS;
   const uint32_t n = (uint64_t)p.size[0] - r0 < (uint64_t)IXG_ROWS ? (uint32_t)((uint64_t)p.size[0] - r0) : (uint32_t)IXG_ROWS;
   const int64_t *tab0 = p.offsets[0] + r0;
   // span of the slice of the table
   long long lo = 0x7FFFFFFFFFFFFFFFll, hi = -0x7FFFFFFFFFFFFFFFll - 1;
   for (uint32_t i0 = threadIdx.x; i0 < n; i0 += IXG_T * GU) {
      long long t[GU];
#pragma unroll
      for (int u = 0; u < GU; u++) { const uint32_t i = i0 + u * IXG_T; t[u] = i < n ? __ldg(tab0 + i) : lo; }
#pragma unroll
      for (int u = 0; u < GU; u++) { lo = t[u] < lo ? t[u] : lo; hi = (i0 + u * IXG_T < n && t[u] > hi) ? t[u] : hi; }
   }
#pragma unroll
   for (int d = 16; d >= 1; d >>= 1) {
      const long long l2 = __shfl_xor_sync(0xFFFFFFFFu, lo, d), h2 = __shfl_xor_sync(0xFFFFFFFFu, hi, d);
      lo = l2 < lo ? l2 : lo; hi = h2 > hi ? h2 : hi;
   }
   if ((threadIdx.x & 31) == 0) { red_lo[threadIdx.x >> 5] = lo; red_hi[threadIdx.x >> 5] = hi; }
   __syncthreads();
#pragma unroll
   for (int w = 0; w < IXG_T / 32; w++) { lo = red_lo[w] < lo ? red_lo[w] : lo; hi = red_hi[w] > hi ? red_hi[w] : hi; }
   const unsigned long long span = (unsigned long long)(hi - lo) + ES;
   const bool staged = span <= (unsigned long long)IXG_WINDOW;
   // the slice as 32-bit offsets from its lowest entry, in registers for all the runs of this block
   uint32_t rel[IXG_PER];
   if (staged) {
#pragma unroll
      for (int j = 0; j < IXG_PER; j++) { const uint32_t i = threadIdx.x + j * IXG_T; rel[j] = i < n ? (uint32_t)(__ldg(tab0 + i) - lo) : 0u; }
   }
   // offsets of run g of this block in the indexed tensor and in the destination
   auto run_offsets = [&](int g, int64_t &o1, int64_t &o2) -> bool {
      uint64_t r = run_begin + (uint64_t)g;
      if (r >= run_end) return false;
      o1 = 0; o2 = 0;
      for (int d = 1; d < p.ndims; d++) {
         const uint64_t q = udiv64(r, (uint64_t)p.size[d]), c = r - q * (uint64_t)p.size[d]; r = q;
         const int64_t *tab = p.offsets[d];
         o1 += tab ? __ldg(tab + c) : (int64_t)c * p.stride1[d];
         o2 += (int64_t)c * p.stride2[d];
      }
      return true;
   };
   if (staged) {
      // Shared-memory byte `pad + k` of a buffer mirrors source byte `lo + k` of the run, so that 16-byte chunks line
      // up.  Whole chunks travel with cp.async (no registers, the copy of the NEXT run's span overlaps the gather of
      // this one when two spans fit the window), the ragged head and tail with ordinary accesses.
      const bool two = span <= (unsigned long long)(IXG_WINDOW / 2);        // each half is IXG_WINDOW / 2 + 16 bytes, pad < 16
      auto stage = [&](int64_t o1, unsigned char *buf) -> uint32_t {
         const char *first = p.ptr1 + o1 + lo;
         const uint32_t pad = (uint32_t)(reinterpret_cast<uintptr_t>(first) & 15u);
         const uint32_t total = pad + (uint32_t)span;                               // end of the mirrored bytes
         const uint32_t head_end = pad == 0 ? 0u : (16u < total ? 16u : total);     // bytes [pad, head_end): before the first whole chunk
         const uint32_t body_end = total & ~15u;                                    // whole chunks end here
         const char *abase = first - pad;                                           // 16-byte aligned
         const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(buf);
         for (uint32_t k = (pad == 0 ? 0u : 16u) + threadIdx.x * 16u; k + 16u <= body_end; k += IXG_T * 16u)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(sbase + k), "l"(abase + k) : "memory");
         asm volatile("cp.async.commit_group;" ::: "memory");
         for (uint32_t k = pad + threadIdx.x * CS; k < head_end; k += IXG_T * CS)
            *reinterpret_cast<C *>(buf + k) = *reinterpret_cast<const C *>(abase + k);
         const uint32_t tail_from = body_end > head_end ? body_end : head_end;
         for (uint32_t k = tail_from + threadIdx.x * CS; k < total; k += IXG_T * CS)
            *reinterpret_cast<C *>(buf + k) = *reinterpret_cast<const C *>(abase + k);
         return pad;
      };
      const uint32_t second = two ? (uint32_t)(IXG_WINDOW / 2 + 16) : 0u;        // offset of the second buffer (none: the same)
      auto buffer = [&](int g) -> unsigned char * { return ixg_smem + ((g & 1) ? second : 0u); };
      int64_t o1 = 0, o2 = 0, n1 = 0, n2 = 0;
      bool have = run_offsets(0, o1, o2);
      uint32_t pad = have ? stage(o1, buffer(0)) : 0u;
      for (int g = 0; have; g++) {
         // with two buffers the next run's span is requested before this one is consumed
         bool next = run_offsets(g + 1, n1, n2);
         uint32_t npad = 0;
         if (next && two) { npad = stage(n1, buffer(g + 1)); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
         else asm volatile("cp.async.wait_group 0;" ::: "memory");
         __syncthreads();
         const unsigned char *buf = buffer(g);
         char *dst = p.ptr2 + o2 + (int64_t)r0 * ES;
#pragma unroll
         for (int j0 = 0; j0 < IXG_PER; j0 += GU) {
            RawElem<CS, NC> e[GU];
#pragma unroll
            for (int u = 0; u < GU; u++) {
               const C *q = reinterpret_cast<const C *>(buf + pad + rel[j0 + u]);
#pragma unroll
               for (int k = 0; k < NC; k++) e[u].c[k] = q[k];
            }
#pragma unroll
            for (int u = 0; u < GU; u++) {
               const uint32_t i = threadIdx.x + (j0 + u) * IXG_T;
               if (i < n) { C *o = reinterpret_cast<C *>(dst + (uint64_t)i * ES);
#pragma unroll
                  for (int k = 0; k < NC; k++) o[k] = e[u].c[k]; }
            }
         }
         __syncthreads();                                      // this buffer may be overwritten from now on
         if (next && !two) npad = stage(n1, buffer(0));
         have = next; o1 = n1; o2 = n2; pad = npad;
      }
   } else {
      for (int g = 0; ; g++) {
         int64_t o1, o2;
         if (!run_offsets(g, o1, o2)) break;
         const char *src = p.ptr1 + o1;
         char *dst = p.ptr2 + o2 + (int64_t)r0 * ES;
         for (uint32_t i0 = threadIdx.x; i0 < n; i0 += IXG_T * GU) {
            long long t[GU]; RawElem<CS, NC> e[GU];
#pragma unroll
            for (int u = 0; u < GU; u++) { const uint32_t i = i0 + u * IXG_T; t[u] = i < n ? __ldg(tab0 + i) : lo; }
#pragma unroll
            for (int u = 0; u < GU; u++) {
               const C *q = reinterpret_cast<const C *>(src + t[u]);
#pragma unroll
               for (int k = 0; k < NC; k++) e[u].c[k] = q[k];
            }
#pragma unroll
            for (int u = 0; u < GU; u++) {
               const uint32_t i = i0 + u * IXG_T;
               if (i < n) { C *o = reinterpret_cast<C *>(dst + (uint64_t)i * ES);
#pragma unroll
                  for (int k = 0; k < NC; k++) o[k] = e[u].c[k]; }
            }
         }
      }
   }
}

template <int CS, int NC, int MODE>
int index_launch(int ndims, const size_t *size, solid_int64 **offsets, const ptrdiff_t *strides1, void *ptr1,
                 const ptrdiff_t *strides2, void *ptr2, const solid_scalar *value, cudaStream_t stream)
{
   constexpr int ES = CS * NC;
   constexpr int V = 16 / ES > 1 ? 16 / ES : 1;
   if (ndims < 0 || ndims > MAXD) SD_ERROR("Number of dimensions (%d) exceeds the maximum of %d", ndims, MAXD);
   IndexParams p; memset(&p, 0, sizeof(p));
   p.ndims = ndims; p.nelem = 1; p.ptr1 = (char *)ptr1; p.ptr2 = (char *)ptr2;
   for (int d = 0; d < ndims; d++) {
      p.size[d] = (int64_t)size[d]; p.nelem *= (uint64_t)size[d];
      p.offsets[d] = offsets ? offsets[d] : nullptr;
      p.stride1[d] = strides1 ? strides1[d] : 0;
      p.stride2[d] = (MODE != IX_FILL && strides2) ? strides2[d] : 0;
   }
   if (p.nelem == 0) return 0;
   if (!aligned_to(ptr1, CS) || (MODE != IX_FILL && !aligned_to(ptr2, CS))) SD_ERROR("Tensor data must be aligned to the element size");
   RawElem<CS, NC> v; memset(&v, 0, sizeof(v));
   if (value) memcpy(&v, value, sizeof(v));
   // whole runs along dimension 0 (no table there, both sides contiguous, at least 1 KB long): copied as bytes
   if (ndims > 0 && (offsets == nullptr || offsets[0] == nullptr) && p.stride1[0] == ES &&
       (MODE == IX_FILL || p.stride2[0] == ES) && (uint64_t)size[0] * ES >= 1024) {
      const uint64_t span = (uint64_t)IX_THREADS * IXR_U * 16;
      const uint64_t pieces = ((uint64_t)size[0] * ES + span - 1) / span;
      const uint64_t runs = p.nelem / (uint64_t)size[0];
      if (pieces <= 0xFFFFFFFFull && runs * pieces <= 0x7FFFFFFFull) {
         uint4 value16;
         for (int i = 0; i < 16 / ES; i++) memcpy(reinterpret_cast<char *>(&value16) + i * ES, &v, ES);
         index_runs_kernel<CS, NC, MODE><<<(unsigned)(runs * pieces), IX_THREADS, 0, stream>>>(p, value16, (uint32_t)pieces);
         SD_LAUNCH_CHECK();
         return 0;
      }
   }
   // gather along dimension 0 into a destination that is contiguous there
   if (MODE == IX_GET && ndims > 0 && offsets != nullptr && offsets[0] != nullptr && p.stride2[0] == ES && size[0] >= 256) {
      const uint64_t chunks = ((uint64_t)size[0] + IXG_ROWS - 1) / IXG_ROWS;
      const uint64_t runs = p.nelem / (uint64_t)size[0];
      // one resident wave of blocks: each keeps its slice of the table for an even share of the runs (at least
      // IXG_RUNS of them, so that the two passes over the slice are spread over several runs)
      DeviceInfo dev;
      if (current_device_info(&dev) != 0) return -1;
      uint64_t shares = (uint64_t)dev.sms * IXG_MINB / chunks;
      if (shares > (runs + IXG_RUNS - 1) / IXG_RUNS) shares = (runs + IXG_RUNS - 1) / IXG_RUNS;
      if (shares < 1) shares = 1;
      if (chunks <= 0xFFFFFFFFull && shares * chunks <= 0x7FFFFFFFull) {
         static bool attr_set = false;
         const size_t smem = IXG_WINDOW + 32;                   // one span of up to 64 KB, or two of up to 32 KB, each with its alignment pad
         if (!attr_set) {
            SD_CUDA_CHECK(cudaFuncSetAttribute(index_gather0_kernel<CS, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            attr_set = true;
         }
         index_gather0_kernel<CS, NC><<<(unsigned)(shares * chunks), IXG_T, smem, stream>>>(p, (uint32_t)chunks, runs, (uint32_t)shares);
         SD_LAUNCH_CHECK();
         return 0;
      }
   }
   // groups of V along dimension 0: the dense-strided side must be contiguous there and 16-byte aligned everywhere
   bool vec = V > 1 && ndims > 0 && size[0] % V == 0;
   if (vec && MODE != IX_FILL) {
      vec = p.stride2[0] == ES && aligned_to(ptr2, 16);
      for (int d = 1; d < ndims && vec; d++) if (p.stride2[d] % 16 != 0) vec = false;
   }
   const uint64_t groups = p.nelem / (vec ? V : 1);
   const uint64_t blocks = (groups + IX_THREADS * IX_U - 1) / (IX_THREADS * IX_U);
   if (blocks > 0x7FFFFFFFull) SD_ERROR("Indexed tensor too large for one launch");
   if (vec) index_kernel<CS, NC, MODE, V><<<(unsigned)blocks, IX_THREADS, 0, stream>>>(p, v);
   else     index_kernel<CS, NC, MODE, 1><<<(unsigned)blocks, IX_THREADS, 0, stream>>>(p, v);
   SD_LAUNCH_CHECK();
   return 0;
}

// element layouts of the fifteen types: component bytes, component count
template <class T> struct elem_layout { static constexpr int CS = sizeof(T), NC = 1; };
template <class E> struct elem_layout<Cplx<E>> { static constexpr int CS = sizeof(E), NC = 2; };

// ---- add_if_negative: x < 0 ? x + value : x, in place (signed integers; used to wrap negative indices)
template <class T> struct AddIfNegativeApply {
   static constexpr int NIN = 1;
   using in1_t = T; using in2_t = Nothing; using out_t = T;
   T v;
   SD_D T operator()(T x, Nothing) const { return x < 0 ? (T)(x + v) : x; }
};

// ---- index_to_offset: out[e] = sum_i strides[i] * index[e][i]
struct OffsetParams { int nstrides; int64_t strides[MAXD]; int64_t stride_reduce, stride1, stride2; uint64_t nelem; const char *src; char *dst; };
template <class T>
__global__ void __launch_bounds__(256) index_to_offset_kernel(const OffsetParams p)
{
   const uint64_t e = (uint64_t)blockIdx.x * 256 + threadIdx.x;
   if (e >= p.nelem) return;
   const char *q = p.src + (int64_t)e * p.stride1;
   int64_t s = 0;
   for (int i = 0; i < p.nstrides; i++) s += p.strides[i] * (int64_t)ld_one<T>(q + i * p.stride_reduce);
   *reinterpret_cast<int64_t *>(p.dst + (int64_t)e * p.stride2) = s;
}

} // namespace sd

#define SD_IX_TYPE(TYPE) sd::ctype_of_##TYPE
namespace sd {
using ctype_of_bool = Bool; using ctype_of_uint8 = uint8_t; using ctype_of_uint16 = uint16_t; using ctype_of_uint32 = uint32_t;
using ctype_of_uint64 = uint64_t; using ctype_of_int8 = int8_t; using ctype_of_int16 = int16_t; using ctype_of_int32 = int32_t;
using ctype_of_int64 = int64_t; using ctype_of_half = Half; using ctype_of_float = float; using ctype_of_double = double;
using ctype_of_chalf = CHalf; using ctype_of_cfloat = CFloat; using ctype_of_cdouble = CDouble;
}

#define SD_DEFINE_INDEX(U, TYPE)                                                                                      \
   extern "C" int solid_gpu_get_index_##TYPE(SOLID_GPU_ARGS_INDEX2)                                                   \
   {  using L = sd::elem_layout<SD_IX_TYPE(TYPE)>;                                                                    \
      return sd::index_launch<L::CS, L::NC, sd::IX_GET>(ndims, size, offsets, strides1, ptr1, strides2, ptr2, nullptr, stream); } \
   extern "C" int solid_gpu_set_index_##TYPE(SOLID_GPU_ARGS_INDEX2)                                                   \
   {  using L = sd::elem_layout<SD_IX_TYPE(TYPE)>;                                                                    \
      return sd::index_launch<L::CS, L::NC, sd::IX_SET>(ndims, size, offsets, strides1, ptr1, strides2, ptr2, nullptr, stream); } \
   extern "C" int solid_gpu_fill_index_##TYPE(SOLID_GPU_ARGS_FILL_INDEX)                                              \
   {  using L = sd::elem_layout<SD_IX_TYPE(TYPE)>;                                                                    \
      return sd::index_launch<L::CS, L::NC, sd::IX_FILL>(ndims, size, offsets, strides, ptr, nullptr, nullptr, &value, stream); }
SOLID_TYPES_all(SD_DEFINE_INDEX, u)

#define SD_DEFINE_ADD_IF_NEGATIVE(U, TYPE)                                                                            \
   extern "C" int solid_gpu_add_if_negative_##TYPE(SOLID_GPU_ARGS_ADD_IF_NEGATIVE)                                    \
   {  using T = SD_IX_TYPE(TYPE);                                                                                     \
      const ptrdiff_t *st[2] = { strides, strides }; void *pt[2] = { ptr, ptr };                                      \
      sd::Layout<2> L;                                                                                                \
      if (sd::make_layout<2>(L, ndims, size, st, pt, 1) != 0) return -1;                                              \
      sd::AddIfNegativeApply<T> ap; memcpy(&ap.v, &value, sizeof(T));                                                 \
      return sd::ew_launch(ap, L, stream); }
SOLID_TYPES_sint(SD_DEFINE_ADD_IF_NEGATIVE, u)

#define SD_DEFINE_INDEX_TO_OFFSET(U, TYPE)                                                                            \
   extern "C" int solid_gpu_index_to_offset_##TYPE(SOLID_GPU_ARGS_INDEX_TO_OFFSET)                                    \
   {  using T = SD_IX_TYPE(TYPE);                                                                                     \
      if (nstrides < 0 || nstrides > sd::MAXD) SD_ERROR("Number of strides (%d) exceeds the maximum of %d", nstrides, sd::MAXD); \
      if (nelem == 0) return 0;                                                                                       \
      if (!sd::aligned_to(ptr1, sizeof(T)) || !sd::aligned_to(ptr2, 8)) SD_ERROR("Tensor data must be aligned to the element size"); \
      sd::OffsetParams p; memset(&p, 0, sizeof(p));                                                                   \
      p.nstrides = nstrides; for (int i = 0; i < nstrides; i++) p.strides[i] = strides[i];                            \
      p.stride_reduce = strideReduce; p.stride1 = stride1; p.stride2 = stride2; p.nelem = nelem;                      \
      p.src = (const char *)ptr1; p.dst = (char *)ptr2;                                                               \
      const uint64_t blocks = ((uint64_t)nelem + 255) / 256;                                                          \
      if (blocks > 0x7FFFFFFFull) SD_ERROR("index_to_offset: too many elements for one launch");                      \
      sd::index_to_offset_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(p);                                         \
      SD_LAUNCH_CHECK();                                                                                              \
      return 0; }
SOLID_TYPES_integer(SD_DEFINE_INDEX_TO_OFFSET, u)
