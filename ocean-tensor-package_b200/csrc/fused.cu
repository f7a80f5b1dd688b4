// Fused entry points that the reference can only express as sequences of kernels
// with temporaries:
//
//   solid_gpu_axpy_sums_<float|double>   z = a*x + y, sum(z), sum(z*z) in one pass
//        (reference: OcTensor_multiplyScalar -> Tensor_scale, Tensor_add,
//         Tensor_sum, Tensor_norm2: src/core/interface/tensor_itf.c:4221-4251,
//         5299-5351,5405-5447; 28 bytes of traffic per element against 12 here)
//   solid_gpu_mixed_multiply_add         dst = (dsttype)((ctype)a * (ctype)b + (ctype)c)
//        with per-operand dtype, byte order, alignment and strides
//        (reference: every operand is first converted into a temporary of the
//         common type by Tensor_copy, src/core/generic/tensor_op.c:170-186, then
//         Tensor_scale, Tensor_add and a final converting copy)
//
// Both reproduce the reference's sequence of roundings: the product is rounded
// to the compute type before the addition (no FMA), and the result is rounded
// once more when it is stored in a narrower type.
#include "solid_core_gpu.h"
#include "dtypes.cuh"
#include "layout.h"
#include "reduce.cuh"

namespace sd {

// ===========================================================================
// axpy + sums
// ===========================================================================
#ifndef AX_THREADS_N
#define AX_THREADS_N 256
#endif
#ifndef AX_VECTORS
#define AX_VECTORS 4
#endif
// 256 threads x 4 vectors per operand (16 KB of x per block).  Other shapes on 2^30 floats, stand-alone: 256 x 2 7061,
// 256 x 8 7076, 128 x 4 7039, 512 x 4 7109, 512 x 2 7159, 1024 x 2 5849 against 7091 GB/s; 512 x 2 was then tried in
// the bench and was 0.2-0.4 % SLOWER there (7.269 against 7.258 ms on 2^32 elements), so the shape stayed.
constexpr int AX_THREADS = AX_THREADS_N;
constexpr int AX_U = AX_VECTORS;             // 16-byte vectors per thread and operand
constexpr int AX_FOLD = 1024;                // per-block pairs folded into one second-level pair

template <class T> struct Sums { T s, s2; };

// Fold of `count` pairs starting at `part`, by the whole block, in a fixed order: thread t adds entries t,
// t + 256, ..., the block tree joins the threads.  Thread 0 returns the result.
template <class T>
SD_D Sums<T> axpy_fold(const Sums<T> *part, uint64_t count, Sums<T> *smem)
{
   // Four pairs per thread are fetched before any is added (one load per pair): the fold is a chain of memory
   // latencies, not of bandwidth.  The order of the additions is fixed by the indices alone.
   using Pair = typename chunk_of<sizeof(Sums<T>) >= 16 ? 16 : 8>::type;
   static_assert(sizeof(Sums<T>) == sizeof(Pair), "a pair is one 8- or 16-byte access");
   T s = 0, s2 = 0;
   for (uint64_t i = threadIdx.x; i < count; i += 4 * AX_THREADS) {
      Pair raw[4];
#pragma unroll
      for (int k = 0; k < 4; k++)                                        // possibly written by other blocks: past the L1 cache
         if (i + (uint64_t)k * AX_THREADS < count) raw[k] = __ldcg(reinterpret_cast<const Pair *>(part + i + (uint64_t)k * AX_THREADS));
#pragma unroll
      for (int k = 0; k < 4; k++)
         if (i + (uint64_t)k * AX_THREADS < count) { Sums<T> v; memcpy(&v, &raw[k], sizeof(v)); s += v.s; s2 += v.s2; }
   }
#pragma unroll
   for (int d = 16; d >= 1; d >>= 1) {
      s  += __shfl_down_sync(0xFFFFFFFFu, s, d);
      s2 += __shfl_down_sync(0xFFFFFFFFu, s2, d);
   }
   const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
   __syncthreads();                              // smem may still be read from the previous use
   if (lane == 0) { smem[warp].s = s; smem[warp].s2 = s2; }
   __syncthreads();
   if (threadIdx.x == 0) for (int w = 1; w < AX_THREADS / 32; w++) { s += smem[w].s; s2 += smem[w].s2; }
   Sums<T> r; r.s = s; r.s2 = s2;
   return r;
}

template <class T>
__global__ void __launch_bounds__(AX_THREADS) axpy_sums_kernel(uint64_t n, T a, const T *__restrict__ x,
                                                               const T *__restrict__ y, T *__restrict__ z,
                                                               Sums<T> *__restrict__ partials)
{
   constexpr int VEC = 16 / sizeof(T), U = AX_U;
   __shared__ Sums<T> smem[AX_THREADS / 32];
   const uint64_t nvec = n / VEC;
   const uint64_t chunk = (uint64_t)AX_THREADS * U;
   T s = 0, s2 = 0;
   for (uint64_t base = (uint64_t)blockIdx.x * chunk; base < nvec; base += (uint64_t)gridDim.x * chunk) {
      Vec<T, VEC> vx[U], vy[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
         uint64_t i = base + (uint64_t)u * AX_THREADS + threadIdx.x;
         if (i < nvec) { vx[u] = ld_vec<T, VEC>(x + i * VEC); vy[u] = ld_vec<T, VEC>(y + i * VEC); }
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
         uint64_t i = base + (uint64_t)u * AX_THREADS + threadIdx.x;
         if (i < nvec) {
            Vec<T, VEC> vz;
#pragma unroll
            for (int j = 0; j < VEC; j++) {
               T p = a * vx[u].v[j];            // rounded product (Tensor_scale)
               T w = p + vy[u].v[j];            // rounded sum (Tensor_add)
               vz.v[j] = w; s += w; s2 += w * w;
            }
            st_vec<T, VEC>(z + i * VEC, vz);
         }
      }
   }
   if (blockIdx.x == 0) {                        // ragged tail
      uint64_t i = nvec * VEC + threadIdx.x;
      if (i < n) { T p = a * x[i]; T w = p + y[i]; z[i] = w; s += w; s2 += w * w; }
   }
   // block fold in fixed order
#pragma unroll
   for (int d = 16; d >= 1; d >>= 1) {
      s  += __shfl_down_sync(0xFFFFFFFFu, s, d);
      s2 += __shfl_down_sync(0xFFFFFFFFu, s2, d);
   }
   const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
   if (lane == 0) { smem[warp].s = s; smem[warp].s2 = s2; }
   __syncthreads();
   if (threadIdx.x == 0) {
      for (int w = 1; w < AX_THREADS / 32; w++) { s += smem[w].s; s2 += smem[w].s2; }
      partials[blockIdx.x].s = s; partials[blockIdx.x].s2 = s2;
   }
}

// Both fold levels in ONE launch: block g folds the pairs of group g (AX_FOLD of them) into a second-level pair and
// announces it on the stream's arrival counter; the block that arrives last folds the second-level pairs into the
// result and leaves the counter at zero.  WHICH block does the last fold depends on timing, WHAT it adds and in which
// order does not, so the sums are the same on every run (and the same as with the two separate fold launches).
// (Counting arrivals inside the streaming kernel instead, one atomic per 16 KB block, was measured: 3.7 % slower on
// 2^32 elements, far more than the launch it saves.)
template <class T>
__global__ void __launch_bounds__(AX_THREADS) axpy_sums_fold(uint64_t nparts, unsigned int ngroups, unsigned int *ticket,
                                                             const Sums<T> *__restrict__ partials,
                                                             Sums<T> *__restrict__ level2, Sums<T> *__restrict__ out)
{
   __shared__ Sums<T> smem[AX_THREADS / 32];
   __shared__ unsigned int arrived;
   const uint64_t first = (uint64_t)blockIdx.x * AX_FOLD;
   const uint64_t count = nparts - first < (uint64_t)AX_FOLD ? nparts - first : (uint64_t)AX_FOLD;
   Sums<T> g = axpy_fold<T>(partials + first, count, smem);
   if (ngroups == 1u) { if (threadIdx.x == 0) *out = g; return; }
   if (threadIdx.x == 0) { level2[blockIdx.x] = g; __threadfence(); arrived = atomicAdd(ticket, 1u) + 1u; }
   __syncthreads();
   if (arrived != ngroups) return;
   __threadfence();
   g = axpy_fold<T>(level2, ngroups, smem);
   if (threadIdx.x == 0) { *out = g; *ticket = 0u; }
}

// Fold of the per-block partials, in fixed order: block b takes partials [b*fold, (b+1)*fold), thread t
// of it adds entries t, t+256, ... and the block tree joins the threads.  The streaming kernel runs one
// chunk per block (measured on B200: 7.1 TB/s against 6.4 TB/s for a grid of resident blocks that
// stride through the arrays), so a large tensor leaves up to a million partials; they are folded in two
// levels, AX_FOLD to one and then the rest in a single block.
template <class T>
__global__ void __launch_bounds__(AX_THREADS) axpy_sums_finish(uint64_t nparts, int fold,
                                                               const Sums<T> *__restrict__ partials,
                                                               Sums<T> *__restrict__ out)
{
   __shared__ Sums<T> smem[AX_THREADS / 32];
   const uint64_t first = (uint64_t)blockIdx.x * fold;
   uint64_t last = first + fold; if (last > nparts) last = nparts;
   T s = 0, s2 = 0;
   for (uint64_t i = first + threadIdx.x; i < last; i += AX_THREADS) { s += partials[i].s; s2 += partials[i].s2; }
#pragma unroll
   for (int d = 16; d >= 1; d >>= 1) {
      s  += __shfl_down_sync(0xFFFFFFFFu, s, d);
      s2 += __shfl_down_sync(0xFFFFFFFFu, s2, d);
   }
   const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
   if (lane == 0) { smem[warp].s = s; smem[warp].s2 = s2; }
   __syncthreads();
   if (threadIdx.x == 0) {
      for (int w = 1; w < AX_THREADS / 32; w++) { s += smem[w].s; s2 += smem[w].s2; }
      out[blockIdx.x].s = s; out[blockIdx.x].s2 = s2;
   }
}

// Blocks of the streaming kernel for n elements of `elemsize` bytes: one chunk each, within the grid limit.
static uint64_t axpy_sums_blocks(uint64_t n, size_t elemsize)
{
   const uint64_t vec = 16 / elemsize, chunk = (uint64_t)AX_THREADS * AX_U * vec;
   uint64_t blocks = (n + chunk - 1) / chunk;
   if (blocks < 1) blocks = 1;
   if (blocks > 0x7FFFFFFFull) blocks = 0x7FFFFFFFull;
   return blocks;
}
static uint64_t axpy_sums_level2(uint64_t blocks) { return blocks > (uint64_t)AX_FOLD ? (blocks + AX_FOLD - 1) / AX_FOLD : 0; }

template <class T>
int axpy_sums(size_t n, T a, const void *x, const void *y, void *z, void *sums, void *partials, cudaStream_t stream)
{
   if (!aligned_to(x, 16) || !aligned_to(y, 16) || !aligned_to(z, 16))
      SD_ERROR("axpy_sums needs 16-byte aligned tensors");
   if (sums == nullptr || partials == nullptr) SD_ERROR("axpy_sums needs the sums and partials buffers");
   const uint64_t blocks = axpy_sums_blocks((uint64_t)n, sizeof(T)), level2 = axpy_sums_level2(blocks);
   Sums<T> *p1 = (Sums<T> *)partials, *p2 = p1 + blocks;
   axpy_sums_kernel<T><<<(unsigned)blocks, AX_THREADS, 0, stream>>>((uint64_t)n, a, (const T *)x, (const T *)y, (T *)z, p1);
   SD_LAUNCH_CHECK();
   // one fold launch when the stream has an arrival counter (every stream but the per-thread default one)
   const uint64_t ngroups = (blocks + AX_FOLD - 1) / AX_FOLD;
   unsigned int *ticket = ngroups > 1 ? red_ticket_for_stream(stream) : nullptr;
   if (ngroups == 1 || ticket != nullptr) {
      axpy_sums_fold<T><<<(unsigned)ngroups, AX_THREADS, 0, stream>>>(blocks, (unsigned)ngroups, ticket, p1, p2, (Sums<T> *)sums);
      SD_LAUNCH_CHECK();
      return 0;
   }
   if (level2) {
      axpy_sums_finish<T><<<(unsigned)level2, AX_THREADS, 0, stream>>>(blocks, AX_FOLD, p1, p2);
      SD_LAUNCH_CHECK();
      axpy_sums_finish<T><<<1, AX_THREADS, 0, stream>>>(level2, (int)level2, p2, (Sums<T> *)sums);
   } else {
      axpy_sums_finish<T><<<1, AX_THREADS, 0, stream>>>(blocks, (int)blocks, p1, (Sums<T> *)sums);
   }
   SD_LAUNCH_CHECK();
   return 0;
}

// ===========================================================================
// mixed multiply-add
// ===========================================================================
struct MixParams {
   char    *ptr[4];             // a, b, c, dst
   int      dtype[4];
   int      swap[4];
   int      unal[4];
   int      comp[4];            // bytes of one real component
   int64_t  stride[4][MAXD];
   int64_t  size[MAXD];
   int      ndims;
   int      dt;                 // dimension along which the staged operands are dense
   uint32_t staged;             // bit k: operand k goes through the shared-memory tile
   uint64_t nelem;
   uint64_t tiles0, tilest;
   FastDiv  div_tiles0, div_tilest;   // the grid has fewer than 2^31 blocks, so both counts fit 32 bits
   int      anyunal;            // some operand is not aligned to its component size
};

// Operand access is split in two so that a thread can issue many loads before it
// consumes any: load_bits fetches the raw bytes of one real component (complex
// operands contribute their real part only), bits_as converts them to the compute
// type.  Both switch on values that are uniform over the launch.
SD_D uint64_t load_bits(const char *p, int comp_size, bool unal)
{
   if (unal) {
      uint64_t r = 0;
      for (int i = 0; i < comp_size; i++) r |= (uint64_t)__ldg(reinterpret_cast<const uint8_t *>(p) + i) << (8 * i);
      return r;
   }
   switch (comp_size) {
      case 1:  return ld_one<uint8_t>(p);
      case 2:  return ld_one<uint16_t>(p);
      case 4:  return ld_one<uint32_t>(p);
      default: return ld_one<uint64_t>(p);
   }
}
template <class S> SD_D S bits_typed(uint64_t raw, bool swap)
{
   typename raw_of<sizeof(S)>::type u = (typename raw_of<sizeof(S)>::type)raw;
   S x; memcpy(&x, &u, sizeof(S));
   if (swap) x = bswap_real(x);
   return x;
}
// Raw component bits of runtime type `dtype` as compute type C.
template <class C> SD_D C bits_as(uint64_t raw, int dtype, bool swap)
{
   switch (dtype) {
      case 0:  return convert<C>(bits_typed<Bool>(raw, swap));
      case 1:  return convert<C>(bits_typed<uint8_t>(raw, swap));
      case 2:  return convert<C>(bits_typed<uint16_t>(raw, swap));
      case 3:  return convert<C>(bits_typed<uint32_t>(raw, swap));
      case 4:  return convert<C>(bits_typed<uint64_t>(raw, swap));
      case 5:  return convert<C>(bits_typed<int8_t>(raw, swap));
      case 6:  return convert<C>(bits_typed<int16_t>(raw, swap));
      case 7:  return convert<C>(bits_typed<int32_t>(raw, swap));
      case 8:  return convert<C>(bits_typed<int64_t>(raw, swap));
      case 9:  case 12: return convert<C>(bits_typed<Half>(raw, swap));
      case 10: case 13: return convert<C>(bits_typed<float>(raw, swap));
      default: return convert<C>(bits_typed<double>(raw, swap));
   }
}
// Array forms: ONE switch around the unrolled element loop.  (A switch per element inside a
// fully unrolled loop multiplies the code of every case by the unroll factor; the kernels then
// stall on instruction fetch instead of on memory.)
template <int N> SD_D void load_bits_n(const char *const (&q)[N], const bool (&ok)[N], int comp_size, bool unal, uint64_t (&raw)[N])
{
   if (unal) {
#pragma unroll
      for (int j = 0; j < N; j++) raw[j] = ok[j] ? load_bits(q[j], comp_size, true) : 0;
      return;
   }
   switch (comp_size) {
      case 1:
#pragma unroll
         for (int j = 0; j < N; j++) raw[j] = ok[j] ? ld_one<uint8_t>(q[j]) : 0;
         break;
      case 2:
#pragma unroll
         for (int j = 0; j < N; j++) raw[j] = ok[j] ? ld_one<uint16_t>(q[j]) : 0;
         break;
      case 4:
#pragma unroll
         for (int j = 0; j < N; j++) raw[j] = ok[j] ? ld_one<uint32_t>(q[j]) : 0;
         break;
      default:
#pragma unroll
         for (int j = 0; j < N; j++) raw[j] = ok[j] ? ld_one<uint64_t>(q[j]) : 0;
         break;
   }
}
#define SD_BITS_CASE(TYPE)                                                             \
   _Pragma("unroll") for (int j = 0; j < N; j++) out[j] = convert<C>(bits_typed<TYPE>(raw[j], swap)); break;
template <class C, int N> SD_D void bits_as_n(const uint64_t (&raw)[N], int dtype, bool swap, C (&out)[N])
{
   switch (dtype) {
      case 0:  SD_BITS_CASE(Bool)
      case 1:  SD_BITS_CASE(uint8_t)
      case 2:  SD_BITS_CASE(uint16_t)
      case 3:  SD_BITS_CASE(uint32_t)
      case 4:  SD_BITS_CASE(uint64_t)
      case 5:  SD_BITS_CASE(int8_t)
      case 6:  SD_BITS_CASE(int16_t)
      case 7:  SD_BITS_CASE(int32_t)
      case 8:  SD_BITS_CASE(int64_t)
      case 9:  case 12: SD_BITS_CASE(Half)
      case 10: case 13: SD_BITS_CASE(float)
      default: SD_BITS_CASE(double)
   }
}
#undef SD_BITS_CASE
template <class D, class C> SD_D void store_typed(char *p, C v, bool swap, bool unal)
{
   D y = convert<D>(v);
   if (swap) y = bswap<D>(y);
   if (!unal) st_one<D>(p, y);
   else { uint8_t b[sizeof(D)]; memcpy(b, &y, sizeof(D));
#pragma unroll
      for (int i = 0; i < (int)sizeof(D); i++) reinterpret_cast<uint8_t *>(p)[i] = b[i]; }
}
#define SD_STORE_CASE(TYPE)                                                            \
   _Pragma("unroll") for (int j = 0; j < N; j++) if (ok[j]) store_typed<TYPE>(q[j], v[j], swap, unal); break;
template <class C, int N> SD_D void store_as_n(char *const (&q)[N], const bool (&ok)[N], int dtype, const C (&v)[N], bool swap, bool unal)
{
   switch (dtype) {
      case 0:  SD_STORE_CASE(Bool)
      case 1:  SD_STORE_CASE(uint8_t)
      case 2:  SD_STORE_CASE(uint16_t)
      case 3:  SD_STORE_CASE(uint32_t)
      case 4:  SD_STORE_CASE(uint64_t)
      case 5:  SD_STORE_CASE(int8_t)
      case 6:  SD_STORE_CASE(int16_t)
      case 7:  SD_STORE_CASE(int32_t)
      case 8:  SD_STORE_CASE(int64_t)
      case 9:  SD_STORE_CASE(Half)
      case 10: SD_STORE_CASE(float)
      case 11: SD_STORE_CASE(double)
      case 12: SD_STORE_CASE(CHalf)
      case 13: SD_STORE_CASE(CFloat)
      default: SD_STORE_CASE(CDouble)
   }
}
#undef SD_STORE_CASE
template <class C> SD_D void store_as(char *p, int dtype, C v, bool swap, bool unal)
{
   switch (dtype) {
      case 0:  store_typed<Bool>(p, v, swap, unal); break;
      case 1:  store_typed<uint8_t>(p, v, swap, unal); break;
      case 2:  store_typed<uint16_t>(p, v, swap, unal); break;
      case 3:  store_typed<uint32_t>(p, v, swap, unal); break;
      case 4:  store_typed<uint64_t>(p, v, swap, unal); break;
      case 5:  store_typed<int8_t>(p, v, swap, unal); break;
      case 6:  store_typed<int16_t>(p, v, swap, unal); break;
      case 7:  store_typed<int32_t>(p, v, swap, unal); break;
      case 8:  store_typed<int64_t>(p, v, swap, unal); break;
      case 9:  store_typed<Half>(p, v, swap, unal); break;
      case 10: store_typed<float>(p, v, swap, unal); break;
      case 11: store_typed<double>(p, v, swap, unal); break;
      case 12: store_typed<CHalf>(p, v, swap, unal); break;
      case 13: store_typed<CFloat>(p, v, swap, unal); break;
      default: store_typed<CDouble>(p, v, swap, unal); break;
   }
}

// Linear variant for one merged dimension: a block handles 256 x MR consecutive elements, a
// thread MR of them 256 apart (coalesced), all loads issued before the first conversion.
// Tile of the tiled variant.  Measured on B200 (4096^2, f64 transposed x i32 byte-swapped + f32 row -> f32): the
// shape (16x128, 32x64, 64x32) makes no difference, resident warps do: 3, 4, 5, 6 blocks of 256 threads per
// multiprocessor ran at 78, 68, 62, 65 us, so the kernel is built for five (48 registers, a few spills).
#ifndef MIX_M0
#define MIX_M0 32
#define MIX_M1 64
#define MIX_NT 256
#ifndef MIX_BLOCKS
#define MIX_BLOCKS 5
#endif
#endif
constexpr int M0 = MIX_M0;                  // tile extent along dimension 0
constexpr int M1 = MIX_M1;                  // tile extent along dimension dt
constexpr int MT = MIX_NT;                  // threads of a tile
#ifndef MIX_MR
#define MIX_MR 8
#endif
constexpr int MR = MIX_MR;                  // elements per thread and operand
static_assert(M0 * M1 == MT * MR, "tile and thread count do not match");
constexpr int MP1 = MT / M1;                // rows of dimension 0 per pass of phase 1
constexpr int MP2 = MT / M0;                // rows of dimension dt per pass of phase 2

template <class C>
__global__ void __launch_bounds__(256) mix_linear(const MixParams p)
{
   const uint64_t chunk = 256ull * MR;
   for (uint64_t base = (uint64_t)blockIdx.x * chunk; base < p.nelem; base += (uint64_t)gridDim.x * chunk) {
      bool ok[MR];
#pragma unroll
      for (int j = 0; j < MR; j++) ok[j] = base + threadIdx.x + 256ull * j < p.nelem;
      C acc[MR];
#pragma unroll
      for (int k = 0; k < 3; k++) {
         const char *q[MR];
#pragma unroll
         for (int j = 0; j < MR; j++) q[j] = p.ptr[k] + (int64_t)(base + threadIdx.x + 256ull * j) * p.stride[k][0];
         uint64_t raw[MR]; C v[MR];
         load_bits_n<MR>(q, ok, p.comp[k], p.unal[k], raw);
         bits_as_n<C, MR>(raw, p.dtype[k], p.swap[k], v);
#pragma unroll
         for (int j = 0; j < MR; j++) acc[j] = (k == 0) ? v[j] : (k == 1 ? acc[j] * v[j] : acc[j] + v[j]);
      }
      char *qo[MR];
#pragma unroll
      for (int j = 0; j < MR; j++) qo[j] = p.ptr[3] + (int64_t)(base + threadIdx.x + 256ull * j) * p.stride[3][0];
      store_as_n<C, MR>(qo, ok, p.dtype[3], acc, p.swap[3], p.unal[3]);
   }
}

// Byte reversal under a run-time flag without a second copy of the code: the permutation selector is data.
template <class S> SD_D S maybe_bswap(S x, bool swap)
{
   if constexpr (sizeof(S) == 1) return x;
   else if constexpr (sizeof(S) == 2) {
      uint16_t u; memcpy(&u, &x, 2);
      u = (uint16_t)__byte_perm((uint32_t)u, 0u, swap ? 0x3201u : 0x3210u);
      memcpy(&x, &u, 2); return x;
   } else if constexpr (sizeof(S) == 4) {
      uint32_t u; memcpy(&u, &x, 4);
      u = __byte_perm(u, 0u, swap ? 0x0123u : 0x3210u);
      memcpy(&x, &u, 4); return x;
   } else {
      uint64_t u; memcpy(&u, &x, 8);
      const uint32_t lo = (uint32_t)u, hi = (uint32_t)(u >> 32), sel = swap ? 0x0123u : 0x3210u;
      u = (uint64_t)__byte_perm(swap ? hi : lo, 0u, sel) | ((uint64_t)__byte_perm(swap ? lo : hi, 0u, sel) << 32);
      memcpy(&x, &u, 8); return x;
   }
}
// N aligned elements of storage type S (the real part where the operand is complex) as compute type C: native-width
// loads, all issued before the first conversion.
template <class C, class S, int N> SD_D void load_typed_n(const char *q, int64_t step, bool swap, C (&out)[N])
{
   S x[N];
#pragma unroll
   for (int j = 0; j < N; j++, q += step) x[j] = ld_one<S>(q);
   // (a branch on the uniform flag instead of the selects of the 8-byte case was measured: 59.7 against 54.3 us)
#pragma unroll
   for (int j = 0; j < N; j++) out[j] = convert<C>(maybe_bswap(x[j], swap));
}
template <class C, int N> SD_D void load_as_n(const char *q, int64_t step, int dtype, bool swap, C (&out)[N])
{
   switch (dtype) {
      case 0:  load_typed_n<C, Bool, N>(q, step, swap, out); break;
      case 1:  load_typed_n<C, uint8_t, N>(q, step, swap, out); break;
      case 2:  load_typed_n<C, uint16_t, N>(q, step, swap, out); break;
      case 3:  load_typed_n<C, uint32_t, N>(q, step, swap, out); break;
      case 4:  load_typed_n<C, uint64_t, N>(q, step, swap, out); break;
      case 5:  load_typed_n<C, int8_t, N>(q, step, swap, out); break;
      case 6:  load_typed_n<C, int16_t, N>(q, step, swap, out); break;
      case 7:  load_typed_n<C, int32_t, N>(q, step, swap, out); break;
      case 8:  load_typed_n<C, int64_t, N>(q, step, swap, out); break;
      case 9:  case 12: load_typed_n<C, Half, N>(q, step, swap, out); break;
      case 10: case 13: load_typed_n<C, float, N>(q, step, swap, out); break;
      default: load_typed_n<C, double, N>(q, step, swap, out); break;
   }
}
template <class C, class D, int N> SD_D void store_typed_n(char *q, int64_t step, bool swap, const C (&v)[N])
{
#pragma unroll
   for (int j = 0; j < N; j++, q += step) {
      D y = convert<D>(v[j]);
      if constexpr (is_cplx<D>) { y.re = maybe_bswap(y.re, swap); y.im = maybe_bswap(y.im, swap); }
      else y = maybe_bswap(y, swap);
      st_one<D>(q, y);
   }
}
template <class C, int N> SD_D void store_aligned_n(char *q, int64_t step, int dtype, bool swap, const C (&v)[N])
{
   switch (dtype) {
      case 0:  store_typed_n<C, Bool, N>(q, step, swap, v); break;
      case 1:  store_typed_n<C, uint8_t, N>(q, step, swap, v); break;
      case 2:  store_typed_n<C, uint16_t, N>(q, step, swap, v); break;
      case 3:  store_typed_n<C, uint32_t, N>(q, step, swap, v); break;
      case 4:  store_typed_n<C, uint64_t, N>(q, step, swap, v); break;
      case 5:  store_typed_n<C, int8_t, N>(q, step, swap, v); break;
      case 6:  store_typed_n<C, int16_t, N>(q, step, swap, v); break;
      case 7:  store_typed_n<C, int32_t, N>(q, step, swap, v); break;
      case 8:  store_typed_n<C, int64_t, N>(q, step, swap, v); break;
      case 9:  store_typed_n<C, Half, N>(q, step, swap, v); break;
      case 10: store_typed_n<C, float, N>(q, step, swap, v); break;
      case 11: store_typed_n<C, double, N>(q, step, swap, v); break;
      case 12: store_typed_n<C, CHalf, N>(q, step, swap, v); break;
      case 13: store_typed_n<C, CFloat, N>(q, step, swap, v); break;
      default: store_typed_n<C, CDouble, N>(q, step, swap, v); break;
   }
}

// Tiled variant for two or more dimensions: a tile of 32 (dimension 0) x 64 (dimension dt)
// elements, 256 threads, 8 elements per thread and operand.  Operands that are dense along dt
// (a transposed matrix) are first read with 64 lanes running along dt, converted and parked in
// shared memory; then 32 lanes run along dimension 0, the remaining operands are read
// directly (coalesced) and the result is stored.  STAGED (the set of operands that go through shared memory)
// is a template parameter, so each operand has the code of one path only.
//
// Interior tiles of aligned operands, i.e. nearly all the work, take mix_tile_fast: unrolled, one type switch per
// operand and thread around native-width loads.  Edge tiles and unaligned operands take mix_tile_slow, a rolled
// loop over the thread's elements that is small rather than fast.  (ncu on the earlier single body, which carried
// raw 64-bit words, bounds predicates and alignment tests through the unrolled loops: 636 instructions per thread
// for 8 elements, issue slots 60 % busy, DRAM 43 %.)
template <class C, int STAGED>
SD_D void mix_tile_fast(const MixParams &p, C (*tile)[M0][M1 + 1], const int64_t (&off)[4], int64_t i0, int64_t it)
{
   if constexpr (STAGED != 0) {                            // phase 1: 64 lanes along dt, 4 rows of dimension 0 per pass
      const int tx = threadIdx.x & (M1 - 1), ty = threadIdx.x / M1;
      int slot = 0;
#pragma unroll
      for (int k = 0; k < 3; k++) {
         if (!(STAGED & (1 << k))) continue;
         C v[MR];
         load_as_n<C, MR>(p.ptr[k] + off[k] + (it + tx) * p.stride[k][p.dt] + (i0 + ty) * p.stride[k][0],
                          MP1 * p.stride[k][0], p.dtype[k], p.swap[k] != 0, v);
#pragma unroll
         for (int j = 0; j < MR; j++) tile[slot][ty + MP1 * j][tx] = v[j];
         slot++;
      }
      __syncthreads();
   }
   // phase 2: 32 lanes along dimension 0, 8 columns of dt per pass
   const int tx = threadIdx.x & (M0 - 1), ty = threadIdx.x / M0;
   C acc[MR];
   int slot = 0;
#pragma unroll
   for (int k = 0; k < 3; k++) {                           // unrolled: k selects the arithmetic at compile time
      C v[MR];
      if (STAGED & (1 << k)) {
#pragma unroll
         for (int j = 0; j < MR; j++) v[j] = tile[slot][tx][ty + MP2 * j];
         slot++;
      } else {
         load_as_n<C, MR>(p.ptr[k] + off[k] + (i0 + tx) * p.stride[k][0] + (it + ty) * p.stride[k][p.dt],
                          MP2 * p.stride[k][p.dt], p.dtype[k], p.swap[k] != 0, v);
      }
#pragma unroll
      for (int j = 0; j < MR; j++) acc[j] = (k == 0) ? v[j] : (k == 1 ? acc[j] * v[j] : acc[j] + v[j]);   // rounded product, rounded sum
   }
   store_aligned_n<C, MR>(p.ptr[3] + off[3] + (i0 + tx) * p.stride[3][0] + (it + ty) * p.stride[3][p.dt],
                          MP2 * p.stride[3][p.dt], p.dtype[3], p.swap[3] != 0, acc);
}

template <class C, int STAGED>
SD_D void mix_tile_slow(const MixParams &p, C (*tile)[M0][M1 + 1], const int64_t (&off)[4],
                        int64_t i0, int64_t it, int64_t n0, int64_t nt)
{
   if constexpr (STAGED != 0) {
      const int tx = threadIdx.x & (M1 - 1), ty = threadIdx.x / M1;
      int slot = 0;
#pragma unroll
      for (int k = 0; k < 3; k++) {
         if (!(STAGED & (1 << k))) continue;
         const char *q = p.ptr[k] + off[k] + (it + tx) * p.stride[k][p.dt] + (i0 + ty) * p.stride[k][0];
#pragma unroll 1
         for (int j = 0; j < MR; j++, q += MP1 * p.stride[k][0]) {
            const bool ok = (i0 + ty + MP1 * j < n0) && (it + tx < nt);
            tile[slot][ty + MP1 * j][tx] = ok ? bits_as<C>(load_bits(q, p.comp[k], p.unal[k] != 0), p.dtype[k], p.swap[k] != 0) : C(0);
         }
         slot++;
      }
      __syncthreads();
   }
   const int tx = threadIdx.x & (M0 - 1), ty = threadIdx.x / M0;
   if (i0 + tx >= n0) return;
#pragma unroll 1
   for (int j = 0; j < MR; j++) {
      const int64_t t = it + ty + MP2 * j;
      if (t >= nt) break;
      C acc = C(0);
      int slot = 0;
#pragma unroll
      for (int k = 0; k < 3; k++) {
         C v;
         if (STAGED & (1 << k)) { v = tile[slot][tx][ty + MP2 * j]; slot++; }
         else v = bits_as<C>(load_bits(p.ptr[k] + off[k] + (i0 + tx) * p.stride[k][0] + t * p.stride[k][p.dt], p.comp[k], p.unal[k] != 0),
                             p.dtype[k], p.swap[k] != 0);
         acc = (k == 0) ? v : (k == 1 ? acc * v : acc + v);
      }
      store_as<C>(p.ptr[3] + off[3] + (i0 + tx) * p.stride[3][0] + t * p.stride[3][p.dt], p.dtype[3], acc, p.swap[3] != 0, p.unal[3] != 0);
   }
}

template <class C, int STAGED>
__global__ void __launch_bounds__(MT, MIX_BLOCKS) mix_tiled(const MixParams p)
{
   extern __shared__ __align__(16) unsigned char mix_smem[];
   C (*tile)[M0][M1 + 1] = reinterpret_cast<C (*)[M0][M1 + 1]>(mix_smem);
   uint32_t bid = blockIdx.x;
   uint32_t bq = fastdiv(bid, p.div_tiles0);
   const uint32_t t0 = bid - bq * (uint32_t)p.tiles0; bid = bq;
   bq = fastdiv(bid, p.div_tilest);
   const uint32_t tt = bid - bq * (uint32_t)p.tilest; bid = bq;
   int64_t off[4] = {0, 0, 0, 0};
   for (int d = 1; d < p.ndims; d++) {
      if (d == p.dt) continue;
      uint32_t q = bid / (uint32_t)p.size[d]; uint32_t c = bid - q * (uint32_t)p.size[d]; bid = q;   // bid < size[d] * (the rest) < 2^31
#pragma unroll
      for (int k = 0; k < 4; k++) off[k] += (int64_t)c * p.stride[k][d];
   }
   const int64_t i0 = (int64_t)t0 * M0, it = (int64_t)tt * M1;
   const int64_t n0 = p.size[0], nt = p.size[p.dt];
   if (i0 + M0 <= n0 && it + M1 <= nt && !p.anyunal) mix_tile_fast<C, STAGED>(p, tile, off, i0, it);
   else                                              mix_tile_slow<C, STAGED>(p, tile, off, i0, it, n0, nt);
}

template <class C, int STAGED>
int mix_tiled_launch(const MixParams &p, uint64_t blocks, size_t smem, cudaStream_t stream)
{
   static bool attr_set = false;
   if (smem > 48 * 1024 && !attr_set) {
      SD_CUDA_CHECK(cudaFuncSetAttribute(mix_tiled<C, STAGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * M0 * (M1 + 1) * (int)sizeof(C)));
      attr_set = true;
   }
   mix_tiled<C, STAGED><<<(unsigned)blocks, MT, smem, stream>>>(p);
   return 0;
}

template <class C>
int mixed_multiply_add(int ndims, const size_t *size, const solid_gpu_operand *const ops[4], cudaStream_t stream)
{
   const ptrdiff_t *st[4]; void *pt[4];
   for (int k = 0; k < 4; k++) {
      if (ops[k] == nullptr || ops[k]->ptr == nullptr) SD_ERROR("mixed_multiply_add: operand %d is missing", k);
      if (ops[k]->dtype < 0 || ops[k]->dtype >= SOLID_NUM_TYPES) SD_ERROR("Invalid type index %d", ops[k]->dtype);
      st[k] = ops[k]->strides; pt[k] = ops[k]->ptr;
   }
   Layout<4> L;
   if (make_layout<4>(L, ndims, size, st, pt, 3) != 0) return -1;
   if (L.nelem == 0) return 0;
   DeviceInfo dev;
   if (current_device_info(&dev) != 0) return -1;
   MixParams p; memset(&p, 0, sizeof(p));
   p.ndims = L.ndims; p.nelem = (uint64_t)L.nelem;
   for (int d = 0; d < L.ndims; d++) p.size[d] = L.size[d];
   for (int k = 0; k < 4; k++) {
      p.ptr[k] = L.ptr[k]; p.dtype[k] = ops[k]->dtype; p.swap[k] = ops[k]->byteswapped ? 1 : 0;
      int es = solid_gpu_type_size[p.dtype[k]];
      int comp = p.dtype[k] >= SD_CHALF ? es / 2 : es;            // accesses are per real component
      bool bad = !aligned_to(p.ptr[k], (size_t)comp);
      for (int d = 0; d < L.ndims; d++) { p.stride[k][d] = L.stride[k][d]; if (L.stride[k][d] % comp) bad = true; }
      p.unal[k] = bad ? 1 : 0;
      p.comp[k] = comp;
   }
   // operands that step by more than a few elements along dimension 0 but are dense
   // along some other dimension are staged through shared memory
   int dt = -1; uint32_t staged = 0;
   for (int k = 0; k < 3 && L.ndims >= 2; k++) {
      int es = solid_gpu_type_size[p.dtype[k]];
      int64_t s0 = L.stride[k][0] < 0 ? -L.stride[k][0] : L.stride[k][0];
      if (s0 == 0 || s0 <= 2 * es) continue;                       // dense enough or broadcast along dim 0
      for (int d = 1; d < L.ndims; d++) {
         int64_t sd_ = L.stride[k][d] < 0 ? -L.stride[k][d] : L.stride[k][d];
         if (sd_ == es && L.size[d] >= 16 && (dt < 0 || dt == d)) { dt = d; staged |= (1u << k); break; }
      }
   }
   if (L.ndims >= 2) {
      if (!staged) dt = 1;                                           // plain 2-D tiling, nothing staged
      p.dt = dt; p.staged = staged;
      p.tiles0 = ((uint64_t)L.size[0] + M0 - 1) / M0; p.tilest = ((uint64_t)L.size[dt] + M1 - 1) / M1;
      uint64_t blocks = p.tiles0 * p.tilest;
      for (int d = 1; d < L.ndims; d++) if (d != dt) blocks *= (uint64_t)L.size[d];
      if (blocks > 0x7FFFFFFFull) SD_ERROR("mixed_multiply_add: grid too large");
      int nstaged = 0;
      for (int k = 0; k < 3; k++) if (staged & (1u << k)) nstaged++;
      size_t smem = (size_t)nstaged * M0 * (M1 + 1) * sizeof(C);            // up to 3 x 16.3 KB
      p.div_tiles0 = make_fastdiv((uint32_t)p.tiles0); p.div_tilest = make_fastdiv((uint32_t)p.tilest);
      p.anyunal = (p.unal[0] | p.unal[1] | p.unal[2] | p.unal[3]) ? 1 : 0;
      int rc = 0;
      switch (staged) {                                              // one kernel per set of staged operands
         case 0: rc = mix_tiled_launch<C, 0>(p, blocks, smem, stream); break;
         case 1: rc = mix_tiled_launch<C, 1>(p, blocks, smem, stream); break;
         case 2: rc = mix_tiled_launch<C, 2>(p, blocks, smem, stream); break;
         case 3: rc = mix_tiled_launch<C, 3>(p, blocks, smem, stream); break;
         case 4: rc = mix_tiled_launch<C, 4>(p, blocks, smem, stream); break;
         case 5: rc = mix_tiled_launch<C, 5>(p, blocks, smem, stream); break;
         case 6: rc = mix_tiled_launch<C, 6>(p, blocks, smem, stream); break;
         default: rc = mix_tiled_launch<C, 7>(p, blocks, smem, stream); break;
      }
      if (rc != 0) return rc;
   } else {
      uint64_t blocks = (p.nelem + 256ull * MR - 1) / (256ull * MR);
      if (blocks > 0x7FFFFFFFull) blocks = 0x7FFFFFFFull;            // one chunk per block
      mix_linear<C><<<(unsigned)blocks, 256, 0, stream>>>(p);
   }
   SD_LAUNCH_CHECK();
   return 0;
}

} // namespace sd

extern "C" int solid_gpu_axpy_sums_buffer_size(int device, size_t n, size_t *size)
{
   (void)device;                                  // the partial count depends on the length only
   if (size == nullptr) { SD_ERROR("axpy_sums_buffer_size needs a result pointer"); }
   const uint64_t blocks = sd::axpy_sums_blocks((uint64_t)n, sizeof(double));   // double has the most blocks
   *size = (size_t)(blocks + sd::axpy_sums_level2(blocks)) * sizeof(sd::Sums<double>);
   return 0;
}
extern "C" int solid_gpu_axpy_sums_float(SOLID_GPU_ARGS_AXPY_SUMS)
{  return sd::axpy_sums<float>(n, a._float, x, y, z, sums, partials, stream); }
extern "C" int solid_gpu_axpy_sums_double(SOLID_GPU_ARGS_AXPY_SUMS)
{  return sd::axpy_sums<double>(n, a._double, x, y, z, sums, partials, stream); }

extern "C" int solid_gpu_mixed_multiply_add(int ndims, const size_t *size,
                                            const solid_gpu_operand *a, const solid_gpu_operand *b,
                                            const solid_gpu_operand *c, const solid_gpu_operand *dst,
                                            int ctype, cudaStream_t stream)
{
   const solid_gpu_operand *ops[4] = { a, b, c, dst };
   if (ctype == SD_FLOAT)  return sd::mixed_multiply_add<float>(ndims, size, ops, stream);
   if (ctype == SD_DOUBLE) return sd::mixed_multiply_add<double>(ndims, size, ops, stream);
   SD_ERROR("mixed_multiply_add: compute type must be float or double (got index %d)", ctype);
}
