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
constexpr int AX_THREADS = 256;

template <class T> struct Sums { T s, s2; };

template <class T>
__global__ void __launch_bounds__(AX_THREADS) axpy_sums_kernel(uint64_t n, T a, const T *__restrict__ x,
                                                               const T *__restrict__ y, T *__restrict__ z,
                                                               Sums<T> *__restrict__ partials)
{
   constexpr int VEC = 16 / sizeof(T), U = 4;
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

// Single block: thread t folds partials t, t+256, ... in order, then the block tree.
template <class T>
__global__ void __launch_bounds__(AX_THREADS) axpy_sums_finish(int nparts, const Sums<T> *__restrict__ partials,
                                                               T *__restrict__ sums)
{
   __shared__ Sums<T> smem[AX_THREADS / 32];
   T s = 0, s2 = 0;
   for (int i = threadIdx.x; i < nparts; i += AX_THREADS) { s += partials[i].s; s2 += partials[i].s2; }
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
      sums[0] = s; sums[1] = s2;
   }
}

static int axpy_sums_blocks(const DeviceInfo &dev) { return dev.sms * (dev.max_threads_per_sm / AX_THREADS); }

template <class T>
int axpy_sums(size_t n, T a, const void *x, const void *y, void *z, void *sums, void *partials, cudaStream_t stream)
{
   if (!aligned_to(x, 16) || !aligned_to(y, 16) || !aligned_to(z, 16))
      SD_ERROR("axpy_sums needs 16-byte aligned tensors");
   if (sums == nullptr || partials == nullptr) SD_ERROR("axpy_sums needs the sums and partials buffers");
   DeviceInfo dev;
   if (current_device_info(&dev) != 0) return -1;
   const int blocks = axpy_sums_blocks(dev);
   axpy_sums_kernel<T><<<blocks, AX_THREADS, 0, stream>>>((uint64_t)n, a, (const T *)x, (const T *)y, (T *)z,
                                                        (Sums<T> *)partials);
   SD_LAUNCH_CHECK();
   axpy_sums_finish<T><<<1, AX_THREADS, 0, stream>>>(blocks, (const Sums<T> *)partials, (T *)sums);
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
template <class C> SD_D C load_as(const char *p, int dtype, int comp_size, bool swap, bool unal)
{  return bits_as<C>(load_bits(p, comp_size, unal), dtype, swap); }
template <class D, class C> SD_D void store_typed(char *p, C v, bool swap, bool unal)
{
   D y = convert<D>(v);
   if (swap) y = bswap<D>(y);
   if (!unal) st_one<D>(p, y);
   else { uint8_t b[sizeof(D)]; memcpy(b, &y, sizeof(D));
#pragma unroll
      for (int i = 0; i < (int)sizeof(D); i++) reinterpret_cast<uint8_t *>(p)[i] = b[i]; }
}
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

// Linear variant: no operand needs staging.  One element per thread-iteration,
// adjacent threads adjacent along dimension 0.
template <class C>
__global__ void __launch_bounds__(256) mix_linear(const MixParams p)
{
   for (uint64_t idx = (uint64_t)blockIdx.x * 256 + threadIdx.x; idx < p.nelem; idx += (uint64_t)gridDim.x * 256) {
      int64_t off[4] = {0, 0, 0, 0};
      uint64_t r = idx;
      for (int d = 0; d < p.ndims - 1; d++) {
         uint64_t q = r / (uint64_t)p.size[d]; uint64_t c = r - q * (uint64_t)p.size[d]; r = q;
#pragma unroll
         for (int k = 0; k < 4; k++) off[k] += (int64_t)c * p.stride[k][d];
      }
#pragma unroll
      for (int k = 0; k < 4; k++) off[k] += (int64_t)r * p.stride[k][p.ndims - 1];
      uint64_t ra = load_bits(p.ptr[0] + off[0], p.comp[0], p.unal[0]);
      uint64_t rb = load_bits(p.ptr[1] + off[1], p.comp[1], p.unal[1]);
      uint64_t rc = load_bits(p.ptr[2] + off[2], p.comp[2], p.unal[2]);
      C a = bits_as<C>(ra, p.dtype[0], p.swap[0]);
      C b = bits_as<C>(rb, p.dtype[1], p.swap[1]);
      C c = bits_as<C>(rc, p.dtype[2], p.swap[2]);
      C prod = a * b;
      C sum = prod + c;
      store_as<C>(p.ptr[3] + off[3], p.dtype[3], sum, p.swap[3], p.unal[3]);
   }
}

// Tiled variant: a 64 x 64 tile over (dimension 0, dimension dt), 256 threads, 16 elements
// per thread and operand.  Operands that are dense along dt are first read with lanes
// running along dt (coalesced), converted and parked in shared memory; then lanes run
// along dimension 0, the remaining operands are read directly (coalesced) and the result
// is stored.  In both phases a thread issues all of its loads before it consumes any of
// them, so sixteen independent requests per operand are in flight per thread.
constexpr int MT = 64;                      // tile edge
constexpr int MR = 16;                      // elements per thread (MT * MT / 256)

template <class C>
__global__ void __launch_bounds__(256) mix_tiled(const MixParams p)
{
   extern __shared__ __align__(16) unsigned char mix_smem[];
   C (*tile)[MT][MT + 1] = reinterpret_cast<C (*)[MT][MT + 1]>(mix_smem);
   const int tx = threadIdx.x & (MT - 1), ty = threadIdx.x / MT;      // 64 x 4
   uint64_t bid = blockIdx.x;
   const uint64_t t0 = bid % p.tiles0; bid /= p.tiles0;
   const uint64_t tt = bid % p.tilest; bid /= p.tilest;
   int64_t off[4] = {0, 0, 0, 0};
   for (int d = 1; d < p.ndims; d++) {
      if (d == p.dt) continue;
      uint64_t q = bid / (uint64_t)p.size[d]; uint64_t c = bid - q * (uint64_t)p.size[d]; bid = q;
#pragma unroll
      for (int k = 0; k < 4; k++) off[k] += (int64_t)c * p.stride[k][d];
   }
   const int64_t i0 = (int64_t)t0 * MT, it = (int64_t)tt * MT;
   const int64_t n0 = p.size[0], nt = p.size[p.dt];

   // phase 1: lanes along dt; tile slot of operand k is the number of staged operands below k
   int slot = 0;
#pragma unroll
   for (int k = 0; k < 3; k++) {
      if (!(p.staged & (1u << k))) continue;
      uint64_t raw[MR];
      const char *base = p.ptr[k] + off[k] + (it + tx) * p.stride[k][p.dt];
#pragma unroll
      for (int j = 0; j < MR; j++) {
         int64_t a0 = i0 + ty + 4 * j;
         raw[j] = (a0 < n0 && it + tx < nt) ? load_bits(base + a0 * p.stride[k][0], p.comp[k], p.unal[k]) : 0;
      }
#pragma unroll
      for (int j = 0; j < MR; j++) tile[slot][ty + 4 * j][tx] = bits_as<C>(raw[j], p.dtype[k], p.swap[k]);
      slot++;
   }
   __syncthreads();
   // phase 2: lanes along dimension 0
   uint64_t raw[3][MR];
#pragma unroll
   for (int k = 0; k < 3; k++) {
      if (p.staged & (1u << k)) continue;
      const char *base = p.ptr[k] + off[k] + (i0 + tx) * p.stride[k][0];
#pragma unroll
      for (int j = 0; j < MR; j++) {
         int64_t at = it + ty + 4 * j;
         raw[k][j] = (i0 + tx < n0 && at < nt) ? load_bits(base + at * p.stride[k][p.dt], p.comp[k], p.unal[k]) : 0;
      }
   }
   C v[3][MR];
   slot = 0;
#pragma unroll
   for (int k = 0; k < 3; k++) {
      if (p.staged & (1u << k)) {
#pragma unroll
         for (int j = 0; j < MR; j++) v[k][j] = tile[slot][tx][ty + 4 * j];
         slot++;
      } else {
#pragma unroll
         for (int j = 0; j < MR; j++) v[k][j] = bits_as<C>(raw[k][j], p.dtype[k], p.swap[k]);
      }
   }
   char *obase = p.ptr[3] + off[3] + (i0 + tx) * p.stride[3][0];
#pragma unroll
   for (int j = 0; j < MR; j++) {
      int64_t at = it + ty + 4 * j;
      if (i0 + tx < n0 && at < nt) {
         C prod = v[0][j] * v[1][j];
         C sum = prod + v[2][j];
         store_as<C>(obase + at * p.stride[3][p.dt], p.dtype[3], sum, p.swap[3], p.unal[3]);
      }
   }
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
   if (staged) {
      p.dt = dt; p.staged = staged;
      p.tiles0 = ((uint64_t)L.size[0] + MT - 1) / MT; p.tilest = ((uint64_t)L.size[dt] + MT - 1) / MT;
      uint64_t blocks = p.tiles0 * p.tilest;
      for (int d = 1; d < L.ndims; d++) if (d != dt) blocks *= (uint64_t)L.size[d];
      if (blocks > 0x7FFFFFFFull) SD_ERROR("mixed_multiply_add: grid too large");
      int nstaged = 0;
      for (int k = 0; k < 3; k++) if (staged & (1u << k)) nstaged++;
      size_t smem = (size_t)nstaged * MT * (MT + 1) * sizeof(C);            // up to 3 x 33 KB
      static bool attr_set[2] = { false, false };
      if (smem > 48 * 1024 && !attr_set[sizeof(C) == 8]) {
         SD_CUDA_CHECK(cudaFuncSetAttribute(mix_tiled<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * MT * (MT + 1) * (int)sizeof(C)));
         attr_set[sizeof(C) == 8] = true;
      }
      mix_tiled<C><<<(unsigned)blocks, 256, smem, stream>>>(p);
   } else {
      uint64_t blocks = (p.nelem + 255) / 256;
      uint64_t cap = (uint64_t)dev.sms * (dev.max_threads_per_sm / 256) * 4;
      if (blocks > cap) blocks = cap;
      mix_linear<C><<<(unsigned)blocks, 256, 0, stream>>>(p);
   }
   SD_LAUNCH_CHECK();
   return 0;
}

} // namespace sd

extern "C" int solid_gpu_axpy_sums_buffer_size(int device, size_t *size)
{
   solid_gpu_properties *prop = solid_gpu_get_device_properties(device);
   if (prop == nullptr) return -1;
   *size = (size_t)prop->multiprocessor_count * (prop->max_threads_per_multiprocessor / sd::AX_THREADS) * 16;
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
