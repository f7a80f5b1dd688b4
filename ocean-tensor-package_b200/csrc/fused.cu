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
   int64_t  stride[4][MAXD];
   int64_t  size[MAXD];
   int      ndims;
   int      dt;                 // dimension along which the staged operands are dense
   uint32_t staged;             // bit k: operand k goes through the shared-memory tile
   uint64_t nelem;
   uint64_t tiles0, tilest;
};

// Load `es` raw bytes (possibly unaligned) into the low bytes of a 16-byte buffer.
template <int ES> SD_D void load_raw(const char *p, bool unal, void *out)
{
   using raw = typename raw_of<ES>::type;
   raw r;
   if (!unal) r = ld_one<raw>(p);
   else { uint8_t b[ES];
#pragma unroll
      for (int i = 0; i < ES; i++) b[i] = __ldg(reinterpret_cast<const uint8_t *>(p) + i);
      memcpy(&r, b, ES); }
   memcpy(out, &r, ES);
}
template <class S> SD_D S load_typed(const char *p, bool swap, bool unal)
{
   S x;
   if constexpr (is_cplx<S>) {
      using E = elem_t<S>;
      load_raw<sizeof(E)>(p, unal, &x.re);                 // only the real part is needed
      if constexpr (is_half<E>) x.im.v = 0; else x.im = 0;
      if (swap) x.re = bswap_real(x.re);
   } else {
      load_raw<sizeof(S)>(p, unal, &x);
      if (swap) x = bswap<S>(x);
   }
   return x;
}
// Read one element of runtime type `dtype` as compute type C (real part of complex).
template <class C> SD_D C load_as(const char *p, int dtype, bool swap, bool unal)
{
   switch (dtype) {
      case 0:  return convert<C>(load_typed<Bool>(p, swap, unal));
      case 1:  return convert<C>(load_typed<uint8_t>(p, swap, unal));
      case 2:  return convert<C>(load_typed<uint16_t>(p, swap, unal));
      case 3:  return convert<C>(load_typed<uint32_t>(p, swap, unal));
      case 4:  return convert<C>(load_typed<uint64_t>(p, swap, unal));
      case 5:  return convert<C>(load_typed<int8_t>(p, swap, unal));
      case 6:  return convert<C>(load_typed<int16_t>(p, swap, unal));
      case 7:  return convert<C>(load_typed<int32_t>(p, swap, unal));
      case 8:  return convert<C>(load_typed<int64_t>(p, swap, unal));
      case 9:  return convert<C>(load_typed<Half>(p, swap, unal));
      case 10: return convert<C>(load_typed<float>(p, swap, unal));
      case 11: return convert<C>(load_typed<double>(p, swap, unal));
      case 12: return convert<C>(load_typed<CHalf>(p, swap, unal));
      case 13: return convert<C>(load_typed<CFloat>(p, swap, unal));
      default: return convert<C>(load_typed<CDouble>(p, swap, unal));
   }
}
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
      C a = load_as<C>(p.ptr[0] + off[0], p.dtype[0], p.swap[0], p.unal[0]);
      C b = load_as<C>(p.ptr[1] + off[1], p.dtype[1], p.swap[1], p.unal[1]);
      C c = load_as<C>(p.ptr[2] + off[2], p.dtype[2], p.swap[2], p.unal[2]);
      C prod = a * b;
      C sum = prod + c;
      store_as<C>(p.ptr[3] + off[3], p.dtype[3], sum, p.swap[3], p.unal[3]);
   }
}

// Tiled variant: a 32 x 32 tile over (dimension 0, dimension dt).  Operands that
// are dense along dt are first read with lanes running along dt (coalesced),
// converted and parked in shared memory; then lanes run along dimension 0, the
// remaining operands are read directly (coalesced) and the result is stored.
template <class C>
__global__ void __launch_bounds__(256) mix_tiled(const MixParams p)
{
   __shared__ C tile[3][32][33];
   const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;         // 32 x 8
   uint64_t bid = blockIdx.x;
   const uint64_t t0 = bid % p.tiles0; bid /= p.tiles0;
   const uint64_t tt = bid % p.tilest; bid /= p.tilest;
   // remaining dimensions
   int64_t off[4] = {0, 0, 0, 0};
   for (int d = 1; d < p.ndims; d++) {
      if (d == p.dt) continue;
      uint64_t q = bid / (uint64_t)p.size[d]; uint64_t c = bid - q * (uint64_t)p.size[d]; bid = q;
#pragma unroll
      for (int k = 0; k < 4; k++) off[k] += (int64_t)c * p.stride[k][d];
   }
   const int64_t i0 = (int64_t)t0 * 32, it = (int64_t)tt * 32;
   const int64_t n0 = p.size[0], nt = p.size[p.dt];

   // phase 1: lanes along dt
#pragma unroll
   for (int k = 0; k < 3; k++) {
      if (!(p.staged & (1u << k))) continue;
#pragma unroll
      for (int j = 0; j < 4; j++) {
         int64_t a0 = i0 + ty + 8 * j, at = it + tx;
         if (a0 < n0 && at < nt)
            tile[k][ty + 8 * j][tx] = load_as<C>(p.ptr[k] + off[k] + a0 * p.stride[k][0] + at * p.stride[k][p.dt],
                                                  p.dtype[k], p.swap[k], p.unal[k]);
      }
   }
   __syncthreads();
   // phase 2: lanes along dimension 0
#pragma unroll
   for (int j = 0; j < 4; j++) {
      int64_t a0 = i0 + tx, at = it + ty + 8 * j;
      if (a0 < n0 && at < nt) {
         C v[3];
#pragma unroll
         for (int k = 0; k < 3; k++) {
            if (p.staged & (1u << k)) v[k] = tile[k][tx][ty + 8 * j];
            else v[k] = load_as<C>(p.ptr[k] + off[k] + a0 * p.stride[k][0] + at * p.stride[k][p.dt],
                                   p.dtype[k], p.swap[k], p.unal[k]);
         }
         C prod = v[0] * v[1];
         C sum = prod + v[2];
         store_as<C>(p.ptr[3] + off[3] + a0 * p.stride[3][0] + at * p.stride[3][p.dt], p.dtype[3], sum,
                     p.swap[3], p.unal[3]);
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
      p.tiles0 = ((uint64_t)L.size[0] + 31) / 32; p.tilest = ((uint64_t)L.size[dt] + 31) / 32;
      uint64_t blocks = p.tiles0 * p.tilest;
      for (int d = 1; d < L.ndims; d++) if (d != dt) blocks *= (uint64_t)L.size[d];
      if (blocks > 0x7FFFFFFFull) SD_ERROR("mixed_multiply_add: grid too large");
      mix_tiled<C><<<(unsigned)blocks, 256, 0, stream>>>(p);
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
