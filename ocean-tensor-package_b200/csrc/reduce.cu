// Global reductions solid_gpu_<op>_<SDX> and axis reductions solid_gpu_axis_<op>_<SDX>
// for one element type (both in one unit so that each kernel is built once).
// Replaces solid/src/core/gpu/template_reduce_all.cu:54-437 with the launcher of
// solid/include/solid/core/gpu/reduce_all.h:365-414, and
// solid/src/core/gpu/template_reduce_axis.cu:54-350.
//
// Contract kept from the reference: `result` is a HOST pointer that holds the
// value when the call returns (the kernel writes it into a pinned, device-mapped
// slot which the host polls briefly before it falls back to a stream
// synchronisation), `buffer` is device
// scratch of solid_gpu_reduce_all_buffer_size() bytes, empty tensors yield the
// identity (sum 0, prod 1, any 0, all 1) and are an error for minimum/maximum.
// Not kept: the range tests read BOTH bounds (the reference's GPU wrapper copies
// `lower` into `upper`, template_reduce_all.cu:208-209).
#include <atomic>
#include "reduce_unit.cuh"

namespace sd {
// When set (by solid_gpu_reduce_all_device on this thread) the value is left in
// device memory at this address and nothing synchronises.
extern thread_local void *reduce_all_device_result;
// 64 pinned, device-mapped host bytes per device, created on first use (reduce_plan.cu).
char *reduce_all_host_slot();

template <class R> __global__ void red_identity(const R r, typename R::out_t *dst, const RedParams p)
{
   if constexpr (!R::seeded) *dst = r.finalize(r.init());
   red_signal(p);
}

// Wait until the finishing thread of the launch has set the slot's sequence word.  The value and the word
// are written straight into mapped host memory, so a short poll sees them a few microseconds before a stream
// synchronisation would return; after about a millisecond (long reductions, or a launch that failed and will
// never write) the stream is synchronised instead, which also delivers the error.
inline int reduce_all_wait(const char *host_slot, uint32_t seq, cudaStream_t stream)
{
   const volatile uint32_t *flag = reinterpret_cast<const volatile uint32_t *>(host_slot + 32);
   for (int spin = 0; spin < 50000; spin++) {
      if (*flag == seq) { std::atomic_thread_fence(std::memory_order_acquire); return 0; }
#if defined(__x86_64__)
      __builtin_ia32_pause();
#endif
   }
   SD_CUDA_CHECK(cudaStreamSynchronize(stream));
   if (*flag != seq) SD_ERROR("Global reduction finished without delivering its result");
   return 0;
}

template <class R, class T>
int reduce_all(const R &r, const char *name, int ndims, const size_t *size, const ptrdiff_t *strides, void *ptr,
               void *result, void *buffer, cudaStream_t stream)
{
   using O = typename R::out_t;
   if (buffer == nullptr) SD_ERROR("Global reduction '%s' needs a device scratch buffer", name);
   RedParams p;
   if (red_make_params(p, 0, nullptr, nullptr, ptr, nullptr, buffer, ndims, size, strides) != 0) return -1;
   // Where the value goes: the caller's device address (device-resident form), or this device's
   // pinned, device-mapped host slot, which the last kernel writes directly so that no separate
   // device-to-host copy has to be queued before the synchronisation.
   char *host_slot = nullptr;
   char *slot = (char *)reduce_all_device_result;
   if (slot == nullptr) {
      host_slot = reduce_all_host_slot();
      if (host_slot == nullptr) return -1;
      slot = host_slot;
   }
   p.dst = slot;
   p.buf = (char *)buffer + 16;
   uint32_t sequence = 0;
   if (host_slot != nullptr) {
      uint32_t *counter = reinterpret_cast<uint32_t *>(host_slot + 48);   // host-only word: calls made through this slot
      if (++*counter == 0) *counter = 1;                   // the slot starts out with 0 in its sequence word
      sequence = *counter;
      p.flag = reinterpret_cast<uint32_t *>(host_slot + 32);
      p.flag_value = sequence;
   }
   if (p.relem == 0) {
      if (R::seeded) SD_ERROR("The tensor %s function is undefined on empty tensors", name);
      red_identity<R><<<1, 1, 0, stream>>>(r, reinterpret_cast<O *>(slot), p);
      SD_LAUNCH_CHECK();
   } else {
      DeviceInfo dev;
      if (current_device_info(&dev) != 0) return -1;
      if (red_launch<R, T>(r, p, red_split_cap(1, p.relem, dev.sms), stream) != 0) return -1;
   }
   if (host_slot == nullptr) return 0;
   if (reduce_all_wait(host_slot, sequence, stream) != 0) return -1;
   memcpy(result, host_slot, sizeof(O));
   return 0;
}
} // namespace sd

#define SD_RED_CALL(R_OBJ, RTYPE, NAME) \
   sd::reduce_all<RTYPE, T>(R_OBJ, #NAME, ndims, size, strides, ptr, (void *)result, buffer, stream)

#define SD_DEFINE_PLAIN(ARGS, NAME, GROUP) SD_WHEN(GROUP)(                                        \
   extern "C" int SD_PASTE(solid_gpu_##NAME##_, SDX)(ARGS)                                         \
   {  return SD_RED_CALL(sdu::R_##NAME(), sdu::R_##NAME, NAME); })
#define SD_DEFINE_BOOL(NAME, GROUP) SD_DEFINE_PLAIN(SOLID_GPU_ARGS_REDUCE_BOOL, NAME, GROUP)
#define SD_DEFINE_U64(NAME, GROUP)  SD_DEFINE_PLAIN(SOLID_GPU_ARGS_REDUCE_U64, NAME, GROUP)
#define SD_DEFINE_VOID(NAME, GROUP) SD_DEFINE_PLAIN(SOLID_GPU_ARGS_REDUCE_VOID, NAME, GROUP)
SOLID_GPU_REDUCE_BOOL_OPS(SD_DEFINE_BOOL)
SOLID_GPU_REDUCE_U64_OPS(SD_DEFINE_U64)
SOLID_GPU_REDUCE_VOID_OPS(SD_DEFINE_VOID)

#define SD_DEFINE_NORM(NAME, GROUP)                                                               \
   extern "C" int SD_PASTE(solid_gpu_##NAME##_, SDX)(SOLID_GPU_ARGS_REDUCE_NORM)                   \
   {  return SD_RED_CALL(sdu::make_norm<sdu::R_##NAME>(p), sdu::R_##NAME, NAME); }
SOLID_GPU_REDUCE_NORM_OPS(SD_DEFINE_NORM)

// one-sided range tests: lt/le bound from above, gt/ge from below
#define SD_DEFINE_BOUND1(NAME, LO, HI)                                                            \
   extern "C" int SD_PASTE(solid_gpu_##NAME##_, SDX)(SOLID_GPU_ARGS_REDUCE_BOUND1)                 \
   {  using R = sd::r_range<T, LO, HI>; R r;                                                       \
      r.pred.lower = sdu::bound_value(bound); r.pred.upper = r.pred.lower;                         \
      return SD_RED_CALL(r, R, NAME); }
SD_DEFINE_BOUND1(all_lt, 0, 1) SD_DEFINE_BOUND1(all_le, 0, 2)
SD_DEFINE_BOUND1(all_gt, 1, 0) SD_DEFINE_BOUND1(all_ge, 2, 0)

#define SD_DEFINE_BOUND2(NAME, LO, HI)                                                            \
   extern "C" int SD_PASTE(solid_gpu_##NAME##_, SDX)(SOLID_GPU_ARGS_REDUCE_BOUND2)                 \
   {  using R = sd::r_range<T, LO, HI>; R r;                                                       \
      r.pred.lower = sdu::bound_value(lower); r.pred.upper = sdu::bound_value(upper);              \
      return SD_RED_CALL(r, R, NAME); }
SD_DEFINE_BOUND2(all_gtlt, 1, 1) SD_DEFINE_BOUND2(all_gtle, 1, 2)
SD_DEFINE_BOUND2(all_gelt, 2, 1) SD_DEFINE_BOUND2(all_gele, 2, 2)

// ---------------------------------------------------------------------------
// Axis reductions.  The caller has run solid_gpu_reduce_axis_prepare(), which
// stored the tensor description in config->data and the scratch requirement in
// config->bufferSize, and has put the scratch pointer into config->data.ptrBuffer.
// Everything is asynchronous on config->stream.
// ---------------------------------------------------------------------------

#define SD_DEFINE_AXIS(NAME, GROUP) SD_WHEN(GROUP)(                                               \
   extern "C" int SD_PASTE(solid_gpu_axis_##NAME##_, SDX)(SOLID_GPU_ARGS_AXIS)                     \
   {  return sd::reduce_axis<sdu::R_##NAME, T>(sdu::R_##NAME(), config); })
SD_DEFINE_AXIS(any, all) SD_DEFINE_AXIS(all, all)
SD_DEFINE_AXIS(all_finite, float) SD_DEFINE_AXIS(any_inf, float) SD_DEFINE_AXIS(any_nan, float)
SD_DEFINE_AXIS(nnz, all) SD_DEFINE_AXIS(nnz_nan, all)
SD_DEFINE_AXIS(sum, all) SD_DEFINE_AXIS(sum_nan, all) SD_DEFINE_AXIS(prod, all) SD_DEFINE_AXIS(prod_nan, all)
SD_DEFINE_AXIS(sum_abs, all) SD_DEFINE_AXIS(sum_abs_nan, all)
SD_DEFINE_AXIS(maximum, all) SD_DEFINE_AXIS(minimum, all)
SD_DEFINE_AXIS(maximum_abs, all) SD_DEFINE_AXIS(minimum_abs, all)
SD_DEFINE_AXIS(norm2, all) SD_DEFINE_AXIS(norm2_nan, all)

#define SD_DEFINE_AXIS_NORM(NAME)                                                                 \
   extern "C" int SD_PASTE(solid_gpu_axis_##NAME##_, SDX)(SOLID_GPU_ARGS_AXIS_NORM)                \
   {  return sd::reduce_axis<sdu::R_##NAME, T>(sdu::make_norm<sdu::R_##NAME>(p), config); }
SD_DEFINE_AXIS_NORM(norm) SD_DEFINE_AXIS_NORM(norm_nan)
