// solid_gpu_axis_sum_float_noalloc: the float axis sum for callers that must not allocate.
//
// Who needs it: code that runs where device memory cannot be requested -- a callback or a
// destructor that may run while the allocator is locked, a latency-critical loop that cannot
// afford the device-wide synchronisation that cudaMalloc and cudaFree imply, or an embedding
// whose memory budget was handed out completely at start-up.  The regular entry
// point (solid_gpu_axis_sum_float) is given its scratch by the caller, who normally obtains it
// from cudaMalloc or a caching allocator.  This variant brings its own: a fixed array that is
// part of the library image, so the call itself requests no memory from anyone.
//
// The price: the array is SOLID_GPU_NOALLOC_SCRATCH_BYTES large on every device that loads the
// library, for as long as the process lives; a reduction whose plan needs more scratch than that
// is refused with an error (use the regular entry point then); and because every call uses the
// same array, two calls that overlap in time on one device -- on different streams, or from
// different threads -- would overwrite each other's partial results.  Issue them on one stream.
// The array keeps whatever the previous call left in it; that is harmless here because every
// partial result slot that the second pass reads is written by the first pass of the same call,
// so nothing has to be cleared.
//
// The first call on a device looks up the device address of the array (the array's name is a
// host-side handle in host code, not an address a kernel could use).  Make that first call
// before any stream capture begins.  First calls do two more one-time things that a restricted
// context may not tolerate, so make them outside it as well: the CUDA runtime loads each kernel
// the first time it is launched, and a reduction to a SINGLE output registers the stream it runs
// on in a fixed table of the library (a lock and one table entry, no allocation) the first time
// it sees that stream.  The table of resolved addresses is written without a lock: every thread
// would store the same value.
#include "solid_core_gpu.h"
#include "reduce.cuh"
#include "ops_reduce.cuh"

#ifndef SOLID_GPU_NOALLOC_SCRATCH_BYTES
#define SOLID_GPU_NOALLOC_SCRATCH_BYTES (1u << 20)
#endif

static __device__ __align__(256) unsigned char solid_gpu_noalloc_scratch[SOLID_GPU_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
void *scratch_address[MAX_DEVICES] = { nullptr };

// Device address of the array on the CURRENT device, resolved once per device.
int scratch_for_current_device(void **out)
{
   int device = -1;
   SD_CUDA_CHECK(cudaGetDevice(&device));
   if (device < 0 || device >= MAX_DEVICES) SD_ERROR("Device index %d is out of range", device);
   if (scratch_address[device] == nullptr) {
      void *ptr = nullptr;
      cudaError_t st = cudaGetSymbolAddress(&ptr, solid_gpu_noalloc_scratch);
      if (st != cudaSuccess || ptr == nullptr)
         SD_ERROR("Cannot resolve the built-in scratch array on device %d (%s)", device, cudaGetErrorString(st));
      scratch_address[device] = ptr;
   }
   *out = scratch_address[device];
   return 0;
}
} // namespace

extern "C" int solid_gpu_noalloc_scratch_size(void) { return (int)SOLID_GPU_NOALLOC_SCRATCH_BYTES; }

extern "C" int solid_gpu_axis_sum_float_noalloc(solid_gpu_reduce_axis_config *config)
{
   if (config == nullptr) SD_ERROR("The reduction configuration is missing");
   if (config->bufferSize > (size_t)SOLID_GPU_NOALLOC_SCRATCH_BYTES)
      SD_ERROR("This axis sum needs %zu bytes of scratch but the built-in array holds %u; "
               "use solid_gpu_axis_sum_float with a caller-provided buffer",
               config->bufferSize, (unsigned)SOLID_GPU_NOALLOC_SCRATCH_BYTES);
   void *scratch = nullptr;
   if (scratch_for_current_device(&scratch) != 0) return -1;
   solid_gpu_reduce_axis_config local = *config;              // the caller's structure is left untouched
   local.data.ptrBuffer = config->bufferSize ? (char *)scratch : nullptr;
   return sd::reduce_axis<sd::r_sum<float>, float>(sd::r_sum<float>(), &local);
}
