// Type-independent parts of the reduction interface: scratch sizes, the axis
// reduction planner and the device-resident form of the global reductions.
// Counterparts: solid/src/core/gpu/op/reduce_all.c:77-123 (buffer size),
// solid/src/core/gpu/op/reduce_axis.c:22-315 (solid_gpu_reduce_axis_prepare).
#include <cstring>
#include <mutex>
#include "solid_core_gpu.h"
#include "reduce.cuh"

namespace sd {
thread_local void *reduce_all_device_result = nullptr;

// Result slot of the host-returning global reductions: 64 bytes of pinned host memory per
// (host thread, device), mapped into the device address space (unified addressing makes the
// host pointer valid in kernels).  Bytes 0-15 receive the value, the word at byte 32 the
// sequence number of the call once the value is in place; the word at byte 48 is the host's
// count of calls, from which the sequence numbers are taken.  Created the first time a thread
// runs such a reduction on a device and kept until exit.
char *reduce_all_host_slot()
{
   static thread_local char *slots[64] = {nullptr};
   int device;
   if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
      snprintf(solid_errmsg, SOLID_ERRMSG_SIZE, "Error getting the current device");
      return nullptr;
   }
   if (slots[device] == nullptr) {
      void *p = nullptr;
      cudaError_t st = cudaHostAlloc(&p, 64, cudaHostAllocMapped | cudaHostAllocPortable);
      if (st != cudaSuccess) {
         snprintf(solid_errmsg, SOLID_ERRMSG_SIZE, "Error allocating the pinned result slot (%s)", cudaGetErrorString(st));
         return nullptr;
      }
      memset(p, 0, 64);
      slots[device] = (char *)p;
   }
   return slots[device];
}

// Arrival counters of the single-pass folds: one word per stream of a device, in a device array
// that the module loader zeroes; the last block of every launch writes its word back to zero.
// Launches of one stream run one after another, so they can share a word; two streams never do.
constexpr int RED_TICKETS = 1024;
__device__ unsigned int red_ticket_pool[RED_TICKETS];

unsigned int *red_ticket_for_stream(cudaStream_t stream)
{
   // fixed tables, no container: a call from a context that must not allocate (the no-alloc entry point) takes the
   // lock and at most writes one table entry
   struct PerDevice { unsigned int *base; int used; cudaStream_t streams[RED_TICKETS]; };
   static PerDevice table[64];
   static std::mutex lock;
   if (stream == cudaStreamPerThread) return nullptr;       // one handle, a different stream in every host thread
   if (stream == cudaStreamLegacy) stream = nullptr;        // both name the legacy default stream
   int device;
   if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
   std::lock_guard<std::mutex> guard(lock);
   PerDevice &t = table[device];
   if (t.base == nullptr) {
      void *p = nullptr;
      if (cudaGetSymbolAddress(&p, red_ticket_pool) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
      t.base = (unsigned int *)p;
   }
   for (int i = 0; i < t.used; i++) if (t.streams[i] == stream) return t.base + i;
   if (t.used >= RED_TICKETS) return nullptr;               // table full: the caller falls back to the two-pass form
   t.streams[t.used] = stream;
   return t.base + t.used++;
}
} // namespace sd

// 16 bytes for the result slot, then one accumulator (at most 16 bytes) per block
// that can share the single output.
extern "C" int solid_gpu_reduce_all_buffer_size(size_t nelem, int device, size_t *size)
{
   solid_gpu_properties *prop = solid_gpu_get_device_properties(device);
   if (prop == nullptr) return -1;
   uint32_t cap = sd::red_split_cap(1, nelem, prop->multiprocessor_count);
   *size = 16 + (size_t)cap * 16;
   return 0;
}

// Record the tensors and decide how much scratch the launch may use.  The kernel
// family itself is chosen at launch time, when the element type is known; only
// the bound on blocks-per-output has to be fixed here because it sizes the
// buffer: bufferSize = outputs * split * elemsize, or 0 when every output is
// produced by a single block.
extern "C" int solid_gpu_reduce_axis_prepare(solid_gpu_reduce_axis_config *config, int elemsize,
                                             int ndims, const size_t *size, const ptrdiff_t *strides1,
                                             void *ptr1, const ptrdiff_t *strides2, void *ptr2,
                                             int rdims, const size_t *rsize, const ptrdiff_t *rstrides,
                                             cudaStream_t stream)
{
   if (ndims < 0 || ndims > SOLID_MAX_TENSOR_DIMS || rdims < 0 || rdims > SOLID_MAX_TENSOR_DIMS)
      SD_ERROR("Number of dimensions exceeds the maximum of %d", SOLID_MAX_TENSOR_DIMS);
   if (elemsize <= 0 || elemsize > 16) SD_ERROR("Invalid accumulator size %d", elemsize);
   sd::DeviceInfo dev;
   if (sd::current_device_info(&dev) != 0) return -1;
   memset(config, 0, sizeof(*config));
   solid_gpu_reduce_axis_data &d = config->data;
   size_t nelem = 1, relem = 1;
   for (int i = 0; i < ndims; i++) { d.size[i] = size[i]; d.strides1[i] = strides1[i]; d.strides2[i] = strides2[i]; nelem *= size[i]; }
   for (int i = 0; i < rdims; i++) { d.rsize[i] = rsize[i]; d.rstrides[i] = rstrides[i]; relem *= rsize[i]; }
   d.ptr1 = (char *)ptr1; d.ptr2 = (char *)ptr2; d.ptrBuffer = nullptr;
   d.nelem = nelem; d.relem = relem; d.ndims = ndims; d.rdims = rdims;
   uint32_t cap = (nelem && relem) ? sd::red_split_cap(nelem, relem, dev.sms) : 1;
   config->mode = cap > 1 ? 3 : 2;                 // 3: partials + finalize pass, 2: single pass
   config->sharedMem = cap;                        // read back by solid_gpu_axis_<op>_<type>
   config->sharedMemFinalize = (size_t)elemsize;
   config->bufferSize = cap > 1 ? (size_t)nelem * cap * (size_t)elemsize : 0;
   config->blockSize = dim3(sd::RED_THREADS, 1, 1);
   config->gridSize = dim3(1, 1, 1);
   config->blockSizeFinalize = dim3(sd::RED_THREADS, 1, 1);
   config->gridSizeFinalize = dim3(1, 1, 1);
   config->stream = stream;
   return 0;
}

// Device-resident global reduction: look the operation up by name and run it
// with the result slot redirected to `result` (device memory).
namespace {
struct NamedTable { const char *name; void *const *table; int kind; };   // kind 0: bool, 1: uint64, 2: void result
#define SD_NAMED(KIND, NAME, GROUP) { #NAME, (void *const *)solid_gpu_##NAME, KIND },
#define SD_NAMED_BOOL(NAME, GROUP) SD_NAMED(0, NAME, GROUP)
#define SD_NAMED_U64(NAME, GROUP)  SD_NAMED(1, NAME, GROUP)
#define SD_NAMED_VOID(NAME, GROUP) SD_NAMED(2, NAME, GROUP)
const NamedTable named_tables[] = {
   SOLID_GPU_REDUCE_BOOL_OPS(SD_NAMED_BOOL)
   SOLID_GPU_REDUCE_U64_OPS(SD_NAMED_U64)
   SOLID_GPU_REDUCE_VOID_OPS(SD_NAMED_VOID)
};
} // namespace

extern "C" int solid_gpu_reduce_all_device(const char *op, int dtype, SOLID_GPU_ARGS_REDUCE_HEAD,
                                           void *result, void *buffer, cudaStream_t stream)
{
   if (dtype < 0 || dtype >= SOLID_NUM_TYPES) SD_ERROR("Invalid type index %d", dtype);
   if (result == nullptr) SD_ERROR("Device result pointer is NULL");
   for (const NamedTable &t : named_tables) {
      if (strcmp(t.name, op) != 0) continue;
      void *fn = t.table[dtype];
      if (fn == nullptr) SD_ERROR("Reduction '%s' is not available for type index %d", op, dtype);
      sd::reduce_all_device_result = result;
      // the three signatures differ only in the static type of the result pointer
      int status = ((solid_funptr_gpu_sum)fn)(ndims, size, strides, ptr, nullptr, buffer, stream);
      sd::reduce_all_device_result = nullptr;
      return status;
   }
   SD_ERROR("Unknown reduction '%s'", op);
}
