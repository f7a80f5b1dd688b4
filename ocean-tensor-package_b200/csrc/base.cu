// Library-level entry points: error text, device property cache, type sizes,
// start-up kernel.  Counterparts in the reference: solid/src/base/gpu/solid_gpu.c,
// solid/src/base/generic/error.c:19-20, solid/src/core/gpu/template_dtype.cu:21-55,
// solid/src/core/gpu/template_dummy.cu:21-37.
#include <cstdlib>
#include <mutex>
#include "solid_core_gpu.h"
#include "layout.h"

static char solid_errmsg_buffer[SOLID_ERRMSG_SIZE] = "";
extern "C" __attribute__((weak)) char *solid_errmsg = solid_errmsg_buffer;

extern "C" const int solid_gpu_type_size[]     = { 1, 1, 2, 4, 8, 1, 2, 4, 8, 2, 4, 8, 4, 8, 16 };
// work types: bool -> bool, half -> float, chalf -> cfloat (solid/include/solid/base/gpu/dtype_gpu.h:83-85)
extern "C" const int solid_gpu_worktype_size[] = { 1, 1, 2, 4, 8, 1, 2, 4, 8, 4, 4, 8, 8, 8, 16 };

namespace {
std::mutex            g_lock;
solid_gpu_properties *g_props = nullptr;
int                   g_count = 0;
int                   g_refs  = 0;

int load_properties()
{
   int n = 0;
   cudaGetLastError();
   cudaError_t st = cudaGetDeviceCount(&n);
   if (st != cudaSuccess) {
      if (st != cudaErrorNoDevice && st != cudaErrorInsufficientDriver)
         SD_ERROR("Error determining the number of GPU devices (%s)", cudaGetErrorString(st));
      cudaGetLastError();
      n = 0;
   }
   if (n == 0) { g_count = 0; return 0; }
   g_props = (solid_gpu_properties *)calloc((size_t)n, sizeof(solid_gpu_properties));
   if (!g_props) SD_ERROR("Error allocating the device property table");
   for (int d = 0; d < n; d++) {
      cudaDeviceProp prop;
      if (cudaGetDeviceProperties(&prop, d) != cudaSuccess) {
         free(g_props); g_props = nullptr;
         SD_ERROR("Error reading the properties of device %d", d);
      }
      solid_gpu_properties &p = g_props[d];
      p.major = prop.major; p.minor = prop.minor;
      p.multiprocessor_count = prop.multiProcessorCount;
      p.max_threads_per_block = prop.maxThreadsPerBlock;
      p.max_threads_per_multiprocessor = prop.maxThreadsPerMultiProcessor;
      p.max_blocks_per_multiprocessor = prop.maxBlocksPerMultiProcessor;
      p.max_warps_per_multiprocessor = prop.maxThreadsPerMultiProcessor / 32;
      p.max_resident_blocks_per_device = p.max_blocks_per_multiprocessor * p.multiprocessor_count;
      p.max_shared_mem_per_multiprocessor = (int)prop.sharedMemPerMultiprocessor;
      p.max_shared_mem_per_threadblock = (int)prop.sharedMemPerBlock;
      for (int i = 0; i < 3; i++) { p.max_gridsize[i] = prop.maxGridSize[i]; p.max_blocksize[i] = prop.maxThreadsDim[i]; }
   }
   g_count = n;
   return 0;
}
} // namespace

extern "C" int solid_gpu_initialize(void)
{
   std::lock_guard<std::mutex> guard(g_lock);
   if (g_refs++ == 0 && g_props == nullptr) {
      if (load_properties() != 0) { g_refs--; return -1; }
   }
   return 0;
}

extern "C" void solid_gpu_finalize(void)
{
   std::lock_guard<std::mutex> guard(g_lock);
   if (g_refs > 0 && --g_refs == 0) { free(g_props); g_props = nullptr; g_count = 0; }
}

extern "C" int solid_gpu_check_status(void)
{
   cudaError_t st = cudaGetLastError();
   if (st != cudaSuccess) SD_ERROR("Cuda error: %s", cudaGetErrorString(st));
   return 0;
}

extern "C" int solid_gpu_get_current_device(int *device)
{
   if (cudaGetDevice(device) != cudaSuccess) SD_ERROR("Error getting the current device");
   return 0;
}

extern "C" solid_gpu_properties *solid_gpu_get_device_properties(int device)
{
   {  std::lock_guard<std::mutex> guard(g_lock);
      if (g_props == nullptr && load_properties() != 0) return nullptr;     // usable without initialize()
   }
   if (device < 0 || device >= g_count) {
      snprintf(solid_errmsg, SOLID_ERRMSG_SIZE, "Invalid device index %d", device);
      return nullptr;
   }
   return &g_props[device];
}

extern "C" solid_gpu_properties *solid_gpu_get_current_device_properties(void)
{
   int device;
   if (solid_gpu_get_current_device(&device) != 0) return nullptr;
   return solid_gpu_get_device_properties(device);
}

extern "C" int solid_gpu_multiprocessor_count(int device)
{
   solid_gpu_properties *p = solid_gpu_get_device_properties(device);
   return p ? p->multiprocessor_count : -1;
}

extern "C" int solid_gpu_max_threads_per_multiprocessor(int device)
{
   solid_gpu_properties *p = solid_gpu_get_device_properties(device);
   return p ? p->max_threads_per_multiprocessor : -1;
}

int sd::current_device_info(sd::DeviceInfo *info)
{
   int device;
   if (solid_gpu_get_current_device(&device) != 0) return -1;
   solid_gpu_properties *p = solid_gpu_get_device_properties(device);
   if (!p) return -1;
   info->device = device;
   info->sms = p->multiprocessor_count;
   info->max_threads_per_sm = p->max_threads_per_multiprocessor;
   return 0;
}

static __global__ void solid_gpu_warmup_kernel(int *flag) { if (flag) *flag = 1; }

extern "C" int solid_gpu_dummy_kernel(void)
{
   solid_gpu_warmup_kernel<<<1, 1>>>(nullptr);
   SD_LAUNCH_CHECK();
   return 0;
}
