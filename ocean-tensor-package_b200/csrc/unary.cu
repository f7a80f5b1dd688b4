// solid_gpu_<unary op>_<SDX> for one element type (list: SOLID_GPU_UNARY_OPS).
// Replaces solid/src/core/gpu/template_unary.cu:52-246 for that type.
#include "unit.cuh"
#include "elemwise.cuh"
#include "ops_unary.cuh"

#define SD_DEFINE_UNARY(NAME, GROUP) SD_WHEN(GROUP)(                                              \
   extern "C" int SD_PASTE(solid_gpu_##NAME##_, SDX)(SOLID_GPU_ARGS_UNARY)                         \
   {  return sd::launch_unary<sd::u_##NAME, T>(ndims, size, strides1, ptr1, strides2, ptr2, stream); })

SOLID_GPU_UNARY_OPS(SD_DEFINE_UNARY)
