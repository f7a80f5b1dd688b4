/*
 * Binding of the B200 dispatch library into Ocean: the OcModuleCore entries of device type "GPU"
 * for the elementwise, copy / fill and reduction path.
 *
 * This file takes the place of six files of the reference's GPU module,
 *    src/core/gpu/op/tensor_{unary,binary,copy,fill,reduce_all,reduce_axis}_gpu.c,
 * and is compiled with the REST of that module unchanged (device, stream and storage management in
 * src/core/gpu; GEMM, ranges and indexed access in src/core/gpu/op/tensor_{blas,steps,index}_gpu.c).
 * It defines the six registration functions that src/core/gpu/tensor_gpu.c:35-50 calls; each one
 * fills its share of the module table (include/ocean/core/interface/module_core.h:43-164) with an
 * adaptor that describes the OcTensor arguments as OcTensorView (dtype, sizes, byte strides, data
 * pointer, device, byte order, CUDA stream and event of the storage) and calls the function of the
 * same Ocean name in libocean_gpu_b200.so (include/ocean_gpu_b200.h), which looks the Solid kernel
 * up, activates the device, orders the streams and launches.  Errors come back as text and are
 * raised through OcError, as the reference's dispatch does.
 *
 * Two things the reference's GPU module does not have are switched on here, because the kernels
 * below support them:
 *   - Tensor_byteswapNoFlag is registered and Tensor_copy accepts byte-swapped tensors (the
 *     reference refuses them, src/core/gpu/op/tensor_copy_gpu.c:102-105, and the interface layer
 *     detours through the CPU, src/core/interface/tensor_itf.c:930-965);
 *   - GPU devices no longer require aligned data (src/core/gpu/device_gpu.c:96 sets the flag): the
 *     copy family reads and writes any address, and elementwise operations still get aligned
 *     operands because OcTensorOp_alignTensors clones unaligned ones through Tensor_copy.
 *
 * Needs the Ocean headers of a checkout, so it is built where one is present (oracle/build_ocean.py).
 */
#include "ocean/core/gpu/op/tensor_unary_gpu.h"
#include "ocean/core/gpu/op/tensor_binary_gpu.h"
#include "ocean/core/gpu/op/tensor_copy_gpu.h"
#include "ocean/core/gpu/op/tensor_fill_gpu.h"
#include "ocean/core/gpu/op/tensor_reduce_all_gpu.h"
#include "ocean/core/gpu/op/tensor_reduce_axis_gpu.h"
#include "ocean/core/interface/tensor_itf.h"
#include "ocean/core/gpu/tensor_gpu.h"
#include "ocean/core/gpu/storage_gpu.h"
#include "ocean/core/gpu/device_gpu.h"
#include "ocean/core/gpu/cuda.h"
#include "ocean/base/shape.h"
#include "ocean/base/error.h"
#include "ocean/external/ocean-solid/ocean_solid.h"

#include "ocean_gpu_b200.h"

#include <string.h>


/* ------------------------------------------------------------------------------------------ */
/* Adaptors                                                                                   */
/* ------------------------------------------------------------------------------------------ */

static void view_of(OcTensor *t, OcTensorView *v)
{  int i;

   v -> dtype = (int)(t -> dtype);                       /* OcDType and solid_type_index share their order */
   v -> ndims = t -> ndims;
   for (i = 0; i < t -> ndims; i++)
   {  v -> size[i]    = (size_t)(t -> size[i]);
      v -> strides[i] = (ptrdiff_t)(t -> strides[i]);
   }
   v -> data        = (void *)OcTensor_data(t);
   v -> device      = t -> device -> index;
   v -> byteswapped = OcTensor_isByteswapped(t) ? 1 : 0;
   v -> stream      = OcTensorGPU_cudaStream(t);
   v -> event       = ((OcEventGPU *)(t -> storage -> event)) -> cudaEvent;
}

static void scalar_of(OcScalar *s, OcScalarView *v)
{
   v -> dtype = (int)(s -> dtype);
   memset(&(v -> value), 0, sizeof(v -> value));
   memcpy(&(v -> value), OcScalar_data(s), (size_t)OcDType_size(s -> dtype));
}

static int report(int status)
{
   if (status != 0) OcError(-1, "%s", OcGPU_errorMessage());
   return 0;
}


/* ------------------------------------------------------------------------------------------ */
/* Unary and binary elementwise operations                                                    */
/* ------------------------------------------------------------------------------------------ */

/* The table look-up is repeated here with the reference's own macro so that a missing type raises the reference's  */
/* message, description included ("The unary negative function is not available for type uint8 on GPU").            */
#define OC_TEMPLATE(NAME, SOLID_OP, CHECK, DESC) \
static int b200_##NAME(OcTensor *src, OcTensor *dst) \
{  OcTensorView vs, vd; \
   solid_funptr_gpu_##SOLID_OP funptr; \
   OC_SOLID_FUNPTR(DESC, solid_gpu_##SOLID_OP, funptr, src -> dtype, "GPU"); \
   if (funptr == 0) return -1; \
   view_of(src, &vs); view_of(dst, &vd); \
   return report(OcTensorGPU_##NAME(&vs, &vd)); \
}
#include "ocean/core/generic/generate_tensor_unary.h"
#undef OC_TEMPLATE

void OcTensorGPU_initializeUnaryOps(OcModuleCore *module)
{
   #define OC_TEMPLATE(NAME, SOLID_OP, CHECK, DESC) module -> Tensor_##NAME = b200_##NAME;
   #include "ocean/core/generic/generate_tensor_unary.h"
   #undef OC_TEMPLATE
}

#define OC_TEMPLATE(NAME, SOLID_OP, CHECK, DESC) \
static int b200_##NAME(OcTensor *src1, OcTensor *src2, OcTensor *dst) \
{  OcTensorView v1, v2, vd; \
   solid_funptr_gpu_##SOLID_OP funptr; \
   OC_SOLID_FUNPTR(DESC, solid_gpu_##SOLID_OP, funptr, src1 -> dtype, "GPU"); \
   if (funptr == 0) return -1; \
   view_of(src1, &v1); view_of(src2, &v2); view_of(dst, &vd); \
   return report(OcTensorGPU_##NAME(&v1, &v2, &vd)); \
}
#include "ocean/core/generic/generate_tensor_binary.h"
#undef OC_TEMPLATE

void OcTensorGPU_initializeBinaryOps(OcModuleCore *module)
{
   #define OC_TEMPLATE(NAME, SOLID_OP, CHECK, DESC) module -> Tensor_##NAME = b200_##NAME;
   #include "ocean/core/generic/generate_tensor_binary.h"
   #undef OC_TEMPLATE
}


/* ------------------------------------------------------------------------------------------ */
/* Fill                                                                                       */
/* ------------------------------------------------------------------------------------------ */

static int b200_fill(OcTensor *tensor, OcScalar *scalar)
{  OcTensorView v; OcScalarView s;
   view_of(tensor, &v); scalar_of(scalar, &s);
   return report(OcTensorGPU_fill(&v, &s));
}

static int b200_fillNaN(OcTensor *tensor, OcScalar *scalar)
{  OcTensorView v; OcScalarView s;
   view_of(tensor, &v); scalar_of(scalar, &s);
   return report(OcTensorGPU_fillNaN(&v, &s));
}

static int b200_maskedFill(OcTensor *tensor, OcTensor *mask, OcScalar *scalar)
{  OcTensorView v, m; OcScalarView s;
   view_of(tensor, &v); view_of(mask, &m); scalar_of(scalar, &s);
   return report(OcTensorGPU_maskedFill(&v, &m, &s));
}

void OcTensorGPU_initializeFillOps(OcModuleCore *module)
{
   module -> Tensor_fill       = b200_fill;
   module -> Tensor_fillNaN    = b200_fillNaN;
   module -> Tensor_maskedFill = b200_maskedFill;
}


/* ------------------------------------------------------------------------------------------ */
/* Copy                                                                                       */
/* ------------------------------------------------------------------------------------------ */

/* Same element type, same byte order, same dense layout: the bytes can move as one block */
static int block_copyable(OcTensor *src, OcTensor *dst)
{
   return ((src -> dtype == dst -> dtype) &&
           (OcTensors_haveSameByteOrder(src, dst)) &&
           (OcTensor_isContiguous(src)) &&
           (OcTensors_haveCompatibleLayout(src, dst)));
}

static void block_extent(OcTensor *src, OcTensor *dst, OcSize *offset1, OcSize *offset2, OcSize *extent)
{
   OcShape_extent(src -> ndims, src -> size, src -> strides, src -> elemsize, offset1, extent);
   OcShape_extent(dst -> ndims, dst -> size, dst -> strides, dst -> elemsize, offset2, NULL);
}

static int b200_copy(OcTensor *src, OcTensor *dst)
{  OcTensorView vs, vd;
   OcSize o1, o2, extent;

   /* The interface layer guarantees a writable destination without zero strides or self overlap, equal */
   /* element counts and no overlap between the tensors; dtype, byte order and device may all differ.   */
   if (block_copyable(src, dst))
   {  block_extent(src, dst, &o1, &o2, &extent);
      return OcBufferGPU_copy(src -> storage, OcTensor_data(src) - o1,
                              dst -> storage, OcTensor_data(dst) - o2, OcDTypeInt8, extent);
   }

   /* Conversion, byte order, strides, alignment and a source on another GPU are all handled by the copy kernel */
   view_of(src, &vs); view_of(dst, &vd);
   return report(OcTensorGPU_copy(&vs, &vd));
}

static int b200_copyFromCPU(OcTensor *src, OcTensor *dst)
{  OcSize o1, o2, extent;

   if (block_copyable(src, dst))
   {  block_extent(src, dst, &o1, &o2, &extent);
      return OcBufferGPU_copyFromCPU(src -> storage, OcTensor_data(src) - o1,
                                     dst -> storage, OcTensor_data(dst) - o2, OcDTypeInt8, extent);
   }
   return OcTensor_intrnlCopyDevices(src, dst);          /* through dense temporaries on both sides */
}

static int b200_copyToCPU(OcTensor *src, OcTensor *dst)
{  OcSize o1, o2, extent;

   if (block_copyable(src, dst) && OcTensors_haveIdenticalLayout(src, dst))
   {  block_extent(src, dst, &o1, &o2, &extent);
      return OcBufferGPU_copyToCPU(src -> storage, OcTensor_data(src) - o1,
                                   dst -> storage, OcTensor_data(dst) - o2, OcDTypeInt8, extent);
   }
   return OcTensor_intrnlCopyDevices(src, dst);
}

static int b200_byteswapNoFlag(OcTensor *tensor)
{  OcTensorView v;
   view_of(tensor, &v);
   return report(OcTensorGPU_byteswapNoFlag(&v));
}

void OcTensorGPU_initializeCopyOps(OcModuleCore *module)
{  OcDeviceType *type;
   int i;

   module -> Tensor_copy           = b200_copy;
   module -> Tensor_copyFromCPU    = b200_copyFromCPU;
   module -> Tensor_copyToCPU      = b200_copyToCPU;
   module -> Tensor_byteswapNoFlag = b200_byteswapNoFlag;

   /* The device instances exist by now (OcInitDevicesGPU runs before the module is filled) */
   type = OcDeviceTypeByName("GPU");
   for (i = 0; (type != NULL) && (i < OcDeviceType_deviceCount(type)); i++)
   {  OcDevice *device = OcDeviceType_getDevice(type, i);
      if (device) device -> requiresAlignedData = 0;
   }
}


/* ------------------------------------------------------------------------------------------ */
/* Global reductions                                                                          */
/* ------------------------------------------------------------------------------------------ */

#define B200_REDUCE_INT(NAME) \
static int b200_##NAME(OcTensor *tensor, int *result) \
{  OcTensorView v; \
   view_of(tensor, &v); \
   return report(OcTensorGPU_##NAME(&v, result)); \
}
B200_REDUCE_INT(any) B200_REDUCE_INT(all) B200_REDUCE_INT(allFinite) B200_REDUCE_INT(anyInf) B200_REDUCE_INT(anyNaN)

#define B200_REDUCE_U64(NAME) \
static int b200_##NAME(OcTensor *tensor, OcUInt64 *result) \
{  OcTensorView v; solid_uint64 value = 0; int status; \
   view_of(tensor, &v); \
   status = OcTensorGPU_##NAME(&v, &value); \
   if (status == 0) *result = (OcUInt64)value; \
   return report(status); \
}
B200_REDUCE_U64(nnz) B200_REDUCE_U64(nnzNaN)

/* The caller has set result -> dtype to the reduction's result type; the value goes into its union */
static int scalar_result(int status, OcScalarView *value, OcScalar *result)
{
   if (status == 0) memcpy(OcScalar_data(result), &(value -> value), (size_t)OcDType_size(result -> dtype));
   return report(status);
}

#define B200_REDUCE_SCALAR(NAME) \
static int b200_##NAME(OcTensor *tensor, OcScalar *result) \
{  OcTensorView v; OcScalarView value; \
   view_of(tensor, &v); \
   return scalar_result(OcTensorGPU_##NAME(&v, &value), &value, result); \
}
B200_REDUCE_SCALAR(sum)     B200_REDUCE_SCALAR(prod)    B200_REDUCE_SCALAR(sumNaN)     B200_REDUCE_SCALAR(prodNaN)
B200_REDUCE_SCALAR(sumAbs)  B200_REDUCE_SCALAR(sumAbsNaN)
B200_REDUCE_SCALAR(maximum) B200_REDUCE_SCALAR(minimum) B200_REDUCE_SCALAR(maximumAbs) B200_REDUCE_SCALAR(minimumAbs)
B200_REDUCE_SCALAR(norm2)   B200_REDUCE_SCALAR(norm2NaN)

#define B200_REDUCE_NORM(NAME) \
static int b200_##NAME(OcTensor *tensor, double p, OcScalar *result) \
{  OcTensorView v; OcScalarView value; \
   view_of(tensor, &v); \
   return scalar_result(OcTensorGPU_##NAME(&v, p, &value), &value, result); \
}
B200_REDUCE_NORM(norm) B200_REDUCE_NORM(normNaN)

#define B200_REDUCE_BOUND1(NAME) \
static int b200_##NAME(OcTensor *tensor, OcScalar *bound, int *result) \
{  OcTensorView v; OcScalarView b; \
   view_of(tensor, &v); scalar_of(bound, &b); \
   return report(OcTensorGPU_##NAME(&v, &b, result)); \
}
B200_REDUCE_BOUND1(allLT) B200_REDUCE_BOUND1(allLE) B200_REDUCE_BOUND1(allGT) B200_REDUCE_BOUND1(allGE)

#define B200_REDUCE_BOUND2(NAME) \
static int b200_##NAME(OcTensor *tensor, OcScalar *lower, OcScalar *upper, int *result) \
{  OcTensorView v; OcScalarView lo, hi; \
   view_of(tensor, &v); scalar_of(lower, &lo); scalar_of(upper, &hi); \
   return report(OcTensorGPU_##NAME(&v, &lo, &hi, result)); \
}
B200_REDUCE_BOUND2(allGTLT) B200_REDUCE_BOUND2(allGTLE) B200_REDUCE_BOUND2(allGELT) B200_REDUCE_BOUND2(allGELE)

void OcTensorGPU_initializeReduceAllOps(OcModuleCore *module)
{
   #define B200_SET(NAME) module -> Tensor_##NAME = b200_##NAME;
   B200_SET(any)     B200_SET(all)     B200_SET(allFinite)  B200_SET(anyInf)     B200_SET(anyNaN)
   B200_SET(nnz)     B200_SET(nnzNaN)
   B200_SET(sum)     B200_SET(prod)    B200_SET(sumNaN)     B200_SET(prodNaN)    B200_SET(sumAbs)   B200_SET(sumAbsNaN)
   B200_SET(maximum) B200_SET(minimum) B200_SET(maximumAbs) B200_SET(minimumAbs)
   B200_SET(norm2)   B200_SET(norm2NaN) B200_SET(norm)      B200_SET(normNaN)
   B200_SET(allLT)   B200_SET(allLE)   B200_SET(allGT)      B200_SET(allGE)
   B200_SET(allGTLT) B200_SET(allGTLE) B200_SET(allGELT)    B200_SET(allGELE)
   #undef B200_SET
}


/* ------------------------------------------------------------------------------------------ */
/* Axis reductions                                                                            */
/* ------------------------------------------------------------------------------------------ */

#define B200_AXIS(NAME) \
static int b200_##NAME(OcTensor *src, int n, int *axes, OcTensor *dst) \
{  OcTensorView vs, vd; \
   view_of(src, &vs); view_of(dst, &vd); \
   return report(OcTensorGPU_##NAME(&vs, n, axes, &vd)); \
}
B200_AXIS(axisAny)     B200_AXIS(axisAll)     B200_AXIS(axisAllFinite)  B200_AXIS(axisAnyInf)     B200_AXIS(axisAnyNaN)
B200_AXIS(axisNnz)     B200_AXIS(axisNnzNaN)
B200_AXIS(axisSum)     B200_AXIS(axisProd)    B200_AXIS(axisSumNaN)     B200_AXIS(axisProdNaN)
B200_AXIS(axisSumAbs)  B200_AXIS(axisSumAbsNaN)
B200_AXIS(axisMinimum) B200_AXIS(axisMaximum) B200_AXIS(axisMinimumAbs) B200_AXIS(axisMaximumAbs)
B200_AXIS(axisNorm2)   B200_AXIS(axisNorm2NaN)

#define B200_AXIS_NORM(NAME) \
static int b200_##NAME(OcTensor *src, double p, int n, int *axes, OcTensor *dst) \
{  OcTensorView vs, vd; \
   view_of(src, &vs); view_of(dst, &vd); \
   return report(OcTensorGPU_##NAME(&vs, p, n, axes, &vd)); \
}
B200_AXIS_NORM(axisNorm) B200_AXIS_NORM(axisNormNaN)

void OcTensorGPU_initializeReduceAxisOps(OcModuleCore *module)
{
   #define B200_SET(NAME) module -> Tensor_##NAME = b200_##NAME;
   B200_SET(axisAny)     B200_SET(axisAll)     B200_SET(axisAllFinite)  B200_SET(axisAnyInf)     B200_SET(axisAnyNaN)
   B200_SET(axisNnz)     B200_SET(axisNnzNaN)
   B200_SET(axisSum)     B200_SET(axisProd)    B200_SET(axisSumNaN)     B200_SET(axisProdNaN)
   B200_SET(axisSumAbs)  B200_SET(axisSumAbsNaN)
   B200_SET(axisMinimum) B200_SET(axisMaximum) B200_SET(axisMinimumAbs) B200_SET(axisMaximumAbs)
   B200_SET(axisNorm2)   B200_SET(axisNorm2NaN) B200_SET(axisNorm)      B200_SET(axisNormNaN)
   #undef B200_SET
}
