/*
 * Ocean-level GPU dispatch for the elementwise / copy / fill / reduction path: the functions
 * Ocean's interface layer reaches through the OcModuleCore table of device type "GPU"
 * (include/ocean/core/interface/module_core.h:43-164 of the reference), re-implemented on top of
 * the Solid tables of solid_core_gpu.h.  Reference implementations being replaced:
 *   src/core/gpu/op/tensor_unary_gpu.c:59-91        OcTensorGPU_<unary>(src, dst)
 *   src/core/gpu/op/tensor_binary_gpu.c:58-94       OcTensorGPU_<binary>(src1, src2, dst)
 *   src/core/gpu/op/tensor_copy_gpu.c:89-132        OcTensorGPU_copy(src, dst)
 *   src/core/gpu/op/tensor_fill_gpu.c               OcTensorGPU_fill / fillNaN / maskedFill
 *   src/core/gpu/op/tensor_reduce_all_gpu.c:126-397 OcTensorGPU_<reduction>(tensor, result)
 *   src/core/gpu/op/tensor_reduce_axis_gpu.c:127-230 OcTensorGPU_axis<Reduction>(src, n, axes, dst)
 *
 * The reference passes OcTensor objects; a caller outside Ocean has none, so the functions take a
 * plain description of the same facts (OcTensorView).  Names, argument order, preconditions and
 * error behaviour are the reference's:
 *   - operands of elementwise functions have ONE dtype (the interface layer converted them),
 *     one shape (broadcast = zero strides), native byte order and aligned data; only copy
 *     accepts differing dtypes, byte orders, shapes of equal element count and unaligned data;
 *   - return 0, or -1 with the text available from OcGPU_errorMessage();
 *   - work is queued on the DESTINATION's stream; sources written on other streams are waited for
 *     through their events, and the destination's event is recorded afterwards
 *     (OcTensor_startRead / OcTensor_update / OcTensor_finishRead, src/base/storage.c:141-222);
 *   - global reductions return host scalars after one synchronisation; their scratch comes from a
 *     three-slot round-robin cache per device, as Ocean's temporaries do
 *     (src/core/interface/storage_itf.c:61-121), so it is never freed while in use.
 */
#ifndef OCEAN_GPU_B200_H
#define OCEAN_GPU_B200_H

#include "solid_core_gpu.h"

typedef struct {
   int          dtype;                              /* solid_type_index == Ocean's dtype order      */
   int          ndims;
   size_t       size[SOLID_MAX_TENSOR_DIMS];
   ptrdiff_t    strides[SOLID_MAX_TENSOR_DIMS];     /* bytes                                        */
   void        *data;                               /* device address of element (0,...,0)          */
   int          device;                             /* CUDA device index                            */
   int          byteswapped;                        /* stored bytes of each component are reversed  */
   cudaStream_t stream;                             /* stream of the tensor's storage               */
   cudaEvent_t  event;                              /* recorded after each write; may be NULL       */
} OcTensorView;

typedef struct {
   int          dtype;
   solid_scalar value;
} OcScalarView;

SOLID_API const char *OcGPU_errorMessage(void);
SOLID_API int  OcInitGPU_B200(void);                /* property cache, warm-up kernel on every device */
SOLID_API void OcFinalizeGPU_B200(void);            /* releases the scratch caches                     */

/* dst = f(src) -- list SOLID_GPU_UNARY_OPS, Ocean names (bitwise_not -> bitwiseNot, ...) */
#define OCGPU_UNARY_OPS(X) \
   X(negative, negative) X(bitwiseNot, bitwise_not) X(logicalNot, logical_not) X(conj, conj) \
   X(reciprocal, reciprocal) X(sin, sin) X(cos, cos) X(tan, tan) X(sinh, sinh) X(cosh, cosh) X(tanh, tanh) \
   X(arcsin, arcsin) X(arccos, arccos) X(arctan, arctan) X(arcsinh, arcsinh) X(arccosh, arccosh) \
   X(arctanh, arctanh) X(sqrt, sqrt) X(cbrt, cbrt) X(square, square) X(exp, exp) X(exp2, exp2) \
   X(exp10, exp10) X(expm1, expm1) X(log, log) X(log2, log2) X(log10, log10) X(log1p, log1p) \
   X(absolute, absolute) X(fabs, fabs) X(sign, sign) X(ceil, ceil) X(floor, floor) X(trunc, trunc) \
   X(round, round) X(isinf, isinf) X(isnan, isnan) X(isfinite, isfinite) X(isposinf, isposinf) X(isneginf, isneginf)
#define OCGPU_DECLARE_UNARY_(OP, SOLID) SOLID_API int OcTensorGPU_##OP(const OcTensorView *src, const OcTensorView *dst);
OCGPU_UNARY_OPS(OCGPU_DECLARE_UNARY_)

/* dst = f(src1, src2) -- include/ocean/core/generic/generate_tensor_binary.h */
#define OCGPU_BINARY_OPS(X) \
   X(add, add) X(subtract, subtract) X(scale, multiply) X(divide, divide) X(trueDivide, true_divide) \
   X(floorDivide, floor_divide) X(power, power) X(mod, mod) X(fmod, fmod) \
   X(elemwiseMin, min) X(elemwiseMax, max) X(elemwiseFMin, fmin) X(elemwiseFMax, fmax) \
   X(elemwiseLT, lt) X(elemwiseLE, le) X(elemwiseEQ, eq) X(elemwiseNE, ne) X(elemwiseGE, ge) X(elemwiseGT, gt) \
   X(bitwiseAnd, bitwise_and) X(bitwiseOr, bitwise_or) X(bitwiseXor, bitwise_xor) \
   X(logicalAnd, logical_and) X(logicalOr, logical_or) X(logicalXor, logical_xor) \
   X(bitshiftLeft, bitshift_left) X(bitshiftRight, bitshift_right)
#define OCGPU_DECLARE_BINARY_(OP, SOLID) \
   SOLID_API int OcTensorGPU_##OP(const OcTensorView *src1, const OcTensorView *src2, const OcTensorView *dst);
OCGPU_BINARY_OPS(OCGPU_DECLARE_BINARY_)

/* Tensor (op) scalar with the scalar passed by value: the forms behind OcTensor_addScalar, _subtractScalar,      */
/* _multiplyScalar and _bitwise{And,Or,Xor}Scalar (src/core/interface/tensor_itf.c:4215-4251), which the reference */
/* runs as tensor operations on a 0-d device tensor built from the scalar.  The scalar must have the tensor's dtype. */
#define OCGPU_SCALAR_OPS(X) \
   X(addScalar, add_scalar) X(subtractScalar, subtract_scalar) X(multiplyScalar, multiply_scalar) \
   X(bitwiseAndScalar, bitwise_and_scalar) X(bitwiseOrScalar, bitwise_or_scalar) X(bitwiseXorScalar, bitwise_xor_scalar)
#define OCGPU_DECLARE_SCALAR_(OP, SOLID) \
   SOLID_API int OcTensorGPU_##OP(const OcTensorView *src, const OcScalarView *scalar, const OcTensorView *dst);
OCGPU_SCALAR_OPS(OCGPU_DECLARE_SCALAR_)

/* Ranges (src/core/gpu/op/tensor_steps_gpu.c:52-140): element i = offset + i * step.  As in the reference the  */
/* tensor is first reduced to its memory layout (unit and zero-stride dimensions dropped, negative strides made   */
/* positive, dimensions sorted by stride and merged: OcSolid_analyzeElemwise1), so i counts in memory order.      */
SOLID_API int OcTensorGPU_stepsInt64(const OcTensorView *tensor, solid_int64 offset, solid_int64 step);
SOLID_API int OcTensorGPU_stepsDouble(const OcTensorView *tensor, solid_double offset, solid_double step);
SOLID_API int OcTensorGPU_stepsCDouble(const OcTensorView *tensor, solid_cdouble offset, solid_cdouble step);

/* Indexed access (src/core/gpu/op/tensor_index_gpu.c:58-260).  An index view is the indexed tensor plus, per         */
/* dimension, either NULL (the dimension is addressed by its stride) or a 1-D contiguous int64 tensor on the same     */
/* device holding one BYTE offset per selected position; `size` is the shape of the selection.                        */
typedef struct {
   OcTensorView        view;          /* the indexed tensor (its strides serve the dimensions without a table)      */
   int                 ndims;         /* dimensions of the selection                                                 */
   size_t              size[8];       /* shape of the selection                                                      */
   const OcTensorView *offsets[8];    /* per dimension: NULL or the table                                            */
} OcIndexView;
SOLID_API int OcTensorGPU_getIndex(const OcIndexView *index, const OcTensorView *dst);        /* dst = view[index]   */
SOLID_API int OcTensorGPU_setIndex(const OcIndexView *index, const OcTensorView *src);        /* view[index] = src   */
SOLID_API int OcTensorGPU_fillIndex(const OcIndexView *index, const OcScalarView *scalar);    /* view[index] = value */
SOLID_API int OcTensorGPU_addIfNegative(const OcTensorView *tensor, const OcScalarView *scalar);
/* tensor: nstrides x nelem (or 1-D: nelem) integer indices; offsets: nelem int64 results, sum strides[i] * index[i] */
SOLID_API int OcTensorGPU_indexToOffset(const OcTensorView *tensor, const solid_int64 *strides, const OcTensorView *offsets);

SOLID_API int OcTensorGPU_copy(const OcTensorView *src, const OcTensorView *dst);
SOLID_API int OcTensorGPU_byteswapNoFlag(const OcTensorView *tensor);   /* reverses the stored bytes in place */
SOLID_API int OcTensorGPU_fill(const OcTensorView *tensor, const OcScalarView *scalar);
SOLID_API int OcTensorGPU_fillNaN(const OcTensorView *tensor, const OcScalarView *scalar);
SOLID_API int OcTensorGPU_maskedFill(const OcTensorView *tensor, const OcTensorView *mask, const OcScalarView *scalar);

/* global reductions: int / OcUInt64 / scalar results on the HOST */
#define OCGPU_REDUCE_BOOL_OPS(X)  X(any, any) X(all, all) X(allFinite, all_finite) X(anyInf, any_inf) X(anyNaN, any_nan)
#define OCGPU_REDUCE_SCALAR_OPS(X) \
   X(sum, sum) X(prod, prod) X(sumNaN, sum_nan) X(prodNaN, prod_nan) X(sumAbs, sum_abs) X(sumAbsNaN, sum_abs_nan) \
   X(maximum, maximum) X(minimum, minimum) X(maximumAbs, maximum_abs) X(minimumAbs, minimum_abs) \
   X(norm2, norm2) X(norm2NaN, norm2_nan)
#define OCGPU_DECLARE_RBOOL_(OP, SOLID)   SOLID_API int OcTensorGPU_##OP(const OcTensorView *tensor, int *result);
#define OCGPU_DECLARE_RSCALAR_(OP, SOLID) SOLID_API int OcTensorGPU_##OP(const OcTensorView *tensor, OcScalarView *result);
OCGPU_REDUCE_BOOL_OPS(OCGPU_DECLARE_RBOOL_)
OCGPU_REDUCE_SCALAR_OPS(OCGPU_DECLARE_RSCALAR_)
SOLID_API int OcTensorGPU_nnz(const OcTensorView *tensor, solid_uint64 *result);
SOLID_API int OcTensorGPU_nnzNaN(const OcTensorView *tensor, solid_uint64 *result);
SOLID_API int OcTensorGPU_norm(const OcTensorView *tensor, double p, OcScalarView *result);
SOLID_API int OcTensorGPU_normNaN(const OcTensorView *tensor, double p, OcScalarView *result);
SOLID_API int OcTensorGPU_allLT(const OcTensorView *tensor, const OcScalarView *bound, int *result);
SOLID_API int OcTensorGPU_allLE(const OcTensorView *tensor, const OcScalarView *bound, int *result);
SOLID_API int OcTensorGPU_allGT(const OcTensorView *tensor, const OcScalarView *bound, int *result);
SOLID_API int OcTensorGPU_allGE(const OcTensorView *tensor, const OcScalarView *bound, int *result);
SOLID_API int OcTensorGPU_allGTLT(const OcTensorView *tensor, const OcScalarView *lower, const OcScalarView *upper, int *result);
SOLID_API int OcTensorGPU_allGTLE(const OcTensorView *tensor, const OcScalarView *lower, const OcScalarView *upper, int *result);
SOLID_API int OcTensorGPU_allGELT(const OcTensorView *tensor, const OcScalarView *lower, const OcScalarView *upper, int *result);
SOLID_API int OcTensorGPU_allGELE(const OcTensorView *tensor, const OcScalarView *lower, const OcScalarView *upper, int *result);

/* axis reductions: dst holds the kept dimensions in order (result dtype as reduce_ops.h defines it) */
#define OCGPU_AXIS_OPS(X) \
   X(axisAny, axis_any) X(axisAll, axis_all) X(axisAllFinite, axis_all_finite) X(axisAnyInf, axis_any_inf) \
   X(axisAnyNaN, axis_any_nan) X(axisNnz, axis_nnz) X(axisNnzNaN, axis_nnz_nan) X(axisSum, axis_sum) \
   X(axisProd, axis_prod) X(axisSumNaN, axis_sum_nan) X(axisProdNaN, axis_prod_nan) X(axisSumAbs, axis_sum_abs) \
   X(axisSumAbsNaN, axis_sum_abs_nan) X(axisMinimum, axis_minimum) X(axisMaximum, axis_maximum) \
   X(axisMinimumAbs, axis_minimum_abs) X(axisMaximumAbs, axis_maximum_abs) X(axisNorm2, axis_norm2) X(axisNorm2NaN, axis_norm2_nan)
#define OCGPU_DECLARE_AXIS_(OP, SOLID) \
   SOLID_API int OcTensorGPU_##OP(const OcTensorView *src, int n, const int *axes, const OcTensorView *dst);
OCGPU_AXIS_OPS(OCGPU_DECLARE_AXIS_)
SOLID_API int OcTensorGPU_axisNorm(const OcTensorView *src, double p, int n, const int *axes, const OcTensorView *dst);
SOLID_API int OcTensorGPU_axisNormNaN(const OcTensorView *src, double p, int n, const int *axes, const OcTensorView *dst);

/* result dtype of a reduction named as in the Solid tables ("sum", "axis_norm2", ...) over `dtype`; -1 if unknown */
SOLID_API int OcGPU_reductionResultType(const char *solid_name, int dtype);

#endif
