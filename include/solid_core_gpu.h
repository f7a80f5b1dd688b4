/*
 * C-ABI of the B200 Solid GPU core: the elementwise, copy/convert/fill and
 * reduction entry points that Ocean's GPU module binds.
 *
 * For every operation NAME listed below the library exports
 *     int solid_gpu_NAME_<type>(...)            one function per supported type
 *     solid_funptr_gpu_NAME solid_gpu_NAME[15]  table indexed by solid_type_index
 *                                               (NULL where the type is unsupported)
 * exactly as the header generated from the reference's
 * solid/src/core/gpu/solid_core_gpu.src does (generator: solid/bin/generate.py:194-432).
 * copy / copy_regular have two type indices: solid_gpu_copy[src][dst].
 *
 * Conventions (solid/src/core/gpu/solid_core_gpu.src:9-23, solid/include/solid/base/generic/error.h:22-35):
 *   - return 0 on success, -1 on error with the text in solid_errmsg;
 *   - strides in bytes; ndims == 0 means one element; any size[i] == 0 is a no-op;
 *   - all pointers are device pointers of the CURRENT device, except the
 *     `result` and bound/scalar arguments of the global reductions (host);
 *   - launches are asynchronous on `stream`; a global reduction returns after
 *     its value has reached the host;
 *   - nothing is allocated: scratch memory is passed in by the caller.
 *
 * The lists are X-macros: OPS(X) calls X(name, group) for each operation, and
 * SOLID_TYPES_<group>(F, name) calls F(name, type) for each type of the group.
 */
#ifndef SOLID_CORE_GPU_H
#define SOLID_CORE_GPU_H

#include "solid_gpu_types.h"

/* ------------------------------------------------------------------------ */
/* Type groups (solid/bin/generate.py:88-109)                               */
/* ------------------------------------------------------------------------ */
#define SOLID_TYPES_bool(F,N)    F(N,bool)
#define SOLID_TYPES_uint(F,N)    F(N,uint8) F(N,uint16) F(N,uint32) F(N,uint64)
#define SOLID_TYPES_sint(F,N)    F(N,int8) F(N,int16) F(N,int32) F(N,int64)
#define SOLID_TYPES_real(F,N)    F(N,half) F(N,float) F(N,double)
#define SOLID_TYPES_complex(F,N) F(N,chalf) F(N,cfloat) F(N,cdouble)
#define SOLID_TYPES_integer(F,N)       SOLID_TYPES_uint(F,N) SOLID_TYPES_sint(F,N)
#define SOLID_TYPES_float(F,N)         SOLID_TYPES_real(F,N) SOLID_TYPES_complex(F,N)
#define SOLID_TYPES_integer_bool(F,N)  SOLID_TYPES_bool(F,N) SOLID_TYPES_integer(F,N)
#define SOLID_TYPES_all(F,N)           SOLID_TYPES_bool(F,N) SOLID_TYPES_integer(F,N) SOLID_TYPES_float(F,N)
#define SOLID_TYPES_all_nobool(F,N)    SOLID_TYPES_integer(F,N) SOLID_TYPES_float(F,N)
#define SOLID_TYPES_all_nouint(F,N)    SOLID_TYPES_bool(F,N) SOLID_TYPES_sint(F,N) SOLID_TYPES_float(F,N)
#define SOLID_TYPES_all_nocomplex(F,N) SOLID_TYPES_bool(F,N) SOLID_TYPES_integer(F,N) SOLID_TYPES_real(F,N)
/* second copy of the full list, for the inner level of the two-type tables */
#define SOLID_TYPES2_all(F,N) \
   F(N,bool) F(N,uint8) F(N,uint16) F(N,uint32) F(N,uint64) F(N,int8) F(N,int16) F(N,int32) F(N,int64) \
   F(N,half) F(N,float) F(N,double) F(N,chalf) F(N,cfloat) F(N,cdouble)

/* ------------------------------------------------------------------------ */
/* Operation lists                                                          */
/* ------------------------------------------------------------------------ */

/* In-place with one scalar: (ndims,size,strides,ptr,value,stream)  -- .src:42-45 */
#define SOLID_GPU_FILL_OPS(X) \
   X(fill, all) X(fill_nan, float)

/* dst = f(src): (ndims,size,strides1,ptr1,strides2,ptr2,stream)    -- .src:105-189 */
#define SOLID_GPU_UNARY_OPS(X) \
   X(negative, all_nouint) X(conj, complex) X(reciprocal, all_nobool) \
   X(bitwise_not, integer_bool) X(logical_not, bool) \
   X(sin, all_nobool) X(cos, all_nobool) X(tan, all_nobool) \
   X(sinh, all_nobool) X(cosh, all_nobool) X(tanh, all_nobool) \
   X(arcsin, all_nobool) X(arccos, all_nobool) X(arctan, all_nobool) \
   X(arcsinh, all_nobool) X(arccosh, all_nobool) X(arctanh, all_nobool) \
   X(sqrt, all_nobool) X(cbrt, all_nobool) X(square, all_nobool) \
   X(exp, all_nobool) X(exp2, all_nobool) X(exp10, all_nobool) X(expm1, all_nobool) \
   X(log, all_nobool) X(log2, all_nobool) X(log10, all_nobool) X(log1p, all_nobool) \
   X(fabs, all) X(sign, all) \
   X(ceil, float) X(floor, float) X(trunc, float) X(round, float) \
   X(isinf, all) X(isnan, all) X(isfinite, all) \
   X(isposinf, all_nocomplex) X(isneginf, all_nocomplex) \
   X(absolute, all)

/* dst = f(a,b): (ndims,size,strides1,ptr1,strides2,ptr2,strides3,ptr3,stream) -- .src:196-283 */
/* Comparisons write bool.  bitshift_* take an int8 shift operand and power on */
/* bool/integer bases an int16 exponent (solid/src/core/gpu/template_binary.cu:201,260-264). */
#define SOLID_GPU_BINARY_OPS(X) \
   X(add, all) X(subtract, all) X(multiply, all) X(divide, all) X(true_divide, all) \
   X(floor_divide, all_nocomplex) X(mod, all_nocomplex) X(fmod, all_nocomplex) \
   X(bitwise_and, integer_bool) X(bitwise_or, integer_bool) X(bitwise_xor, integer_bool) \
   X(logical_and, bool) X(logical_or, bool) X(logical_xor, bool) \
   X(lt, all) X(le, all) X(ge, all) X(gt, all) X(eq, all) X(ne, all) \
   X(min, all) X(max, all) X(fmin, all) X(fmax, all) \
   X(bitshift_left, integer_bool) X(bitshift_right, integer_bool) \
   X(power, all)

/* Unary functions with a domain, fused with the domain test that Ocean runs as a separate global reduction      */
/* before them (OcTensor_sqrt and relatives, src/core/interface/tensor_itf.c:3822-3871: anyLTZero, anyLTNegOne,     */
/* anyLTOne, anyGTOneAbs; OcTensor_reciprocal :3786-3810: anyEQZero).  No counterpart in the reference's Solid      */
/* layer.  The result is that of the plain function; `outside` (device int, zeroed by the caller) is set to 1      */
/* when an element fails the test the reference applies: x < 0 for sqrt/log/log2/log10, x < -1 for log1p, x < 1     */
/* for arccosh, x < -1 or x > 1 for arcsin/arccos/arctanh, x == 0 for reciprocal (a NaN passes all of them, as in   */
/* the reference's all_ge / all_gele reductions).  One pass over the data instead of two.  Real floating types.     */
#define SOLID_GPU_CHECKED_OPS(X) \
   X(sqrt_checked, real) X(log_checked, real) X(log2_checked, real) X(log10_checked, real) X(log1p_checked, real) \
   X(arccosh_checked, real) X(arcsin_checked, real) X(arccos_checked, real) X(arctanh_checked, real) \
   X(reciprocal_checked, real)

/* Binary operations with the second operand a scalar passed BY VALUE: dst = op(src, value).      */
/* No counterpart in the reference's Solid layer: Ocean's addScalar, subtractScalar, multiplyScalar */
/* and bitwise{And,Or,Xor}Scalar build a 0-d device tensor from the scalar and call the tensor     */
/* operation (src/core/interface/tensor_itf.c:4215-4251, "Possible optimization"); these entry     */
/* points skip that tensor.  Results are those of the tensor operation with a broadcast operand.   */
#define SOLID_GPU_SCALAR_OPS(X) \
   X(add_scalar, all) X(subtract_scalar, all) X(multiply_scalar, all) \
   X(bitwise_and_scalar, integer_bool) X(bitwise_or_scalar, integer_bool) X(bitwise_xor_scalar, integer_bool)

/* Global reductions -- .src:293-366.  `result` is a HOST pointer, `buffer` device scratch */
/* of at least solid_gpu_reduce_all_buffer_size() bytes.                                   */
#define SOLID_GPU_REDUCE_BOOL_OPS(X)   /* (..., solid_bool *result, buffer, stream) */ \
   X(any, all) X(all, all) X(all_finite, float) X(any_inf, float) X(any_nan, float)
#define SOLID_GPU_REDUCE_BOUND1_OPS(X) /* (..., solid_scalar *bound, solid_bool *result, buffer, stream) */ \
   X(all_lt, all) X(all_le, all) X(all_gt, all) X(all_ge, all)
#define SOLID_GPU_REDUCE_BOUND2_OPS(X) /* (..., solid_scalar *lower, solid_scalar *upper, solid_bool *result, buffer, stream) */ \
   X(all_gtlt, all) X(all_gtle, all) X(all_gelt, all) X(all_gele, all)
#define SOLID_GPU_REDUCE_U64_OPS(X)    /* (..., solid_uint64 *result, buffer, stream) */ \
   X(nnz, all) X(nnz_nan, all)
#define SOLID_GPU_REDUCE_VOID_OPS(X)   /* (..., void *result, buffer, stream) */ \
   X(sum, all) X(sum_nan, all) X(prod, all) X(prod_nan, all) \
   X(sum_abs, all) X(sum_abs_nan, all) \
   X(maximum, all) X(minimum, all) X(maximum_abs, all) X(minimum_abs, all) \
   X(norm2, all) X(norm2_nan, all)
#define SOLID_GPU_REDUCE_NORM_OPS(X)   /* (..., double p, void *result, buffer, stream) */ \
   X(norm, all) X(norm_nan, all)

/* Axis reductions -- .src:380-412 */
#define SOLID_GPU_AXIS_OPS(X)          /* (solid_gpu_reduce_axis_config *config) */ \
   X(axis_any, all) X(axis_all, all) \
   X(axis_all_finite, float) X(axis_any_inf, float) X(axis_any_nan, float) \
   X(axis_nnz, all) X(axis_nnz_nan, all) \
   X(axis_sum, all) X(axis_sum_nan, all) X(axis_prod, all) X(axis_prod_nan, all) \
   X(axis_sum_abs, all) X(axis_sum_abs_nan, all) \
   X(axis_maximum, all) X(axis_minimum, all) X(axis_maximum_abs, all) X(axis_minimum_abs, all) \
   X(axis_norm2, all) X(axis_norm2_nan, all)
#define SOLID_GPU_AXIS_NORM_OPS(X)     /* (solid_gpu_reduce_axis_config *config, double p) */ \
   X(axis_norm, all) X(axis_norm_nan, all)

/* ------------------------------------------------------------------------ */
/* Argument lists                                                           */
/* ------------------------------------------------------------------------ */
#define SOLID_GPU_ARGS_FILL \
   int ndims, const size_t *size, const ptrdiff_t *strides, void *ptr, \
   const solid_scalar value, cudaStream_t stream
#define SOLID_GPU_ARGS_MASKED_FILL \
   int ndims, const size_t *size, const ptrdiff_t *strides1, void *ptr1, \
   const ptrdiff_t *strides2, void *ptr2, const solid_scalar value, cudaStream_t stream
#define SOLID_GPU_ARGS_UNARY \
   int ndims, const size_t *size, const ptrdiff_t *strides1, void *ptr1, \
   const ptrdiff_t *strides2, void *ptr2, cudaStream_t stream
#define SOLID_GPU_ARGS_UNARY_CHECKED \
   int ndims, const size_t *size, const ptrdiff_t *strides1, void *ptr1, \
   const ptrdiff_t *strides2, void *ptr2, int *outside, cudaStream_t stream
#define SOLID_GPU_ARGS_BINARY \
   int ndims, const size_t *size, const ptrdiff_t *strides1, void *ptr1, \
   const ptrdiff_t *strides2, void *ptr2, const ptrdiff_t *strides3, void *ptr3, \
   cudaStream_t stream
#define SOLID_GPU_ARGS_SCALAR_OP \
   int ndims, const size_t *size, const ptrdiff_t *strides1, void *ptr1, \
   const solid_scalar value, const ptrdiff_t *strides2, void *ptr2, cudaStream_t stream
#define SOLID_GPU_ARGS_STEPS_HEAD \
   int ndims, const size_t *size, const ptrdiff_t *strides, void *ptr
#define SOLID_GPU_ARGS_STEPS_INT64   SOLID_GPU_ARGS_STEPS_HEAD, solid_int64 offset, solid_int64 step, cudaStream_t stream
#define SOLID_GPU_ARGS_STEPS_DOUBLE  SOLID_GPU_ARGS_STEPS_HEAD, solid_double offset, solid_double step, cudaStream_t stream
#define SOLID_GPU_ARGS_STEPS_CDOUBLE SOLID_GPU_ARGS_STEPS_HEAD, solid_cdouble offset, solid_cdouble step, cudaStream_t stream
#define SOLID_GPU_ARGS_INDEX2 \
   int ndims, const size_t *size, solid_int64 **offsets, const ptrdiff_t *strides1, void *ptr1, \
   const ptrdiff_t *strides2, void *ptr2, cudaStream_t stream
#define SOLID_GPU_ARGS_FILL_INDEX \
   int ndims, const size_t *size, solid_int64 **offsets, const ptrdiff_t *strides, void *ptr, \
   const solid_scalar value, cudaStream_t stream
#define SOLID_GPU_ARGS_ADD_IF_NEGATIVE \
   int ndims, const size_t *size, const ptrdiff_t *strides, void *ptr, const solid_scalar value, cudaStream_t stream
#define SOLID_GPU_ARGS_INDEX_TO_OFFSET \
   int nstrides, solid_int64 *strides, ptrdiff_t strideReduce, size_t nelem, \
   ptrdiff_t stride1, void *ptr1, ptrdiff_t stride2, void *ptr2, cudaStream_t stream
#define SOLID_GPU_ARGS_GEMM \
   char transA, char transB, size_t M, size_t N, size_t K, void *ptrAlpha, void *ptrA, ptrdiff_t ldA, \
   void *ptrB, ptrdiff_t ldB, void *ptrBeta, void *ptrC, ptrdiff_t ldC, int scalarModeHost, cudaStream_t stream
#define SOLID_GPU_ARGS_GEMM_WITH_PLAN \
   solid_gpu_gemm_plan *plan, void *ptrAlpha, void *ptrA, ptrdiff_t ldA, void *ptrB, ptrdiff_t ldB, \
   void *ptrBeta, void *ptrC, ptrdiff_t ldC, int scalarModeHost, cudaStream_t stream
#define SOLID_GPU_ARGS_COPY \
   int ndims1, const size_t *size1, const ptrdiff_t *strides1, void *ptr1, \
   int ndims2, const size_t *size2, const ptrdiff_t *strides2, void *ptr2, \
   cudaStream_t stream
#define SOLID_GPU_ARGS_BYTESWAP \
   int ndims, const size_t *size, const ptrdiff_t *strides, void *ptr, cudaStream_t stream
#define SOLID_GPU_ARGS_REDUCE_HEAD \
   int ndims, const size_t *size, const ptrdiff_t *strides, void *ptr
#define SOLID_GPU_ARGS_REDUCE_BOOL \
   SOLID_GPU_ARGS_REDUCE_HEAD, solid_bool *result, void *buffer, cudaStream_t stream
#define SOLID_GPU_ARGS_REDUCE_BOUND1 \
   SOLID_GPU_ARGS_REDUCE_HEAD, solid_scalar *bound, solid_bool *result, void *buffer, cudaStream_t stream
#define SOLID_GPU_ARGS_REDUCE_BOUND2 \
   SOLID_GPU_ARGS_REDUCE_HEAD, solid_scalar *lower, solid_scalar *upper, solid_bool *result, \
   void *buffer, cudaStream_t stream
#define SOLID_GPU_ARGS_REDUCE_U64 \
   SOLID_GPU_ARGS_REDUCE_HEAD, solid_uint64 *result, void *buffer, cudaStream_t stream
#define SOLID_GPU_ARGS_REDUCE_VOID \
   SOLID_GPU_ARGS_REDUCE_HEAD, void *result, void *buffer, cudaStream_t stream
#define SOLID_GPU_ARGS_REDUCE_NORM \
   SOLID_GPU_ARGS_REDUCE_HEAD, double p, void *result, void *buffer, cudaStream_t stream
#define SOLID_GPU_ARGS_AXIS       solid_gpu_reduce_axis_config *config
#define SOLID_GPU_ARGS_AXIS_NORM  solid_gpu_reduce_axis_config *config, double p

/* ------------------------------------------------------------------------ */
/* Declarations: typedef, table and per-type functions                      */
/* ------------------------------------------------------------------------ */
#define SOLID_GPU_DECLARE_FN_(NAME, TYPE)  SOLID_API int solid_gpu_##NAME##_##TYPE(SOLID_GPU_ARGS_CURRENT_);
#define SOLID_GPU_DECLARE_(NAME, GROUP) \
   typedef int (*solid_funptr_gpu_##NAME)(SOLID_GPU_ARGS_CURRENT_); \
   SOLID_API solid_funptr_gpu_##NAME solid_gpu_##NAME[SOLID_NUM_TYPES]; \
   SOLID_TYPES_##GROUP(SOLID_GPU_DECLARE_FN_, NAME)

#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_FILL
SOLID_GPU_FILL_OPS(SOLID_GPU_DECLARE_)
#undef SOLID_GPU_ARGS_CURRENT_

/* masked_fill: ptr1[i] = value where the bool tensor ptr2[i] is set -- .src:46-48 */
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_MASKED_FILL
SOLID_GPU_DECLARE_(masked_fill, all)
#undef SOLID_GPU_ARGS_CURRENT_

#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_UNARY
SOLID_GPU_UNARY_OPS(SOLID_GPU_DECLARE_)
#undef SOLID_GPU_ARGS_CURRENT_

#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_UNARY_CHECKED
SOLID_GPU_CHECKED_OPS(SOLID_GPU_DECLARE_)
#undef SOLID_GPU_ARGS_CURRENT_

#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_BINARY
SOLID_GPU_BINARY_OPS(SOLID_GPU_DECLARE_)
#undef SOLID_GPU_ARGS_CURRENT_

/* Ranges: element i (column-major position in the tensor's own dimensions) = offset + i * step, evaluated */
/* in int64, double or complex double and cast to the element type -- solid_core_gpu.src:61-68,            */
/* template_steps.cu:30-122.  steps_cdouble exists for the complex types only, as in the reference.       */
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_STEPS_INT64
SOLID_GPU_DECLARE_(steps_int64, all)
#undef SOLID_GPU_ARGS_CURRENT_
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_STEPS_DOUBLE
SOLID_GPU_DECLARE_(steps_double, all)
#undef SOLID_GPU_ARGS_CURRENT_
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_STEPS_CDOUBLE
SOLID_GPU_DECLARE_(steps_cdouble, complex)
#undef SOLID_GPU_ARGS_CURRENT_

/* Indexed access -- solid_core_gpu.src:72-99, template_index.cu:30-185.  `offsets` is a HOST array of ndims     */
/* pointers; entry d is NULL (dimension d of the indexed tensor ptr1 is addressed by strides1[d]) or points to    */
/* size[d] int64 BYTE offsets in DEVICE memory.  get: ptr2 = ptr1[index]; set: ptr1[index] = ptr2; fill:          */
/* ptr[index] = value.  add_if_negative wraps negative indices (x < 0: x += value) in place; index_to_offset      */
/* turns nelem index tuples (component i at ptr1 + e*stride1 + i*strideReduce) into int64 offsets sum strides[i]*index. */
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_INDEX2
SOLID_GPU_DECLARE_(get_index, all)
SOLID_GPU_DECLARE_(set_index, all)
#undef SOLID_GPU_ARGS_CURRENT_
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_FILL_INDEX
SOLID_GPU_DECLARE_(fill_index, all)
#undef SOLID_GPU_ARGS_CURRENT_
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_ADD_IF_NEGATIVE
SOLID_GPU_DECLARE_(add_if_negative, sint)
#undef SOLID_GPU_ARGS_CURRENT_
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_INDEX_TO_OFFSET
SOLID_GPU_DECLARE_(index_to_offset, integer)
#undef SOLID_GPU_ARGS_CURRENT_

/* Integer and boolean matrix product C = alpha * op(A) * op(B) + beta * C in the wrap-around arithmetic of the     */
/* element type (bool: and / or) -- solid_core_gpu.src:415-440, template_blas.cu:26-259.  Column-major, leading     */
/* dimensions in elements, trans 'N' or 'T'; alpha and beta are read from HOST memory when scalarModeHost is set,   */
/* from DEVICE memory otherwise; a NULL scalar stands for alpha = 1, beta = 0.  The plan has the reference's layout. */
typedef struct
{  char    transA, transB;
   size_t  M, N, K;
   dim3    gridsize;
   dim3    blocksize;
   int     tilesize;
   int     sharedmem;
} solid_gpu_gemm_plan;
SOLID_API int solid_gpu_gemm_create_plan(char transA, char transB, size_t M, size_t N, size_t K,
                                         int elemsize, int device, solid_gpu_gemm_plan *plan);
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_GEMM
SOLID_GPU_DECLARE_(gemm, integer_bool)
#undef SOLID_GPU_ARGS_CURRENT_
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_GEMM_WITH_PLAN
SOLID_GPU_DECLARE_(gemm_with_plan, integer_bool)
#undef SOLID_GPU_ARGS_CURRENT_

/* strides2 == NULL and ptr2 == NULL: in place */
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_SCALAR_OP
SOLID_GPU_SCALAR_OPS(SOLID_GPU_DECLARE_)
#undef SOLID_GPU_ARGS_CURRENT_

#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_REDUCE_BOOL
SOLID_GPU_REDUCE_BOOL_OPS(SOLID_GPU_DECLARE_)
#undef SOLID_GPU_ARGS_CURRENT_
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_REDUCE_BOUND1
SOLID_GPU_REDUCE_BOUND1_OPS(SOLID_GPU_DECLARE_)
#undef SOLID_GPU_ARGS_CURRENT_
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_REDUCE_BOUND2
SOLID_GPU_REDUCE_BOUND2_OPS(SOLID_GPU_DECLARE_)
#undef SOLID_GPU_ARGS_CURRENT_
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_REDUCE_U64
SOLID_GPU_REDUCE_U64_OPS(SOLID_GPU_DECLARE_)
#undef SOLID_GPU_ARGS_CURRENT_
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_REDUCE_VOID
SOLID_GPU_REDUCE_VOID_OPS(SOLID_GPU_DECLARE_)
#undef SOLID_GPU_ARGS_CURRENT_
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_REDUCE_NORM
SOLID_GPU_REDUCE_NORM_OPS(SOLID_GPU_DECLARE_)
#undef SOLID_GPU_ARGS_CURRENT_

#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_AXIS
SOLID_GPU_AXIS_OPS(SOLID_GPU_DECLARE_)
#undef SOLID_GPU_ARGS_CURRENT_
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_AXIS_NORM
SOLID_GPU_AXIS_NORM_OPS(SOLID_GPU_DECLARE_)
#undef SOLID_GPU_ARGS_CURRENT_

/* Type-converting copies: solid_gpu_copy[src][dst](...) -- .src:54-58.  copy accepts     */
/* tensors of different shape and equal element count (elements pair up in column-major   */
/* order of each tensor); copy_regular requires one shared shape.                         */
#define SOLID_GPU_DECLARE_COPY_FN2_(SRC, DST) \
   SOLID_API int solid_gpu_copy_##SRC##_##DST(SOLID_GPU_ARGS_COPY); \
   SOLID_API int solid_gpu_copy_regular_##SRC##_##DST(SOLID_GPU_ARGS_UNARY); \
   SOLID_API int solid_gpu_byteswap_copy_##SRC##_##DST(SOLID_GPU_ARGS_COPY);
#define SOLID_GPU_DECLARE_COPY_FN_(UNUSED, SRC)  SOLID_TYPES2_all(SOLID_GPU_DECLARE_COPY_FN2_, SRC)
typedef int (*solid_funptr_gpu_copy)(SOLID_GPU_ARGS_COPY);
typedef int (*solid_funptr_gpu_copy_regular)(SOLID_GPU_ARGS_UNARY);
SOLID_API solid_funptr_gpu_copy         solid_gpu_copy[SOLID_NUM_TYPES][SOLID_NUM_TYPES];
SOLID_API solid_funptr_gpu_copy_regular solid_gpu_copy_regular[SOLID_NUM_TYPES][SOLID_NUM_TYPES];
SOLID_TYPES_all(SOLID_GPU_DECLARE_COPY_FN_, unused)

/* ------------------------------------------------------------------------ */
/* Byte-order entry points.  The reference has these on the CPU only        */
/* (solid/src/core/cpu/solid_core_cpu.src:49-52 byteswap, byteswap_copy;     */
/* its GPU copy rejects byteswapped tensors, src/core/gpu/op/tensor_copy_gpu.c:102-105). */
/*   byteswap:       reverse the bytes of every real component in place      */
/*   byteswap_copy:  the SOURCE bytes are reversed; swap, then convert       */
/* Source and destination pointers and strides of the copy family need not   */
/* be multiples of the element size.                                         */
/* ------------------------------------------------------------------------ */
typedef int (*solid_funptr_gpu_byteswap)(SOLID_GPU_ARGS_BYTESWAP);
typedef int (*solid_funptr_gpu_byteswap_copy)(SOLID_GPU_ARGS_COPY);
SOLID_API solid_funptr_gpu_byteswap      solid_gpu_byteswap[SOLID_NUM_TYPES];
SOLID_API solid_funptr_gpu_byteswap_copy solid_gpu_byteswap_copy[SOLID_NUM_TYPES][SOLID_NUM_TYPES];
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_BYTESWAP
SOLID_TYPES_all(SOLID_GPU_DECLARE_FN_, byteswap)
#undef SOLID_GPU_ARGS_CURRENT_

/* General form behind all of the above: either side may be byte-reversed.   */
/* flags: bit 0 = source bytes reversed, bit 1 = write destination reversed. */
#define SOLID_GPU_COPY_SRC_SWAPPED 1
#define SOLID_GPU_COPY_DST_SWAPPED 2
SOLID_API int solid_gpu_copy_ex(int srctype, int dsttype, int flags, SOLID_GPU_ARGS_COPY);

/* ------------------------------------------------------------------------ */
/* Library-level functions                                                  */
/* ------------------------------------------------------------------------ */
SOLID_API char *solid_errmsg;                       /* solid/include/solid/base/generic/error.h:26 */
SOLID_API const int solid_gpu_type_size[];          /* solid/src/core/gpu/template_dtype.cu:21-55  */
SOLID_API const int solid_gpu_worktype_size[];
SOLID_API int  solid_gpu_dummy_kernel(void);        /* solid/src/core/gpu/template_dummy.cu:21-37  */

/* solid/include/solid_gpu.h:48-57 */
SOLID_API int  solid_gpu_initialize(void);
SOLID_API void solid_gpu_finalize(void);
SOLID_API int  solid_gpu_check_status(void);
SOLID_API int  solid_gpu_get_current_device(int *device);
SOLID_API int  solid_gpu_multiprocessor_count(int device);
SOLID_API int  solid_gpu_max_threads_per_multiprocessor(int device);
SOLID_API solid_gpu_properties *solid_gpu_get_device_properties(int device);
SOLID_API solid_gpu_properties *solid_gpu_get_current_device_properties(void);

/* Scratch size of a global reduction over nelem elements (solid/src/core/gpu/op/reduce_all.c:111-123) */
SOLID_API int solid_gpu_reduce_all_buffer_size(size_t nelem, int device, size_t *size);

/* Plan an axis reduction (solid/src/core/gpu/op/reduce_axis.c:22-315).  `elemsize` is the  */
/* work-type size of the DESTINATION dtype (solid_gpu_worktype_size[dsttype]).               */
SOLID_API int solid_gpu_reduce_axis_prepare(solid_gpu_reduce_axis_config *config, int elemsize,
                                            int ndims, const size_t *size, const ptrdiff_t *strides1,
                                            void *ptr1, const ptrdiff_t *strides2, void *ptr2,
                                            int rdims, const size_t *rsize, const ptrdiff_t *rstrides,
                                            cudaStream_t stream);

/* ------------------------------------------------------------------------ */
/* Fused entry points (extensions; the reference computes each of these as   */
/* a sequence of separate kernels with temporaries, src/core/interface/      */
/* tensor_itf.c:4221-4251 and src/core/generic/tensor_op.c:170-186, and the  */
/* results here reproduce that sequence rounding for rounding).              */
/* ------------------------------------------------------------------------ */

/* z = a*x + y in the element type, the product rounded to the element type before the add */
/* (Tensor_scale followed by Tensor_add).  Real floating-point types only.                 */
#define SOLID_GPU_ARGS_AXPY \
   int ndims, const size_t *size, const solid_scalar a, const ptrdiff_t *strides1, void *ptr1, \
   const ptrdiff_t *strides2, void *ptr2, const ptrdiff_t *strides3, void *ptr3, cudaStream_t stream
typedef int (*solid_funptr_gpu_axpy)(SOLID_GPU_ARGS_AXPY);
SOLID_API solid_funptr_gpu_axpy solid_gpu_axpy[SOLID_NUM_TYPES];
#define SOLID_GPU_ARGS_CURRENT_ SOLID_GPU_ARGS_AXPY
SOLID_TYPES_real(SOLID_GPU_DECLARE_FN_, axpy)
#undef SOLID_GPU_ARGS_CURRENT_

/* z = a*x + y over n contiguous elements together with sum(z) and sum(z*z) in one pass.    */
/* `partials` (device, solid_gpu_axpy_sums_buffer_size(device, n) bytes: one pair per 16 KB */
/* of x, 8 MiB for 2^32 floats) receives the per-block partial sums; `sums` (device, 2      */
/* elements) receives { sum(z), sum(z*z) } folded in a fixed order by one or two small      */
/* kernels, so that a collective can add the pairs of several GPUs before the square root   */
/* is taken.  Nothing is copied to the host.  float and double.                             */
#define SOLID_GPU_ARGS_AXPY_SUMS \
   size_t n, const solid_scalar a, const void *x, const void *y, void *z, \
   void *sums, void *partials, cudaStream_t stream
SOLID_API int solid_gpu_axpy_sums_buffer_size(int device, size_t n, size_t *size);
SOLID_API int solid_gpu_axpy_sums_float(SOLID_GPU_ARGS_AXPY_SUMS);
SOLID_API int solid_gpu_axpy_sums_double(SOLID_GPU_ARGS_AXPY_SUMS);

/* dst = (dsttype)( (ctype)a * (ctype)b + (ctype)c ) over one shared shape; every operand   */
/* has its own dtype, byte order, strides and alignment and is converted on load with the   */
/* rules of solid_gpu_copy.  `ctype` (SD_FLOAT or SD_DOUBLE) is the common type Ocean would  */
/* have promoted to; product and sum are rounded separately.                                 */
SOLID_API int solid_gpu_mixed_multiply_add(int ndims, const size_t *size,
                                           const solid_gpu_operand *a, const solid_gpu_operand *b,
                                           const solid_gpu_operand *c, const solid_gpu_operand *dst,
                                           int ctype, cudaStream_t stream);

/* Device-resident variants of the global reductions: the value stays in `result` (device,  */
/* 16 bytes) and nothing synchronises.  op is one of the names of SOLID_GPU_REDUCE_VOID_OPS, */
/* SOLID_GPU_REDUCE_BOOL_OPS or SOLID_GPU_REDUCE_U64_OPS.                                    */
SOLID_API int solid_gpu_reduce_all_device(const char *op, int dtype, SOLID_GPU_ARGS_REDUCE_HEAD,
                                          void *result, void *buffer, cudaStream_t stream);

/* ------------------------------------------------------------------------ */
/* Sum of a pair of per-GPU partial results over the GPUs of one node through  */
/* peer memory: the exchange at the end of a sharded reduction (sum, norm2) as  */
/* ONE small kernel instead of a library all-reduce.  No counterpart in the     */
/* reference, which has no collectives (its only cross-device traffic is         */
/* cudaMemcpyPeerAsync, src/core/gpu/storage_gpu.c:140-143).                     */
/*   - every GPU provides a zero-initialised exchange buffer of                  */
/*     solid_gpu_peer_sum_buffer_size(world, &bytes) bytes that the others can  */
/*     address (peer access, CUDA IPC or symmetric memory); buffers[r] is GPU   */
/*     r's buffer as mapped in the calling process, buffers[rank] its own;      */
/*   - sequence is 1, 2, 3, ... and the same on every GPU for the same exchange;*/
/*   - local holds count (1 or 2) floats on this GPU; result receives the sums  */
/*     over all GPUs, added in rank order (the same bits everywhere), with the  */
/*     square root taken of value i when bit i of sqrt_mask is set;             */
/*   - the wait for the peers is bounded: after limit_us microseconds (0: two   */
/*     seconds) the kernel sets *status (device int, may be NULL) to 1 and      */
/*     returns; result is then meaningless and the buffers must be zeroed and   */
/*     the sequence restarted before the next use.                              */
SOLID_API int solid_gpu_peer_sum_buffer_size(int world, size_t *size);
SOLID_API int solid_gpu_peer_sum_float(int world, int rank, void *const *buffers, unsigned int sequence, int count,
                                       const float *local, float *result, int sqrt_mask, unsigned int limit_us,
                                       int *status, cudaStream_t stream);

/* ------------------------------------------------------------------------ */
/* Axis sum of float tensors for callers that may not allocate.  It has no    */
/* counterpart in the reference.  Some callers cannot obtain device memory at  */
/* the point where they reduce: a callback or destructor that runs while an    */
/* allocator lock is held, a latency-critical loop that must not take the      */
/* device-wide synchronisation cudaMalloc/cudaFree imply, a process whose      */
/* memory budget was handed out completely at start-up.  For them this variant */
/* uses a scratch array that is part of the library image instead of           */
/* config->data.ptrBuffer.                                                     */
/*   - config comes from solid_gpu_reduce_axis_prepare as usual; source and    */
/*     destination are the caller's; data.ptrBuffer is ignored and not modified */
/*   - a plan whose bufferSize exceeds solid_gpu_noalloc_scratch_size() bytes   */
/*     (1 MiB per device, held from library load to process exit) is refused    */
/*     with -1 and a message                                                    */
/*   - all calls on a device share the array: calls that overlap in time        */
/*     (different streams or threads) race; issue them on one stream            */
/*   - the first call on each device resolves the array's device address with   */
/*     cudaGetSymbolAddress; make that first call before any stream capture     */
/*   - no cudaMalloc, cudaFree or other allocating call is made                 */
/* ------------------------------------------------------------------------ */
SOLID_API int solid_gpu_noalloc_scratch_size(void);
SOLID_API int solid_gpu_axis_sum_float_noalloc(solid_gpu_reduce_axis_config *config);

#endif
