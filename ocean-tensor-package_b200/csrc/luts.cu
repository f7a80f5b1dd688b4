// Function tables: solid_gpu_<op>[15] and solid_gpu_copy[15][15] etc., indexed by
// solid_type_index, NULL where a type is not supported.  The reference generates
// the same tables from its .src file (solid/bin/generate.py:396-432).
#include "solid_core_gpu.h"
#include "layout.h"

#define Z 0
#define SD_LUT_all(P)           { P##bool, P##uint8, P##uint16, P##uint32, P##uint64, P##int8, P##int16, P##int32, P##int64, P##half, P##float, P##double, P##chalf, P##cfloat, P##cdouble }
#define SD_LUT_all_nobool(P)    { Z,       P##uint8, P##uint16, P##uint32, P##uint64, P##int8, P##int16, P##int32, P##int64, P##half, P##float, P##double, P##chalf, P##cfloat, P##cdouble }
#define SD_LUT_all_nouint(P)    { P##bool, Z, Z, Z, Z,                                P##int8, P##int16, P##int32, P##int64, P##half, P##float, P##double, P##chalf, P##cfloat, P##cdouble }
#define SD_LUT_all_nocomplex(P) { P##bool, P##uint8, P##uint16, P##uint32, P##uint64, P##int8, P##int16, P##int32, P##int64, P##half, P##float, P##double, Z, Z, Z }
#define SD_LUT_integer_bool(P)  { P##bool, P##uint8, P##uint16, P##uint32, P##uint64, P##int8, P##int16, P##int32, P##int64, Z, Z, Z, Z, Z, Z }
#define SD_LUT_sint(P)          { Z, Z, Z, Z, Z, P##int8, P##int16, P##int32, P##int64, Z, Z, Z, Z, Z, Z }
#define SD_LUT_integer(P)       { Z, P##uint8, P##uint16, P##uint32, P##uint64, P##int8, P##int16, P##int32, P##int64, Z, Z, Z, Z, Z, Z }
#define SD_LUT_bool(P)          { P##bool, Z, Z, Z, Z, Z, Z, Z, Z, Z, Z, Z, Z, Z, Z }
#define SD_LUT_float(P)         { Z, Z, Z, Z, Z, Z, Z, Z, Z, P##half, P##float, P##double, P##chalf, P##cfloat, P##cdouble }
#define SD_LUT_real(P)          { Z, Z, Z, Z, Z, Z, Z, Z, Z, P##half, P##float, P##double, Z, Z, Z }
#define SD_LUT_complex(P)       { Z, Z, Z, Z, Z, Z, Z, Z, Z, Z, Z, Z, P##chalf, P##cfloat, P##cdouble }

#define SD_DEFINE_LUT(NAME, GROUP) \
   extern "C" solid_funptr_gpu_##NAME solid_gpu_##NAME[SOLID_NUM_TYPES] = SD_LUT_##GROUP(solid_gpu_##NAME##_);

SOLID_GPU_FILL_OPS(SD_DEFINE_LUT)
SD_DEFINE_LUT(masked_fill, all)
SOLID_GPU_UNARY_OPS(SD_DEFINE_LUT)
SOLID_GPU_CHECKED_OPS(SD_DEFINE_LUT)
SOLID_GPU_BINARY_OPS(SD_DEFINE_LUT)
SOLID_GPU_SCALAR_OPS(SD_DEFINE_LUT)
SD_DEFINE_LUT(steps_int64, all)
SD_DEFINE_LUT(steps_double, all)
SD_DEFINE_LUT(steps_cdouble, complex)
SD_DEFINE_LUT(gemm, integer_bool)
SD_DEFINE_LUT(gemm_with_plan, integer_bool)
SD_DEFINE_LUT(get_index, all)
SD_DEFINE_LUT(set_index, all)
SD_DEFINE_LUT(fill_index, all)
SD_DEFINE_LUT(add_if_negative, sint)
SD_DEFINE_LUT(index_to_offset, integer)
SOLID_GPU_REDUCE_BOOL_OPS(SD_DEFINE_LUT)
SOLID_GPU_REDUCE_BOUND1_OPS(SD_DEFINE_LUT)
SOLID_GPU_REDUCE_BOUND2_OPS(SD_DEFINE_LUT)
SOLID_GPU_REDUCE_U64_OPS(SD_DEFINE_LUT)
SOLID_GPU_REDUCE_VOID_OPS(SD_DEFINE_LUT)
SOLID_GPU_REDUCE_NORM_OPS(SD_DEFINE_LUT)
SOLID_GPU_AXIS_OPS(SD_DEFINE_LUT)
SOLID_GPU_AXIS_NORM_OPS(SD_DEFINE_LUT)
SD_DEFINE_LUT(byteswap, all)
SD_DEFINE_LUT(axpy, real)

#define SD_ROW_(P, SRC) SD_LUT_all(P##SRC##_),
#define SD_ROW_COPY(U, SRC)     SD_ROW_(solid_gpu_copy_, SRC)
#define SD_ROW_REGULAR(U, SRC)  SD_ROW_(solid_gpu_copy_regular_, SRC)
#define SD_ROW_BSCOPY(U, SRC)   SD_ROW_(solid_gpu_byteswap_copy_, SRC)
extern "C" solid_funptr_gpu_copy solid_gpu_copy[SOLID_NUM_TYPES][SOLID_NUM_TYPES] = { SOLID_TYPES2_all(SD_ROW_COPY, u) };
extern "C" solid_funptr_gpu_copy_regular solid_gpu_copy_regular[SOLID_NUM_TYPES][SOLID_NUM_TYPES] = { SOLID_TYPES2_all(SD_ROW_REGULAR, u) };
extern "C" solid_funptr_gpu_byteswap_copy solid_gpu_byteswap_copy[SOLID_NUM_TYPES][SOLID_NUM_TYPES] = { SOLID_TYPES2_all(SD_ROW_BSCOPY, u) };

// solid_gpu_copy_ex: any source type, any destination type, either byte order
typedef int (*copy_ex_row)(int dsttype, int flags, SOLID_GPU_ARGS_COPY);
#define SD_DECL_EX(U, SRC) extern "C" int solid_gpu_copy_ex_from_##SRC(int dsttype, int flags, SOLID_GPU_ARGS_COPY);
SOLID_TYPES2_all(SD_DECL_EX, u)
#define SD_EX_ENTRY(U, SRC) solid_gpu_copy_ex_from_##SRC,
static const copy_ex_row copy_ex_rows[SOLID_NUM_TYPES] = { SOLID_TYPES2_all(SD_EX_ENTRY, u) };

extern "C" int solid_gpu_copy_ex(int srctype, int dsttype, int flags, SOLID_GPU_ARGS_COPY)
{
   if (srctype < 0 || srctype >= SOLID_NUM_TYPES) SD_ERROR("Invalid source type index %d", srctype);
   return copy_ex_rows[srctype](dsttype, flags, ndims1, size1, strides1, ptr1, ndims2, size2, strides2, ptr2, stream);
}
