/*
 * ABI data types of the Solid GPU function tables.
 *
 * Every structure here is laid out exactly as the Ocean tensor library
 * expects it, because the caller (the files of Ocean's src/core/gpu/op) fills or
 * reads the fields directly:
 *   - element types and complex structs   solid/include/solid/base/generic/types.h:30-45
 *   - dtype index order (LUT index)       solid/include/solid/base/generic/dtype.h:23-38
 *   - solid_scalar union                  solid/include/solid/base/generic/scalar.h:27-43
 *   - SOLID_MAX_TENSOR_DIMS               solid/include/solid/base/generic/const.h:20
 *   - solid_gpu_reduce_axis_config        solid/include/solid/core/gpu/reduce_axis.h:38-64
 *   - solid_gpu_properties                solid/include/solid_gpu.h:27-41
 *   - error convention (0 / -1 + text)    solid/include/solid/base/generic/error.h:22-35
 *
 * All strides are in BYTES (ptrdiff_t), sizes are size_t, at most 8 dimensions.
 */
#ifndef SOLID_GPU_TYPES_H
#define SOLID_GPU_TYPES_H

#include <stddef.h>
#include <stdint.h>
#include <cuda_runtime_api.h>

/*
 * Inside an Ocean build the Solid headers of the checkout are on the include
 * path, and Ocean's own files include them before (or after) this one
 * (include/ocean/external/ocean-solid/ocean_solid.h:20-21 pulls in solid.h).
 * A C translation unit may define each of these anonymous struct types only
 * once, so in that case the checkout's definitions are used -- the very
 * headers the reference's generated solid_core_gpu.h includes
 * (solid/src/core/gpu/solid_core_gpu.src:27-31) -- and nothing is defined here.
 * Without them (this library's own build, bindings from other languages) the
 * same types are defined below.  Define SOLID_B200_STANDALONE_TYPES to force
 * the definitions below even when Solid headers can be found.
 */
#if !defined(SOLID_B200_STANDALONE_TYPES) && defined(__has_include)
#  if __has_include("solid_gpu.h") && __has_include("solid/base/gpu/types_gpu.h") && \
      __has_include("solid/core/gpu/reduce_axis.h")
#    define SOLID_B200_USING_OCEAN_SOLID_HEADERS 1
#  endif
#endif

#ifdef SOLID_B200_USING_OCEAN_SOLID_HEADERS

#include "solid_gpu.h"                      /* solid.h: element types, solid_scalar, SD_* ; solid_gpu_properties */
#include "solid/base/gpu/types_gpu.h"       /* solid_gpu_config                                                  */
#include "solid/core/gpu/reduce_all.h"
#include "solid/core/gpu/reduce_axis.h"     /* solid_gpu_reduce_axis_data, solid_gpu_reduce_axis_config          */
#define SOLID_NUM_TYPES 15

#else  /* stand-alone definitions */

#ifdef __cplusplus
#define SOLID_API extern "C"
#else
#define SOLID_API extern
#endif

#define SOLID_MAX_TENSOR_DIMS 8
#define SOLID_ERRMSG_SIZE     512

typedef size_t    solid_size;
typedef ptrdiff_t solid_index;
typedef uint8_t   solid_bool;
typedef uint8_t   solid_uint8;
typedef uint16_t  solid_uint16;
typedef uint32_t  solid_uint32;
typedef uint64_t  solid_uint64;
typedef int8_t    solid_int8;
typedef int16_t   solid_int16;
typedef int32_t   solid_int32;
typedef int64_t   solid_int64;
typedef uint16_t  solid_half;      /* raw IEEE binary16 bits */
typedef float     solid_float;
typedef double    solid_double;
typedef struct { solid_half   real; solid_half   imag; } solid_chalf;
typedef struct { solid_float  real; solid_float  imag; } solid_cfloat;
typedef struct { solid_double real; solid_double imag; } solid_cdouble;

/* Index of each element type in every function table */
typedef enum {
   SD_BOOL = 0, SD_UINT8 = 1, SD_UINT16 = 2, SD_UINT32 = 3, SD_UINT64 = 4,
   SD_INT8 = 5, SD_INT16 = 6, SD_INT32 = 7, SD_INT64 = 8,
   SD_HALF = 9, SD_FLOAT = 10, SD_DOUBLE = 11,
   SD_CHALF = 12, SD_CFLOAT = 13, SD_CDOUBLE = 14
} solid_type_index;
#define SOLID_NUM_TYPES 15

typedef union {
   solid_bool    _bool;
   solid_uint8   _uint8;
   solid_uint16  _uint16;
   solid_uint32  _uint32;
   solid_uint64  _uint64;
   solid_int8    _int8;
   solid_int16   _int16;
   solid_int32   _int32;
   solid_int64   _int64;
   solid_half    _half;
   solid_float   _float;
   solid_double  _double;
   solid_chalf   _chalf;
   solid_cfloat  _cfloat;
   solid_cdouble _cdouble;
} solid_scalar;

/* Launch shape handed back to callers that inspect it */
typedef struct {
   dim3 blocks;
   dim3 threads;
} solid_gpu_config;

/* Axis reduction: tensor description followed by the launch plan.  The     */
/* caller runs solid_gpu_reduce_axis_prepare, allocates bufferSize bytes of  */
/* device scratch when that is non-zero, stores it in data.ptrBuffer and     */
/* only then calls solid_gpu_axis_<op>_<type>(config).                       */
typedef struct {
   size_t     size[SOLID_MAX_TENSOR_DIMS];       /* kept (outer) dimensions            */
   size_t     rsize[SOLID_MAX_TENSOR_DIMS];      /* reduced dimensions                 */
   ptrdiff_t  strides1[SOLID_MAX_TENSOR_DIMS];   /* source strides of the outer dims   */
   ptrdiff_t  strides2[SOLID_MAX_TENSOR_DIMS];   /* destination strides                */
   ptrdiff_t  rstrides[SOLID_MAX_TENSOR_DIMS];   /* source strides of the reduced dims */
   char      *ptr1;                              /* source                             */
   char      *ptr2;                              /* destination                        */
   char      *ptrBuffer;                         /* device scratch (bufferSize bytes)  */
   size_t     nelem;                             /* number of outputs                  */
   size_t     relem;                             /* elements reduced per output        */
   int        ndims;
   int        rdims;
} solid_gpu_reduce_axis_data;

typedef struct {
   solid_gpu_reduce_axis_data data;
   int          mode;
   dim3         gridSize;
   dim3         blockSize;
   dim3         gridSizeFinalize;
   dim3         blockSizeFinalize;
   size_t       bufferSize;
   size_t       sharedMem;
   size_t       sharedMemFinalize;
   cudaStream_t stream;
} solid_gpu_reduce_axis_config;

typedef struct {
   int major;
   int minor;
   int multiprocessor_count;
   int max_threads_per_block;
   int max_threads_per_multiprocessor;
   int max_blocks_per_multiprocessor;
   int max_warps_per_multiprocessor;
   int max_resident_blocks_per_device;
   int max_shared_mem_per_multiprocessor;
   int max_shared_mem_per_threadblock;
   int max_gridsize[3];
   int max_blocksize[3];
} solid_gpu_properties;

#endif /* stand-alone definitions */

/* One operand of the mixed-dtype fused entry points (an extension; the      */
/* reference has no counterpart because it converts every operand to a       */
/* common dtype through temporaries first).  `strides` has one byte stride   */
/* per dimension of the shared `size` vector; 0 broadcasts.  `byteswapped`   */
/* says the stored bytes of each real component are reversed.  `ptr` need    */
/* not be aligned to the element size.                                       */
typedef struct {
   void            *ptr;
   const ptrdiff_t *strides;
   int              dtype;        /* solid_type_index */
   int              byteswapped;  /* 0 or 1 */
} solid_gpu_operand;

#endif
