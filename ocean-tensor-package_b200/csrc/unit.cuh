// Shared prologue of the per-type translation units.  Each unit is compiled once
// per element type with -DSDX=<type name> -DSDX_KIND=<0 bool,1 uint,2 sint,3 real,4 complex>
// and defines the solid_gpu_<op>_<type> entry points of that type.
#pragma once
#include "solid_core_gpu.h"
#include "dtypes.cuh"

#ifndef SDX
#error "compile with -DSDX=<type> -DSDX_KIND=<kind>"
#endif

#define SD_PASTE_(A, B) A##B
#define SD_PASTE(A, B)  SD_PASTE_(A, B)
#define SD_T(NAME)      sd::SD_PASTE(t_, NAME)

// membership of SDX in each type group, as literal 0/1 tokens
#define SD_IN_all 1
#if SDX_KIND == 0
#define SD_IN_bool 1
#define SD_IN_all_nobool 0
#define SD_IN_integer_bool 1
#define SD_IN_float 0
#define SD_IN_complex 0
#define SD_IN_real 0
#define SD_IN_all_nouint 1
#define SD_IN_all_nocomplex 1
#elif SDX_KIND == 1
#define SD_IN_bool 0
#define SD_IN_all_nobool 1
#define SD_IN_integer_bool 1
#define SD_IN_float 0
#define SD_IN_complex 0
#define SD_IN_real 0
#define SD_IN_all_nouint 0
#define SD_IN_all_nocomplex 1
#elif SDX_KIND == 2
#define SD_IN_bool 0
#define SD_IN_all_nobool 1
#define SD_IN_integer_bool 1
#define SD_IN_float 0
#define SD_IN_complex 0
#define SD_IN_real 0
#define SD_IN_all_nouint 1
#define SD_IN_all_nocomplex 1
#elif SDX_KIND == 3
#define SD_IN_bool 0
#define SD_IN_all_nobool 1
#define SD_IN_integer_bool 0
#define SD_IN_float 1
#define SD_IN_complex 0
#define SD_IN_real 1
#define SD_IN_all_nouint 1
#define SD_IN_all_nocomplex 1
#else
#define SD_IN_bool 0
#define SD_IN_all_nobool 1
#define SD_IN_integer_bool 0
#define SD_IN_float 1
#define SD_IN_complex 1
#define SD_IN_real 0
#define SD_IN_all_nouint 1
#define SD_IN_all_nocomplex 0
#endif

// SD_WHEN(group)(text) expands to text when SDX belongs to the group
#define SD_WHEN_1(...) __VA_ARGS__
#define SD_WHEN_0(...)
#define SD_WHEN__(FLAG) SD_WHEN_##FLAG
#define SD_WHEN_(FLAG)  SD_WHEN__(FLAG)
#define SD_WHEN(GROUP)  SD_WHEN_(SD_IN_##GROUP)

using T = SD_T(SDX);
