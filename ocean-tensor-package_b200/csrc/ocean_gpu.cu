// Ocean-level GPU dispatch (declared in include/ocean_gpu_b200.h): table lookup by dtype,
// device activation, stream ordering, scratch from a per-device cache, host results -- what
// src/core/gpu/op/tensor_{unary,binary,copy,fill,reduce_all,reduce_axis}_gpu.c do in the
// reference.  Layout simplification (OcSolid_analyze*, src/external/ocean-solid/ocean_solid.c)
// is done inside the Solid entry points here, so the views are passed through as they are.
#include <cstdio>
#include <cstdarg>
#include <cstring>
#include <cstdlib>
#include <mutex>
#include <utility>
#include "ocean_gpu_b200.h"

namespace {

thread_local char g_error[SOLID_ERRMSG_SIZE] = "";

int fail(const char *fmt, ...)
{
   va_list ap; va_start(ap, fmt);
   vsnprintf(g_error, sizeof(g_error), fmt, ap);
   va_end(ap);
   return -1;
}
int fail_solid() { snprintf(g_error, sizeof(g_error), "%s", solid_errmsg); return -1; }     // OC_SOLID_ERRMSG
int fail_cuda(cudaError_t st, const char *what) { return fail("%s: %s", what, cudaGetErrorString(st)); }

const char *const dtype_names[SOLID_NUM_TYPES] = {
   "bool", "uint8", "uint16", "uint32", "uint64", "int8", "int16", "int32", "int64",
   "half", "float", "double", "complex-half", "complex-float", "complex-double" };

bool valid_dtype(int t) { return t >= 0 && t < SOLID_NUM_TYPES; }

// OC_SOLID_FUNPTR (src/external/ocean-solid/ocean_solid.h:131-140): NULL entry -> typed error
template <class F> F lookup(F const *table, int dtype, const char *desc)
{
   if (!valid_dtype(dtype)) { fail("Invalid data type index %d", dtype); return nullptr; }
   F f = table[dtype];
   if (f == nullptr) fail("The %s function is not available for type %s on GPU", desc, dtype_names[dtype]);
   return f;
}

int set_device(int device)                                             // OcCuda_setDevice
{
   cudaError_t st = cudaSetDevice(device);
   return st == cudaSuccess ? 0 : fail_cuda(st, "Error activating the GPU device");
}

// Stream protocol of src/base/storage.c:141-222 on the facts a view carries.
int start_read(const OcTensorView *dst, const OcTensorView *src)
{
   if (src->stream == dst->stream || src->event == nullptr) return 0;
   cudaError_t st = cudaStreamWaitEvent(dst->stream, src->event, 0);
   return st == cudaSuccess ? 0 : fail_cuda(st, "Error synchronizing streams");
}
int update(const OcTensorView *dst)
{
   if (dst->event == nullptr) return 0;
   cudaError_t st = cudaEventRecord(dst->event, dst->stream);
   return st == cudaSuccess ? 0 : fail_cuda(st, "Error recording the tensor event");
}
int finish_read(const OcTensorView *dst, const OcTensorView *src)
{
   // the source must not be overwritten before this read has completed: its stream waits for the
   // destination's event, and its own event is recorded again behind that wait, so that a third stream
   // about to write the source (which waits on the source's event) is held back as well
   // (OcStorage_finishRead, src/base/storage.c:176-190)
   if (src->stream == dst->stream || dst->event == nullptr) return 0;
   cudaError_t st = cudaStreamWaitEvent(src->stream, dst->event, 0);
   if (st == cudaSuccess && src->event != nullptr && src->device == dst->device) st = cudaEventRecord(src->event, src->stream);
   return st == cudaSuccess ? 0 : fail_cuda(st, "Error synchronizing streams");
}

bool same_shape(const OcTensorView *a, const OcTensorView *b)
{
   if (a->ndims != b->ndims) return false;
   for (int i = 0; i < a->ndims; i++) if (a->size[i] != b->size[i]) return false;
   return true;
}
int check_view(const OcTensorView *t, const char *what)
{
   if (t == nullptr) return fail("Missing %s tensor", what);
   if (t->ndims < 0 || t->ndims > SOLID_MAX_TENSOR_DIMS) return fail("Invalid number of dimensions (%d)", t->ndims);
   if (!valid_dtype(t->dtype)) return fail("Invalid data type index %d", t->dtype);
   return 0;
}
// Preconditions the interface layer guarantees for elementwise kernels (tensor_op.c:346-409)
int check_elemwise(const OcTensorView *t, const char *what)
{
   if (check_view(t, what) != 0) return -1;
   if (t->byteswapped) return fail("The %s tensor must be in native byte order", what);
   return 0;
}

// ---- scratch: three round-robin slots per device (src/core/interface/storage_itf.c:61-121) ----
// A slot is handed out again after two other requests, possibly while the kernels of its previous user are still
// queued on some other stream.  Each slot therefore carries an event: the user records it on its stream behind its
// last launch that touches the slot (scratch_done), and the next user's stream waits for it before it may write
// the slot (Ocean's temporaries get the same ordering from the event of their OcStorage, src/base/storage.c:193-222).
struct Slot { void *ptr; size_t size; cudaEvent_t done; bool recorded; };
struct DeviceCache { Slot slot[3]; int next; };
DeviceCache g_cache[64];
std::mutex g_cache_lock;

// `device` must be current.  The returned slot index goes to scratch_done.
int temporary(int device, size_t bytes, cudaStream_t stream, void **out, int *slot_index)
{
   if (device < 0 || device >= 64) return fail("Invalid device index %d", device);
   std::lock_guard<std::mutex> guard(g_cache_lock);
   DeviceCache &c = g_cache[device];
   const int k = c.next;
   Slot &s = c.slot[k];
   c.next = (c.next + 1) % 3;
   if (s.done == nullptr) {
      cudaError_t st = cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming);
      if (st != cudaSuccess) { s.done = nullptr; return fail_cuda(st, "Error creating an event"); }
   }
   if (s.size < bytes) {
      // replace the buffer once its last user has finished with it
      if (s.ptr) {
         if (s.recorded) cudaEventSynchronize(s.done);
         cudaFree(s.ptr); s.ptr = nullptr; s.size = 0; s.recorded = false;
      }
      size_t want = bytes < (1u << 16) ? (1u << 16) : bytes;
      cudaError_t st = cudaMalloc(&s.ptr, want);
      if (st != cudaSuccess) { s.ptr = nullptr; return fail_cuda(st, "Error allocating a temporary buffer"); }
      s.size = want;
   }
   if (s.recorded) {
      cudaError_t st = cudaStreamWaitEvent(stream, s.done, 0);
      if (st != cudaSuccess) return fail_cuda(st, "Error synchronizing streams");
   }
   *out = s.ptr;
   *slot_index = k;
   return 0;
}

// Everything queued on `stream` (a stream of `device`, which must be current) so far is the slot's last use.
int scratch_done(int device, int slot_index, cudaStream_t stream)
{
   std::lock_guard<std::mutex> guard(g_cache_lock);
   Slot &s = g_cache[device].slot[slot_index];
   cudaError_t st = cudaEventRecord(s.done, stream);
   if (st != cudaSuccess) return fail_cuda(st, "Error recording an event");
   s.recorded = true;
   return 0;
}

// result dtypes of reductions (solid/include/solid/core/generic/reduce_ops.h:607-617,798-837,1004-1255)
bool is_intlike(int t) { return t <= SD_INT64; }
bool is_complex(int t) { return t >= SD_CHALF; }
int elem_type(int t) { return is_complex(t) ? t - 3 : t; }
int abs_type(int t) { return (t >= SD_INT8 && t <= SD_INT64) ? t - 4 : elem_type(t); }
int sum_type(int t) { return t <= SD_UINT64 ? SD_UINT64 : (t <= SD_INT64 ? SD_INT64 : t); }


// Operand and result types of the elementwise tables.  The Solid function is chosen by the FIRST operand's type and
// reads and writes the others as the types listed here, so anything else would run past the end of a buffer:
//   unary    is* -> bool, absolute -> real type of a complex source, everything else the source type
//            (solid/src/core/gpu/template_unary.cu:176-246)
//   binary   comparisons -> bool; shifts take an int8 count and may write the other signedness of the same width
//            (src/core/interface/tensor_itf.c:4660-4727); power on a bool / integer base takes an int16 exponent
//            (solid/src/core/gpu/template_binary.cu:201,260-264); everything else one type throughout
int unary_result_type(const char *solid, int t)
{
   if (!strncmp(solid, "is", 2)) return SD_BOOL;
   if (!strcmp(solid, "absolute")) return elem_type(t);
   return t;
}
int check_unary_types(const char *op, const char *solid, const OcTensorView *src, const OcTensorView *dst)
{
   const int want = unary_result_type(solid, src->dtype);
   if (dst->dtype != want)
      return fail("The destination of %s on type %s must have type %s, not %s", op, dtype_names[src->dtype], dtype_names[want], dtype_names[dst->dtype]);
   if (src->device != dst->device) return fail("All tensors of %s must be on the device of the destination", op);
   return 0;
}
int check_binary_types(const char *op, const char *solid, const OcTensorView *a, const OcTensorView *b, const OcTensorView *dst)
{
   int want_b = a->dtype, want_dst = a->dtype;
   bool dst_width_only = false;
   if (!strcmp(solid, "lt") || !strcmp(solid, "le") || !strcmp(solid, "eq") || !strcmp(solid, "ne") || !strcmp(solid, "ge") || !strcmp(solid, "gt"))
      want_dst = SD_BOOL;
   else if (!strncmp(solid, "bitshift", 8)) { want_b = SD_INT8; dst_width_only = true; }
   else if (!strcmp(solid, "power") && is_intlike(a->dtype)) want_b = SD_INT16;
   if (b->dtype != want_b)
      return fail("The second operand of %s on type %s must have type %s, not %s", op, dtype_names[a->dtype], dtype_names[want_b], dtype_names[b->dtype]);
   const bool dst_ok = dst_width_only ? (is_intlike(dst->dtype) && solid_gpu_type_size[dst->dtype] == solid_gpu_type_size[a->dtype])
                                      : dst->dtype == want_dst;
   if (!dst_ok)
      return fail("The destination of %s on type %s must have type %s, not %s", op, dtype_names[a->dtype], dtype_names[want_dst], dtype_names[dst->dtype]);
   if (a->device != dst->device || b->device != dst->device) return fail("All tensors of %s must be on the device of the destination", op);
   return 0;
}

} // namespace

extern "C" int OcGPU_reductionResultType(const char *name, int t)
{
   if (!valid_dtype(t) || name == nullptr) return -1;
   if (strncmp(name, "axis_", 5) == 0) name += 5;
   if (!strncmp(name, "any", 3) || !strncmp(name, "all", 3)) return SD_BOOL;
   if (!strncmp(name, "nnz", 3)) return SD_UINT64;
   if (!strcmp(name, "sum") || !strcmp(name, "sum_nan") || !strcmp(name, "prod") || !strcmp(name, "prod_nan")) return sum_type(t);
   if (!strcmp(name, "sum_abs") || !strcmp(name, "sum_abs_nan")) return is_intlike(t) ? SD_UINT64 : abs_type(t);
   if (!strcmp(name, "maximum") || !strcmp(name, "minimum")) return t;
   if (!strcmp(name, "maximum_abs") || !strcmp(name, "minimum_abs")) return abs_type(t);
   if (!strncmp(name, "norm", 4)) return is_intlike(t) ? SD_DOUBLE : abs_type(t);
   return -1;
}

extern "C" const char *OcGPU_errorMessage(void) { return g_error; }

extern "C" int OcInitGPU_B200(void)
{
   if (solid_gpu_initialize() != 0) return fail_solid();
   int n = 0;
   if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); n = 0; }
   int current = 0; cudaGetDevice(&current);
   for (int d = 0; d < n; d++) {                        // warm-up as OcInitDevicesGPU does (device_gpu.c:155-196)
      if (set_device(d) != 0) return -1;
      if (solid_gpu_dummy_kernel() != 0) return fail_solid();
   }
   if (n) cudaSetDevice(current);
   return 0;
}

extern "C" void OcFinalizeGPU_B200(void)
{
   std::lock_guard<std::mutex> guard(g_cache_lock);
   int current = 0; cudaGetDevice(&current);
   for (int d = 0; d < 64; d++) for (Slot &s : g_cache[d].slot) if (s.ptr || s.done) {
      cudaSetDevice(d);
      if (s.recorded) cudaEventSynchronize(s.done);
      if (s.ptr) cudaFree(s.ptr);
      if (s.done) cudaEventDestroy(s.done);
      s.ptr = nullptr; s.size = 0; s.done = nullptr; s.recorded = false; }
   cudaSetDevice(current);
   solid_gpu_finalize();
}

// ---------------------------------------------------------------------------------- unary
#define OCGPU_DEFINE_UNARY(OP, SOLID)                                                              \
extern "C" int OcTensorGPU_##OP(const OcTensorView *src, const OcTensorView *dst)                  \
{                                                                                                  \
   if (check_elemwise(src, "source") != 0 || check_elemwise(dst, "destination") != 0) return -1;   \
   if (!same_shape(src, dst)) return fail("Tensor size mismatch in " #OP);                         \
   solid_funptr_gpu_##SOLID f = lookup(solid_gpu_##SOLID, src->dtype, #OP);                        \
   if (f == nullptr) return -1;                                                                    \
   if (check_unary_types(#OP, #SOLID, src, dst) != 0) return -1;                                   \
   if (set_device(dst->device) != 0) return -1;                                                    \
   if (start_read(dst, src) != 0) return -1;                                                       \
   if (f(src->ndims, src->size, src->strides, src->data, dst->strides, dst->data, dst->stream) != 0) return fail_solid(); \
   if (update(dst) != 0) return -1;                                                                \
   return finish_read(dst, src);                                                                   \
}
OCGPU_UNARY_OPS(OCGPU_DEFINE_UNARY)

// ---------------------------------------------------------------------------------- binary
#define OCGPU_DEFINE_BINARY(OP, SOLID)                                                             \
extern "C" int OcTensorGPU_##OP(const OcTensorView *src1, const OcTensorView *src2, const OcTensorView *dst) \
{                                                                                                  \
   if (check_elemwise(src1, "first source") != 0 || check_elemwise(src2, "second source") != 0 ||  \
       check_elemwise(dst, "destination") != 0) return -1;                                         \
   if (!same_shape(src1, dst) || !same_shape(src2, dst)) return fail("Tensor size mismatch in " #OP); \
   solid_funptr_gpu_##SOLID f = lookup(solid_gpu_##SOLID, src1->dtype, #OP);                       \
   if (f == nullptr) return -1;                                                                    \
   if (check_binary_types(#OP, #SOLID, src1, src2, dst) != 0) return -1;                           \
   if (set_device(dst->device) != 0) return -1;                                                    \
   if (start_read(dst, src1) != 0 || start_read(dst, src2) != 0) return -1;                        \
   if (f(dst->ndims, dst->size, src1->strides, src1->data, src2->strides, src2->data,              \
         dst->strides, dst->data, dst->stream) != 0) return fail_solid();                          \
   if (update(dst) != 0) return -1;                                                                \
   if (finish_read(dst, src2) != 0) return -1;                                                     \
   return finish_read(dst, src1);                                                                  \
}
OCGPU_BINARY_OPS(OCGPU_DEFINE_BINARY)

// ---------------------------------------------------------------------------------- tensor (op) scalar
#define OCGPU_DEFINE_SCALAR(OP, SOLID)                                                             \
extern "C" int OcTensorGPU_##OP(const OcTensorView *src, const OcScalarView *scalar, const OcTensorView *dst) \
{                                                                                                  \
   if (check_elemwise(src, "source") != 0 || check_elemwise(dst, "destination") != 0) return -1;   \
   if (scalar == nullptr) return fail("Missing scalar in " #OP);                                   \
   if (!same_shape(src, dst)) return fail("Tensor size mismatch in " #OP);                         \
   if (scalar->dtype != src->dtype || dst->dtype != src->dtype) return fail("Data type mismatch in " #OP); \
   solid_funptr_gpu_##SOLID f = lookup(solid_gpu_##SOLID, src->dtype, #OP);                        \
   if (f == nullptr) return -1;                                                                    \
   if (set_device(dst->device) != 0) return -1;                                                    \
   if (start_read(dst, src) != 0) return -1;                                                       \
   if (f(dst->ndims, dst->size, src->strides, src->data, scalar->value,                            \
         dst->strides, dst->data, dst->stream) != 0) return fail_solid();                          \
   if (update(dst) != 0) return -1;                                                                \
   return finish_read(dst, src);                                                                   \
}
OCGPU_SCALAR_OPS(OCGPU_DEFINE_SCALAR)

// ---------------------------------------------------------------------------------- ranges
// The memory layout of one tensor (OcSolid_analyzeElemwise1, src/external/ocean-solid/ocean_solid.c:85-130):
// no unit or repeated dimensions, positive strides in increasing order, contiguous neighbours merged.
struct Analyzed { int ndims; size_t size[8]; ptrdiff_t strides[8]; char *ptr; };
static void analyze1(const OcTensorView *t, Analyzed *a)
{
   a->ptr = (char *)t->data; a->ndims = 0;
   size_t nelem = 1;
   for (int i = 0; i < t->ndims; i++) nelem *= t->size[i];
   if (nelem == 0) { a->ndims = 1; a->size[0] = 0; a->strides[0] = 0; return; }
   int n = 0;
   for (int i = 0; i < t->ndims; i++) {
      ptrdiff_t r = t->strides[i]; const size_t sz = t->size[i];
      if (sz == 1 || r == 0) continue;
      if (r < 0) { a->ptr += r * (ptrdiff_t)(sz - 1); r = -r; }
      a->size[n] = sz; a->strides[n] = r; n++;
   }
   for (int i = 1; i < n; i++)                                          // insertion sort by stride
      for (int j = i; j > 0 && a->strides[j] < a->strides[j - 1]; j--) {
         std::swap(a->strides[j], a->strides[j - 1]); std::swap(a->size[j], a->size[j - 1]); }
   int m = 0;
   for (int i = 0; i < n; i++) {
      if (m > 0 && a->strides[i] == a->strides[m - 1] * (ptrdiff_t)a->size[m - 1]) a->size[m - 1] *= a->size[i];
      else { a->size[m] = a->size[i]; a->strides[m] = a->strides[i]; m++; }
   }
   a->ndims = m;
}
#define OCGPU_DEFINE_STEPS(OP, SOLID, PTYPE)                                                       \
extern "C" int OcTensorGPU_##OP(const OcTensorView *tensor, PTYPE offset, PTYPE step)              \
{                                                                                                  \
   if (check_elemwise(tensor, "destination") != 0) return -1;                                      \
   solid_funptr_gpu_##SOLID f = lookup(solid_gpu_##SOLID, tensor->dtype, #OP);                     \
   if (f == nullptr) return -1;                                                                    \
   if (set_device(tensor->device) != 0) return -1;                                                 \
   Analyzed a; analyze1(tensor, &a);                                                               \
   if (f(a.ndims, a.size, a.strides, a.ptr, offset, step, tensor->stream) != 0) return fail_solid(); \
   return update(tensor);                                                                          \
}
OCGPU_DEFINE_STEPS(stepsInt64, steps_int64, solid_int64)
OCGPU_DEFINE_STEPS(stepsDouble, steps_double, solid_double)
OCGPU_DEFINE_STEPS(stepsCDouble, steps_cdouble, solid_cdouble)

// ---------------------------------------------------------------------------------- indexed access
static int index_prepare(const OcIndexView *ix, const OcTensorView *other, const char *what, solid_int64 **tables)
{
   if (ix == nullptr) return fail("Missing index view in %s", what);
   if (check_elemwise(&ix->view, "indexed") != 0) return -1;
   if (ix->ndims < 0 || ix->ndims > 8) return fail("Invalid number of index dimensions in %s", what);
   if (ix->ndims != ix->view.ndims) return fail("The index must cover every dimension of the tensor in %s", what);
   for (int d = 0; d < ix->ndims; d++) {
      const OcTensorView *t = ix->offsets[d];
      tables[d] = nullptr;
      if (t == nullptr) continue;
      if (check_view(t, "offset") != 0) return -1;
      if (t->dtype != SD_INT64 || t->ndims != 1 || t->size[0] != ix->size[d] || (t->size[0] > 1 && t->strides[0] != 8) || t->byteswapped)
         return fail("Offset tables must be contiguous native int64 vectors with one entry per selected position");
      if (t->device != ix->view.device) return fail("Offset tables must be on the device of the indexed tensor");
      tables[d] = (solid_int64 *)t->data;
   }
   if (other) {
      if (other->ndims != ix->ndims) return fail("Tensor size mismatch in %s", what);
      for (int d = 0; d < ix->ndims; d++) if (other->size[d] != ix->size[d]) return fail("Tensor size mismatch in %s", what);
      if (other->dtype != ix->view.dtype) return fail("Data type mismatch in %s", what);
      if (other->device != ix->view.device) return fail("Device mismatch in %s", what);
   }
   return 0;
}
static int index_tables_wait(const OcTensorView *writer, const OcIndexView *ix, bool before)
{
   for (int d = 0; d < ix->ndims; d++) {
      if (ix->offsets[d] == nullptr) continue;
      if ((before ? start_read(writer, ix->offsets[d]) : finish_read(writer, ix->offsets[d])) != 0) return -1;
   }
   return 0;
}

extern "C" int OcTensorGPU_getIndex(const OcIndexView *ix, const OcTensorView *dst)
{
   solid_int64 *tables[8];
   if (check_elemwise(dst, "destination") != 0 || index_prepare(ix, dst, "getIndex", tables) != 0) return -1;
   solid_funptr_gpu_get_index f = lookup(solid_gpu_get_index, dst->dtype, "getIndex");
   if (f == nullptr || set_device(dst->device) != 0) return -1;
   if (start_read(dst, &ix->view) != 0 || index_tables_wait(dst, ix, true) != 0) return -1;
   if (f(ix->ndims, ix->size, tables, ix->view.strides, ix->view.data, dst->strides, dst->data, dst->stream) != 0) return fail_solid();
   if (update(dst) != 0 || finish_read(dst, &ix->view) != 0) return -1;
   return index_tables_wait(dst, ix, false);
}
extern "C" int OcTensorGPU_setIndex(const OcIndexView *ix, const OcTensorView *src)
{
   solid_int64 *tables[8];
   if (check_elemwise(src, "source") != 0 || index_prepare(ix, src, "setIndex", tables) != 0) return -1;
   const OcTensorView *dst = &ix->view;
   solid_funptr_gpu_set_index f = lookup(solid_gpu_set_index, dst->dtype, "setIndex");
   if (f == nullptr || set_device(dst->device) != 0) return -1;
   if (start_read(dst, src) != 0 || index_tables_wait(dst, ix, true) != 0) return -1;
   if (f(ix->ndims, ix->size, tables, dst->strides, dst->data, src->strides, src->data, dst->stream) != 0) return fail_solid();
   if (update(dst) != 0 || finish_read(dst, src) != 0) return -1;
   return index_tables_wait(dst, ix, false);
}
extern "C" int OcTensorGPU_fillIndex(const OcIndexView *ix, const OcScalarView *s)
{
   solid_int64 *tables[8];
   if (index_prepare(ix, nullptr, "fillIndex", tables) != 0) return -1;
   const OcTensorView *dst = &ix->view;
   if (s == nullptr || s->dtype != dst->dtype) return fail("The scalar must have the data type of the tensor");
   solid_funptr_gpu_fill_index f = lookup(solid_gpu_fill_index, dst->dtype, "fillIndex");
   if (f == nullptr || set_device(dst->device) != 0) return -1;
   if (index_tables_wait(dst, ix, true) != 0) return -1;
   if (f(ix->ndims, ix->size, tables, dst->strides, dst->data, s->value, dst->stream) != 0) return fail_solid();
   if (update(dst) != 0) return -1;
   return index_tables_wait(dst, ix, false);
}
extern "C" int OcTensorGPU_addIfNegative(const OcTensorView *t, const OcScalarView *s)
{
   if (check_elemwise(t, "input") != 0) return -1;
   if (s == nullptr || s->dtype != t->dtype) return fail("The scalar must have the data type of the tensor");
   solid_funptr_gpu_add_if_negative f = lookup(solid_gpu_add_if_negative, t->dtype, "addIfNegative");
   if (f == nullptr || set_device(t->device) != 0) return -1;
   if (f(t->ndims, t->size, t->strides, t->data, s->value, t->stream) != 0) return fail_solid();
   return update(t);
}
extern "C" int OcTensorGPU_indexToOffset(const OcTensorView *t, const solid_int64 *strides, const OcTensorView *offsets)
{
   if (check_elemwise(t, "index") != 0 || check_elemwise(offsets, "offset") != 0) return -1;
   if (strides == nullptr) return fail("Missing strides in indexToOffset");
   if (offsets->dtype != SD_INT64 || offsets->ndims != 1) return fail("The offsets must be a vector of int64");
   if (t->ndims != 1 && t->ndims != 2) return fail("The index tensor must have one or two dimensions");
   solid_funptr_gpu_index_to_offset f = lookup(solid_gpu_index_to_offset, t->dtype, "indexToOffset");
   if (f == nullptr || set_device(offsets->device) != 0) return -1;
   ptrdiff_t stride1, stride_reduce; size_t nelem; int nstrides;           // tensor_index_gpu.c:107-118
   if (t->ndims == 1) { stride1 = t->strides[0]; stride_reduce = 0; nstrides = 1; nelem = t->size[0]; }
   else { stride1 = t->strides[1]; stride_reduce = t->strides[0]; nstrides = (int)t->size[0]; nelem = t->size[1]; }
   if (offsets->size[0] != nelem) return fail("Tensor size mismatch in indexToOffset");
   if (start_read(offsets, t) != 0) return -1;
   if (f(nstrides, const_cast<solid_int64 *>(strides), stride_reduce, nelem, stride1, t->data,
         offsets->strides[0], offsets->data, offsets->stream) != 0) return fail_solid();
   if (update(offsets) != 0) return -1;
   return finish_read(offsets, t);
}

// Two events per ordered (source device, destination device) pair, created once: `on_src` lives on the source
// device and marks "the source stream's earlier work is done", `on_dst` on the destination device marks "the copy
// has run".  An event can only be recorded on a stream of its own device, hence one of each.
struct PairEvents { cudaEvent_t on_src, on_dst; bool ready; };
static PairEvents *pair_events(int src_device, int dst_device)
{
   static PairEvents table[64][64];
   static std::mutex lock;
   if (src_device < 0 || src_device >= 64 || dst_device < 0 || dst_device >= 64) { fail("Invalid device index"); return nullptr; }
   std::lock_guard<std::mutex> guard(lock);
   PairEvents &p = table[src_device][dst_device];
   if (!p.ready) {
      int current = 0; cudaGetDevice(&current);
      bool ok = cudaSetDevice(src_device) == cudaSuccess && cudaEventCreateWithFlags(&p.on_src, cudaEventDisableTiming) == cudaSuccess &&
                cudaSetDevice(dst_device) == cudaSuccess && cudaEventCreateWithFlags(&p.on_dst, cudaEventDisableTiming) == cudaSuccess;
      cudaSetDevice(current);
      if (!ok) { (void)cudaGetLastError(); fail("Error creating an event"); return nullptr; }
      p.ready = true;
   }
   return &p;
}

// OCEAN_B200_FORCE_STAGED_COPY=1 sends every cross-device copy through the dense temporaries even where peer
// loads are possible, so that the staged path can be exercised on machines whose GPUs all see each other.
static bool force_staged_copy()
{
   static const bool forced = [] { const char *e = getenv("OCEAN_B200_FORCE_STAGED_COPY"); return e && e[0] == '1'; }();
   return forced;
}

// Can kernels on device `reader` load memory of device `owner`?  Asked of the runtime once per pair; peer access is
// switched on at that moment (another library in the process may have done so already, which is not an error).
static bool peer_readable(int reader, int owner)
{
   static signed char known[64][64];                       // 0 not asked, 1 yes, -1 no
   static std::mutex lock;
   if (reader < 0 || reader >= 64 || owner < 0 || owner >= 64) return false;
   std::lock_guard<std::mutex> guard(lock);
   if (known[reader][owner] == 0) {
      int can = 0, current = -1;
      known[reader][owner] = -1;
      if (cudaDeviceCanAccessPeer(&can, reader, owner) == cudaSuccess && can && cudaGetDevice(&current) == cudaSuccess) {
         if (cudaSetDevice(reader) == cudaSuccess) {
            cudaError_t st = cudaDeviceEnablePeerAccess(owner, 0);
            if (st == cudaSuccess || st == cudaErrorPeerAccessAlreadyEnabled) known[reader][owner] = 1;
            (void)cudaGetLastError();
         }
         cudaSetDevice(current);
      } else (void)cudaGetLastError();
   }
   return known[reader][owner] > 0;
}

// ---------------------------------------------------------------------------------- copy / fill
extern "C" int OcTensorGPU_copy(const OcTensorView *src, const OcTensorView *dst)
{
   if (check_view(src, "source") != 0 || check_view(dst, "destination") != 0) return -1;
   size_t n1 = 1, n2 = 1;
   for (int i = 0; i < src->ndims; i++) n1 *= src->size[i];
   for (int i = 0; i < dst->ndims; i++) n2 *= dst->size[i];
   if (n1 != n2) return fail("Mismatch in number of elements in tensor copy");
   if (set_device(dst->device) != 0) return -1;
   if (start_read(dst, src) != 0) return -1;
   const int flags = (src->byteswapped ? SOLID_GPU_COPY_SRC_SWAPPED : 0) | (dst->byteswapped ? SOLID_GPU_COPY_DST_SWAPPED : 0);
   if (src->device == dst->device) {
      if (solid_gpu_copy_ex(src->dtype, dst->dtype, flags, src->ndims, src->size, src->strides, src->data,
                            dst->ndims, dst->size, dst->strides, dst->data, dst->stream) != 0) return fail_solid();
   } else if (!force_staged_copy() && peer_readable(dst->device, src->device)) {
      // other device, readable through a peer mapping (NVLink on the HGX boards): the converting copy kernel runs on
      // the destination device and loads the source over the link with plain loads -- one pass, no temporaries on
      // either side.  The two streams belong to different devices, so they are ordered by the pair's own events:
      // the kernel starts after the source stream's earlier work, and the source stream continues after the kernel.
      PairEvents *ev = pair_events(src->device, dst->device);
      if (ev == nullptr) return -1;
      if (set_device(src->device) != 0) return -1;
      cudaEventRecord(ev->on_src, src->stream);
      if (set_device(dst->device) != 0) return -1;
      cudaStreamWaitEvent(dst->stream, ev->on_src, 0);
      if (solid_gpu_copy_ex(src->dtype, dst->dtype, flags, src->ndims, src->size, src->strides, src->data,
                            dst->ndims, dst->size, dst->strides, dst->data, dst->stream) != 0) return fail_solid();
      cudaEventRecord(ev->on_dst, dst->stream);
      cudaStreamWaitEvent(src->stream, ev->on_dst, 0);
   } else {
      // other device without peer access: gather into a dense buffer of the source type on the source device, move it
      // with one peer copy, convert on the destination (OcTensor_intrnlCopyDevices, tensor_itf.c:895-1041)
      const size_t bytes = n1 * (size_t)solid_gpu_type_size[src->dtype];
      void *tmp_src = nullptr, *tmp_dst = nullptr;
      int slot_src = 0, slot_dst = 0;
      size_t dense[1] = { n1 }; ptrdiff_t step[1] = { solid_gpu_type_size[src->dtype] };
      PairEvents *ev = pair_events(src->device, dst->device);
      if (ev == nullptr) return -1;
      if (set_device(src->device) != 0 || temporary(src->device, bytes, src->stream, &tmp_src, &slot_src) != 0) return -1;
      if (solid_gpu_copy_ex(src->dtype, src->dtype, 0, src->ndims, src->size, src->strides, src->data,
                            1, dense, step, tmp_src, src->stream) != 0) return fail_solid();
      cudaEventRecord(ev->on_src, src->stream);
      if (set_device(dst->device) != 0 || temporary(dst->device, bytes, dst->stream, &tmp_dst, &slot_dst) != 0) return -1;
      cudaStreamWaitEvent(dst->stream, ev->on_src, 0);
      cudaError_t st = cudaMemcpyPeerAsync(tmp_dst, dst->device, tmp_src, src->device, bytes, dst->stream);
      if (st != cudaSuccess) return fail_cuda(st, "Error copying between devices");
      // the source-side buffer is free once the transfer has run: the source stream waits for it, and the slot's
      // event is recorded behind that wait
      cudaEventRecord(ev->on_dst, dst->stream);
      if (solid_gpu_copy_ex(src->dtype, dst->dtype, flags, 1, dense, step, tmp_dst,
                            dst->ndims, dst->size, dst->strides, dst->data, dst->stream) != 0) return fail_solid();
      if (scratch_done(dst->device, slot_dst, dst->stream) != 0) return -1;
      if (set_device(src->device) != 0) return -1;
      cudaStreamWaitEvent(src->stream, ev->on_dst, 0);
      if (scratch_done(src->device, slot_src, src->stream) != 0) return -1;
      if (set_device(dst->device) != 0) return -1;
   }
   if (update(dst) != 0) return -1;
   return finish_read(dst, src);
}

extern "C" int OcTensorGPU_byteswapNoFlag(const OcTensorView *t)
{
   if (check_view(t, "input") != 0) return -1;
   solid_funptr_gpu_byteswap f = lookup(solid_gpu_byteswap, t->dtype, "byteswap");
   if (f == nullptr || set_device(t->device) != 0) return -1;
   if (f(t->ndims, t->size, t->strides, t->data, t->stream) != 0) return fail_solid();
   return update(t);
}

// The scalar arrives as the bytes to store: for a byte-swapped tensor the interface layer has already reversed them
// (OcTensor_fill, src/core/interface/tensor_itf.c:2770-2784), so the destination's byte order does not matter here.
static int fill_common(const OcTensorView *t, const OcScalarView *s, solid_funptr_gpu_fill const *table, const char *desc)
{
   if (check_view(t, "destination") != 0) return -1;
   if (s == nullptr || s->dtype != t->dtype) return fail("The scalar must have the data type of the tensor");
   solid_funptr_gpu_fill f = lookup(table, t->dtype, desc);
   if (f == nullptr || set_device(t->device) != 0) return -1;
   if (f(t->ndims, t->size, t->strides, t->data, s->value, t->stream) != 0) return fail_solid();
   return update(t);
}
extern "C" int OcTensorGPU_fill(const OcTensorView *t, const OcScalarView *s) { return fill_common(t, s, solid_gpu_fill, "fill"); }
extern "C" int OcTensorGPU_fillNaN(const OcTensorView *t, const OcScalarView *s) { return fill_common(t, s, solid_gpu_fill_nan, "fillNaN"); }

extern "C" int OcTensorGPU_maskedFill(const OcTensorView *t, const OcTensorView *mask, const OcScalarView *s)
{
   if (check_view(t, "destination") != 0 || check_elemwise(mask, "mask") != 0) return -1;
   if (mask->dtype != SD_BOOL) return fail("The mask must have type bool");
   if (!same_shape(t, mask)) return fail("Tensor size mismatch in maskedFill");
   if (s == nullptr || s->dtype != t->dtype) return fail("The scalar must have the data type of the tensor");
   solid_funptr_gpu_masked_fill f = lookup(solid_gpu_masked_fill, t->dtype, "maskedFill");
   if (f == nullptr || set_device(t->device) != 0) return -1;
   if (start_read(t, mask) != 0) return -1;
   if (f(t->ndims, t->size, t->strides, t->data, mask->strides, mask->data, s->value, t->stream) != 0) return fail_solid();
   if (update(t) != 0) return -1;
   return finish_read(t, mask);
}

// ---------------------------------------------------------------------------------- global reductions
namespace {
struct ReduceSetup { void *buffer; int slot; };
int reduce_begin(const OcTensorView *t, ReduceSetup *rs)             // OcTensorGPU_intrnlInitializeReduce
{
   if (check_elemwise(t, "input") != 0) return -1;
   if (set_device(t->device) != 0) return -1;
   size_t n = 1, bytes = 0;
   for (int i = 0; i < t->ndims; i++) n *= t->size[i];
   if (solid_gpu_reduce_all_buffer_size(n, t->device, &bytes) != 0) return fail_solid();
   return temporary(t->device, bytes, t->stream, &rs->buffer, &rs->slot);
}
// the scratch is free again once everything queued on the tensor's stream so far has run
int reduce_end(const OcTensorView *t, const ReduceSetup *rs, int status)
{
   if (status != 0) { fail_solid(); scratch_done(t->device, rs->slot, t->stream); return -1; }
   return scratch_done(t->device, rs->slot, t->stream);
}
} // namespace

#define OCGPU_DEFINE_RBOOL(OP, SOLID)                                                              \
extern "C" int OcTensorGPU_##OP(const OcTensorView *t, int *result)                                \
{                                                                                                  \
   ReduceSetup rs; solid_bool value = 0;                                                           \
   if (reduce_begin(t, &rs) != 0) return -1;                                                       \
   solid_funptr_gpu_##SOLID f = lookup(solid_gpu_##SOLID, t->dtype, #OP);                          \
   if (f == nullptr) return -1;                                                                    \
   if (reduce_end(t, &rs, f(t->ndims, t->size, t->strides, t->data, &value, rs.buffer, t->stream)) != 0) return -1; \
   *result = value ? 1 : 0;                                                                        \
   return 0;                                                                                       \
}
OCGPU_REDUCE_BOOL_OPS(OCGPU_DEFINE_RBOOL)

#define OCGPU_DEFINE_RSCALAR(OP, SOLID)                                                            \
extern "C" int OcTensorGPU_##OP(const OcTensorView *t, OcScalarView *result)                       \
{                                                                                                  \
   ReduceSetup rs;                                                                                 \
   if (reduce_begin(t, &rs) != 0) return -1;                                                       \
   solid_funptr_gpu_##SOLID f = lookup(solid_gpu_##SOLID, t->dtype, #OP);                          \
   if (f == nullptr) return -1;                                                                    \
   memset(&result->value, 0, sizeof(result->value));                                               \
   result->dtype = OcGPU_reductionResultType(#SOLID, t->dtype);                                    \
   if (reduce_end(t, &rs, f(t->ndims, t->size, t->strides, t->data, &result->value, rs.buffer, t->stream)) != 0) return -1; \
   return 0;                                                                                       \
}
OCGPU_REDUCE_SCALAR_OPS(OCGPU_DEFINE_RSCALAR)

#define OCGPU_DEFINE_RNNZ(OP, SOLID)                                                               \
extern "C" int OcTensorGPU_##OP(const OcTensorView *t, solid_uint64 *result)                       \
{                                                                                                  \
   ReduceSetup rs;                                                                                 \
   if (reduce_begin(t, &rs) != 0) return -1;                                                       \
   solid_funptr_gpu_##SOLID f = lookup(solid_gpu_##SOLID, t->dtype, #OP);                          \
   if (f == nullptr) return -1;                                                                    \
   if (reduce_end(t, &rs, f(t->ndims, t->size, t->strides, t->data, result, rs.buffer, t->stream)) != 0) return -1; \
   return 0;                                                                                       \
}
OCGPU_DEFINE_RNNZ(nnz, nnz) OCGPU_DEFINE_RNNZ(nnzNaN, nnz_nan)

#define OCGPU_DEFINE_RNORM(OP, SOLID)                                                              \
extern "C" int OcTensorGPU_##OP(const OcTensorView *t, double p, OcScalarView *result)             \
{                                                                                                  \
   ReduceSetup rs;                                                                                 \
   if (reduce_begin(t, &rs) != 0) return -1;                                                       \
   solid_funptr_gpu_##SOLID f = lookup(solid_gpu_##SOLID, t->dtype, #OP);                          \
   if (f == nullptr) return -1;                                                                    \
   memset(&result->value, 0, sizeof(result->value));                                               \
   result->dtype = OcGPU_reductionResultType(#SOLID, t->dtype);                                    \
   if (reduce_end(t, &rs, f(t->ndims, t->size, t->strides, t->data, p, &result->value, rs.buffer, t->stream)) != 0) return -1; \
   return 0;                                                                                       \
}
OCGPU_DEFINE_RNORM(norm, norm) OCGPU_DEFINE_RNORM(normNaN, norm_nan)

#define OCGPU_DEFINE_BOUND1(OP, SOLID)                                                             \
extern "C" int OcTensorGPU_##OP(const OcTensorView *t, const OcScalarView *bound, int *result)     \
{                                                                                                  \
   ReduceSetup rs; solid_bool value = 0;                                                           \
   if (reduce_begin(t, &rs) != 0) return -1;                                                       \
   if (bound == nullptr || bound->dtype != t->dtype) return fail("The bound must have the data type of the tensor"); \
   solid_funptr_gpu_##SOLID f = lookup(solid_gpu_##SOLID, t->dtype, #OP);                          \
   if (f == nullptr) return -1;                                                                    \
   solid_scalar b = bound->value;                                                                  \
   if (reduce_end(t, &rs, f(t->ndims, t->size, t->strides, t->data, &b, &value, rs.buffer, t->stream)) != 0) return -1; \
   *result = value ? 1 : 0;                                                                        \
   return 0;                                                                                       \
}
OCGPU_DEFINE_BOUND1(allLT, all_lt) OCGPU_DEFINE_BOUND1(allLE, all_le) OCGPU_DEFINE_BOUND1(allGT, all_gt) OCGPU_DEFINE_BOUND1(allGE, all_ge)

#define OCGPU_DEFINE_BOUND2(OP, SOLID)                                                             \
extern "C" int OcTensorGPU_##OP(const OcTensorView *t, const OcScalarView *lower, const OcScalarView *upper, int *result) \
{                                                                                                  \
   ReduceSetup rs; solid_bool value = 0;                                                           \
   if (reduce_begin(t, &rs) != 0) return -1;                                                       \
   if (lower == nullptr || upper == nullptr || lower->dtype != t->dtype || upper->dtype != t->dtype) \
      return fail("The bounds must have the data type of the tensor");                             \
   solid_funptr_gpu_##SOLID f = lookup(solid_gpu_##SOLID, t->dtype, #OP);                          \
   if (f == nullptr) return -1;                                                                    \
   solid_scalar lo = lower->value, hi = upper->value;                                              \
   if (reduce_end(t, &rs, f(t->ndims, t->size, t->strides, t->data, &lo, &hi, &value, rs.buffer, t->stream)) != 0) return -1; \
   *result = value ? 1 : 0;                                                                        \
   return 0;                                                                                       \
}
OCGPU_DEFINE_BOUND2(allGTLT, all_gtlt) OCGPU_DEFINE_BOUND2(allGTLE, all_gtle)
OCGPU_DEFINE_BOUND2(allGELT, all_gelt) OCGPU_DEFINE_BOUND2(allGELE, all_gele)

// ---------------------------------------------------------------------------------- axis reductions
namespace {
// Split src into kept and reduced dimensions, plan, fetch scratch (OcTensorGPU_intrnlAxisReduce,
// tensor_reduce_axis_gpu.c:127-158).
int axis_begin(const OcTensorView *src, int n, const int *axes, const OcTensorView *dst, const char *solid_name,
               solid_gpu_reduce_axis_config *config, int *slot)
{
   *slot = -1;
   if (check_elemwise(src, "source") != 0 || check_elemwise(dst, "destination") != 0) return -1;
   bool reduced[SOLID_MAX_TENSOR_DIMS] = { false };
   for (int i = 0; i < n; i++) {
      if (axes[i] < 0 || axes[i] >= src->ndims) return fail("Axis index %d out of range", axes[i]);
      if (reduced[axes[i]]) return fail("Duplicate axis %d", axes[i]);
      reduced[axes[i]] = true;
   }
   size_t size[SOLID_MAX_TENSOR_DIMS], rsize[SOLID_MAX_TENSOR_DIMS];
   ptrdiff_t st1[SOLID_MAX_TENSOR_DIMS], st2[SOLID_MAX_TENSOR_DIMS], rst[SOLID_MAX_TENSOR_DIMS];
   int nd = 0, rd = 0;
   for (int i = 0; i < src->ndims; i++) {
      if (reduced[i]) { rsize[rd] = src->size[i]; rst[rd] = src->strides[i]; rd++; }
      else { size[nd] = src->size[i]; st1[nd] = src->strides[i]; nd++; }
   }
   // the destination either drops the reduced dimensions or keeps them with extent one
   int j = 0;
   if (dst->ndims == nd) { for (int i = 0; i < nd; i++) st2[i] = dst->strides[i]; }
   else if (dst->ndims == src->ndims) { for (int i = 0; i < src->ndims; i++) if (!reduced[i]) st2[j++] = dst->strides[i]; }
   else return fail("Destination dimensions do not match the reduction");
   j = 0;
   for (int i = 0; i < dst->ndims; i++) {
      size_t expect = (dst->ndims == nd) ? size[i] : (reduced[i] ? 1 : src->size[i]);
      if (dst->size[i] != expect) return fail("Destination size mismatch in axis reduction");
   }
   int rtype = OcGPU_reductionResultType(solid_name, src->dtype);
   if (dst->dtype != rtype) return fail("The destination must have type %s", rtype >= 0 ? dtype_names[rtype] : "?");
   if (set_device(dst->device) != 0) return -1;
   if (solid_gpu_reduce_axis_prepare(config, solid_gpu_worktype_size[rtype], nd, size, st1, src->data, st2, dst->data,
                                     rd, rsize, rst, dst->stream) != 0) return fail_solid();
   if (config->bufferSize > 0) {
      void *buf = nullptr;
      if (temporary(dst->device, config->bufferSize, dst->stream, &buf, slot) != 0) return -1;
      config->data.ptrBuffer = (char *)buf;
   }
   return start_read(dst, src);
}
int axis_end(const OcTensorView *src, const OcTensorView *dst, int slot, int status)
{
   if (status != 0) fail_solid();
   if (slot >= 0 && scratch_done(dst->device, slot, dst->stream) != 0) return -1;
   if (status != 0) return -1;
   if (update(dst) != 0) return -1;
   return finish_read(dst, src);
}
} // namespace

#define OCGPU_DEFINE_AXIS(OP, SOLID)                                                               \
extern "C" int OcTensorGPU_##OP(const OcTensorView *src, int n, const int *axes, const OcTensorView *dst) \
{                                                                                                  \
   solid_gpu_reduce_axis_config config; int slot;                                                  \
   solid_funptr_gpu_##SOLID f = lookup(solid_gpu_##SOLID, src ? src->dtype : -1, #OP);             \
   if (f == nullptr) return -1;                                                                    \
   if (axis_begin(src, n, axes, dst, #SOLID, &config, &slot) != 0) return -1;                      \
   return axis_end(src, dst, slot, f(&config));                                                    \
}
OCGPU_AXIS_OPS(OCGPU_DEFINE_AXIS)

#define OCGPU_DEFINE_AXIS_NORM(OP, SOLID)                                                          \
extern "C" int OcTensorGPU_##OP(const OcTensorView *src, double p, int n, const int *axes, const OcTensorView *dst) \
{                                                                                                  \
   solid_gpu_reduce_axis_config config; int slot;                                                  \
   solid_funptr_gpu_##SOLID f = lookup(solid_gpu_##SOLID, src ? src->dtype : -1, #OP);             \
   if (f == nullptr) return -1;                                                                    \
   if (axis_begin(src, n, axes, dst, #SOLID, &config, &slot) != 0) return -1;                      \
   return axis_end(src, dst, slot, f(&config, p));                                                 \
}
OCGPU_DEFINE_AXIS_NORM(axisNorm, axis_norm) OCGPU_DEFINE_AXIS_NORM(axisNormNaN, axis_norm_nan)
