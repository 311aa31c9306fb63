/* THCl.h — the host-facing C API of the B200 backend for torch.ClTensor.
 *
 * Function names, argument order, 0-based dimension arguments, struct field
 * order and ownership rules are those of cltorch's libTHCl (hughperkins/cltorch,
 * paths below are relative to its root), so that its Lua binding
 * (src/init.cpp, src/TensorMath.lua, src/FFI.lua) can sit on top unchanged.
 * Behind them are CUDA kernels for sm_100a reached through include/thb200.h.
 *
 * Differences a caller can observe:
 *  - THClStorage::wrapper holds the device address (float* in HBM) instead of an
 *    EasyCL CLWrapper*, and THClStorage::cl the per-device context. `data` (the
 *    host mirror of the reference) is NULL: host copies go through the copy
 *    functions, which move only the addressed sub-range.
 *  - Errors: the reference calls THError (Torch7's handler, which does not
 *    return). Here a failing call runs the handler installed with
 *    THClSetErrorHandler; the default prints the message and aborts. A handler
 *    that returns makes the failing call return early (0 / NULL where a value is
 *    expected) with the message kept for THClLastError().
 *  - All work of one device is ordered on one CUDA stream (the reference: one
 *    in-order OpenCL queue per device, src/lib/THClGeneral.h:87-88). Only the
 *    functions that return a float/int to the host, the to-host copies and
 *    THClSynchronize block.
 */
#ifndef THCL_B200_INC
#define THCL_B200_INC

#include <stddef.h>

#ifdef __cplusplus
#define THCL_API extern "C"
#else
#define THCL_API extern
#endif

/* ---- the slice of Torch7's TH that the API mentions ------------------------
 * When the real TH headers are included first (TH_GENERAL_INC defined) these
 * are skipped; layouts are those of torch7 lib/TH/generic/THStorage.h and
 * THTensor.h. The THLongStorage functions below are weak symbols, so a process
 * that also loads libTH uses libTH's. */
#ifndef TH_GENERAL_INC
typedef struct THAllocator THAllocator;
#define THCL_DECLARE_TH_TYPES(Name, real)                                                    \
  typedef struct TH##Name##Storage {                                                         \
    real* data; long size; int refcount; char flag;                                          \
    THAllocator* allocator; void* allocatorContext; struct TH##Name##Storage* view;          \
  } TH##Name##Storage;                                                                       \
  typedef struct TH##Name##Tensor {                                                          \
    long* size; long* stride; int nDimension;                                                \
    TH##Name##Storage* storage; long storageOffset; int refcount; char flag;                 \
  } TH##Name##Tensor;
THCL_DECLARE_TH_TYPES(Byte, unsigned char)
THCL_DECLARE_TH_TYPES(Char, char)
THCL_DECLARE_TH_TYPES(Short, short)
THCL_DECLARE_TH_TYPES(Int, int)
THCL_DECLARE_TH_TYPES(Long, long)
THCL_DECLARE_TH_TYPES(Float, float)
THCL_DECLARE_TH_TYPES(Double, double)
THCL_API THLongStorage* THLongStorage_newWithSize(long size);
THCL_API void THLongStorage_free(THLongStorage* storage);
#endif

#define TH_STORAGE_REFCOUNTED 1
#define TH_STORAGE_RESIZABLE 2
#define TH_STORAGE_FREEMEM 4
#define TH_TENSOR_REFCOUNTED 1

/* ---- state: src/lib/THClGeneral.h:60-131 ----------------------------------- */

struct THClDeviceContext; /* stream, scratch and device properties of one GPU */

typedef struct THClScratchSpace {
  float* wrapper; /* device memory */
  float* data;    /* pinned host memory of the same size, for read-backs */
} THClScratchSpace;

typedef struct THClState {
  int initialized;
  int allowNonGpus; /* kept for the binding; there is no non-GPU device here */
  int allocatedDevices;
  int currentDevice;
  int trace;           /* 1: print every device allocation, free and host<->device copy */
  int addFinish;       /* 1: synchronise the stream after every launch (debugging) */
  int detailedTimings; /* kept for the binding */
  struct THClScratchSpace** scratchSpaceByDevice;
  struct THClDeviceContext** contextByDevice; /* reference: deviceInfoByDevice + clByDevice */
} THClState;

THCL_API void THClInit(THClState* state);               /* src/lib/THClGeneral.cpp:58-71 */
THCL_API void THCl_initializeState(THClState* state);   /* :19-50 */
THCL_API void THClShutdown(THClState* state);           /* :73-101 */
THCL_API void THClSetAllowNonGpus(THClState* state, int allowNonGpus);
THCL_API int THClState_getNumDevices(THClState* state);
THCL_API void THClState_setDevice(THClState* state, int device);
THCL_API int THClState_getDevice(THClState* state);
THCL_API struct THClScratchSpace* THClState_getDeviceScratchSpace(THClState* state, int device, int stream);
THCL_API size_t THClState_getDeviceScratchSpaceSize(THClState* state, int device);
/* the deprecated current-device forms, src/lib/THClGeneral.h:128-130 */
THCL_API struct THClScratchSpace* THClState_getCurrentDeviceScratchSpace(THClState* state);
THCL_API size_t THClState_getCurrentDeviceScratchSpaceSize(THClState* state);
/* cltorch.synchronize / cltorch.finish, src/init.cpp:72-78 */
THCL_API void THClSynchronize(THClState* state);
/* The CUDA stream (cudaStream_t as void*) that carries device `device`'s work.
 * setStream adopts a caller-owned stream, e.g. the one of the framework that
 * owns the process. No counterpart in the reference (one queue per device). */
THCL_API void* THClState_getStream(THClState* state, int device);
THCL_API void THClState_setStream(THClState* state, int device, void* stream);

typedef void (*THClErrorHandler)(const char* msg, void* data);
THCL_API void THClSetErrorHandler(THClErrorHandler handler, void* data);
THCL_API const char* THClLastError(void); /* "" if the last call on this thread succeeded */
THCL_API void THClClearError(void);

/* ---- storage: src/lib/THClStorage.h:13-59, src/FFI.lua:6-18 ---------------- */

typedef struct THClStorage {
  int device;
  float* data;                   /* NULL (no host mirror) */
  struct THClDeviceContext* cl;  /* reference: EasyCL* */
  float* wrapper;                /* device memory; reference: CLWrapper* */
  long size;
  int refcount;
  char flag;
  THAllocator* allocator;
  void* allocatorContext;
  struct THClStorage* view;
} THClStorage;

THCL_API float* THClStorage_data(THClState* state, const THClStorage*);
THCL_API long THClStorage_size(THClState* state, const THClStorage*);
THCL_API void THClStorage_set(THClState* state, THClStorage*, long, float);
THCL_API float THClStorage_get(THClState* state, const THClStorage*, long);
THCL_API THClStorage* THClStorage_new(THClState* state);
THCL_API THClStorage* THClStorage_newv2(THClState* state, int device);
THCL_API THClStorage* THClStorage_newWithSize(THClState* state, int device, long size);
THCL_API THClStorage* THClStorage_newWithSize1(THClState* state, int device, float);
THCL_API THClStorage* THClStorage_newWithSize2(THClState* state, int device, float, float);
THCL_API THClStorage* THClStorage_newWithSize3(THClState* state, int device, float, float, float);
THCL_API THClStorage* THClStorage_newWithSize4(THClState* state, int device, float, float, float, float);
/* takes ownership of the malloc'ed host array `data`: uploads it, then frees it */
THCL_API THClStorage* THClStorage_newWithData(THClState* state, int device, float* data, long size);
/* wraps device memory that the caller owns and keeps alive (not freed, not
 * resizable); no counterpart in the reference */
THCL_API THClStorage* THClStorage_newWithDevicePointer(THClState* state, int device, float* devptr, long size);
THCL_API void THClStorage_setFlag(THClState* state, THClStorage* storage, const char flag);
THCL_API void THClStorage_clearFlag(THClState* state, THClStorage* storage, const char flag);
THCL_API void THClStorage_retain(THClState* state, THClStorage* storage);
THCL_API void THClStorage_free(THClState* state, THClStorage* storage);
/* grows only; contents are not preserved (src/lib/THClStorage.cpp:236-252) */
THCL_API void THClStorage_resize(THClState* state, THClStorage* storage, long size);
THCL_API void THClStorage_fill(THClState* state, THClStorage* storage, float value);

/* src/lib/THClStorageCopy.h */
THCL_API void THClStorage_rawCopy(THClState* state, THClStorage* storage, float* src); /* host -> device, `size` floats */
THCL_API void THClStorage_copy(THClState* state, THClStorage* storage, THClStorage* src);
THCL_API void THClStorage_copyCl(THClState* state, THClStorage* storage, THClStorage* src);
THCL_API void THClStorage_copyFloat(THClState* state, THClStorage* storage, struct THFloatStorage* src);
THCL_API void THFloatStorage_copyCl(THClState* state, struct THFloatStorage* self, struct THClStorage* src);

/* ---- tensor: src/lib/THClTensor.h:14-145, src/FFI.lua:20-33 ---------------- */

typedef struct THClTensor {
  long* size;
  long* stride;
  int nDimension;
  THClStorage* storage;
  long storageOffset;
  int refcount;
  char flag;
  int device;
} THClTensor;

THCL_API THClStorage* THClTensor_storage(THClState* state, const THClTensor* self);
THCL_API long THClTensor_storageOffset(THClState* state, const THClTensor* self);
THCL_API int THClTensor_nDimension(THClState* state, const THClTensor* self);
THCL_API long THClTensor_size(THClState* state, const THClTensor* self, int dim);
THCL_API long THClTensor_stride(THClState* state, const THClTensor* self, int dim);
THCL_API THLongStorage* THClTensor_newSizeOf(THClState* state, THClTensor* self);
THCL_API THLongStorage* THClTensor_newStrideOf(THClState* state, THClTensor* self);
THCL_API float* THClTensor_data(THClState* state, const THClTensor* self); /* device address of element 0 */
/* src/lib/THClTensor.h:40 (returns the storage's CLWrapper there): the device address of the
 * storage's first float, NOT offset by storageOffset; NULL without storage. */
THCL_API float* THClTensor_wrapper(THClState* state, const THClTensor* self);
THCL_API void THClTensor_setFlag(THClState* state, THClTensor* self, const char flag);
THCL_API void THClTensor_clearFlag(THClState* state, THClTensor* self, const char flag);

THCL_API THClTensor* THClTensor_new(THClState* state);
THCL_API THClTensor* THClTensor_newv2(THClState* state, int device);
THCL_API THClTensor* THClTensor_newWithTensor(THClState* state, THClTensor* tensor);
THCL_API THClTensor* THClTensor_newWithStorage(THClState* state, int device, THClStorage* storage_, long storageOffset_, THLongStorage* size_, THLongStorage* stride_);
THCL_API THClTensor* THClTensor_newWithStorage1d(THClState* state, int device, THClStorage* storage_, long storageOffset_, long size0_, long stride0_);
THCL_API THClTensor* THClTensor_newWithStorage2d(THClState* state, int device, THClStorage* storage_, long storageOffset_, long size0_, long stride0_, long size1_, long stride1_);
THCL_API THClTensor* THClTensor_newWithStorage3d(THClState* state, int device, THClStorage* storage_, long storageOffset_, long size0_, long stride0_, long size1_, long stride1_, long size2_, long stride2_);
THCL_API THClTensor* THClTensor_newWithStorage4d(THClState* state, int device, THClStorage* storage_, long storageOffset_, long size0_, long stride0_, long size1_, long stride1_, long size2_, long stride2_, long size3_, long stride3_);
THCL_API THClTensor* THClTensor_newWithSize(THClState* state, int device, THLongStorage* size_, THLongStorage* stride_);
THCL_API THClTensor* THClTensor_newWithSize1d(THClState* state, int device, long size0_);
THCL_API THClTensor* THClTensor_newWithSize2d(THClState* state, int device, long size0_, long size1_);
THCL_API THClTensor* THClTensor_newWithSize3d(THClState* state, int device, long size0_, long size1_, long size2_);
THCL_API THClTensor* THClTensor_newWithSize4d(THClState* state, int device, long size0_, long size1_, long size2_, long size3_);
THCL_API THClTensor* THClTensor_newClone(THClState* state, THClTensor* self);
THCL_API THClTensor* THClTensor_newContiguous(THClState* state, THClTensor* tensor);
THCL_API THClTensor* THClTensor_newSelect(THClState* state, THClTensor* tensor, int dimension_, long sliceIndex_);
THCL_API THClTensor* THClTensor_newNarrow(THClState* state, THClTensor* tensor, int dimension_, long firstIndex_, long size_);
THCL_API THClTensor* THClTensor_newTranspose(THClState* state, THClTensor* tensor, int dimension1_, int dimension2_);
THCL_API THClTensor* THClTensor_newUnfold(THClState* state, THClTensor* tensor, int dimension_, long size_, long step_);

THCL_API void THClTensor_resize(THClState* state, THClTensor* tensor, THLongStorage* size, THLongStorage* stride);
THCL_API void THClTensor_resizeAs(THClState* state, THClTensor* tensor, THClTensor* src);
THCL_API void THClTensor_resize0d(THClState* state, THClTensor* tensor); /* point tensor: 0 dims, 1 float */
THCL_API void THClTensor_resize1d(THClState* state, THClTensor* tensor, long size0_);
THCL_API void THClTensor_resize2d(THClState* state, THClTensor* tensor, long size0_, long size1_);
THCL_API void THClTensor_resize3d(THClState* state, THClTensor* tensor, long size0_, long size1_, long size2_);
THCL_API void THClTensor_resize4d(THClState* state, THClTensor* tensor, long size0_, long size1_, long size2_, long size3_);
THCL_API void THClTensor_resize5d(THClState* state, THClTensor* tensor, long size0_, long size1_, long size2_, long size3_, long size4_);

THCL_API void THClTensor_set(THClState* state, THClTensor* self, THClTensor* src);
THCL_API void THClTensor_setStorage(THClState* state, THClTensor* self, THClStorage* storage_, long storageOffset_, THLongStorage* size_, THLongStorage* stride_);
THCL_API void THClTensor_setStorage1d(THClState* state, THClTensor* self, THClStorage* storage_, long storageOffset_, long size0_, long stride0_);
THCL_API void THClTensor_setStorage2d(THClState* state, THClTensor* self, THClStorage* storage_, long storageOffset_, long size0_, long stride0_, long size1_, long stride1_);
THCL_API void THClTensor_setStorage3d(THClState* state, THClTensor* self, THClStorage* storage_, long storageOffset_, long size0_, long stride0_, long size1_, long stride1_, long size2_, long stride2_);
THCL_API void THClTensor_setStorage4d(THClState* state, THClTensor* self, THClStorage* storage_, long storageOffset_, long size0_, long stride0_, long size1_, long stride1_, long size2_, long stride2_, long size3_, long stride3_);

THCL_API void THClTensor_narrow(THClState* state, THClTensor* self, THClTensor* src, int dimension_, long firstIndex_, long size_);
THCL_API void THClTensor_select(THClState* state, THClTensor* self, THClTensor* src, int dimension_, long sliceIndex_);
THCL_API void THClTensor_transpose(THClState* state, THClTensor* self, THClTensor* src, int dimension1_, int dimension2_);
THCL_API void THClTensor_unfold(THClState* state, THClTensor* self, THClTensor* src, int dimension_, long size_, long step_);
THCL_API void THClTensor_squeeze(THClState* state, THClTensor* self, THClTensor* src);
THCL_API void THClTensor_squeeze1d(THClState* state, THClTensor* self, THClTensor* src, int dimension_);

THCL_API int THClTensor_isContiguous(THClState* state, const THClTensor* self);
THCL_API int THClTensor_isSameSizeAs(THClState* state, const THClTensor* self, const THClTensor* src);
THCL_API long THClTensor_nElement(THClState* state, const THClTensor* self); /* 0 for a 0-dim tensor */
THCL_API void THClTensor_retain(THClState* state, THClTensor* self);
THCL_API void THClTensor_free(THClState* state, THClTensor* self);
THCL_API void THClTensor_freeCopyTo(THClState* state, THClTensor* self, THClTensor* dst);

THCL_API void THClTensor_set1d(THClState* state, THClTensor* tensor, long x0, float value);
THCL_API void THClTensor_set2d(THClState* state, THClTensor* tensor, long x0, long x1, float value);
THCL_API void THClTensor_set3d(THClState* state, THClTensor* tensor, long x0, long x1, long x2, float value);
THCL_API void THClTensor_set4d(THClState* state, THClTensor* tensor, long x0, long x1, long x2, long x3, float value);
THCL_API float THClTensor_get1d(THClState* state, const THClTensor* tensor, long x0);
THCL_API float THClTensor_get2d(THClState* state, const THClTensor* tensor, long x0, long x1);
THCL_API float THClTensor_get3d(THClState* state, const THClTensor* tensor, long x0, long x1, long x2);
THCL_API float THClTensor_get4d(THClState* state, const THClTensor* tensor, long x0, long x1, long x2, long x3);

THCL_API int THClTensor_getDevice(THClState* state, const THClTensor* self);
THCL_API int THClTensor_checkGPU(THClState* state, unsigned int nTensors, ...);

/* ---- copies: src/lib/THClTensorCopy.h:7-23 --------------------------------- */

THCL_API void THClTensor_copy(THClState* state, THClTensor* self, THClTensor* src);
THCL_API void THClTensor_copyCl(THClState* state, THClTensor* self, THClTensor* src);
THCL_API void THClTensor_copyIgnoringOverlaps(THClState* state, THClTensor* dst, THClTensor* src);
#define THCL_DECLARE_HOST_COPY(Name)                                                             \
  THCL_API void THClTensor_copy##Name(THClState* state, THClTensor* self, TH##Name##Tensor* src); \
  THCL_API void TH##Name##Tensor_copyCl(THClState* state, TH##Name##Tensor* self, THClTensor* src);
THCL_DECLARE_HOST_COPY(Byte)
THCL_DECLARE_HOST_COPY(Char)
THCL_DECLARE_HOST_COPY(Short)
THCL_DECLARE_HOST_COPY(Int)
THCL_DECLARE_HOST_COPY(Long)
THCL_DECLARE_HOST_COPY(Float)
THCL_DECLARE_HOST_COPY(Double)
/* Extension (the reference's host copies all block, src/lib/THClTensorCopy.cpp:18-115): the upload of `n`
 * floats from page-locked host memory into a contiguous tensor of n elements is enqueued on `stream` (a
 * cudaStream_t of the tensor's device; NULL = the device's THCl stream) and the call returns; the host
 * memory must stay as it is until the stream has passed the copy. With a stream of its own a caller uploads
 * the next input while kernels work on the previous one on the THCl stream, with events of its own between
 * the two (THClState_setStream is no substitute: it waits for the stream it replaces). */
THCL_API void THClTensor_copyFloatAsync(THClState* state, THClTensor* self, const float* src, long n, void* stream);

/* ---- pointwise math: src/lib/THClTensorMath.h:7-155 ------------------------ */

THCL_API void THClTensor_fill(THClState* state, THClTensor* self, float value);
THCL_API void THClTensor_zero(THClState* state, THClTensor* self);
THCL_API void THClTensor_zeros(THClState* state, THClTensor* r_, THLongStorage* size);
THCL_API void THClTensor_ones(THClState* state, THClTensor* r_, THLongStorage* size);
THCL_API void THClTensor_reshape(THClState* state, THClTensor* r_, THClTensor* t, THLongStorage* size);
THCL_API long THClTensor_numel(THClState* state, THClTensor* t);

THCL_API void THClTensor_add(THClState* state, THClTensor* self, THClTensor* src, float value);
THCL_API void THClTensor_sub(THClState* state, THClTensor* self, THClTensor* src, float value);
THCL_API void THClTensor_mul(THClState* state, THClTensor* self, THClTensor* src, float value);
THCL_API void THClTensor_div(THClState* state, THClTensor* self, THClTensor* src, float value); /* multiplies by 1.0f/value */
THCL_API void THClTensor_cadd(THClState* state, THClTensor* self, THClTensor* src1, float value, THClTensor* src2);
THCL_API void THClTensor_csub(THClState* state, THClTensor* self, THClTensor* src1, float value, THClTensor* src2);
THCL_API void THClTensor_cmul(THClState* state, THClTensor* self, THClTensor* src1, THClTensor* src2);
THCL_API void THClTensor_cdiv(THClState* state, THClTensor* self, THClTensor* src1, THClTensor* src2);
THCL_API void THClTensor_cpow(THClState* state, THClTensor* self, THClTensor* src1, THClTensor* src2);
THCL_API void THClTensor_addcmul(THClState* state, THClTensor* self, THClTensor* t, float value, THClTensor* src1, THClTensor* src2);
THCL_API void THClTensor_addcdiv(THClState* state, THClTensor* self, THClTensor* t, float value, THClTensor* src1, THClTensor* src2);
THCL_API void THClTensor_cmin(THClState* state, THClTensor* self, THClTensor* src1, THClTensor* src2);
THCL_API void THClTensor_cmax(THClState* state, THClTensor* self, THClTensor* src1, THClTensor* src2);
THCL_API void THClTensor_cminValue(THClState* state, THClTensor* self, THClTensor* src, float value);
THCL_API void THClTensor_cmaxValue(THClState* state, THClTensor* self, THClTensor* src, float value);

/* self = f(src), in place when self == src (src/lib/THClTensorMathPointwise.cpp:18-78) */
#define THCL_DECLARE_UNARY(NAME) THCL_API void THClTensor_##NAME(THClState* state, THClTensor* self, THClTensor* src);
THCL_DECLARE_UNARY(log) THCL_DECLARE_UNARY(log1p) THCL_DECLARE_UNARY(exp) THCL_DECLARE_UNARY(cos)
THCL_DECLARE_UNARY(acos) THCL_DECLARE_UNARY(cosh) THCL_DECLARE_UNARY(sin) THCL_DECLARE_UNARY(asin)
THCL_DECLARE_UNARY(sinh) THCL_DECLARE_UNARY(tan) THCL_DECLARE_UNARY(atan) THCL_DECLARE_UNARY(tanh)
THCL_DECLARE_UNARY(sqrt) THCL_DECLARE_UNARY(ceil) THCL_DECLARE_UNARY(floor) THCL_DECLARE_UNARY(abs)
THCL_DECLARE_UNARY(round) THCL_DECLARE_UNARY(neg) THCL_DECLARE_UNARY(cinv) THCL_DECLARE_UNARY(sigmoid)
THCL_DECLARE_UNARY(sign)

THCL_API void THClTensor_pow(THClState* state, THClTensor* self, THClTensor* src, float value);
THCL_API void THClTensor_tpow(THClState* state, THClTensor* self, float value, THClTensor* src);
THCL_API void THClTensor_clamp(THClState* state, THClTensor* self, THClTensor* src, float min_value, float max_value);
THCL_API void THClTensor_atan2(THClState* state, THClTensor* r_, THClTensor* tx, THClTensor* ty);

/* comparisons produce 0.0f / 1.0f (src/lib/THClTensorMathCompare.cpp, THClTensorMathCompareT.cpp) */
#define THCL_DECLARE_COMPARE(NAME)                                                                                   \
  THCL_API void THClTensor_##NAME##Value(THClState* state, THClTensor* self_, THClTensor* src, float value);          \
  THCL_API void THClTensor_##NAME##Tensor(THClState* state, THClTensor* self_, THClTensor* src1, THClTensor* src2);   \
  THCL_API void THClTensor_##NAME##PointTensor(THClState* state, THClTensor* self_, THClTensor* src, THClTensor* value);
THCL_DECLARE_COMPARE(lt) THCL_DECLARE_COMPARE(gt) THCL_DECLARE_COMPARE(le)
THCL_DECLARE_COMPARE(ge) THCL_DECLARE_COMPARE(eq) THCL_DECLARE_COMPARE(ne)

/* user expressions over x (self, read/write), y, z: apply_on_gpu / map_on_gpu /
 * map2_on_gpu (src/lib/THClTensorMathPointwise.cpp:79-146, src/TensorMath.lua:591-620) */
THCL_API void THClTensor_apply(THClState* state, THClTensor* self, char const* operation1);
THCL_API void THClTensor_map(THClState* state, THClTensor* self, THClTensor* two, char const* operation2);
THCL_API void THClTensor_map2(THClState* state, THClTensor* self, THClTensor* in1, THClTensor* in2, char const* operation3);

/* operations whose scalar operand is a point tensor that stays on the device */
THCL_API void THClTensor_add_gpu(THClState* state, THClTensor* self, THClTensor* src, THClTensor* value);
THCL_API void THClTensor_sub_gpu(THClState* state, THClTensor* self, THClTensor* src, THClTensor* value);
THCL_API void THClTensor_mul_gpu(THClState* state, THClTensor* self, THClTensor* src, THClTensor* value);
THCL_API void THClTensor_div_gpu(THClState* state, THClTensor* self, THClTensor* src, THClTensor* value); /* true division */
THCL_API void THClTensor_fill_gpu(THClState* state, THClTensor* self, THClTensor* value);

/* ---- reductions ------------------------------------------------------------ */

/* whole tensor -> host scalar (blocks until the value is back) */
THCL_API float THClTensor_sumall(THClState* state, THClTensor* self);
THCL_API float THClTensor_prodall(THClState* state, THClTensor* self);
THCL_API float THClTensor_minall(THClState* state, THClTensor* self);
THCL_API float THClTensor_maxall(THClState* state, THClTensor* self);
THCL_API float THClTensor_meanall(THClState* state, THClTensor* self);
THCL_API float THClTensor_varall(THClState* state, THClTensor* self);
THCL_API float THClTensor_stdall(THClState* state, THClTensor* self);
THCL_API float THClTensor_normall(THClState* state, THClTensor* self, float value);
THCL_API int THClTensor_logicalall(THClState* state, THClTensor* self);
THCL_API int THClTensor_logicalany(THClState* state, THClTensor* self);
THCL_API float THClTensor_as_float(THClState* state, THClTensor* self); /* value of a point tensor */

/* whole tensor -> point tensor `self` (0 dims), no host synchronisation */
THCL_API void THClTensor_sumall_gpu(THClState* state, THClTensor* self, THClTensor* src);
THCL_API void THClTensor_prodall_gpu(THClState* state, THClTensor* self, THClTensor* src);
THCL_API void THClTensor_minall_gpu(THClState* state, THClTensor* self, THClTensor* src);
THCL_API void THClTensor_maxall_gpu(THClState* state, THClTensor* self, THClTensor* src);
THCL_API void THClTensor_logicalall_gpu(THClState* state, THClTensor* self, THClTensor* src);
THCL_API void THClTensor_logicalany_gpu(THClState* state, THClTensor* self, THClTensor* src);
/* mean / var / std as point tensors. The reference declares meanall/varall/stdall
 * (src/lib/THClTensorMath.h:88-93) but ships only the host-scalar meanall; these
 * follow its commented specification (src/lib/THClTensorMath2.cpp:181-229):
 * mean = sum / n, var = sum((x - mean)^2) / (n - 1), std = sqrt(var). var and std read the
 * input once (shifted sums of x and x^2 kept in double) instead of twice. */
THCL_API void THClTensor_meanall_gpu(THClState* state, THClTensor* self, THClTensor* src);
THCL_API void THClTensor_varall_gpu(THClState* state, THClTensor* self, THClTensor* src);
THCL_API void THClTensor_stdall_gpu(THClState* state, THClTensor* self, THClTensor* src);

/* along one dimension (0-based); `self` gets src's shape with size 1 at `dim` */
THCL_API void THClTensor_sum(THClState* state, THClTensor* self, THClTensor* src, long dim);
THCL_API void THClTensor_prod(THClState* state, THClTensor* self, THClTensor* src, long dim);
THCL_API void THClTensor_mean(THClState* state, THClTensor* self, THClTensor* src, long dim);
THCL_API void THClTensor_norm(THClState* state, THClTensor* self, THClTensor* src, float value, long dimension);
/* indices are 1-based positions stored as fp32; first occurrence wins ties */
THCL_API void THClTensor_max(THClState* state, THClTensor* values, THClTensor* indices, THClTensor* src, long dim);
THCL_API void THClTensor_min(THClState* state, THClTensor* values, THClTensor* indices, THClTensor* src, long dim);

/* Variance / standard deviation along `dim` (0-based); flag != 0 divides by n instead of n - 1.
 * Declared in src/lib/THClTensorMath.h:93-95; the reference's implementation
 * (src/lib/THClTensorMath2.cpp:293-333, kernels src/lib/THClTensorMath2.cl:5-108) is commented
 * out and serves as the specification. `self` keeps the dimension with size 1. */
THCL_API void THClTensor_var(THClState* state, THClTensor* self, THClTensor* src, long dim, int flag);
THCL_API void THClTensor_std(THClState* state, THClTensor* self, THClTensor* src, long dim, int flag);
/* Inclusive scans along `dim` (src/lib/THClTensorMathScan.cpp:144-156); self is resized like src. */
THCL_API void THClTensor_cumsum(THClState* state, THClTensor* self, THClTensor* src, long dim);
THCL_API void THClTensor_cumprod(THClState* state, THClTensor* self, THClTensor* src, long dim);
/* Every sub-tensor along `dimension` whose p-norm (p = value > 0) exceeds max_norm is scaled to
 * max_norm (src/lib/THClTensorMath.h:98; specification src/lib/THClTensorMath2.cpp:414-446). */
THCL_API void THClTensor_renorm(THClState* state, THClTensor* self, THClTensor* src, float value, long dimension, float max_norm);
/* (sum |self - src|^value)^(1/value) (src/lib/THClTensorMath.h:99; specification
 * src/lib/THClTensorMath2.cpp:448-475); the _gpu form leaves the result in a point tensor. */
THCL_API float THClTensor_dist(THClState* state, THClTensor* self, THClTensor* src, float value);
THCL_API void THClTensor_dist_gpu(THClState* state, THClTensor* res, THClTensor* self, THClTensor* src, float value);

/* ---- BLAS front-ends: src/lib/THClTensorMathBlas.cpp ----------------------- */

THCL_API void THClTensor_addmm(THClState* state, THClTensor* self, float beta, THClTensor* t, float alpha, THClTensor* mat1, THClTensor* mat2);
THCL_API void THClTensor_baddbmm(THClState* state, THClTensor* result, float beta, THClTensor* t, float alpha, THClTensor* batch1, THClTensor* batch2);
/* self = beta * t + alpha * mat * vec (src/lib/THClTensorMathBlas.cpp:43-105) */
THCL_API void THClTensor_addmv(THClState* state, THClTensor* self, float beta, THClTensor* t, float alpha, THClTensor* mat, THClTensor* vec);
/* self = beta * t + alpha * vec1 (x) vec2 (src/lib/THClTensorMathBlas.cpp:216-277) */
THCL_API void THClTensor_addr(THClState* state, THClTensor* self, float beta, THClTensor* t, float alpha, THClTensor* vec1, THClTensor* vec2);
/* sum of self[i] * src[i] over all elements, returned to the host (src/lib/THClTensorMathBlas.cpp:17-41) */
THCL_API float THClTensor_dot(THClState* state, THClTensor* self, THClTensor* src);

#endif /* THCL_B200_INC */
