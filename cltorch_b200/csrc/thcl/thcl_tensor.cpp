// THClTensor: size/stride/offset views over a THClStorage
// (reference src/lib/THClTensor.cpp). Pure host bookkeeping except for the
// element accessors and the functions that copy.
#include "thcl_internal.h"

#include <cstdarg>
#include <cstdlib>
#include <cstring>

using namespace thcl;

namespace thcl {

void View::set(const THClTensor* x) {
  t.ndim = x->nDimension > 0 ? x->nDimension : 0;
  if (t.ndim > THB200_MAX_DIMS) raise("tensor too large or too many (>%d) dimensions", THB200_MAX_DIMS);
  for (int d = 0; d < t.ndim; ++d) {
    size[d] = x->size[d];
    stride[d] = x->stride[d];
  }
  t.data = (x->storage && x->storage->wrapper) ? x->storage->wrapper + x->storageOffset : nullptr;
}

}  // namespace thcl

// A new tensor has nDimension -1 and no storage (reference src/lib/THClTensor.cpp:628-639).
static void raw_init(int device, THClTensor* self) {
  self->refcount = 1;
  self->storage = nullptr;
  self->storageOffset = 0;
  self->size = nullptr;
  self->stride = nullptr;
  self->nDimension = -1;
  self->flag = TH_TENSOR_REFCOUNTED;
  self->device = device;
}

// Sizes are read up to the first non-positive entry; missing strides are the
// contiguous ones; the storage grows to hold the last addressed element, and at
// least one float for a 0-dim tensor (reference src/lib/THClTensor.cpp:671-736).
static void raw_resize(THClState* state, THClTensor* self, int nDimension, const long* size, const long* stride) {
  int nd = 0;
  bool correct = true;
  for (int d = 0; d < nDimension; ++d) {
    if (size[d] > 0) {
      ++nd;
      if (self->nDimension > d && size[d] != self->size[d]) correct = false;
      if (self->nDimension > d && stride && stride[d] >= 0 && stride[d] != self->stride[d]) correct = false;
    } else {
      break;
    }
  }
  nDimension = nd;
  if (nDimension != self->nDimension) correct = false;
  if (correct) return;

  if (nDimension != self->nDimension) {
    self->size = (long*)realloc(self->size, sizeof(long) * (nDimension > 0 ? nDimension : 1));
    self->stride = (long*)realloc(self->stride, sizeof(long) * (nDimension > 0 ? nDimension : 1));
    self->nDimension = nDimension;
  }
  long total = 1;
  for (int d = nDimension - 1; d >= 0; --d) {
    self->size[d] = size[d];
    if (stride && stride[d] >= 0) self->stride[d] = stride[d];
    else self->stride[d] = (d == nDimension - 1) ? 1 : self->size[d + 1] * self->stride[d + 1];
    total += (self->size[d] - 1) * self->stride[d];
  }
  if (total + self->storageOffset > 0) {
    if (!self->storage) self->storage = THClStorage_newv2(state, self->device);
    if (total + self->storageOffset > self->storage->size) THClStorage_resize(state, self->storage, total + self->storageOffset);
  }
}

static void raw_set(THClState* state, THClTensor* self, THClStorage* storage, long storageOffset, int nDimension,
                    const long* size, const long* stride) {
  if (self->storage != storage) {
    if (self->storage) THClStorage_free(state, self->storage);
    self->storage = storage;
    if (storage) THClStorage_retain(state, storage);
  }
  if (storageOffset < 0) raise("Tensor: invalid storage offset");
  self->storageOffset = storageOffset;
  raw_resize(state, self, nDimension, size, stride);
}

static THClTensor* alloc_tensor(int device) {
  THClTensor* t = (THClTensor*)malloc(sizeof(THClTensor));
  raw_init(device, t);
  return t;
}

static void check_index(const THClTensor* t, int nidx, const long* x) {
  arg_check(t->nDimension == nidx, 1, "tensor has a different number of dimensions");
  for (int d = 0; d < nidx; ++d) arg_check(x[d] >= 0 && x[d] < t->size[d], 2 + d, "out of range");
}

extern "C" {

THClStorage* THClTensor_storage(THClState*, const THClTensor* self) { return self->storage; }
long THClTensor_storageOffset(THClState*, const THClTensor* self) { return self->storageOffset; }
int THClTensor_nDimension(THClState*, const THClTensor* self) { return self->nDimension; }

long THClTensor_size(THClState*, const THClTensor* self, int dim) {
  THCL_BEGIN
  arg_check(dim >= 0 && dim < self->nDimension, 2, "out of range");
  return self->size[dim];
  THCL_END(0)
}
long THClTensor_stride(THClState*, const THClTensor* self, int dim) {
  THCL_BEGIN
  arg_check(dim >= 0 && dim < self->nDimension, 2, "out of range");
  return self->stride[dim];
  THCL_END(0)
}

THLongStorage* THClTensor_newSizeOf(THClState*, THClTensor* self) {
  int n = self->nDimension > 0 ? self->nDimension : 0;
  THLongStorage* s = THLongStorage_newWithSize(n);
  for (int d = 0; d < n; ++d) s->data[d] = self->size[d];
  return s;
}
THLongStorage* THClTensor_newStrideOf(THClState*, THClTensor* self) {
  int n = self->nDimension > 0 ? self->nDimension : 0;
  THLongStorage* s = THLongStorage_newWithSize(n);
  for (int d = 0; d < n; ++d) s->data[d] = self->stride[d];
  return s;
}

float* THClTensor_data(THClState*, const THClTensor* self) {
  return (self->storage && self->storage->wrapper) ? self->storage->wrapper + self->storageOffset : nullptr;
}

float* THClTensor_wrapper(THClState*, const THClTensor* self) { return self->storage ? self->storage->wrapper : nullptr; }

void THClTensor_setFlag(THClState*, THClTensor* self, const char flag) { self->flag |= flag; }
void THClTensor_clearFlag(THClState*, THClTensor* self, const char flag) { self->flag &= ~flag; }

THClTensor* THClTensor_newv2(THClState*, int device) { return alloc_tensor(device); }
THClTensor* THClTensor_new(THClState* state) { return alloc_tensor(state->currentDevice); }

THClTensor* THClTensor_newWithTensor(THClState* state, THClTensor* tensor) {
  THCL_BEGIN
  THClTensor* self = alloc_tensor(tensor->device);
  raw_set(state, self, tensor->storage, tensor->storageOffset, tensor->nDimension, tensor->size, tensor->stride);
  return self;
  THCL_END(nullptr)
}

THClTensor* THClTensor_newWithStorage(THClState* state, int device, THClStorage* storage, long storageOffset,
                                      THLongStorage* size, THLongStorage* stride) {
  THCL_BEGIN
  if (size && stride) arg_check(size->size == stride->size, 4, "inconsistent size");
  THClTensor* self = alloc_tensor(device);
  raw_set(state, self, storage, storageOffset, (int)(size ? size->size : (stride ? stride->size : 0)),
          size ? size->data : nullptr, stride ? stride->data : nullptr);
  return self;
  THCL_END(nullptr)
}

THClTensor* THClTensor_newWithStorage4d(THClState* state, int device, THClStorage* storage, long storageOffset,
                                        long size0, long stride0, long size1, long stride1, long size2, long stride2,
                                        long size3, long stride3) {
  THCL_BEGIN
  long size[4] = {size0, size1, size2, size3};
  long stride[4] = {stride0, stride1, stride2, stride3};
  THClTensor* self = alloc_tensor(device);
  raw_set(state, self, storage, storageOffset, 4, size, stride);
  return self;
  THCL_END(nullptr)
}
THClTensor* THClTensor_newWithStorage1d(THClState* state, int device, THClStorage* storage, long storageOffset,
                                        long size0, long stride0) {
  return THClTensor_newWithStorage4d(state, device, storage, storageOffset, size0, stride0, -1, -1, -1, -1, -1, -1);
}
THClTensor* THClTensor_newWithStorage2d(THClState* state, int device, THClStorage* storage, long storageOffset,
                                        long size0, long stride0, long size1, long stride1) {
  return THClTensor_newWithStorage4d(state, device, storage, storageOffset, size0, stride0, size1, stride1, -1, -1, -1, -1);
}
THClTensor* THClTensor_newWithStorage3d(THClState* state, int device, THClStorage* storage, long storageOffset,
                                        long size0, long stride0, long size1, long stride1, long size2, long stride2) {
  return THClTensor_newWithStorage4d(state, device, storage, storageOffset, size0, stride0, size1, stride1, size2, stride2, -1, -1);
}

THClTensor* THClTensor_newWithSize(THClState* state, int device, THLongStorage* size, THLongStorage* stride) {
  return THClTensor_newWithStorage(state, device, nullptr, 0, size, stride);
}
THClTensor* THClTensor_newWithSize4d(THClState* state, int device, long size0, long size1, long size2, long size3) {
  THCL_BEGIN
  long size[4] = {size0, size1, size2, size3};
  THClTensor* self = alloc_tensor(device);
  raw_resize(state, self, 4, size, nullptr);
  return self;
  THCL_END(nullptr)
}
THClTensor* THClTensor_newWithSize1d(THClState* state, int device, long size0) {
  return THClTensor_newWithSize4d(state, device, size0, -1, -1, -1);
}
THClTensor* THClTensor_newWithSize2d(THClState* state, int device, long size0, long size1) {
  return THClTensor_newWithSize4d(state, device, size0, size1, -1, -1);
}
THClTensor* THClTensor_newWithSize3d(THClState* state, int device, long size0, long size1, long size2) {
  return THClTensor_newWithSize4d(state, device, size0, size1, size2, -1);
}

THClTensor* THClTensor_newClone(THClState* state, THClTensor* self) {
  THCL_BEGIN
  THClTensor* t = alloc_tensor(self->device);
  THClTensor_resizeAs(state, t, self);
  THClTensor_copy(state, t, self);
  return t;
  THCL_END(nullptr)
}

THClTensor* THClTensor_newContiguous(THClState* state, THClTensor* self) {
  THCL_BEGIN
  if (!THClTensor_isContiguous(state, self)) return THClTensor_newClone(state, self);
  THClTensor_retain(state, self);
  return self;
  THCL_END(nullptr)
}

THClTensor* THClTensor_newSelect(THClState* state, THClTensor* tensor, int dimension, long sliceIndex) {
  THCL_BEGIN
  THClTensor* self = THClTensor_newWithTensor(state, tensor);
  THClTensor_select(state, self, nullptr, dimension, sliceIndex);
  return self;
  THCL_END(nullptr)
}
THClTensor* THClTensor_newNarrow(THClState* state, THClTensor* tensor, int dimension, long firstIndex, long size) {
  THCL_BEGIN
  THClTensor* self = THClTensor_newWithTensor(state, tensor);
  THClTensor_narrow(state, self, nullptr, dimension, firstIndex, size);
  return self;
  THCL_END(nullptr)
}
THClTensor* THClTensor_newTranspose(THClState* state, THClTensor* tensor, int dimension1, int dimension2) {
  THCL_BEGIN
  THClTensor* self = THClTensor_newWithTensor(state, tensor);
  THClTensor_transpose(state, self, nullptr, dimension1, dimension2);
  return self;
  THCL_END(nullptr)
}
THClTensor* THClTensor_newUnfold(THClState* state, THClTensor* tensor, int dimension, long size, long step) {
  THCL_BEGIN
  THClTensor* self = THClTensor_newWithTensor(state, tensor);
  THClTensor_unfold(state, self, nullptr, dimension, size, step);
  return self;
  THCL_END(nullptr)
}

void THClTensor_resize(THClState* state, THClTensor* self, THLongStorage* size, THLongStorage* stride) {
  THCL_BEGIN
  arg_check(size != nullptr, 2, "invalid size");
  if (stride) arg_check(stride->size == size->size, 3, "invalid stride");
  raw_resize(state, self, (int)size->size, size->data, stride ? stride->data : nullptr);
  THCL_END_VOID
}

void THClTensor_resizeAs(THClState* state, THClTensor* self, THClTensor* src) {
  THCL_BEGIN
  bool same = self->nDimension == src->nDimension;
  for (int d = 0; same && d < self->nDimension; ++d) same = self->size[d] == src->size[d];
  if (!same) raw_resize(state, self, src->nDimension, src->size, nullptr);
  THCL_END_VOID
}

void THClTensor_resize5d(THClState* state, THClTensor* self, long size0, long size1, long size2, long size3, long size4) {
  THCL_BEGIN
  long size[5] = {size0, size1, size2, size3, size4};
  raw_resize(state, self, 5, size, nullptr);
  THCL_END_VOID
}
void THClTensor_resize4d(THClState* state, THClTensor* self, long size0, long size1, long size2, long size3) {
  THClTensor_resize5d(state, self, size0, size1, size2, size3, -1);
}
void THClTensor_resize0d(THClState* state, THClTensor* self) { THClTensor_resize5d(state, self, -1, -1, -1, -1, -1); }
void THClTensor_resize1d(THClState* state, THClTensor* self, long size0) { THClTensor_resize5d(state, self, size0, -1, -1, -1, -1); }
void THClTensor_resize2d(THClState* state, THClTensor* self, long size0, long size1) { THClTensor_resize5d(state, self, size0, size1, -1, -1, -1); }
void THClTensor_resize3d(THClState* state, THClTensor* self, long size0, long size1, long size2) { THClTensor_resize5d(state, self, size0, size1, size2, -1, -1); }

void THClTensor_set(THClState* state, THClTensor* self, THClTensor* src) {
  THCL_BEGIN
  if (self != src) raw_set(state, self, src->storage, src->storageOffset, src->nDimension, src->size, src->stride);
  THCL_END_VOID
}

void THClTensor_setStorage(THClState* state, THClTensor* self, THClStorage* storage, long storageOffset,
                           THLongStorage* size, THLongStorage* stride) {
  THCL_BEGIN
  if (size && stride) arg_check(size->size == stride->size, 5, "inconsistent size/stride sizes");
  raw_set(state, self, storage, storageOffset, (int)(size ? size->size : (stride ? stride->size : 0)),
          size ? size->data : nullptr, stride ? stride->data : nullptr);
  THCL_END_VOID
}
void THClTensor_setStorage4d(THClState* state, THClTensor* self, THClStorage* storage, long storageOffset, long size0,
                             long stride0, long size1, long stride1, long size2, long stride2, long size3, long stride3) {
  THCL_BEGIN
  long size[4] = {size0, size1, size2, size3};
  long stride[4] = {stride0, stride1, stride2, stride3};
  raw_set(state, self, storage, storageOffset, 4, size, stride);
  THCL_END_VOID
}
void THClTensor_setStorage1d(THClState* state, THClTensor* self, THClStorage* storage, long storageOffset, long size0, long stride0) {
  THClTensor_setStorage4d(state, self, storage, storageOffset, size0, stride0, -1, -1, -1, -1, -1, -1);
}
void THClTensor_setStorage2d(THClState* state, THClTensor* self, THClStorage* storage, long storageOffset, long size0, long stride0, long size1, long stride1) {
  THClTensor_setStorage4d(state, self, storage, storageOffset, size0, stride0, size1, stride1, -1, -1, -1, -1);
}
void THClTensor_setStorage3d(THClState* state, THClTensor* self, THClStorage* storage, long storageOffset, long size0, long stride0, long size1, long stride1, long size2, long stride2) {
  THClTensor_setStorage4d(state, self, storage, storageOffset, size0, stride0, size1, stride1, size2, stride2, -1, -1);
}

void THClTensor_narrow(THClState* state, THClTensor* self, THClTensor* src, int dimension, long firstIndex, long size) {
  THCL_BEGIN
  if (!src) src = self;
  arg_check(dimension >= 0 && dimension < src->nDimension, 3, "out of range");
  arg_check(firstIndex >= 0 && firstIndex < src->size[dimension], 4, "out of range");
  arg_check(size > 0 && firstIndex + size <= src->size[dimension], 5, "out of range");
  THClTensor_set(state, self, src);
  if (firstIndex > 0) self->storageOffset += firstIndex * self->stride[dimension];
  self->size[dimension] = size;
  THCL_END_VOID
}

void THClTensor_select(THClState* state, THClTensor* self, THClTensor* src, int dimension, long sliceIndex) {
  THCL_BEGIN
  if (!src) src = self;
  arg_check(src->nDimension > 1, 1, "cannot select on a vector");
  arg_check(dimension >= 0 && dimension < src->nDimension, 3, "out of range");
  arg_check(sliceIndex >= 0 && sliceIndex < src->size[dimension], 4, "out of range");
  THClTensor_set(state, self, src);
  THClTensor_narrow(state, self, nullptr, dimension, sliceIndex, 1);
  for (int d = dimension; d < self->nDimension - 1; ++d) {
    self->size[d] = self->size[d + 1];
    self->stride[d] = self->stride[d + 1];
  }
  self->nDimension--;
  THCL_END_VOID
}

void THClTensor_transpose(THClState* state, THClTensor* self, THClTensor* src, int dimension1, int dimension2) {
  THCL_BEGIN
  if (!src) src = self;
  arg_check(dimension1 >= 0 && dimension1 < src->nDimension, 1, "out of range");
  arg_check(dimension2 >= 0 && dimension2 < src->nDimension, 2, "out of range");
  THClTensor_set(state, self, src);
  if (dimension1 == dimension2) return;
  long z = self->stride[dimension1];
  self->stride[dimension1] = self->stride[dimension2];
  self->stride[dimension2] = z;
  z = self->size[dimension1];
  self->size[dimension1] = self->size[dimension2];
  self->size[dimension2] = z;
  THCL_END_VOID
}

void THClTensor_unfold(THClState* state, THClTensor* self, THClTensor* src, int dimension, long size, long step) {
  THCL_BEGIN
  if (!src) src = self;
  arg_check(src->nDimension > 0, 1, "cannot unfold an empty tensor");
  arg_check(dimension >= 0 && dimension < src->nDimension, 2, "out of range");
  arg_check(size <= src->size[dimension], 3, "out of range");
  arg_check(step > 0, 4, "invalid step");
  THClTensor_set(state, self, src);
  const int nd = self->nDimension;
  long* newSize = (long*)malloc(sizeof(long) * (nd + 1));
  long* newStride = (long*)malloc(sizeof(long) * (nd + 1));
  newSize[nd] = size;
  newStride[nd] = self->stride[dimension];
  for (int d = 0; d < nd; ++d) {
    if (d == dimension) {
      newSize[d] = (self->size[d] - size) / step + 1;
      newStride[d] = step * self->stride[d];
    } else {
      newSize[d] = self->size[d];
      newStride[d] = self->stride[d];
    }
  }
  free(self->size);
  free(self->stride);
  self->size = newSize;
  self->stride = newStride;
  self->nDimension = nd + 1;
  THCL_END_VOID
}

void THClTensor_squeeze(THClState* state, THClTensor* self, THClTensor* src) {
  THCL_BEGIN
  if (!src) src = self;
  THClTensor_set(state, self, src);
  int nd = 0;
  for (int d = 0; d < src->nDimension; ++d) {
    if (src->size[d] != 1) {
      if (d != nd) {
        self->size[nd] = src->size[d];
        self->stride[nd] = src->stride[d];
      }
      ++nd;
    }
  }
  if (nd == 0 && src->nDimension > 0) {  // all dims were 1: keep one
    self->size[0] = 1;
    self->stride[0] = 1;
    nd = 1;
  }
  self->nDimension = nd;
  THCL_END_VOID
}

void THClTensor_squeeze1d(THClState* state, THClTensor* self, THClTensor* src, int dimension) {
  THCL_BEGIN
  if (!src) src = self;
  arg_check(dimension >= 0 && dimension < src->nDimension, 3, "dimension out of range");
  THClTensor_set(state, self, src);
  if (src->size[dimension] == 1 && src->nDimension > 1) {
    for (int d = dimension; d < self->nDimension - 1; ++d) {
      self->size[d] = self->size[d + 1];
      self->stride[d] = self->stride[d + 1];
    }
    self->nDimension--;
  }
  THCL_END_VOID
}

int THClTensor_isContiguous(THClState*, const THClTensor* self) {
  long z = 1;
  for (int d = self->nDimension - 1; d >= 0; --d) {
    if (self->size[d] != 1) {
      if (self->stride[d] == z) z *= self->size[d];
      else return 0;
    }
  }
  return 1;
}

int THClTensor_isSameSizeAs(THClState*, const THClTensor* self, const THClTensor* src) {
  if (self->nDimension != src->nDimension) return 0;
  for (int d = 0; d < self->nDimension; ++d)
    if (self->size[d] != src->size[d]) return 0;
  return 1;
}

long THClTensor_nElement(THClState*, const THClTensor* self) {
  if (self->nDimension <= 0) return 0;
  long n = 1;
  for (int d = 0; d < self->nDimension; ++d) n *= self->size[d];
  return n;
}

void THClTensor_retain(THClState*, THClTensor* self) {
  if (self->flag & TH_TENSOR_REFCOUNTED) __sync_add_and_fetch(&self->refcount, 1);
}

void THClTensor_free(THClState* state, THClTensor* self) {
  THCL_BEGIN
  if (!self || !(self->flag & TH_TENSOR_REFCOUNTED)) return;
  if (__sync_sub_and_fetch(&self->refcount, 1) == 0) {
    free(self->size);
    free(self->stride);
    if (self->storage) THClStorage_free(state, self->storage);
    free(self);
  }
  THCL_END_VOID
}

void THClTensor_freeCopyTo(THClState* state, THClTensor* self, THClTensor* dst) {
  THCL_BEGIN
  if (self != dst) THClTensor_copy(state, dst, self);
  THClTensor_free(state, self);
  THCL_END_VOID
}

static long element_offset(const THClTensor* t, int n, const long* x) {
  check_index(t, n, x);
  long off = t->storageOffset;
  for (int d = 0; d < n; ++d) off += x[d] * t->stride[d];
  return off;
}

void THClTensor_set1d(THClState* state, THClTensor* t, long x0, float value) {
  THCL_BEGIN
  long x[1] = {x0};
  THClStorage_set(state, t->storage, element_offset(t, 1, x), value);
  THCL_END_VOID
}
void THClTensor_set2d(THClState* state, THClTensor* t, long x0, long x1, float value) {
  THCL_BEGIN
  long x[2] = {x0, x1};
  THClStorage_set(state, t->storage, element_offset(t, 2, x), value);
  THCL_END_VOID
}
void THClTensor_set3d(THClState* state, THClTensor* t, long x0, long x1, long x2, float value) {
  THCL_BEGIN
  long x[3] = {x0, x1, x2};
  THClStorage_set(state, t->storage, element_offset(t, 3, x), value);
  THCL_END_VOID
}
void THClTensor_set4d(THClState* state, THClTensor* t, long x0, long x1, long x2, long x3, float value) {
  THCL_BEGIN
  long x[4] = {x0, x1, x2, x3};
  THClStorage_set(state, t->storage, element_offset(t, 4, x), value);
  THCL_END_VOID
}
float THClTensor_get1d(THClState* state, const THClTensor* t, long x0) {
  THCL_BEGIN
  long x[1] = {x0};
  return THClStorage_get(state, t->storage, element_offset(t, 1, x));
  THCL_END(0.f)
}
float THClTensor_get2d(THClState* state, const THClTensor* t, long x0, long x1) {
  THCL_BEGIN
  long x[2] = {x0, x1};
  return THClStorage_get(state, t->storage, element_offset(t, 2, x));
  THCL_END(0.f)
}
float THClTensor_get3d(THClState* state, const THClTensor* t, long x0, long x1, long x2) {
  THCL_BEGIN
  long x[3] = {x0, x1, x2};
  return THClStorage_get(state, t->storage, element_offset(t, 3, x));
  THCL_END(0.f)
}
float THClTensor_get4d(THClState* state, const THClTensor* t, long x0, long x1, long x2, long x3) {
  THCL_BEGIN
  long x[4] = {x0, x1, x2, x3};
  return THClStorage_get(state, t->storage, element_offset(t, 4, x));
  THCL_END(0.f)
}

int THClTensor_getDevice(THClState*, const THClTensor* self) { return self->device; }

// All operands on one device (reference src/lib/THClTensor.cpp:844-873).
int THClTensor_checkGPU(THClState*, unsigned int nTensors, ...) {
  va_list args;
  va_start(args, nTensors);
  int device = -1, ok = 1;
  for (unsigned int i = 0; i < nTensors; ++i) {
    THClTensor* t = va_arg(args, THClTensor*);
    if (!t) continue;
    if (device == -1) device = t->device;
    else if (t->device != device) ok = 0;
  }
  va_end(args);
  return ok;
}

}  // extern "C"
