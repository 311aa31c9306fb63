// THClStorage: a refcounted block of fp32 device memory
// (reference src/lib/THClStorage.cpp, src/lib/THClStorageCopy.cpp).
//
// The reference keeps a host mirror and a dirty flag per storage and moves the
// whole buffer on every host access; here the memory lives in HBM only and is
// allocated from the CUDA stream-ordered pool on the device's stream, so that
// temporaries can be freed without a device-wide synchronisation.
#include "thcl_internal.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>

using namespace thcl;

// Minimal stand-ins for the two THLongStorage functions the API hands out
// objects of; weak, so libTH's definitions win when it is loaded.
extern "C" __attribute__((weak)) THLongStorage* THLongStorage_newWithSize(long size) {
  THLongStorage* s = (THLongStorage*)calloc(1, sizeof(THLongStorage));
  s->data = (long*)calloc(size > 0 ? size : 1, sizeof(long));
  s->size = size;
  s->refcount = 1;
  s->flag = TH_STORAGE_REFCOUNTED | TH_STORAGE_RESIZABLE | TH_STORAGE_FREEMEM;
  return s;
}
extern "C" __attribute__((weak)) void THLongStorage_free(THLongStorage* s) {
  if (!s) return;
  if (__sync_sub_and_fetch(&s->refcount, 1) == 0) {
    free(s->data);
    free(s);
  }
}

static void storage_alloc(THClState* state, THClStorage* s, long size) {
  THClDeviceContext* ctx = context(state, s->device);
  use_device(s->device);
  float* p = nullptr;
  check_cuda(cudaMallocAsync((void**)&p, (size_t)size * sizeof(float), ctx->stream), "cudaMallocAsync(storage)");
  if (state->trace) printf("THCl: alloc %ld floats on device %d -> %p\n", size, s->device, (void*)p);
  s->wrapper = p;
  s->cl = ctx;
  s->size = size;
}

static void storage_release(THClState* state, THClStorage* s) {
  if (s->wrapper && (s->flag & TH_STORAGE_FREEMEM)) {
    THClDeviceContext* ctx = context(state, s->device);
    use_device(s->device);
    if (state->trace) printf("THCl: free %ld floats on device %d (%p)\n", s->size, s->device, (void*)s->wrapper);
    check_cuda(cudaFreeAsync(s->wrapper, ctx->stream), "cudaFreeAsync(storage)");
  }
  s->wrapper = nullptr;
  s->size = 0;
}

extern "C" {

float* THClStorage_data(THClState*, const THClStorage* self) { return self->data; }
long THClStorage_size(THClState*, const THClStorage* self) { return self->size; }

THClStorage* THClStorage_newv2(THClState* state, int device) {
  THCL_BEGIN
  if (!state->initialized) THCl_initializeState(state);
  THClStorage* s = (THClStorage*)calloc(1, sizeof(THClStorage));
  s->device = device;
  s->refcount = 1;
  s->flag = TH_STORAGE_REFCOUNTED | TH_STORAGE_RESIZABLE | TH_STORAGE_FREEMEM;
  return s;
  THCL_END(nullptr)
}

THClStorage* THClStorage_new(THClState* state) { return THClStorage_newv2(state, state->currentDevice); }

THClStorage* THClStorage_newWithSize(THClState* state, int device, long size) {
  THCL_BEGIN
  arg_check(size >= 0, 2, "invalid size");
  THClStorage* s = THClStorage_newv2(state, device);
  if (size > 0) {
    try {
      storage_alloc(state, s, size);
    } catch (...) {
      free(s);
      throw;
    }
  }
  return s;
  THCL_END(nullptr)
}

static THClStorage* new_with_values(THClState* state, int device, const float* v, int n) {
  THClStorage* s = THClStorage_newWithSize(state, device, n);
  THClDeviceContext* ctx = context(state, device);
  check_cuda(cudaMemcpyAsync(s->wrapper, v, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream), "cudaMemcpyAsync");
  sync_stream(ctx);  // `v` is on the caller's stack
  return s;
}

THClStorage* THClStorage_newWithSize1(THClState* state, int device, float a) {
  THCL_BEGIN
  float v[1] = {a};
  return new_with_values(state, device, v, 1);
  THCL_END(nullptr)
}
THClStorage* THClStorage_newWithSize2(THClState* state, int device, float a, float b) {
  THCL_BEGIN
  float v[2] = {a, b};
  return new_with_values(state, device, v, 2);
  THCL_END(nullptr)
}
THClStorage* THClStorage_newWithSize3(THClState* state, int device, float a, float b, float c) {
  THCL_BEGIN
  float v[3] = {a, b, c};
  return new_with_values(state, device, v, 3);
  THCL_END(nullptr)
}
THClStorage* THClStorage_newWithSize4(THClState* state, int device, float a, float b, float c, float d) {
  THCL_BEGIN
  float v[4] = {a, b, c, d};
  return new_with_values(state, device, v, 4);
  THCL_END(nullptr)
}

THClStorage* THClStorage_newWithData(THClState* state, int device, float* data, long size) {
  THCL_BEGIN
  THClStorage* s = THClStorage_newWithSize(state, device, size);
  if (size > 0) {
    THClDeviceContext* ctx = context(state, device);
    check_cuda(cudaMemcpyAsync(s->wrapper, data, (size_t)size * sizeof(float), cudaMemcpyHostToDevice, ctx->stream), "cudaMemcpyAsync");
    sync_stream(ctx);
  }
  free(data);
  return s;
  THCL_END(nullptr)
}

THClStorage* THClStorage_newWithDevicePointer(THClState* state, int device, float* devptr, long size) {
  THCL_BEGIN
  arg_check(size >= 0, 4, "invalid size");
  THClStorage* s = THClStorage_newv2(state, device);
  s->flag = TH_STORAGE_REFCOUNTED;  // neither resizable nor freed
  s->wrapper = devptr;
  s->size = size;
  return s;
  THCL_END(nullptr)
}

void THClStorage_setFlag(THClState*, THClStorage* s, const char flag) { s->flag |= flag; }
void THClStorage_clearFlag(THClState*, THClStorage* s, const char flag) { s->flag &= ~flag; }

void THClStorage_retain(THClState*, THClStorage* s) {
  if (s && (s->flag & TH_STORAGE_REFCOUNTED)) __sync_add_and_fetch(&s->refcount, 1);
}

void THClStorage_free(THClState* state, THClStorage* s) {
  THCL_BEGIN
  if (!s || !(s->flag & TH_STORAGE_REFCOUNTED)) return;
  if (__sync_sub_and_fetch(&s->refcount, 1) == 0) {
    storage_release(state, s);
    free(s);
  }
  THCL_END_VOID
}

void THClStorage_resize(THClState* state, THClStorage* s, long size) {
  THCL_BEGIN
  arg_check(size >= 0, 2, "invalid size");
  if (!(s->flag & TH_STORAGE_RESIZABLE)) raise("Trying to resize storage that is not resizable");
  if (size <= s->size) return;  // grows only
  storage_release(state, s);
  storage_alloc(state, s, size);
  THCL_END_VOID
}

void THClStorage_fill(THClState* state, THClStorage* s, float value) {
  THCL_BEGIN
  if (s->size == 0) return;
  THClDeviceContext* ctx = context(state, s->device);
  use_device(s->device);
  int64_t size = s->size, stride = 1;
  thb200_tensor t{s->wrapper, 1, &size, &stride};
  check_thb(thb200_apply_op(ctx->stream, thb200_op_code("FILL_1"), 1, &t, value, 0.f, nullptr, nullptr));
  after_launch(state, ctx);
  THCL_END_VOID
}

void THClStorage_set(THClState* state, THClStorage* s, long index, float value) {
  THCL_BEGIN
  arg_check(index >= 0 && index < s->size, 2, "index out of bounds");
  THClDeviceContext* ctx = context(state, s->device);
  use_device(s->device);
  int64_t size = 1, stride = 1;
  thb200_tensor t{s->wrapper + index, 1, &size, &stride};
  check_thb(thb200_apply_op(ctx->stream, thb200_op_code("FILL_1"), 1, &t, value, 0.f, nullptr, nullptr));
  after_launch(state, ctx);
  THCL_END_VOID
}

float THClStorage_get(THClState* state, const THClStorage* s, long index) {
  THCL_BEGIN
  arg_check(index >= 0 && index < s->size, 2, "index out of bounds");
  THClDeviceContext* ctx = context(state, s->device);
  use_device(s->device);
  check_cuda(cudaMemcpyAsync(ctx->result_host + 32, s->wrapper + index, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream), "cudaMemcpyAsync");
  sync_stream(ctx);
  return ctx->result_host[32];
  THCL_END(0.f)
}

void THClStorage_rawCopy(THClState* state, THClStorage* self, float* src) {
  THCL_BEGIN
  if (self->size == 0) return;
  THClDeviceContext* ctx = context(state, self->device);
  use_device(self->device);
  if (state->trace) printf("THCl: host -> device %ld floats\n", self->size);
  check_cuda(cudaMemcpyAsync(self->wrapper, src, (size_t)self->size * sizeof(float), cudaMemcpyHostToDevice, ctx->stream), "cudaMemcpyAsync");
  sync_stream(ctx);
  THCL_END_VOID
}

void THClStorage_copy(THClState* state, THClStorage* self, THClStorage* src) {
  THCL_BEGIN
  arg_check(self->size == src->size, 2, "size does not match");
  if (self->size == 0) return;
  THClDeviceContext* ctx = context(state, self->device);
  use_device(self->device);
  check_cuda(cudaMemcpyAsync(self->wrapper, src->wrapper, (size_t)self->size * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream), "cudaMemcpyAsync");
  THCL_END_VOID
}

void THClStorage_copyCl(THClState* state, THClStorage* self, THClStorage* src) { THClStorage_copy(state, self, src); }

void THClStorage_copyFloat(THClState* state, THClStorage* self, struct THFloatStorage* src) {
  THCL_BEGIN
  arg_check(self->size == src->size, 2, "size does not match");
  THClStorage_rawCopy(state, self, src->data);
  THCL_END_VOID
}

void THFloatStorage_copyCl(THClState* state, struct THFloatStorage* self, struct THClStorage* src) {
  THCL_BEGIN
  arg_check(self->size == src->size, 2, "size does not match");
  if (src->size == 0) return;
  THClDeviceContext* ctx = context(state, src->device);
  use_device(src->device);
  if (state->trace) printf("THCl: device -> host %ld floats\n", src->size);
  check_cuda(cudaMemcpyAsync(self->data, src->wrapper, (size_t)src->size * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream), "cudaMemcpyAsync");
  sync_stream(ctx);
  THCL_END_VOID
}

}  // extern "C"
