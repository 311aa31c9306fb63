// Module table of the Lua package `cltorch`, written against libthb200.so.
//
// Not built in this repository (it needs lua.h / luaT.h / TH.h of a Torch7 tree). It keeps the
// function names of the `cltorch` table of cltorch (reference src/init.cpp:207-226) so that
// scripts run unchanged; bodies call include/THCl.h and include/thb200.h. Entries that only
// made sense for OpenCL (setAllowNonGpus, setDetailedTimings) are accepted and ignored.
extern "C" {
#include "lua.h"
#include "lauxlib.h"
#include "luaT.h"
}
#include <cuda_runtime.h>
#include <cstdlib>
#include <string>
#include <vector>

#include "THCl.h"
#include "thb200.h"

// registered by the unchanged binding sources (Storage.cpp, Tensor.cpp, generated TensorMath.c, ...)
extern "C" {
void cltorch_ClStorage_init(lua_State* L);
void cltorch_ClTensor_init(lua_State* L);
void cltorch_ClTensorMath_init(lua_State* L);
void cltorch_ClTensorOperator_init(lua_State* L);
void cltorch_UserKernel_init(lua_State* L);
}

namespace {

THClState* state_of(lua_State* L) {
  lua_getglobal(L, "cltorch");
  lua_getfield(L, -1, "_state");
  THClState* s = (THClState*)lua_touserdata(L, -1);
  lua_pop(L, 2);
  return s;
}

// The library reports errors through a handler; raising a Lua error from it unwinds like THError does.
void raise_lua_error(const char* msg, void* L) { luaL_error((lua_State*)L, "%s", msg); }

int l_get_device_count(lua_State* L) {
  lua_pushinteger(L, THClState_getNumDevices(state_of(L)));
  return 1;
}
int l_get_device(lua_State* L) {
  lua_pushinteger(L, THClState_getDevice(state_of(L)) + 1);     // Lua counts from 1
  return 1;
}
int l_set_device(lua_State* L) {
  THClState_setDevice(state_of(L), (int)luaL_checkinteger(L, 1) - 1);
  return 0;
}
int l_synchronize(lua_State* L) {
  THClSynchronize(state_of(L));
  return 0;
}
int l_set_trace(lua_State* L) {
  state_of(L)->trace = (int)luaL_checkinteger(L, 1);
  return 0;
}
int l_set_add_finish(lua_State* L) {
  state_of(L)->addFinish = (int)luaL_checkinteger(L, 1);
  return 0;
}
int l_ignored(lua_State*) { return 0; }

// setProfiling / setEnableTiming -> device time per library call; dumpProfiling / dumpTimings print it
int l_set_profiling(lua_State* L) {
  thb200_timing_enable((int)luaL_checkinteger(L, 1));
  return 0;
}
int l_dump_profiling(lua_State* L) {
  std::vector<char> text(thb200_timing_report(nullptr, 0) + 4096);
  thb200_timing_report(text.data(), text.size());
  thb200_timing_reset();
  printf("entry point, calls, device milliseconds\n%s", text.data());
  lua_pushstring(L, text.data());
  return 1;
}

void set_number(lua_State* L, const char* key, double v) {
  lua_pushnumber(L, v);
  lua_setfield(L, -2, key);
}
int l_get_device_properties(lua_State* L) {
  const int device = (int)luaL_checkinteger(L, 1) - 1;
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, device) != cudaSuccess) return luaL_error(L, "no such device: %d", device + 1);
  lua_newtable(L);
  lua_pushstring(L, "GPU");
  lua_setfield(L, -2, "deviceType");
  lua_pushstring(L, p.name);
  lua_setfield(L, -2, "deviceName");
  set_number(L, "globalMemSizeMB", (double)(p.totalGlobalMem >> 20));
  set_number(L, "localMemSizeKB", (double)(p.sharedMemPerBlockOptin >> 10));
  set_number(L, "maxComputeUnits", p.multiProcessorCount);
  set_number(L, "maxWorkGroupSize", p.maxThreadsPerBlock);
  set_number(L, "maxClockFrequency", p.clockRate / 1000.0);
  set_number(L, "computeCapability", p.major * 10 + p.minor);
  return 1;
}
int l_get_state(lua_State* L) {
  lua_getglobal(L, "cltorch");
  lua_getfield(L, -1, "_state");
  lua_remove(L, -2);
  return 1;
}
int l_about(lua_State*) {
  printf("cltorch on libthb200: CUDA kernels for sm_100a behind the THCl C API\n");
  return 0;
}

const luaL_Reg kTable[] = {
    {"getDeviceCount", l_get_device_count}, {"getDevice", l_get_device}, {"setDevice", l_set_device},
    {"synchronize", l_synchronize}, {"finish", l_synchronize}, {"getDeviceProperties", l_get_device_properties},
    {"getState", l_get_state}, {"setTrace", l_set_trace}, {"setAddFinish", l_set_add_finish},
    {"setProfiling", l_set_profiling}, {"setEnableTiming", l_set_profiling}, {"setTiming", l_set_profiling},
    {"dumpProfiling", l_dump_profiling}, {"dumpTimings", l_dump_profiling},
    {"setAllowNonGpus", l_ignored}, {"setDetailedTimings", l_ignored}, {"about", l_about}, {NULL, NULL}};

}  // namespace

extern "C" int luaopen_libcltorch(lua_State* L) {
  lua_newtable(L);
  luaL_setfuncs(L, kTable, 0);
  THClState* state = (THClState*)malloc(sizeof(THClState));
  THClInit(state);
  THClSetErrorHandler(raise_lua_error, L);
  cltorch_ClStorage_init(L);
  cltorch_ClTensor_init(L);
  cltorch_ClTensorMath_init(L);
  cltorch_ClTensorOperator_init(L);
  cltorch_UserKernel_init(L);
  lua_pushlightuserdata(L, state);
  lua_setfield(L, -2, "_state");
  return 1;
}
