// Run-time bindings to the CUDA driver, NVRTC and NCCL.  The libraries are opened with
// dlopen so that the backend's shared object loads (and its symbols can be inspected, and
// routines can be compiled to sm_100a machine code) on a machine without a GPU driver.
#pragma once
#include <cuda.h>
#include <nccl.h>
#include <nvrtc.h>

#include <string>

#include "ir.hpp"

namespace b200 {

#define B200_CU_FUNCS(X)                                                                                              \
  X(cuInit) X(cuDeviceGetCount) X(cuDeviceGet) X(cuDeviceGetName) X(cuDeviceGetAttribute) X(cuDeviceTotalMem)         \
  X(cuDevicePrimaryCtxRetain) X(cuCtxSetCurrent) X(cuStreamCreate) X(cuStreamSynchronize) X(cuStreamQuery)            \
  X(cuStreamWaitEvent) X(cuMemAlloc) X(cuMemFree) X(cuMemsetD8Async) X(cuMemcpyHtoDAsync) X(cuMemcpyDtoHAsync)         \
  X(cuMemcpyDtoDAsync) X(cuMemcpyPeerAsync) X(cuMemHostAlloc) X(cuMemFreeHost) X(cuMemHostGetDevicePointer)            \
  X(cuMemGetInfo) X(cuEventCreate) X(cuEventRecord) X(cuEventQuery) X(cuEventSynchronize) X(cuEventDestroy)            \
  X(cuEventElapsedTime) X(cuModuleLoadData) X(cuModuleUnload) X(cuModuleGetFunction) X(cuLaunchKernel)                 \
  X(cuFuncSetAttribute) X(cuFuncGetAttribute) X(cuGetErrorString) X(cuTensorMapEncodeTiled) X(cuStreamBeginCapture)    \
  X(cuStreamEndCapture) X(cuGraphInstantiateWithFlags) X(cuGraphLaunch) X(cuGraphExecDestroy) X(cuGraphDestroy)        \
  X(cuDeviceCanAccessPeer) X(cuCtxEnablePeerAccess) X(cuModuleGetGlobal) X(cuLaunchKernelEx) X(cuOccupancyMaxActiveClusters) X(cuStreamDestroy)

#define B200_NVRTC_FUNCS(X)                                                                                  \
  X(nvrtcCreateProgram) X(nvrtcCompileProgram) X(nvrtcDestroyProgram) X(nvrtcGetCUBINSize) X(nvrtcGetCUBIN)  \
  X(nvrtcGetProgramLogSize) X(nvrtcGetProgramLog) X(nvrtcGetErrorString) X(nvrtcVersion)

#define B200_NCCL_FUNCS(X)                                                                              \
  X(ncclGetUniqueId) X(ncclCommInitRank) X(ncclCommDestroy) X(ncclAllReduce) X(ncclGetErrorString)      \
  X(ncclCommAbort) X(ncclCommGetAsyncError) X(ncclCommInitAll) X(ncclGroupStart) X(ncclGroupEnd)

struct CuApi {
#define X(name) decltype(&::name) name##_ = nullptr;
  B200_CU_FUNCS(X)
#undef X
  bool loaded = false;
  std::string why;
};
struct NvrtcApi {
#define X(name) decltype(&::name) name##_ = nullptr;
  B200_NVRTC_FUNCS(X)
#undef X
  bool loaded = false;
  std::string why;
};
struct NcclApi {
#define X(name) decltype(&::name) name##_ = nullptr;
  B200_NCCL_FUNCS(X)
#undef X
  bool loaded = false;
  std::string why;
};

CuApi& cu();        // loads libcuda.so.1 on first use; `loaded` false when unavailable
NvrtcApi& nvrtc();  // loads libnvrtc.so.12
NcclApi& nccl();    // loads libnccl.so.2

void cu_check(CUresult r, const char* what);  // throws Error(positive code)

// Compiles one translation unit to sm_100a machine code (cached by source text).
// Throws Error(-2) when NVRTC is unavailable and Error(positive) with the log on failure.
const std::string& compile_cubin(const std::string& source, const std::string& name, std::string* log = nullptr);

}  // namespace b200
