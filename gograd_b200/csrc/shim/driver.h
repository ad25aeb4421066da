// CUDA driver API, bound at run time with dlopen("libcuda.so.1"): the library has no
// link-time dependency on the driver, so it loads (and every symbol resolves) on a
// machine without a GPU, and fails with a clear message only when a device call is made.
// The reference binds its NVIDIA libraries the same lazy way (cuda/cuda_windows.go:136-195).
#ifndef OE_DRIVER_H
#define OE_DRIVER_H

#include <cuda.h>

#define OE_DRIVER_FUNCS(X)                   \
    X(cuInit)                                \
    X(cuDriverGetVersion)                    \
    X(cuDeviceGet)                           \
    X(cuDeviceGetCount)                      \
    X(cuDeviceGetAttribute)                  \
    X(cuDeviceGetName)                       \
    X(cuDevicePrimaryCtxRetain)              \
    X(cuDevicePrimaryCtxRelease)             \
    X(cuCtxPushCurrent)                      \
    X(cuCtxPopCurrent)                       \
    X(cuCtxGetCurrent)                       \
    X(cuModuleLoadData)                      \
    X(cuModuleUnload)                        \
    X(cuModuleGetFunction)                   \
    X(cuFuncGetAttribute)                    \
    X(cuOccupancyMaxActiveBlocksPerMultiprocessor) \
    X(cuLaunchKernel)                        \
    X(cuMemAlloc)                            \
    X(cuMemFree)                             \
    X(cuMemAllocHost)                        \
    X(cuMemFreeHost)                         \
    X(cuMemHostRegister)                     \
    X(cuMemHostUnregister)                   \
    X(cuMemcpyHtoDAsync)                     \
    X(cuMemcpyDtoHAsync)                     \
    X(cuMemcpyDtoDAsync)                     \
    X(cuMemcpyAsync)                         \
    X(cuMemsetD32Async)                      \
    X(cuMemsetD8Async)                       \
    X(cuMemGetInfo)                          \
    X(cuMemGetAddressRange)                  \
    X(cuStreamCreate)                        \
    X(cuStreamDestroy)                       \
    X(cuStreamSynchronize)                   \
    X(cuStreamWaitEvent)                     \
    X(cuStreamIsCapturing)                   \
    X(cuEventCreate)                         \
    X(cuEventDestroy)                        \
    X(cuEventRecord)                         \
    X(cuEventSynchronize)                    \
    X(cuEventQuery)                          \
    X(cuEventElapsedTime)                    \
    X(cuIpcGetMemHandle)                     \
    X(cuIpcOpenMemHandle)                    \
    X(cuIpcCloseMemHandle)                   \
    X(cuDeviceCanAccessPeer)                 \
    X(cuCtxEnablePeerAccess)                 \
    X(cuGetErrorString)                      \
    X(cuGetErrorName)

struct oe_driver {
#define OE_DECL(name) decltype(&name) name##_;
    OE_DRIVER_FUNCS(OE_DECL)
#undef OE_DECL
};

// Loads libcuda once per process and calls cuInit(0). Returns nullptr and sets *why
// (a static string or a dlerror text) when the driver is not available.
const oe_driver* oe_driver_get(const char** why);

#endif
