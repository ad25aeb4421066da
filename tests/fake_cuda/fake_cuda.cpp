// A stand-in for libcuda.so.1 that runs on a machine without a GPU (test infrastructure).
//
// liboptengine.so binds the CUDA driver at run time; pointed at this library (environment
// variable OE_CUDA_DRIVER_LIBRARY) its host logic can be exercised on the CPU: "device memory"
// is host memory, copies are memcpy, kernels are not executed but every launch is recorded
// (kernel name, grid, block), and any driver entry point can be told to fail on its n-th call.
// Nothing here computes an optimizer step: parity is never checked through this library.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace {
std::mutex g_mu;
struct Fail {
    int countdown;  // fails when it reaches 0
    int code;
    bool sticky;    // keeps failing afterwards
};
std::map<std::string, Fail> g_fail;
std::map<std::string, long> g_calls;
struct Launch {
    std::string name;
    unsigned grid, block;
};
std::vector<Launch> g_launches;
std::map<void*, size_t> g_device_allocs;
size_t g_device_bytes = 0;
struct FakeFunction {
    std::string name;
};
std::map<std::string, FakeFunction*> g_functions;
int g_cc_major = 10, g_cc_minor = 0, g_sms = 148;

CUresult enter(const char* api) {
    std::lock_guard<std::mutex> lock(g_mu);
    g_calls[api]++;
    auto it = g_fail.find(api);
    if (it == g_fail.end()) return CUDA_SUCCESS;
    if (it->second.countdown > 0) {
        it->second.countdown--;
        return CUDA_SUCCESS;
    }
    CUresult r = (CUresult)it->second.code;
    if (!it->second.sticky) g_fail.erase(it);
    return r;
}
#define ENTER(api)                            \
    do {                                      \
        CUresult fake_r_ = enter(api);        \
        if (fake_r_ != CUDA_SUCCESS) return fake_r_; \
    } while (0)
}  // namespace

extern "C" {

// ---- controls for the tests ----------------------------------------------------------------
// The call number `after` + 1 of `api` (counted from now) fails with `code`; sticky keeps it failing.
void fake_cuda_fail(const char* api, int after, int code, int sticky) {
    std::lock_guard<std::mutex> lock(g_mu);
    g_fail[api] = Fail{after, code, sticky != 0};
}
void fake_cuda_clear_failures(void) {
    std::lock_guard<std::mutex> lock(g_mu);
    g_fail.clear();
}
long fake_cuda_calls(const char* api) {
    std::lock_guard<std::mutex> lock(g_mu);
    return g_calls[api];
}
int fake_cuda_launch_count(void) {
    std::lock_guard<std::mutex> lock(g_mu);
    return (int)g_launches.size();
}
// Name, grid and block of recorded launch i; returns 0 when i is out of range.
int fake_cuda_launch(int i, char* name_out, int capacity, unsigned* grid, unsigned* block) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (i < 0 || i >= (int)g_launches.size()) return 0;
    strncpy(name_out, g_launches[(size_t)i].name.c_str(), (size_t)capacity - 1);
    name_out[capacity - 1] = 0;
    *grid = g_launches[(size_t)i].grid;
    *block = g_launches[(size_t)i].block;
    return 1;
}
void fake_cuda_reset_launches(void) {
    std::lock_guard<std::mutex> lock(g_mu);
    g_launches.clear();
}
long fake_cuda_live_allocations(void) {
    std::lock_guard<std::mutex> lock(g_mu);
    return (long)g_device_allocs.size();
}
void fake_cuda_set_device(int major, int minor, int sms) {
    g_cc_major = major;
    g_cc_minor = minor;
    g_sms = sms;
}

// ---- the driver entry points liboptengine.so binds ----------------------------------------------
CUresult CUDAAPI cuInit(unsigned) { ENTER("cuInit"); return CUDA_SUCCESS; }
CUresult CUDAAPI cuDriverGetVersion(int* v) { *v = 12090; return CUDA_SUCCESS; }
CUresult CUDAAPI cuDeviceGet(CUdevice* d, int ordinal) { ENTER("cuDeviceGet"); *d = ordinal; return CUDA_SUCCESS; }
CUresult CUDAAPI cuDeviceGetCount(int* n) { *n = 2; return CUDA_SUCCESS; }
CUresult CUDAAPI cuDeviceGetAttribute(int* v, CUdevice_attribute a, CUdevice) {
    if (a == CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR) *v = g_cc_major;
    else if (a == CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR) *v = g_cc_minor;
    else if (a == CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT) *v = g_sms;
    else *v = 0;
    return CUDA_SUCCESS;
}
CUresult CUDAAPI cuDeviceGetName(char* name, int len, CUdevice) { strncpy(name, "fake B200", (size_t)len); return CUDA_SUCCESS; }
CUresult CUDAAPI cuDevicePrimaryCtxRetain(CUcontext* c, CUdevice d) { *c = (CUcontext)(uintptr_t)(0x1000 + d); return CUDA_SUCCESS; }
CUresult CUDAAPI cuDevicePrimaryCtxRelease(CUdevice) { return CUDA_SUCCESS; }
CUresult CUDAAPI cuCtxPushCurrent(CUcontext) { return CUDA_SUCCESS; }
CUresult CUDAAPI cuCtxPopCurrent(CUcontext* c) { *c = nullptr; return CUDA_SUCCESS; }
CUresult CUDAAPI cuCtxGetCurrent(CUcontext* c) { *c = nullptr; return CUDA_SUCCESS; }
CUresult CUDAAPI cuModuleLoadData(CUmodule* m, const void*) { ENTER("cuModuleLoadData"); *m = (CUmodule)(uintptr_t)0x2000; return CUDA_SUCCESS; }
CUresult CUDAAPI cuModuleUnload(CUmodule) { return CUDA_SUCCESS; }
CUresult CUDAAPI cuModuleGetFunction(CUfunction* f, CUmodule, const char* name) {
    ENTER("cuModuleGetFunction");
    std::lock_guard<std::mutex> lock(g_mu);
    FakeFunction*& fn = g_functions[name];
    if (!fn) fn = new FakeFunction{name};
    *f = (CUfunction)fn;
    return CUDA_SUCCESS;
}
CUresult CUDAAPI cuFuncGetAttribute(int* v, CUfunction_attribute, CUfunction) { *v = 0; return CUDA_SUCCESS; }
CUresult CUDAAPI cuOccupancyMaxActiveBlocksPerMultiprocessor(int* n, CUfunction, int, size_t) { *n = 2; return CUDA_SUCCESS; }
CUresult CUDAAPI cuLaunchKernel(CUfunction f, unsigned gx, unsigned, unsigned, unsigned bx, unsigned, unsigned, unsigned, CUstream,
                                void**, void**) {
    ENTER("cuLaunchKernel");
    std::lock_guard<std::mutex> lock(g_mu);
    g_launches.push_back(Launch{((FakeFunction*)f)->name, gx, bx});
    return CUDA_SUCCESS;
}
CUresult CUDAAPI cuMemAlloc(CUdeviceptr* p, size_t n) {
    ENTER("cuMemAlloc");
    void* m = nullptr;
    if (posix_memalign(&m, 512, n ? n : 1) != 0) return CUDA_ERROR_OUT_OF_MEMORY;
    memset(m, 0xcd, n);
    std::lock_guard<std::mutex> lock(g_mu);
    g_device_allocs[m] = n;
    g_device_bytes += n;
    *p = (CUdeviceptr)(uintptr_t)m;
    return CUDA_SUCCESS;
}
CUresult CUDAAPI cuMemFree(CUdeviceptr p) {
    ENTER("cuMemFree");
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_device_allocs.find((void*)(uintptr_t)p);
    if (it == g_device_allocs.end()) return CUDA_ERROR_INVALID_VALUE;
    g_device_bytes -= it->second;
    free(it->first);
    g_device_allocs.erase(it);
    return CUDA_SUCCESS;
}
CUresult CUDAAPI cuMemAllocHost(void** p, size_t n) {
    ENTER("cuMemAllocHost");
    *p = malloc(n ? n : 1);
    return *p ? CUDA_SUCCESS : CUDA_ERROR_OUT_OF_MEMORY;
}
CUresult CUDAAPI cuMemFreeHost(void* p) { free(p); return CUDA_SUCCESS; }
CUresult CUDAAPI cuMemHostRegister(void*, size_t, unsigned) { return CUDA_SUCCESS; }
CUresult CUDAAPI cuMemHostUnregister(void*) { return CUDA_SUCCESS; }
CUresult CUDAAPI cuMemcpyHtoDAsync(CUdeviceptr d, const void* s, size_t n, CUstream) {
    ENTER("cuMemcpyHtoDAsync");
    memcpy((void*)(uintptr_t)d, s, n);
    return CUDA_SUCCESS;
}
CUresult CUDAAPI cuMemcpyDtoHAsync(void* d, CUdeviceptr s, size_t n, CUstream) {
    ENTER("cuMemcpyDtoHAsync");
    memcpy(d, (const void*)(uintptr_t)s, n);
    return CUDA_SUCCESS;
}
CUresult CUDAAPI cuMemcpyDtoDAsync(CUdeviceptr d, CUdeviceptr s, size_t n, CUstream) {
    memmove((void*)(uintptr_t)d, (const void*)(uintptr_t)s, n);
    return CUDA_SUCCESS;
}
CUresult CUDAAPI cuMemcpyAsync(CUdeviceptr d, CUdeviceptr s, size_t n, CUstream) {
    ENTER("cuMemcpyAsync");
    memmove((void*)(uintptr_t)d, (const void*)(uintptr_t)s, n);
    return CUDA_SUCCESS;
}
CUresult CUDAAPI cuMemsetD32Async(CUdeviceptr d, unsigned v, size_t n, CUstream) {
    unsigned* p = (unsigned*)(uintptr_t)d;
    for (size_t i = 0; i < n; i++) p[i] = v;
    return CUDA_SUCCESS;
}
CUresult CUDAAPI cuMemsetD8Async(CUdeviceptr d, unsigned char v, size_t n, CUstream) {
    ENTER("cuMemsetD8Async");
    memset((void*)(uintptr_t)d, v, n);
    return CUDA_SUCCESS;
}
CUresult CUDAAPI cuMemGetInfo(size_t* f, size_t* t) { *t = (size_t)180 << 30; *f = *t - g_device_bytes; return CUDA_SUCCESS; }
CUresult CUDAAPI cuMemGetAddressRange(CUdeviceptr* base, size_t* size, CUdeviceptr p) {
    std::lock_guard<std::mutex> lock(g_mu);
    for (auto& kv : g_device_allocs) {
        uintptr_t b = (uintptr_t)kv.first;
        if ((uintptr_t)p >= b && (uintptr_t)p < b + kv.second) {
            *base = (CUdeviceptr)b;
            *size = kv.second;
            return CUDA_SUCCESS;
        }
    }
    return CUDA_ERROR_INVALID_VALUE;
}
CUresult CUDAAPI cuStreamCreate(CUstream* s, unsigned) { *s = (CUstream)(uintptr_t)0x3000; return CUDA_SUCCESS; }
CUresult CUDAAPI cuStreamDestroy(CUstream) { return CUDA_SUCCESS; }
CUresult CUDAAPI cuStreamSynchronize(CUstream) { ENTER("cuStreamSynchronize"); return CUDA_SUCCESS; }
CUresult CUDAAPI cuStreamWaitEvent(CUstream, CUevent, unsigned) { return CUDA_SUCCESS; }
CUresult CUDAAPI cuStreamIsCapturing(CUstream, CUstreamCaptureStatus* s) { *s = CU_STREAM_CAPTURE_STATUS_NONE; return CUDA_SUCCESS; }
CUresult CUDAAPI cuEventCreate(CUevent* e, unsigned) { ENTER("cuEventCreate"); *e = (CUevent)malloc(8); return CUDA_SUCCESS; }
CUresult CUDAAPI cuEventDestroy(CUevent e) { free(e); return CUDA_SUCCESS; }
CUresult CUDAAPI cuEventRecord(CUevent, CUstream) { ENTER("cuEventRecord"); return CUDA_SUCCESS; }
CUresult CUDAAPI cuEventSynchronize(CUevent) { return CUDA_SUCCESS; }
CUresult CUDAAPI cuEventQuery(CUevent) { return CUDA_SUCCESS; }
CUresult CUDAAPI cuEventElapsedTime(float* ms, CUevent, CUevent) { *ms = 0.0f; return CUDA_SUCCESS; }
CUresult CUDAAPI cuIpcGetMemHandle(CUipcMemHandle* h, CUdeviceptr p) { memset(h, 0, sizeof(*h)); memcpy(h, &p, sizeof(p)); return CUDA_SUCCESS; }
CUresult CUDAAPI cuIpcOpenMemHandle(CUdeviceptr* p, CUipcMemHandle h, unsigned) { memcpy(p, &h, sizeof(*p)); return CUDA_SUCCESS; }
CUresult CUDAAPI cuIpcCloseMemHandle(CUdeviceptr) { return CUDA_SUCCESS; }
CUresult CUDAAPI cuDeviceCanAccessPeer(int* can, CUdevice, CUdevice) { *can = 1; return CUDA_SUCCESS; }
CUresult CUDAAPI cuCtxEnablePeerAccess(CUcontext, unsigned) { return CUDA_SUCCESS; }
CUresult CUDAAPI cuGetErrorString(CUresult r, const char** s) { *s = r == CUDA_ERROR_OUT_OF_MEMORY ? "out of memory" : "fake driver error"; return CUDA_SUCCESS; }
CUresult CUDAAPI cuGetErrorName(CUresult r, const char** s) { *s = r == CUDA_ERROR_OUT_OF_MEMORY ? "CUDA_ERROR_OUT_OF_MEMORY" : "CUDA_ERROR_FAKE"; return CUDA_SUCCESS; }

}  // extern "C"
