#include "driver.h"

#include <dlfcn.h>
#include <stdlib.h>

#include <mutex>
#include <string>

namespace {
oe_driver g_driver;
bool g_ok = false;
std::string g_why;
std::once_flag g_once;

// cuda.h maps the public names to versioned entry points with macros
// (cuMemAlloc -> cuMemAlloc_v2, ...); stringifying after expansion binds the same
// symbol the header's prototype describes.
#define OE_STR2(x) #x
#define OE_STR(x) OE_STR2(x)

void load() {
    // OE_CUDA_DRIVER_LIBRARY names the driver library to bind instead of the system's libcuda.so.1:
    // a driver installed in an unusual place, or the recording stand-in the CPU tests use.
    const char* chosen = getenv("OE_CUDA_DRIVER_LIBRARY");
    void* h = nullptr;
    if (chosen && *chosen) {
        h = dlopen(chosen, RTLD_NOW | RTLD_LOCAL);
        if (!h) {
            const char* e = dlerror();
            g_why = std::string("CUDA driver library named by OE_CUDA_DRIVER_LIBRARY could not be loaded: ") + (e ? e : chosen);
            return;
        }
    }
    if (!h) h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        const char* e = dlerror();
        g_why = std::string("CUDA driver library not found (libcuda.so.1): ") + (e ? e : "dlopen failed");
        return;
    }
#define OE_LOAD(name)                                                              \
    g_driver.name##_ = reinterpret_cast<decltype(&name)>(dlsym(h, OE_STR(name))); \
    if (!g_driver.name##_) {                                                       \
        g_why = std::string("CUDA driver lacks symbol ") + OE_STR(name);           \
        return;                                                                    \
    }
    OE_DRIVER_FUNCS(OE_LOAD)
#undef OE_LOAD
    CUresult r = g_driver.cuInit_(0);
    if (r != CUDA_SUCCESS) {
        const char* s = nullptr;
        g_driver.cuGetErrorString_(r, &s);
        g_why = std::string("cuInit failed: ") + (s ? s : "unknown error");
        return;
    }
    g_ok = true;
}
}  // namespace

const oe_driver* oe_driver_get(const char** why) {
    std::call_once(g_once, load);
    if (!g_ok) {
        if (why) *why = g_why.c_str();
        return nullptr;
    }
    return &g_driver;
}
