// oe_grad_norm_static: the gradient-norm reduction for callers that must not allocate.
//
// Every other entry point of this library works on a plan, and a plan owns device
// memory obtained with cuMemAlloc (its tables and the per-CTA partial sums of the
// reduction). Some hosts cannot afford that call: a trainer that has handed the whole
// GPU to its own arena up front, so that any later driver allocation fails or evicts
// what the arena holds; or a step loop that may not take the device-wide
// synchronisation an allocation or a free implies. For them this file offers the norm
// of ONE contiguous fp32 gradient buffer with no allocation at all: the partial sums
// and the arrival counter live in a file-scope __device__ array that is part of the
// library image, so every GPU that loads the library carries these 257 KB until the
// process exits.
//
// Consequences of the shared array, which callers have to respect:
//  * one reduction at a time per device: two calls whose kernels overlap on the GPU
//    (different streams, or different host threads) race on the array and both results
//    are undefined; calls on one stream are ordered and safe;
//  * the array keeps what the last call left in it; the entry point clears the only
//    word that has to start at zero (the arrival counter) on the caller's stream before
//    every launch, and every partial sum that is read was written by the same launch;
//  * the size is fixed: at most OE_STATIC_NORM_MAX_ELEMS elements per call.
//
// The first call on a device checks that it is an sm_100 part, looks up the array's device
// address (cudaGetSymbolAddress), which makes the CUDA runtime load this module, and asks for the
// kernel's occupancy; do that first call during start-up, outside any stream capture. No cudaMalloc, cudaFree or other
// allocating routine is called here, on the first call or later.
//
// This entry point has no counterpart in the reference.
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>

#include "../../../include/optengine.h"

extern "C" void oe_internal_set_error(const char* message);  // engine.cpp: feeds oe_last_error()

namespace {

constexpr int kThreads = 256;
constexpr uint32_t kSpanElems = 65536;  // elements behind one partial sum, for buffers that need all the slots
constexpr uint32_t kShortSpanElems = 8192;  // ... for buffers short enough to afford finer spans (better balance)
constexpr uint32_t kMaxSpans = 32768;   // partial sums the array can hold
constexpr uint64_t kMaxElems = (uint64_t)kSpanElems * kMaxSpans;  // 2^31 elements, 8 GiB of fp32
constexpr size_t kHeaderBytes = 256;    // arrival counter, padded to the array's alignment
constexpr size_t kScratchBytes = kHeaderBytes + (size_t)kMaxSpans * sizeof(double);

static_assert(kMaxElems == OE_STATIC_NORM_MAX_ELEMS, "header and kernel disagree on the maximum size");

// The scratch memory. In host code this name is only a handle for cudaGetSymbolAddress;
// it is not a device address and is never passed to a kernel.
static __device__ __align__(256) unsigned char oe_static_norm_scratch[kScratchBytes];

__device__ __forceinline__ double block_sum(double x, double* warp_sums) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) x += __shfl_down_sync(0xffffffffu, x, off);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = x;
    __syncthreads();
    double total = 0.0;
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 0; w < kThreads / 32; w++) total += warp_sums[w];
    }
    __syncthreads();
    return total;  // valid in thread 0
}

// A persistent grid (resident CTAs x SMs, fewer for a short buffer) strides over the spans of
// span_elems elements; a CTA reduces each of its spans to one float64 partial sum in the span's
// own slot of the array. The span is 8192 elements while the buffer fits the array's 32768 slots
// that way (up to 2^28 elements: many spans per CTA, so the last sweep of the grid is short) and
// 65536 beyond. Float64 accumulation as in the plan-based reduction; the CTA that arrives last
// adds the partial sums in span order, so the result depends only on the data and its length,
// not on the grid or on timing.
__global__ void __launch_bounds__(kThreads, 4)
oe_static_sumsq(const float* __restrict__ g, uint64_t numel, uint32_t n_spans, uint32_t span_elems, unsigned char* scratch,
                float* norm_out) {
    __shared__ double warp_sums[kThreads / 32];
    __shared__ uint32_t is_last;
    uint32_t* ticket = (uint32_t*)scratch;
    double* partials = (double*)(scratch + kHeaderBytes);
    const bool vector_path = (((uint64_t)g) & 15u) == 0;  // spans start at multiples of 8192 elements: same alignment as g

    for (uint32_t span = blockIdx.x; span < n_spans; span += gridDim.x) {
        const uint64_t begin = (uint64_t)span * span_elems;
        const uint64_t left = begin < numel ? numel - begin : 0;
        const uint32_t n = left < span_elems ? (uint32_t)left : span_elems;
        const float* __restrict__ x = g + begin;
        double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
        uint32_t done = 0;
        if (vector_path) {
            const uint32_t nvec = n >> 2;
            const float4* x4 = (const float4*)x;
            for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += kThreads * 4) {
                float4 v[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    uint32_t i = i0 + u * kThreads;
                    v[u] = i < nvec ? __ldcs(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    double p = (double)v[u].x, q = (double)v[u].y, r = (double)v[u].z, s = (double)v[u].w;
                    a0 = fma(p, p, a0);
                    a1 = fma(q, q, a1);
                    a2 = fma(r, r, a2);
                    a3 = fma(s, s, a3);
                }
            }
            done = nvec << 2;
        }
        for (uint32_t i = done + threadIdx.x; i < n; i += kThreads) {
            double p = (double)x[i];
            a0 = fma(p, p, a0);
        }
        double block = block_sum((a0 + a1) + (a2 + a3), warp_sums);
        if (threadIdx.x == 0) partials[span] = block;
    }
    if (threadIdx.x == 0) {
        __threadfence();
        is_last = (atomicAdd(ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    double s = 0.0;
    for (uint32_t i = threadIdx.x; i < n_spans; i += kThreads) s += __ldcg(partials + i);
    double total = block_sum(s, warp_sums);
    if (threadIdx.x == 0) {
        *norm_out = (float)sqrt(total);
        *ticket = 0u;
    }
}

std::mutex g_mu;
unsigned char* g_scratch_address[64] = {nullptr};  // per device, filled by the first call on it
uint32_t g_persistent_grid[64] = {0};               // resident CTAs of the kernel on the whole device

int fail(int code, const std::string& message) {
    oe_internal_set_error(message.c_str());
    return code;
}

int fail_rt(cudaError_t e, const char* op) {
    return fail((int)e, std::string(op) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
}

// Restores the caller's current device when the call returns.
struct DeviceGuard {
    int previous = -1;
    bool changed = false;
    cudaError_t enter(int device) {
        cudaError_t e = cudaGetDevice(&previous);
        if (e != cudaSuccess) return e;
        if (previous != device) {
            e = cudaSetDevice(device);
            changed = e == cudaSuccess;
        }
        return e;
    }
    ~DeviceGuard() {
        if (changed) cudaSetDevice(previous);
    }
};

}  // namespace

extern "C" OE_API int oe_grad_norm_static(int device, uint64_t grad, uint64_t numel, uint64_t norm_out,
                                          uint64_t stream) {
    if (device < 0 || device >= 64) return fail(OE_ERR_INVALID, "oe_grad_norm_static: device ordinal out of range");
    if (norm_out == 0 || (norm_out & 3u)) return fail(OE_ERR_INVALID, "oe_grad_norm_static: norm_out must be a 4-byte aligned device address");
    if (numel > 0 && (grad == 0 || (grad & 3u))) return fail(OE_ERR_INVALID, "oe_grad_norm_static: grad must be a 4-byte aligned device address");
    if (numel > kMaxElems)
        return fail(OE_ERR_LIMIT, "oe_grad_norm_static: " + std::to_string(numel) + " elements exceed the fixed scratch array's maximum of " +
                                      std::to_string(kMaxElems) + "; use a plan (oe_grad_norm) for larger inputs");
    DeviceGuard guard;
    cudaError_t e = guard.enter(device);
    if (e != cudaSuccess) return fail_rt(e, "cudaSetDevice");
    unsigned char* scratch = nullptr;
    uint32_t persistent = 0;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (g_scratch_address[device] == nullptr) {
            // Set-up, once per device, with that device current. This entry point does not need
            // oe_init, so it checks the architecture itself: the image holds sm_100a code only.
            int major = 0, minor = 0, sms = 0, resident = 0;
            if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device)) != cudaSuccess ||
                (e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device)) != cudaSuccess ||
                (e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess)
                return fail_rt(e, "cudaDeviceGetAttribute");
            if (major != 10 || minor != 0)
                return fail(OE_ERR_ARCH, "oe_grad_norm_static: device " + std::to_string(device) + " is sm_" + std::to_string(major) +
                                             std::to_string(minor) + "; this library carries sm_100a code only");
            // The array's name is a host-side handle; its address on this device comes from the runtime.
            void* address = nullptr;
            e = cudaGetSymbolAddress(&address, oe_static_norm_scratch);
            if (e != cudaSuccess) return fail_rt(e, "cudaGetSymbolAddress(oe_static_norm_scratch)");
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, oe_static_sumsq, kThreads, 0);
            if (e != cudaSuccess) return fail_rt(e, "cudaOccupancyMaxActiveBlocksPerMultiprocessor");
            g_persistent_grid[device] = (uint32_t)(sms > 0 ? sms : 1) * (uint32_t)(resident > 0 ? resident : 1);
            g_scratch_address[device] = (unsigned char*)address;
        }
        scratch = g_scratch_address[device];
        persistent = g_persistent_grid[device];
    }
    cudaStream_t s = (cudaStream_t)stream;
    // The arrival counter is the only word that must start at zero; a launch that was
    // interrupted earlier could have left it half-counted.
    e = cudaMemsetAsync(scratch, 0, sizeof(uint32_t), s);
    if (e != cudaSuccess) return fail_rt(e, "cudaMemsetAsync(arrival counter)");
    uint32_t span_elems = numel <= (uint64_t)kShortSpanElems * kMaxSpans ? kShortSpanElems : kSpanElems;
    uint32_t spans = (uint32_t)((numel + span_elems - 1) / span_elems);  // 0 for an empty gradient: norm 0
    uint32_t grid = spans < persistent ? spans : persistent;
    if (grid == 0) grid = 1;
    const float* g = (const float*)grad;
    float* out = (float*)norm_out;
    void* args[] = {&g, &numel, &spans, &span_elems, &scratch, &out};
    // The launch call's own return value: a sticky error left by an earlier, unrelated call is
    // neither reported under this kernel's name nor cleared here.
    e = cudaLaunchKernel((const void*)oe_static_sumsq, dim3(grid), dim3(kThreads), args, 0, s);
    if (e != cudaSuccess) return fail_rt(e, "oe_static_sumsq launch");
    return 0;
}
