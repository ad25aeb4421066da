// Host side of liboptengine.so: plans (device tables), launches and the small set of
// driver calls a host without a CUDA binding needs. Everything goes through the CUDA
// driver API bound at run time (driver.h); the kernels come from an sm_100a cubin
// embedded in the library (cubin_blob.S).
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <map>
#include <mutex>
#include <new>
#include <string>
#include <utility>
#include <vector>

#include "../../../include/optengine.h"
#include "driver.h"
#include "oe_table.h"

extern "C" const unsigned char oe_cubin_start[];
extern "C" const unsigned char oe_cubin_end[];

namespace {

constexpr uint32_t kThreads = 256;             // must equal OE_THREADS of the kernels
constexpr uint32_t kDefaultChunkElems = 4096;  // one pass of the update CTA: 256 threads x 4 vectors x 4 floats
constexpr int kMaxDevices = 64;
constexpr uint32_t kNormSpan = 2;               // must equal OE_NORM_SPAN of the kernels

thread_local std::string t_error;

int fail(int code, const std::string& message) {
    t_error = message;
    return code;
}

int fail_cu(const oe_driver* d, CUresult r, const char* op) {
    const char* name = nullptr;
    const char* text = nullptr;
    d->cuGetErrorName_(r, &name);
    d->cuGetErrorString_(r, &text);
    t_error = std::string(op) + ": " + (name ? name : "CUDA_ERROR") + " (" + (text ? text : "?") + ")";
    return (int)r;
}

#define OE_CU(call, op)                                       \
    do {                                                      \
        CUresult oe_r_ = (call);                              \
        if (oe_r_ != CUDA_SUCCESS) return fail_cu(d, oe_r_, op); \
    } while (0)

struct KernelSet {
    CUfunction adamw[4] = {nullptr, nullptr, nullptr, nullptr};  // "", u1, u2, u8
    CUfunction adamw_peers[3] = {nullptr, nullptr, nullptr};  // 4, 2, 8 vectors in flight per thread
    CUfunction sgd_peers = nullptr, peer_reduce[3] = {nullptr, nullptr, nullptr};  // n <= 2, 4, 8
    CUfunction step_increment = nullptr, sgd = nullptr, sumsq = nullptr, norm_finalize = nullptr,
               scale = nullptr, zero = nullptr, cast = nullptr, rank_exchange = nullptr, probe_stores = nullptr;
};
const char* const kAdamwNames[4] = {"oe_adamw_fused", "oe_adamw_fused_u1", "oe_adamw_fused_u2", "oe_adamw_fused_u8"};
const char* const kVariantKeys[4] = {"", "u1", "u2", "u8"};
const char* const kAdamwPeerNames[3] = {"oe_adamw_fused_peers", "oe_adamw_fused_peers_u2", "oe_adamw_fused_peers_u8"};

struct DeviceCtx {
    bool ready = false;
    int ordinal = -1;
    CUdevice dev = 0;
    CUcontext ctx = nullptr;
    CUmodule module = nullptr;
    int sm_count = 0;
    KernelSet k;
    int occ_adamw[4] = {0, 0, 0, 0};
    int occ_adamw_peers[3] = {0, 0, 0}, occ_sgd_peers = 0, occ_peer_reduce[3] = {0, 0, 0};
    int occ_sgd = 0, occ_sumsq = 0, occ_scale = 0, occ_zero = 0, occ_cast = 0;
};

std::mutex g_mu;
DeviceCtx g_dev[kMaxDevices];
std::atomic<int> g_live_plans{0};  // plans hold their device's context and kernel handles
std::map<std::string, int64_t> g_launches;

// Pushes the device's primary context for the lifetime of the guard and pops it
// again, so the caller's current context is never changed behind its back.
struct CtxGuard {
    const oe_driver* d;
    bool pushed = false;
    CtxGuard(const oe_driver* drv, CUcontext ctx) : d(drv) { pushed = d->cuCtxPushCurrent_(ctx) == CUDA_SUCCESS; }
    ~CtxGuard() {
        if (pushed) {
            CUcontext old;
            d->cuCtxPopCurrent_(&old);
        }
    }
};

const oe_driver* driver_or_fail(int* rc) {
    const char* why = nullptr;
    const oe_driver* d = oe_driver_get(&why);
    if (!d) *rc = fail(OE_ERR_NO_DRIVER, why ? why : "CUDA driver unavailable");
    return d;
}

DeviceCtx* device_or_fail(int device, int* rc) {
    if (device < 0 || device >= kMaxDevices) {
        *rc = fail(OE_ERR_INVALID, "device ordinal out of range");
        return nullptr;
    }
    DeviceCtx* dc = &g_dev[device];
    bool ready;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        ready = dc->ready;
    }
    if (!ready) {
        *rc = fail(OE_ERR_NOT_INIT, "oe_init was not called for device " + std::to_string(device));
        return nullptr;
    }
    return dc;
}

void count_launch(const char* name) {
    std::lock_guard<std::mutex> lock(g_mu);
    g_launches[name] += 1;
}

// Optional per-launch timing (the reference's EnableGPUProfile / timedGPU, autograd/cuda_kernels.go:24-82):
// two events around the launch and a wait for the second one, summed per kernel name. Like the
// reference's it serialises every launch, so it is a diagnostic and must stay off under stream capture.
std::atomic<bool> g_profiling{false};
std::map<std::string, double> g_profile_ms;  // guarded by g_mu

int launch(const oe_driver* d, CUfunction f, const char* name, uint32_t grid, uint32_t block, CUstream stream,
           void** args) {
    if (!g_profiling.load(std::memory_order_relaxed)) {
        OE_CU(d->cuLaunchKernel_(f, grid, 1, 1, block, 1, 1, 0, stream, args, nullptr), name);
        count_launch(name);
        return 0;
    }
    CUevent start = nullptr, end = nullptr;
    OE_CU(d->cuEventCreate_(&start, CU_EVENT_DEFAULT), "cuEventCreate(profile)");
    CUresult r = d->cuEventCreate_(&end, CU_EVENT_DEFAULT);
    if (r == CUDA_SUCCESS) r = d->cuEventRecord_(start, stream);
    if (r == CUDA_SUCCESS) r = d->cuLaunchKernel_(f, grid, 1, 1, block, 1, 1, 0, stream, args, nullptr);
    bool launched = r == CUDA_SUCCESS;
    if (r == CUDA_SUCCESS) r = d->cuEventRecord_(end, stream);
    if (r == CUDA_SUCCESS) r = d->cuEventSynchronize_(end);
    float ms = 0.0f;
    if (r == CUDA_SUCCESS) r = d->cuEventElapsedTime_(&ms, start, end);
    d->cuEventDestroy_(start);
    if (end) d->cuEventDestroy_(end);
    if (launched) count_launch(name);
    if (r != CUDA_SUCCESS) return fail_cu(d, r, name);
    std::lock_guard<std::mutex> lock(g_mu);
    g_profile_ms[name] += (double)ms;
    return 0;
}

bool finite_nonneg(float x) { return isfinite(x) && x >= 0.0f; }

}  // namespace

// -------------------------------------------------------------------------------------
// plan
// -------------------------------------------------------------------------------------
struct oe_plan {
    DeviceCtx* dc = nullptr;
    uint32_t chunk_elems = kDefaultChunkElems;
    int variant = 0;
    float grad_scale = 1.0f;            // every kernel of the plan reads a gradient element as (float)(g * grad_scale)
    std::vector<oe_tensor_desc> descs;  // every parameter, with or without a gradient
    uint32_t n_active = 0;              // parameters with a gradient = rows of the device tensor table
    uint64_t n_chunks = 0;
    uint64_t active_elems = 0;
    bool all_adamw_state = true;        // every active tensor has state1 and state2
    // device side
    CUdeviceptr d_tensors = 0, d_chunks = 0, d_norm = 0, d_partials = 0;
    size_t cap_tensors = 0, cap_chunks = 0;  // capacities in entries
    uint32_t max_grid = 0;
    // page-locked staging for the tables, and the event that guards its reuse
    void* h_stage = nullptr;
    size_t h_stage_bytes = 0;
    CUevent staged = nullptr;
    bool staged_pending = false;
    int64_t uploads = 0;
    bool tables_valid = false;  // the device tables describe `descs`; false after a failed update
    // tuning knobs of the peer kernels (0 = the library's choice); none changes a result
    uint32_t tune_reduce_grid = 0, tune_update_grid = 0, tune_reduce_first = 0, tune_push_warp_rotate = 0;
    uint32_t tune_reduce_warp_rotate = 0;  // pull-reduce: every warp starts at another source
    uint32_t tune_peer_unroll = 0;  // shape of the sharded AdamW update: 0 = 4 vectors in flight, 1 = 2, 2 = 8
    uint32_t tune_step_grid = 0;  // single-GPU update / scale launches: 0 = persistent grid, 1 = one CTA per work unit
    uint64_t status_word = 0;   // device address of a sharded step's status word, 0 = none
};

namespace {

int validate_descs(const oe_tensor_desc* t, uint32_t n, uint32_t chunk_elems) {
    if (n > 0 && t == nullptr) return fail(OE_ERR_INVALID, "tensor descriptors are NULL");
    for (uint32_t i = 0; i < n; i++) {
        const oe_tensor_desc& x = t[i];
        std::string at = "tensor " + std::to_string(i) + ": ";
        if (x.numel == 0) return fail(OE_ERR_INVALID, at + "numel is 0");
        if (x.param == 0) return fail(OE_ERR_INVALID, at + "param address is 0");
        if ((x.param | x.grad | x.state1 | x.state2) & 3u) return fail(OE_ERR_INVALID, at + "fp32 address not 4-byte aligned");
        if (x.shadow & 1u) return fail(OE_ERR_INVALID, at + "bf16 shadow address not 2-byte aligned");
        if (!finite_nonneg(x.lr_scale)) return fail(OE_ERR_INVALID, at + "invalid parameter group learning-rate scale");
        if (!finite_nonneg(x.weight_decay)) return fail(OE_ERR_INVALID, at + "invalid parameter group weight decay");
        if ((x.numel + chunk_elems - 1) / chunk_elems > 0xffffffffull) return fail(OE_ERR_LIMIT, at + "too many chunks");
    }
    return 0;
}

// Fills the staging buffer with the tensor table followed by the chunk table.
void build_tables(oe_plan* p, oe_dev_tensor* tt, oe_dev_chunk* ck) {
    uint32_t row = 0;
    uint64_t c = 0;
    for (const oe_tensor_desc& x : p->descs) {
        if (x.grad == 0) continue;
        oe_dev_tensor& o = tt[row];
        o.param = x.param;
        o.grad = x.grad;
        o.state1 = x.state1;
        o.state2 = x.state2;
        o.shadow = x.shadow;
        o.numel = x.numel;
        o.lr_scale = x.lr_scale == 0.0f ? 1.0f : x.lr_scale;
        o.weight_decay = x.weight_decay;
        // 128-bit path: fp32 streams 16-byte aligned, the bf16 stream 8-byte aligned.
        // Bit 0 covers param, grad, state1 and the shadow; bit 1 adds state2, which is
        // a full-size stream for AdamW (v) but a one-float flag for SGD.
        bool aligned = ((x.param | x.grad | x.state1) & 15u) == 0 && (x.shadow & 7u) == 0;
        o.aligned = (aligned ? OE_ALIGNED_BASE : 0u) | ((aligned && (x.state2 & 15u) == 0) ? OE_ALIGNED_STATE2 : 0u);
        o.reserved = 0;
        uint64_t nck = (x.numel + p->chunk_elems - 1) / p->chunk_elems;
        for (uint64_t j = 0; j < nck; j++) {
            ck[c].tensor = row;
            ck[c].chunk = (uint32_t)j;
            c++;
        }
        row++;
    }
}

void count_active(oe_plan* p) {
    p->n_active = 0;
    p->n_chunks = 0;
    p->active_elems = 0;
    p->all_adamw_state = true;
    for (const oe_tensor_desc& x : p->descs) {
        if (x.grad == 0) continue;
        p->n_active++;
        p->n_chunks += (x.numel + p->chunk_elems - 1) / p->chunk_elems;
        p->active_elems += x.numel;
        if (x.state1 == 0 || x.state2 == 0) p->all_adamw_state = false;
    }
}

// Makes room for the current tables on the device and in the staging buffer. Only
// called outside stream capture paths that must not allocate: capacities never shrink.
int ensure_capacity(const oe_driver* d, oe_plan* p) {
    // A table that has to grow is allocated before the old one is released, and the plan's
    // fields change only once the new allocation exists: a failed allocation leaves the plan
    // exactly as it was (capacities, addresses and all).
    size_t need_t = p->n_active ? p->n_active : 1, need_c = p->n_chunks ? p->n_chunks : 1;
    if (need_t > p->cap_tensors) {
        size_t cap = need_t + need_t / 4 + 8;
        CUdeviceptr fresh = 0;
        OE_CU(d->cuMemAlloc_(&fresh, cap * sizeof(oe_dev_tensor)), "cuMemAlloc(tensor table)");
        if (p->d_tensors) d->cuMemFree_(p->d_tensors);
        p->d_tensors = fresh;
        p->cap_tensors = cap;
    }
    if (need_c > p->cap_chunks) {
        size_t cap = need_c + need_c / 4 + 64;
        CUdeviceptr fresh = 0;
        OE_CU(d->cuMemAlloc_(&fresh, cap * sizeof(oe_dev_chunk)), "cuMemAlloc(chunk table)");
        if (p->d_chunks) d->cuMemFree_(p->d_chunks);
        p->d_chunks = fresh;
        p->cap_chunks = cap;
    }
    size_t bytes = p->cap_tensors * sizeof(oe_dev_tensor) + p->cap_chunks * sizeof(oe_dev_chunk);
    if (bytes > p->h_stage_bytes) {
        if (p->staged_pending) {
            OE_CU(d->cuEventSynchronize_(p->staged), "cuEventSynchronize(table upload)");
            p->staged_pending = false;
        }
        void* fresh = nullptr;
        OE_CU(d->cuMemAllocHost_(&fresh, bytes), "cuMemAllocHost(staging)");
        if (p->h_stage) d->cuMemFreeHost_(p->h_stage);
        p->h_stage = fresh;
        p->h_stage_bytes = bytes;
    }
    return 0;
}

int upload_tables(const oe_driver* d, oe_plan* p, CUstream stream) {
    // From here until the copies are enqueued the device tables may describe neither the old nor
    // the new descriptors: every launch path refuses a plan whose tables are not valid.
    p->tables_valid = false;
    int rc = ensure_capacity(d, p);
    if (rc) return rc;
    if (p->staged_pending) {
        // The previous upload may still be reading the staging buffer.
        OE_CU(d->cuEventSynchronize_(p->staged), "cuEventSynchronize(table upload)");
        p->staged_pending = false;
    }
    oe_dev_tensor* tt = (oe_dev_tensor*)p->h_stage;
    oe_dev_chunk* ck = (oe_dev_chunk*)((char*)p->h_stage + p->cap_tensors * sizeof(oe_dev_tensor));
    build_tables(p, tt, ck);
    if (p->n_active) {
        OE_CU(d->cuMemcpyHtoDAsync_(p->d_tensors, tt, p->n_active * sizeof(oe_dev_tensor), stream),
              "cuMemcpyHtoDAsync(tensor table)");
        OE_CU(d->cuMemcpyHtoDAsync_(p->d_chunks, ck, p->n_chunks * sizeof(oe_dev_chunk), stream),
              "cuMemcpyHtoDAsync(chunk table)");
        OE_CU(d->cuEventRecord_(p->staged, stream), "cuEventRecord(table upload)");
        p->staged_pending = true;
    }
    p->uploads++;
    p->tables_valid = true;
    return 0;
}

uint32_t grid_for(const oe_plan* p, int occupancy);

// Launch shape of an update that also stores into the peers' buffers. The caller's knobs win; where
// they are unset the library chooses by the number of ranks, from measurements on 8-GPU B200 boxes
// (`bench.py --gpus N --sweep`): with four ranks the AdamW update pushes 676-695 GB/s from one CTA
// per SM whose warps start their round of stores at different targets, against 621 GB/s from the
// persistent default; with two or eight ranks no shape beat the default.
struct PeerLaunchShape {
    uint32_t grid;
    bool warp_rotate;
};
PeerLaunchShape peer_update_shape(const oe_plan* p, int occupancy, uint32_t n_ranks, bool adamw) {
    PeerLaunchShape shape;
    shape.grid = grid_for(p, occupancy);
    const bool four = adamw && n_ranks == 4 && p->tune_peer_unroll == 0;
    if (p->tune_update_grid) {
        if (p->tune_update_grid < shape.grid) shape.grid = p->tune_update_grid;
    } else if (four && (uint32_t)p->dc->sm_count < shape.grid) {
        shape.grid = (uint32_t)p->dc->sm_count;
    }
    if (p->tune_push_warp_rotate)
        shape.warp_rotate = p->tune_push_warp_rotate == 1;
    else
        shape.warp_rotate = four && shape.grid == (uint32_t)p->dc->sm_count;
    return shape;
}

uint32_t grid_for(const oe_plan* p, int occupancy) {
    uint64_t persistent = (uint64_t)p->dc->sm_count * (uint64_t)(occupancy > 0 ? occupancy : 1);
    uint64_t g = p->n_chunks < persistent ? p->n_chunks : persistent;
    if (g == 0) g = 1;
    if (g > p->max_grid) g = p->max_grid;
    return (uint32_t)g;
}

void destroy_plan(const oe_driver* d, oe_plan* p) {
    if (p->staged_pending) d->cuEventSynchronize_(p->staged);
    if (p->staged) d->cuEventDestroy_(p->staged);
    if (p->h_stage) d->cuMemFreeHost_(p->h_stage);
    if (p->d_tensors) d->cuMemFree_(p->d_tensors);
    if (p->d_chunks) d->cuMemFree_(p->d_chunks);
    if (p->d_norm) d->cuMemFree_(p->d_norm);
    if (p->d_partials) d->cuMemFree_(p->d_partials);
    delete p;
    g_live_plans.fetch_sub(1);
}

// Work-unit size when the caller leaves it to the library. Sets that stream from HBM use
// 4096 elements (one pass of an update CTA at four vectors per thread). A set too small to give
// every SM two such units is latency-bound: halve the unit (down to 1024) until it does, so the
// one launch spreads over the machine (measured on a captured step of a 0.2 M-parameter
// set: 8.2 us per replay at 4096, 6.2 us at 2048 and 1024).
uint32_t default_chunk_elems(const oe_tensor_desc* t, uint32_t n, int sm_count) {
    if (!t) return kDefaultChunkElems;
    uint32_t chunk = kDefaultChunkElems;
    const uint64_t want = 2ull * (uint64_t)(sm_count > 0 ? sm_count : 1);
    while (chunk > 1024) {
        uint64_t units = 0;
        for (uint32_t i = 0; i < n && units < want; i++) units += (t[i].numel + chunk - 1) / chunk;
        if (units >= want) break;
        chunk >>= 1;
    }
    return chunk;
}

bool same_descs(const std::vector<oe_tensor_desc>& a, const oe_tensor_desc* b, uint32_t n) {
    if (a.size() != n) return false;
    return n == 0 || memcmp(a.data(), b, (size_t)n * sizeof(oe_tensor_desc)) == 0;
}

}  // namespace

// -------------------------------------------------------------------------------------
// library
// -------------------------------------------------------------------------------------
extern "C" int oe_abi_version(void) { return OE_ABI_VERSION; }

extern "C" const char* oe_last_error(void) { return t_error.c_str(); }

extern "C" int oe_init(int device) {
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    if (device < 0 || device >= kMaxDevices) return fail(OE_ERR_INVALID, "device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceCtx* dc = &g_dev[device];
    if (dc->ready) return 0;
    int count = 0;
    OE_CU(d->cuDeviceGetCount_(&count), "cuDeviceGetCount");
    if (device >= count) return fail(OE_ERR_INVALID, "no such CUDA device: " + std::to_string(device));
    OE_CU(d->cuDeviceGet_(&dc->dev, device), "cuDeviceGet");
    int major = 0, minor = 0;
    OE_CU(d->cuDeviceGetAttribute_(&major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, dc->dev), "cuDeviceGetAttribute");
    OE_CU(d->cuDeviceGetAttribute_(&minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, dc->dev), "cuDeviceGetAttribute");
    if (major != 10 || minor != 0)
        return fail(OE_ERR_ARCH, "device " + std::to_string(device) + " is sm_" + std::to_string(major) +
                                     std::to_string(minor) + "; this library carries sm_100a code only");
    OE_CU(d->cuDeviceGetAttribute_(&dc->sm_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, dc->dev),
          "cuDeviceGetAttribute");
    OE_CU(d->cuDevicePrimaryCtxRetain_(&dc->ctx, dc->dev), "cuDevicePrimaryCtxRetain");
    CtxGuard guard(d, dc->ctx);
    CUresult r = d->cuModuleLoadData_(&dc->module, oe_cubin_start);
    if (r != CUDA_SUCCESS) {
        d->cuDevicePrimaryCtxRelease_(dc->dev);
        return fail_cu(d, r, "cuModuleLoadData(embedded sm_100a cubin)");
    }
    struct {
        CUfunction* f;
        const char* name;
        int* occ;
    } table[] = {
        {&dc->k.adamw[0], kAdamwNames[0], &dc->occ_adamw[0]}, {&dc->k.adamw[1], kAdamwNames[1], &dc->occ_adamw[1]},
        {&dc->k.adamw[2], kAdamwNames[2], &dc->occ_adamw[2]}, {&dc->k.adamw[3], kAdamwNames[3], &dc->occ_adamw[3]},
        {&dc->k.adamw_peers[0], kAdamwPeerNames[0], &dc->occ_adamw_peers[0]},
        {&dc->k.adamw_peers[1], kAdamwPeerNames[1], &dc->occ_adamw_peers[1]},
        {&dc->k.adamw_peers[2], kAdamwPeerNames[2], &dc->occ_adamw_peers[2]},
        {&dc->k.peer_reduce[0], "oe_peer_reduce_sumsq_n2", &dc->occ_peer_reduce[0]},
        {&dc->k.peer_reduce[1], "oe_peer_reduce_sumsq_n4", &dc->occ_peer_reduce[1]},
        {&dc->k.peer_reduce[2], "oe_peer_reduce_sumsq_n8", &dc->occ_peer_reduce[2]},
        {&dc->k.step_increment, "oe_step_increment", nullptr}, {&dc->k.sgd, "oe_sgd_fused", &dc->occ_sgd},
        {&dc->k.sgd_peers, "oe_sgd_fused_peers", &dc->occ_sgd_peers},
        {&dc->k.sumsq, "oe_grad_sumsq", &dc->occ_sumsq},
        {&dc->k.norm_finalize, "oe_norm_finalize", nullptr},   {&dc->k.scale, "oe_scale_grads", &dc->occ_scale},
        {&dc->k.zero, "oe_zero_grads", &dc->occ_zero},         {&dc->k.cast, "oe_cast_bf16", &dc->occ_cast},
        {&dc->k.rank_exchange, "oe_rank_exchange", nullptr},
        {&dc->k.probe_stores, "oe_probe_peer_stores", nullptr},
    };
    for (auto& e : table) {
        r = d->cuModuleGetFunction_(e.f, dc->module, e.name);
        if (r == CUDA_SUCCESS && e.occ)
            r = d->cuOccupancyMaxActiveBlocksPerMultiprocessor_(e.occ, *e.f, (int)kThreads, 0);
        if (r != CUDA_SUCCESS) {
            d->cuModuleUnload_(dc->module);
            d->cuDevicePrimaryCtxRelease_(dc->dev);
            dc->module = nullptr;
            return fail_cu(d, r, e.name);
        }
    }
    dc->ordinal = device;
    dc->ready = true;
    return 0;
}

extern "C" int oe_shutdown(void) {
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    if (g_live_plans.load() > 0)
        return fail(OE_ERR_INVALID, "oe_shutdown: " + std::to_string(g_live_plans.load()) + " plan(s) still alive; destroy them first");
    std::lock_guard<std::mutex> lock(g_mu);
    for (DeviceCtx& dc : g_dev) {
        if (!dc.ready) continue;
        {
            CtxGuard guard(d, dc.ctx);
            d->cuModuleUnload_(dc.module);
        }
        d->cuDevicePrimaryCtxRelease_(dc.dev);
        dc = DeviceCtx();
    }
    return 0;
}

extern "C" int oe_device_count(int* count_out) {
    if (!count_out) return fail(OE_ERR_INVALID, "count_out is NULL");
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    OE_CU(d->cuDeviceGetCount_(count_out), "cuDeviceGetCount");
    return 0;
}

extern "C" int oe_enable_peer_access(int device, int peer_device) {
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    DeviceCtx* dc = device_or_fail(device, &rc);
    if (!dc) return rc;
    DeviceCtx* peer = device_or_fail(peer_device, &rc);
    if (!peer) return rc;
    if (device == peer_device) return 0;
    int can = 0;
    OE_CU(d->cuDeviceCanAccessPeer_(&can, dc->dev, peer->dev), "cuDeviceCanAccessPeer");
    if (!can) return fail(OE_ERR_INVALID, "device " + std::to_string(device) + " cannot address the memory of device " + std::to_string(peer_device));
    CtxGuard guard(d, dc->ctx);
    CUresult r = d->cuCtxEnablePeerAccess_(peer->ctx, 0);
    if (r != CUDA_SUCCESS && r != CUDA_ERROR_PEER_ACCESS_ALREADY_ENABLED) return fail_cu(d, r, "cuCtxEnablePeerAccess");
    return 0;
}

extern "C" int oe_device_sm_count(int device) {
    int rc = 0;
    DeviceCtx* dc = device_or_fail(device, &rc);
    return dc ? dc->sm_count : rc;
}

// -------------------------------------------------------------------------------------
// plans
// -------------------------------------------------------------------------------------
extern "C" int oe_plan_create(int device, const oe_tensor_desc* tensors, uint32_t n_tensors, uint32_t chunk_elems,
                              oe_plan** out) {
    if (!out) return fail(OE_ERR_INVALID, "out is NULL");
    *out = nullptr;
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    DeviceCtx* dc = device_or_fail(device, &rc);
    if (!dc) return rc;
    if (chunk_elems == 0) chunk_elems = default_chunk_elems(tensors, n_tensors, dc->sm_count);
    if (chunk_elems % 1024 != 0 || chunk_elems > (1u << 24))
        return fail(OE_ERR_INVALID, "chunk_elems must be a multiple of 1024, at most 2^24");
    if ((rc = validate_descs(tensors, n_tensors, chunk_elems)) != 0) return rc;
    oe_plan* p = new (std::nothrow) oe_plan();
    if (!p) return fail(OE_ERR_INVALID, "out of host memory");
    g_live_plans.fetch_add(1);
    p->dc = dc;
    p->chunk_elems = chunk_elems;
    p->descs.assign(tensors, tensors + n_tensors);
    count_active(p);
    CtxGuard guard(d, dc->ctx);
    int occ_max = dc->occ_sumsq;
    for (int o : dc->occ_adamw) occ_max = o > occ_max ? o : occ_max;
    for (int o : {dc->occ_sgd, dc->occ_scale, dc->occ_zero}) occ_max = o > occ_max ? o : occ_max;
    p->max_grid = (uint32_t)dc->sm_count * (uint32_t)(occ_max > 0 ? occ_max : 1);
    CUresult r = d->cuMemAlloc_(&p->d_norm, sizeof(oe_dev_norm));
    if (r == CUDA_SUCCESS) r = d->cuMemAlloc_(&p->d_partials, (size_t)p->max_grid * sizeof(double));
    if (r == CUDA_SUCCESS) r = d->cuEventCreate_(&p->staged, CU_EVENT_DISABLE_TIMING);
    if (r == CUDA_SUCCESS) r = d->cuMemsetD8Async_(p->d_norm, 0, sizeof(oe_dev_norm), nullptr);
    if (r != CUDA_SUCCESS) {
        rc = fail_cu(d, r, "oe_plan_create(allocate)");
        destroy_plan(d, p);
        return rc;
    }
    rc = upload_tables(d, p, nullptr);
    if (rc == 0) {
        r = d->cuStreamSynchronize_(nullptr);
        if (r != CUDA_SUCCESS) rc = fail_cu(d, r, "cuStreamSynchronize");
        p->staged_pending = false;
    }
    if (rc) {
        std::string keep = t_error;
        destroy_plan(d, p);
        t_error = keep;
        return rc;
    }
    *out = p;
    return 0;
}

extern "C" int oe_plan_update(oe_plan* plan, const oe_tensor_desc* tensors, uint32_t n_tensors, uint64_t stream) {
    if (!plan) return fail(OE_ERR_INVALID, "plan is NULL");
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    if (plan->tables_valid && same_descs(plan->descs, tensors, n_tensors)) return 0;
    if ((rc = validate_descs(tensors, n_tensors, plan->chunk_elems)) != 0) return rc;
    // The new descriptors are adopted only together with their uploaded tables. When a driver call
    // fails on the way, the plan keeps no descriptors at all: the next update (with any list, the
    // same one included) uploads again, and until one succeeds every launch is refused.
    plan->descs.assign(tensors, tensors + n_tensors);
    count_active(plan);
    CtxGuard guard(d, plan->dc->ctx);
    rc = upload_tables(d, plan, (CUstream)stream);
    if (rc) {
        plan->descs.clear();
        count_active(plan);
        plan->tables_valid = false;
    }
    return rc;
}

extern "C" int oe_plan_destroy(oe_plan* plan) {
    if (!plan) return 0;
    if (plan->status_word != 0)
        return fail(OE_ERR_INVALID, "oe_plan_destroy: a sharded step (oe_zero1) is still bound to this plan; destroy it first");
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    CtxGuard guard(d, plan->dc->ctx);
    destroy_plan(d, plan);
    return 0;
}

extern "C" int64_t oe_plan_info(const oe_plan* plan, int what) {
    if (!plan) return -1;
    switch (what) {
        case 0: return plan->n_active;
        case 1: return (int64_t)plan->n_chunks;
        case 2: return (int64_t)plan->active_elems;
        case 3: return grid_for(plan, plan->dc->occ_adamw[plan->variant]);
        case 4: return grid_for(plan, plan->dc->occ_sumsq);
        case 5: return plan->chunk_elems;
        case 6: return plan->uploads;
        default: return -1;
    }
}

extern "C" uint64_t oe_plan_norm_address(const oe_plan* plan) { return plan ? (uint64_t)plan->d_norm : 0; }

extern "C" int oe_plan_set_variant(oe_plan* plan, const char* variant) {
    if (!plan || !variant) return fail(OE_ERR_INVALID, "plan or variant is NULL");
    for (int i = 0; i < 4; i++) {
        if (strcmp(variant, kVariantKeys[i]) == 0) {
            plan->variant = i;
            return 0;
        }
    }
    return fail(OE_ERR_INVALID, std::string("unknown update-kernel variant: ") + variant);
}

extern "C" int oe_plan_set_grad_scale(oe_plan* plan, const float* scale) {
    if (!plan || !scale) return fail(OE_ERR_INVALID, "plan or scale is NULL");
    if (!isfinite(*scale) || !(*scale > 0.0f)) return fail(OE_ERR_INVALID, "gradient scale must be finite and positive");
    plan->grad_scale = *scale;
    return 0;
}

extern "C" int oe_plan_set_tuning(oe_plan* plan, int what, uint64_t value) {
    if (!plan) return fail(OE_ERR_INVALID, "plan is NULL");
    if (value > 0x7fffffffull) return fail(OE_ERR_INVALID, "oe_plan_set_tuning: value out of range");
    switch (what) {
        case OE_TUNE_PEER_REDUCE_GRID: plan->tune_reduce_grid = (uint32_t)value; return 0;
        case OE_TUNE_PEER_UPDATE_GRID: plan->tune_update_grid = (uint32_t)value; return 0;
        case OE_TUNE_PEER_REDUCE_FIRST: plan->tune_reduce_first = (uint32_t)value % OE_MAX_PEERS; return 0;
        case OE_TUNE_PEER_PUSH_WARP_ROTATE:
            if (value > 2) return fail(OE_ERR_INVALID, "oe_plan_set_tuning: warp rotation is 0 (library's choice), 1 (on) or 2 (off)");
            plan->tune_push_warp_rotate = (uint32_t)value;
            return 0;
        case OE_TUNE_STEP_GRID: plan->tune_step_grid = value ? 1u : 0u; return 0;
        case OE_TUNE_PEER_REDUCE_WARP_ROTATE: plan->tune_reduce_warp_rotate = value ? 1u : 0u; return 0;
        case OE_TUNE_PEER_UPDATE_VECTORS:
            if (value != 0 && value != 2 && value != 4 && value != 8)
                return fail(OE_ERR_INVALID, "oe_plan_set_tuning: the sharded update is built for 2, 4 or 8 vectors in flight");
            plan->tune_peer_unroll = value == 2 ? 1u : value == 8 ? 2u : 0u;
            return 0;
        default: return fail(OE_ERR_INVALID, "oe_plan_set_tuning: unknown knob");
    }
}

// -------------------------------------------------------------------------------------
// norm and clip
// -------------------------------------------------------------------------------------
namespace {
int launch_sumsq(const oe_driver* d, oe_plan* p, uint32_t flags, CUstream stream) {
    uint32_t n_chunks = (uint32_t)p->n_chunks, chunk_elems = p->chunk_elems;
    float gscale = p->grad_scale;
    void* args[] = {&p->d_tensors, &p->d_chunks, &n_chunks, &chunk_elems, &p->d_norm, &p->d_partials, &flags, &gscale};
    uint32_t grid = grid_for(p, p->dc->occ_sumsq);
    uint32_t spans = (n_chunks + kNormSpan - 1) / kNormSpan;  // the kernel walks the table in spans of work units
    if (grid > spans) grid = spans ? spans : 1;
    return launch(d, p->dc->k.sumsq, "oe_grad_sumsq", grid, kThreads, stream, args);
}

// Every launch path passes through here: a plan whose last table upload failed has no usable
// tables, and a grid dimension (oe_zero_grads launches one CTA per work unit) ends at 2^31-1.
int check_chunk_count(const oe_plan* p) {
    if (!p->tables_valid)
        return fail(OE_ERR_INVALID, "the plan's device tables are stale (the last oe_plan_update failed); update the plan again");
    if (p->n_chunks > 0x7fffffffull) return fail(OE_ERR_LIMIT, "plan has more than 2^31-1 work units; use a larger chunk_elems");
    return 0;
}
}  // namespace

extern "C" int oe_grad_norm(oe_plan* plan, uint32_t flags, uint64_t stream) {
    if (!plan) return fail(OE_ERR_INVALID, "plan is NULL");
    if (flags & ~OE_PARTIAL_ONLY) return fail(OE_ERR_INVALID, "oe_grad_norm: unknown flag");
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    if ((rc = check_chunk_count(plan)) != 0) return rc;
    CtxGuard guard(d, plan->dc->ctx);
    return launch_sumsq(d, plan, flags, (CUstream)stream);
}

extern "C" int oe_norm_finalize(oe_plan* plan, uint64_t stream) {
    if (!plan) return fail(OE_ERR_INVALID, "plan is NULL");
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    CtxGuard guard(d, plan->dc->ctx);
    void* args[] = {&plan->d_norm};
    return launch(d, plan->dc->k.norm_finalize, "oe_norm_finalize", 1, 32, (CUstream)stream, args);
}

extern "C" int oe_clip_grad_norm(oe_plan* plan, const float* max_norm, uint32_t flags, uint64_t stream) {
    if (!plan || !max_norm) return fail(OE_ERR_INVALID, "plan or max_norm is NULL");
    if (flags & ~OE_CLIP_DEVFORM) return fail(OE_ERR_INVALID, "oe_clip_grad_norm: unknown flag");
    if (isnan(*max_norm)) return fail(OE_ERR_INVALID, "max_norm is NaN");
    // The in-place clip rewrites the stored gradients; with a pending scale the next kernel
    // would apply the scale a second time. The folded clip of the update kernels is the way.
    if (plan->grad_scale != 1.0f && *max_norm > 0.0f)
        return fail(OE_ERR_INVALID, "oe_clip_grad_norm: in-place clip with a gradient scale other than 1; use the clip folded into the step");
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    if ((rc = check_chunk_count(plan)) != 0) return rc;
    CtxGuard guard(d, plan->dc->ctx);
    if ((rc = launch_sumsq(d, plan, 0, (CUstream)stream)) != 0) return rc;
    if (!(*max_norm > 0.0f) || plan->n_chunks == 0) return 0;  // norm only (autograd/cuda_clip.go:130)
    uint32_t n_chunks = (uint32_t)plan->n_chunks, chunk_elems = plan->chunk_elems;
    float mx = *max_norm;
    void* args[] = {&plan->d_tensors, &plan->d_chunks, &n_chunks, &chunk_elems, &plan->d_norm, &mx, &flags};
    return launch(d, plan->dc->k.scale, "oe_scale_grads", plan->tune_step_grid == 1 ? n_chunks : grid_for(plan, plan->dc->occ_scale),
                  kThreads, (CUstream)stream, args);
}

extern "C" int oe_read_norm(oe_plan* plan, float* norm_out, double* sumsq_out, uint64_t stream) {
    if (!plan) return fail(OE_ERR_INVALID, "plan is NULL");
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    CtxGuard guard(d, plan->dc->ctx);
    oe_dev_norm rec;
    OE_CU(d->cuMemcpyDtoHAsync_(&rec, plan->d_norm, sizeof(rec), (CUstream)stream), "cuMemcpyDtoHAsync(norm)");
    OE_CU(d->cuStreamSynchronize_((CUstream)stream), "cuStreamSynchronize");
    if (norm_out) *norm_out = rec.norm;
    if (sumsq_out) *sumsq_out = rec.sumsq;
    return 0;
}

// -------------------------------------------------------------------------------------
// updates
// -------------------------------------------------------------------------------------
namespace {
int validate_adamw(const oe_plan* p, const oe_adamw_hparams* hp) {
    if (!hp) return fail(OE_ERR_INVALID, "hyper-parameters are NULL");
    if (!finite_nonneg(hp->lr)) return fail(OE_ERR_INVALID, "invalid learning rate");
    if (!(hp->beta1 >= 0.0f && hp->beta1 < 1.0f) || !(hp->beta2 >= 0.0f && hp->beta2 < 1.0f) || !(hp->eps > 0.0f) ||
        !isfinite(hp->eps))
        return fail(OE_ERR_INVALID, "invalid optimizer configuration");
    if (hp->step_dev == 0 && (!(hp->bc1 > 0.0f) || !(hp->bc2 > 0.0f) || !isfinite(hp->bc1) || !isfinite(hp->bc2)))
        return fail(OE_ERR_INVALID, "bias corrections must be positive and finite (step >= 1)");
    if ((hp->step_dev | hp->lr_dev) & 3u) return fail(OE_ERR_INVALID, "step_dev / lr_dev not 4-byte aligned");
    if (isnan(hp->max_norm)) return fail(OE_ERR_INVALID, "max_norm is NaN");
    if (hp->flags & ~(OE_CLIP_DEVFORM | OE_WRITE_SHADOW | OE_ZERO_GRAD))
        return fail(OE_ERR_INVALID, "oe_adamw_step: unknown flag");
    if (!p->all_adamw_state) return fail(OE_ERR_INVALID, "AdamW needs m (state1) and v (state2) for every parameter with a gradient");
    return check_chunk_count(p);
}

int launch_adamw(const oe_driver* d, oe_plan* p, const oe_adamw_hparams* hp, CUstream stream,
                 const oe_peer_set* peers = nullptr, uint64_t first_chunk = 0, uint64_t range_chunks = UINT64_MAX) {
    if (p->n_chunks == 0) {
        // Nothing to update, but a captured step still counts (autograd/nn.go:476-479).
        if (!hp->step_dev) return 0;
        uint64_t sd = hp->step_dev;
        void* inc_args[] = {&sd};
        return launch(d, p->dc->k.step_increment, "oe_step_increment", 1, 32, stream, inc_args);
    }
    oe_adamw_args a;
    memset(&a, 0, sizeof(a));
    a.lr = hp->lr;
    a.beta1 = hp->beta1;
    a.beta2 = hp->beta2;
    a.eps = hp->eps;
    a.bc1 = hp->bc1;
    a.bc2 = hp->bc2;
    a.max_norm = hp->max_norm;
    a.flags = hp->flags;
    a.norm = hp->max_norm > 0.0f ? (uint64_t)p->d_norm : 0;
    a.step_dev = hp->step_dev;
    a.lr_dev = hp->lr_dev;
    a.grad_scale = p->grad_scale;
    a.ticket = (uint64_t)p->d_norm + offsetof(oe_dev_norm, step_ticket);
    a.status = peers ? p->status_word : 0;
    uint32_t n_chunks = (uint32_t)p->n_chunks, chunk_elems = p->chunk_elems;
    CUdeviceptr chunk_table = p->d_chunks;
    if (range_chunks != UINT64_MAX) {  // a contiguous range of the chunk table
        chunk_table += first_chunk * sizeof(oe_dev_chunk);
        n_chunks = (uint32_t)range_chunks;
        if (n_chunks == 0) return 0;
    }
    if (peers) {
        oe_peer_set ps = *peers;
        const uint32_t variant = p->tune_peer_unroll;
        const PeerLaunchShape shape = peer_update_shape(p, p->dc->occ_adamw_peers[variant], ps.n, !(ps.mode & OE_PEER_MULTICAST));
        if (shape.warp_rotate) ps.mode |= OE_PEER_WARP_ROTATE;
        void* peer_args[] = {&p->d_tensors, &chunk_table, &n_chunks, &chunk_elems, &a, &ps};
        return launch(d, p->dc->k.adamw_peers[variant], kAdamwPeerNames[variant], shape.grid, kThreads, stream, peer_args);
    }
    uint32_t grid = grid_for(p, p->dc->occ_adamw[p->variant]);
    if (grid > n_chunks || p->tune_step_grid == 1) grid = n_chunks;
    void* args[] = {&p->d_tensors, &chunk_table, &n_chunks, &chunk_elems, &a};
    return launch(d, p->dc->k.adamw[p->variant], kAdamwNames[p->variant], grid, kThreads, stream, args);
}
}  // namespace

extern "C" int oe_adamw_step(oe_plan* plan, const oe_adamw_hparams* hp, uint64_t stream) {
    if (!plan) return fail(OE_ERR_INVALID, "plan is NULL");
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    if ((rc = validate_adamw(plan, hp)) != 0) return rc;
    CtxGuard guard(d, plan->dc->ctx);
    return launch_adamw(d, plan, hp, (CUstream)stream);
}

extern "C" int oe_adamw_step_chunks(oe_plan* plan, const oe_adamw_hparams* hp, uint64_t first_chunk, uint64_t n_chunks,
                                    uint64_t stream) {
    if (!plan) return fail(OE_ERR_INVALID, "plan is NULL");
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    if ((rc = validate_adamw(plan, hp)) != 0) return rc;
    if (hp->step_dev != 0) return fail(OE_ERR_INVALID, "oe_adamw_step_chunks: a device step counter cannot be split over calls");
    if (first_chunk > plan->n_chunks || n_chunks > plan->n_chunks - first_chunk)
        return fail(OE_ERR_INVALID, "oe_adamw_step_chunks: range outside the plan's work units");
    CtxGuard guard(d, plan->dc->ctx);
    return launch_adamw(d, plan, hp, (CUstream)stream, nullptr, first_chunk, n_chunks);
}

namespace {
int validate_sgd(const oe_plan* plan, const oe_sgd_hparams* hp) {
    if (!plan || !hp) return fail(OE_ERR_INVALID, "plan or hyper-parameters are NULL");
    // SGDOptions.validate (autograd/sgd.go:21-31)
    for (float v : {hp->lr, hp->momentum, hp->dampening})
        if (!finite_nonneg(v)) return fail(OE_ERR_INVALID, "invalid SGD configuration");
    if ((hp->flags & OE_NESTEROV) && (!(hp->momentum > 0.0f) || hp->dampening != 0.0f))
        return fail(OE_ERR_INVALID, "Nesterov needs positive momentum and zero dampening");
    if (isnan(hp->max_norm)) return fail(OE_ERR_INVALID, "max_norm is NaN");
    if (hp->flags & ~(OE_NESTEROV | OE_MAXIMIZE | OE_CLIP_DEVFORM | OE_WRITE_SHADOW | OE_ZERO_GRAD))
        return fail(OE_ERR_INVALID, "oe_sgd_step: unknown flag");
    if (hp->momentum > 0.0f) {
        for (const oe_tensor_desc& x : plan->descs)
            if (x.grad != 0 && (x.state1 == 0 || x.state2 == 0))
                return fail(OE_ERR_INVALID, "incomplete SGD device storage: momentum needs a buffer and a flag per parameter");
    }
    if ((hp->step_dev | hp->lr_dev) & 3u) return fail(OE_ERR_INVALID, "step_dev / lr_dev not 4-byte aligned");
    return check_chunk_count(plan);
}

int sgd_step(oe_plan* plan, const oe_sgd_hparams* hp, uint64_t stream, const oe_peer_set* peers) {
    int rc = validate_sgd(plan, hp);
    if (rc) return rc;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    CtxGuard guard(d, plan->dc->ctx);
    if (plan->n_chunks == 0) {
        if (!hp->step_dev) return 0;
        uint64_t sd = hp->step_dev;
        void* inc_args[] = {&sd};
        return launch(d, plan->dc->k.step_increment, "oe_step_increment", 1, 32, (CUstream)stream, inc_args);
    }
    oe_sgd_args a;
    memset(&a, 0, sizeof(a));
    a.lr = hp->lr;
    a.momentum = hp->momentum;
    a.dampening = hp->dampening;
    a.max_norm = hp->max_norm;
    a.flags = hp->flags;
    a.norm = hp->max_norm > 0.0f ? (uint64_t)plan->d_norm : 0;
    a.lr_dev = hp->lr_dev;
    a.grad_scale = plan->grad_scale;
    a.step_dev = hp->step_dev;
    a.ticket = (uint64_t)plan->d_norm + offsetof(oe_dev_norm, step_ticket);
    a.n_tensors = plan->n_active;
    a.status = peers ? plan->status_word : 0;
    uint32_t n_chunks = (uint32_t)plan->n_chunks, chunk_elems = plan->chunk_elems;
    if (peers) {
        oe_peer_set ps = *peers;
        const PeerLaunchShape shape = peer_update_shape(plan, plan->dc->occ_sgd_peers, ps.n, false);  // not measured for SGD: knobs only
        if (shape.warp_rotate) ps.mode |= OE_PEER_WARP_ROTATE;
        void* peer_args[] = {&plan->d_tensors, &plan->d_chunks, &n_chunks, &chunk_elems, &a, &ps};
        return launch(d, plan->dc->k.sgd_peers, "oe_sgd_fused_peers", shape.grid, kThreads, (CUstream)stream, peer_args);
    }
    void* args[] = {&plan->d_tensors, &plan->d_chunks, &n_chunks, &chunk_elems, &a};
    return launch(d, plan->dc->k.sgd, "oe_sgd_fused", plan->tune_step_grid == 1 ? n_chunks : grid_for(plan, plan->dc->occ_sgd),
                  kThreads, (CUstream)stream, args);
}

int peer_set_from(const int64_t* shadow_deltas, uint32_t n_ranks, const char* who, oe_peer_set* ps,
                  const int64_t* mc_delta = nullptr) {
    if (!shadow_deltas) return fail(OE_ERR_INVALID, std::string(who) + ": NULL argument");
    if (n_ranks < 1 || n_ranks > OE_MAX_PEERS) return fail(OE_ERR_LIMIT, std::string(who) + ": 1 to 8 ranks are supported");
    memset(ps, 0, sizeof(*ps));
    ps->n = n_ranks;
    for (uint32_t k = 0; k < n_ranks; k++) {
        if (shadow_deltas[k] & 1) return fail(OE_ERR_INVALID, std::string(who) + ": odd byte distance to a bf16 buffer");
        // an 8-byte store needs every target as aligned as the local one
        if (shadow_deltas[k] & 7) return fail(OE_ERR_INVALID, std::string(who) + ": shadow buffers must be mutually 8-byte aligned");
        ps->delta[k] = shadow_deltas[k];
    }
    if (mc_delta) {
        if (*mc_delta == 0 || (*mc_delta & 7)) return fail(OE_ERR_INVALID, std::string(who) + ": bad distance to the multicast mapping");
        ps->mode |= OE_PEER_MULTICAST;
        ps->mc_delta = *mc_delta;
    }
    return 0;
}
}  // namespace

extern "C" int oe_sgd_step(oe_plan* plan, const oe_sgd_hparams* hp, uint64_t stream) {
    return sgd_step(plan, hp, stream, nullptr);
}

extern "C" int oe_sgd_step_peers(oe_plan* plan, const oe_sgd_hparams* hp, const int64_t* shadow_deltas, uint32_t n_ranks,
                                 uint64_t stream) {
    oe_peer_set ps;
    int rc = peer_set_from(shadow_deltas, n_ranks, "oe_sgd_step_peers", &ps);
    if (rc) return rc;
    return sgd_step(plan, hp, stream, &ps);
}

extern "C" int oe_zero_grads(oe_plan* plan, uint64_t stream) {
    if (!plan) return fail(OE_ERR_INVALID, "plan is NULL");
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    if ((rc = check_chunk_count(plan)) != 0) return rc;
    if (plan->n_chunks == 0) return 0;
    CtxGuard guard(d, plan->dc->ctx);
    uint32_t n_chunks = (uint32_t)plan->n_chunks, chunk_elems = plan->chunk_elems;
    void* args[] = {&plan->d_tensors, &plan->d_chunks, &n_chunks, &chunk_elems};
    // One CTA per work unit, dispatched in table order: for a write-only stream a compact window that
    // sweeps the addresses in order measured 7.5 TB/s on B200 against 6.1 TB/s for a persistent grid
    // whose CTAs drift apart (the read-modify-write kernels measured the same either way).
    return launch(d, plan->dc->k.zero, "oe_zero_grads", n_chunks, kThreads, (CUstream)stream, args);
}

extern "C" int oe_cast_bf16(int device, uint64_t src, uint64_t dst, uint64_t numel, uint64_t stream) {
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    DeviceCtx* dc = device_or_fail(device, &rc);
    if (!dc) return rc;
    if (numel == 0) return 0;  // an empty launch is not an error (kernels/kernels_test.go:153-174)
    if (src == 0 || dst == 0 || (src & 3u) || (dst & 1u)) return fail(OE_ERR_INVALID, "oe_cast_bf16: bad address");
    CtxGuard guard(d, dc->ctx);
    // One CTA per tile of 256 threads x 4 vectors x 4 elements, in address order (see the kernel: a
    // compact window sweeping the buffer beats a persistent grid by a quarter for this stream).
    uint64_t blocks = (numel + 4095) / 4096;
    uint32_t grid = (uint32_t)(blocks < 0x7fffffffull ? blocks : 0x7fffffffull);
    void* args[] = {&src, &dst, &numel};
    return launch(d, dc->k.cast, "oe_cast_bf16", grid, kThreads, (CUstream)stream, args);
}

extern "C" int oe_adamw_step_from_host(oe_plan* plan, const oe_adamw_hparams* hp, const float* const* host_grads,
                                       uint32_t n_tensors, float* norm_out, uint64_t stream) {
    if (!plan) return fail(OE_ERR_INVALID, "plan is NULL");
    if (n_tensors != plan->descs.size()) return fail(OE_ERR_INVALID, "host gradient count differs from the plan's");
    if (n_tensors > 0 && !host_grads) return fail(OE_ERR_INVALID, "host_grads is NULL");
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    if ((rc = validate_adamw(plan, hp)) != 0) return rc;
    CtxGuard guard(d, plan->dc->ctx);
    CUstream s = (CUstream)stream;
    for (uint32_t i = 0; i < n_tensors; i++) {
        const oe_tensor_desc& x = plan->descs[i];
        if (x.grad == 0 || host_grads[i] == nullptr) continue;
        OE_CU(d->cuMemcpyHtoDAsync_((CUdeviceptr)x.grad, host_grads[i], x.numel * sizeof(float), s),
              "cuMemcpyHtoDAsync(gradient)");
    }
    if ((rc = launch_sumsq(d, plan, 0, s)) != 0) return rc;
    if ((rc = launch_adamw(d, plan, hp, s)) != 0) return rc;
    oe_dev_norm rec;
    OE_CU(d->cuMemcpyDtoHAsync_(&rec, plan->d_norm, sizeof(rec), s), "cuMemcpyDtoHAsync(norm)");
    OE_CU(d->cuStreamSynchronize_(s), "cuStreamSynchronize");
    if (norm_out) *norm_out = rec.norm;
    return 0;
}

// -------------------------------------------------------------------------------------
// launch counters
// -------------------------------------------------------------------------------------
extern "C" int64_t oe_launch_count(const char* kernel_name) {
    std::lock_guard<std::mutex> lock(g_mu);
    int64_t total = 0;
    for (const auto& kv : g_launches)
        if (!kernel_name || kv.first == kernel_name) total += kv.second;
    return total;
}

extern "C" void oe_launch_count_reset(void) {
    std::lock_guard<std::mutex> lock(g_mu);
    g_launches.clear();
}

extern "C" void oe_profile_enable(int enabled) {
    if (enabled) {  // enabling starts a fresh profile, as EnableGPUProfile(true) does
        std::lock_guard<std::mutex> lock(g_mu);
        g_profile_ms.clear();
        g_launches.clear();
    }
    g_profiling.store(enabled != 0);
}

extern "C" int oe_profile_get(const char* kernel_name, int64_t* count_out, double* ms_out) {
    std::lock_guard<std::mutex> lock(g_mu);
    int64_t count = 0;
    double ms = 0.0;
    for (const auto& kv : g_launches)
        if (!kernel_name || kv.first == kernel_name) count += kv.second;
    for (const auto& kv : g_profile_ms)
        if (!kernel_name || kv.first == kernel_name) ms += kv.second;
    if (count_out) *count_out = count;
    if (ms_out) *ms_out = ms;
    return 0;
}

// -------------------------------------------------------------------------------------
// device plumbing
// -------------------------------------------------------------------------------------
#define OE_DEVICE_PROLOGUE                          \
    int rc = 0;                                     \
    const oe_driver* d = driver_or_fail(&rc);       \
    if (!d) return rc;                              \
    DeviceCtx* dc = device_or_fail(device, &rc);    \
    if (!dc) return rc;                             \
    CtxGuard guard(d, dc->ctx)

extern "C" int oe_mem_alloc(int device, uint64_t bytes, uint64_t* address_out) {
    if (!address_out || bytes == 0) return fail(OE_ERR_INVALID, "oe_mem_alloc: bad argument");
    OE_DEVICE_PROLOGUE;
    CUdeviceptr p = 0;
    OE_CU(d->cuMemAlloc_(&p, bytes), "cuMemAlloc");
    *address_out = (uint64_t)p;
    return 0;
}
extern "C" int oe_mem_free(int device, uint64_t address) {
    if (address == 0) return 0;
    OE_DEVICE_PROLOGUE;
    OE_CU(d->cuMemFree_((CUdeviceptr)address), "cuMemFree");
    return 0;
}
extern "C" int oe_mem_info(int device, uint64_t* free_out, uint64_t* total_out) {
    OE_DEVICE_PROLOGUE;
    size_t f = 0, t = 0;
    OE_CU(d->cuMemGetInfo_(&f, &t), "cuMemGetInfo");
    if (free_out) *free_out = f;
    if (total_out) *total_out = t;
    return 0;
}
extern "C" int oe_memcpy_h2d(int device, uint64_t dst, const void* src, uint64_t bytes, uint64_t stream) {
    if (bytes == 0) return 0;
    if (!dst || !src) return fail(OE_ERR_INVALID, "oe_memcpy_h2d: NULL address");
    OE_DEVICE_PROLOGUE;
    OE_CU(d->cuMemcpyHtoDAsync_((CUdeviceptr)dst, src, bytes, (CUstream)stream), "cuMemcpyHtoDAsync");
    return 0;
}
extern "C" int oe_memcpy_d2h(int device, void* dst, uint64_t src, uint64_t bytes, uint64_t stream) {
    if (bytes == 0) return 0;
    if (!dst || !src) return fail(OE_ERR_INVALID, "oe_memcpy_d2h: NULL address");
    OE_DEVICE_PROLOGUE;
    OE_CU(d->cuMemcpyDtoHAsync_(dst, (CUdeviceptr)src, bytes, (CUstream)stream), "cuMemcpyDtoHAsync");
    return 0;
}
extern "C" int oe_memcpy_d2d(int device, uint64_t dst, uint64_t src, uint64_t bytes, uint64_t stream) {
    if (bytes == 0) return 0;
    if (!dst || !src) return fail(OE_ERR_INVALID, "oe_memcpy_d2d: NULL address");
    OE_DEVICE_PROLOGUE;
    // the unified-address form: either side may be a peer's buffer mapped on this device
    OE_CU(d->cuMemcpyAsync_((CUdeviceptr)dst, (CUdeviceptr)src, bytes, (CUstream)stream), "cuMemcpyAsync");
    return 0;
}
extern "C" int oe_memset_u32(int device, uint64_t dst, uint32_t value, uint64_t count, uint64_t stream) {
    if (count == 0) return 0;
    if (!dst || (dst & 3u)) return fail(OE_ERR_INVALID, "oe_memset_u32: bad address");
    OE_DEVICE_PROLOGUE;
    OE_CU(d->cuMemsetD32Async_((CUdeviceptr)dst, value, count, (CUstream)stream), "cuMemsetD32Async");
    return 0;
}
extern "C" int oe_host_alloc(int device, uint64_t bytes, void** out) {
    if (!out || bytes == 0) return fail(OE_ERR_INVALID, "oe_host_alloc: bad argument");
    OE_DEVICE_PROLOGUE;
    OE_CU(d->cuMemAllocHost_(out, bytes), "cuMemAllocHost");
    return 0;
}
extern "C" int oe_host_free(int device, void* ptr) {
    if (!ptr) return 0;
    OE_DEVICE_PROLOGUE;
    OE_CU(d->cuMemFreeHost_(ptr), "cuMemFreeHost");
    return 0;
}
extern "C" int oe_stream_create(int device, uint64_t* stream_out) {
    if (!stream_out) return fail(OE_ERR_INVALID, "stream_out is NULL");
    OE_DEVICE_PROLOGUE;
    CUstream s = nullptr;
    OE_CU(d->cuStreamCreate_(&s, CU_STREAM_NON_BLOCKING), "cuStreamCreate");
    *stream_out = (uint64_t)s;
    return 0;
}
extern "C" int oe_stream_destroy(int device, uint64_t stream) {
    if (!stream) return 0;
    OE_DEVICE_PROLOGUE;
    OE_CU(d->cuStreamDestroy_((CUstream)stream), "cuStreamDestroy");
    return 0;
}
extern "C" int oe_stream_sync(int device, uint64_t stream) {
    OE_DEVICE_PROLOGUE;
    OE_CU(d->cuStreamSynchronize_((CUstream)stream), "cuStreamSynchronize");
    return 0;
}
extern "C" int oe_event_create(int device, uint64_t* event_out) {
    if (!event_out) return fail(OE_ERR_INVALID, "event_out is NULL");
    OE_DEVICE_PROLOGUE;
    CUevent e = nullptr;
    OE_CU(d->cuEventCreate_(&e, CU_EVENT_DEFAULT), "cuEventCreate");
    *event_out = (uint64_t)e;
    return 0;
}
extern "C" int oe_event_destroy(int device, uint64_t event) {
    if (!event) return 0;
    OE_DEVICE_PROLOGUE;
    OE_CU(d->cuEventDestroy_((CUevent)event), "cuEventDestroy");
    return 0;
}
extern "C" int oe_event_record(int device, uint64_t event, uint64_t stream) {
    OE_DEVICE_PROLOGUE;
    OE_CU(d->cuEventRecord_((CUevent)event, (CUstream)stream), "cuEventRecord");
    return 0;
}
extern "C" int oe_event_sync(int device, uint64_t event) {
    OE_DEVICE_PROLOGUE;
    OE_CU(d->cuEventSynchronize_((CUevent)event), "cuEventSynchronize");
    return 0;
}
extern "C" int oe_event_elapsed_ms(int device, uint64_t start, uint64_t stop, float* ms_out) {
    if (!ms_out) return fail(OE_ERR_INVALID, "ms_out is NULL");
    OE_DEVICE_PROLOGUE;
    OE_CU(d->cuEventElapsedTime_(ms_out, (CUevent)start, (CUevent)stop), "cuEventElapsedTime");
    return 0;
}

// -------------------------------------------------------------------------------------
// sharded step (ZeRO-1 style): peer-memory kernels and the IPC plumbing they need
// -------------------------------------------------------------------------------------
namespace {
int peer_reduce(oe_plan* plan, const uint64_t* rank_bases, uint32_t n_ranks, uint64_t first_elem, uint64_t numel, uint64_t out,
                const float* scale, uint32_t flags, uint64_t stream);
}

extern "C" int oe_peer_reduce_grads(oe_plan* plan, const uint64_t* rank_bases, uint32_t n_ranks, uint64_t first_elem,
                                    uint64_t numel, uint64_t out, const float* scale, uint32_t flags, uint64_t stream) {
    if (flags & ~(OE_PARTIAL_ONLY | OE_ACCUMULATE)) return fail(OE_ERR_INVALID, "oe_peer_reduce_grads: unknown flag");
    return peer_reduce(plan, rank_bases, n_ranks, first_elem, numel, out, scale, flags, stream);
}

namespace {
// flags may carry the kernel-side bits of oe_table.h beside the public ones
int peer_reduce(oe_plan* plan, const uint64_t* rank_bases, uint32_t n_ranks, uint64_t first_elem, uint64_t numel, uint64_t out,
                const float* scale, uint32_t flags, uint64_t stream) {
    if (!plan || !rank_bases || !scale) return fail(OE_ERR_INVALID, "oe_peer_reduce_grads: NULL argument");
    if (n_ranks < 1 || n_ranks > OE_MAX_PEERS) return fail(OE_ERR_LIMIT, "oe_peer_reduce_grads: 1 to 8 ranks are supported");
    if (!isfinite(*scale)) return fail(OE_ERR_INVALID, "oe_peer_reduce_grads: scale is not finite");
    // This kernel writes the scaled sum in place and takes its own factor; a plan-level scale
    // would be applied again by the update that follows.
    if (plan->grad_scale != 1.0f)
        return fail(OE_ERR_INVALID, "oe_peer_reduce_grads: the plan has a gradient scale other than 1; fold it into this call's scale");
    if (numel > 0 && (out == 0 || (out & 3u))) return fail(OE_ERR_INVALID, "oe_peer_reduce_grads: bad output address");
    oe_peer_grads pg;
    memset(&pg, 0, sizeof(pg));
    pg.n = n_ranks;
    pg.flags = flags;
    pg.scale = *scale;
    pg.rot = plan->tune_reduce_first;
    if (plan->tune_reduce_warp_rotate) pg.flags |= OE_F_WARP_ROTATE;
    pg.status = plan->status_word;
    for (uint32_t k = 0; k < n_ranks; k++) {
        if (rank_bases[k] == 0 || (rank_bases[k] & 3u)) return fail(OE_ERR_INVALID, "oe_peer_reduce_grads: bad gradient base of rank " + std::to_string(k));
        pg.base[k] = rank_bases[k];
    }
    for (uint32_t k = n_ranks; k < OE_MAX_PEERS; k++) pg.base[k] = rank_bases[0];
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    DeviceCtx* dc = plan->dc;
    CtxGuard guard(d, dc->ctx);
    int which = n_ranks <= 2 ? 0 : n_ranks <= 4 ? 1 : 2;
    static const char* const names[3] = {"oe_peer_reduce_sumsq_n2", "oe_peer_reduce_sumsq_n4", "oe_peer_reduce_sumsq_n8"};
    uint64_t vec_threads = numel / 4 / 2 + 1;
    uint64_t blocks = (vec_threads + kThreads - 1) / kThreads;
    uint64_t persistent = (uint64_t)dc->sm_count * (uint64_t)(dc->occ_peer_reduce[which] > 0 ? dc->occ_peer_reduce[which] : 1);
    uint64_t grid = blocks < persistent ? blocks : persistent;
    if (grid > plan->max_grid) grid = plan->max_grid;
    if (plan->tune_reduce_grid && plan->tune_reduce_grid < grid) grid = plan->tune_reduce_grid;
    if (grid == 0) grid = 1;
    void* args[] = {&pg, &first_elem, &numel, &out, &plan->d_norm, &plan->d_partials};
    return launch(d, dc->k.peer_reduce[which], names[which], (uint32_t)grid, kThreads, (CUstream)stream, args);
}
}  // namespace

extern "C" int oe_link_probe_reads(oe_plan* plan, const uint64_t* rank_bases, uint32_t n_ranks, uint64_t first_elem,
                                   uint64_t numel, uint64_t stream) {
    if (!plan || !rank_bases) return fail(OE_ERR_INVALID, "oe_link_probe_reads: NULL argument");
    // the pull-reduce with its stores switched off: every load of the real launch, nothing written but the plan's norm record
    const float one = 1.0f;
    uint64_t anywhere = rank_bases[0] + 4ull * first_elem;
    return peer_reduce(plan, rank_bases, n_ranks, first_elem, numel, anywhere, &one, OE_PARTIAL_ONLY | OE_F_NO_STORE, stream);
}

extern "C" int oe_link_probe_stores(oe_plan* plan, uint64_t shadow_shard, const int64_t* shadow_deltas, uint32_t n_ranks,
                                    uint64_t numel, uint64_t stream) {
    if (!plan || !shadow_deltas) return fail(OE_ERR_INVALID, "oe_link_probe_stores: NULL argument");
    if (shadow_shard == 0 || (shadow_shard & 7u) || (numel & 3u))
        return fail(OE_ERR_INVALID, "oe_link_probe_stores: the range must start on an 8-byte boundary and hold a multiple of 4 elements");
    oe_peer_set all;
    int rc = peer_set_from(shadow_deltas, n_ranks, "oe_link_probe_stores", &all);
    if (rc) return rc;
    oe_peer_set ps;   // every target but the caller's own buffer
    memset(&ps, 0, sizeof(ps));
    for (uint32_t k = 0; k < all.n; k++)
        if (all.delta[k] != 0) ps.delta[ps.n++] = all.delta[k];
    if (ps.n == 0 || numel == 0) return 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    CtxGuard guard(d, plan->dc->ctx);
    const PeerLaunchShape shape = peer_update_shape(plan, plan->dc->occ_adamw_peers[0], n_ranks, true);
    if (shape.warp_rotate) ps.mode |= OE_PEER_WARP_ROTATE;
    uint64_t n_vec = numel / 4;
    uint64_t tiles = (n_vec + 1023) / 1024;
    uint32_t grid = (uint32_t)(tiles < shape.grid ? tiles : shape.grid);
    void* args[] = {&shadow_shard, &n_vec, &ps};
    return launch(d, plan->dc->k.probe_stores, "oe_probe_peer_stores", grid ? grid : 1, kThreads, (CUstream)stream, args);
}

extern "C" int oe_adamw_step_peers(oe_plan* plan, const oe_adamw_hparams* hp, const int64_t* shadow_deltas,
                                   uint32_t n_ranks, uint64_t stream) {
    if (!plan) return fail(OE_ERR_INVALID, "oe_adamw_step_peers: NULL argument");
    oe_peer_set ps;
    int rc = peer_set_from(shadow_deltas, n_ranks, "oe_adamw_step_peers", &ps);
    if (rc) return rc;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    if ((rc = validate_adamw(plan, hp)) != 0) return rc;
    CtxGuard guard(d, plan->dc->ctx);
    return launch_adamw(d, plan, hp, (CUstream)stream, &ps);
}

extern "C" int oe_adamw_step_multicast(oe_plan* plan, const oe_adamw_hparams* hp, const int64_t* shadow_deltas,
                                       uint32_t n_ranks, const int64_t* mc_delta, uint64_t stream) {
    if (!plan || !mc_delta) return fail(OE_ERR_INVALID, "oe_adamw_step_multicast: NULL argument");
    oe_peer_set ps;
    int rc = peer_set_from(shadow_deltas, n_ranks, "oe_adamw_step_multicast", &ps, mc_delta);
    if (rc) return rc;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    if ((rc = validate_adamw(plan, hp)) != 0) return rc;
    CtxGuard guard(d, plan->dc->ctx);
    return launch_adamw(d, plan, hp, (CUstream)stream, &ps);
}

extern "C" int oe_sgd_step_multicast(oe_plan* plan, const oe_sgd_hparams* hp, const int64_t* shadow_deltas,
                                     uint32_t n_ranks, const int64_t* mc_delta, uint64_t stream) {
    if (!mc_delta) return fail(OE_ERR_INVALID, "oe_sgd_step_multicast: NULL argument");
    oe_peer_set ps;
    int rc = peer_set_from(shadow_deltas, n_ranks, "oe_sgd_step_multicast", &ps, mc_delta);
    if (rc) return rc;
    return sgd_step(plan, hp, stream, &ps);
}

// -------------------------------------------------------------------------------------
// sharded step driven by the library alone: the exchanges between the ranks are kernels too
// -------------------------------------------------------------------------------------
struct oe_zero1 {
    oe_plan* plan = nullptr;
    oe_zero1_desc desc;
    uint32_t epoch = 0;
    float mean_scale = 1.0f;
    // copy-engine assistance, resolved from the descriptor when the context is made
    uint32_t ce_pull = 0;      // peers whose range a copy stages before the pull kernel
    bool ce_pull_writes = false;  // the staged ranges are written by their owners into this rank's staging
    uint32_t staged_count = 0;    // reduce phases begun in that form: the epoch of the staging exchange
    uint64_t ce_slot = 0;      // bytes of one staged range
    uint32_t ce_push = 0;      // ranks served by a copy after the update kernel
    bool ce_push_auto = false; // the library chose: small shards stay on the kernel's stores
    int64_t runs_for_upload = -1;                      // plan->uploads the runs below were derived from
    std::vector<std::pair<uint64_t, uint64_t>> runs;   // this rank's shadow values as (address, bytes) ranges
};

namespace {
int launch_exchange(const oe_driver* d, oe_zero1* z, uint32_t phase, bool with_norm, CUstream stream) {
    oe_sync_args a;
    memset(&a, 0, sizeof(a));
    a.rank = z->desc.rank;
    a.world = z->desc.world;
    a.phase = phase;
    // the staging exchange counts the reduce phases (one per step, more when a caller times the phase on its own)
    a.epoch = phase == OE_SYNC_STAGED ? z->staged_count : z->epoch;
    for (uint32_t k = 0; k < OE_MAX_PEERS; k++) a.block[k] = z->desc.sync_blocks[k < z->desc.world ? k : z->desc.rank];
    a.norm_rec = with_norm ? (uint64_t)z->plan->d_norm : 0;
    uint64_t ms = z->desc.timeout_ms ? z->desc.timeout_ms : 10000u;
    a.timeout_ns = ms * 1000000ull;
    uint64_t polls = ms * 4000ull;  // a poll takes a microsecond or so once the wait backs off
    a.max_polls = polls > 0x7fffffffull ? 0x7fffffffu : (uint32_t)polls;
    void* args[] = {&a};
    return launch(d, z->plan->dc->k.rank_exchange, "oe_rank_exchange", 1, 32, stream, args);
}

constexpr size_t kMaxShadowRuns = 64;                  // more ranges than this per target: the kernel stores them itself
constexpr uint64_t kCopyEngineMinBytes = 64ull << 20;  // the library's own choice leaves smaller shards to the kernels

// The bf16 shadow values this rank's update writes, as maximal contiguous ranges of its shadow buffer.
void shadow_runs(oe_zero1* z) {
    const oe_plan* plan = z->plan;
    if (z->runs_for_upload == plan->uploads) return;
    z->runs.clear();
    std::vector<std::pair<uint64_t, uint64_t>> pieces;
    for (const oe_tensor_desc& t : plan->descs)
        if (t.grad && t.shadow) pieces.emplace_back(t.shadow, 2ull * t.numel);
    std::sort(pieces.begin(), pieces.end());
    for (const auto& p : pieces) {
        if (!z->runs.empty() && z->runs.back().first + z->runs.back().second == p.first)
            z->runs.back().second += p.second;
        else
            z->runs.push_back(p);
    }
    z->runs_for_upload = plan->uploads;
}

// The reduce phase: staged copies (if any), then the pull kernel that leaves the mean in place and this
// rank's partial sum of squares in the plan's norm record.
int zero1_reduce(const oe_driver* d, oe_zero1* z, uint64_t stream) {
    const oe_zero1_desc& D = z->desc;
    oe_plan* plan = z->plan;
    CUstream s = (CUstream)stream;
    uint64_t out = D.grad_bases[D.rank] + 4ull * D.first_elem;
    uint64_t bases[OE_MAX_PEERS];
    for (uint32_t k = 0; k < OE_MAX_PEERS; k++) bases[k] = D.grad_bases[k];
    if (z->ce_pull && D.numel && !z->ce_pull_writes) {
        // Window j: every rank copies from the rank j+1 places after it, so each GPU serves one reader at a
        // time. The pull kernel then finds those ranges in local memory, under the source rank's slot of the sum.
        CtxGuard guard(d, plan->dc->ctx);
        for (uint32_t j = 0; j < z->ce_pull; j++) {
            const uint32_t src = (D.rank + 1 + j) % D.world;
            const uint64_t dst = D.staging + (uint64_t)j * z->ce_slot;
            OE_CU(d->cuMemcpyAsync_((CUdeviceptr)dst, (CUdeviceptr)(D.grad_bases[src] + 4ull * D.first_elem), 4ull * D.numel, s),
                  "cuMemcpyAsync(stage gradients)");
            bases[src] = dst - 4ull * D.first_elem;
        }
    } else if (z->ce_pull && D.numel) {
        // The same windows with the copies going the other way: in window j this rank writes the range that
        // belongs to the rank j+1 places after it into slot j of that rank's staging, so each GPU serves one
        // writer at a time; slot j of this rank's staging is filled by the rank j+1 places BEFORE it. An
        // exchange tells every rank that its staging is complete.
        {
            CtxGuard guard(d, plan->dc->ctx);
            for (uint32_t j = 0; j < z->ce_pull; j++) {
                const uint32_t to = (D.rank + 1 + j) % D.world;
                const uint64_t dst = D.staging_bases[to] + (uint64_t)j * z->ce_slot;
                const uint64_t src = D.grad_bases[D.rank] + 4ull * D.numel * to;
                OE_CU(d->cuMemcpyAsync_((CUdeviceptr)dst, (CUdeviceptr)src, 4ull * D.numel, s), "cuMemcpyAsync(stage gradients at the owner)");
                const uint32_t from = (D.rank + D.world - 1 - j) % D.world;
                bases[from] = D.staging + (uint64_t)j * z->ce_slot - 4ull * D.first_elem;
            }
            z->staged_count += 1;
            int rc = launch_exchange(d, z, OE_SYNC_STAGED, false, s);
            if (rc) return rc;
        }
    }
    return oe_peer_reduce_grads(plan, bases, D.world, D.first_elem, D.numel, out, &z->mean_scale, OE_PARTIAL_ONLY, stream);
}

// The update phase: the fused update storing the shadow to this rank and the next `stored` ranks, then copies
// of this rank's shadow ranges to the remaining ones.
int zero1_update(const oe_driver* d, oe_zero1* z, const oe_adamw_hparams* ahp, const oe_sgd_hparams* shp, uint64_t stream) {
    const oe_zero1_desc& D = z->desc;
    oe_plan* plan = z->plan;
    CUstream s = (CUstream)stream;
    const int64_t* mc = D.shadow_mc_delta ? &D.shadow_mc_delta : nullptr;
    const uint32_t hp_flags = ahp ? ahp->flags : shp->flags;
    uint32_t copied = (mc || !(hp_flags & OE_WRITE_SHADOW)) ? 0 : z->ce_push;   // no shadow written: nothing to deliver
    if (copied) {
        shadow_runs(z);
        uint64_t bytes = 0;
        for (const auto& r : z->runs) bytes += r.second;
        if (z->runs.empty() || z->runs.size() > kMaxShadowRuns || (z->ce_push_auto && bytes < kCopyEngineMinBytes)) copied = 0;
    }
    const uint32_t stored = D.world - 1 - copied;
    int64_t deltas[OE_MAX_PEERS];
    deltas[0] = 0;
    for (uint32_t j = 0; j < stored; j++) deltas[1 + j] = D.shadow_deltas[(D.rank + 1 + j) % D.world];
    const int64_t* use = copied ? deltas : D.shadow_deltas;
    const uint32_t n_use = copied ? stored + 1 : D.world;
    int rc;
    if (ahp)
        rc = mc ? oe_adamw_step_multicast(plan, ahp, D.shadow_deltas, D.world, mc, stream) : oe_adamw_step_peers(plan, ahp, use, n_use, stream);
    else
        rc = mc ? oe_sgd_step_multicast(plan, shp, D.shadow_deltas, D.world, mc, stream) : oe_sgd_step_peers(plan, shp, use, n_use, stream);
    if (rc || !copied) return rc;
    // After an exchange that gave up the kernel above did nothing, and these copies carry the values every
    // rank already holds.
    CtxGuard guard(d, plan->dc->ctx);
    for (uint32_t j = stored; j + 1 < D.world; j++) {
        const int64_t delta = D.shadow_deltas[(D.rank + 1 + j) % D.world];
        for (const auto& r : z->runs)
            OE_CU(d->cuMemcpyAsync_((CUdeviceptr)(r.first + (uint64_t)delta), (CUdeviceptr)r.first, r.second, s), "cuMemcpyAsync(shadow)");
    }
    return 0;
}

int zero1_phase_prologue(oe_zero1* z, const oe_adamw_hparams* ahp, const oe_sgd_hparams* shp, const oe_driver** d_out) {
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    // everything that can be refused is checked before the first launch
    if (ahp && (rc = validate_adamw(z->plan, ahp)) != 0) return rc;
    if (shp && (rc = validate_sgd(z->plan, shp)) != 0) return rc;
    *d_out = d;
    return 0;
}

int zero1_step(oe_zero1* z, const oe_adamw_hparams* ahp, const oe_sgd_hparams* shp, uint64_t stream) {
    if (!z || (!ahp && !shp)) return fail(OE_ERR_INVALID, "oe_zero1 step: NULL argument");
    const oe_driver* d = nullptr;
    int rc = zero1_phase_prologue(z, ahp, shp, &d);
    if (rc) return rc;
    oe_plan* plan = z->plan;
    CUstream s = (CUstream)stream;
    z->epoch += 1;
    {
        CtxGuard guard(d, plan->dc->ctx);
        if (!(z->desc.flags & OE_ZERO1_NO_ENTRY_EXCHANGE) && (rc = launch_exchange(d, z, OE_SYNC_GRADS_READY, false, s)) != 0) return rc;
    }
    if ((rc = zero1_reduce(d, z, stream)) != 0) return rc;
    {
        CtxGuard guard(d, plan->dc->ctx);
        if ((rc = launch_exchange(d, z, OE_SYNC_REDUCED, true, s)) != 0) return rc;
    }
    if ((rc = zero1_update(d, z, ahp, shp, stream)) != 0) return rc;
    CtxGuard guard(d, plan->dc->ctx);
    return launch_exchange(d, z, OE_SYNC_PUSHED, false, s);
}
}  // namespace

extern "C" int oe_zero1_create(oe_plan* plan, const oe_zero1_desc* desc, oe_zero1** out) {
    if (!out) return fail(OE_ERR_INVALID, "out is NULL");
    *out = nullptr;
    if (!plan || !desc) return fail(OE_ERR_INVALID, "oe_zero1_create: NULL argument");
    if (desc->world < 1 || desc->world > OE_MAX_PEERS) return fail(OE_ERR_LIMIT, "oe_zero1_create: 1 to 8 ranks are supported");
    if (desc->rank >= desc->world) return fail(OE_ERR_INVALID, "oe_zero1_create: rank out of range");
    if (desc->flags & ~OE_ZERO1_NO_ENTRY_EXCHANGE) return fail(OE_ERR_INVALID, "oe_zero1_create: unknown flag");
    for (uint32_t k = 0; k < desc->world; k++) {
        if (desc->grad_bases[k] == 0 || (desc->grad_bases[k] & 3u))
            return fail(OE_ERR_INVALID, "oe_zero1_create: bad gradient base of rank " + std::to_string(k));
        if (desc->sync_blocks[k] == 0 || (desc->sync_blocks[k] & 255u))
            return fail(OE_ERR_INVALID, "oe_zero1_create: exchange area of rank " + std::to_string(k) + " missing or not 256-byte aligned");
        if (desc->shadow_deltas[k] & 7) return fail(OE_ERR_INVALID, "oe_zero1_create: shadow buffers must be mutually 8-byte aligned");
    }
    if (desc->shadow_deltas[desc->rank] != 0) return fail(OE_ERR_INVALID, "oe_zero1_create: the rank's own shadow distance must be 0");
    if (plan->status_word != 0) return fail(OE_ERR_INVALID, "oe_zero1_create: the plan already drives a sharded step");
    // copy-engine assistance: an explicit request is honoured or refused, the library's own choice adapts
    const uint32_t others = desc->world - 1;
    const uint64_t slot = (4ull * desc->numel + 255ull) & ~255ull;
    if (desc->staging & 15u) return fail(OE_ERR_INVALID, "oe_zero1_create: staging must be 16-byte aligned");
    const uint64_t slots = (desc->staging && slot) ? desc->staging_bytes / slot : 0;
    uint32_t pull = 0, push = 0;
    if (desc->ce_pull_sources == 0) {
        if (desc->world >= 4 && 4ull * desc->numel >= kCopyEngineMinBytes) pull = (uint32_t)std::min<uint64_t>(others - 1, slots);
    } else if (desc->ce_pull_sources != OE_ZERO1_CE_NONE) {
        if (desc->ce_pull_sources > others) return fail(OE_ERR_INVALID, "oe_zero1_create: ce_pull_sources exceeds the number of peers");
        if (desc->ce_pull_sources > slots)
            return fail(OE_ERR_INVALID, "oe_zero1_create: staging holds " + std::to_string(slots) + " gradient ranges of " +
                                            std::to_string(slot) + " bytes, ce_pull_sources asks for " + std::to_string(desc->ce_pull_sources));
        pull = desc->ce_pull_sources;
    }
    if (desc->ce_push_targets == 0) {
        // a caller that gives no staging has not asked for copies at all: all-zero fields mean the kernels alone
        if (desc->world >= 8 && desc->staging != 0) push = others - 3;
    } else if (desc->ce_push_targets != OE_ZERO1_CE_NONE) {
        if (desc->ce_push_targets > others) return fail(OE_ERR_INVALID, "oe_zero1_create: ce_push_targets exceeds the number of peers");
        push = desc->ce_push_targets;
    }
    // staging_bases: all peers' entries set = the owners write the staged ranges; all zero = this rank reads them
    uint32_t shared = 0;
    for (uint32_t k = 0; k < desc->world; k++)
        if (k != desc->rank && desc->staging_bases[k] != 0) shared++;
    bool writes = false;
    if (shared != 0 && pull != 0) {
        if (shared != others) return fail(OE_ERR_INVALID, "oe_zero1_create: staging_bases must name every peer's staging or none");
        for (uint32_t k = 0; k < desc->world; k++)
            if (k != desc->rank && (desc->staging_bases[k] & 15u))
                return fail(OE_ERR_INVALID, "oe_zero1_create: staging of rank " + std::to_string(k) + " is not 16-byte aligned");
        if (desc->first_elem != (uint64_t)desc->rank * desc->numel)
            return fail(OE_ERR_INVALID, "oe_zero1_create: staging written by the owners needs equal shards in rank order (first_elem = rank * numel)");
        writes = true;
    }
    oe_zero1* z = new (std::nothrow) oe_zero1();
    if (!z) return fail(OE_ERR_INVALID, "out of host memory");
    z->plan = plan;
    z->desc = *desc;
    z->ce_pull_writes = writes;
    z->mean_scale = (float)(1.0 / (double)desc->world);
    z->ce_slot = (4ull * desc->numel + 255ull) & ~255ull;
    z->ce_pull = pull;
    z->ce_push = push;
    z->ce_push_auto = desc->ce_push_targets == 0;
    plan->status_word = desc->sync_blocks[desc->rank] + offsetof(oe_sync_block, status);
    *out = z;
    return 0;
}

extern "C" int oe_zero1_destroy(oe_zero1* z) {
    if (!z) return 0;
    if (z->plan) z->plan->status_word = 0;
    delete z;
    return 0;
}

extern "C" int oe_zero1_adamw_step(oe_zero1* z, const oe_adamw_hparams* hp, uint64_t stream) {
    return zero1_step(z, hp, nullptr, stream);
}

extern "C" int oe_zero1_sgd_step(oe_zero1* z, const oe_sgd_hparams* hp, uint64_t stream) {
    return zero1_step(z, nullptr, hp, stream);
}

extern "C" int64_t oe_zero1_info(const oe_zero1* z, int what) {
    if (!z) return -1;
    switch (what) {
        case 0: return z->ce_pull;
        case 1: return (z->desc.shadow_mc_delta != 0) ? 0 : z->ce_push;
        case 2: return z->epoch;
        case 3: return z->ce_pull_writes ? 1 : 0;
        default: return -1;
    }
}

extern "C" int oe_zero1_reduce(oe_zero1* z, uint64_t stream) {
    if (!z) return fail(OE_ERR_INVALID, "oe_zero1_reduce: NULL argument");
    const oe_driver* d = nullptr;
    int rc = zero1_phase_prologue(z, nullptr, nullptr, &d);
    return rc ? rc : zero1_reduce(d, z, stream);
}

extern "C" int oe_zero1_adamw_update(oe_zero1* z, const oe_adamw_hparams* hp, uint64_t stream) {
    if (!z || !hp) return fail(OE_ERR_INVALID, "oe_zero1_adamw_update: NULL argument");
    const oe_driver* d = nullptr;
    int rc = zero1_phase_prologue(z, hp, nullptr, &d);
    return rc ? rc : zero1_update(d, z, hp, nullptr, stream);
}

extern "C" int oe_zero1_sgd_update(oe_zero1* z, const oe_sgd_hparams* hp, uint64_t stream) {
    if (!z || !hp) return fail(OE_ERR_INVALID, "oe_zero1_sgd_update: NULL argument");
    const oe_driver* d = nullptr;
    int rc = zero1_phase_prologue(z, nullptr, hp, &d);
    return rc ? rc : zero1_update(d, z, nullptr, hp, stream);
}

extern "C" int oe_zero1_exchange(oe_zero1* z, uint32_t phase, uint64_t stream) {
    if (!z) return fail(OE_ERR_INVALID, "oe_zero1_exchange: NULL argument");
    if (phase > OE_SYNC_PUSHED) return fail(OE_ERR_INVALID, "oe_zero1_exchange: unknown phase");  // the staging exchange belongs to the reduce phase
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    if (phase == OE_SYNC_GRADS_READY) z->epoch += 1;  // a step begins with this exchange
    CtxGuard guard(d, z->plan->dc->ctx);
    return launch_exchange(d, z, phase, phase == OE_SYNC_REDUCED, (CUstream)stream);
}

extern "C" int oe_zero1_status(oe_zero1* z, uint32_t* status_out, uint64_t stream) {
    if (!z || !status_out) return fail(OE_ERR_INVALID, "oe_zero1_status: NULL argument");
    int rc = 0;
    const oe_driver* d = driver_or_fail(&rc);
    if (!d) return rc;
    CtxGuard guard(d, z->plan->dc->ctx);
    uint32_t word = 0;
    OE_CU(d->cuMemcpyDtoHAsync_(&word, (CUdeviceptr)z->plan->status_word, sizeof(word), (CUstream)stream), "cuMemcpyDtoHAsync(status)");
    OE_CU(d->cuStreamSynchronize_((CUstream)stream), "cuStreamSynchronize");
    *status_out = word;
    if (word != 0)
        return fail(OE_ERR_DEVICE, "sharded step: rank " + std::to_string((word >> 16) & 0xff) + " did not arrive at exchange " +
                                       std::to_string((word >> 8) & 0xff) + " within the limit; the step's later launches did nothing");
    return 0;
}

extern "C" int oe_ipc_export(int device, uint64_t address, void* handle_out, uint64_t* offset_out) {
    if (!address || !handle_out || !offset_out) return fail(OE_ERR_INVALID, "oe_ipc_export: NULL argument");
    static_assert(sizeof(CUipcMemHandle) == 64, "IPC handle is 64 bytes");
    OE_DEVICE_PROLOGUE;
    CUdeviceptr base = 0;
    size_t size = 0;
    OE_CU(d->cuMemGetAddressRange_(&base, &size, (CUdeviceptr)address), "cuMemGetAddressRange");
    CUipcMemHandle h;
    OE_CU(d->cuIpcGetMemHandle_(&h, base), "cuIpcGetMemHandle");
    memcpy(handle_out, &h, sizeof(h));
    *offset_out = (uint64_t)address - (uint64_t)base;
    return 0;
}

extern "C" int oe_ipc_import(int device, const void* handle, uint64_t* base_out) {
    if (!handle || !base_out) return fail(OE_ERR_INVALID, "oe_ipc_import: NULL argument");
    OE_DEVICE_PROLOGUE;
    CUipcMemHandle h;
    memcpy(&h, handle, sizeof(h));
    CUdeviceptr p = 0;
    OE_CU(d->cuIpcOpenMemHandle_(&p, h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS), "cuIpcOpenMemHandle");
    *base_out = (uint64_t)p;
    return 0;
}

extern "C" int oe_ipc_close(int device, uint64_t base) {
    if (!base) return 0;
    OE_DEVICE_PROLOGUE;
    OE_CU(d->cuIpcCloseMemHandle_((CUdeviceptr)base), "cuIpcCloseMemHandle");
    return 0;
}


// Lets other translation units of the library report through oe_last_error().
extern "C" void oe_internal_set_error(const char* message) { t_error = message ? message : ""; }
