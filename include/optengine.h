/*
 * optengine — C ABI of the B200 optimizer-step engine (liboptengine.so).
 *
 * The library replaces, for NVIDIA B200 (sm_100a), the device side of gograd's
 * training hot path: the AdamW / SGD parameter update, the global gradient-norm
 * clip and the fp32-master -> bf16-shadow cast. It is what gograd's Go host code
 * binds instead of compiling CUDA C with NVRTC at run time: prebuilt sm_100a
 * cubins are embedded in the library and loaded through the CUDA driver API.
 *
 * Calling convention. Every argument is an integer, a pointer, or a pointer to a
 * plain struct; floating-point values travel inside structs, never as direct
 * arguments, so that a cgo-free Go binding (purego.SyscallN, the mechanism of
 * vulkan/loader_linux.go:16-47) can call every entry point. Device addresses and
 * streams are passed as uint64_t (CUdeviceptr / CUstream values; 0 = the default
 * stream). Every function returns 0 on success, a positive CUresult when a driver
 * call failed, or a negative OE_ERR_* code; oe_last_error() returns the message of
 * the calling thread's last failure. Nothing here aborts, exits or throws.
 *
 * Ownership. The caller owns parameters, gradients, optimizer state and shadows;
 * the library borrows their addresses for the duration of a call and owns only its
 * plans (device tables, the norm record, reduction scratch). There is no CPU
 * fallback: without a CUDA driver and a B200 every device call fails.
 *
 * Threading. A plan may be used from any thread, by one thread and one stream at a
 * time. The library never changes the caller's current context: it pushes the
 * device's primary context for the duration of a call and pops it again.
 *
 * Stream capture. oe_grad_norm, oe_norm_finalize, oe_adamw_step, oe_sgd_step, oe_zero_grads and
 * oe_cast_bf16 only enqueue launches: they allocate nothing and never synchronise, and the
 * counters the kernels use re-arm themselves, so the calls may be recorded in a stream capture
 * and replayed. A recorded launch carries the plan's table addresses, its number of work units,
 * its gradient scale and the hyper-parameter block as they were when it was recorded (step_dev
 * and lr_dev are the two values a replay reads afresh): create or update the plan before
 * capturing, and capture again after oe_plan_update changed the tensors.
 */
#ifndef OPTENGINE_H
#define OPTENGINE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OE_ABI_VERSION 1

#if defined(__GNUC__)
#define OE_API __attribute__((visibility("default")))
#else
#define OE_API
#endif

/* negative engine error codes (positive return values are CUresult codes) */
#define OE_ERR_INVALID   (-1) /* bad argument; nothing was launched or changed           */
#define OE_ERR_NO_DRIVER (-2) /* libcuda.so.1 missing or cuInit failed                   */
#define OE_ERR_NOT_INIT  (-3) /* oe_init was not called for the device                   */
#define OE_ERR_ARCH      (-4) /* the device is not sm_100 (the cubins are sm_100a only)  */
#define OE_ERR_LIMIT     (-5) /* a size exceeds what the entry point supports            */
#define OE_ERR_DEVICE    (-6) /* a kernel reported an error in its status word           */

/* flag bits (oe_adamw_hparams.flags, oe_sgd_hparams.flags, oe_grad_norm flags) */
#define OE_CLIP_DEVFORM  0x1u  /* clip coefficient fminf(1, max/(norm+1e-6)) as the reference's CUDA
                                  kernels do (autograd/cuda_kernels.go:676); default is the host rule
                                  "scale only if norm > max_norm" (autograd/nn.go:327-328)           */
#define OE_WRITE_SHADOW  0x2u  /* write the bf16 shadow of every tensor that has one                 */
#define OE_ZERO_GRAD     0x4u  /* store zeros over each gradient after it was consumed               */
#define OE_NESTEROV      0x8u  /* SGDOptions.Nesterov (autograd/sgd.go:16-19)                        */
#define OE_MAXIMIZE      0x10u /* SGDOptions.Maximize                                                */
#define OE_PARTIAL_ONLY  0x20u /* oe_grad_norm: leave the sum of squares, do not take the root       */
#define OE_ACCUMULATE    0x40u /* oe_peer_reduce_grads: add this call's sum of squares to the record     */

/* One optimizer parameter. Mirrors what the reference keeps per parameter:
 * Tensor.buf / Tensor.gradBuf (autograd/tensor.go:19-52), AdamW.mGPU/vGPU
 * (autograd/nn.go:336-346) or SGD.bufferGPU/initializedGPU (autograd/sgd.go:33-45), the
 * bf16 shadow (autograd/cuda_autocast.go:15-60) and the resolved group of the
 * parameter (autograd/param_groups.go:30-35). */
typedef struct oe_tensor_desc {
    uint64_t param;     /* float[numel]  master weights, device address                              */
    uint64_t grad;      /* float[numel]  gradient, or 0 when the parameter has none: it is then
                           skipped by every entry point, as a nil gradBuf is in the reference        */
    uint64_t state1;    /* AdamW: m.   SGD: momentum buffer, or 0 when momentum == 0                 */
    uint64_t state2;    /* AdamW: v.   SGD: device float holding 0/1 "buffer initialised", or 0      */
    uint64_t shadow;    /* uint16[numel] bf16 shadow, or 0                                           */
    uint64_t numel;     /* elements, > 0                                                             */
    float lr_scale;     /* ParameterGroup.LRScale after normalisation (0 is taken as 1)              */
    float weight_decay; /* ParameterGroup.WeightDecay                                                */
} oe_tensor_desc;

/* AdamW hyper-parameters of one step. The caller advances its step counter and
 * computes the bias corrections exactly as AdamW.Step does (autograd/nn.go:492-494):
 * bc = float32(1 - pow(float64(beta), float64(step))). */
typedef struct oe_adamw_hparams {
    float lr;          /* AdamW.LR (base rate; the group scale is applied on the device)             */
    float beta1, beta2, eps;
    float bc1, bc2;    /* bias corrections; ignored when step_dev != 0                               */
    float max_norm;    /* > 0: fold the clip coefficient of the plan's last oe_grad_norm into the
                          update (g*coef in registers); <= 0: no clipping                            */
    uint32_t flags;    /* OE_CLIP_DEVFORM | OE_WRITE_SHADOW | OE_ZERO_GRAD                           */
    uint64_t step_dev; /* device int32 step counter for captured steps (AdamW.PrepareGraph,
                          autograd/nn.go:350-361): incremented on the device, bias corrections
                          computed there; 0 = eager mode                                             */
    uint64_t lr_dev;   /* device float holding the base rate, read by the kernel instead of lr when
                          non-zero: a captured step then follows a schedule (OneCycle.Step ->
                          SetLearningRate, autograd/nn.go:571) without being captured again, which the
                          reference cannot do (it bakes lr into the launch, autograd/nn.go:480-483)          */
} oe_adamw_hparams;

/* SGD hyper-parameters of one step (SGDOptions, autograd/sgd.go:16-19). */
typedef struct oe_sgd_hparams {
    float lr;          /* SGD.LR (base rate)                                                         */
    float momentum, dampening;
    float max_norm;    /* as in oe_adamw_hparams                                                     */
    uint32_t flags;    /* OE_NESTEROV | OE_MAXIMIZE | OE_CLIP_DEVFORM | OE_WRITE_SHADOW | OE_ZERO_GRAD */
    uint32_t reserved;
    uint64_t step_dev; /* device int32 step counter incremented by a captured step (SGD.PrepareGraph,
                          sgd_step, autograd/cuda_sgd.go:18,99-125); 0 = eager mode                        */
    uint64_t lr_dev;   /* as in oe_adamw_hparams                                                     */
} oe_sgd_hparams;

typedef struct oe_plan oe_plan;

/* ---- library ------------------------------------------------------------------------------------ */

/* ABI version of the loaded library (OE_ABI_VERSION it was built with). */
OE_API int oe_abi_version(void);

/* Message of the calling thread's last failed call ("" when none). Replaces the
 * *cuda.Error{Op,Code,Message} values of cuda/cuda_windows.go:24-36. */
OE_API const char* oe_last_error(void);

/* Binds the CUDA driver, retains the device's primary context and loads the embedded
 * sm_100a cubin into it. Idempotent per device. Replaces the lazy NVRTC compile +
 * cuModuleLoadData of cuda.Compile (cuda/kernel_windows.go:131-228) and the per-device
 * kernel cache (cuda/device_cache.go:23-68). */
OE_API int oe_init(int device);

/* Unloads the modules and releases the primary contexts retained by oe_init. Plans
 * must be destroyed first. */
OE_API int oe_shutdown(void);

/* Number of CUDA devices the driver offers. */
OE_API int oe_device_count(int* count_out);

/* Lets `device` address memory allocated on `peer_device` (both initialised): what a single process
 * that drives several GPUs — one OS thread per device, as autograd/cuda_context.go:29-54 — needs
 * before it hands one device's buffers to kernels of another. Processes that own one GPU each
 * use oe_ipc_* instead, which brings the access with the mapping. Enabling twice is not an error. */
OE_API int oe_enable_peer_access(int device, int peer_device);

/* Number of SMs of an initialised device (148 on B200); < 0 on error. */
OE_API int oe_device_sm_count(int device);

/* ---- plans -------------------------------------------------------------------------------------- */

/* Builds the device-side tensor table and chunk table for a parameter list: the
 * multi-tensor replacement of the reference's one-launch-per-tensor loops
 * (autograd/nn.go:495-505, autograd/cuda_sgd.go:71-97) and of its clip pointer table
 * (getClipPlan, autograd/cuda_clip.go:66-113, one write_clip_entry launch per tensor).
 * Parameters with grad == 0 stay in the plan but are left out of the tables.
 * chunk_elems = 0 selects the default work-unit size (4096 elements; 2048 or 1024 for a
 * parameter list too small to give every SM two units); otherwise a multiple of 1024. The size
 * is fixed for the life of the plan and never changes results. Validates every descriptor
 * before allocating anything. */
OE_API int oe_plan_create(int device, const oe_tensor_desc* tensors, uint32_t n_tensors, uint32_t chunk_elems,
                   oe_plan** out);

/* Replaces the descriptors (gradients appear or disappear, the pool hands out other
 * addresses, a group's decay changes). Like getClipPlan's cache check
 * (autograd/cuda_clip.go:80-93) it compares addresses and sizes and re-uploads the
 * tables on `stream` only when something changed. */
OE_API int oe_plan_update(oe_plan* plan, const oe_tensor_desc* tensors, uint32_t n_tensors, uint64_t stream);

OE_API int oe_plan_destroy(oe_plan* plan);

/* Plan facts: what = 0 tensors with a gradient, 1 chunks, 2 elements with a gradient,
 * 3 grid size of the update launch, 4 grid size of the norm launch, 5 chunk_elems,
 * 6 number of table uploads so far. Returns -1 for an unknown query. */
OE_API int64_t oe_plan_info(const oe_plan* plan, int what);

/* Device address of the plan's norm record: a float32 norm at byte offset 8 and the
 * float64 sum of squares at offset 0. Replaces clipState.norm (autograd/cuda_clip.go:22). */
OE_API uint64_t oe_plan_norm_address(const oe_plan* plan);

/* Selects one of the built shapes of the update kernel by name suffix ("" default,
 * "u1", "u2", "u8"); a tuning knob, results are identical. */
OE_API int oe_plan_set_variant(oe_plan* plan, const char* variant);

/* Gradient scale of the plan (default 1): from now on oe_grad_norm, oe_adamw_step*, oe_sgd_step and
 * oe_adamw_step_from_host read every gradient element as (float)(g * *scale) — one fp32 rounding,
 * before the clip coefficient — so norm and update are those of the reference optimizer fed with
 * gradients stored at that scale. It folds the 1/groups factor of gradient accumulation
 * (GradAccumulator.Backward seeds differentiation with it, autograd/accumulate.go:31-44; for a power
 * of two the results are identical to seeding) or an unscale factor into the pass that reads the
 * gradients anyway. A scale of 1 changes no bit. *scale must be finite and positive. While it is not
 * 1, the in-place clip (oe_clip_grad_norm with max_norm > 0) and oe_peer_reduce_grads, which
 * rewrite the stored gradients, are refused with OE_ERR_INVALID. The float travels by pointer like
 * every float of this interface. */
OE_API int oe_plan_set_grad_scale(oe_plan* plan, const float* scale);

/* ---- gradient norm and clip --------------------------------------------------------------------- */

/* Global L2 norm over every present gradient of the plan: per-CTA float64 partial
 * sums, finalised by the last CTA to arrive (deterministic, no memset, no host
 * sync). Replaces norm.Memset + global_norm_parts + kernels.SqrtScalar
 * (autograd/cuda_clip.go:120-129, autograd/cuda_kernels.go:675, kernels/optim.go:56-64).
 * flags: OE_PARTIAL_ONLY leaves only the sum of squares (for a cross-rank reduction). */
OE_API int oe_grad_norm(oe_plan* plan, uint32_t flags, uint64_t stream);

/* norm = (float)sqrt(sum of squares) for a sum completed outside (after an all-reduce
 * of the record's float64 field). */
OE_API int oe_norm_finalize(oe_plan* plan, uint64_t stream);

/* ClipGradNorm on the device (autograd/nn.go:310-317, autograd/cuda_clip.go:114-134): the
 * norm as oe_grad_norm, then, when max_norm > 0, every present gradient scaled in
 * place (scale_all_grads, autograd/cuda_kernels.go:676). max_norm travels by pointer. */
OE_API int oe_clip_grad_norm(oe_plan* plan, const float* max_norm, uint32_t flags, uint64_t stream);

/* Blocking read of the last norm (GradientNormToHost, autograd/nn.go:17-27). */
OE_API int oe_read_norm(oe_plan* plan, float* norm_out, double* sumsq_out, uint64_t stream);

/* ---- updates ------------------------------------------------------------------------------------ */

/* One fused AdamW step over the whole plan in one launch: reads p, g, m, v with
 * 128-bit loads, updates in fp32 registers in the operation order of the reference's
 * host loop (autograd/nn.go:519-528), writes p, m, v and — with OE_WRITE_SHADOW — the
 * round-to-nearest-even bf16 shadow. Replaces the per-tensor kernels.AdamWUpdate
 * launches (autograd/nn.go:495-505, kernels/optim.go:69-82), graph_adamw
 * (autograd/cuda_kernels.go:597) and the later f32_to_bf16 pass per weight
 * (autograd/cuda_autocast.go:15-20). */
OE_API int oe_adamw_step(oe_plan* plan, const oe_adamw_hparams* hp, uint64_t stream);

/* One fused SGD step (autograd/sgd.go:192-225 semantics; replaces sgd_update + sgd_mark
 * per tensor, autograd/cuda_sgd.go:66-98) in ONE launch: the CTA that finishes last sets the
 * per-tensor "initialised" flags, which the reference does with one sgd_mark launch per tensor. */
OE_API int oe_sgd_step(oe_plan* plan, const oe_sgd_hparams* hp, uint64_t stream);

/* Zero every present gradient in one launch (AdamW.ZeroGrad, autograd/nn.go:533-537). */
OE_API int oe_zero_grads(oe_plan* plan, uint64_t stream);

/* Stand-alone fp32 -> bf16 cast of one buffer (castBF16 / f32_to_bf16,
 * autograd/cuda_autocast.go:15-20, autograd/cuda_kernels.go:86). */
OE_API int oe_cast_bf16(int device, uint64_t src, uint64_t dst, uint64_t numel, uint64_t stream);

/* ---- host-buffer step --------------------------------------------------------------------------- */

/* The whole step for a caller whose gradients live in host memory (Tensor.Grad):
 * copies host_grads[i] (float[numel], page-locked for full speed; NULL = keep what is
 * on the device) into each present gradient buffer, computes the norm, runs the fused
 * AdamW step with the clip folded in, reads the pre-clip norm back into *norm_out and
 * waits for the stream. n_tensors must equal the plan's. */
OE_API int oe_adamw_step_from_host(oe_plan* plan, const oe_adamw_hparams* hp, const float* const* host_grads,
                            uint32_t n_tensors, float* norm_out, uint64_t stream);

/* ---- sharded step (ZeRO-1 style) over peer memory ------------------------------------------------ */
/* The reference has no distributed code at all (no collective, no sharding); these entry points
 * have no counterpart there. Every rank (one process per GPU) keeps a full flat fp32 gradient
 * buffer and a full flat bf16 shadow buffer of one common layout, and owns one contiguous shard of
 * master weights, m and v. Buffers of other ranks are reached through CUDA IPC mappings (plain peer
 * loads and stores only). None of the kernels in this group waits on another rank: the caller orders them
 * with stream-ordered collectives of its own, or uses the oe_zero1_* group below, which brings its own
 * (bounded) exchanges. */

/* Pull reduce-scatter fused with the norm pass. rank_bases[k] is the address, valid on this GPU, of
 * rank k's gradient buffer; the kernel reads elements [first_elem, first_elem+numel) of each, adds
 * them in ascending rank order (deterministic), multiplies by *scale (1/n for a mean), writes the
 * reduced shard to `out` (may be this rank's own range, in place) and leaves the float64 sum of
 * squares of the reduced shard in the plan's norm record (and the norm, unless OE_PARTIAL_ONLY).
 * With OE_ACCUMULATE the sum is added to the record instead of replacing it, so a shard can be
 * reduced piece by piece. The bases may equally point at local staging copies of the peers' ranges:
 * only the address arithmetic base + 4*(first_elem + i) matters. */
OE_API int oe_peer_reduce_grads(oe_plan* plan, const uint64_t* rank_bases, uint32_t n_ranks, uint64_t first_elem,
                                uint64_t numel, uint64_t out, const float* scale, uint32_t flags, uint64_t stream);

/* oe_adamw_step over a contiguous range of the plan's work units (first_chunk .. first_chunk+n_chunks of
 * oe_plan_info(plan, 1) units, in parameter order): lets a caller pipeline the update piece by piece
 * against copies of the pieces already updated. Eager mode only (step_dev must be 0). */
OE_API int oe_adamw_step_chunks(oe_plan* plan, const oe_adamw_hparams* hp, uint64_t first_chunk, uint64_t n_chunks,
                                uint64_t stream);

/* oe_adamw_step whose bf16 shadow stores go to every rank's shadow buffer: shadow_deltas[k] is the
 * byte distance from this rank's shadow buffer to rank k's mapping (0 for the rank itself). The
 * all-gather of the shadows is these stores, overlapped with the update's own HBM traffic. */
OE_API int oe_adamw_step_peers(oe_plan* plan, const oe_adamw_hparams* hp, const int64_t* shadow_deltas,
                               uint32_t n_ranks, uint64_t stream);

/* The same for oe_sgd_step: the sharded form of SGD.Step, momentum buffers and init flags per piece of a
 * tensor inside the rank's shard. */
OE_API int oe_sgd_step_peers(oe_plan* plan, const oe_sgd_hparams* hp, const int64_t* shadow_deltas, uint32_t n_ranks,
                             uint64_t stream);

/* The same two steps with the shadow stores sent through an NVLink multicast mapping: *mc_delta is the byte
 * distance from this rank's shadow buffer to a multicast address that is bound to every rank's shadow
 * buffer (cuMulticastCreate / cuMulticastBindMem, or torch's symmetric memory). Each 8-byte vector
 * leaves this GPU once (multimem.st) and the switch delivers it to every rank, this one included; the
 * few single elements at the end of a tensor whose length is no multiple of 4 take the plain stores
 * through shadow_deltas. Results are those of oe_adamw_step_peers / oe_sgd_step_peers. */
OE_API int oe_adamw_step_multicast(oe_plan* plan, const oe_adamw_hparams* hp, const int64_t* shadow_deltas,
                                   uint32_t n_ranks, const int64_t* mc_delta, uint64_t stream);
OE_API int oe_sgd_step_multicast(oe_plan* plan, const oe_sgd_hparams* hp, const int64_t* shadow_deltas,
                                 uint32_t n_ranks, const int64_t* mc_delta, uint64_t stream);

/* Tuning knobs of the peer kernels; none changes a result. value 0 restores the library's choice.
 *   OE_TUNE_PEER_REDUCE_GRID       CTAs of the pull-reduce launch (at most the persistent grid)
 *   OE_TUNE_PEER_UPDATE_GRID       CTAs of the update launches that store into peers' buffers
 *   OE_TUNE_PEER_REDUCE_FIRST      rank whose gradient is loaded first for every element (the adds keep
 *                                  ascending rank order); ranks that pass their own rank + 1 do not all
 *                                  address the same source first
 *   OE_TUNE_PEER_PUSH_WARP_ROTATE  1: warp w of a CTA starts its round of shadow stores at target w mod n instead of
 *                                  target 0; 2: it does not; 0: the library's choice
 * Where OE_TUNE_PEER_UPDATE_GRID and OE_TUNE_PEER_PUSH_WARP_ROTATE are left at 0 the library chooses by the number
 * of ranks from measurements on 8-GPU B200 boxes: with four ranks the AdamW update runs one CTA per SM with rotated
 * warps (676-695 GB/s pushed against 621), otherwise the persistent grid without rotation.
 * The update kernels issue their plain shadow stores in the order of shadow_deltas, which the caller may
 * rotate by rank for the same reason. */
#define OE_TUNE_PEER_REDUCE_GRID      1
#define OE_TUNE_PEER_UPDATE_GRID      2
#define OE_TUNE_PEER_REDUCE_FIRST     3
#define OE_TUNE_PEER_PUSH_WARP_ROTATE 4
#define OE_TUNE_PEER_UPDATE_VECTORS   6 /* sharded AdamW update: 2, 4 (default) or 8 128-bit vectors in flight per thread and
                                           stream (3, 2 or 1 resident CTAs per SM) */
#define OE_TUNE_PEER_REDUCE_WARP_ROTATE 7 /* pull-reduce: non-zero makes warp w of a CTA issue its loads starting w
                                             sources after OE_TUNE_PEER_REDUCE_FIRST (the adds keep rank order) */
#define OE_TUNE_STEP_GRID             5 /* single-GPU update and in-place clip launches: 0 = a persistent grid strides
                                           over the work units, 1 = one CTA per work unit in table order */
OE_API int oe_plan_set_tuning(oe_plan* plan, int what, uint64_t value);

/* Link-rate probes: what the NVLink fabric gives the two access patterns of the sharded step when nothing else
 * rides on them, to rate the step's kernels against (run them on every rank at the same time, as the step does).
 * oe_link_probe_reads issues every load of oe_peer_reduce_grads over the same range and stores no element (the
 * plan's norm record is overwritten). oe_link_probe_stores writes bf16 ZEROS over [shadow_shard, shadow_shard +
 * 2*numel) of every OTHER rank's shadow buffer, in the launch shape the update would use: call it only where a
 * following step rewrites that range. */
OE_API int oe_link_probe_reads(oe_plan* plan, const uint64_t* rank_bases, uint32_t n_ranks, uint64_t first_elem,
                               uint64_t numel, uint64_t stream);
OE_API int oe_link_probe_stores(oe_plan* plan, uint64_t shadow_shard, const int64_t* shadow_deltas, uint32_t n_ranks,
                                uint64_t numel, uint64_t stream);

/* ---- sharded step driven through this interface alone -------------------------------------------- */
/* For a host with no collective library (the reference has none: one OS thread per device,
 * autograd/cuda_context.go:29-54). The points at which the ranks of a step must meet (three, or four when
 * staged gradient ranges are written by their owners, below) are small kernels of the library: every rank announces its arrival with plain stores into an exchange area in
 * each rank's memory, then waits for the others' announcements in its own area. The wait is bounded:
 * after timeout_ms (or an equivalent number of polls) the kernel records the missing rank in the area's
 * status word and returns; every later launch of the sharded step (pull-reduce, update, exchanges) sees
 * the word and does nothing, so a rank that never arrives costs a time-out, never a hung GPU. The host
 * reads the word with oe_zero1_status.
 *
 * Set-up: every rank allocates OE_ZERO1_SYNC_BYTES of zeroed device memory (256-byte aligned), exports it
 * with oe_ipc_export like its gradient and shadow buffers, and maps the others' (oe_ipc_import). All
 * ranks must call the step the same number of times. A rank's kernels wait on kernels of OTHER GPUs
 * only: never run two ranks of one step on the same GPU. The step number each exchange waits for is a
 * launch parameter that the host advances per call, so these calls cannot be recorded once in a stream
 * capture and replayed. */
#define OE_ZERO1_SYNC_BYTES 512
#define OE_ZERO1_NO_ENTRY_EXCHANGE 0x1u /* the caller already knows that every rank's gradients are complete */

typedef struct oe_zero1_desc {
    uint32_t rank, world;          /* world <= 8, one node                                             */
    uint64_t first_elem, numel;    /* this rank's shard of the flat layout                             */
    uint64_t grad_bases[8];        /* rank k's flat gradient buffer as mapped on this GPU              */
    int64_t shadow_deltas[8];      /* byte distance from this rank's shadow buffer to rank k's (own: 0) */
    int64_t shadow_mc_delta;       /* distance to a multicast mapping of the shadow buffer, 0 = none   */
    uint64_t sync_blocks[8];       /* rank k's exchange area as mapped on this GPU                     */
    uint32_t timeout_ms;           /* limit of every wait, 0 = 10000                                   */
    uint32_t flags;                /* OE_ZERO1_NO_ENTRY_EXCHANGE                                       */
    /* Copy-engine assistance (see below); all of it may be 0.                                         */
    uint64_t staging;              /* caller-owned device scratch, 16-byte aligned, or 0               */
    uint64_t staging_bytes;
    uint32_t ce_pull_sources;      /* peers whose gradient range a copy brings into staging before the
                                      pull kernel runs: 0 = the library's choice, OE_ZERO1_CE_NONE = none */
    uint32_t ce_push_targets;      /* ranks that receive their shadow copy from a copy after the update
                                      kernel: 0 = the library's choice, OE_ZERO1_CE_NONE = none          */
    uint64_t staging_bases[8];     /* rank k's staging as mapped on this GPU (own entry = staging), or all 0:
                                      with them the staged ranges are WRITTEN by their owners (see below)  */
} oe_zero1_desc;
#define OE_ZERO1_CE_NONE 0xffffffffu
/* Copy-engine assistance. With all GPUs of a box reading (or writing) each other at once, SM-issued loads
 * reach about 665 GB/s and stores about 620 GB/s per GPU; copies issued in RING order — in window j every rank
 * talks to the rank j+1 places after it, so every GPU serves one reader and one writer at a time — reach
 * 740 GB/s when they read from the peer and 770 GB/s when they write to it. So from four ranks on the step lets copies carry part of the traffic, all on the caller's
 * stream, in whole-shard pieces:
 *   reduce: the ranges of the first ce_pull_sources ranks after this one are copied into `staging` (4*numel
 *           bytes each), then the pull kernel reads those locally and the remaining peers over NVLink — same
 *           ascending-rank-order sum, bit for bit. With staging_bases set (every rank's staging mapped on
 *           every GPU, all of one size) the copies go the other way: each rank writes its own gradient ranges
 *           into the staging of the ce_pull_sources ranks after it — a copy that writes to a peer runs at
 *           770 GB/s where one that reads from it runs at 740 — and one more exchange (phase 3) tells every
 *           rank that its staging is complete. That form needs equal shards in rank order
 *           (first_elem = rank * numel on every rank) and the same ce_pull_sources on every rank;
 *   update: the kernel stores the shadow to this rank and the next world-1-ce_push_targets ranks, then copies
 *           deliver this rank's shard to the remaining ranks.
 * The library's choice (measured on 8-GPU B200 boxes), made only for a caller that provides staging: eight
 * ranks: all but one peer through staging, four shadow copies; four to seven ranks: all but one peer through
 * staging, no shadow copies; fewer: none. With staging for fewer ranges than that, as many as fit are staged.
 * A descriptor whose copy fields are all zero runs on the kernels alone. */

typedef struct oe_zero1 oe_zero1;

/* Binds a plan (whose tensors are the pieces of this rank's shard) to the ranks' buffers. Allocates
 * nothing on the device. One binding per plan; destroy it before the plan (oe_plan_destroy refuses a
 * plan that is still bound). */
OE_API int oe_zero1_create(oe_plan* plan, const oe_zero1_desc* desc, oe_zero1** out);
OE_API int oe_zero1_destroy(oe_zero1* z);

/* One sharded step, enqueued on `stream` without a host wait: exchange "gradients ready" -> pull-reduce
 * of this rank's shard (mean in ascending rank order) with its sum of squares -> exchange of the partial
 * sums, added in rank order into the global norm -> fused update with the clip folded in, shadow stored
 * to every rank -> exchange "stores performed". hp as for oe_adamw_step / oe_sgd_step.
 * One host thread may enqueue the steps of several ranks (devices) one after the other as long as the context
 * uses no copies. With copies and several ranks in ONE process, issue each rank's call from a thread of its own
 * and on a stream created for it (oe_stream_create), not the device's default stream: a copy between two devices
 * of one process is work for both, it may keep the host in the call until the work queued before it has run, and
 * on a default stream it is ordered after that device's own step, which waits for the other ranks (measured: the
 * exchanges then run into their limit). Ranks in processes of their own need neither. */
OE_API int oe_zero1_adamw_step(oe_zero1* z, const oe_adamw_hparams* hp, uint64_t stream);
OE_API int oe_zero1_sgd_step(oe_zero1* z, const oe_sgd_hparams* hp, uint64_t stream);

/* The phases on their own, for a caller that enqueues them itself (and for timing them one by one): one
 * exchange (phase 0 gradients ready — it also begins a new step —, 1 reduced, 2 stored); the reduce phase
 * (staged copies, if the context uses them, then the pull kernel); the update phase (fused update and shadow
 * stores, then shadow copies, if the context uses them). A step is exchange 0, reduce, exchange 1, update,
 * exchange 2 in that order on one stream. */
OE_API int oe_zero1_exchange(oe_zero1* z, uint32_t phase, uint64_t stream);
OE_API int oe_zero1_reduce(oe_zero1* z, uint64_t stream);
OE_API int oe_zero1_adamw_update(oe_zero1* z, const oe_adamw_hparams* hp, uint64_t stream);
OE_API int oe_zero1_sgd_update(oe_zero1* z, const oe_sgd_hparams* hp, uint64_t stream);

/* what: 0 peers staged by a copy in the reduce phase, 1 ranks served by a shadow copy in the update phase (as
 * resolved when the context was made; the library's own choice still leaves shadow ranges under 64 MiB to the
 * kernel), 2 steps begun so far, 3 whether the staged ranges are written by their owners (1) or read by this rank
 * (0). -1 for anything else. */
OE_API int64_t oe_zero1_info(const oe_zero1* z, int what);

/* Waits for `stream` and reads the status word: 0 and *status_out = 0 when every exchange so far
 * completed; otherwise OE_ERR_DEVICE, *status_out = 1 | phase << 8 | missing rank << 16, and the message
 * names the rank. The word is sticky: rebuild the ranks' state before stepping again. */
OE_API int oe_zero1_status(oe_zero1* z, uint32_t* status_out, uint64_t stream);

/* CUDA IPC plumbing: export the allocation that contains `address` (64-byte handle + offset of
 * the address inside it), map a peer's allocation on this device, unmap it. */
OE_API int oe_ipc_export(int device, uint64_t address, void* handle_out, uint64_t* offset_out);
OE_API int oe_ipc_import(int device, const void* handle, uint64_t* base_out);
OE_API int oe_ipc_close(int device, uint64_t base);

/* ---- allocation-free norm ------------------------------------------------------------------------ */

/* Largest input of oe_grad_norm_static: 2^31 elements (8 GiB of fp32). */
#define OE_STATIC_NORM_MAX_ELEMS 2147483648ull

/* L2 norm of ONE contiguous fp32 gradient buffer, written as a float to the device address
 * norm_out, without allocating anything: no plan, no cuMemAlloc/cudaMalloc, no free. It exists
 * for hosts that cannot allocate once training runs — a process that gave the whole GPU to its
 * own arena, so that a later driver allocation fails, or a step loop that must not take the
 * device-wide synchronisation an allocation implies. The reduction's scratch (32768 float64
 * partial sums — one per 8192 elements, or per 65536 for buffers beyond 2^28 elements — plus an
 * arrival counter, 257 KB) is a fixed __device__ array
 * inside the library image: every GPU that loads the library holds it until the process ends,
 * and numel above OE_STATIC_NORM_MAX_ELEMS is refused with OE_ERR_LIMIT.
 * All calls on a device share that array and it keeps the previous call's contents (the entry
 * point re-zeroes the counter on `stream` before each launch): calls whose kernels could overlap
 * on the GPU — other streams, other threads — race and must be serialised by the caller. The
 * first call on a device also resolves the array's device address, which loads the module: make
 * it at start-up, before any stream capture begins.
 * No counterpart in the reference; same result as oe_grad_norm on a one-tensor plan up to the
 * summation order of the float64 partial sums. This one entry point uses the CUDA runtime: a positive
 * return value is a cudaError_t, which has the same numbering as CUresult for every code that can occur
 * here (invalid value 1, out of memory 2, no kernel image 209, invalid device 101, launch failures 7xx). */
OE_API int oe_grad_norm_static(int device, uint64_t grad, uint64_t numel, uint64_t norm_out, uint64_t stream);

/* ---- launch counters ---------------------------------------------------------------------------- */

/* Launches of the named kernel since the last reset (all devices). The reference's
 * tests assert "kernel X ran" through its profile counts (autograd/cuda_kernels.go:11-82,
 * autograd/sgd_test.go:119-121). name NULL = all kernels. */
OE_API int64_t oe_launch_count(const char* kernel_name);
OE_API void oe_launch_count_reset(void);

/* Optional timing of every launch (EnableGPUProfile / GPUProfile, autograd/cuda_kernels.go:24-82): while
 * enabled each launch is bracketed by two events and waited for, and its device time is added to the
 * total of its kernel name. Enabling clears counts and times. A diagnostic: it serialises the stream
 * and must stay off inside a stream capture. oe_profile_get reads count and milliseconds of one
 * kernel (name NULL = all kernels); either output may be NULL. */
OE_API void oe_profile_enable(int enabled);
OE_API int oe_profile_get(const char* kernel_name, int64_t* count_out, double* ms_out);

/* ---- device plumbing for a host without a CUDA binding ------------------------------------------ */
/* The reference's cuda package only exists for Windows (cuda/cuda_stub.go:1-25); these
 * are the few calls its optimizer path needs on Linux (cuda.Alloc / Buffer.Free /
 * CopyFromHost / CopyToHost / Memset, cuda/cuda_windows.go:324-700; Stream and Event,
 * cuda/cuda_windows.go:700-900). */
OE_API int oe_mem_alloc(int device, uint64_t bytes, uint64_t* address_out);
OE_API int oe_mem_free(int device, uint64_t address);
OE_API int oe_mem_info(int device, uint64_t* free_out, uint64_t* total_out);
OE_API int oe_memcpy_h2d(int device, uint64_t dst, const void* src, uint64_t bytes, uint64_t stream);
OE_API int oe_memcpy_d2h(int device, void* dst, uint64_t src, uint64_t bytes, uint64_t stream);
/* either side may be a peer's buffer mapped on `device` (oe_ipc_import, oe_enable_peer_access) */
OE_API int oe_memcpy_d2d(int device, uint64_t dst, uint64_t src, uint64_t bytes, uint64_t stream);
OE_API int oe_memset_u32(int device, uint64_t dst, uint32_t value, uint64_t count, uint64_t stream);
OE_API int oe_host_alloc(int device, uint64_t bytes, void** out); /* page-locked host memory */
OE_API int oe_host_free(int device, void* ptr);
OE_API int oe_stream_create(int device, uint64_t* stream_out);
OE_API int oe_stream_destroy(int device, uint64_t stream);
OE_API int oe_stream_sync(int device, uint64_t stream);
OE_API int oe_event_create(int device, uint64_t* event_out);
OE_API int oe_event_destroy(int device, uint64_t event);
OE_API int oe_event_record(int device, uint64_t event, uint64_t stream);
OE_API int oe_event_sync(int device, uint64_t event);
OE_API int oe_event_elapsed_ms(int device, uint64_t start, uint64_t stop, float* ms_out);

#ifdef __cplusplus
}
#endif
#endif /* OPTENGINE_H */
