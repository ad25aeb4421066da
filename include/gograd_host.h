/*
 * gograd_host — flat C handle API over the C++ host mirror of gograd's optimizer surface
 * (gograd_b200/csrc/host/autograd.hpp). It exists so that the behaviour a Go host keeps
 * around the device work — constructor validation, parameter groups, the shared step
 * counter, absent gradients, lazily initialised momentum, state snapshots and the
 * safetensors checkpoint layout — can be driven and tested from any language without a Go
 * toolchain. Every function returns 0 on success and non-zero on failure (the message is
 * gg_last_error()); a failed call leaves optimizer and tensors unchanged. Floats travel by
 * pointer, as in optengine.h.
 *
 * Reference surface mirrored (yh2237/gograd): autograd/nn.go:296-571 (Parameter, ClipGradNorm,
 * AdamW, OneCycle), autograd/sgd.go, autograd/param_groups.go, autograd/optimizer.go,
 * autograd/optimizer_state.go, autograd/sgd_state.go, autograd/training_checkpoint.go.
 */
#ifndef GOGRAD_HOST_H
#define GOGRAD_HOST_H

#include <stdint.h>

#include "optengine.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct gg_tensor gg_tensor;
typedef struct gg_optimizer gg_optimizer;

typedef struct gg_sgd_options { /* SGDOptions, autograd/sgd.go:16-19 */
    float lr, momentum, dampening, weight_decay;
    int32_t nesterov, maximize;
} gg_sgd_options;

typedef struct gg_onecycle { /* OneCycle, autograd/nn.go:539-542 */
    double max_lr, pct_start, div_factor, final_div_factor;
    int32_t total, step_count;
} gg_onecycle;

typedef struct gg_accumulator { /* GradAccumulator, autograd/accumulate.go:15-18 */
    int32_t groups, pending;
} gg_accumulator;

/* Parameter groups as flat arrays: group g is named group_names[g], owns the parameters
 * members[offsets[g] .. offsets[g+1]) (indexes into the parameter list), scales the base rate
 * by lr_scales[g] (0 selects 1) and decays with decays[g] (ParameterGroupSpec,
 * autograd/param_groups.go:21-26). */
typedef struct gg_groups {
    int32_t n_groups;
    const char* const* group_names;
    const int32_t* offsets; /* n_groups + 1 entries */
    const int32_t* members;
    const float* lr_scales;
    const float* decays;
} gg_groups;

OE_API const char* gg_last_error(void);

/* ---- tensors: contiguous float32 CUDA leaves (autograd/tensor.go:19-52) ---- */
OE_API int gg_tensor_new(const float* values, const int32_t* shape, int32_t rank, int32_t device, int32_t requires_grad,
                         gg_tensor** out);
OE_API void gg_tensor_free(gg_tensor* t);
OE_API int64_t gg_tensor_numel(const gg_tensor* t);
OE_API int gg_tensor_to_host(const gg_tensor* t, float* out);
OE_API int gg_tensor_copy_from_host(gg_tensor* t, const float* values);
OE_API int gg_tensor_has_grad(const gg_tensor* t);                 /* 1 when a gradient buffer exists */
OE_API int gg_tensor_set_grad(gg_tensor* t, const float* values);  /* NULL makes the gradient absent */
OE_API int gg_tensor_ensure_grad(gg_tensor* t);                    /* present and zero when it was absent */
OE_API int gg_tensor_grad_to_host(const gg_tensor* t, float* out);
OE_API int gg_tensor_shadow_to_host(const gg_tensor* t, uint16_t* out);
OE_API int gg_tensor_shadow_current(const gg_tensor* t);           /* 1 when the bf16 shadow matches the value */
OE_API uint64_t gg_tensor_address(const gg_tensor* t, int32_t which); /* 0 value, 1 gradient, 2 shadow */
OE_API int gg_tensor_grad_known_zero(const gg_tensor* t);          /* 1 while the gradient is known to hold zeros */
/* bf16 shadow leases (autograd/cuda_autocast.go:77-94): a reader that keeps the shadow's address across an
 * optimizer step takes a lease; the step then writes a fresh buffer and the leased one stays valid until
 * released. gg_tensor_shadow_lease returns the leased device address (0 when there is no shadow). */
OE_API uint64_t gg_tensor_shadow_lease(gg_tensor* t);
OE_API void gg_tensor_shadow_release(gg_tensor* t, uint64_t address);
OE_API int gg_tensor_leased_shadows(const gg_tensor* t); /* buffers currently kept alive by leases */

/* ---- optimizers (autograd/nn.go:385-537, autograd/sgd.go:76-257) ---- */
OE_API int gg_adamw_new(const char* const* names, gg_tensor* const* tensors, int32_t n, const float* lr,
                        const float* decay, gg_optimizer** out);            /* NewAdamW */
OE_API int gg_adamw_new_groups(const char* const* names, gg_tensor* const* tensors, int32_t n, const float* lr,
                               const gg_groups* groups, gg_optimizer** out); /* NewAdamWGroups */
OE_API int gg_adamw_set_config(gg_optimizer* o, const float* beta1, const float* beta2, const float* eps); /* exported fields */
OE_API int gg_sgd_new(const char* const* names, gg_tensor* const* tensors, int32_t n, const gg_sgd_options* options,
                      gg_optimizer** out);                                   /* NewSGD */
OE_API int gg_sgd_new_groups(const char* const* names, gg_tensor* const* tensors, int32_t n,
                             const gg_sgd_options* options, const gg_groups* groups, gg_optimizer** out);
OE_API int gg_opt_set_engine(gg_optimizer* o, int32_t write_shadow, int32_t clip_devform);
/* Step stores zeros over every gradient it has read, and the next ZeroGrad launches nothing while no
 * gradient was written since (ZeroGrad at the start of a group, autograd/training_loop.go:125-133).
 * An eager SGD refuses to step with it: its ZeroGrad makes gradients absent (autograd/sgd.go:231-246),
 * and a zeroed buffer is not an absent one; once prepared for graphs SGD zeroes too and accepts it. */
OE_API int gg_opt_set_zero_grad_in_step(gg_optimizer* o, int32_t on);
/* Step and step_clipped read every gradient element as (float)(g * *scale) from now on (default 1):
 * the 1/groups factor of gradient accumulation folded into the pass that reads the gradients. */
OE_API int gg_opt_set_grad_scale(gg_optimizer* o, const float* scale);
OE_API int gg_opt_step(gg_optimizer* o);                                /* Step */
OE_API int gg_opt_step_clipped(gg_optimizer* o, const float* max_norm); /* norm + Step with the clip folded in */
OE_API int gg_opt_last_norm(gg_optimizer* o, float* out);
OE_API int gg_opt_zero_grad(gg_optimizer* o);                           /* ZeroGrad */
OE_API int gg_opt_get_lr(const gg_optimizer* o, float* out);            /* LearningRate */
OE_API int gg_opt_set_lr(gg_optimizer* o, const float* lr);             /* SetLearningRate */
OE_API int64_t gg_opt_step_count(const gg_optimizer* o);
OE_API int gg_opt_close(gg_optimizer* o);                               /* Close: idempotent */
OE_API void gg_opt_free(gg_optimizer* o);
/* state of parameter `index`: which = 0 AdamW m, 1 AdamW v, 2 SGD momentum buffer; *initialized
 * receives the SGD flag (always 1 for AdamW). out may be NULL to query the flag only. */
OE_API int gg_opt_state(gg_optimizer* o, int32_t index, int32_t which, float* out, int32_t* initialized);
OE_API int gg_opt_group_scale(const gg_optimizer* o, int32_t index, float* step_size, float* decay); /* groupScale */
OE_API int gg_opt_save(gg_optimizer* o, const char* path);              /* SaveSafeTensors */
OE_API int gg_opt_load(gg_optimizer* o, const char* path);              /* LoadSafeTensors */
OE_API int gg_opt_prepare_graph(gg_optimizer* o);                       /* AdamW.PrepareGraph / SGD.PrepareGraph */
OE_API int gg_opt_step_captured(gg_optimizer* o);                       /* the capture branch of Step */
OE_API int gg_opt_graph_step_count(gg_optimizer* o, int32_t* out);      /* GraphStepCount */
OE_API int gg_adamw_prepare_graph(gg_optimizer* o);                     /* the three above, AdamW only */
OE_API int gg_adamw_step_captured(gg_optimizer* o);
OE_API int gg_adamw_graph_step_count(gg_optimizer* o, int32_t* out);

/* PartitionParameters (autograd/param_groups.go:63-102): labels[i] is what the caller's assign(name)
 * returns for parameter i. Writes the resulting specs, in order of first appearance of each label, as
 * JSON [{"Name":label,"Params":[names...]},...] into out. */
OE_API int gg_partition_parameters(const char* const* names, gg_tensor* const* tensors, const char* const* labels,
                                   int32_t n, char* out, int32_t capacity);

/* ---- clip (autograd/nn.go:310-334, autograd/cuda_clip.go) ---- */
OE_API int gg_clip_grad_norm(gg_tensor* const* tensors, int32_t n, const float* max_norm);
OE_API int gg_gradient_norm_to_host(float* out);
OE_API void gg_release_clip_state(void);

/* ---- gradient accumulation bookkeeping (autograd/accumulate.go:21-71) ----
 * gg_accumulator_micro_batch is what GradAccumulator.Backward does around the differentiation
 * itself: it writes the seed 1/groups, counts the micro-batch and reports (1/0) whether the group
 * is complete. Pending and Groups are the struct's fields; reset is Reset. */
OE_API int gg_accumulator_new(int32_t groups, gg_accumulator* out);
OE_API int gg_accumulator_micro_batch(gg_accumulator* a, float* seed_out, int32_t* complete_out);
OE_API void gg_accumulator_reset(gg_accumulator* a);

/* ---- the loop that calls the optimizer (TrainingLoop.Run, autograd/training_loop.go:53-214) ----
 * Reader, sampler, step, report and save belong to the caller and arrive as callbacks (user is passed
 * back to each). Statuses of next and step: 0 = a batch was read / the micro-batch was back-propagated,
 * GG_LOOP_END_OF_EPOCH (next only, io.EOF), GG_LOOP_CANCELLED (a context error: the run stops, unfinished
 * gradients are dropped and save receives the starting position of the unfinished group),
 * GG_LOOP_FAILED (any other error: the run returns it without saving); on a non-zero status the
 * callback may leave a message with gg_loop_set_error. step back-propagates with the seed it is given
 * (1/accumulate, GradAccumulator.Backward). position writes the sampler's payload (at most capacity
 * bytes) and its length; NULL = no sampler. report and save may be NULL; save's savepoint is NULL when
 * there is nothing to rewind. schedule may be NULL. applied is advanced by the run.
 * Returns 0 when the planned updates were applied, GG_LOOP_CANCELLED after a cancellation, 1 for any
 * other error (gg_last_error). */
#define GG_LOOP_END_OF_EPOCH 1
#define GG_LOOP_CANCELLED 2
#define GG_LOOP_FAILED 3
typedef struct gg_training_loop {
    void* user;
    int (*next)(void* user);
    int (*next_epoch)(void* user);
    int (*position)(void* user, char* out, int32_t capacity, int32_t* length);
    int (*step)(void* user, const float* seed, double* loss);
    void (*report)(void* user, int32_t update, const double* loss);
    int (*save)(void* user, const char* savepoint, int32_t length);
    gg_optimizer* optimizer;
    gg_onecycle* schedule;
    int32_t updates, applied, accumulate, log_every;
} gg_training_loop;
OE_API int gg_training_loop_run(gg_training_loop* loop);
OE_API void gg_loop_set_error(const char* message);

/* ---- schedule and training checkpoint (autograd/nn.go:539-571, autograd/training_checkpoint.go) ---- */
OE_API int gg_onecycle_new(const double* max_lr, int32_t total, const double* pct_start, gg_onecycle* out);
OE_API int gg_onecycle_lr(const gg_onecycle* c, double* out);
OE_API int gg_onecycle_step(gg_onecycle* c, gg_optimizer* o);
OE_API int gg_save_training_checkpoint(const char* path, const char* const* names, gg_tensor* const* tensors, int32_t n,
                                       gg_optimizer* o, const gg_onecycle* scheduler, const char* const* user_keys,
                                       const char* const* user_values, int32_t n_user);
/* user_json receives the caller metadata as a JSON object text (truncated to capacity). */
OE_API int gg_load_training_checkpoint(const char* path, const char* const* names, gg_tensor* const* tensors, int32_t n,
                                       gg_optimizer* o, gg_onecycle* scheduler, char* user_json, int32_t capacity);

/* ---- safetensors container, host only (autograd/safetensors.go:30-98, safetensors_stream.go:28-96) ---- */
/* Writes F32 entries (entry i: names[i], data[i], shape = shapes[shape_offsets[i] .. shape_offsets[i+1])) and
 * string metadata exactly as the reference's writer lays them out. Needs no GPU. */
OE_API int gg_safetensors_write(const char* path, const char* const* names, const float* const* data,
                                const int32_t* shapes, const int32_t* shape_offsets, int32_t n,
                                const char* const* meta_keys, const char* const* meta_values, int32_t n_meta);
/* Writes an AdamW state file ("gograd-adamw": entries m.<i>, v.<i> of shape [numel], metadata with the
 * optimizer configuration, autograd/optimizer_state.go:142-160) from host arrays: the export path of a
 * sharded optimizer whose gathered moments never lived in one AdamW object. Needs no GPU. */
typedef struct gg_adamw_config {
    int32_t step_count;
    float lr, weight_decay, beta1, beta2, eps;
} gg_adamw_config;
OE_API int gg_adamw_state_write(const char* path, int32_t n, const char* const* names, const int32_t* shapes,
                                const int32_t* shape_offsets, const float* const* m, const float* const* v,
                                const gg_adamw_config* config, const gg_groups* groups);
/* The same file written front to back without holding the moments: begin with names, shapes,
 * configuration and groups (the header and its offsets are fixed by them), then hand over the
 * values entry by entry in the order the file stores them (sorted names: m.0, m.1, m.10, ...;
 * gg_state_stream_next names the entry the file wants and how many of its values are missing, an
 * empty name at the end). An entry may arrive in consecutive pieces, so a sharded optimizer passes
 * each owner's piece as it is gathered. finish checks that everything arrived, fsyncs and renames
 * the temporary file into place; finish and abort free the handle. Byte for byte the file
 * gg_adamw_state_write produces. Needs no GPU. */
typedef struct gg_state_stream gg_state_stream;
OE_API int gg_adamw_state_stream_begin(const char* path, int32_t n, const char* const* names, const int32_t* shapes,
                                       const int32_t* shape_offsets, const gg_adamw_config* config,
                                       const gg_groups* groups, gg_state_stream** out);
/* The same for an SGD state file ("gograd-sgd": one entry buffer.<i> of shape [numel] per parameter whose
 * momentum buffer is initialised, the flags, options and groups in the metadata,
 * autograd/sgd_state.go:27-67,150-194). initialized[i] != 0 marks the parameters that have a buffer; the
 * values follow through gg_state_stream_next / append / finish as above. */
typedef struct gg_sgd_config {
    int32_t step_count;
    float lr, momentum, dampening, weight_decay;
    int32_t nesterov, maximize;
} gg_sgd_config;
OE_API int gg_sgd_state_stream_begin(const char* path, int32_t n, const char* const* names, const int32_t* shapes,
                                     const int32_t* shape_offsets, const gg_sgd_config* config,
                                     const uint8_t* initialized, const gg_groups* groups, gg_state_stream** out);
OE_API int gg_state_stream_next(const gg_state_stream* s, char* name_out, int32_t capacity, int64_t* remaining_out);
OE_API int gg_state_stream_append(gg_state_stream* s, const char* entry, const float* values, int64_t count);
OE_API int gg_state_stream_finish(gg_state_stream* s);
OE_API void gg_state_stream_abort(gg_state_stream* s);
/* Validates a file with the reference reader's rules and returns a JSON description
 * {"entries":{name:{"shape":[..],"sum":float64 sum of the values}},"metadata":{..}} in out. */
OE_API int gg_safetensors_describe(const char* path, char* out, int32_t capacity);

#ifdef __cplusplus
}
#endif
#endif /* GOGRAD_HOST_H */
