/* Device-table layouts shared by the host shim and the sm_100a kernels.
 * Plain C, fixed-width fields only: the same bytes are written by the host and
 * read by the device. */
#ifndef OE_TABLE_H
#define OE_TABLE_H

#include <stdint.h>

/* One optimizer parameter with a present gradient. 64 bytes, 16-byte aligned. */
typedef struct oe_dev_tensor {
    uint64_t param;   /* float*    master weights                               */
    uint64_t grad;    /* float*    gradient (never 0 inside a device table)     */
    uint64_t state1;  /* float*    AdamW m  | SGD momentum buffer (0 = none)    */
    uint64_t state2;  /* float*    AdamW v  | SGD float init flag (0 = none)    */
    uint64_t shadow;  /* uint16_t* bf16 shadow (0 = do not write one)           */
    uint64_t numel;
    float lr_scale;     /* group LRScale, already normalised (0 -> 1)           */
    float weight_decay; /* group WeightDecay                                    */
    uint32_t aligned;   /* OE_ALIGNED_* bits: which streams allow 128-bit access */
    uint32_t reserved;
} oe_dev_tensor;

/* One unit of work: chunk `chunk` (of plan->chunk_elems elements) of tensor `tensor`. */
typedef struct oe_dev_chunk {
    uint32_t tensor;
    uint32_t chunk;
} oe_dev_chunk;

/* Result record of the norm reduction, 32 bytes in device memory. */
typedef struct oe_dev_norm {
    double sumsq;     /* sum of squares of every present gradient element        */
    float norm;       /* (float)sqrt(sumsq)                                      */
    uint32_t ticket;  /* arrival counter of the reduction; 0 between launches    */
    uint32_t error;   /* sticky device-side error word (0 = none)                */
    uint32_t step_ticket; /* arrival counter of an update launch; 0 between launches */
    uint32_t pad[2];
} oe_dev_norm;

#define OE_ALIGNED_BASE   0x1u /* param, grad, state1 16-byte and shadow 8-byte aligned */
#define OE_ALIGNED_STATE2 0x2u /* ... and state2 16-byte aligned as well                */

/* Kernel parameter blocks (passed by value through cuLaunchKernel). */
typedef struct oe_adamw_args {
    float lr, beta1, beta2, eps;
    float bc1, bc2;
    float max_norm;   /* > 0 folds the clip coefficient read from *norm          */
    uint32_t flags;
    int64_t step;     /* host step counter (after increment); used when step_dev == 0 */
    uint64_t norm;    /* const oe_dev_norm* or 0                                 */
    uint64_t step_dev;/* const int32_t* device step counter (capture mode) or 0  */
    uint64_t lr_dev;  /* const float* device-resident base rate, or 0 = use lr    */
    float grad_scale; /* every gradient element is read as (float)(g * grad_scale) */
    uint32_t pad;
    uint64_t ticket;  /* uint32_t* arrival counter used to advance *step_dev (capture mode) */
} oe_adamw_args;

typedef struct oe_sgd_args {
    float lr, momentum, dampening;
    float max_norm;
    uint32_t flags;   /* OE_F_NESTEROV | OE_F_MAXIMIZE | clip/shadow bits        */
    float grad_scale; /* every gradient element is read as (float)(g * grad_scale) */
    uint64_t norm;
    uint64_t lr_dev;  /* const float* device-resident base rate, or 0 = use lr    */
    uint64_t step_dev;/* int32_t* device step counter advanced by the launch, or 0 */
    uint64_t ticket;  /* uint32_t* arrival counter: the last CTA marks the momentum buffers initialised */
    uint32_t n_tensors; /* rows of the tensor table */
    uint32_t pad;
} oe_sgd_args;

/* Ranks of a sharded step: byte distance from this rank's buffer to rank k's buffer of the
 * same layout (0 for the rank itself). */
#define OE_MAX_PEERS 8
typedef struct oe_peer_set {
    uint32_t n;
    uint32_t pad;
    int64_t delta[OE_MAX_PEERS];
} oe_peer_set;

/* Arguments of the pull-reduce kernel: rank k's gradient buffer base, as seen from this GPU. */
typedef struct oe_peer_grads {
    uint32_t n;
    uint32_t flags;
    float scale;      /* multiplies the fixed-order sum (1/n for a mean, 1 for a sum) */
    uint32_t pad;
    uint64_t base[OE_MAX_PEERS];
} oe_peer_grads;

/* flag bits shared with include/optengine.h */
#define OE_F_CLIP_DEVFORM 0x1u  /* coefficient = fminf(1, max/(norm+1e-6)) instead of the host rule */
#define OE_F_WRITE_SHADOW 0x2u  /* write the bf16 shadow where a tensor has one  */
#define OE_F_ZERO_GRAD    0x4u  /* store zeros over the gradient after reading it */
#define OE_F_NESTEROV     0x8u
#define OE_F_MAXIMIZE     0x10u
#define OE_F_PARTIAL_ONLY 0x20u /* norm pass: leave sumsq, do not finalise        */
#define OE_F_ACCUMULATE   0x40u /* reduce pass: add to the record's sumsq instead of replacing it */

#endif
