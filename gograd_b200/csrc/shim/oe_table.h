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
    uint64_t status;  /* const uint32_t* or 0: a non-zero word (a failed exchange between ranks) skips the launch */
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
    uint64_t status;  /* as in oe_adamw_args */
} oe_sgd_args;

/* Ranks of a sharded step: byte distance from this rank's buffer to rank k's buffer of the
 * same layout (0 for the rank itself). */
#define OE_MAX_PEERS 8
typedef struct oe_peer_set {
    uint32_t n;
    uint32_t mode;    /* OE_PEER_* bits */
    int64_t delta[OE_MAX_PEERS];
    int64_t mc_delta; /* OE_PEER_MULTICAST: byte distance to a multicast mapping of the buffer */
} oe_peer_set;
#define OE_PEER_MULTICAST 0x1u /* 8-byte vectors go out as one multimem.st through mc_delta, replicated to
                                  every rank by the switch; single elements still take the plain stores */
#define OE_PEER_WARP_ROTATE 0x2u /* warp w of a CTA starts its round of stores at target w mod n       */

/* Arguments of the pull-reduce kernel: rank k's gradient buffer base, as seen from this GPU. */
typedef struct oe_peer_grads {
    uint32_t n;
    uint32_t flags;
    float scale;      /* multiplies the fixed-order sum (1/n for a mean, 1 for a sum) */
    uint32_t rot;     /* the loads of one element are issued starting at rank `rot`; the adds keep rank order */
    uint64_t base[OE_MAX_PEERS];
    uint64_t status;  /* const uint32_t* or 0: a non-zero word skips the launch */
} oe_peer_grads;

/* Exchange area of one rank of a sharded step: 512 bytes of device memory, zero before the first
 * step, mapped by every other rank. Rank r announces that it reached point `phase` of step `epoch`
 * by storing the epoch into arrive[phase][r] of EVERY rank's area (its own included) and then waits,
 * with a limit, until its own area shows that epoch in every column. The middle exchange also
 * carries each rank's float64 partial sum of squares. */
#define OE_SYNC_PHASES 4
#define OE_SYNC_GRADS_READY 0  /* this rank's gradients are complete: the others may pull them      */
#define OE_SYNC_REDUCED     1  /* this rank's pull is over and its partial sum is published          */
#define OE_SYNC_PUSHED      2  /* this rank's shadow stores are performed on every GPU               */
#define OE_SYNC_STAGED      3  /* this rank's gradient copies into the others' staging are complete  */
typedef struct oe_sync_block {
    uint32_t arrive[OE_SYNC_PHASES][OE_MAX_PEERS]; /* 128 B */
    double partial[2][OE_MAX_PEERS];               /* 128 B, indexed by epoch parity */
    uint32_t status;   /* sticky: OE_SYNC_TIMEOUT | phase << 8 | first missing rank << 16; 0 = fine */
    uint32_t pad[63];
} oe_sync_block;
#define OE_SYNC_TIMEOUT 0x1u

typedef struct oe_sync_args {
    uint32_t rank, world, phase, epoch;
    uint64_t block[OE_MAX_PEERS]; /* every rank's oe_sync_block as mapped on this GPU */
    uint64_t norm_rec;            /* oe_dev_norm* for OE_SYNC_REDUCED (partial in, total and norm out), else 0 */
    uint64_t timeout_ns;          /* the wait gives up after this long ...                     */
    uint32_t max_polls;           /* ... or after this many polls, whichever comes first      */
    uint32_t pad;
} oe_sync_args;

/* flag bits shared with include/optengine.h */
#define OE_F_CLIP_DEVFORM 0x1u  /* coefficient = fminf(1, max/(norm+1e-6)) instead of the host rule */
#define OE_F_WRITE_SHADOW 0x2u  /* write the bf16 shadow where a tensor has one  */
#define OE_F_ZERO_GRAD    0x4u  /* store zeros over the gradient after reading it */
#define OE_F_NESTEROV     0x8u
#define OE_F_MAXIMIZE     0x10u
#define OE_F_PARTIAL_ONLY 0x20u /* norm pass: leave sumsq, do not finalise        */
#define OE_F_ACCUMULATE   0x40u /* reduce pass: add to the record's sumsq instead of replacing it */
#define OE_F_WARP_ROTATE  0x80u /* reduce pass (kernel side only): warp w issues its loads starting w sources later */
#define OE_F_NO_STORE     0x100u /* reduce pass (kernel side only): read and add, write no element (link-rate probe) */

#endif
