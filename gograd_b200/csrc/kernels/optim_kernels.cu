// Optimizer-step kernels for sm_100a (B200): multi-tensor AdamW / SGD update with the
// clip coefficient folded in and the bf16 shadow written in the same pass, the
// two-level gradient-norm reduction, the in-place gradient scale and the stand-alone
// fp32 -> bf16 cast. Compiled to a cubin and loaded by the shim through the driver API;
// this file holds device code only.
//
// Work layout. The host builds two device tables: one oe_dev_tensor per parameter
// with a present gradient and one oe_dev_chunk per `chunk_elems` elements of such a
// tensor. Every kernel is one launch over the whole parameter set: a persistent grid
// (a multiple of the SM count) strides over the chunk table, so a 2048-element norm
// weight and a 65M-element embedding cost the same per element.
//
// Arithmetic. The update follows the reference's host (CPU) optimizer operation for
// operation with explicit round-to-nearest intrinsics, so that no multiply-add is
// contracted: the results are meant to be bit-identical to that code, not merely
// close (autograd/nn.go:519-528, autograd/sgd.go:205-220, autograd/nn.go:318-333).
// The path is HBM-bound (about 0.3 flop per byte): no tensor cores, no shared-memory
// staging; the design goal is bytes in flight — 128-bit streaming loads, several per
// thread before the first use, streaming stores.
#include <stdint.h>

#include "../shim/oe_table.h"

#define OE_THREADS 256
#ifndef OE_UNROLL
#define OE_UNROLL 4
#endif
#ifndef OE_NORM_UNROLL
#define OE_NORM_UNROLL 4
#endif
#ifndef OE_NORM_SPAN
#define OE_NORM_SPAN 2
#endif

// ---------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------

// fp32 -> bf16, round to nearest even: the reference's integer formula
// (autograd/cuda_kernels.go:86-87) for every non-NaN input; NaN becomes a quiet NaN
// with the input's sign instead of wrapping into an infinity or a zero.
__device__ __forceinline__ uint32_t oe_bf16_rne(float x) {
    uint32_t bits = __float_as_uint(x);
    uint32_t r = (bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16;
    if ((bits & 0x7fffffffu) > 0x7f800000u) r = ((bits >> 16) & 0x8000u) | 0x7fc0u;
    return r & 0xffffu;
}

// Clip coefficient from the norm record of the reduction. Host rule
// (autograd/nn.go:327-328): scale only when norm > max_norm > 0. Device-form rule
// (autograd/cuda_kernels.go:676): fminf(1, max_norm/(norm+1e-6)) whenever max_norm > 0.
__device__ __forceinline__ float oe_clip_coefficient(const oe_dev_norm* norm, float max_norm, uint32_t flags) {
    if (norm == nullptr || !(max_norm > 0.0f)) return 1.0f;
    float n = norm->norm;
    float c = __fdiv_rn(max_norm, __fadd_rn(n, 1e-6f));
    if (flags & OE_F_CLIP_DEVFORM) return fminf(1.0f, c);
    return n > max_norm ? c : 1.0f;
}

struct oe_chunk_view {
    const oe_dev_tensor* t;
    uint64_t base;  // first element of the chunk inside the tensor
    uint32_t n;     // elements in this chunk
};

__device__ __forceinline__ oe_chunk_view oe_view(const oe_dev_tensor* tensors, const oe_dev_chunk* chunks, uint32_t c,
                                                 uint32_t chunk_elems) {
    oe_dev_chunk ck = chunks[c];
    oe_chunk_view v;
    v.t = tensors + ck.tensor;
    v.base = (uint64_t)ck.chunk * chunk_elems;
    uint64_t left = v.t->numel - v.base;
    v.n = left < chunk_elems ? (uint32_t)left : chunk_elems;
    return v;
}

// ---------------------------------------------------------------------------------
// AdamW
// ---------------------------------------------------------------------------------
struct oe_adamw_consts {
    float b1, b2, omb1, omb2, eps, bc1, bc2, coef, gscale;
};

// One element of AdamW.Step's host loop (autograd/nn.go:522-527), g already the
// stored gradient: g*coef rounds exactly like the in-place clip followed by a reload.
__device__ __forceinline__ void oe_adamw_one(float& p, float g, float& m, float& v, const oe_adamw_consts& k,
                                             float step, float one_minus_decay) {
    g = __fmul_rn(g, k.coef);
    float mi = __fadd_rn(__fmul_rn(k.b1, m), __fmul_rn(k.omb1, g));
    float vi = __fadd_rn(__fmul_rn(k.b2, v), __fmul_rn(__fmul_rn(k.omb2, g), g));
    m = mi;
    v = vi;
    float root = __fsqrt_rn(__fdiv_rn(vi, k.bc2));
    float update = __fdiv_rn(__fmul_rn(step, __fdiv_rn(mi, k.bc1)), __fadd_rn(root, k.eps));
    p = __fsub_rn(__fmul_rn(p, one_minus_decay), update);
}

// Where the bf16 shadow of a chunk goes. Single GPU: the tensor's own shadow buffer.
// Sharded step: every rank keeps a full shadow with the same layout, and the rank that
// owns a shard stores its bf16 values into all of them (its own included) — the
// all-gather of the shadows is these stores, overlapped with the update's HBM traffic.
// Peer buffers are plain peer-mapped device memory reached with ordinary stores.
// Peer modes. Plain: one ordinary store per target, in the order of peers.delta (the caller
// chooses the order; with OE_PEER_WARP_ROTATE warp w of the CTA starts its round at target
// w mod n, so the warps of a CTA do not all address the same GPU at the same moment).
// Multicast: peers.mc_delta leads to a multicast mapping of the buffer (every rank's copy bound
// to one NVLink multicast object); one multimem.st leaves this GPU once and the switch
// delivers it to every rank, the storing one included. The instruction has no 16-bit form,
// so the few single elements (tails of tensors whose length is no multiple of 4) keep the
// plain stores.
template <bool PEERS>
__device__ __forceinline__ void oe_store_shadow4(uint16_t* sh, uint32_t vec_index, uint2 packed, const oe_peer_set& peers) {
    if (PEERS) {
        if (peers.mode & OE_PEER_MULTICAST) {
            uint2* dst = (uint2*)((char*)sh + peers.mc_delta) + vec_index;
            asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(dst), "f"(__uint_as_float(packed.x)),
                         "f"(__uint_as_float(packed.y))
                         : "memory");
            return;
        }
        uint32_t k = (peers.mode & OE_PEER_WARP_ROTATE) ? (threadIdx.x >> 5) % peers.n : 0u;
        for (uint32_t j = 0; j < peers.n; j++) {
            __stcs((uint2*)((char*)sh + peers.delta[k]) + vec_index, packed);
            if (++k == peers.n) k = 0;
        }
    } else {
        __stcs((uint2*)sh + vec_index, packed);
    }
}

template <bool PEERS>
__device__ __forceinline__ void oe_store_shadow1(uint16_t* sh, uint32_t index, uint16_t value, const oe_peer_set& peers) {
    if (PEERS) {
        for (uint32_t k = 0; k < peers.n; k++) ((uint16_t*)((char*)sh + peers.delta[k]))[index] = value;
    } else {
        sh[index] = value;
    }
}

// The plan's gradient scale: a gradient element is read as (float)(g*scale), rounded on its
// own before anything else, so the update sees what it would have seen had the gradient
// been stored at that scale. Bodies are built with and without the multiply; a scale of
// exactly 1 (the default) runs the body without it.
template <bool SCALED>
__device__ __forceinline__ void oe_scale4(float4& g, float s) {
    if (SCALED) {
        g.x = __fmul_rn(g.x, s);
        g.y = __fmul_rn(g.y, s);
        g.z = __fmul_rn(g.z, s);
        g.w = __fmul_rn(g.w, s);
    }
}

template <int UNROLL, bool PEERS, bool SCALED>
__device__ __forceinline__ void oe_adamw_body(const oe_dev_tensor* __restrict__ tensors,
                                              const oe_dev_chunk* __restrict__ chunks, uint32_t n_chunks,
                                              uint32_t chunk_elems, const oe_adamw_args& a, const oe_peer_set& peers) {
    // Sharded step: an exchange between the ranks that gave up leaves a non-zero status word;
    // every later launch of that step then does nothing (the word is uniform over the grid).
    if (a.status != 0 && *(const volatile uint32_t*)a.status != 0u) return;
    oe_adamw_consts k;
    k.b1 = a.beta1;
    k.b2 = a.beta2;
    k.omb1 = __fsub_rn(1.0f, a.beta1);
    k.omb2 = __fsub_rn(1.0f, a.beta2);
    k.eps = a.eps;
    k.bc1 = a.bc1;
    k.bc2 = a.bc2;
    int32_t step_now = 0;
    if (a.step_dev != 0) {
        // Capture mode: the step counter lives on the device. This launch is step
        // counter+1 (the reference advances it with a launch of its own first,
        // graph_adam_inc, autograd/cuda_kernels.go:595; here the CTA that finishes last
        // stores the new value, see the end of this function). Bias correction as on
        // the host, in double (autograd/nn.go:493-494).
        step_now = *(const int32_t*)a.step_dev + 1;
        double t = (double)step_now;
        // The two double-precision pow calls are the longest dependent chain of a small launch:
        // two warps take one each.
        __shared__ float bc_shared[2];
        if (threadIdx.x == 0) bc_shared[0] = (float)(1.0 - pow((double)a.beta1, t));
        if (threadIdx.x == 32) bc_shared[1] = (float)(1.0 - pow((double)a.beta2, t));
        __syncthreads();
        k.bc1 = bc_shared[0];
        k.bc2 = bc_shared[1];
    }
    k.coef = oe_clip_coefficient((const oe_dev_norm*)a.norm, a.max_norm, a.flags);
    k.gscale = a.grad_scale;
    const bool want_shadow = (a.flags & OE_F_WRITE_SHADOW) != 0;
    const bool zero_grad = (a.flags & OE_F_ZERO_GRAD) != 0;
    // A captured step bakes its launch parameters into the graph; a device-resident rate
    // lets a schedule change it between replays without capturing again.
    const float base_lr = a.lr_dev != 0 ? *(const float*)a.lr_dev : a.lr;

    for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        oe_chunk_view cv = oe_view(tensors, chunks, c, chunk_elems);
        const oe_dev_tensor* t = cv.t;
        float* __restrict__ p = (float*)t->param + cv.base;
        float* __restrict__ g = (float*)t->grad + cv.base;
        float* __restrict__ m = (float*)t->state1 + cv.base;
        float* __restrict__ v = (float*)t->state2 + cv.base;
        uint16_t* __restrict__ sh = (want_shadow && t->shadow) ? (uint16_t*)t->shadow + cv.base : nullptr;
        // Group scaling in fp32 exactly as AdamW.groupScale (autograd/nn.go:461-465).
        const float step = __fmul_rn(base_lr, t->lr_scale);
        const float omd = __fsub_rn(1.0f, __fmul_rn(step, t->weight_decay));
        uint32_t done = 0;
        if ((t->aligned & (OE_ALIGNED_BASE | OE_ALIGNED_STATE2)) == (OE_ALIGNED_BASE | OE_ALIGNED_STATE2)) {
            const uint32_t nvec = cv.n >> 2;
            float4* p4 = (float4*)p;
            float4* g4 = (float4*)g;
            float4* m4 = (float4*)m;
            float4* v4 = (float4*)v;
            for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += OE_THREADS * UNROLL) {
                float4 P[UNROLL], G[UNROLL], M[UNROLL], V[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    uint32_t i = i0 + u * OE_THREADS;
                    if (i < nvec) {
                        G[u] = __ldcs(g4 + i);
                        P[u] = __ldcs(p4 + i);
                        M[u] = __ldcs(m4 + i);
                        V[u] = __ldcs(v4 + i);
                    }
                }
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    uint32_t i = i0 + u * OE_THREADS;
                    if (i < nvec) {
                        oe_scale4<SCALED>(G[u], k.gscale);
                        oe_adamw_one(P[u].x, G[u].x, M[u].x, V[u].x, k, step, omd);
                        oe_adamw_one(P[u].y, G[u].y, M[u].y, V[u].y, k, step, omd);
                        oe_adamw_one(P[u].z, G[u].z, M[u].z, V[u].z, k, step, omd);
                        oe_adamw_one(P[u].w, G[u].w, M[u].w, V[u].w, k, step, omd);
                        __stcs(p4 + i, P[u]);
                        __stcs(m4 + i, M[u]);
                        __stcs(v4 + i, V[u]);
                        if (sh) {
                            uint2 packed;
                            packed.x = oe_bf16_rne(P[u].x) | (oe_bf16_rne(P[u].y) << 16);
                            packed.y = oe_bf16_rne(P[u].z) | (oe_bf16_rne(P[u].w) << 16);
                            oe_store_shadow4<PEERS>(sh, i, packed, peers);
                        }
                        if (zero_grad) __stcs(g4 + i, make_float4(0.f, 0.f, 0.f, 0.f));
                    }
                }
            }
            done = nvec << 2;
        }
        // Scalar path: the tail of an aligned chunk (< 4 elements) or a whole chunk
        // of a tensor whose pointers do not allow 128-bit accesses.
        for (uint32_t i = done + threadIdx.x; i < cv.n; i += OE_THREADS) {
            float pi = p[i], mi = m[i], vi = v[i];
            oe_adamw_one(pi, SCALED ? __fmul_rn(g[i], k.gscale) : g[i], mi, vi, k, step, omd);
            p[i] = pi;
            m[i] = mi;
            v[i] = vi;
            if (sh) oe_store_shadow1<PEERS>(sh, i, (uint16_t)oe_bf16_rne(pi), peers);
            if (zero_grad) g[i] = 0.0f;
        }
    }
    // Peer stores must be performed before the kernel is reported complete to other devices.
    if (PEERS) __threadfence_system();
    if (a.step_dev != 0) {
        // Every CTA read the counter before it got here, so the one that arrives last may
        // store the new value; it also re-arms the arrival counter for the next replay.
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t* ticket = (uint32_t*)a.ticket;
            __threadfence();
            if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
                *ticket = 0u;
                *(int32_t*)a.step_dev = step_now;
            }
        }
    }
}

// The update kernel is built in a few shapes (vectors in flight per thread x resident
// CTAs per SM); the shim picks one per plan. All shapes compute identical results.
#define OE_ADAMW_VARIANT(name, unroll, min_blocks)                                                         \
    extern "C" __global__ void __launch_bounds__(OE_THREADS, min_blocks)                                   \
    name(const oe_dev_tensor* __restrict__ tensors, const oe_dev_chunk* __restrict__ chunks,               \
         uint32_t n_chunks, uint32_t chunk_elems, oe_adamw_args a) {                                       \
        oe_peer_set none;                                                                                  \
        none.n = 0;                                                                                        \
        if (a.grad_scale == 1.0f)                                                                          \
            oe_adamw_body<unroll, false, false>(tensors, chunks, n_chunks, chunk_elems, a, none);          \
        else                                                                                               \
            oe_adamw_body<unroll, false, true>(tensors, chunks, n_chunks, chunk_elems, a, none);           \
    }
// Default: four 128-bit vectors per stream in flight per thread, two CTAs per SM (measured
// fastest on B200: fewer, fatter threads keep more bytes in flight than more CTAs do).
OE_ADAMW_VARIANT(oe_adamw_fused, 4, 2)
OE_ADAMW_VARIANT(oe_adamw_fused_u1, 1, 4)
OE_ADAMW_VARIANT(oe_adamw_fused_u2, 2, 3)
OE_ADAMW_VARIANT(oe_adamw_fused_u8, 8, 1)

// Sharded step: same update, shadow stored into every rank's shadow buffer. Built in the same
// shapes as the single-GPU kernel (vectors in flight per thread x resident CTAs per SM); which one
// keeps the NVLink stores flowing best depends on the number of ranks, so the shim exposes the choice.
#define OE_ADAMW_PEERS_VARIANT(name, unroll, min_blocks)                                                    \
    extern "C" __global__ void __launch_bounds__(OE_THREADS, min_blocks)                                    \
    name(const oe_dev_tensor* __restrict__ tensors, const oe_dev_chunk* __restrict__ chunks, uint32_t n_chunks, \
         uint32_t chunk_elems, oe_adamw_args a, const __grid_constant__ oe_peer_set peers) {                \
        if (a.grad_scale == 1.0f)                                                                           \
            oe_adamw_body<unroll, true, false>(tensors, chunks, n_chunks, chunk_elems, a, peers);           \
        else                                                                                                \
            oe_adamw_body<unroll, true, true>(tensors, chunks, n_chunks, chunk_elems, a, peers);            \
    }
OE_ADAMW_PEERS_VARIANT(oe_adamw_fused_peers, 4, 2)
OE_ADAMW_PEERS_VARIANT(oe_adamw_fused_peers_u2, 2, 3)
OE_ADAMW_PEERS_VARIANT(oe_adamw_fused_peers_u8, 8, 1)

// Advances a device step counter on its own: used when a captured step has no work unit
// at all (no parameter has a gradient), so no update launch could do it.
extern "C" __global__ void oe_step_increment(int32_t* step) {
    if (blockIdx.x == 0 && threadIdx.x == 0) step[0] += 1;
}

// ---------------------------------------------------------------------------------
// SGD (PyTorch semantics: coupled decay, momentum, dampening, Nesterov, maximize)
// ---------------------------------------------------------------------------------
struct oe_sgd_consts {
    float momentum, one_minus_damp, coef, gscale;
    bool nesterov, maximize;
};

// One element of SGD.Step's host loop (autograd/sgd.go:205-220).
__device__ __forceinline__ void oe_sgd_one(float& p, float g, float& b, const oe_sgd_consts& k, float lr, float decay,
                                           bool first) {
    g = __fmul_rn(g, k.coef);
    if (k.maximize) g = -g;
    g = __fadd_rn(g, __fmul_rn(decay, p));
    if (k.momentum > 0.0f) {
        float nb = first ? g : __fadd_rn(__fmul_rn(k.momentum, b), __fmul_rn(k.one_minus_damp, g));
        b = nb;
        g = k.nesterov ? __fadd_rn(g, __fmul_rn(k.momentum, nb)) : nb;
    }
    p = __fsub_rn(p, __fmul_rn(lr, g));
}

template <bool SCALED, bool PEERS>
__device__ __forceinline__ void oe_sgd_body(const oe_dev_tensor* __restrict__ tensors,
                                            const oe_dev_chunk* __restrict__ chunks, uint32_t n_chunks,
                                            uint32_t chunk_elems, const oe_sgd_args& a, const oe_peer_set& peers) {
    if (a.status != 0 && *(const volatile uint32_t*)a.status != 0u) return;
    oe_sgd_consts k;
    k.momentum = a.momentum;
    k.one_minus_damp = __fsub_rn(1.0f, a.dampening);
    k.coef = oe_clip_coefficient((const oe_dev_norm*)a.norm, a.max_norm, a.flags);
    k.gscale = a.grad_scale;
    k.nesterov = (a.flags & OE_F_NESTEROV) != 0;
    k.maximize = (a.flags & OE_F_MAXIMIZE) != 0;
    const bool want_shadow = (a.flags & OE_F_WRITE_SHADOW) != 0;
    const bool zero_grad = (a.flags & OE_F_ZERO_GRAD) != 0;
    const float base_lr = a.lr_dev != 0 ? *(const float*)a.lr_dev : a.lr;

    for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        oe_chunk_view cv = oe_view(tensors, chunks, c, chunk_elems);
        const oe_dev_tensor* t = cv.t;
        float* __restrict__ p = (float*)t->param + cv.base;
        float* __restrict__ g = (float*)t->grad + cv.base;
        const bool has_buf = k.momentum > 0.0f && t->state1 != 0;
        float* __restrict__ b = has_buf ? (float*)t->state1 + cv.base : nullptr;
        // The per-tensor device flag says whether the momentum buffer holds a value
        // yet (autograd/cuda_sgd.go:14); the last CTA of this launch sets it.
        const bool first = has_buf && t->state2 != 0 ? (*(const float*)t->state2 == 0.0f) : true;
        uint16_t* __restrict__ sh = (want_shadow && t->shadow) ? (uint16_t*)t->shadow + cv.base : nullptr;
        // SGD.groupScale (autograd/sgd.go:127-130): the decay is not scaled by the rate.
        const float lr = __fmul_rn(base_lr, t->lr_scale);
        const float decay = t->weight_decay;
        uint32_t done = 0;
        if (t->aligned & OE_ALIGNED_BASE) {
            const uint32_t nvec = cv.n >> 2;
            float4* p4 = (float4*)p;
            float4* g4 = (float4*)g;
            float4* b4 = (float4*)b;
            for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += OE_THREADS * OE_UNROLL) {
                float4 P[OE_UNROLL], G[OE_UNROLL], B[OE_UNROLL];
#pragma unroll
                for (int u = 0; u < OE_UNROLL; u++) {
                    uint32_t i = i0 + u * OE_THREADS;
                    if (i < nvec) {
                        G[u] = __ldcs(g4 + i);
                        P[u] = __ldcs(p4 + i);
                        B[u] = (has_buf && !first) ? __ldcs(b4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
#pragma unroll
                for (int u = 0; u < OE_UNROLL; u++) {
                    uint32_t i = i0 + u * OE_THREADS;
                    if (i < nvec) {
                        oe_scale4<SCALED>(G[u], k.gscale);
                        oe_sgd_one(P[u].x, G[u].x, B[u].x, k, lr, decay, first);
                        oe_sgd_one(P[u].y, G[u].y, B[u].y, k, lr, decay, first);
                        oe_sgd_one(P[u].z, G[u].z, B[u].z, k, lr, decay, first);
                        oe_sgd_one(P[u].w, G[u].w, B[u].w, k, lr, decay, first);
                        __stcs(p4 + i, P[u]);
                        if (has_buf) __stcs(b4 + i, B[u]);
                        if (sh) {
                            uint2 packed;
                            packed.x = oe_bf16_rne(P[u].x) | (oe_bf16_rne(P[u].y) << 16);
                            packed.y = oe_bf16_rne(P[u].z) | (oe_bf16_rne(P[u].w) << 16);
                            oe_store_shadow4<PEERS>(sh, i, packed, peers);
                        }
                        if (zero_grad) __stcs(g4 + i, make_float4(0.f, 0.f, 0.f, 0.f));
                    }
                }
            }
            done = nvec << 2;
        }
        for (uint32_t i = done + threadIdx.x; i < cv.n; i += OE_THREADS) {
            float pi = p[i];
            float bi = (has_buf && !first) ? b[i] : 0.0f;
            oe_sgd_one(pi, SCALED ? __fmul_rn(g[i], k.gscale) : g[i], bi, k, lr, decay, first);
            p[i] = pi;
            if (has_buf) b[i] = bi;
            if (sh) oe_store_shadow1<PEERS>(sh, i, (uint16_t)oe_bf16_rne(pi), peers);
            if (zero_grad) g[i] = 0.0f;
        }
    }
    // Peer stores must be performed before the kernel is reported complete to other devices.
    if (PEERS) __threadfence_system();
    if (k.momentum > 0.0f) {
        // Every tensor that took part now has an initialised momentum buffer (the reference's
        // sgd_mark, one launch per tensor, autograd/cuda_sgd.go:14-16). Every CTA read the flags
        // of its work units before it got here, so the CTA that arrives last may set them all;
        // it also re-arms the arrival counter.
        __shared__ uint32_t is_last;
        uint32_t* ticket = (uint32_t*)a.ticket;
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            is_last = (atomicAdd(ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
        }
        __syncthreads();
        if (is_last) {
            for (uint32_t i = threadIdx.x; i < a.n_tensors; i += OE_THREADS)
                if (tensors[i].state1 != 0 && tensors[i].state2 != 0) *(float*)tensors[i].state2 = 1.0f;
            if (threadIdx.x == 0) *ticket = 0u;
        }
    }
}

extern "C" __global__ void __launch_bounds__(OE_THREADS, 2)
oe_sgd_fused(const oe_dev_tensor* __restrict__ tensors, const oe_dev_chunk* __restrict__ chunks, uint32_t n_chunks,
             uint32_t chunk_elems, oe_sgd_args a) {
    // Capture mode: the launch advances the device step counter (the reference's sgd_step,
    // autograd/cuda_sgd.go:18); nothing in the update reads it.
    if (a.step_dev != 0 && blockIdx.x == 0 && threadIdx.x == 0) *(int32_t*)a.step_dev += 1;
    oe_peer_set none;
    none.n = 0;
    if (a.grad_scale == 1.0f)
        oe_sgd_body<false, false>(tensors, chunks, n_chunks, chunk_elems, a, none);
    else
        oe_sgd_body<true, false>(tensors, chunks, n_chunks, chunk_elems, a, none);
}

// Sharded step: same update, shadow stored into every rank's shadow buffer.
extern "C" __global__ void __launch_bounds__(OE_THREADS, 2)
oe_sgd_fused_peers(const oe_dev_tensor* __restrict__ tensors, const oe_dev_chunk* __restrict__ chunks, uint32_t n_chunks,
                   uint32_t chunk_elems, oe_sgd_args a, const __grid_constant__ oe_peer_set peers) {
    if (a.step_dev != 0 && blockIdx.x == 0 && threadIdx.x == 0) *(int32_t*)a.step_dev += 1;
    if (a.grad_scale == 1.0f)
        oe_sgd_body<false, true>(tensors, chunks, n_chunks, chunk_elems, a, peers);
    else
        oe_sgd_body<true, true>(tensors, chunks, n_chunks, chunk_elems, a, peers);
}

// ---------------------------------------------------------------------------------
// gradient norm: sum of squares in double, two levels, deterministic
// ---------------------------------------------------------------------------------
__device__ __forceinline__ double oe_block_sum(double x, double* warp_sums) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) x += __shfl_down_sync(0xffffffffu, x, off);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) warp_sums[warp] = x;
    __syncthreads();
    double total = 0.0;
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 0; w < OE_THREADS / 32; w++) total += warp_sums[w];
    }
    __syncthreads();
    return total;  // valid in thread 0
}

// One CTA's share of the sum: OE_NORM_SPAN consecutive work units at a time (for a read-only
// 4 B/param stream a longer contiguous run per CTA measured ~6 % faster than single
// 4096-element units). SCALED: the norm of the gradient as the update will read it,
// (float)(g*scale) converted to double.
template <bool SCALED>
__device__ __forceinline__ double oe_sumsq_walk(const oe_dev_tensor* __restrict__ tensors,
                                                const oe_dev_chunk* __restrict__ chunks, uint32_t n_chunks,
                                                uint32_t chunk_elems, float gscale) {
    double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
    const uint32_t n_spans = (n_chunks + OE_NORM_SPAN - 1) / OE_NORM_SPAN;
    for (uint32_t sp = blockIdx.x; sp < n_spans; sp += gridDim.x)
    for (uint32_t c = sp * OE_NORM_SPAN; c < n_chunks && c < (sp + 1) * OE_NORM_SPAN; c++) {
        oe_chunk_view cv = oe_view(tensors, chunks, c, chunk_elems);
        const float* __restrict__ g = (const float*)cv.t->grad + cv.base;
        uint32_t done = 0;
        if (cv.t->aligned & OE_ALIGNED_BASE) {
            const uint32_t nvec = cv.n >> 2;
            const float4* g4 = (const float4*)g;
            for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += OE_THREADS * OE_NORM_UNROLL) {
                float4 G[OE_NORM_UNROLL];
#pragma unroll
                for (int u = 0; u < OE_NORM_UNROLL; u++) {
                    uint32_t i = i0 + u * OE_THREADS;
                    G[u] = i < nvec ? __ldcs(g4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < OE_NORM_UNROLL; u++) {
                    oe_scale4<SCALED>(G[u], gscale);
                    double x = (double)G[u].x, y = (double)G[u].y, z = (double)G[u].z, w = (double)G[u].w;
                    a0 = fma(x, x, a0);
                    a1 = fma(y, y, a1);
                    a2 = fma(z, z, a2);
                    a3 = fma(w, w, a3);
                }
            }
            done = nvec << 2;
        }
        for (uint32_t i = done + threadIdx.x; i < cv.n; i += OE_THREADS) {
            double x = (double)(SCALED ? __fmul_rn(g[i], gscale) : g[i]);
            a0 = fma(x, x, a0);
        }
    }
    return (a0 + a1) + (a2 + a3);
}

// Level 1: every CTA accumulates its chunks in double (the reference's host code sums in
// float64 too, autograd/nn.go:319-324) and writes one partial. Level 2: the CTA that
// arrives last adds the partials in index order, so the result depends only on the
// grid size, never on timing; it stores sum, norm = (float)sqrt(sum) and re-arms the
// ticket, so the launch needs no memset and can be captured in a graph.
extern "C" __global__ void __launch_bounds__(OE_THREADS, 4)
oe_grad_sumsq(const oe_dev_tensor* __restrict__ tensors, const oe_dev_chunk* __restrict__ chunks, uint32_t n_chunks,
              uint32_t chunk_elems, oe_dev_norm* out, double* partials, uint32_t flags, float gscale) {
    __shared__ double warp_sums[OE_THREADS / 32];
    __shared__ uint32_t is_last;
    const double mine = gscale == 1.0f ? oe_sumsq_walk<false>(tensors, chunks, n_chunks, chunk_elems, gscale)
                                       : oe_sumsq_walk<true>(tensors, chunks, n_chunks, chunk_elems, gscale);
    double block = oe_block_sum(mine, warp_sums);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = block;
        __threadfence();
        uint32_t ticket = atomicAdd(&out->ticket, 1u);
        is_last = (ticket == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    double s = 0.0;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += OE_THREADS) s += __ldcg(partials + i);
    double total = oe_block_sum(s, warp_sums);
    if (threadIdx.x == 0) {
        out->sumsq = total;
        if (!(flags & OE_F_PARTIAL_ONLY)) out->norm = (float)sqrt(total);
        out->ticket = 0u;
    }
}

// norm = (float)sqrt(sumsq) for a sum that was completed elsewhere (for instance by
// an all-reduce over the ranks of a sharded step).
extern "C" __global__ void oe_norm_finalize(oe_dev_norm* out) {
    if (blockIdx.x == 0 && threadIdx.x == 0) out->norm = (float)sqrt(out->sumsq);
}

// In-place clip: g *= coefficient (autograd/nn.go:327-333, autograd/cuda_kernels.go:676).
// A coefficient of exactly 1 writes nothing.
extern "C" __global__ void __launch_bounds__(OE_THREADS, 4)
oe_scale_grads(const oe_dev_tensor* __restrict__ tensors, const oe_dev_chunk* __restrict__ chunks, uint32_t n_chunks,
               uint32_t chunk_elems, const oe_dev_norm* norm, float max_norm, uint32_t flags) {
    const float coef = oe_clip_coefficient(norm, max_norm, flags);
    if (coef == 1.0f) return;
    for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        oe_chunk_view cv = oe_view(tensors, chunks, c, chunk_elems);
        float* __restrict__ g = (float*)cv.t->grad + cv.base;
        uint32_t done = 0;
        if (cv.t->aligned & OE_ALIGNED_BASE) {
            const uint32_t nvec = cv.n >> 2;
            float4* g4 = (float4*)g;
            for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += OE_THREADS * OE_NORM_UNROLL) {
                float4 G[OE_NORM_UNROLL];
#pragma unroll
                for (int u = 0; u < OE_NORM_UNROLL; u++) {
                    uint32_t i = i0 + u * OE_THREADS;
                    if (i < nvec) G[u] = __ldcs(g4 + i);
                }
#pragma unroll
                for (int u = 0; u < OE_NORM_UNROLL; u++) {
                    uint32_t i = i0 + u * OE_THREADS;
                    if (i < nvec) {
                        G[u].x = __fmul_rn(G[u].x, coef);
                        G[u].y = __fmul_rn(G[u].y, coef);
                        G[u].z = __fmul_rn(G[u].z, coef);
                        G[u].w = __fmul_rn(G[u].w, coef);
                        __stcs(g4 + i, G[u]);
                    }
                }
            }
            done = nvec << 2;
        }
        for (uint32_t i = done + threadIdx.x; i < cv.n; i += OE_THREADS) g[i] = __fmul_rn(g[i], coef);
    }
}

// Zero every present gradient in one launch (AdamW.ZeroGrad keeps the buffers and
// memsets each of them, autograd/nn.go:533-537, autograd/tensor.go:407-420).
extern "C" __global__ void __launch_bounds__(OE_THREADS, 4)
oe_zero_grads(const oe_dev_tensor* __restrict__ tensors, const oe_dev_chunk* __restrict__ chunks, uint32_t n_chunks,
              uint32_t chunk_elems) {
    for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        oe_chunk_view cv = oe_view(tensors, chunks, c, chunk_elems);
        float* __restrict__ g = (float*)cv.t->grad + cv.base;
        uint32_t done = 0;
        if (cv.t->aligned & OE_ALIGNED_BASE) {
            const uint32_t nvec = cv.n >> 2;
            float4* g4 = (float4*)g;
            for (uint32_t i = threadIdx.x; i < nvec; i += OE_THREADS) __stcs(g4 + i, make_float4(0.f, 0.f, 0.f, 0.f));
            done = nvec << 2;
        }
        for (uint32_t i = done + threadIdx.x; i < cv.n; i += OE_THREADS) g[i] = 0.0f;
    }
}

// ---------------------------------------------------------------------------------
// stand-alone fp32 -> bf16 cast (the reference's f32_to_bf16, one tensor per call)
// ---------------------------------------------------------------------------------
// One CTA per tile of OE_THREADS x OE_UNROLL vectors (16 KB read, 8 KB written, both contiguous), launched
// in address order WITHOUT a persistent grid: for this 2:1 read/write stream a compact window of
// CTAs that sweeps the buffer in order measured 7.1 TB/s on B200 (6.3 TB/s on a 65 M-element tensor,
// a 62 us launch), against 5.7 / 5.5 TB/s for a persistent grid striding over the same tiles and 5.8
// for per-thread grid strides. Four 128-bit loads are in flight per thread before the first use. The
// loop only matters beyond 2^31-1 tiles, where the host caps the grid.
extern "C" __global__ void __launch_bounds__(OE_THREADS, 4)
oe_cast_bf16(const float* __restrict__ src, uint16_t* __restrict__ dst, uint64_t n) {
    const bool aligned = (((uint64_t)src & 15u) == 0) && (((uint64_t)dst & 7u) == 0);
    uint64_t done = 0;
    if (aligned) {
        const uint64_t nvec = n >> 2;
        const float4* s4 = (const float4*)src;
        uint2* d2 = (uint2*)dst;
        const uint64_t tile = (uint64_t)OE_THREADS * OE_UNROLL;
        for (uint64_t t0 = (uint64_t)blockIdx.x * tile; t0 < nvec; t0 += (uint64_t)gridDim.x * tile) {
            float4 x[OE_UNROLL];
#pragma unroll
            for (int u = 0; u < OE_UNROLL; u++) {
                uint64_t i = t0 + (uint64_t)u * OE_THREADS + threadIdx.x;
                if (i < nvec) x[u] = __ldcs(s4 + i);
            }
#pragma unroll
            for (int u = 0; u < OE_UNROLL; u++) {
                uint64_t i = t0 + (uint64_t)u * OE_THREADS + threadIdx.x;
                if (i < nvec) {
                    uint2 packed;
                    packed.x = oe_bf16_rne(x[u].x) | (oe_bf16_rne(x[u].y) << 16);
                    packed.y = oe_bf16_rne(x[u].z) | (oe_bf16_rne(x[u].w) << 16);
                    __stcs(d2 + i, packed);
                }
            }
        }
        done = nvec << 2;
    }
    const uint64_t tid = (uint64_t)blockIdx.x * OE_THREADS + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * OE_THREADS;
    for (uint64_t i = done + tid; i < n; i += stride) dst[i] = (uint16_t)oe_bf16_rne(src[i]);
}

// ---------------------------------------------------------------------------------
// sharded step: pull reduce-scatter of the gradients fused with the norm pass
// ---------------------------------------------------------------------------------
// Every rank holds a full flat gradient buffer of the same layout. The rank that owns
// the shard [first, first+numel) reads that range from every rank's buffer with plain
// 128-bit loads (its own from HBM, the others over NVLink through peer-mapped
// addresses), adds them in ascending rank order — so the sum is the same on every run
// and can be reproduced on the host —, scales the sum (1/n for a mean), writes the
// reduced shard to `out` and accumulates its sum of squares in double in the same pass:
// the reduce-scatter and the 4 B/param norm read of the single-GPU step become one
// kernel. `out` may be this rank's own range (in place): a thread reads every element it
// writes before it writes it, and no other rank reads that range of this buffer.
// No flag or barrier is waited on here; ordering against the other ranks is the host's
// job (stream-ordered collectives before and after).
// The streaming part of the reduction for one order of issue: returns this thread's sum of squares.
template <int NP, int U, int ROT>
__device__ __forceinline__ double oe_peer_reduce_stream(const oe_peer_grads& pg, uint64_t first, uint64_t numel,
                                                        float* __restrict__ out) {
    const uint32_t n = pg.n;
    const float scale = pg.scale;
    double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
    bool aligned = (((uint64_t)out | (first * 4u)) & 15u) == 0;
#pragma unroll
    for (int k = 0; k < NP; k++)
        if (k < (int)n) aligned = aligned && ((pg.base[k] & 15u) == 0);
    const uint64_t tid = (uint64_t)blockIdx.x * OE_THREADS + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * OE_THREADS;
    uint64_t done = 0;
    if (aligned) {
        const uint64_t nvec = numel >> 2;
        float4* o4 = (float4*)out;
        // U x n 128-bit loads are issued before the first add: a remote load takes a few
        // microseconds, so bytes in flight per SM decide the NVLink throughput.
        // Loads go through L2 only (ld.global.cg): peer data must not linger in L1, and on B200 this
        // flavour pulls 4 % faster over NVLink than streaming (.cs) loads (656 vs 629 GB/s).
        for (uint64_t i0 = tid; i0 < nvec; i0 += (uint64_t)U * stride) {
            float4 v[U][NP];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const uint64_t i = i0 + (uint64_t)u * stride;
                // Issue order: rank ROT first, then upwards and around. The slot of a value is its
                // rank, whatever the order of issue, so the adds below stay in ascending rank order.
#pragma unroll
                for (int kk = 0; kk < NP; kk++) {
                    const int k = (kk + ROT) % NP;
                    if (k < (int)n && i < nvec) v[u][k] = __ldcg((const float4*)((const float*)pg.base[k] + first) + i);
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const uint64_t i = i0 + (uint64_t)u * stride;
                if (i < nvec) {
                    float4 s = v[u][0];
#pragma unroll
                    for (int k = 1; k < NP; k++) {
                        if (k < (int)n) {
                            s.x = __fadd_rn(s.x, v[u][k].x);
                            s.y = __fadd_rn(s.y, v[u][k].y);
                            s.z = __fadd_rn(s.z, v[u][k].z);
                            s.w = __fadd_rn(s.w, v[u][k].w);
                        }
                    }
                    s.x = __fmul_rn(s.x, scale);
                    s.y = __fmul_rn(s.y, scale);
                    s.z = __fmul_rn(s.z, scale);
                    s.w = __fmul_rn(s.w, scale);
                    if (!(pg.flags & OE_F_NO_STORE)) __stcs(o4 + i, s);
                    double x = (double)s.x, y = (double)s.y, z = (double)s.z, w = (double)s.w;
                    a0 = fma(x, x, a0);
                    a1 = fma(y, y, a1);
                    a2 = fma(z, z, a2);
                    a3 = fma(w, w, a3);
                }
            }
        }
        done = nvec << 2;
    }
    for (uint64_t i = done + tid; i < numel; i += stride) {
        float s = __ldcg((const float*)pg.base[0] + first + i);
        for (uint32_t k = 1; k < n; k++) s = __fadd_rn(s, __ldcg((const float*)pg.base[k] + first + i));
        s = __fmul_rn(s, scale);
        if (!(pg.flags & OE_F_NO_STORE)) out[i] = s;
        double x = (double)s;
        a0 = fma(x, x, a0);
    }
    return (a0 + a1) + (a2 + a3);
}

// One instance of the streaming part per first-issued rank. pg.rot is uniform over the grid (the host
// passes the rank's own number + 1, so the ranks of a step do not all address the same source first);
// with OE_F_WARP_ROTATE every warp of a CTA adds its own number, so the warps of a CTA do not either.
// The choice is uniform over a warp, so the switch costs nothing; block-wide barriers come after it.
template <int NP, int U>
__device__ __forceinline__ void oe_peer_reduce_body(const oe_peer_grads& pg, uint64_t first, uint64_t numel,
                                                    float* __restrict__ out, oe_dev_norm* rec, double* partials) {
    __shared__ double warp_sums[OE_THREADS / 32];
    __shared__ uint32_t is_last;
    if (pg.status != 0 && *(const volatile uint32_t*)pg.status != 0u) return;  // a failed exchange: skip
    const uint32_t rot = (pg.rot + ((pg.flags & OE_F_WARP_ROTATE) ? (threadIdx.x >> 5) : 0u)) % NP;
    double mine;
    switch (rot) {
        case 1: mine = oe_peer_reduce_stream<NP, U, 1 % NP>(pg, first, numel, out); break;
        case 2: mine = oe_peer_reduce_stream<NP, U, 2 % NP>(pg, first, numel, out); break;
        case 3: mine = oe_peer_reduce_stream<NP, U, 3 % NP>(pg, first, numel, out); break;
        case 4: mine = oe_peer_reduce_stream<NP, U, 4 % NP>(pg, first, numel, out); break;
        case 5: mine = oe_peer_reduce_stream<NP, U, 5 % NP>(pg, first, numel, out); break;
        case 6: mine = oe_peer_reduce_stream<NP, U, 6 % NP>(pg, first, numel, out); break;
        case 7: mine = oe_peer_reduce_stream<NP, U, 7 % NP>(pg, first, numel, out); break;
        default: mine = oe_peer_reduce_stream<NP, U, 0>(pg, first, numel, out); break;
    }
    double block = oe_block_sum(mine, warp_sums);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = block;
        __threadfence();
        uint32_t ticket = atomicAdd(&rec->ticket, 1u);
        is_last = (ticket == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    double s = 0.0;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += OE_THREADS) s += __ldcg(partials + i);
    double total = oe_block_sum(s, warp_sums);
    if (threadIdx.x == 0) {
        // A shard reduced piece by piece (one launch per staged piece) adds up in launch order.
        if (pg.flags & OE_F_ACCUMULATE) total = rec->sumsq + total;
        rec->sumsq = total;
        if (!(pg.flags & OE_F_PARTIAL_ONLY)) rec->norm = (float)sqrt(total);
        rec->ticket = 0u;
    }
}

#define OE_PEER_REDUCE_VARIANT(name, np, unroll)                                                               \
    extern "C" __global__ void __launch_bounds__(OE_THREADS, 2)                                       \
    name(const __grid_constant__ oe_peer_grads pg, uint64_t first, uint64_t numel, float* out, oe_dev_norm* rec, double* partials) { \
        oe_peer_reduce_body<np, unroll>(pg, first, numel, out, rec, partials);                             \
    }
OE_PEER_REDUCE_VARIANT(oe_peer_reduce_sumsq_n2, 2, 8)
OE_PEER_REDUCE_VARIANT(oe_peer_reduce_sumsq_n4, 4, 4)
OE_PEER_REDUCE_VARIANT(oe_peer_reduce_sumsq_n8, 8, 2)

// Link-rate probe for the stores of the sharded update: bf16 zeros over [0, n_vec) 8-byte vectors of every
// target in peers.delta, issued like the update kernel issues its shadow stores (four vectors per thread,
// one round of targets per vector, optional warp rotation) with no other memory traffic beside them.
extern "C" __global__ void __launch_bounds__(OE_THREADS, 2)
oe_probe_peer_stores(uint16_t* sh, uint64_t n_vec, const __grid_constant__ oe_peer_set peers) {
    const uint2 zero = make_uint2(0u, 0u);
    const uint64_t tile = (uint64_t)OE_THREADS * OE_UNROLL;
    for (uint64_t t0 = (uint64_t)blockIdx.x * tile; t0 < n_vec; t0 += (uint64_t)gridDim.x * tile) {
#pragma unroll
        for (int u = 0; u < OE_UNROLL; u++) {
            const uint64_t i = t0 + (uint64_t)u * OE_THREADS + threadIdx.x;
            if (i < n_vec) {
                uint32_t k = (peers.mode & OE_PEER_WARP_ROTATE) ? (threadIdx.x >> 5) % peers.n : 0u;
                for (uint32_t j = 0; j < peers.n; j++) {
                    __stcs((uint2*)((char*)sh + peers.delta[k]) + i, zero);
                    if (++k == peers.n) k = 0;
                }
            }
        }
    }
    __threadfence_system();
}

// ---------------------------------------------------------------------------------
// sharded step: exchange between the ranks without a collective library
// ---------------------------------------------------------------------------------
// One warp. Lane k speaks to rank k: it publishes this rank's arrival (and, at the middle
// exchange, its float64 partial sum of squares) in rank k's area with plain peer stores, then
// waits until rank k's arrival shows in this rank's own area. The wait is bounded twice, by the
// device clock and by a poll count: when either runs out the lane records which rank was
// missing in the sticky status word and the kernel returns; nothing spins for ever. After the
// middle exchange lane 0 adds the partial sums in rank order, so every rank computes the same
// total and the same norm, bit for bit.
__device__ __forceinline__ uint32_t oe_ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void oe_st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t oe_globaltimer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

extern "C" __global__ void __launch_bounds__(32, 1) oe_rank_exchange(const __grid_constant__ oe_sync_args a) {
    const uint32_t lane = threadIdx.x;
    oe_sync_block* own = (oe_sync_block*)a.block[a.rank];
    oe_dev_norm* rec = (oe_dev_norm*)a.norm_rec;
    if (*(volatile uint32_t*)&own->status != 0u) return;  // an earlier exchange already gave up
    const uint32_t parity = a.epoch & 1u;
    bool failed = false;
    if (lane < a.world) {
        oe_sync_block* theirs = (oe_sync_block*)a.block[lane];
        if (rec != nullptr) theirs->partial[parity][a.rank] = *(volatile double*)&rec->sumsq;
        // the stores of the kernels before this one on the stream, and the partial above, come first
        __threadfence_system();
        oe_st_release_sys(&theirs->arrive[a.phase][a.rank], a.epoch);
        const uint32_t* flag = &own->arrive[a.phase][lane];
        const uint64_t t0 = oe_globaltimer();
        uint32_t polls = 0;
        while ((int32_t)(oe_ld_acquire_sys(flag) - a.epoch) < 0) {
            if (++polls >= a.max_polls || oe_globaltimer() - t0 > a.timeout_ns) {
                failed = true;
                break;
            }
            __nanosleep(polls < 64 ? 100 : 1000);
        }
        if (failed) atomicCAS(&own->status, 0u, OE_SYNC_TIMEOUT | (a.phase << 8) | (lane << 16));
    }
    const bool any_failed = __any_sync(0xffffffffu, failed);
    __syncwarp();  // what the other lanes acquired is ordered before lane 0's reads below
    if (lane == 0 && rec != nullptr) {
        if (any_failed) {
            rec->error = OE_SYNC_TIMEOUT;
        } else {
            double total = 0.0;
            for (uint32_t r = 0; r < a.world; r++) total += *(volatile double*)&own->partial[parity][r];
            rec->sumsq = total;
            rec->norm = (float)sqrt(total);
        }
    }
}
