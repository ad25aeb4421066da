/*
 * CPU oracle for the optimizer-step path of yh2237/gograd.
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, operation for operation, the
 * reference's CPU (host) arithmetic so that the CUDA engine can be checked
 * against it. Nothing in the shipped library links, loads or calls it; only the
 * test-suite, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Parity pin: the reference itself (Go) cannot be built in this image, so the
 * restatement is pinned against the reference's own golden vectors
 * (testdata/sgd.json, testdata/param_groups.json, testdata/nn_conv_step.json and
 * the inline vectors of kernels/kernels_test.go:117-151,
 * autograd/audit_cuda_regression_test.go:66-178) by tests/test_oracle_golden.py.
 * The bf16 rounding formula has no golden vector in the reference; it is pinned
 * against an independent float->bfloat16 round-to-nearest-even conversion.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math (see oracle/Makefile). Every
 * variable is IEEE binary32 unless it says double; every operation rounds to
 * binary32 at once, exactly like Go on amd64 (which does not fuse a*b+c).
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* ---- bias correction: autograd/nn.go:493-494 ---------------------------------
 * bc = float32(1 - math.Pow(float64(beta), float64(t))) : double pow, one rounding. */
void oracle_bias_corrections(float beta1, float beta2, int64_t t, float *bc1, float *bc2) {
    *bc1 = (float)(1.0 - pow((double)beta1, (double)t));
    *bc2 = (float)(1.0 - pow((double)beta2, (double)t));
}

/* ---- group scaling ------------------------------------------------------------
 * AdamW: autograd/nn.go:461-465   step = LR*LRScale ; decay = step*WeightDecay
 * SGD:   autograd/sgd.go:127-130  lr   = LR*LRScale ; decay = WeightDecay
 * LRScale == 0 selects 1 (autograd/param_groups.go:46-54). */
float oracle_normalize_lr_scale(float scale) { return scale == 0.0f ? 1.0f : scale; }

void oracle_adamw_group_scale(float lr, float lr_scale, float weight_decay, float *step, float *decay) {
    float s = lr * lr_scale;
    *step = s;
    *decay = s * weight_decay;
}

void oracle_sgd_group_scale(float lr, float lr_scale, float weight_decay, float *step, float *decay) {
    *step = lr * lr_scale;
    *decay = weight_decay;
}

/* ---- AdamW element loop: autograd/nn.go:519-528 ------------------------------- */
static void adamw_range(float *data, const float *grad, float *m, float *v, size_t start, size_t end,
                        float b1, float b2, float eps, float step, float decay, float bc1, float bc2) {
    const float one_minus_b1 = 1.0f - b1, one_minus_b2 = 1.0f - b2;
    for (size_t i = start; i < end; i++) {
        float g = grad[i];
        float mi = b1 * m[i] + one_minus_b1 * g;
        float vi = b2 * v[i] + (one_minus_b2 * g) * g; /* Go parses a*b*c as (a*b)*c */
        m[i] = mi;
        v[i] = vi;
        /* float32(math.Sqrt(float64(x))) is the correctly rounded binary32 root. */
        float root = (float)sqrt((double)(vi / bc2));
        data[i] = data[i] * (1.0f - decay) - (step * (mi / bc1)) / (root + eps);
    }
}

void oracle_adamw_update(float *data, const float *grad, float *m, float *v, size_t n, float b1, float b2,
                         float eps, float step, float decay, float bc1, float bc2) {
    adamw_range(data, grad, m, v, 0, n, b1, b2, eps, step, decay, bc1, bc2);
}

/* The reference's CUDA kernel (kernels/optim.go:12-23, called from
 * autograd/nn.go:501 with stepSize/bc1) uses another operation order; kept here so
 * that tests can show how far the two reference forms lie apart. No FMA either. */
void oracle_adamw_update_devform(float *p, const float *g, float *m, float *v, size_t n, float norm,
                                 float b1, float b2, float step_over_bc1, float bc2, float decay, float eps,
                                 float max_norm) {
    float coefficient = max_norm > 0.0f ? fminf(1.0f, max_norm / (norm + 1e-6f)) : 1.0f;
    for (size_t i = 0; i < n; i++) {
        float grad = g[i] * coefficient;
        m[i] = b1 * m[i] + (1.0f - b1) * grad;
        v[i] = b2 * v[i] + ((1.0f - b2) * grad) * grad;
        float denom = sqrtf(v[i] / bc2) + eps;
        p[i] = p[i] * (1.0f - decay) - (step_over_bc1 * m[i]) / denom;
    }
}

/* ---- parallelFor: autograd/tensor.go:625-644 ----------------------------------
 * workers = min(GOMAXPROCS, n, n/65536); fewer than two runs inline; worker w gets
 * [n*w/workers, n*(w+1)/workers). Only the timed baseline uses it; the split does
 * not change any result because elements are independent. */
typedef struct {
    float *data, *m, *v;
    const float *grad;
    size_t start, end;
    float b1, b2, eps, step, decay, bc1, bc2;
} adamw_job;

static void *adamw_worker(void *arg) {
    adamw_job *j = (adamw_job *)arg;
    adamw_range(j->data, j->grad, j->m, j->v, j->start, j->end, j->b1, j->b2, j->eps, j->step, j->decay, j->bc1,
                j->bc2);
    return NULL;
}

int oracle_parallel_workers(size_t n, int max_procs) {
    size_t workers = (size_t)(max_procs > 0 ? max_procs : 1);
    if (n < workers) workers = n;
    if (n / 65536 < workers) workers = n / 65536;
    return (int)workers;
}

void oracle_adamw_update_parallel(float *data, const float *grad, float *m, float *v, size_t n, float b1,
                                  float b2, float eps, float step, float decay, float bc1, float bc2,
                                  int max_procs) {
    int workers = oracle_parallel_workers(n, max_procs);
    if (workers < 2) {
        adamw_range(data, grad, m, v, 0, n, b1, b2, eps, step, decay, bc1, bc2);
        return;
    }
    if (workers > 256) workers = 256;
    pthread_t threads[256];
    adamw_job jobs[256];
    for (int w = 0; w < workers; w++) {
        adamw_job j = {data, m, v, grad, n * (size_t)w / (size_t)workers, n * (size_t)(w + 1) / (size_t)workers,
                       b1,   b2, eps, step, decay, bc1, bc2};
        jobs[w] = j;
        pthread_create(&threads[w], NULL, adamw_worker, &jobs[w]);
    }
    for (int w = 0; w < workers; w++) pthread_join(threads[w], NULL);
}

/* ---- SGD element loop: autograd/sgd.go:205-220 --------------------------------
 * first != 0 means the parameter's momentum buffer has not been initialised yet.
 * The explicit float32(...) conversions of the reference are the natural binary32
 * roundings here. buffer may be NULL when momentum == 0. */
void oracle_sgd_update(float *data, const float *grad, float *buffer, size_t n, int first, float lr,
                       float momentum, float dampening, float decay, int nesterov, int maximize) {
    for (size_t i = 0; i < n; i++) {
        float g = grad[i];
        if (maximize) g = -g;
        g += decay * data[i];
        if (momentum > 0.0f) {
            if (first) {
                buffer[i] = g;
            } else {
                float a = momentum * buffer[i];
                float b = (1.0f - dampening) * g;
                buffer[i] = a + b;
            }
            if (nesterov) {
                float c = momentum * buffer[i];
                g += c;
            } else {
                g = buffer[i];
            }
        }
        float d = lr * g;
        data[i] -= d;
    }
}

/* ---- ClipGradNorm, CPU: autograd/nn.go:318-333 --------------------------------
 * Serial float64 sum of squares over the present gradients in list order;
 * norm = float32(sqrt(sum)); scale in place only when norm > max_norm > 0.
 * Returns the pre-clip norm. *scale_out receives the factor applied (1 if none). */
double oracle_sum_squares(const float *const *grads, const size_t *sizes, size_t count) {
    double sum = 0.0;
    for (size_t t = 0; t < count; t++) {
        const float *g = grads[t];
        for (size_t i = 0; i < sizes[t]; i++) sum += (double)g[i] * (double)g[i];
    }
    return sum;
}

float oracle_clip_coefficient(float norm, float max_norm) {
    if (norm > max_norm && max_norm > 0.0f) return max_norm / (norm + 1e-6f);
    return 1.0f;
}

/* The reference's CUDA kernels scale unconditionally by fminf(1, max/(norm+1e-6))
 * when max_norm > 0 (autograd/cuda_kernels.go:676, autograd/cuda_clip.go:130). */
float oracle_clip_coefficient_devform(float norm, float max_norm) {
    if (max_norm > 0.0f) return fminf(1.0f, max_norm / (norm + 1e-6f));
    return 1.0f;
}

float oracle_clip_grad_norm(float *const *grads, const size_t *sizes, size_t count, float max_norm,
                            float *scale_out) {
    double sum = oracle_sum_squares((const float *const *)grads, sizes, count);
    float norm = (float)sqrt(sum);
    float scale = 1.0f;
    if (norm > max_norm && max_norm > 0.0f) {
        scale = max_norm / (norm + 1e-6f);
        for (size_t t = 0; t < count; t++) {
            float *g = grads[t];
            for (size_t i = 0; i < sizes[t]; i++) g[i] *= scale;
        }
    }
    if (scale_out) *scale_out = scale;
    return norm;
}

void oracle_scale(float *g, size_t n, float scale) {
    for (size_t i = 0; i < n; i++) g[i] *= scale;
}

/* ---- fp32 -> bf16: autograd/cuda_kernels.go:86-87 -----------------------------
 * (bits + 0x7fff + ((bits >> 16) & 1)) >> 16, round-to-nearest-even for every
 * finite input and for infinities. For NaN inputs whose low mantissa bits make the
 * integer sum carry out of the mantissa the reference formula produces an infinity
 * or a zero of the opposite sign; the engine returns a quiet NaN with the input's
 * sign (sign | 0x7fc0) for every NaN instead, and so does this function when
 * nan_canonical != 0. With nan_canonical == 0 it is the raw reference formula. */
uint16_t oracle_f32_to_bf16_one(float x, int nan_canonical) {
    uint32_t bits;
    memcpy(&bits, &x, 4);
    if (nan_canonical && (bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)(((bits >> 16) & 0x8000u) | 0x7fc0u);
    return (uint16_t)((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
}

void oracle_f32_to_bf16(const float *x, uint16_t *y, size_t n, int nan_canonical) {
    for (size_t i = 0; i < n; i++) y[i] = oracle_f32_to_bf16_one(x[i], nan_canonical);
}

/* ---- AdamW state validation: autograd/optimizer_state.go:251-256 --------------
 * Returns the index of the first element with a non-finite m, or a non-finite or
 * negative v; n when all are valid. */
size_t oracle_first_invalid_moment(const float *m, const float *v, size_t n) {
    for (size_t i = 0; i < n; i++) {
        if (isnan(m[i]) || isinf(m[i]) || isnan(v[i]) || isinf(v[i]) || v[i] < 0.0f) return i;
    }
    return n;
}
