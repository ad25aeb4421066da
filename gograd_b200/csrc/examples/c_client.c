/*
 * A plain-C client of liboptengine.so: what a foreign-language binding does, without any Python.
 * It allocates two two-element parameters through the library, gives them present all-zero
 * gradients, decay 2 and group rate scales 1 and 0.5 at base rate 0.2, runs four AdamW steps and
 * checks p = p0 * 0.6^4 and p0 * 0.8^4 — the analytic case of the reference's
 * TestAuditAdamWCapturedDecayCUDA (autograd/audit_cuda_regression_test.go:66-119). Then it clips a
 * (3, 4) gradient to norm 1 in place and reads the norm 5 back (:121-178).
 *
 *   cc c_client.c -I../../../include -L../.. -loptengine -Wl,-rpath,../.. -lm -o c_client && ./c_client
 */
#include <math.h>
#include <stdio.h>
#include <string.h>

#include "optengine.h"

#define CHECK(call)                                                          \
    do {                                                                     \
        int rc_ = (call);                                                    \
        if (rc_ != 0) {                                                      \
            fprintf(stderr, "%s failed (%d): %s\n", #call, rc_, oe_last_error()); \
            return 1;                                                        \
        }                                                                    \
    } while (0)

int main(void) {
    const int dev = 0;
    CHECK(oe_init(dev));
    uint64_t p[2], g[2], m[2], v[2];
    const float init[2] = {2.0f, -3.0f};
    for (int i = 0; i < 2; i++) {
        CHECK(oe_mem_alloc(dev, 8, &p[i]));
        CHECK(oe_mem_alloc(dev, 8, &g[i]));
        CHECK(oe_mem_alloc(dev, 8, &m[i]));
        CHECK(oe_mem_alloc(dev, 8, &v[i]));
        CHECK(oe_memcpy_h2d(dev, p[i], init, 8, 0));
        CHECK(oe_memset_u32(dev, g[i], 0, 2, 0));
        CHECK(oe_memset_u32(dev, m[i], 0, 2, 0));
        CHECK(oe_memset_u32(dev, v[i], 0, 2, 0));
    }
    oe_tensor_desc t[2];
    memset(t, 0, sizeof t);
    for (int i = 0; i < 2; i++) {
        t[i].param = p[i];
        t[i].grad = g[i];
        t[i].state1 = m[i];
        t[i].state2 = v[i];
        t[i].numel = 2;
        t[i].lr_scale = i == 0 ? 1.0f : 0.5f;
        t[i].weight_decay = 2.0f;
    }
    oe_plan* plan = NULL;
    CHECK(oe_plan_create(dev, t, 2, 0, &plan));
    for (int step = 1; step <= 4; step++) {
        oe_adamw_hparams hp;
        memset(&hp, 0, sizeof hp);
        hp.lr = 0.2f;
        hp.beta1 = 0.9f;
        hp.beta2 = 0.999f;
        hp.eps = 1e-8f;
        hp.bc1 = (float)(1.0 - pow((double)hp.beta1, (double)step));
        hp.bc2 = (float)(1.0 - pow((double)hp.beta2, (double)step));
        CHECK(oe_adamw_step(plan, &hp, 0));
    }
    float out[2][2];
    for (int i = 0; i < 2; i++) CHECK(oe_memcpy_d2h(dev, out[i], p[i], 8, 0));
    CHECK(oe_stream_sync(dev, 0));
    const double factor[2] = {pow(0.6, 4), pow(0.8, 4)};
    for (int i = 0; i < 2; i++)
        for (int j = 0; j < 2; j++) {
            double want = init[j] * factor[i];
            if (fabs(out[i][j] - want) > 2e-6 + 2e-6 * fabs(want)) {
                fprintf(stderr, "decay: p[%d][%d] = %.9g, want %.9g\n", i, j, out[i][j], want);
                return 1;
            }
        }
    /* clip: gradient (3, 4) on the first parameter, none on the second */
    const float grad[2] = {3.0f, 4.0f};
    CHECK(oe_memcpy_h2d(dev, g[0], grad, 8, 0));
    t[1].grad = 0;
    CHECK(oe_plan_update(plan, t, 2, 0));
    const float max_norm = 1.0f;
    CHECK(oe_clip_grad_norm(plan, &max_norm, 0, 0));
    float norm = 0.0f, clipped[2];
    CHECK(oe_read_norm(plan, &norm, NULL, 0));
    CHECK(oe_memcpy_d2h(dev, clipped, g[0], 8, 0));
    CHECK(oe_stream_sync(dev, 0));
    const float coef = 1.0f / (5.0f + 1e-6f);
    if (norm != 5.0f || clipped[0] != 3.0f * coef || clipped[1] != 4.0f * coef) {
        fprintf(stderr, "clip: norm %.9g, gradient (%.9g, %.9g)\n", norm, clipped[0], clipped[1]);
        return 1;
    }
    if (oe_launch_count("oe_adamw_fused") != 4) {
        fprintf(stderr, "expected 4 update launches, counted %lld\n", (long long)oe_launch_count("oe_adamw_fused"));
        return 1;
    }
    CHECK(oe_plan_destroy(plan));
    for (int i = 0; i < 2; i++) {
        CHECK(oe_mem_free(dev, p[i]));
        CHECK(oe_mem_free(dev, g[i]));
        CHECK(oe_mem_free(dev, m[i]));
        CHECK(oe_mem_free(dev, v[i]));
    }
    CHECK(oe_shutdown());
    printf("c_client ok: decay-only AdamW matches 0.6^4 / 0.8^4, clip of (3,4) gives norm 5\n");
    return 0;
}
