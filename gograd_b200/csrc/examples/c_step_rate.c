/*
 * What one eager optimizer step costs when it is issued from C, without an interpreter in between:
 * the 2-layer MLP parameter set (784x256 + 256 + 256x10 + 10 = 203,530 fp32 parameters, AdamW),
 * one oe_adamw_step per step, bias corrections computed on the host as AdamW.Step does
 * (autograd/nn.go:493-494). Prints the host's issue time per step and the time per step with the
 * device drained at the end.
 *
 *   cc -std=gnu11 c_step_rate.c -I../../../include -L../.. -loptengine -Wl,-rpath,../.. -lm -o c_step_rate
 */
#include <math.h>
#include <stdio.h>
#include <string.h>
#include <time.h>

#include "optengine.h"

#define CHECK(call)                                                          \
    do {                                                                     \
        int rc_ = (call);                                                    \
        if (rc_ != 0) {                                                      \
            fprintf(stderr, "%s failed (%d): %s\n", #call, rc_, oe_last_error()); \
            return 1;                                                        \
        }                                                                    \
    } while (0)

static double now_us(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec * 1e6 + ts.tv_nsec * 1e-3;
}

int main(void) {
    const int dev = 0;
    const uint64_t numel[4] = {784 * 256, 256, 256 * 10, 10};
    CHECK(oe_init(dev));
    oe_tensor_desc t[4];
    memset(t, 0, sizeof t);
    for (int i = 0; i < 4; i++) {
        uint64_t* slot[4] = {&t[i].param, &t[i].grad, &t[i].state1, &t[i].state2};
        for (int k = 0; k < 4; k++) {
            CHECK(oe_mem_alloc(dev, numel[i] * 4, slot[k]));
            /* p = 0.5 (bit pattern), g = 2^-10, m = v = 0 */
            uint32_t fill = k == 0 ? 0x3f000000u : k == 1 ? 0x3a800000u : 0u;
            CHECK(oe_memset_u32(dev, *slot[k], fill, numel[i], 0));
        }
        t[i].numel = numel[i];
        t[i].lr_scale = 1.0f;
        t[i].weight_decay = 0.01f;
    }
    oe_plan* plan = NULL;
    CHECK(oe_plan_create(dev, t, 4, 0, &plan));
    oe_adamw_hparams hp;
    memset(&hp, 0, sizeof hp);
    hp.lr = 1e-3f;
    hp.beta1 = 0.9f;
    hp.beta2 = 0.999f;
    hp.eps = 1e-8f;
    const int warmup = 200, steps = 5000;
    int step = 0;
    double t0 = 0, t_issued = 0, t_done = 0;
    for (int k = 0; k < warmup + steps; k++) {
        if (k == warmup) {
            CHECK(oe_stream_sync(dev, 0));
            t0 = now_us();
        }
        step++;
        hp.bc1 = (float)(1.0 - pow((double)hp.beta1, (double)step));
        hp.bc2 = (float)(1.0 - pow((double)hp.beta2, (double)step));
        CHECK(oe_adamw_step(plan, &hp, 0));
    }
    t_issued = now_us();
    CHECK(oe_stream_sync(dev, 0));
    t_done = now_us();
    float first = 0.0f;
    CHECK(oe_memcpy_d2h(dev, &first, t[0].param, 4, 0));
    CHECK(oe_stream_sync(dev, 0));
    if (!(first < 0.5f) || !isfinite(first)) {
        fprintf(stderr, "the parameters did not move as expected: p[0] = %.9g\n", first);
        return 1;
    }
    if (oe_launch_count(NULL) != warmup + steps) {
        fprintf(stderr, "expected one launch per step, counted %lld\n", (long long)oe_launch_count(NULL));
        return 1;
    }
    printf("c_step_rate ok: %d eager AdamW steps over 203530 parameters, host issue %.2f us/step, "
           "with the device drained %.2f us/step\n",
           steps, (t_issued - t0) / steps, (t_done - t0) / steps);
    CHECK(oe_plan_destroy(plan));
    for (int i = 0; i < 4; i++) {
        CHECK(oe_mem_free(dev, t[i].param));
        CHECK(oe_mem_free(dev, t[i].grad));
        CHECK(oe_mem_free(dev, t[i].state1));
        CHECK(oe_mem_free(dev, t[i].state2));
    }
    CHECK(oe_shutdown());
    return 0;
}
