/*
 * A plain-C host drives the sharded (ZeRO-1 style) AdamW step on every GPU of the box from ONE
 * process and ONE thread, with no collective library and no Python: what gograd's Go host would do
 * (one device per OS thread, no collectives anywhere in the repository). Per rank it allocates a flat
 * gradient buffer, a flat bf16 shadow buffer, its shard of master weights and moments and a 512-byte
 * exchange area through the library, lets the devices address one another's memory, and then issues
 * ONE call per rank and step: oe_zero1_adamw_step. The calls only enqueue work; rank 0's first
 * exchange kernel waits (bounded) on its GPU until rank 1's step has been enqueued on the next GPU a
 * few microseconds later. With a single GPU the world has one rank and the exchanges meet themselves.
 * Run as "c_zero1 copies" it asks for the copy-assisted form of the step and issues each rank's call
 * from a thread of its own (see the comment at the call).
 *
 * The result is checked on the host against the same arithmetic written out in C: the mean of the
 * ranks' gradients added in ascending rank order, the global norm from a float64 sum, the clip
 * coefficient of the host rule, AdamW in the operation order of autograd/nn.go:519-528, and the bf16
 * shadow as round-to-nearest-even of the master — bit for bit, on every rank.
 *
 *   cc -std=c11 -ffp-contract=off c_zero1.c -I../../../include -L../.. -loptengine -Wl,-rpath,../.. -lm -lpthread -o c_zero1 && ./c_zero1
 */
#include <math.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
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

#define MAX_RANKS 8
#define SHARD 12288u /* elements per rank: three work units */
#define STEPS 3

static float grad_value(int rank, int step, uint32_t i) {
    /* any deterministic pattern with mixed signs and magnitudes */
    uint32_t h = (uint32_t)(i * 2654435761u) ^ (uint32_t)(rank * 40503u + step * 9973u);
    h ^= h >> 13;
    h *= 2246822519u;
    h ^= h >> 16;
    return ((float)(h & 0xffff) - 32768.0f) * (1.0f / 32768.0f) * 1e-3f;
}

static uint16_t bf16_rne(float x) {
    uint32_t bits;
    memcpy(&bits, &x, 4);
    return (uint16_t)((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
}

/* One rank's step call, for the mode that gives every rank a host thread of its own. */
typedef struct rank_call {
    oe_zero1* z;
    const oe_adamw_hparams* hp;
    uint64_t stream;
    int rc;
} rank_call;

static void* rank_step(void* arg) {
    rank_call* c = (rank_call*)arg;
    c->rc = oe_zero1_adamw_step(c->z, c->hp, c->stream);
    return NULL;
}

int main(int argc, char** argv) {
    /* "copies": ask for the copy-assisted form of the step (all peers' gradient ranges but one staged by copies,
     * the last rank of the ring served by a shadow copy), which the library would not choose for shards this small */
    const int copies = argc > 1 && strcmp(argv[1], "copies") == 0;
    int devices = 0;
    CHECK(oe_device_count(&devices));
    int world = devices > MAX_RANKS ? MAX_RANKS : devices;
    if (world < 1) {
        fprintf(stderr, "no CUDA device\n");
        return 1;
    }
    const uint32_t total = SHARD * (uint32_t)world;
    const float lr = 3e-4f, beta1 = 0.9f, beta2 = 0.95f, eps = 1e-8f, decay = 0.1f, max_norm = 0.01f;
    uint64_t grad[MAX_RANKS], shadow[MAX_RANKS], master[MAX_RANKS], m[MAX_RANKS], v[MAX_RANKS], sync[MAX_RANKS];
    uint64_t staging[MAX_RANKS], stream[MAX_RANKS];
    const uint32_t staged = (copies && world > 1) ? (uint32_t)(world > 2 ? world - 2 : 1) : 0;
    oe_plan* plan[MAX_RANKS];
    oe_zero1* z[MAX_RANKS];
    float* host = (float*)malloc(sizeof(float) * total);
    float* ref_p = (float*)malloc(sizeof(float) * total);
    float* ref_m = (float*)calloc(total, sizeof(float));
    float* ref_v = (float*)calloc(total, sizeof(float));
    float* mean = (float*)malloc(sizeof(float) * total);
    if (!host || !ref_p || !ref_m || !ref_v || !mean) return 1;
    for (uint32_t i = 0; i < total; i++) ref_p[i] = 0.02f * (float)((int)(i % 201) - 100) * 0.01f;

    for (int r = 0; r < world; r++) CHECK(oe_init(r));
    for (int r = 0; r < world; r++)
        for (int q = 0; q < world; q++) CHECK(oe_enable_peer_access(r, q));
    for (int r = 0; r < world; r++) {
        CHECK(oe_mem_alloc(r, 4ull * total, &grad[r]));
        CHECK(oe_mem_alloc(r, 2ull * total, &shadow[r]));
        CHECK(oe_mem_alloc(r, 4ull * SHARD, &master[r]));
        CHECK(oe_mem_alloc(r, 4ull * SHARD, &m[r]));
        CHECK(oe_mem_alloc(r, 4ull * SHARD, &v[r]));
        CHECK(oe_mem_alloc(r, OE_ZERO1_SYNC_BYTES, &sync[r]));
        staging[r] = 0;
        stream[r] = 0; /* the device's default stream, unless the step uses copies (below) */
        if (staged) {
            CHECK(oe_mem_alloc(r, 4ull * SHARD * staged, &staging[r]));
            CHECK(oe_stream_create(r, &stream[r]));
        }
        CHECK(oe_memset_u32(r, shadow[r], 0, total / 2, 0));
        CHECK(oe_memset_u32(r, m[r], 0, SHARD, 0));
        CHECK(oe_memset_u32(r, v[r], 0, SHARD, 0));
        CHECK(oe_memset_u32(r, sync[r], 0, OE_ZERO1_SYNC_BYTES / 4, 0));
        CHECK(oe_memcpy_h2d(r, master[r], ref_p + (size_t)r * SHARD, 4ull * SHARD, 0));
        CHECK(oe_stream_sync(r, 0));
    }
    for (int r = 0; r < world; r++) {
        oe_tensor_desc t;
        memset(&t, 0, sizeof t);
        t.param = master[r];
        t.grad = grad[r] + 4ull * r * SHARD; /* the owner's range of its own gradient buffer */
        t.state1 = m[r];
        t.state2 = v[r];
        t.shadow = shadow[r] + 2ull * r * SHARD;
        t.numel = SHARD;
        t.lr_scale = 1.0f;
        t.weight_decay = decay;
        CHECK(oe_plan_create(r, &t, 1, 0, &plan[r]));
        oe_zero1_desc d;
        memset(&d, 0, sizeof d);
        d.rank = (uint32_t)r;
        d.world = (uint32_t)world;
        d.first_elem = (uint64_t)r * SHARD;
        d.numel = SHARD;
        for (int q = 0; q < world; q++) {
            d.grad_bases[q] = grad[q];
            d.shadow_deltas[q] = (int64_t)(shadow[q] - shadow[r]);
            d.sync_blocks[q] = sync[q];
        }
        d.timeout_ms = 10000;
        if (staged) {
            d.staging = staging[r];
            d.staging_bytes = 4ull * SHARD * staged; /* 4 * SHARD is a multiple of 256: one slot per staged peer */
            d.ce_pull_sources = staged;
            d.ce_push_targets = 1;
        } else {
            d.ce_pull_sources = d.ce_push_targets = OE_ZERO1_CE_NONE;
        }
        CHECK(oe_zero1_create(plan[r], &d, &z[r]));
        if (oe_zero1_info(z[r], 0) != (int64_t)staged || oe_zero1_info(z[r], 1) != (staged ? 1 : 0)) {
            fprintf(stderr, "rank %d: the context did not take the requested copy plan\n", r);
            return 1;
        }
    }

    for (int step = 1; step <= STEPS; step++) {
        for (int r = 0; r < world; r++) {
            for (uint32_t i = 0; i < total; i++) host[i] = grad_value(r, step, i);
            CHECK(oe_memcpy_h2d(r, grad[r], host, 4ull * total, 0));
        }
        for (int r = 0; r < world; r++) CHECK(oe_stream_sync(r, 0));
        oe_adamw_hparams hp;
        memset(&hp, 0, sizeof hp);
        hp.lr = lr;
        hp.beta1 = beta1;
        hp.beta2 = beta2;
        hp.eps = eps;
        hp.bc1 = (float)(1.0 - pow((double)beta1, (double)step));
        hp.bc2 = (float)(1.0 - pow((double)beta2, (double)step));
        hp.max_norm = max_norm;
        hp.flags = OE_WRITE_SHADOW;
        if (!copies) {
            for (int r = 0; r < world; r++) CHECK(oe_zero1_adamw_step(z[r], &hp, 0)); /* enqueue only */
        } else {
            /* A copy between two devices of ONE process is work for both devices: it may keep the host in the
             * call until the work queued before it has run, and on a device's default stream it is ordered after
             * that device's own step, which waits for the other rank. So here each rank's call comes from a thread
             * of its own, as gograd pins one OS thread per device, on a stream created for it. (Ranks in
             * processes of their own, the usual case, need nothing of the kind.) */
            pthread_t th[MAX_RANKS];
            rank_call call[MAX_RANKS];
            for (int r = 0; r < world; r++) {
                call[r].z = z[r];
                call[r].hp = &hp;
                call[r].stream = stream[r];
                call[r].rc = -1;
                if (pthread_create(&th[r], NULL, rank_step, &call[r]) != 0) return 1;
            }
            for (int r = 0; r < world; r++) pthread_join(th[r], NULL);
            for (int r = 0; r < world; r++)
                if (call[r].rc != 0) {
                    fprintf(stderr, "rank %d: oe_zero1_adamw_step failed (%d): %s\n", r, call[r].rc, oe_last_error());
                    return 1;
                }
        }
        for (int r = 0; r < world; r++) {
            uint32_t status = 0;
            CHECK(oe_zero1_status(z[r], &status, stream[r]));
        }
        /* the same step on the host */
        double sumsq = 0.0;
        const float inv = (float)(1.0 / (double)world);
        for (uint32_t i = 0; i < total; i++) {
            float s = grad_value(0, step, i);
            for (int r = 1; r < world; r++) s = s + grad_value(r, step, i);
            mean[i] = s * inv;
            sumsq += (double)mean[i] * (double)mean[i];
        }
        const float norm = (float)sqrt(sumsq);
        const float coef = norm > max_norm ? max_norm / (norm + 1e-6f) : 1.0f;
        const float step_size = lr * 1.0f, omd = 1.0f - step_size * decay;
        const float omb1 = 1.0f - beta1, omb2 = 1.0f - beta2;
        for (uint32_t i = 0; i < total; i++) {
            float g = mean[i] * coef;
            float mi = beta1 * ref_m[i] + omb1 * g;
            float t2 = omb2 * g;
            float vi = beta2 * ref_v[i] + t2 * g;
            ref_m[i] = mi;
            ref_v[i] = vi;
            float root = (float)sqrt((double)(vi / hp.bc2));
            float upd = step_size * (mi / hp.bc1);
            ref_p[i] = ref_p[i] * omd - upd / (root + eps);
        }
        float got_norm = 0.0f;
        CHECK(oe_read_norm(plan[0], &got_norm, NULL, 0));
        if (fabsf(got_norm - norm) > 1e-6f * norm) {
            fprintf(stderr, "step %d: norm %.9g, host %.9g\n", step, got_norm, norm);
            return 1;
        }
    }
    /* every rank's master shard and every rank's whole shadow */
    uint16_t* sh = (uint16_t*)malloc(2ull * total);
    if (!sh) return 1;
    for (int r = 0; r < world; r++) {
        CHECK(oe_memcpy_d2h(r, host, master[r], 4ull * SHARD, 0));
        CHECK(oe_memcpy_d2h(r, sh, shadow[r], 2ull * total, 0));
        CHECK(oe_stream_sync(r, 0));
        if (memcmp(host, ref_p + (size_t)r * SHARD, 4ull * SHARD) != 0) {
            fprintf(stderr, "rank %d: master weights differ from the host loop\n", r);
            return 1;
        }
        for (uint32_t i = 0; i < total; i++)
            if (sh[i] != bf16_rne(ref_p[i])) {
                fprintf(stderr, "rank %d: shadow[%u] = %04x, want %04x\n", r, i, sh[i], bf16_rne(ref_p[i]));
                return 1;
            }
    }
    const long long exchanges = (long long)oe_launch_count("oe_rank_exchange");
    if (exchanges != 3LL * STEPS * world) {
        fprintf(stderr, "expected %d exchange launches, counted %lld\n", 3 * STEPS * world, exchanges);
        return 1;
    }
    for (int r = 0; r < world; r++) {
        CHECK(oe_zero1_destroy(z[r]));
        CHECK(oe_plan_destroy(plan[r]));
        CHECK(oe_mem_free(r, grad[r]));
        CHECK(oe_mem_free(r, shadow[r]));
        CHECK(oe_mem_free(r, master[r]));
        CHECK(oe_mem_free(r, m[r]));
        CHECK(oe_mem_free(r, v[r]));
        CHECK(oe_mem_free(r, sync[r]));
        if (staging[r]) CHECK(oe_mem_free(r, staging[r]));
        if (stream[r]) CHECK(oe_stream_destroy(r, stream[r]));
    }
    CHECK(oe_shutdown());
    printf("c_zero1 ok: %d rank(s), %d sharded AdamW steps driven from C, master weights and every rank's bf16 shadow equal the host loop bit for bit\n",
           world, STEPS);
    free(sh);
    free(host);
    free(ref_p);
    free(ref_m);
    free(ref_v);
    free(mean);
    return 0;
}
