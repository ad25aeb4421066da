"""Host-logic cases of liboptengine.so run against the recording stand-in driver (child process of
tests/test_shim_host_logic_cpu.py; prints one JSON object). No GPU, no arithmetic."""
import ctypes as C
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from gograd_b200 import _lib  # noqa: E402

fake = C.CDLL(os.environ["OE_CUDA_DRIVER_LIBRARY"])
fake.fake_cuda_calls.restype = C.c_long
fake.fake_cuda_calls.argtypes = [C.c_char_p]
fake.fake_cuda_fail.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int]
fake.fake_cuda_live_allocations.restype = C.c_long
lib = _lib.lib()
out = {}


def launches():
    rec = []
    name, grid, block = C.create_string_buffer(64), C.c_uint(), C.c_uint()
    i = 0
    while fake.fake_cuda_launch(i, name, 64, C.byref(grid), C.byref(block)):
        rec.append((name.value.decode(), grid.value, block.value))
        i += 1
    return rec


def err():
    return lib.oe_last_error().decode()


class Buffers:
    """"Device" buffers from the stand-in's allocator (host memory), kept alive for the run."""

    def __init__(self):
        self.addresses = []

    def alloc(self, nbytes):
        a = C.c_uint64()
        assert lib.oe_mem_alloc(0, nbytes, C.byref(a)) == 0, err()
        self.addresses.append(a.value)
        return a.value


assert lib.oe_init(0) == 0, err()
assert lib.oe_device_sm_count(0) == 148
buf = Buffers()


def desc(numel, with_grad=True, wd=0.1, misalign=0):
    p, g, m, v, sh = (buf.alloc(4 * numel + 64) for _ in range(5))
    return _lib.oe_tensor_desc(p, (g + misalign) if with_grad else 0, m, v, sh, numel, 1.0, wd)


def descs(*items):
    arr = (_lib.oe_tensor_desc * len(items))(*items)
    return arr, len(items)


hp = _lib.oe_adamw_hparams(1e-3, 0.9, 0.999, 1e-8, 0.1, 0.001, 1.0, _lib.OE_WRITE_SHADOW, 0, 0)

# ---- 1. tables: one row per tensor with a gradient, one work unit per chunk_elems elements ---------
a, b, c = desc(10_000), desc(5, with_grad=False), desc(4096 * 3 + 1, misalign=4)
arr, n = descs(a, b, c)
plan = C.c_void_p()
assert lib.oe_plan_create(0, arr, n, 4096, C.byref(plan)) == 0, err()
out["tables"] = {"active": lib.oe_plan_info(plan, 0), "chunks": lib.oe_plan_info(plan, 1),
                 "elems": lib.oe_plan_info(plan, 2), "uploads": lib.oe_plan_info(plan, 6)}
fake.fake_cuda_reset_launches()
assert lib.oe_grad_norm(plan, 0, 0) == 0, err()
assert lib.oe_adamw_step(plan, C.byref(hp), 0) == 0, err()
assert lib.oe_zero_grads(plan, 0) == 0, err()
out["launches"] = launches()

# ---- 2. an unchanged list uploads nothing; a changed one uploads once --------------------------------
before = lib.oe_plan_info(plan, 6)
assert lib.oe_plan_update(plan, arr, n, 0) == 0
same = lib.oe_plan_info(plan, 6) - before
b2 = desc(5)                       # the second parameter now has a gradient
arr2, _ = descs(a, b2, c)
assert lib.oe_plan_update(plan, arr2, n, 0) == 0, err()
out["uploads"] = {"unchanged": same, "changed": lib.oe_plan_info(plan, 6) - before, "active": lib.oe_plan_info(plan, 0)}

# ---- 3. a failed table growth: nothing launches until an update succeeds -----------------------------
big = [desc(4096 * 40) for _ in range(12)]   # needs more rows and more work units than the tables hold
arr3, n3 = descs(*big)
fake.fake_cuda_fail(b"cuMemAlloc", 0, 2, 0)   # the next device allocation reports out of memory
rc_update = lib.oe_plan_update(plan, arr3, n3, 0)
message = err()
fake.fake_cuda_reset_launches()
rc_step = lib.oe_adamw_step(plan, C.byref(hp), 0)
step_message = err()
rc_norm = lib.oe_grad_norm(plan, 0, 0)
rc_zero = lib.oe_zero_grads(plan, 0)
rc_same = lib.oe_plan_update(plan, arr3, n3, 0)           # the same list again: must upload, not return early
assert lib.oe_adamw_step(plan, C.byref(hp), 0) == 0, err()
out["failed_growth"] = {"update": rc_update, "message": message, "step": rc_step, "step_message": step_message,
                        "norm": rc_norm, "zero": rc_zero, "retry": rc_same, "launches_after_retry": launches(),
                        "active": lib.oe_plan_info(plan, 0)}

# ---- 4. a failed copy of the tables (the allocation succeeded): same rule ------------------------------
arr4, n4 = descs(a, c)
fake.fake_cuda_fail(b"cuMemcpyHtoDAsync", 0, 719, 0)
rc_update = lib.oe_plan_update(plan, arr4, n4, 0)
fake.fake_cuda_reset_launches()
rc_step = lib.oe_adamw_step(plan, C.byref(hp), 0)
launched = len(launches())
rc_retry = lib.oe_plan_update(plan, arr4, n4, 0)
rc_step2 = lib.oe_adamw_step(plan, C.byref(hp), 0)
out["failed_copy"] = {"update": rc_update, "step": rc_step, "launched": launched, "retry": rc_retry, "step_after": rc_step2,
                      "active": lib.oe_plan_info(plan, 0)}

# ---- 5. validation happens before anything is launched or changed -----------------------------------
fake.fake_cuda_reset_launches()
bad = _lib.oe_adamw_hparams(1e-3, 1.5, 0.999, 1e-8, 0.1, 0.001, 1.0, 0, 0, 0)
rc_bad = lib.oe_adamw_step(plan, C.byref(bad), 0)
odd = _lib.oe_tensor_desc(buf.alloc(64) + 2, 0, 0, 0, 0, 4, 1.0, 0.0)
arr5, _ = descs(odd)
uploads = lib.oe_plan_info(plan, 6)
rc_odd = lib.oe_plan_update(plan, arr5, 1, 0)
out["validation"] = {"bad_beta": rc_bad, "odd_address": rc_odd, "launched": len(launches()),
                     "uploads_unchanged": lib.oe_plan_info(plan, 6) == uploads, "still_steps": lib.oe_adamw_step(plan, C.byref(hp), 0)}

# ---- 6. the sharded step driven through the library alone: five launches in order ---------------------
z = C.c_void_p()
d = _lib.oe_zero1_desc()
d.rank, d.world, d.first_elem, d.numel = 1, 2, 4096, 4096
grads = [buf.alloc(4 * 8192), buf.alloc(4 * 8192)]
shadow = [buf.alloc(2 * 8192), buf.alloc(2 * 8192)]
sync = [buf.alloc(512), buf.alloc(512)]
for k in range(2):
    d.grad_bases[k], d.sync_blocks[k] = grads[k], sync[k]
    d.shadow_deltas[k] = shadow[k] - shadow[1]
shard = _lib.oe_tensor_desc(buf.alloc(4 * 4096), grads[1] + 4 * 4096, buf.alloc(4 * 4096), buf.alloc(4 * 4096),
                            shadow[1] + 2 * 4096, 4096, 1.0, 0.1)
arr6, _ = descs(shard)
plan2 = C.c_void_p()
assert lib.oe_plan_create(0, arr6, 1, 0, C.byref(plan2)) == 0, err()
assert lib.oe_zero1_create(plan2, C.byref(d), C.byref(z)) == 0, err()
twice = lib.oe_zero1_create(plan2, C.byref(d), C.byref(C.c_void_p()))
fake.fake_cuda_reset_launches()
assert lib.oe_zero1_adamw_step(z, C.byref(hp), 0) == 0, err()
seq = [x[0] for x in launches()]
fake.fake_cuda_reset_launches()
rc_bad_step = lib.oe_zero1_adamw_step(z, C.byref(bad), 0)   # refused before the first launch of the step
bad_launched = len(launches())
d_bad = _lib.oe_zero1_desc.from_buffer_copy(d)
d_bad.rank = 2
rc_rank = lib.oe_zero1_create(plan2, C.byref(d_bad), C.byref(C.c_void_p()))
rc_plan_first = lib.oe_plan_destroy(plan2)                  # refused while the sharded step is bound to it
assert lib.oe_zero1_destroy(z) == 0
out["zero1"] = {"plan_destroyed_first": rc_plan_first, "sequence": seq, "second_create": twice, "bad_step": rc_bad_step, "bad_launched": bad_launched,
                "bad_rank": rc_rank}

# ---- 6b. launch shape of the sharded update: the library's choice by the number of ranks, and the knobs ----
wide = desc(4096 * 400)
arr7, _ = descs(wide)
plan3 = C.c_void_p()
assert lib.oe_plan_create(0, arr7, 1, 4096, C.byref(plan3)) == 0, err()
shapes = {}
for ranks in (2, 4, 8):
    deltas = (C.c_int64 * ranks)(*([0] * ranks))
    fake.fake_cuda_reset_launches()
    assert lib.oe_adamw_step_peers(plan3, C.byref(hp), deltas, ranks, 0) == 0, err()
    shapes[str(ranks)] = launches()[0][1]
assert lib.oe_plan_set_tuning(plan3, 2, 100) == 0          # OE_TUNE_PEER_UPDATE_GRID
deltas = (C.c_int64 * 4)(0, 0, 0, 0)
fake.fake_cuda_reset_launches()
assert lib.oe_adamw_step_peers(plan3, C.byref(hp), deltas, 4, 0) == 0, err()
shapes["4 with the grid knob at 100"] = launches()[0][1]
shapes["bad knob"] = lib.oe_plan_set_tuning(plan3, 4, 3)   # warp rotation takes 0, 1 or 2
assert lib.oe_plan_destroy(plan3) == 0
out["peer_shapes"] = shapes

# ---- 6c. copy-engine assistance of the sharded step: which copies are issued, from where to where ---------
def copy_plan_case(W, R, pull, push, SH=4096, writers=False):
    """Rank R of W with `pull` staged sources and `push` copied shadow targets, asked for explicitly; with
    `writers` every rank's staging is known and the staged ranges are written by their owners."""
    g = [buf.alloc(4 * SH * W) for _ in range(W)]
    s_ = [buf.alloc(2 * SH * W) for _ in range(W)]
    y = [buf.alloc(512) for _ in range(W)]
    stages = [buf.alloc(pull * 4 * SH) for _ in range(W)]
    stage = stages[R]
    for k in range(W):                                        # rank k's gradient bytes read 16 k + t inside shard t
        for t in range(W):
            C.memset(g[k] + 4 * SH * t, 16 * k + t, 4 * SH)
        C.memset(stages[k], 0xff, pull * 4 * SH)
        C.memset(s_[k], 0, 2 * SH * W)
    C.memset(s_[R] + 2 * SH * R, 0x5a, 2 * SH)                # "this rank's updated shadow values" (no kernel runs here)
    d = _lib.oe_zero1_desc()
    d.rank, d.world, d.first_elem, d.numel = R, W, SH * R, SH
    for k in range(W):
        d.grad_bases[k], d.sync_blocks[k], d.shadow_deltas[k] = g[k], y[k], s_[k] - s_[R]
    d.staging, d.staging_bytes, d.ce_pull_sources, d.ce_push_targets = stage, pull * 4 * SH, pull, push
    if writers:
        for k in range(W):
            d.staging_bases[k] = stages[k]
    own = _lib.oe_tensor_desc(buf.alloc(4 * SH), g[R] + 4 * SH * R, buf.alloc(4 * SH), buf.alloc(4 * SH), s_[R] + 2 * SH * R, SH, 1.0, 0.1)
    arr, _ = descs(own)
    plan = C.c_void_p()
    assert lib.oe_plan_create(0, arr, 1, 0, C.byref(plan)) == 0, err()
    too_many = _lib.oe_zero1_desc.from_buffer_copy(d)
    too_many.ce_pull_sources = pull + 1
    rc_too_many = lib.oe_zero1_create(plan, C.byref(too_many), C.byref(C.c_void_p()))
    odd = _lib.oe_zero1_desc.from_buffer_copy(d)
    odd.staging = stage + 4
    rc_odd = lib.oe_zero1_create(plan, C.byref(odd), C.byref(C.c_void_p()))
    z = C.c_void_p()
    assert lib.oe_zero1_create(plan, C.byref(d), C.byref(z)) == 0, err()
    before = fake.fake_cuda_calls(b"cuMemcpyAsync")
    fake.fake_cuda_reset_launches()
    assert lib.oe_zero1_adamw_step(z, C.byref(hp), 0) == 0, err()
    seq = launches()
    if writers:   # slot j of the rank j + 1 places after this one holds this rank's gradient bytes; its own staging is untouched
        staged = [C.string_at(stages[(R + 1 + j) % W] + j * 4 * SH, 4 * SH) for j in range(pull)]
        untouched = C.string_at(stage, pull * 4 * SH) == b"\xff" * (pull * 4 * SH)
    else:
        staged = [C.string_at(stage + j * 4 * SH, 4 * SH) for j in range(pull)]
    served = {k: C.string_at(s_[k] + 2 * SH * R, 2 * SH) == b"\x5a" * (2 * SH) for k in range(W)}
    result = {"too_many": rc_too_many, "odd_staging": rc_odd, "copies": fake.fake_cuda_calls(b"cuMemcpyAsync") - before,
              "sequence": [x[0] for x in seq], "info": [lib.oe_zero1_info(z, 0), lib.oe_zero1_info(z, 1), lib.oe_zero1_info(z, 3)],
              # (rank the bytes come from, shard they were taken from) per slot, and that each slot holds one whole range
              "staged_from": [[x[0] // 16, x[0] % 16] for x in staged], "staged_whole": all(x == bytes([x[0]]) * (4 * SH) for x in staged),
              # the kernel would serve this rank and the next ones; the copies serve the last `push` ranks of the ring
              "served_by_copy": sorted(k for k, ok in served.items() if ok and k != R)}
    if writers:
        result["own_staging_untouched"] = untouched
    assert lib.oe_zero1_destroy(z) == 0
    if writers:   # the owners' form needs every peer's staging and equal shards in rank order
        partial = _lib.oe_zero1_desc.from_buffer_copy(d)
        partial.staging_bases[(R + 1) % W] = 0
        shifted = _lib.oe_zero1_desc.from_buffer_copy(d)
        shifted.first_elem += 4
        result["refused"] = [lib.oe_zero1_create(plan, C.byref(partial), C.byref(C.c_void_p())),
                             lib.oe_zero1_create(plan, C.byref(shifted), C.byref(C.c_void_p()))]
    assert lib.oe_plan_destroy(plan) == 0
    return result


out["zero1_copies"] = {"4": copy_plan_case(4, 1, 2, 1), "8": copy_plan_case(8, 5, 6, 4),
                       "8 writers": copy_plan_case(8, 5, 6, 4, writers=True)}

# the library's own choice by world size, shard size and the staging it was given (contexts made, never stepped)
def library_choice(W, numel, staging_slots):
    d = _lib.oe_zero1_desc()
    d.rank, d.world, d.first_elem, d.numel = 0, W, 0, numel
    for k in range(W):
        d.grad_bases[k], d.sync_blocks[k], d.shadow_deltas[k] = 0x10000000 * (k + 1), 0x1000 * (k + 1), 0x40000000 * k
    d.staging, d.staging_bytes = (0x7000000000, staging_slots * 4 * numel) if staging_slots else (0, 0)
    plan = C.c_void_p()
    arr, _ = descs(desc(4096))
    assert lib.oe_plan_create(0, arr, 1, 0, C.byref(plan)) == 0, err()
    z = C.c_void_p()
    assert lib.oe_zero1_create(plan, C.byref(d), C.byref(z)) == 0, err()
    got = [lib.oe_zero1_info(z, 0), lib.oe_zero1_info(z, 1)]
    assert lib.oe_zero1_destroy(z) == 0 and lib.oe_plan_destroy(plan) == 0
    return got


BIG, SMALL = 1 << 26, 1 << 20     # 256 MiB and 4 MiB of gradients per shard
out["zero1_library_choice"] = {
    "8 ranks": library_choice(8, BIG, 7), "8 ranks, staging for 3": library_choice(8, BIG, 3),
    "8 ranks, no staging": library_choice(8, BIG, 0), "8 ranks, small shard": library_choice(8, SMALL, 7),
    "4 ranks": library_choice(4, BIG, 3), "2 ranks": library_choice(2, BIG, 1), "1 rank": library_choice(1, BIG, 0)}

# ---- 7. shutdown refuses while plans live; everything the library allocated is returned -------------------
rc_shutdown_live = lib.oe_shutdown()
assert lib.oe_plan_destroy(plan) == 0 and lib.oe_plan_destroy(plan2) == 0
for addr in buf.addresses:
    assert lib.oe_mem_free(0, addr) == 0
out["teardown"] = {"shutdown_with_live_plans": rc_shutdown_live, "shutdown": lib.oe_shutdown(),
                   "leaked_allocations": fake.fake_cuda_live_allocations()}

# ---- 8. another architecture is refused ----------------------------------------------------------------------
fake.fake_cuda_set_device(9, 0, 132)
out["arch"] = {"rc": lib.oe_init(1), "message": err()}
print(json.dumps(out))
