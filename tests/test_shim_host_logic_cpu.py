"""Host logic of liboptengine.so on the CPU: the library is pointed at a recording stand-in for the
CUDA driver (tests/fake_cuda/fake_cuda.cpp: device memory is host memory, kernels are recorded, not
run, any driver call can be made to fail), and a child process drives the C ABI through table building,
updates, injected driver failures, validation, the sharded step's launch sequence and teardown."""
import json
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    cxx = shutil.which("g++")
    cuda_h = "/usr/local/cuda/include/cuda.h"
    if cxx is None or not os.path.exists(cuda_h):
        pytest.skip("needs g++ and cuda.h to build the stand-in driver")
    lib = tmp_path_factory.mktemp("fake_cuda") / "libcuda_standin.so"
    subprocess.run([cxx, "-std=c++17", "-O1", "-fPIC", "-shared", "-I/usr/local/cuda/include", "-o", str(lib),
                    os.path.join(ROOT, "tests", "fake_cuda", "fake_cuda.cpp")], check=True)
    env = dict(os.environ, OE_CUDA_DRIVER_LIBRARY=str(lib))
    run = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "fake_cuda", "driver_cases.py")], env=env,
                         capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stderr[-2000:]
    return json.loads(run.stdout.strip().splitlines()[-1])


def test_tables_and_launch_shapes(cases):
    # 10,000 elements = 3 units of 4096; 12,289 = 4 units; the parameter without a gradient has no row
    assert cases["tables"] == {"active": 2, "chunks": 7, "elems": 22_289, "uploads": 1}
    names = [x[0] for x in cases["launches"]]
    assert names == ["oe_grad_sumsq", "oe_adamw_fused", "oe_zero_grads"]
    (_, norm_grid, block), (_, update_grid, _), (_, zero_grid, _) = cases["launches"]
    assert block == 256 and norm_grid == 4 and update_grid == 7 and zero_grid == 7   # spans of two units; one CTA per unit


def test_update_uploads_only_on_change(cases):
    assert cases["uploads"] == {"unchanged": 0, "changed": 1, "active": 3}


def test_a_failed_table_growth_never_launches_with_stale_tables(cases):
    """The allocation of a larger table fails (a caller whose arena owns the GPU sees exactly this):
    the update reports it, every launch path then refuses the plan instead of launching with a missing
    table, and the same descriptor list uploads on the next call instead of being taken for unchanged."""
    f = cases["failed_growth"]
    assert f["update"] == 2 and "cuMemAlloc" in f["message"] and "OUT_OF_MEMORY" in f["message"]
    assert f["step"] == -1 and "stale" in f["step_message"] and f["norm"] == -1 and f["zero"] == -1
    assert f["retry"] == 0 and f["active"] == 12
    assert [x[0] for x in f["launches_after_retry"]] == ["oe_adamw_fused"], "nothing launched before the retry"


def test_a_failed_table_copy_is_handled_the_same_way(cases):
    f = cases["failed_copy"]
    assert f["update"] == 719 and f["step"] == -1 and f["launched"] == 0
    assert f["retry"] == 0 and f["step_after"] == 0 and f["active"] == 2


def test_validation_comes_before_any_launch_or_change(cases):
    v = cases["validation"]
    assert v == {"bad_beta": -1, "odd_address": -1, "launched": 0, "uploads_unchanged": True, "still_steps": 0}


def test_sharded_step_is_five_launches_in_order(cases):
    z = cases["zero1"]
    assert z["sequence"] == ["oe_rank_exchange", "oe_peer_reduce_sumsq_n2", "oe_rank_exchange", "oe_adamw_fused_peers",
                             "oe_rank_exchange"]
    assert z["second_create"] == -1 and z["bad_step"] == -1 and z["bad_launched"] == 0 and z["bad_rank"] == -1
    assert z["plan_destroyed_first"] == -1


def test_sharded_step_with_copy_engine_assistance(cases):
    """Rank 1 of 4 (two staged sources, one copied shadow target) and rank 5 of 8 (six and four): the copies run in
    ring order from the next rank on, the kernels keep their places in the sequence, and a request the staging
    cannot hold is refused."""
    for world, rank, pull, push in ((4, 1, 2, 1), (8, 5, 6, 4)):
        z = cases["zero1_copies"][str(world)]
        assert z["too_many"] == -1 and z["odd_staging"] == -1
        assert z["copies"] == pull + push and z["info"] == [pull, push, 0]
        assert z["sequence"] == ["oe_rank_exchange", f"oe_peer_reduce_sumsq_n{world}", "oe_rank_exchange", "oe_adamw_fused_peers",
                                 "oe_rank_exchange"]
        # slot j: this rank's shard as the rank j + 1 places after it holds it
        assert z["staged_from"] == [[(rank + 1 + j) % world, rank] for j in range(pull)] and z["staged_whole"]
        assert z["served_by_copy"] == sorted((rank + 1 + j) % world for j in range(world - 1 - push, world - 1))


def test_sharded_step_with_staging_written_by_the_owners(cases):
    """Rank 5 of 8 knows every rank's staging: it writes its own gradient ranges into slot j of the rank j + 1 places
    after it (never into its own), one more exchange follows the copies, and the form is refused when a peer's
    staging is missing or the shards are not in rank order."""
    z = cases["zero1_copies"]["8 writers"]
    assert z["copies"] == 6 + 4 and z["info"] == [6, 4, 1]
    assert z["sequence"] == ["oe_rank_exchange", "oe_rank_exchange", "oe_peer_reduce_sumsq_n8", "oe_rank_exchange",
                             "oe_adamw_fused_peers", "oe_rank_exchange"]
    # slot j of the rank j + 1 places after rank 5 holds rank 5's gradients for THAT rank's shard
    assert z["staged_from"] == [[5, (5 + 1 + j) % 8] for j in range(6)] and z["staged_whole"] and z["own_staging_untouched"]
    assert z["refused"] == [-1, -1]


def test_the_librarys_own_copy_plan(cases):
    """[staged sources, copied shadow targets] as oe_zero1_create resolves them when the caller leaves the choice."""
    assert cases["zero1_library_choice"] == {
        "8 ranks": [6, 4], "8 ranks, staging for 3": [3, 4], "8 ranks, no staging": [0, 0], "8 ranks, small shard": [0, 4],
        "4 ranks": [2, 0], "2 ranks": [0, 0], "1 rank": [0, 0]}


def test_sharded_update_launch_shape_follows_the_rank_count(cases):
    """400 work units on a 148-SM device whose kernels fit two CTAs per SM: the persistent grid is 296 CTAs; with
    four ranks the library launches one CTA per SM (the measured optimum there); an explicit knob wins."""
    assert cases["peer_shapes"] == {"2": 296, "4": 148, "8": 296, "4 with the grid knob at 100": 100, "bad knob": -1}


def test_teardown_and_architecture_check(cases):
    t = cases["teardown"]
    assert t["shutdown_with_live_plans"] == -1 and t["shutdown"] == 0 and t["leaked_allocations"] == 0
    assert cases["arch"]["rc"] == -4 and "sm_90" in cases["arch"]["message"]
