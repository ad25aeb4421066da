"""Pins the CPU oracle against every golden vector the reference holds for this path."""
import math

import numpy as np
import pytest

from oracle import oracle
from tests.helpers import assert_close, f32, load_golden

G = load_golden()
VAL = G["tolerances"]["values"]
VTOL = G["tolerances"]["adamw_v"]


@pytest.mark.parametrize("case", G["sgd"], ids=[c["name"] for c in G["sgd"]])
def test_sgd_fixture(case):
    """autograd/sgd_test.go:53-125: 7 configurations x 6 steps, absent and zero gradients, per-step rates."""
    o = case["options"]
    params = [f32(v) for v in case["initial"]]
    opt = oracle.OracleSGD(params, lr=o["LR"], momentum=o["Momentum"], dampening=o["Dampening"],
                           weight_decay=o["WeightDecay"], nesterov=o["Nesterov"], maximize=o["Maximize"])
    for n, step in enumerate(case["steps"]):
        opt.lr = step["lr"]
        opt.step([None if g is None else f32(g) for g in step["gradients"]])
        for i, p in enumerate(params):
            assert_close(f"{case['name']} step {n} value {i}", p, step["values"][i], VAL["atol"], VAL["rtol"])
            want = step["buffers"][i]
            if want is None:
                assert not opt.initialized[i], "momentum initialised without a gradient"
            else:
                assert opt.initialized[i]
                assert_close(f"{case['name']} step {n} buffer {i}", opt.buffers[i], want, VAL["atol"], VAL["rtol"])
    assert opt.step_count == len(case["steps"])


def _groups(case):
    names = [p["name"] for p in case["params"]]
    base = case["groups"][0]["lr"]
    groups = []
    for g in case["groups"]:
        # LRScale = group.lr / groups[0].lr in float32 (autograd/param_groups_test.go:40-52)
        scale = float(np.float32(g["lr"]) / np.float32(base))
        groups.append(oracle.Group(g["name"], [names.index(n) for n in g["params"]], scale, g["weight_decay"]))
    return names, base, groups


def test_param_groups_sgd_fixture():
    """autograd/param_groups_test.go:86-139: momentum .9 + Nesterov, two groups."""
    case = next(c for c in G["param_groups"] if c["kind"] == "sgd")
    names, base, groups = _groups(case)
    params = [f32(p["value"]) for p in case["params"]]
    opt = oracle.OracleSGD(params, lr=base, momentum=0.9, nesterov=True, groups=groups)
    for n, step in enumerate(case["steps"]):
        opt.step([None if g is None else f32(g) for g in step["gradients"]])
        for i, p in enumerate(params):
            assert_close(f"sgd groups step {n} {names[i]}", p, step["values"][i], VAL["atol"], VAL["rtol"])
            if step["buffers"][i] is not None:
                assert_close(f"sgd groups step {n} buffer {names[i]}", opt.buffers[i], step["buffers"][i],
                             VAL["atol"], VAL["rtol"])
            else:
                assert not opt.initialized[i]


def test_param_groups_adamw_fixture():
    """autograd/param_groups_test.go:141-198: defaults beta=(.9,.999), eps 1e-8; v at the tighter bound."""
    case = next(c for c in G["param_groups"] if c["kind"] == "adamw")
    names, base, groups = _groups(case)
    params = [f32(p["value"]) for p in case["params"]]
    opt = oracle.OracleAdamW(params, lr=base, groups=groups)
    for n, step in enumerate(case["steps"]):
        opt.step([None if g is None else f32(g) for g in step["gradients"]])
        for i, p in enumerate(params):
            assert_close(f"adamw groups step {n} {names[i]}", p, step["values"][i], VAL["atol"], VAL["rtol"])
            m, v = step["moments"][i]
            assert_close(f"adamw groups step {n} m {names[i]}", opt.m[i], m, VAL["atol"], VAL["rtol"])
            assert_close(f"adamw groups step {n} v {names[i]}", opt.v[i], v, VTOL["atol"], VTOL["rtol"])


def test_clip_then_adamw_fixture():
    """testdata/nn_conv_step.json: clip_grad_norm_(0.8) then one AdamW(lr .003, wd .01) step, 47 parameters.

    PyTorch clips with max_norm/(norm+1e-6) clamped to 1, the reference CPU path scales only when
    norm > max_norm; both agree here because the fixture's norm exceeds 0.8."""
    c = G["clip_adamw_step"]
    params = [f32(c["parameters"][n]) for n in c["names"]]
    grads = [f32(c["gradients"][n]) for n in c["names"]]
    norm, scale = oracle.clip_grad_norm(grads, c["max_norm"])
    assert norm > c["max_norm"] and scale < 1
    want_norm = math.sqrt(sum(float(x) ** 2 for n in c["names"] for x in c["gradients"][n]))
    assert abs(float(norm) - want_norm) <= 1e-6 * want_norm
    opt = oracle.OracleAdamW(params, lr=c["lr"], weight_decay=c["weight_decay"])
    opt.step(grads)
    for n, p in zip(c["names"], params):
        assert_close(f"clip+adamw {n}", p, c["updated"][n], VAL["atol"], VAL["rtol"])


def test_adamw_kernel_known_answer():
    """kernels/kernels_test.go:117-151: folded clip, norm 1, maxNorm 1 -> coefficient 1/(1+1e-6); 1e-6 abs."""
    p = f32([1, -2, .5, 3])
    g = f32([.1, -.2, .3, -.4])
    m, v = np.zeros(4, np.float32), np.zeros(4, np.float32)
    beta1, beta2, step, bc2, wd, eps, max_norm = .9, .999, .001, .999, .01, 1e-8, 1.0
    oracle.adamw_update_devform(p, g, m, v, 1.0, beta1, beta2, step, bc2, wd, eps, max_norm)
    coefficient = np.float32(min(1.0, max_norm / (1 + 1e-6)))
    for i, (gi, pi) in enumerate(zip([.1, -.2, .3, -.4], [1, -2, .5, 3])):
        grad = np.float32(gi) * coefficient
        mv = np.float32(1 - np.float32(beta1)) * grad
        vv = np.float32(1 - np.float32(beta2)) * grad * grad
        denom = np.float32(math.sqrt(float(vv / np.float32(bc2)))) + np.float32(eps)
        want = np.float32(pi) * np.float32(1 - np.float32(wd)) - np.float32(step) * mv / denom
        assert abs(float(p[i]) - float(want)) <= 1e-6
    # The CPU form with the same coefficient folded in lands within the same bound.
    p2, m2, v2 = f32([1, -2, .5, 3]), np.zeros(4, np.float32), np.zeros(4, np.float32)
    g2 = f32([.1, -.2, .3, -.4])
    oracle.scale_(g2, float(oracle.clip_coefficient(1.0, 1.0, devform=True)))
    # bc1 = 1 so that step/bc1 == step, as the kernel test passes stepSize directly.
    oracle.lib().oracle_adamw_update(oracle._ptr(p2), oracle._ptr(g2), oracle._ptr(m2), oracle._ptr(v2), 4,
                                     beta1, beta2, eps, step, wd, 1.0, bc2)
    assert np.max(np.abs(p2.astype(np.float64) - p.astype(np.float64))) <= 1e-6


def test_decay_only_analytic():
    """autograd/audit_cuda_regression_test.go:66-119: zero grads, wd 2, lr .2 / .1 -> p * .6^4 / .8^4."""
    params = [f32([2, -3]), f32([2, -3])]
    groups = [oracle.Group("fast", [0], 1.0, 2.0), oracle.Group("slow", [1], 0.5, 2.0)]
    opt = oracle.OracleAdamW(params, lr=.2, groups=groups)
    for _ in range(4):
        opt.step([np.zeros(2, np.float32), np.zeros(2, np.float32)])
    for p, base in zip(params, (.6, .8)):
        factor = np.float32(base ** 4)
        assert_close("analytic decay", p, [2 * factor, -3 * factor], 2e-6, 2e-6)


def test_clip_known_answers():
    """autograd/audit_cuda_regression_test.go:121-178: norm of (3,4) is 5; absent grads are not
    counted; maxNorm 0 stores the norm without scaling; all-absent -> 0."""
    g = [f32([3, 4]), None, None]
    norm, scale = oracle.clip_grad_norm(g, 1.0)
    assert abs(float(norm) - 5) <= 1e-5
    assert_close("clipped", g[0], f32([3, 4]) * (np.float32(1) / (np.float32(5) + np.float32(1e-6))), 0, 0)
    g = [f32([3, 4])]
    norm, scale = oracle.clip_grad_norm(g, 0.0)
    assert float(norm) == 5 and float(scale) == 1 and list(g[0]) == [3, 4]
    norm, _ = oracle.clip_grad_norm([None, None], 1.0)
    assert float(norm) == 0
    # CPU rule: norm == max_norm does not scale; the device form multiplies by max/(norm+1e-6) < 1.
    assert float(oracle.clip_coefficient(1.0, 1.0)) == 1.0
    assert float(oracle.clip_coefficient(1.0, 1.0, devform=True)) < 1.0


def test_lr_scale_arithmetic_exact():
    """autograd/param_groups_test.go:458-505: group rate is LR*LRScale in float32; 0 selects 1."""
    assert float(oracle.lib().oracle_normalize_lr_scale(0.0)) == 1.0
    s, d = oracle.C.c_float(), oracle.C.c_float()
    oracle.lib().oracle_adamw_group_scale(0.3, 0.25, 0.1, s, d)
    assert np.float32(s.value) == np.float32(0.3) * np.float32(0.25)
    assert np.float32(d.value) == np.float32(s.value) * np.float32(0.1)
    oracle.lib().oracle_sgd_group_scale(0.3, 0.25, 0.1, s, d)
    assert np.float32(s.value) == np.float32(0.3) * np.float32(0.25) and np.float32(d.value) == np.float32(0.1)


def test_bias_correction_double_pow():
    """autograd/nn.go:493-494."""
    for t in (1, 2, 7, 100, 10000):
        bc1, bc2 = oracle.bias_corrections(0.9, 0.999, t)
        assert bc1 == np.float32(1 - float(np.float32(0.9)) ** t)
        assert bc2 == np.float32(1 - float(np.float32(0.999)) ** t)


def test_bf16_formula_is_rne():
    """autograd/cuda_kernels.go:86: the integer formula equals round-to-nearest-even for every
    non-NaN input; checked against torch's conversion on random bit patterns and edge cases."""
    import torch
    rng = np.random.default_rng(5)
    bits = rng.integers(0, 2 ** 32, size=1 << 20, dtype=np.uint64).astype(np.uint32)
    edge = np.array([0, 0x80000000, 0x7F800000, 0xFF800000, 0x00000001, 0x00008000, 0x00018000, 0x3F808000,
                     0x3F818000, 0x7F7FFFFF, 0x7F7F8000, 0x7F7F7FFF, 0x3F80FFFF, 0x0000FFFF], np.uint32)
    bits = np.concatenate([bits, edge])
    x = bits.view(np.float32)
    finite_or_inf = ~np.isnan(x)
    got = oracle.f32_to_bf16(x, nan_canonical=False)
    want = torch.from_numpy(x.copy()).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got[finite_or_inf], want[finite_or_inf])
    # NaN policy of the engine: quiet NaN carrying the input's sign.
    nan_bits = np.array([0x7FFFFFFF, 0xFFFFFFFF, 0x7FC00000, 0x7F800001, 0xFF800001], np.uint32)
    y = oracle.f32_to_bf16(nan_bits.view(np.float32), nan_canonical=True)
    assert list(y) == [0x7FC0, 0xFFC0, 0x7FC0, 0x7FC0, 0xFFC0]
    # The raw reference formula turns the all-ones NaN into -0: documented divergence.
    assert int(oracle.f32_to_bf16(nan_bits[:1].view(np.float32), nan_canonical=False)[0]) == 0x8000


def test_torch_cross_check_random():
    """Secondary sanity check: the same library family that wrote the fixtures, on larger random
    tensors, over several steps (not the oracle of record)."""
    import torch
    torch.manual_seed(3)
    shapes = [(64, 33), (257,), (5, 7, 3)]
    tp = [torch.nn.Parameter(torch.randn(s) * 0.05) for s in shapes]
    params = [p.detach().numpy().copy().reshape(-1) for p in tp]
    topt = torch.optim.AdamW(tp, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opt = oracle.OracleAdamW(params, lr=1e-3, weight_decay=0.1, beta2=0.95)
    for _ in range(10):
        grads = [torch.randn(s) * 0.01 for s in shapes]
        for p, g in zip(tp, grads):
            p.grad = g.clone()
        topt.step()
        opt.step([g.numpy().reshape(-1).copy() for g in grads])
    for p, q in zip(tp, params):
        assert_close("torch adamw", q, p.detach().numpy(), 5e-7, 3e-5)
    # SGD momentum + nesterov + decay
    tp = [torch.nn.Parameter(torch.randn(s) * 0.05) for s in shapes]
    params = [p.detach().numpy().copy().reshape(-1) for p in tp]
    topt = torch.optim.SGD(tp, lr=0.05, momentum=0.9, weight_decay=5e-4, nesterov=True)
    opt = oracle.OracleSGD(params, lr=0.05, momentum=0.9, weight_decay=5e-4, nesterov=True)
    for _ in range(10):
        grads = [torch.randn(s) * 0.02 for s in shapes]
        for p, g in zip(tp, grads):
            p.grad = g.clone()
        topt.step()
        opt.step([g.numpy().reshape(-1).copy() for g in grads])
    for p, q in zip(tp, params):
        assert_close("torch sgd", q, p.detach().numpy(), 5e-7, 3e-5)


def test_parallel_split_matches_serial():
    """autograd/tensor.go:625-644: the worker split never changes a value."""
    assert oracle.lib().oracle_parallel_workers(65535, 8) == 0
    assert oracle.lib().oracle_parallel_workers(131072, 8) == 2
    assert oracle.lib().oracle_parallel_workers(1 << 20, 8) == 8
    rng = np.random.default_rng(0)
    n = 300_001
    p = rng.normal(0, .02, n).astype(np.float32)
    g = rng.normal(0, .01, n).astype(np.float32)
    a = oracle.OracleAdamW([p.copy()], lr=1e-3, weight_decay=.01, max_procs=1)
    b = oracle.OracleAdamW([p.copy()], lr=1e-3, weight_decay=.01, max_procs=4)
    for _ in range(3):
        a.step([g])
        b.step([g])
    assert np.array_equal(a.params[0], b.params[0]) and np.array_equal(a.m[0], b.m[0])
