"""Parity of the CUDA engine (called through the C ABI) against the CPU oracle.

Tolerances are the ones stated for this path: fp32 p/m/v within 1e-6 relative after one
step and 1e-5 after 100; the gradient norm within 1e-6 relative; the bf16 shadow
bit-exact to round-to-nearest-even of the GPU's own master. Because the kernels keep the
host loop's operation order without fused multiply-adds, the tests also require the
fp32 results to be bit-identical and fail if they ever drift.
"""
import math

import numpy as np
import pytest

from tests.helpers import assert_close, f32, load_golden, ulp_distance

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def eng():
    import gograd_b200 as g
    g.init(0)
    return g


@pytest.fixture(scope="module")
def orc():
    from oracle import oracle
    return oracle


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def rel_close(name, got, want, rtol, scale_atol=0.0):
    """|got-want| <= rtol*|want| + rtol*scale: relative to the element, with an absolute floor
    tied to the tensor's own magnitude for elements near zero."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    floor = rtol * (scale_atol if scale_atol else float(np.max(np.abs(want))) if want.size else 0.0)
    bad = np.abs(got - want) > rtol * np.abs(want) + floor
    assert not bad.any(), f"{name}: {int(bad.sum())} of {got.size} outside {rtol} (worst {np.max(np.abs(got - want)):.3g})"


def bc(beta1, beta2, t):
    from gograd_b200.workload import bias_corrections
    return bias_corrections(beta1, beta2, t)


# --------------------------------------------------------------------------------------
# AdamW on the MLP parameter set: 100 steps, fresh gradients every step
# --------------------------------------------------------------------------------------
def test_mlp_adamw_100_steps(eng, orc):
    from gograd_b200 import paramsets
    ps = paramsets.get("mlp")
    rng = np.random.default_rng(0)
    host_p = []
    for s in ps.params:
        if s.init == "uniform":
            host_p.append(rng.uniform(-s.init_scale, s.init_scale, s.numel).astype(np.float32))
        else:
            host_p.append(np.zeros(s.numel, np.float32))
    hp = ps.hparams
    wd = ps.groups[0].weight_decay
    ref = orc.OracleAdamW([p.copy() for p in host_p], lr=hp["lr"], weight_decay=wd, beta1=hp["beta1"],
                          beta2=hp["beta2"], eps=hp["eps"])
    p = [dev(x) for x in host_p]
    g = [torch.zeros_like(x) for x in p]
    m = [torch.zeros_like(x) for x in p]
    v = [torch.zeros_like(x) for x in p]
    plan = eng.Plan([eng.TensorDesc(p[i], g[i], m[i], v[i], None, 1.0, wd) for i in range(len(p))])
    eng.launch_count_reset()
    grng = np.random.default_rng(ps.grad_seed)
    for t in range(1, ps.steps + 1):
        grads = [grng.normal(0, ps.grad_std, s.numel).astype(np.float32) for s in ps.params]
        for gi, x in zip(g, grads):
            gi.copy_(torch.from_numpy(x))
        b1, b2 = bc(hp["beta1"], hp["beta2"], t)
        plan.adamw_step(eng.AdamWHParams(hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], b1, b2))
        ref.step(grads)
        if t in (1, ps.steps):
            rtol = 1e-6 if t == 1 else 1e-5
            for i in range(len(p)):
                rel_close(f"p[{i}] step {t}", host(p[i]), ref.params[i], rtol)
                rel_close(f"m[{i}] step {t}", host(m[i]), ref.m[i], rtol)
                rel_close(f"v[{i}] step {t}", host(v[i]), ref.v[i], rtol)
    for i in range(len(p)):
        assert ulp_distance(host(p[i]), ref.params[i]).max() == 0, "p not bit-identical to the host loop"
        assert ulp_distance(host(m[i]), ref.m[i]).max() == 0
        assert ulp_distance(host(v[i]), ref.v[i]).max() == 0
    # one launch per step for the whole parameter set
    assert eng.launch_count("oe_adamw_fused") == ps.steps
    assert eng.launch_count() == ps.steps
    plan.close()


# --------------------------------------------------------------------------------------
# SGD on the CNN parameter set: momentum .9, wd 5e-4, 200 steps
# --------------------------------------------------------------------------------------
def test_cnn_sgd_200_steps(eng, orc):
    from gograd_b200 import paramsets
    ps = paramsets.get("cnn")
    rng = np.random.default_rng(11)
    host_p = []
    for s in ps.params:
        if s.init == "uniform":
            host_p.append(rng.uniform(-s.init_scale, s.init_scale, s.numel).astype(np.float32))
        elif s.init == "ones":
            host_p.append(np.ones(s.numel, np.float32))
        else:
            host_p.append(np.zeros(s.numel, np.float32))
    hp = ps.hparams
    wd = ps.groups[0].weight_decay
    ref = orc.OracleSGD([x.copy() for x in host_p], lr=hp["lr"], momentum=hp["momentum"], weight_decay=wd)
    p = [dev(x) for x in host_p]
    g = [torch.zeros_like(x) for x in p]
    buf = [torch.zeros_like(x) for x in p]
    flag = [torch.zeros(1, device="cuda") for _ in p]
    plan = eng.Plan([eng.TensorDesc(p[i], g[i], buf[i], flag[i], None, 1.0, wd) for i in range(len(p))])
    eng.launch_count_reset()
    grng = np.random.default_rng(ps.grad_seed)
    for t in range(1, ps.steps + 1):
        grads = [grng.normal(0, ps.grad_std, s.numel).astype(np.float32) for s in ps.params]
        for gi, x in zip(g, grads):
            gi.copy_(torch.from_numpy(x))
        plan.sgd_step(eng.SGDHParams(hp["lr"], hp["momentum"], hp["dampening"]))
        ref.step(grads)
        if t in (1, 100, ps.steps):
            rtol = 1e-6 if t == 1 else 1e-5
            for i in range(len(p)):
                rel_close(f"p[{i}] step {t}", host(p[i]), ref.params[i], rtol)
                rel_close(f"buffer[{i}] step {t}", host(buf[i]), ref.buffers[i], rtol)
    for i in range(len(p)):
        assert ulp_distance(host(p[i]), ref.params[i]).max() == 0
        assert ulp_distance(host(buf[i]), ref.buffers[i]).max() == 0
        assert float(flag[i].item()) == 1.0
    # one launch per step instead of two per tensor: the update's last CTA also marks the momentum
    # buffers initialised
    assert eng.launch_count("oe_sgd_fused") == ps.steps and eng.launch_count() == ps.steps
    plan.close()


# --------------------------------------------------------------------------------------
# the reference's golden vectors, driven through the C ABI
# --------------------------------------------------------------------------------------
G = load_golden()
VAL = G["tolerances"]["values"]
VTOL = G["tolerances"]["adamw_v"]


@pytest.mark.parametrize("case", G["sgd"], ids=[c["name"] for c in G["sgd"]])
def test_sgd_fixture_on_device(eng, case):
    """autograd/sgd_test.go:53-125 on the device: absent gradients leave the parameter and its
    flag untouched, zero gradients update, the rate changes per step (including 0)."""
    o = case["options"]
    p = [dev(f32(v)) for v in case["initial"]]
    use_mom = o["Momentum"] > 0
    buf = [torch.zeros_like(x) if use_mom else None for x in p]
    flag = [torch.zeros(1, device="cuda") if use_mom else None for x in p]
    gbuf = [torch.zeros_like(x) for x in p]
    flags = (eng.engine.OE_NESTEROV if o["Nesterov"] else 0) | (eng.engine.OE_MAXIMIZE if o["Maximize"] else 0)
    plan = None
    for n, step in enumerate(case["steps"]):
        descs = []
        for i, gr in enumerate(step["gradients"]):
            if gr is not None:
                gbuf[i].copy_(torch.from_numpy(f32(gr)))
            descs.append(eng.TensorDesc(p[i], gbuf[i] if gr is not None else None, buf[i], flag[i], None, 1.0,
                                        o["WeightDecay"]))
        if plan is None:
            plan = eng.Plan(descs)
        else:
            plan.update(descs)
        plan.sgd_step(eng.SGDHParams(step["lr"], o["Momentum"], o["Dampening"], 0.0, flags))
        for i in range(len(p)):
            assert_close(f"{case['name']} step {n} value {i}", host(p[i]), step["values"][i], VAL["atol"], VAL["rtol"])
            want = step["buffers"][i]
            if use_mom:
                assert float(flag[i].item()) == (0.0 if want is None else 1.0)
                if want is not None:
                    assert_close(f"{case['name']} step {n} buffer {i}", host(buf[i]), want, VAL["atol"], VAL["rtol"])
    plan.close()


def _group_case(kind):
    case = next(c for c in G["param_groups"] if c["kind"] == kind)
    names = [q["name"] for q in case["params"]]
    base = case["groups"][0]["lr"]
    per_param = {}
    for grp in case["groups"]:
        for n in grp["params"]:
            per_param[n] = (float(np.float32(grp["lr"]) / np.float32(base)), grp["weight_decay"])
    return case, names, base, per_param


def test_param_groups_adamw_on_device(eng):
    """autograd/param_groups_test.go:141-198."""
    case, names, base, per_param = _group_case("adamw")
    p = [dev(f32(q["value"])) for q in case["params"]]
    g = [torch.zeros_like(x) for x in p]
    m = [torch.zeros_like(x) for x in p]
    v = [torch.zeros_like(x) for x in p]
    plan = eng.Plan([eng.TensorDesc(p[i], g[i], m[i], v[i], None, *per_param[names[i]]) for i in range(len(p))])
    for t, step in enumerate(case["steps"], 1):
        for i, gr in enumerate(step["gradients"]):
            g[i].copy_(torch.from_numpy(f32(gr)))
        b1, b2 = bc(0.9, 0.999, t)
        plan.adamw_step(eng.AdamWHParams(base, 0.9, 0.999, 1e-8, b1, b2))
        for i in range(len(p)):
            assert_close(f"adamw groups step {t} {names[i]}", host(p[i]), step["values"][i], VAL["atol"], VAL["rtol"])
            assert_close(f"m {names[i]}", host(m[i]), step["moments"][i][0], VAL["atol"], VAL["rtol"])
            assert_close(f"v {names[i]}", host(v[i]), step["moments"][i][1], VTOL["atol"], VTOL["rtol"])
    plan.close()


def test_param_groups_sgd_on_device(eng):
    """autograd/param_groups_test.go:86-139: momentum .9 + Nesterov, absent gradients."""
    case, names, base, per_param = _group_case("sgd")
    p = [dev(f32(q["value"])) for q in case["params"]]
    g = [torch.zeros_like(x) for x in p]
    buf = [torch.zeros_like(x) for x in p]
    flag = [torch.zeros(1, device="cuda") for _ in p]
    plan = None
    for t, step in enumerate(case["steps"], 1):
        descs = []
        for i, gr in enumerate(step["gradients"]):
            if gr is not None:
                g[i].copy_(torch.from_numpy(f32(gr)))
            descs.append(eng.TensorDesc(p[i], g[i] if gr is not None else None, buf[i], flag[i], None,
                                        *per_param[names[i]]))
        plan = eng.Plan(descs) if plan is None else (plan.update(descs) or plan)
        plan.sgd_step(eng.SGDHParams(base, 0.9, 0.0, 0.0, eng.engine.OE_NESTEROV))
        for i in range(len(p)):
            assert_close(f"sgd groups step {t} {names[i]}", host(p[i]), step["values"][i], VAL["atol"], VAL["rtol"])
            if step["buffers"][i] is not None:
                assert_close(f"buffer {names[i]}", host(buf[i]), step["buffers"][i], VAL["atol"], VAL["rtol"])
            else:
                assert float(flag[i].item()) == 0.0
    plan.close()


def test_clip_then_adamw_fixture_on_device(eng, orc):
    """testdata/nn_conv_step.json: clip 0.8 then one AdamW step; unfused (in-place clip, then step)
    and fused (norm, then step with the coefficient folded in) must agree bit for bit."""
    c = G["clip_adamw_step"]
    results = []
    for fused in (False, True):
        p = [dev(f32(c["parameters"][n])) for n in c["names"]]
        g = [dev(f32(c["gradients"][n])) for n in c["names"]]
        m = [torch.zeros_like(x) for x in p]
        v = [torch.zeros_like(x) for x in p]
        plan = eng.Plan([eng.TensorDesc(p[i], g[i], m[i], v[i], None, 1.0, c["weight_decay"]) for i in range(len(p))])
        b1, b2 = bc(0.9, 0.999, 1)
        if fused:
            plan.grad_norm()
            plan.adamw_step(eng.AdamWHParams(c["lr"], 0.9, 0.999, 1e-8, b1, b2, max_norm=c["max_norm"]))
        else:
            plan.clip_grad_norm(c["max_norm"])
            plan.adamw_step(eng.AdamWHParams(c["lr"], 0.9, 0.999, 1e-8, b1, b2))
        norm, _ = plan.read_norm()
        want_norm = math.sqrt(sum(float(x) ** 2 for n in c["names"] for x in c["gradients"][n]))
        assert abs(norm - want_norm) <= 1e-6 * want_norm
        for n, x in zip(c["names"], p):
            assert_close(f"clip+adamw {n}", host(x), c["updated"][n], VAL["atol"], VAL["rtol"])
        results.append([host(x).copy() for x in p])
        plan.close()
    for a, b in zip(*results):
        assert np.array_equal(a, b), "folded clip differs from in-place clip + step"


def test_decay_only_analytic_on_device(eng):
    """autograd/audit_cuda_regression_test.go:66-119: present zero gradients, wd 2, lr .2 with
    group scales 1 and .5: p * .6^4 and p * .8^4 after four steps."""
    p = [dev(f32([2, -3])), dev(f32([2, -3]))]
    g = [torch.zeros_like(x) for x in p]
    m = [torch.zeros_like(x) for x in p]
    v = [torch.zeros_like(x) for x in p]
    plan = eng.Plan([eng.TensorDesc(p[0], g[0], m[0], v[0], None, 1.0, 2.0),
                     eng.TensorDesc(p[1], g[1], m[1], v[1], None, 0.5, 2.0)])
    for t in range(1, 5):
        b1, b2 = bc(0.9, 0.999, t)
        plan.adamw_step(eng.AdamWHParams(0.2, 0.9, 0.999, 1e-8, b1, b2))
    for x, base in zip(p, (.6, .8)):
        factor = np.float32(base ** 4)
        assert_close("analytic decay", host(x), [2 * factor, -3 * factor], 2e-6, 2e-6)
    plan.close()


def test_clip_known_answers_on_device(eng):
    """autograd/audit_cuda_regression_test.go:121-178: norm of (3,4) is 5 at 1e-5; absent gradients
    are not counted and not created; max_norm 0 stores the norm without scaling; all absent -> 0."""
    active, unused = dev(f32([1, 2])), dev(f32([7, 8]))
    ga = dev(f32([3, 4]))
    plan = eng.Plan([eng.TensorDesc(active, ga), eng.TensorDesc(unused, None)])
    assert plan.n_active == 1
    plan.clip_grad_norm(1.0)
    norm, sumsq = plan.read_norm()
    assert abs(norm - 5) <= 1e-5 and sumsq == 25.0
    want = f32([3, 4]) * (np.float32(1) / (np.float32(5) + np.float32(1e-6)))
    assert np.array_equal(host(ga), want)
    uploads = plan.uploads
    plan.update([eng.TensorDesc(active, ga), eng.TensorDesc(unused, None)])
    assert plan.uploads == uploads, "unchanged gradients re-uploaded the tables"
    ga.copy_(torch.from_numpy(f32([3, 4])))
    plan.clip_grad_norm(0.0)
    norm, _ = plan.read_norm()
    assert norm == 5.0 and list(host(ga)) == [3, 4]
    gu = dev(f32([0, 12]))
    plan.update([eng.TensorDesc(active, ga), eng.TensorDesc(unused, gu)])
    assert plan.uploads == uploads + 1 and plan.n_active == 2
    plan.grad_norm()
    assert plan.read_norm()[0] == 13.0
    plan.update([eng.TensorDesc(active, None), eng.TensorDesc(unused, None)])
    plan.clip_grad_norm(1.0)
    assert plan.read_norm()[0] == 0.0
    plan.close()


def test_clip_rule_host_vs_devform(eng):
    """norm == max_norm: the host rule leaves gradients alone, the device form scales by
    max/(norm+1e-6) < 1 (autograd/nn.go:327 vs autograd/cuda_kernels.go:676)."""
    for flags, changed in ((0, False), (eng.engine.OE_CLIP_DEVFORM, True)):
        g = dev(f32([0.6, 0.8]))
        plan = eng.Plan([eng.TensorDesc(dev(f32([1, 1])), g)])
        plan.clip_grad_norm(1.0, flags)
        assert plan.read_norm()[0] == 1.0
        got = host(g)
        if changed:
            coef = np.float32(1) / (np.float32(1) + np.float32(1e-6))
            assert np.array_equal(got, f32([0.6, 0.8]) * coef) and got[0] < np.float32(0.6)
        else:
            assert np.array_equal(got, f32([0.6, 0.8]))
        plan.close()


def test_adamw_kernel_known_answer_devform(eng):
    """kernels/kernels_test.go:117-151: norm 1, maxNorm 1, folded coefficient 1/(1+1e-6), 1e-6 abs.
    The norm comes from a real reduction over a gradient whose norm is exactly 1."""
    p = dev(f32([1, -2, .5, 3]))
    g = dev(f32([.1, -.2, .3, -.4]))
    # pad the gradient with a second tensor so that the global norm is exactly 1
    rest = math.sqrt(1.0 - float(np.sum(f32([.1, -.2, .3, -.4]).astype(np.float64) ** 2)))
    pad_p, pad_g = dev(f32([0])), dev(f32([rest]))
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    pm, pv = torch.zeros_like(pad_p), torch.zeros_like(pad_p)
    plan = eng.Plan([eng.TensorDesc(p, g, m, v, None, 1.0, 10.0), eng.TensorDesc(pad_p, pad_g, pm, pv)])
    plan.grad_norm()
    norm, _ = plan.read_norm()
    assert abs(norm - 1.0) <= 1e-6
    # stepSize .001 with bc1 = 1, weightDecay .01 = step * 10
    plan.adamw_step(eng.AdamWHParams(.001, .9, .999, 1e-8, 1.0, .999, max_norm=1.0, flags=eng.engine.OE_CLIP_DEVFORM))
    coefficient = np.float32(min(1.0, 1.0 / (norm + 1e-6)))
    got = host(p)
    for i, (gi, pi) in enumerate(zip([.1, -.2, .3, -.4], [1, -2, .5, 3])):
        grad = np.float32(gi) * coefficient
        mv = np.float32(1 - np.float32(.9)) * grad
        vv = np.float32(1 - np.float32(.999)) * grad * grad
        denom = np.float32(math.sqrt(float(vv / np.float32(.999)))) + np.float32(1e-8)
        want = np.float32(pi) * np.float32(1 - np.float32(.01)) - np.float32(.001) * mv / denom
        assert abs(float(got[i]) - float(want)) <= 1e-6
    plan.close()


# --------------------------------------------------------------------------------------
# ragged sizes, unaligned addresses, guard words
# --------------------------------------------------------------------------------------
SIZES = [1, 2, 3, 4, 5, 31, 255, 256, 257, 1023, 1024, 1025, 4095, 4097, 8191, 8192, 8193, 16385, 70001]


@pytest.mark.parametrize("offset", [0, 1, 2, 3])
def test_ragged_sizes_and_alignment(eng, orc, offset):
    """Every tensor sits `offset` floats past a 16-byte boundary inside a guarded arena:
    offset 0 takes the 128-bit path with scalar tails, the others the scalar path. Guard
    words around every buffer must survive, and all outputs must equal the oracle's."""
    rng = np.random.default_rng(100 + offset)
    guard = np.float32(-777.25)
    guard_bf16 = -21555  # int16 pattern

    def arena(arrays, dtype=np.float32, fill=guard):
        # layout: [guard x 8 + offset][data][guard x 8] per tensor, each start 16-byte aligned + offset
        parts, starts = [], []
        pos = 0
        for a in arrays:
            pad = (-pos) % 8
            pos += pad
            parts.append(np.full(pad + 8 + offset, fill, dtype))
            pos += 8 + offset
            starts.append(pos)
            parts.append(a.astype(dtype))
            pos += a.size
            parts.append(np.full(8, fill, dtype))
            pos += 8
        return np.concatenate(parts), starts

    hp_ = [rng.normal(0, .02, n).astype(np.float32) for n in SIZES]
    hg_ = [rng.normal(0, .01, n).astype(np.float32) for n in SIZES]
    hm_ = [rng.normal(0, .001, n).astype(np.float32) for n in SIZES]
    hv_ = [np.abs(rng.normal(0, 1e-4, n)).astype(np.float32) for n in SIZES]
    flat = {}
    views = {}
    for key, arrs in (("p", hp_), ("g", hg_), ("m", hm_), ("v", hv_)):
        a, starts = arena(arrs)
        flat[key] = dev(a)
        views[key] = [flat[key][s:s + n] for s, n in zip(starts, SIZES)]
        flat[key + "_starts"] = starts
    sh_host, sh_starts = arena([np.zeros(n, np.int16) for n in SIZES], np.int16, guard_bf16)
    # bf16 offset: 2-byte elements; offset floats -> 2*offset shorts keeps 8-byte alignment only for offset 0, 2
    flat["s"] = dev(sh_host)
    views["s"] = [flat["s"][s:s + n] for s, n in zip(sh_starts, SIZES)]
    descs = [eng.TensorDesc(views["p"][i], views["g"][i], views["m"][i], views["v"][i], views["s"][i], 1.0, 0.1)
             for i in range(len(SIZES))]
    plan = eng.Plan(descs)
    assert plan.active_elems == sum(SIZES)
    ref = orc.OracleAdamW([x.copy() for x in hp_], lr=1e-3, weight_decay=0.1, beta2=0.95,
                          m=[x.copy() for x in hm_], v=[x.copy() for x in hv_])
    ref.step_count = 6
    grads = [x.copy() for x in hg_]
    want_norm, scale = orc.clip_grad_norm(grads, 0.05)
    assert scale < 1
    ref.step(grads)
    b1, b2 = bc(0.9, 0.95, 7)
    plan.grad_norm()
    plan.adamw_step(eng.AdamWHParams(1e-3, 0.9, 0.95, 1e-8, b1, b2, max_norm=0.05, flags=eng.engine.OE_WRITE_SHADOW))
    norm, _ = plan.read_norm()
    assert abs(norm - float(want_norm)) <= 1e-6 * float(want_norm)
    assert np.float32(norm) == want_norm, "norm differs from the float64-accumulated host value"
    for i, n in enumerate(SIZES):
        assert np.array_equal(host(views["p"][i]), ref.params[i]), f"p size {n}"
        assert np.array_equal(host(views["m"][i]), ref.m[i]), f"m size {n}"
        assert np.array_equal(host(views["v"][i]), ref.v[i]), f"v size {n}"
        assert np.array_equal(host(views["g"][i]), hg_[i]), "the folded clip must not modify gradients"
        want_sh = orc.f32_to_bf16(ref.params[i]).view(np.int16)
        assert np.array_equal(host(views["s"][i]), want_sh), f"shadow size {n}"
    # guards: everything outside the views is untouched
    for key, fill in (("p", guard), ("g", guard), ("m", guard), ("v", guard)):
        a = host(flat[key]).copy()
        for s, n in zip(flat[key + "_starts"], SIZES):
            a[s:s + n] = fill
        assert np.all(a == fill), f"guard words of {key} overwritten"
    a = host(flat["s"]).copy()
    for s, n in zip(sh_starts, SIZES):
        a[s:s + n] = guard_bf16
    assert np.all(a == guard_bf16), "guard words of the shadow overwritten"
    plan.close()


def test_sgd_ragged_first_and_later_steps(eng, orc):
    """Momentum + dampening + maximize over ragged sizes: the first step seeds the buffer with
    the decayed gradient, later steps blend; checked bit for bit over three steps with clip."""
    rng = np.random.default_rng(7)
    sizes = [1, 3, 4, 5, 257, 8193, 30000]
    hp_ = [rng.normal(0, .05, n).astype(np.float32) for n in sizes]
    p = [dev(x) for x in hp_]
    g = [torch.zeros_like(x) for x in p]
    buf = [torch.zeros_like(x) for x in p]
    flag = [torch.zeros(1, device="cuda") for _ in p]
    shadow = [torch.zeros(n, dtype=torch.int16, device="cuda") for n in sizes]
    plan = eng.Plan([eng.TensorDesc(p[i], g[i], buf[i], flag[i], shadow[i], 1.0, 0.01) for i in range(len(p))])
    ref = orc.OracleSGD([x.copy() for x in hp_], lr=0.05, momentum=0.8, dampening=0.2, weight_decay=0.01,
                        maximize=True)
    for t in range(3):
        grads = [rng.normal(0, .02, n).astype(np.float32) for n in sizes]
        for gi, x in zip(g, grads):
            gi.copy_(torch.from_numpy(x))
        clipped = [x.copy() for x in grads]
        orc.clip_grad_norm(clipped, 0.5)
        ref.step(clipped)
        plan.grad_norm()
        plan.sgd_step(eng.SGDHParams(0.05, 0.8, 0.2, 0.5, eng.engine.OE_MAXIMIZE | eng.engine.OE_WRITE_SHADOW))
        for i in range(len(p)):
            assert np.array_equal(host(p[i]), ref.params[i]), f"step {t} p[{i}]"
            assert np.array_equal(host(buf[i]), ref.buffers[i]), f"step {t} buffer[{i}]"
            assert np.array_equal(host(shadow[i]), orc.f32_to_bf16(ref.params[i]).view(np.int16))
    plan.close()


def test_zero_grad_flag_and_launch(eng):
    rng = np.random.default_rng(3)
    sizes = [5, 4096, 9000]
    p = [dev(rng.normal(0, 1, n).astype(np.float32)) for n in sizes]
    g = [dev(rng.normal(0, 1, n).astype(np.float32)) for n in sizes]
    m = [torch.zeros_like(x) for x in p]
    v = [torch.zeros_like(x) for x in p]
    plan = eng.Plan([eng.TensorDesc(p[i], g[i], m[i], v[i]) for i in range(3)])
    b1, b2 = bc(0.9, 0.999, 1)
    plan.adamw_step(eng.AdamWHParams(1e-3, 0.9, 0.999, 1e-8, b1, b2, flags=eng.engine.OE_ZERO_GRAD))
    assert all(float(x.abs().max()) == 0.0 for x in g)
    assert all(float(x.abs().max()) > 0.0 for x in m)
    for x in g:
        x.fill_(3.0)
    plan.zero_grads()
    assert all(float(x.abs().max()) == 0.0 for x in g)
    plan.close()


# --------------------------------------------------------------------------------------
# bf16 cast: every fp32 bit pattern
# --------------------------------------------------------------------------------------
def test_bf16_cast_all_bit_patterns(eng, orc):
    """All 2^32 inputs in slices: the kernel equals the reference's integer formula
    (autograd/cuda_kernels.go:86) evaluated independently with integer tensor ops for every
    non-NaN input, and sign|0x7fc0 for NaN. A slice is also compared with the C oracle."""
    n = 1 << 26
    base = torch.arange(n, dtype=torch.int64, device="cuda")
    dst = torch.empty(n, dtype=torch.int16, device="cuda")
    for s in range(64):
        src = base + (s << 26)                                     # the bit patterns, as int64
        as_f32 = torch.where(src >= 2 ** 31, src - 2 ** 32, src).to(torch.int32).view(torch.float32)
        eng.cast_bf16(as_f32, dst)
        formula = ((src + 0x7FFF + ((src >> 16) & 1)) >> 16) & 0xFFFF
        is_nan = (src & 0x7FFFFFFF) > 0x7F800000
        formula = torch.where(is_nan, ((src >> 16) & 0x8000) | 0x7FC0, formula)
        got = dst.to(torch.int64) & 0xFFFF
        assert bool((got == formula).all()), f"slice {s}"
        if s in (0, 31, 63):
            sample = as_f32[:: 4099][:4096].contiguous()
            out = torch.empty(sample.numel(), dtype=torch.int16, device="cuda")
            eng.cast_bf16(sample, out)
            assert np.array_equal(host(out).view(np.uint16), orc.f32_to_bf16(host(sample)))


def test_cast_unaligned_and_empty(eng, orc):
    x = dev(np.random.default_rng(1).normal(0, 1, 10007).astype(np.float32))
    out = torch.full((10007 + 16,), -7, dtype=torch.int16, device="cuda")
    for off_src, off_dst, n in ((0, 0, 10007), (1, 0, 9999), (0, 1, 9999), (3, 3, 5), (2, 5, 4097)):
        out.fill_(-7)
        eng.cast_bf16(x[off_src:off_src + n], out[8 + off_dst:8 + off_dst + n])
        got = host(out)
        assert np.array_equal(got[8 + off_dst:8 + off_dst + n].view(np.uint16), orc.f32_to_bf16(host(x[off_src:off_src + n])))
        assert np.all(got[:8 + off_dst] == -7) and np.all(got[8 + off_dst + n:] == -7)
    eng.cast_bf16(x[:0], out[:0])  # empty launch is not an error


# --------------------------------------------------------------------------------------
# error behaviour: reject before any mutation
# --------------------------------------------------------------------------------------
def test_invalid_arguments_change_nothing(eng):
    from gograd_b200.engine import EngineError
    p, g = dev(f32([1, 2, 3])), dev(f32([1, 1, 1]))
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    plan = eng.Plan([eng.TensorDesc(p, g, m, v)])
    before = eng.launch_count()
    bad = [
        eng.AdamWHParams(float("nan"), 0.9, 0.999, 1e-8, .1, .001),
        eng.AdamWHParams(-1.0, 0.9, 0.999, 1e-8, .1, .001),
        eng.AdamWHParams(1e-3, 1.0, 0.999, 1e-8, .1, .001),
        eng.AdamWHParams(1e-3, 0.9, 0.999, 0.0, .1, .001),
        eng.AdamWHParams(1e-3, 0.9, 0.999, 1e-8, 0.0, .001),
        eng.AdamWHParams(1e-3, 0.9, 0.999, 1e-8, .1, .001, flags=0x8000),
    ]
    for hp in bad:
        with pytest.raises(EngineError) as e:
            plan.adamw_step(hp)
        assert e.value.code == -1 and e.value.message
    with pytest.raises(EngineError):
        plan.sgd_step(eng.SGDHParams(0.1, 0.0, 0.0, 0.0, eng.engine.OE_NESTEROV))  # Nesterov needs momentum
    with pytest.raises(EngineError):
        plan.sgd_step(eng.SGDHParams(0.1, 0.9, 0.1, 0.0, eng.engine.OE_NESTEROV))  # ... and zero dampening
    assert eng.launch_count() == before
    assert list(host(p)) == [1, 2, 3] and float(m.abs().max()) == 0
    # AdamW without moments, SGD momentum without buffer/flag
    plan2 = eng.Plan([eng.TensorDesc(p, g)])
    with pytest.raises(EngineError):
        plan2.adamw_step(eng.AdamWHParams(1e-3, 0.9, 0.999, 1e-8, .1, .001))
    with pytest.raises(EngineError):
        plan2.sgd_step(eng.SGDHParams(0.1, 0.9))
    plan2.sgd_step(eng.SGDHParams(0.1))  # plain SGD needs no state
    assert np.allclose(host(p), [0.9, 1.9, 2.9])
    # descriptors: zero numel, misaligned address, bad group values
    with pytest.raises(EngineError):
        eng.Plan([eng.TensorDesc(p[:0], g[:0])])
    with pytest.raises(EngineError):
        eng.Plan([eng.TensorDesc(p, g, weight_decay=-1.0)])
    with pytest.raises(EngineError):
        eng.Plan([eng.TensorDesc(p, g, lr_scale=float("inf"))])
    plan.close()
    plan2.close()


def test_capture_mode_device_step_counter(eng, orc):
    """A device-resident step counter drives the bias correction (AdamW.PrepareGraph,
    autograd/nn.go:350-361): three steps with step_dev equal three eager steps."""
    rng = np.random.default_rng(9)
    n = 5000
    hp0 = rng.normal(0, .02, n).astype(np.float32)
    grads = [rng.normal(0, .01, n).astype(np.float32) for _ in range(3)]
    ref = orc.OracleAdamW([hp0.copy()], lr=1e-3, weight_decay=0.01)
    p, g = dev(hp0), torch.zeros(n, device="cuda")
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    step = torch.zeros(1, dtype=torch.int32, device="cuda")
    plan = eng.Plan([eng.TensorDesc(p, g, m, v, None, 1.0, 0.01)])
    for gr in grads:
        g.copy_(torch.from_numpy(gr))
        plan.adamw_step(eng.AdamWHParams(1e-3, 0.9, 0.999, 1e-8, step_dev=step.data_ptr()))
        ref.step([gr])
    assert int(step.item()) == 3
    rel_close("captured p", host(p), ref.params[0], 1e-6)
    rel_close("captured m", host(m), ref.m[0], 1e-6)
    rel_close("captured v", host(v), ref.v[0], 1e-6)
    plan.close()


def test_device_step_counter_is_advanced_by_the_update_launch_itself(eng, orc):
    """Capture mode costs no launch of its own: the update launch reads the counter, runs step
    counter+1 and its last CTA stores the new value (any grid size, the sharded shape and SGD
    included). Only a plan without a single gradient needs the stand-alone increment."""
    rng = np.random.default_rng(10)
    sizes = [5000, 300_000, 7]          # 1 unit, many units, a ragged tail: several grid sizes
    for chunk in (0, 1024, 8192):
        hp0 = [rng.normal(0, .02, n).astype(np.float32) for n in sizes]
        ref = orc.OracleAdamW([x.copy() for x in hp0], lr=1e-3, weight_decay=0.01)
        p = [dev(x) for x in hp0]
        g = [torch.zeros_like(x) for x in p]
        m = [torch.zeros_like(x) for x in p]
        v = [torch.zeros_like(x) for x in p]
        step = torch.zeros(1, dtype=torch.int32, device="cuda")
        plan = eng.Plan([eng.TensorDesc(p[i], g[i], m[i], v[i], None, 1.0, 0.01) for i in range(3)], 0, chunk)
        eng.launch_count_reset()
        for t in range(1, 6):
            grads = [rng.normal(0, .01, n).astype(np.float32) for n in sizes]
            for gi, x in zip(g, grads):
                gi.copy_(torch.from_numpy(x))
            if t == 4:   # the sharded shape of the kernel, with this GPU as its only rank
                plan.adamw_step_peers(eng.AdamWHParams(1e-3, 0.9, 0.999, 1e-8, step_dev=step.data_ptr()), [0])
            else:
                plan.adamw_step(eng.AdamWHParams(1e-3, 0.9, 0.999, 1e-8, step_dev=step.data_ptr()))
            ref.step(grads)
            assert int(step.item()) == t
        assert eng.launch_count("oe_step_increment") == 0 and eng.launch_count() == 5
        for i in range(3):
            assert np.array_equal(host(p[i]), ref.params[i]) and np.array_equal(host(v[i]), ref.v[i]), f"chunk {chunk} [{i}]"
        # no gradient anywhere: the step still counts
        plan.update([eng.TensorDesc(p[i], None, m[i], v[i], None, 1.0, 0.01) for i in range(3)])
        plan.adamw_step(eng.AdamWHParams(1e-3, 0.9, 0.999, 1e-8, step_dev=step.data_ptr()))
        assert int(step.item()) == 6 and eng.launch_count("oe_step_increment") == 1
        plan.close()
    # SGD: the update launch advances the counter, one launch more only for the momentum flags
    x = dev(np.ones(5000, np.float32))
    gx = torch.full_like(x, 0.5)
    step = torch.zeros(1, dtype=torch.int32, device="cuda")
    plan = eng.Plan([eng.TensorDesc(x, gx, None, None, None, 1.0, 0.0)])
    eng.launch_count_reset()
    for t in range(1, 4):
        plan.sgd_step(eng.SGDHParams(0.1, step_dev=step.data_ptr()))
        assert int(step.item()) == t
    assert eng.launch_count() == 3 and eng.launch_count("oe_sgd_fused") == 3
    assert float(x[0]) == np.float32(1.0) - np.float32(0.05) - np.float32(0.05) - np.float32(0.05)
    plan.close()


def test_default_work_unit_follows_the_size_of_the_parameter_list(eng):
    """Left to the library, the work unit is 4096 elements for sets that stream from HBM and is halved
    (down to 1024) while the list would give fewer than two units per SM; an explicit size is kept."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count

    def unit_for(numels, chunk=0):
        p = [torch.zeros(n, device="cuda") for n in numels]
        plan = eng.Plan([eng.TensorDesc(x, x.clone(), x.clone(), x.clone()) for x in p], 0, chunk)
        unit, units = plan.info(5), plan.info(1)
        plan.close()
        return unit, units

    assert unit_for([10])[0] == 1024
    assert unit_for([784 * 256, 256, 2560, 10]) == (1024, 196 + 1 + 3 + 1)
    unit, units = unit_for([4096 * 2 * sms])            # exactly two 4096-element units per SM
    assert unit == 4096 and units == 2 * sms
    unit, units = unit_for([4096 * 2 * sms - 4096])     # one short: halve once
    assert unit == 2048 and units >= 2 * sms
    assert unit_for([10], 8192)[0] == 8192
    with pytest.raises(eng.engine.EngineError):
        unit_for([10], 1000)


def test_launch_profile_counts_and_times_kernels(eng):
    """The reference's tests assert that a kernel ran through its profile (EnableGPUProfile / GPUProfile,
    autograd/cuda_kernels.go:24-82, autograd/sgd_test.go:119-121): while enabled every launch is timed
    and summed under its kernel name; enabling starts afresh; disabled, only the counts go on."""
    from gograd_b200 import engine
    n = 1 << 22
    p, g = torch.zeros(n, device="cuda"), torch.full((n,), 1e-3, device="cuda")
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    plan = eng.Plan([eng.TensorDesc(p, g, m, v, None, 1.0, 0.1)])
    hp = eng.AdamWHParams(1e-3, 0.9, 0.999, 1e-8, 0.1, 0.001, max_norm=1.0)
    engine.profile_enable(True)
    for _ in range(3):
        plan.grad_norm()
        plan.adamw_step(hp)
    count, ms = engine.profile("oe_adamw_fused")
    assert count == 3 and 0.0 < ms < 50.0
    assert engine.profile("oe_grad_sumsq")[0] == 3 and engine.profile("oe_sgd_fused") == (0, 0.0)
    total_count, total_ms = engine.profile()
    assert total_count == 6 and total_ms >= ms
    engine.profile_enable(False)
    plan.adamw_step(hp)
    assert engine.profile("oe_adamw_fused") == (4, ms), "counts go on, times stop"
    engine.profile_enable(True)
    assert engine.profile() == (0, 0.0)
    engine.profile_enable(False)
    plan.close()


def test_against_the_library_optimizers_as_a_second_opinion(eng):
    """The oracle restates the reference; the fixtures it is pinned to came from PyTorch. As a second
    opinion the engine is compared with torch.optim.AdamW / SGD and clip_grad_norm_ directly (the same
    library family, other operation order, fused multiply-adds allowed): within 2e-6 relative plus a
    floor tied to each tensor's scale after five clipped steps — a tolerance, not the bit-for-bit
    equality the oracle tests require."""
    rng = np.random.default_rng(77)
    sizes = [5000, 33, 4096, 12001]
    w0 = [rng.normal(0, .05, n).astype(np.float32) for n in sizes]
    grads = [[rng.normal(0, .02, n).astype(np.float32) for n in sizes] for _ in range(5)]

    def close(name, got, want):
        got, want = got.astype(np.float64), want.astype(np.float64)
        floor = 2e-6 * float(np.max(np.abs(want)))
        assert np.all(np.abs(got - want) <= 2e-6 * np.abs(want) + floor), name

    # AdamW, decoupled decay, clip 0.5
    tp = [torch.nn.Parameter(torch.from_numpy(x.copy()).cuda()) for x in w0]
    topt = torch.optim.AdamW(tp, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    p = [dev(x) for x in w0]
    g = [torch.zeros_like(x) for x in p]
    m = [torch.zeros_like(x) for x in p]
    v = [torch.zeros_like(x) for x in p]
    plan = eng.Plan([eng.TensorDesc(p[i], g[i], m[i], v[i], None, 1.0, 0.1) for i in range(len(p))])
    for t, gs in enumerate(grads, start=1):
        for i, x in enumerate(gs):
            tp[i].grad = torch.from_numpy(x.copy()).cuda()
            g[i].copy_(torch.from_numpy(x))
        want_norm = float(torch.nn.utils.clip_grad_norm_(tp, 0.5))
        topt.step()
        b1, b2 = bc(0.9, 0.95, t)
        plan.grad_norm()
        plan.adamw_step(eng.AdamWHParams(1e-3, 0.9, 0.95, 1e-8, b1, b2, max_norm=0.5))
        norm, _ = plan.read_norm()
        assert abs(norm - want_norm) <= 1e-6 * want_norm
    for i in range(len(p)):
        close(f"adamw p[{i}]", host(p[i]), tp[i].detach().cpu().numpy())
        close(f"adamw m[{i}]", host(m[i]), topt.state[tp[i]]["exp_avg"].cpu().numpy())
        close(f"adamw v[{i}]", host(v[i]), topt.state[tp[i]]["exp_avg_sq"].cpu().numpy())
    plan.close()

    # SGD, coupled decay, momentum, Nesterov
    tp = [torch.nn.Parameter(torch.from_numpy(x.copy()).cuda()) for x in w0]
    topt = torch.optim.SGD(tp, lr=0.05, momentum=0.9, nesterov=True, weight_decay=0.01)
    p = [dev(x) for x in w0]
    g = [torch.zeros_like(x) for x in p]
    buf = [torch.zeros_like(x) for x in p]
    flag = [torch.zeros(1, device="cuda") for _ in p]
    plan = eng.Plan([eng.TensorDesc(p[i], g[i], buf[i], flag[i], None, 1.0, 0.01) for i in range(len(p))])
    for gs in grads:
        for i, x in enumerate(gs):
            tp[i].grad = torch.from_numpy(x.copy()).cuda()
            g[i].copy_(torch.from_numpy(x))
        topt.step()
        plan.sgd_step(eng.SGDHParams(0.05, 0.9, 0.0, 0.0, eng.engine.OE_NESTEROV))
    for i in range(len(p)):
        close(f"sgd p[{i}]", host(p[i]), tp[i].detach().cpu().numpy())
        close(f"sgd buffer[{i}]", host(buf[i]), topt.state[tp[i]]["momentum_buffer"].cpu().numpy())
    plan.close()
