"""The host mirror of gograd's optimizer API (C++ over the C ABI), driven the way the reference's
own tests drive `AdamW`, `SGD`, `ClipGradNorm` and the checkpoints."""
import json
import math
import struct

import numpy as np
import pytest

from tests.helpers import assert_close, f32, load_golden

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

G = load_golden()
VAL = G["tolerances"]["values"]
VTOL = G["tolerances"]["adamw_v"]


@pytest.fixture(scope="module")
def ag():
    from gograd_b200 import autograd
    autograd.lib()
    return autograd


def params_of(ag, named):
    return [ag.Parameter(n, ag.Tensor(v)) for n, v in named]


@pytest.mark.parametrize("case", G["sgd"], ids=[c["name"] for c in G["sgd"]])
def test_sgd_matches_pytorch_fixture_and_resumes(ag, case, tmp_path):
    """autograd/sgd_test.go:53-125: values and buffers per step, lazy initialisation flags, and a
    safetensors round trip in the middle that must resume bit for bit."""
    o = case["options"]
    params = params_of(ag, [("weight", case["initial"][0]), ("bias", case["initial"][1])])
    opt = ag.NewSGD(params, ag.SGDOptions(o["LR"], o["Momentum"], o["Dampening"], o["WeightDecay"], o["Nesterov"], o["Maximize"]))
    twin_params = twin = None
    for n, step in enumerate(case["steps"]):
        for runner, ps in ((opt, params), (twin, twin_params)):
            if runner is None:
                continue
            runner.SetLearningRate(step["lr"])
            for p, g in zip(ps, step["gradients"]):
                p.Value.set_grad(None if g is None else f32(g))
            runner.Step()
        for i, p in enumerate(params):
            assert_close(f"{case['name']} step {n} value {i}", p.Value.to_host(), step["values"][i], VAL["atol"], VAL["rtol"])
            buf, init = (opt.Buffer(i) if o["Momentum"] > 0 else (None, False))
            want = step["buffers"][i]
            assert init == (want is not None)
            if want is not None:
                assert_close(f"{case['name']} step {n} buffer {i}", buf, want, VAL["atol"], VAL["rtol"])
            if twin is not None:
                assert np.array_equal(twin_params[i].Value.to_host(), p.Value.to_host()), "resumed run diverged"
        assert opt.StepCount == n + 1
        if n == 2:  # save, load into a fresh optimizer over copies of the parameters, run both on
            path = str(tmp_path / "sgd.safetensors")
            opt.SaveSafeTensors(path)
            twin_params = params_of(ag, [(p.Name, p.Value.to_host()) for p in params])
            twin = ag.NewSGD(twin_params, ag.SGDOptions(LR=9.0, Momentum=o["Momentum"]))  # config comes from the file
            twin.LoadSafeTensors(path)
            assert twin.StepCount == 3 and twin.LearningRate() == np.float32(step["lr"])
            d = ag.safetensors_describe(path)
            assert d["metadata"]["format"] == "gograd-sgd" and d["metadata"]["step_count"] == "3"
            cfg = json.loads(d["metadata"]["optimizer"])
            assert list(cfg) == ["StepCount", "Names", "Shapes", "Options", "Initialized", "Buffers", "Groups"]
            assert cfg["Names"] == ["weight", "bias"] and cfg["Buffers"] is None
            want_entries = [f"buffer.{i}" for i, b in enumerate(step["buffers"]) if b is not None]
            assert sorted(d["entries"]) == want_entries
    # eager ZeroGrad makes gradients absent (set-to-none), autograd/sgd.go:231-246
    opt.ZeroGrad()
    assert not any(p.Value.has_grad for p in params)
    opt.Close()
    opt.Close()  # idempotent
    with pytest.raises(ag.HostError, match="closed"):
        opt.Step()


def _group_case(ag, kind):
    case = next(c for c in G["param_groups"] if c["kind"] == kind)
    params = params_of(ag, [(q["name"], q["value"]) for q in case["params"]])
    by_name = {p.Name: p for p in params}
    base = case["groups"][0]["lr"]
    specs = [ag.ParameterGroupSpec(g["name"], [by_name[n] for n in g["params"]],
                                   float(np.float32(g["lr"]) / np.float32(base)), g["weight_decay"]) for g in case["groups"]]
    return case, params, base, specs


def test_adamw_groups_match_pytorch_fixture(ag, tmp_path):
    """autograd/param_groups_test.go:141-198 plus the grouped state round trip of :288-359."""
    case, params, base, specs = _group_case(ag, "adamw")
    opt = ag.NewAdamWGroups(params, base, specs)
    for t, step in enumerate(case["steps"], 1):
        for p, g in zip(params, step["gradients"]):
            p.Value.set_grad(f32(g))
        opt.Step()
        for i, p in enumerate(params):
            assert_close(f"step {t} {p.Name}", p.Value.to_host(), step["values"][i], VAL["atol"], VAL["rtol"])
            assert_close(f"m {p.Name}", opt.M(i), step["moments"][i][0], VAL["atol"], VAL["rtol"])
            assert_close(f"v {p.Name}", opt.V(i), step["moments"][i][1], VTOL["atol"], VTOL["rtol"])
    # exact group arithmetic (autograd/param_groups_test.go:458-505): step = LR*LRScale, decay = step*wd in float32
    step_size, decay = opt.groupScale(2)
    assert step_size == np.float32(base) * np.float32(0.5) and decay == step_size * np.float32(0)
    step_size, decay = opt.groupScale(0)
    assert step_size == np.float32(base) and decay == np.float32(base) * np.float32(0.02)
    path = str(tmp_path / "adamw.safetensors")
    opt.SaveSafeTensors(path)
    d = ag.safetensors_describe(path)
    assert sorted(d["entries"]) == sorted([f"m.{i}" for i in range(3)] + [f"v.{i}" for i in range(3)])
    cfg = json.loads(d["metadata"]["optimizer"])
    assert list(cfg) == ["StepCount", "Moments", "Names", "Shapes", "LR", "WeightDecay", "Beta1", "Beta2", "Eps", "Groups"]
    assert cfg["Moments"] is None and cfg["StepCount"] == 3 and d["metadata"]["format"] == "gograd-adamw"
    assert [g["Name"] for g in cfg["Groups"]] == ["decay", "no_decay"] and cfg["Groups"][0]["Names"] == ["weight", "bias"]
    assert np.float32(cfg["Beta2"]) == np.float32(0.999) and np.float32(cfg["Eps"]) == np.float32(1e-8)
    # a second optimizer with the same groups resumes bit for bit
    case2, params2, _, specs2 = _group_case(ag, "adamw")
    for p2, p in zip(params2, params):
        p2.Value.copy_from_host(p.Value.to_host())
    opt2 = ag.NewAdamWGroups(params2, 123.0, specs2)
    opt2.LoadSafeTensors(path)
    assert opt2.StepCount == 3 and opt2.LearningRate() == np.float32(base)
    for o_, ps in ((opt, params), (opt2, params2)):
        for p in ps:
            p.Value.set_grad(f32([.25, -.5]))
        o_.Step()
    for p, p2 in zip(params, params2):
        assert np.array_equal(p.Value.to_host(), p2.Value.to_host())
    # a state saved with other groups is rejected before anything changes
    flat = ag.NewAdamW(params_of(ag, [(q["name"], q["value"]) for q in case["params"]]), base, 0.0)
    before = flat.StepCount
    with pytest.raises(ag.HostError, match="parameter groups"):
        flat.LoadSafeTensors(path)
    assert flat.StepCount == before


def test_sgd_groups_match_pytorch_fixture(ag):
    """autograd/param_groups_test.go:86-139: momentum .9 + Nesterov with absent gradients."""
    case, params, base, specs = _group_case(ag, "sgd")
    opt = ag.NewSGDGroups(params, ag.SGDOptions(LR=base, Momentum=0.9, Nesterov=True), specs)
    for t, step in enumerate(case["steps"], 1):
        for p, g in zip(params, step["gradients"]):
            p.Value.set_grad(None if g is None else f32(g))
        opt.Step()
        for i, p in enumerate(params):
            assert_close(f"step {t} {p.Name}", p.Value.to_host(), step["values"][i], VAL["atol"], VAL["rtol"])
            buf, init = opt.Buffer(i)
            assert init == (step["buffers"][i] is not None)
            if init:
                assert_close(f"buffer {p.Name}", buf, step["buffers"][i], VAL["atol"], VAL["rtol"])


def test_constructor_and_group_validation(ag):
    """autograd/nn.go:407-436, autograd/sgd.go:21-31,47-96, autograd/param_groups.go:104-171: every
    rejected configuration names its reason and builds nothing."""
    a, b = ag.Tensor([1, 2]), ag.Tensor([3])
    pa, pb = ag.Parameter("a", a), ag.Parameter("b", b)
    with pytest.raises(ag.HostError, match="distinct named"):
        ag.NewAdamW([pa, ag.Parameter("a", b)], 0.1, 0)
    with pytest.raises(ag.HostError, match="distinct named"):
        ag.NewAdamW([ag.Parameter("", a)], 0.1, 0)
    with pytest.raises(ag.HostError, match="parameter values"):
        ag.NewAdamW([ag.Parameter("x", None)], 0.1, 0)
    for bad in (-1.0, float("nan"), float("inf")):
        with pytest.raises(ag.HostError, match="invalid learning rate"):
            ag.NewAdamW([pa], bad, 0)
    with pytest.raises(ag.HostError, match="weight decay"):
        ag.NewAdamW([pa], 0.1, -0.5)
    with pytest.raises(ag.HostError, match="at least one parameter group"):
        ag.NewAdamWGroups([pa], 0.1, [])
    with pytest.raises(ag.HostError, match="not in any group"):
        ag.NewAdamWGroups([pa, pb], 0.1, [ag.ParameterGroupSpec("g", [pa])])
    with pytest.raises(ag.HostError, match="appears in groups"):
        ag.NewAdamWGroups([pa, pb], 0.1, [ag.ParameterGroupSpec("g", [pa, pb]), ag.ParameterGroupSpec("h", [pa])])
    with pytest.raises(ag.HostError, match="duplicate parameter group"):
        ag.NewAdamWGroups([pa, pb], 0.1, [ag.ParameterGroupSpec("g", [pa]), ag.ParameterGroupSpec("g", [pb])])
    with pytest.raises(ag.HostError, match="has no name"):
        ag.NewAdamWGroups([pa], 0.1, [ag.ParameterGroupSpec("", [pa])])
    with pytest.raises(ag.HostError, match="has no parameters"):
        ag.NewAdamWGroups([pa], 0.1, [ag.ParameterGroupSpec("g", [pa]), ag.ParameterGroupSpec("h", [])])
    with pytest.raises(ag.HostError, match="not part of this optimizer"):
        ag.NewAdamWGroups([pa], 0.1, [ag.ParameterGroupSpec("g", [pa, ag.Parameter("z", ag.Tensor([0]))])])
    with pytest.raises(ag.HostError, match="learning-rate scale"):
        ag.NewAdamWGroups([pa], 0.1, [ag.ParameterGroupSpec("g", [pa], LRScale=-1)])
    # LRScale 0 selects the unscaled base rate
    o = ag.NewAdamWGroups([pa], 0.25, [ag.ParameterGroupSpec("g", [pa], LRScale=0, WeightDecay=0.5)])
    assert o.groupScale(0) == (np.float32(0.25), np.float32(0.125))
    with pytest.raises(ag.HostError, match="Nesterov"):
        ag.NewSGD([pa], ag.SGDOptions(LR=0.1, Nesterov=True))
    with pytest.raises(ag.HostError, match="Nesterov"):
        ag.NewSGD([pa], ag.SGDOptions(LR=0.1, Momentum=0.9, Dampening=0.1, Nesterov=True))
    with pytest.raises(ag.HostError, match="invalid SGD configuration"):
        ag.NewSGD([pa], ag.SGDOptions(LR=-0.1))
    with pytest.raises(ag.HostError, match="parameter groups, not SGDOptions"):
        ag.NewSGDGroups([pa], ag.SGDOptions(LR=0.1, WeightDecay=0.1), [ag.ParameterGroupSpec("g", [pa])])
    with pytest.raises(ag.HostError, match="distinct"):
        ag.NewSGD([pa, ag.Parameter("again", a)], ag.SGDOptions(LR=0.1))  # same storage twice
    with pytest.raises(ag.HostError, match="invalid learning rate"):
        o.SetLearningRate(float("nan"))


def test_clip_grad_norm_absent_gradients(ag):
    """autograd/audit_cuda_regression_test.go:121-178."""
    active, unused, frozen = ag.Tensor([1, 2]), ag.Tensor([7, 8]), ag.Tensor([9, 10], requires_grad=False)
    params = [ag.Parameter("active", active), ag.Parameter("unused", unused), ag.Parameter("frozen", frozen)]
    active.set_grad([3, 4])
    opt = ag.NewSGD(params, ag.SGDOptions(LR=.1, Momentum=.9, WeightDecay=.5))
    assert math.isnan(ag.ClipGradNorm(params, 1))  # the norm stays on the device
    assert not unused.has_grad and not frozen.has_grad, "clipping created an absent gradient"
    assert abs(ag.GradientNormToHost() - 5) <= 1e-5
    coef = np.float32(1) / (np.float32(5) + np.float32(1e-6))
    assert np.array_equal(active.grad_to_host(), f32([3, 4]) * coef)
    ag.ClipGradNorm(params, 0)  # stores the norm of the already clipped gradient, scales nothing
    assert abs(ag.GradientNormToHost() - 1) <= 1e-6
    opt.Step()
    for i in (1, 2):
        buf, init = opt.Buffer(i)
        assert not init, "clipping initialised unused SGD momentum"
    assert list(unused.to_host()) == [7, 8] and list(frozen.to_host()) == [9, 10]
    unused.ensure_grad()
    active.set_grad([3, 4])
    ag.ClipGradNorm(params, 0)
    assert ag.GradientNormToHost() == 5.0  # the new zero gradient is observed and adds nothing
    unused.set_grad(None)
    ag.ClipGradNorm(params[1:], 1)
    assert ag.GradientNormToHost() == 0.0, "all-absent gradient norm"
    ag.ReleaseClipState()


def test_step_clipped_equals_clip_then_step_and_installs_shadow(ag):
    """Folded clip == ClipGradNorm + Step bit for bit; with WriteShadow the step leaves a current
    bf16 shadow (the seam of autograd/cuda_autocast.go:30-60) that a later write invalidates."""
    rng = np.random.default_rng(5)
    values = [rng.normal(0, .05, n).astype(np.float32) for n in (1000, 7, 4096)]
    grads = [rng.normal(0, .5, n).astype(np.float32) for n in (1000, 7, 4096)]
    runs = []
    for fused in (False, True):
        params = params_of(ag, [(f"p{i}", v) for i, v in enumerate(values)])
        opt = ag.NewAdamW(params, 1e-2, 0.1)
        opt.SetConfig(beta2=0.95)
        opt.SetEngine(write_shadow=True)
        for step in range(3):
            for p, g in zip(params, grads):
                p.Value.set_grad(g * np.float32(step + 1))
            if fused:
                opt.StepClipped(1.0)
                norm = opt.LastGradNorm()
            else:
                ag.ClipGradNorm(params, 1.0)
                norm = ag.GradientNormToHost()
                opt.Step()
            want = math.sqrt(sum(float(np.sum((g.astype(np.float64) * (step + 1)) ** 2)) for g in grads))
            assert abs(norm - want) <= 1e-6 * want
        runs.append([p.Value.to_host() for p in params])
        for p in params:
            assert p.Value.shadow_current
            want = torch.from_numpy(p.Value.to_host()).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
            assert np.array_equal(p.Value.shadow_to_host(), want)
        params[0].Value.copy_from_host(values[0])
        assert not params[0].Value.shadow_current, "a write through the tensor must invalidate its shadow"
    for a, b in zip(*runs):
        assert np.array_equal(a, b)
    ag.ReleaseClipState()


def test_captured_step_counter_matches_eager(ag):
    """autograd/audit_cuda_regression_test.go:66-119: present zero gradients, decay 2, rates .2/.1: after
    one eager and three captured steps p = p0 * .6^4 / .8^4, and the device counter reads 4."""
    def make():
        params = params_of(ag, [("fast", [2, -3]), ("slow", [2, -3])])
        for p in params:
            p.Value.ensure_grad()
        return params, ag.NewAdamWGroups(params, .2, [ag.ParameterGroupSpec("fast", params[:1], 1, 2),
                                                      ag.ParameterGroupSpec("slow", params[1:], .5, 2)])
    (cp, captured), (ep, eager) = make(), make()
    captured.Step()
    eager.Step()
    captured.PrepareGraph()
    for _ in range(3):
        captured.StepCaptured()
        eager.Step()
    assert captured.GraphStepCount() == 4
    for i, (p, q) in enumerate(zip(cp, ep)):
        assert_close("captured/eager decay", p.Value.to_host(), q.Value.to_host(), 2e-6, 2e-6)
        factor = np.float32([.6, .8][i] ** 4)
        assert_close("analytic decay", p.Value.to_host(), [2 * factor, -3 * factor], 2e-6, 2e-6)
    captured.Step()  # back to eager: the host counter is synchronised from the device first
    assert captured.StepCount == 5


def test_training_checkpoint_round_trip_and_rejection(ag, tmp_path):
    """autograd/training_checkpoint_test.go:15-141: model + optimizer + schedule + caller metadata in
    one file; a resumed run continues bit for bit; a bad file changes nothing."""
    rng = np.random.default_rng(8)
    shapes = {"layer.weight": (4, 3), "layer.bias": (4,), "bn.running_mean": (4,)}
    init = {k: rng.normal(0, .1, int(np.prod(s))).astype(np.float32) for k, s in shapes.items()}

    def build():
        tensors = {k: ag.Tensor(init[k], shapes[k]) for k in shapes}
        model = [ag.Parameter(k, t) for k, t in tensors.items()]
        trainable = model[:2]
        opt = ag.NewAdamW(trainable, 1e-3, 0.01)
        sched = ag.OneCycle(0.01, 10, 0.3)
        return model, trainable, opt, sched

    def train(model, trainable, opt, sched, steps, seed):
        r = np.random.default_rng(seed)
        for _ in range(steps):
            for p in trainable:
                p.Value.set_grad(r.normal(0, .1, p.Value.numel).astype(np.float32))
            opt.Step()
            sched.Step(opt)

    model, trainable, opt, sched = build()
    train(model, trainable, opt, sched, 3, 1)
    path = str(tmp_path / "train.safetensors")
    ag.SaveTrainingCheckpoint(path, model, opt, sched, {"epoch": "2", "note": "a<b & c"})
    d = ag.safetensors_describe(path)
    assert d["metadata"]["format"] == "gograd-training-1" and d["metadata"]["optimizer_kind"] == "adamw"
    assert sorted(d["entries"]) == sorted([f"model.{k}" for k in shapes] + ["optimizer.m.0", "optimizer.m.1",
                                                                            "optimizer.v.0", "optimizer.v.1"])
    assert d["entries"]["model.layer.weight"]["shape"] == [4, 3]
    sch = json.loads(d["metadata"]["scheduler"])
    assert list(sch) == ["MaxLR", "PctStart", "DivFactor", "FinalDivFactor", "Total", "StepCount"] and sch["StepCount"] == 3
    assert json.loads(d["metadata"]["user"]) == {"epoch": "2", "note": "a<b & c"}
    model2, trainable2, opt2, sched2 = build()
    user = ag.LoadTrainingCheckpoint(path, model2, opt2, sched2)
    assert user == {"epoch": "2", "note": "a<b & c"}
    assert opt2.StepCount == 3 and sched2.fields() == sched.fields() and opt2.LearningRate() == opt.LearningRate()
    train(model, trainable, opt, sched, 2, 2)
    train(model2, trainable2, opt2, sched2, 2, 2)
    for p, q in zip(model, model2):
        assert np.array_equal(p.Value.to_host(), q.Value.to_host()), p.Name
    for i in range(2):
        assert np.array_equal(opt.M(i), opt2.M(i)) and np.array_equal(opt.V(i), opt2.V(i))
    # saving refuses a schedule that is out of step with the optimizer
    sched.StepCount += 1
    with pytest.raises(ag.HostError, match="step mismatch"):
        ag.SaveTrainingCheckpoint(str(tmp_path / "bad.safetensors"), model, opt, sched, {})
    sched.StepCount -= 1
    # a file with a negative second moment is rejected before the model or the optimizer changes
    raw = bytearray(open(path, "rb").read())
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    a, _ = header["optimizer.v.0"]["data_offsets"]
    raw[8 + hlen + a:8 + hlen + a + 4] = struct.pack("<f", -1.0)
    bad = tmp_path / "negative_v.safetensors"
    bad.write_bytes(bytes(raw))
    model3, trainable3, opt3, sched3 = build()
    with pytest.raises(ag.HostError, match="invalid optimizer moment"):
        ag.LoadTrainingCheckpoint(str(bad), model3, opt3, sched3)
    assert opt3.StepCount == 0 and sched3.StepCount == 0
    for k, p in zip(shapes, model3):
        assert np.array_equal(p.Value.to_host(), init[k])
    # an SGD optimizer refuses an AdamW checkpoint
    sgd = ag.NewSGD(trainable3, ag.SGDOptions(LR=0.1))
    with pytest.raises(ag.HostError, match="incompatible SGD snapshot"):
        ag.LoadTrainingCheckpoint(path, model3, sgd, sched3)


def test_onecycle_schedule_values(ag):
    """autograd/nn.go:539-571 restated independently: warm-up to the peak, cosine down to the floor."""
    c = ag.OneCycle(0.1, 20, 0.25)

    def want(step, max_lr=0.1, total=20, pct=0.25, div=25.0, final_div=1e4):
        initial = max_lr / div
        final = initial / final_div
        warm = max(pct * total - 1, 0)
        if step <= warm:
            start, end, p = initial, max_lr, (step / warm if warm > 0 else 0)
        else:
            start, end, p = max_lr, final, (step - warm) / ((total - 1) - warm)
        return end + (start - end) * (1 + math.cos(math.pi * p)) / 2

    for step in range(20):
        c.StepCount = step
        assert abs(c.LR() - want(step)) <= 1e-15
    with pytest.raises(ag.HostError, match="invalid OneCycle"):
        ag.OneCycle(0.1, 1, 0.25)


def test_two_threads_clip_concurrently_and_read_their_own_norm(ag):
    """autograd/cuda_concurrency_test.go:247-304: clip state belongs to the calling OS thread, so two
    training runs clipping at the same time neither share a plan nor read each other's norm."""
    import threading
    results, errors = {}, []
    barrier = threading.Barrier(2)

    def run(tag, scale):
        try:
            rng = np.random.default_rng(hash(tag) % 1000)
            grads = [rng.normal(0, scale, n).astype(np.float32) for n in (50_000, 17, 4096)]
            params = [ag.Parameter(f"{tag}{i}", ag.Tensor(np.zeros(g.size, np.float32))) for i, g in enumerate(grads)]
            want = math.sqrt(sum(float(np.sum(g.astype(np.float64) ** 2)) for g in grads))
            for rep in range(20):
                for p, g in zip(params, grads):
                    p.Value.set_grad(g)
                barrier.wait(timeout=60)
                ag.ClipGradNorm(params, 1.0)
                got = ag.GradientNormToHost()
                assert abs(got - want) <= 1e-4 * want, (tag, rep, got, want)
                coef = np.float32(1.0) / (np.float32(got) + np.float32(1e-6)) if got > 1.0 else np.float32(1.0)
                assert np.array_equal(params[1].Value.grad_to_host(), grads[1] * coef)
            results[tag] = got
            ag.ReleaseClipState()
        except Exception as e:  # surfaced in the main thread below
            errors.append((tag, repr(e)))
            barrier.abort()

    threads = [threading.Thread(target=run, args=("a", 0.5)), threading.Thread(target=run, args=("b", 2.0))]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not errors, errors
    assert set(results) == {"a", "b"} and abs(results["a"] - results["b"]) > 1.0


def test_shadow_lease_survives_an_optimizer_step(ag):
    """autograd/cuda_autocast.go:77-94, autograd/audit_bf16_lease_test.go: a reader that leased the bf16
    shadow before the step (a graph node waiting for its backward pass) keeps a valid, unchanged
    buffer; the step writes its new shadow elsewhere; returning the lease frees the old buffer; with
    no lease out the step rewrites the shadow in place."""
    import ctypes as C
    from gograd_b200 import _lib
    rng = np.random.default_rng(12)
    w = ag.Tensor(rng.normal(0, .05, 5000).astype(np.float32))
    p = [ag.Parameter("w", w)]
    opt = ag.NewAdamW(p, 1e-2, 0.0)
    opt.SetEngine(write_shadow=True)

    def bf16_at(address, n):
        out = np.empty(n, np.uint16)
        _lib.check(_lib.lib().oe_memcpy_d2h(0, out.ctypes.data_as(C.c_void_p), address, 2 * n, 0))
        _lib.check(_lib.lib().oe_stream_sync(0, 0))
        return out

    w.set_grad(rng.normal(0, .1, 5000).astype(np.float32))
    opt.Step()
    first = w.shadow_to_host().copy()
    first_address = w.address(2)
    lease = w.shadow_lease()
    assert lease == first_address and w.leased_shadows == 1
    opt.Step()                                   # must not overwrite the leased buffer
    assert w.address(2) != first_address and w.shadow_current
    assert np.array_equal(bf16_at(lease, 5000), first), "the leased shadow changed under its reader"
    second = w.shadow_to_host()
    assert not np.array_equal(second, first)
    want = torch.from_numpy(w.to_host()).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(second, want)
    assert w.leased_shadows == 1
    w.shadow_release(lease)
    assert w.leased_shadows == 0
    in_place = w.address(2)
    opt.Step()                                   # nobody reads the shadow: rewritten in place
    assert w.address(2) == in_place and w.shadow_current


def test_accumulated_gradients_read_at_the_seed_scale(ag):
    """Four micro-batches (autograd/accumulate_test.go:97-141 splits a batch the same way). One run
    stores each micro-batch gradient at the accumulator's seed 1/4, as Backward would; the other
    stores them raw and hands the seed to the optimizer as its gradient scale. A power-of-two factor
    commutes with the fp32 additions, so both runs end on the same bits, AdamW and SGD alike; an
    invalid scale is refused and leaves the step counter where it was."""
    rng = np.random.default_rng(31)
    sizes = (1000, 7, 4096, 5001)
    values = [rng.normal(0, .05, n).astype(np.float32) for n in sizes]
    micro = [[rng.normal(0, .5, n).astype(np.float32) for n in sizes] for _ in range(8)]
    for kind in ("adamw", "sgd"):
        runs = []
        for folded in (False, True):
            params = params_of(ag, [(f"p{i}", v) for i, v in enumerate(values)])
            if kind == "adamw":
                opt = ag.NewAdamW(params, 1e-2, 0.1)
            else:
                opt = ag.NewSGD(params, ag.SGDOptions(LR=0.05, Momentum=0.9, WeightDecay=0.01))
            acc = ag.GradAccumulator(4)
            if folded:
                opt.SetGradScale(float(acc.MicroBatch()[0]))
                acc.Reset()
            sums = [np.zeros(n, np.float32) for n in sizes]
            for k in range(8):
                seed, complete = acc.MicroBatch()
                for i in range(len(sizes)):
                    g = micro[k][i] if folded else (micro[k][i] * seed).astype(np.float32)
                    sums[i] = (sums[i] + g).astype(np.float32)
                assert complete == (k % 4 == 3)
                if complete:
                    for p, g in zip(params, sums):
                        p.Value.set_grad(g)
                    opt.StepClipped(1.0)
                    sums = [np.zeros(n, np.float32) for n in sizes]
            assert opt.StepCount == 2
            runs.append([p.Value.to_host() for p in params])
            if folded:
                for bad in (0.0, -2.0, float("nan")):
                    with pytest.raises(ag.HostError, match="invalid gradient scale"):
                        opt.SetGradScale(bad)
                opt.StepClipped(1.0)
                assert opt.StepCount == 3
            opt.Close()
        for a, b in zip(*runs):
            assert np.array_equal(a, b), kind


def test_step_zeroes_the_gradients_it_read_and_zero_grad_finds_nothing_to_do(ag):
    """The loop around the optimizer calls ZeroGrad at the start of every group
    (autograd/training_loop.go:125-133) and AdamW.ZeroGrad keeps the buffers and zeroes them
    (autograd/nn.go:533-537). With zeroing folded into Step the gradients are zero when Step returns,
    the following ZeroGrad launches nothing, results are unchanged, and a gradient written afterwards
    is zeroed again the usual way. SGD refuses: its ZeroGrad makes gradients absent."""
    import gograd_b200 as eng
    rng = np.random.default_rng(41)
    sizes = (1000, 7, 4096, 20001)
    values = [rng.normal(0, .05, n).astype(np.float32) for n in sizes]
    grads = [[rng.normal(0, .5, n).astype(np.float32) for n in sizes] for _ in range(3)]
    runs = []
    for fused in (False, True):
        params = params_of(ag, [(f"p{i}", v) for i, v in enumerate(values)])
        opt = ag.NewAdamW(params, 1e-2, 0.1)
        if fused:
            opt.SetZeroGradInStep(True)
        for step in range(3):
            opt.ZeroGrad()
            for p, g in zip(params, grads[step]):
                p.Value.set_grad(g)
            assert not any(p.Value.grad_known_zero for p in params)
            opt.StepClipped(1.0)
            if fused:
                assert all(p.Value.grad_known_zero for p in params)
                assert all(float(np.abs(p.Value.grad_to_host()).max()) == 0.0 for p in params)
                before = eng.launch_count()
                opt.ZeroGrad()
                assert eng.launch_count() == before, "nothing to zero: nothing launched"
            else:
                assert np.array_equal(params[0].Value.grad_to_host(), grads[step][0])
        runs.append([p.Value.to_host() for p in params])
        if fused:
            params[2].Value.set_grad(grads[0][2])
            before = eng.launch_count()
            opt.ZeroGrad()
            assert eng.launch_count() == before + 1 and float(np.abs(params[2].Value.grad_to_host()).max()) == 0.0
            assert all(p.Value.grad_known_zero for p in params)
        opt.Close()
    for a, b in zip(*runs):
        assert np.array_equal(a, b)
    sgd_params = params_of(ag, [("w", values[0])])
    sgd = ag.NewSGD(sgd_params, ag.SGDOptions(LR=0.1))
    sgd.SetZeroGradInStep(True)
    sgd_params[0].Value.set_grad(grads[0][0])
    with pytest.raises(ag.HostError, match="releases its gradients"):
        sgd.Step()
    assert sgd.StepCount == 0 and np.array_equal(sgd_params[0].Value.to_host(), values[0])
    sgd.Close()


def test_sgd_captured_steps_match_eager_and_sync_the_counter(ag):
    """autograd/sgd_test.go:268-333: three captured steps over a stable gradient equal three eager
    steps (weights and momentum), State reads the device counter, an eager step afterwards syncs the
    host count and invalidates the bf16 shadow. Prepared for graphs, ZeroGrad keeps the buffers and
    zeroes them (autograd/sgd.go:228-246), and Step may do that zeroing itself."""
    import gograd_b200 as eng
    initial = np.float32([.3, -.7, .2, .4])
    grad = np.float32([.2, -.3, .1, .4])
    options = ag.SGDOptions(LR=.03, Momentum=.9, Dampening=.2, WeightDecay=.1)
    p, q = ag.Parameter("weight", ag.Tensor(initial, [2, 2])), ag.Parameter("weight", ag.Tensor(initial, [2, 2]))
    o, eager = ag.NewSGD([p], options), ag.NewSGD([q], options)
    with pytest.raises(ag.HostError, match="call SGD.PrepareGraph before capture"):
        o.StepCaptured()
    p.Value.set_grad(grad)
    o.PrepareGraph()
    for _ in range(3):
        o.StepCaptured()
    for _ in range(3):
        eager.ZeroGrad()
        assert not q.Value.has_grad, "eager ZeroGrad makes the gradient absent"
        q.Value.set_grad(grad)
        eager.Step()
    assert o.GraphStepCount() == 3
    assert o.StepCount == 0, "a captured step changes no host state"
    assert np.array_equal(p.Value.to_host(), q.Value.to_host())
    left, right = o.Buffer(0), eager.Buffer(0)
    assert left[1] and right[1] and np.array_equal(left[0], right[0])
    # graph mode: ZeroGrad keeps the buffer and zeroes it
    o.ZeroGrad()
    assert p.Value.has_grad and float(np.abs(p.Value.grad_to_host()).max()) == 0.0
    # an eager step after replay syncs the host count and invalidates the shadow
    o.SetEngine(write_shadow=True)
    p.Value.set_grad(grad)
    o.Step()
    assert o.StepCount == 4 and o.GraphStepCount() == 4 and p.Value.shadow_current
    o.SetEngine(write_shadow=False)
    p.Value.set_grad(grad)
    o.Step()
    assert o.StepCount == 5 and not p.Value.shadow_current, "a step that does not rewrite the shadow invalidates it"
    # zeroing folded into Step is accepted once prepared for graphs, refused by an eager SGD
    o.SetZeroGradInStep(True)
    p.Value.set_grad(grad)
    o.Step()
    assert p.Value.grad_known_zero and float(np.abs(p.Value.grad_to_host()).max()) == 0.0
    before = eng.launch_count()
    o.ZeroGrad()
    assert eng.launch_count() == before and p.Value.has_grad
    eager.SetZeroGradInStep(True)
    q.Value.set_grad(grad)
    with pytest.raises(ag.HostError, match="releases its gradients"):
        eager.Step()
    assert eager.StepCount == 3
    o.Close()
    eager.Close()


def test_a_bf16_gemm_consumes_the_shadow_the_step_wrote(ag):
    """The consumer on the far side of the path: the next forward's matrix multiply takes a lease on the
    weight's bf16 shadow (autograd/cuda_blas.go:97-99,197-203) instead of casting the fp32 master again.
    A library bf16 GEMM over the leased buffer gives the bits of the same GEMM over a fresh cast of the
    master, before and after further steps, and the leased operand stays what the GEMM node captured."""
    class Borrowed:
        def __init__(self, address, shape):
            self.__cuda_array_interface__ = {"shape": shape, "typestr": "<i2", "data": (address, False), "version": 2}

    rng = np.random.default_rng(61)
    rows, cols = 96, 128
    w = ag.Tensor(rng.normal(0, .05, rows * cols).astype(np.float32), [rows, cols])
    opt = ag.NewAdamW([ag.Parameter("w", w)], 1e-2, 0.1)
    opt.SetEngine(write_shadow=True)
    x = torch.from_numpy(rng.normal(0, 1, (32, rows)).astype(np.float32)).cuda().to(torch.bfloat16)

    def forward_with_lease():
        lease = w.shadow_lease()
        weight = torch.as_tensor(Borrowed(lease, (rows, cols)), device="cuda").view(torch.bfloat16)
        return lease, weight, x @ weight

    def forward_with_fresh_cast():
        master = torch.from_numpy(w.to_host()).cuda().view(rows, cols)
        return x @ master.to(torch.bfloat16)

    w.set_grad(rng.normal(0, .1, rows * cols).astype(np.float32))
    opt.StepClipped(1.0)
    lease1, weight1, y1 = forward_with_lease()
    assert torch.equal(y1, forward_with_fresh_cast())
    captured = weight1.clone()
    w.set_grad(rng.normal(0, .1, rows * cols).astype(np.float32))
    opt.StepClipped(1.0)                      # the first forward's node still holds its lease
    assert torch.equal(weight1, captured), "the operand a graph node kept must not change under it"
    lease2, weight2, y2 = forward_with_lease()
    assert lease2 != lease1 and torch.equal(y2, forward_with_fresh_cast()) and not torch.equal(y2, y1)
    w.shadow_release(lease1)
    w.shadow_release(lease2)
    assert w.leased_shadows == 0
    torch.cuda.synchronize()
    opt.Close()
