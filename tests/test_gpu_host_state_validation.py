"""State files that must be rejected before anything changes, legacy layouts that must still load,
and resume of an SGD training checkpoint — the host mirror against the reference's
TestParameterGroupStateValidation (autograd/param_groups_test.go:507-619),
TestSGDValidationVersionsAndSnapshot (autograd/sgd_test.go:199-266) and
TestSGDCheckpointResumeAndLegacyAdamW (autograd/sgd_test.go:127-197)."""
import json
import math
import struct

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def ag():
    from gograd_b200 import autograd
    autograd.lib()
    return autograd


def read_file(path):
    raw = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    metadata = header.pop("__metadata__", None)
    entries = {}
    for name, h in header.items():
        a, b = h["data_offsets"]
        entries[name] = np.frombuffer(raw[8 + hlen + a:8 + hlen + b], dtype="<f4").reshape(h["shape"]).copy()
    return entries, metadata


def rewrite(ag, src, dst, edit_config=None, edit_metadata=None, edit_entries=None):
    entries, metadata = read_file(src)
    if edit_config:
        cfg = json.loads(metadata["optimizer"])
        edit_config(cfg)
        metadata["optimizer"] = json.dumps(cfg, separators=(",", ":"))
    if edit_metadata:
        edit_metadata(metadata)
    if edit_entries:
        edit_entries(entries)
    ag.safetensors_write(dst, entries, metadata)
    return dst


def snapshot(opt, params, sgd=True):
    state = [p.Value.to_host().copy() for p in params]
    for i in range(len(params)):
        state.append(opt.Buffer(i)[0].copy() if sgd else opt.M(i).copy())
        state.append(np.array([opt.Buffer(i)[1]]) if sgd else opt.V(i).copy())
    return state + [np.array([opt.StepCount]), np.array([opt.LearningRate()])] + \
        [np.array(opt.groupScale(i)) for i in range(len(params))]


def same(a, b):
    return len(a) == len(b) and all(np.array_equal(x, y) for x, y in zip(a, b))


def test_group_state_validation_and_legacy_state(ag, tmp_path):
    weight, bias = ag.Parameter("weight", ag.Tensor([1, 2])), ag.Parameter("bias", ag.Tensor([3, 4]))
    params = [weight, bias]
    specs = [ag.ParameterGroupSpec("decay", [weight], LRScale=.5, WeightDecay=.02), ag.ParameterGroupSpec("plain", [bias])]
    opt = ag.NewSGDGroups(params, ag.SGDOptions(LR=.1, Momentum=.9), specs)
    for p in params:
        p.Value.set_grad([.5, -.25])
    opt.Step()
    good = str(tmp_path / "good.safetensors")
    opt.SaveSafeTensors(good)
    before = snapshot(opt, params)

    def renamed_members(c):
        c["Groups"][0]["Names"], c["Groups"][1]["Names"] = ["gain"], ["weight"]

    def renamed_group(c):
        c["Groups"][1]["Name"] = "other"

    def missing_group(c):
        c["Groups"] = c["Groups"][:1]

    def negative_scale(c):
        c["Groups"][0]["LRScale"] = -1

    def negative_decay(c):
        c["Groups"][1]["WeightDecay"] = -1

    def bad_options(c):
        c["Options"]["Nesterov"], c["Options"]["Dampening"] = True, .5

    for k, edit in enumerate((renamed_members, renamed_group, missing_group, negative_scale, negative_decay, bad_options)):
        broken = rewrite(ag, good, str(tmp_path / f"broken{k}.safetensors"), edit_config=edit)
        with pytest.raises(ag.HostError):
            opt.LoadSafeTensors(broken)
        assert same(snapshot(opt, params), before), f"{edit.__name__}: a rejected state changed the optimizer"

    def nan_momentum(entries):
        entries["buffer.0"][0] = np.nan

    with pytest.raises(ag.HostError, match="non-finite SGD momentum"):
        opt.LoadSafeTensors(rewrite(ag, good, str(tmp_path / "nan.safetensors"), edit_entries=nan_momentum))
    assert same(snapshot(opt, params), before)

    # legacy state without groups: fits a single-group optimizer and brings its decay along
    def legacy(c):
        c["Groups"] = None
        c["Options"]["WeightDecay"] = .07

    legacy_path = rewrite(ag, good, str(tmp_path / "legacy.safetensors"), edit_config=legacy)
    flat_params = [ag.Parameter("weight", ag.Tensor([1, 2])), ag.Parameter("bias", ag.Tensor([3, 4]))]
    flat = ag.NewSGD(flat_params, ag.SGDOptions(LR=.1, Momentum=.9, WeightDecay=.3))
    flat.LoadSafeTensors(legacy_path)
    assert flat.groupScale(0)[1] == np.float32(.07) and flat.groupScale(1)[1] == np.float32(.07)
    assert flat.StepCount == 1 and flat.Buffer(0)[1]
    with pytest.raises(ag.HostError, match="no parameter groups"):
        opt.LoadSafeTensors(legacy_path)
    assert same(snapshot(opt, params), before)
    # the grouped file loads back and restores scale and decay of each group
    opt.LoadSafeTensors(good)
    assert opt.groupScale(0) == (np.float32(.1) * np.float32(.5), np.float32(.02)) and opt.groupScale(1)[1] == 0
    # closed optimizers refuse everything
    opt.Close()
    with pytest.raises(ag.HostError, match="closed"):
        opt.SaveSafeTensors(str(tmp_path / "closed.safetensors"))


def test_partition_parameters(ag):
    params = [ag.Parameter("weight", ag.Tensor([1])), ag.Parameter("bias", ag.Tensor([2])), ag.Parameter("gain", ag.Tensor([3]))]
    specs = ag.PartitionParameters(params, lambda name: "plain" if name == "bias" else "decay")
    assert [(s.Name, [p.Name for p in s.Params]) for s in specs] == [("decay", ["weight", "gain"]), ("plain", ["bias"])]
    with pytest.raises(ag.HostError, match="not assigned"):
        ag.PartitionParameters(params, lambda name: "")
    with pytest.raises(ag.HostError, match="no parameters to partition"):
        ag.PartitionParameters([], lambda name: "x")
    with pytest.raises(ag.HostError, match="duplicate parameter name"):
        ag.PartitionParameters(params + [ag.Parameter("bias", ag.Tensor([4]))], lambda name: "x")
    # the specs feed the grouped constructors
    specs[0].WeightDecay, specs[1].LRScale = .1, .5
    opt = ag.NewAdamWGroups(params, .01, specs)
    assert opt.groupScale(1) == (np.float32(.01) * np.float32(.5), np.float32(0))


def test_sgd_training_checkpoint_resume_wrong_kind_and_legacy_adamw(ag, tmp_path):
    """Nesterov SGD driven by OneCycle: loss = sum(p^2) so the gradient is 2p; eight steps with a
    checkpoint after three; the resumed run ends bit-identical. An AdamW optimizer refuses the SGD
    file before the model changes; a training file without optimizer_kind is read as AdamW."""
    def new_run():
        p = ag.Parameter("weight", ag.Tensor([.3, -.7]))
        o = ag.NewSGD([p], ag.SGDOptions(LR=.03, Momentum=.9, Nesterov=True, WeightDecay=.01))
        return [p], o, ag.OneCycle(.03, 8, .3)

    def step(model, o, s):
        o.ZeroGrad()
        for p in model:
            p.Value.set_grad(np.float32(2) * p.Value.to_host())
        o.Step()
        s.Step(o)

    m, o, schedule = new_run()
    o.SetLearningRate(schedule.LR())
    for _ in range(3):
        step(m, o, schedule)
    path = str(tmp_path / "training.safetensors")
    ag.SaveTrainingCheckpoint(path, m, o, schedule, {"sampler": "example"})
    d = ag.safetensors_describe(path)
    assert d["metadata"]["optimizer_kind"] == "sgd" and sorted(d["entries"]) == ["model.weight", "optimizer.buffer.0"]
    n, restored, c = new_run()
    assert ag.LoadTrainingCheckpoint(path, n, restored, c) == {"sampler": "example"}
    for _ in range(3, 8):
        step(m, o, schedule)
        step(n, restored, c)
    assert np.array_equal(m[0].Value.to_host(), n[0].Value.to_host())
    assert np.array_equal(o.Buffer(0)[0], restored.Buffer(0)[0]) and o.StepCount == restored.StepCount == 8
    assert schedule.fields() == c.fields() and o.LearningRate() == restored.LearningRate()
    adam = ag.NewAdamW(n, .1, 0)
    before = n[0].Value.to_host().copy()
    with pytest.raises(ag.HostError, match="incompatible AdamW snapshot"):
        ag.LoadTrainingCheckpoint(path, n, adam, c)
    assert np.array_equal(n[0].Value.to_host(), before), "optimizer kind mismatch changed the model"
    # an older training file has no optimizer_kind: it is AdamW
    legacy = str(tmp_path / "legacy.safetensors")
    adam_schedule = ag.OneCycle(.1, 8, .3)
    ag.SaveTrainingCheckpoint(legacy, n, adam, adam_schedule, None)

    def drop_kind(metadata):
        del metadata["optimizer_kind"]

    rewrite(ag, legacy, legacy, edit_metadata=drop_kind)
    assert "optimizer_kind" not in ag.safetensors_describe(legacy)["metadata"]
    assert ag.LoadTrainingCheckpoint(legacy, n, adam, adam_schedule) == {}


def test_onecycle_single_point_warmup_is_finite(ag):
    """autograd/training_checkpoint_test.go:272-281: a warm-up shorter than one step must not divide by zero."""
    c = ag.OneCycle(.002, 10, .1)
    for i in range(11):
        c.StepCount = i
        lr = c.LR()
        assert math.isfinite(lr) and lr > 0
    c.StepCount = 0
    assert abs(c.LR() - .002 / 25) < 1e-15
    for peak in (0.0, -1.0):
        with pytest.raises(ag.HostError, match="invalid OneCycle"):
            ag.OneCycle(peak, 10, .3)
