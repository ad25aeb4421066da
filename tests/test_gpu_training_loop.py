"""The loop that calls the optimizer (autograd.TrainingLoop, autograd/training_loop.go:53-214), driven
the way autograd/training_loop_test.go drives it: a fixed list of micro-batches per epoch, a sampler
that reports the reader's position, a real AdamW on the device. The step callback stands in for
forward + backward: it adds seed * g(batch) to every gradient buffer."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

SIZES = (12, 4, 4, 1)        # hidden 3x4 + bias, head 4x1 + bias, as the reference's test model


@pytest.fixture(scope="module")
def ag():
    from gograd_b200 import autograd
    autograd.lib()
    return autograd


class Reader:
    """loopReader (autograd/training_loop_test.go:22-60)."""

    def __init__(self, batches, cursor=0, fail_after=0, cancel_at=None):
        self.batches, self.cursor, self.epochs, self.fail_after = batches, cursor, 0, fail_after
        self.cancelled = cancel_at if cancel_at is not None else [False]

    def next(self):
        from gograd_b200.autograd import LoopCancelled
        if self.cancelled[0]:
            raise LoopCancelled("context canceled")
        if self.fail_after > 0 and self.cursor == self.fail_after:
            raise RuntimeError("loop reader failed")
        if self.cursor == len(self.batches):
            raise StopIteration
        self.cursor += 1
        return self.batches[self.cursor - 1]

    def next_epoch(self):
        self.epochs += 1
        self.cursor = 0
        self.fail_after = 0


class Sampler:
    def __init__(self, reader):
        self.reader, self.saves = reader, 0

    def marshal(self):
        self.saves += 1
        return f"position={self.reader.cursor}".encode()


def batches(count):
    rng = np.random.default_rng(5)
    return [[rng.normal(0, 1, n).astype(np.float32) for n in SIZES] for _ in range(count)]


def model(ag, seed):
    rng = np.random.default_rng(seed)
    return [ag.Parameter(f"p{i}", ag.Tensor(rng.normal(0, .5, n).astype(np.float32))) for i, n in enumerate(SIZES)]


def accumulate_step(params):
    def step(batch, seed):
        for p, g in zip(params, batch):
            have = p.Value.grad_to_host() if p.Value.has_grad else np.zeros(g.size, np.float32)
            p.Value.set_grad((have + g * seed).astype(np.float32))
        return float(sum(float(np.abs(g).sum()) for g in batch))
    return step


def test_loop_applies_updates_and_reports(ag):
    """autograd/training_loop_test.go:180-249, plus: the parameters equal a hand-written loop's."""
    params = model(ag, 3)
    initial = [p.Value.to_host() for p in params]
    opt = ag.NewAdamW(params, .01, 0)
    schedule = ag.OneCycle(.01, 6, .5)
    data = batches(3)
    reader = Reader(data, cursor=len(data))
    reported, losses, saved = [], [], []
    loop = ag.TrainingLoop(reader, opt, accumulate_step(params), sampler=Sampler(reader), schedule=schedule, updates=6,
                           accumulate=2, log_every=2, report=lambda u, l: (reported.append(u), losses.append(l)),
                           save=lambda sp: saved.append(sp))
    loop.Run()
    assert loop.Applied == 6 and reader.epochs == 4
    assert schedule.StepCount == 6
    assert reported == [1, 2, 4, 6] and all(l > 0 for l in losses)
    assert saved == [None], "a completed run has nothing to rewind"
    # a completed run leaves the last group's gradients in place
    assert all(float(np.abs(p.Value.grad_to_host()).max()) > 0 for p in params)
    assert all(not np.array_equal(p.Value.to_host(), w) for p, w in zip(params, initial))
    # the same twelve micro-batches through a hand-written loop
    ref = model(ag, 3)
    ref_opt = ag.NewAdamW(ref, .01, 0)
    ref_schedule = ag.OneCycle(.01, 6, .5)
    step = accumulate_step(ref)
    order = [data[k % 3] for k in range(12)]
    for k, batch in enumerate(order):
        if k % 2 == 0:
            ref_opt.ZeroGrad()
        step(batch, np.float32(0.5))
        if k % 2 == 1:
            ref_opt.Step()
            ref_schedule.Step(ref_opt)
    for a, b in zip(params, ref):
        assert np.array_equal(a.Value.to_host(), b.Value.to_host())
    assert opt.LearningRate() == ref_opt.LearningRate()
    opt.Close()
    ref_opt.Close()


def test_loop_validation(ag):
    """autograd/training_loop_test.go:251-282."""
    params = model(ag, 1)
    opt = ag.NewAdamW(params, .01, 0)
    reader = Reader(batches(2))

    def base(**changes):
        kw = dict(reader=reader, optimizer=opt, step=lambda batch, seed: 0.0, sampler=Sampler(reader), updates=2, applied=0)
        kw.update(changes)
        return ag.TrainingLoop(**kw)

    for name, changes in {"reader": dict(reader=None), "optimizer": dict(optimizer=None), "step": dict(step=None),
                          "updates": dict(updates=-1), "applied": dict(applied=3),
                          "sampler": dict(accumulate=2, sampler=None)}.items():
        with pytest.raises(ag.HostError):
            base(**changes).Run()
    # a run whose updates are all applied reads nothing and reports nothing
    reports = []
    before = reader.cursor
    finished = base(updates=2, applied=2, report=lambda u, l: reports.append(u))
    finished.Run()
    assert reports == [] and reader.cursor == before
    opt.Close()


@pytest.mark.parametrize("groups,after,in_step", [(1, 1, False), (3, 4, False), (3, 6, False), (1, 2, True),
                                                  (3, 1, True), (3, 3, True), (3, 5, True)])
def test_loop_interruption(ag, groups, after, in_step):
    """autograd/training_loop_test.go:284-355: cancelled between micro-batches or inside a step. Save runs
    once, with the starting position of the unfinished group (nothing when the last group was complete),
    the applied count stops at the completed groups and no gradient survives."""
    params = model(ag, 7)
    opt = ag.NewAdamW(params, .01, 0)
    cancelled = [False]
    reader = Reader(batches(8), cancel_at=cancelled)
    sampler = Sampler(reader)
    inner = accumulate_step(params)
    micro = [0]
    saved = []

    def step(batch, seed):
        loss = inner(batch, seed)
        micro[0] += 1
        if micro[0] == after:
            cancelled[0] = True
            if in_step:
                raise ag.LoopCancelled("step: context canceled")
        return loss

    loop = ag.TrainingLoop(reader, opt, step, sampler=sampler, updates=8, accumulate=groups, save=lambda sp: saved.append(sp))
    with pytest.raises(ag.LoopStopped, match="context canceled"):
        loop.Run()
    assert len(saved) == 1
    completed = after - 1 if in_step else after
    assert loop.Applied == completed // groups
    want = f"position={completed // groups * groups}".encode() if (in_step or after % groups != 0) else None
    assert saved[0] == want
    for p in params:
        assert float(np.abs(p.Value.grad_to_host()).max()) == 0.0, "unfinished gradients are dropped"
    opt.Close()


def test_loop_read_error_skips_save(ag):
    """autograd/training_loop_test.go:357-385."""
    params = model(ag, 9)
    opt = ag.NewAdamW(params, .01, 0)
    reader = Reader(batches(4), fail_after=2)
    saved = []
    loop = ag.TrainingLoop(reader, opt, accumulate_step(params), sampler=Sampler(reader), updates=4, accumulate=2,
                           save=lambda sp: saved.append(sp))
    with pytest.raises(ag.HostError, match="loop reader failed") as info:
        loop.Run()
    assert not isinstance(info.value, ag.LoopStopped)
    assert loop.Applied == 1 and saved == []
    opt.Close()


def test_loop_rejects_an_epoch_without_batches(ag):
    """autograd/training_loop_test.go:402-434."""
    params = model(ag, 1)
    opt = ag.NewAdamW(params, .01, 0)
    reader = Reader([])
    calls = []
    loop = ag.TrainingLoop(reader, opt, lambda batch, seed: calls.append("step") or 0.0, updates=1,
                           save=lambda sp: calls.append("save"))
    with pytest.raises(ag.HostError, match="training epoch contains no batches"):
        loop.Run()
    assert reader.epochs == 1 and loop.Applied == 0 and calls == []
    opt.Close()


def test_loop_with_zeroing_folded_into_step(ag):
    """The loop's ZeroGrad at the start of a group launches nothing once Step zeroes what it read;
    the run ends on the same parameters."""
    import gograd_b200 as eng
    runs = []
    for fused in (False, True):
        params = model(ag, 11)
        opt = ag.NewAdamW(params, .01, 0.1)
        if fused:
            opt.SetZeroGradInStep(True)
        reader = Reader(batches(4))
        eng.launch_count_reset()
        loop = ag.TrainingLoop(reader, opt, accumulate_step(params), sampler=Sampler(reader), updates=6, accumulate=2)
        loop.Run()
        assert loop.Applied == 6
        runs.append(([p.Value.to_host() for p in params], eng.launch_count("oe_zero_grads"), eng.launch_count()))
        opt.Close()
    for a, b in zip(runs[0][0], runs[1][0]):
        assert np.array_equal(a, b)
    assert runs[0][1] == 5 and runs[1][1] == 0, "five groups start over dirty gradients; none when Step zeroed them"
    assert runs[1][2] == 6, "six updates, six launches"
