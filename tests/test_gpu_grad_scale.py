"""The plan's gradient scale: norm and update read every gradient element as float32(g*scale).

The oracle is the reference's optimizer fed with gradients stored at that scale (each element
rounded once to fp32, then clip and step as always): results must be bit-identical. With a
power-of-two scale this is also what GradAccumulator.Backward's 1/groups seed produces
(autograd/accumulate.go:31-44), shown here by accumulating micro-batch gradients both ways.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

SIZES = [1, 3, 4, 5, 257, 4096, 8193, 30001]


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
    return torch.from_numpy(np.require(a, requirements="C")).cuda()


def host(t):
    return t.detach().cpu().numpy()


def bc(beta1, beta2, t):
    from gograd_b200.workload import bias_corrections
    return bias_corrections(beta1, beta2, t)


def scaled(orc, grads, scale):
    out = [x.copy() for x in grads]
    for x in out:
        orc.scale_(x, scale)          # one fp32 multiply per element, the oracle's own routine
    return out


@pytest.mark.parametrize("scale", [0.25, 1.0 / 3.0, 1.0, 1.0 / 65536.0, 3.0])
def test_adamw_with_clip_reads_scaled_gradients(eng, orc, scale):
    rng = np.random.default_rng(5)
    hp_ = [rng.normal(0, .05, n).astype(np.float32) for n in SIZES]
    p = [dev(x) for x in hp_]
    g = [torch.zeros_like(x) for x in p]
    m = [torch.zeros_like(x) for x in p]
    v = [torch.zeros_like(x) for x in p]
    shadow = [torch.zeros(n, dtype=torch.int16, device="cuda") for n in SIZES]
    plan = eng.Plan([eng.TensorDesc(p[i], g[i], m[i], v[i], shadow[i], 1.0, 0.1) for i in range(len(p))])
    plan.set_grad_scale(scale)
    ref = orc.OracleAdamW([x.copy() for x in hp_], lr=1e-3, weight_decay=0.1, beta1=0.9, beta2=0.95, eps=1e-8)
    max_norm = 0.5 * scale            # clips on every step at every scale
    for t in range(1, 4):
        grads = [rng.normal(0, .02, n).astype(np.float32) for n in SIZES]
        for gi, x in zip(g, grads):
            gi.copy_(torch.from_numpy(x))
        fed = scaled(orc, grads, scale)
        want_norm, coef = orc.clip_grad_norm(fed, max_norm)
        assert coef < 1.0
        ref.step(fed)
        b1, b2 = bc(0.9, 0.95, t)
        plan.grad_norm()
        plan.adamw_step(eng.AdamWHParams(1e-3, 0.9, 0.95, 1e-8, b1, b2, max_norm=max_norm, flags=eng.engine.OE_WRITE_SHADOW))
        norm, _ = plan.read_norm()
        assert abs(norm - float(want_norm)) <= 1e-6 * float(want_norm)
        for i in range(len(p)):
            assert np.array_equal(host(p[i]), ref.params[i]), f"scale {scale} step {t} p[{i}]"
            assert np.array_equal(host(m[i]), ref.m[i]) and np.array_equal(host(v[i]), ref.v[i])
            assert np.array_equal(host(shadow[i]), orc.f32_to_bf16(ref.params[i]).view(np.int16))
            assert np.array_equal(host(g[i]), grads[i]), "the stored gradient is read, never rewritten"
    plan.close()


def test_sgd_reads_scaled_gradients(eng, orc):
    rng = np.random.default_rng(9)
    hp_ = [rng.normal(0, .05, n).astype(np.float32) for n in SIZES]
    p = [dev(x) for x in hp_]
    g = [torch.zeros_like(x) for x in p]
    buf = [torch.zeros_like(x) for x in p]
    flag = [torch.zeros(1, device="cuda") for _ in p]
    plan = eng.Plan([eng.TensorDesc(p[i], g[i], buf[i], flag[i], None, 1.0, 0.01) for i in range(len(p))])
    scale = 1.0 / 6.0
    plan.set_grad_scale(scale)
    ref = orc.OracleSGD([x.copy() for x in hp_], lr=0.05, momentum=0.9, weight_decay=0.01, nesterov=True)
    for t in range(3):
        grads = [rng.normal(0, .02, n).astype(np.float32) for n in SIZES]
        for gi, x in zip(g, grads):
            gi.copy_(torch.from_numpy(x))
        fed = scaled(orc, grads, scale)
        orc.clip_grad_norm(fed, 0.05)
        ref.step(fed)
        plan.grad_norm()
        plan.sgd_step(eng.SGDHParams(0.05, 0.9, 0.0, 0.05, eng.engine.OE_NESTEROV))
        for i in range(len(p)):
            assert np.array_equal(host(p[i]), ref.params[i]), f"step {t} p[{i}]"
            assert np.array_equal(host(buf[i]), ref.buffers[i]), f"step {t} buffer[{i}]"
    plan.close()


def test_power_of_two_scale_equals_seeding_backward_with_it(eng, orc):
    """Four micro-batches. The reference seeds each backward with 1/4, so the buffers accumulate
    g_k/4; here they accumulate the raw g_k and the step reads the sum at scale 1/4. Scaling by a
    power of two commutes with fp32 addition (no underflow at these magnitudes): same bits."""
    rng = np.random.default_rng(21)
    groups = 4
    hp_ = [rng.normal(0, .05, n).astype(np.float32) for n in SIZES]
    micro = [[rng.normal(0, .02, n).astype(np.float32) for n in SIZES] for _ in range(groups)]
    seeded = []
    for i in range(len(SIZES)):
        acc = np.zeros(SIZES[i], np.float32)
        for k in range(groups):
            acc = (acc + micro[k][i] * np.float32(1.0 / groups)).astype(np.float32)
        seeded.append(acc)
    ref = orc.OracleAdamW([x.copy() for x in hp_], lr=1e-3, weight_decay=0.0, beta1=0.9, beta2=0.999, eps=1e-8)
    clipped = [x.copy() for x in seeded]
    orc.clip_grad_norm(clipped, 0.01)
    ref.step(clipped)

    p = [dev(x) for x in hp_]
    g = [torch.zeros_like(x) for x in p]
    m = [torch.zeros_like(x) for x in p]
    v = [torch.zeros_like(x) for x in p]
    for k in range(groups):
        for gi, x in zip(g, micro[k]):
            gi.add_(torch.from_numpy(x).cuda())
    plan = eng.Plan([eng.TensorDesc(p[i], g[i], m[i], v[i], None, 1.0, 0.0) for i in range(len(p))])
    plan.set_grad_scale(1.0 / groups)
    b1, b2 = bc(0.9, 0.999, 1)
    plan.grad_norm()
    plan.adamw_step(eng.AdamWHParams(1e-3, 0.9, 0.999, 1e-8, b1, b2, max_norm=0.01))
    for i in range(len(p)):
        assert np.array_equal(host(p[i]), ref.params[i]), f"p[{i}]"
        assert np.array_equal(host(m[i]), ref.m[i]) and np.array_equal(host(v[i]), ref.v[i])
    plan.close()


def test_scale_rules(eng):
    x = torch.ones(5000, device="cuda")
    g = torch.full((5000,), 2.0, device="cuda")
    m, v = torch.zeros_like(x), torch.zeros_like(x)
    plan = eng.Plan([eng.TensorDesc(x, g, m, v, None, 1.0, 0.0)])
    for bad in (0.0, -1.0, float("nan"), float("inf")):
        with pytest.raises(eng._lib.EngineError, match="finite and positive"):
            plan.set_grad_scale(bad)
    plan.set_grad_scale(0.5)
    plan.grad_norm()
    norm, sumsq = plan.read_norm()
    assert sumsq == 5000.0 and norm == np.float32(np.sqrt(5000.0))
    # norm-only use of the clip entry point still works; an in-place clip would be applied twice
    plan.clip_grad_norm(0.0)
    with pytest.raises(eng._lib.EngineError, match="in-place clip"):
        plan.clip_grad_norm(1.0)
    assert float(g.min()) == 2.0 and float(g.max()) == 2.0
    with pytest.raises(eng._lib.EngineError, match="fold it into this call"):
        plan.peer_reduce_grads([g.data_ptr()], 0, 4096, g.data_ptr(), 1.0, 0)
    plan.set_grad_scale(1.0)
    plan.clip_grad_norm(1.0)
    assert abs(float(g[0]) - 2.0 / (np.sqrt(20000.0) + 1e-6)) < 1e-7
    plan.close()
