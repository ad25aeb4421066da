"""The step entry points inside a CUDA graph: captured once, replayed with new gradients and a new
learning rate each time (autograd/audit_cuda_regression_test.go:180-243, autograd/sgd_test.go:268-333,
autograd/param_groups_test.go:200-286 check the same equivalence for the reference's captured steps)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_captured_adamw_step_follows_schedule_and_counter():
    import gograd_b200 as eng
    from gograd_b200.engine import OE_WRITE_SHADOW
    from gograd_b200.workload import bias_corrections
    from oracle import oracle

    eng.init(0)
    rng = np.random.default_rng(21)
    sizes = [5000, 257, 8192]
    decays = [0.1, 0.0, 0.1]
    scales = [1.0, 0.5, 1.0]
    hp0 = [rng.normal(0, .02, n).astype(np.float32) for n in sizes]
    p = [dev(x) for x in hp0]
    g = [torch.zeros_like(x) for x in p]
    m = [torch.zeros_like(x) for x in p]
    v = [torch.zeros_like(x) for x in p]
    sh = [torch.zeros(n, dtype=torch.int16, device="cuda") for n in sizes]
    plan = eng.Plan([eng.TensorDesc(p[i], g[i], m[i], v[i], sh[i], scales[i], decays[i]) for i in range(3)])
    groups = [oracle.Group(f"g{i}", [i], scales[i], decays[i]) for i in range(3)]
    ref = oracle.OracleAdamW([x.copy() for x in hp0], lr=1e-3, groups=groups, beta2=0.95)
    lrs = [1e-3, 2e-3, 5e-4, 1e-4]
    grads = [[rng.normal(0, .3, n).astype(np.float32) for n in sizes] for _ in lrs]

    def oracle_step(k):
        ref.lr = lrs[k]
        clipped = [x.copy() for x in grads[k]]
        oracle.clip_grad_norm(clipped, 1.0)
        ref.step(clipped)

    # step 1 eagerly (this also loads every kernel before anything is captured)
    for gi, x in zip(g, grads[0]):
        gi.copy_(torch.from_numpy(x))
    b1, b2 = bias_corrections(0.9, 0.95, 1)
    plan.grad_norm()
    plan.adamw_step(eng.AdamWHParams(lrs[0], 0.9, 0.95, 1e-8, b1, b2, 1.0, OE_WRITE_SHADOW))
    oracle_step(0)
    # device-resident step counter and learning rate (what PrepareGraph sets up)
    step_dev = torch.ones(1, dtype=torch.int32, device="cuda")
    lr_dev = torch.zeros(1, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    launches_before = eng.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        plan.grad_norm()
        plan.adamw_step(eng.AdamWHParams(123.0, 0.9, 0.95, 1e-8, max_norm=1.0, flags=OE_WRITE_SHADOW,
                                         step_dev=step_dev.data_ptr(), lr_dev=lr_dev.data_ptr()))
    assert eng.launch_count() - launches_before == 2  # norm and update (which advances the counter): captured, not run
    assert int(step_dev.item()) == 1, "capturing must not execute the step"
    for k in (1, 2, 3):
        for gi, x in zip(g, grads[k]):
            gi.copy_(torch.from_numpy(x))
        lr_dev.fill_(lrs[k])
        graph.replay()
        oracle_step(k)
    torch.cuda.synchronize()
    assert int(step_dev.item()) == 4
    for i in range(3):
        for name, got, want in (("p", p[i], ref.params[i]), ("m", m[i], ref.m[i]), ("v", v[i], ref.v[i])):
            got = got.cpu().numpy()
            scale = float(np.max(np.abs(want)))
            assert np.max(np.abs(got.astype(np.float64) - want) / (np.abs(want) + scale)) <= 1e-6, f"{name}[{i}]"
        assert np.array_equal(sh[i].cpu().numpy().view(np.uint16), oracle.f32_to_bf16(p[i].cpu().numpy()))
    plan.close()


def test_captured_sgd_step_initialises_then_blends():
    """One captured SGD step serves the first (buffer = gradient) and the later (blend) replays: the
    first-step decision is read from the per-tensor device flag inside the kernel."""
    import gograd_b200 as eng
    from gograd_b200.engine import OE_NESTEROV
    from oracle import oracle

    eng.init(0)
    rng = np.random.default_rng(22)
    sizes = [3000, 4100]
    hp0 = [rng.normal(0, .05, n).astype(np.float32) for n in sizes]
    p = [dev(x) for x in hp0]
    g = [torch.zeros_like(x) for x in p]
    buf = [torch.zeros_like(x) for x in p]
    flag = [torch.zeros(1, device="cuda") for _ in p]
    plan = eng.Plan([eng.TensorDesc(p[i], g[i], buf[i], flag[i], None, 1.0, 5e-4) for i in range(2)])
    ref = oracle.OracleSGD([x.copy() for x in hp0], lr=0.05, momentum=0.9, weight_decay=5e-4, nesterov=True)
    step_dev = torch.zeros(1, dtype=torch.int32, device="cuda")
    lr_dev = torch.full((1,), 0.05, dtype=torch.float32, device="cuda")
    # load the kernels outside the capture with a step of zero rate on throw-away state
    warm_p, warm_g = torch.zeros(8, device="cuda"), torch.zeros(8, device="cuda")
    warm_b, warm_f = torch.zeros(8, device="cuda"), torch.zeros(1, device="cuda")
    warm = eng.Plan([eng.TensorDesc(warm_p, warm_g, warm_b, warm_f)])
    warm.sgd_step(eng.SGDHParams(0.0, 0.9, step_dev=step_dev.data_ptr()))
    step_dev.zero_()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        plan.sgd_step(eng.SGDHParams(9.0, 0.9, 0.0, 0.0, OE_NESTEROV, step_dev=step_dev.data_ptr(),
                                     lr_dev=lr_dev.data_ptr()))
    for k in range(3):
        grads = [rng.normal(0, .02, n).astype(np.float32) for n in sizes]
        for gi, x in zip(g, grads):
            gi.copy_(torch.from_numpy(x))
        graph.replay()
        ref.step(grads)
    torch.cuda.synchronize()
    assert int(step_dev.item()) == 3
    for i in range(2):
        assert np.array_equal(p[i].cpu().numpy(), ref.params[i])
        assert np.array_equal(buf[i].cpu().numpy(), ref.buffers[i])
        assert float(flag[i].item()) == 1.0
    plan.close()
    warm.close()
