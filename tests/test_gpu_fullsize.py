"""Full-size checks: the GPT-style set against the oracle over its 50 steps, and the 1.3B set
against the oracle on every tensor plus size-independent properties."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def host(t):
    return t.detach().cpu().numpy()


def test_gpt_set_clip_shadow_groups_against_oracle():
    """109.6M parameters, two groups (decay .1 on matrices, 0 on norms/biases), 2 % of the tensors
    with x100 gradients so that clipping triggers, bf16 shadow: the configuration's 50 steps, every
    element of p, m, v against the oracle after steps 1 and 50 (bit-identical, and within the stated
    1e-6 / 1e-5), the norm within 1e-6 relative at every step, the shadow bit-exact to RNE of the GPU
    master."""
    import gograd_b200 as eng
    from gograd_b200 import paramsets, workload
    from gograd_b200.engine import OE_WRITE_SHADOW
    from oracle import oracle

    ps = paramsets.get("gpt")
    assert ps.numel == paramsets.EXPECTED_NUMEL["gpt"]
    st = workload.materialize(ps, "cuda:0")
    plan = eng.Plan(st.descs())
    names = [s.name for s in ps.params]
    groups = [oracle.Group(g.name, [i for i, s in enumerate(ps.params) if s.group == g.name], g.lr_scale,
                           g.weight_decay) for g in ps.groups]
    hp = ps.hparams
    ref = oracle.OracleAdamW([host(x).copy() for x in st.p], lr=hp["lr"], groups=groups, beta1=hp["beta1"],
                             beta2=hp["beta2"], eps=hp["eps"], max_procs=os.cpu_count() or 1)
    assert len(workload.boosted_indices(ps)) == 3 and ps.steps == 50
    for t in range(1, ps.steps + 1):
        workload.fill_grads(st, t)
        grads = [host(g).copy() for g in st.g]
        want_norm, scale = oracle.clip_grad_norm(grads, ps.max_norm)
        assert scale < 1, "the boosted tensors must make the clip trigger"
        ref.step(grads)
        b1, b2 = workload.bias_corrections(hp["beta1"], hp["beta2"], t)
        plan.grad_norm()
        plan.adamw_step(eng.AdamWHParams(hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], b1, b2, ps.max_norm,
                                         OE_WRITE_SHADOW))
        norm, _ = plan.read_norm()
        assert abs(norm - float(want_norm)) <= 1e-6 * float(want_norm)
        if t in (1, ps.steps):
            worst = 0.0
            for i, name in enumerate(names):
                for kind, got, want in (("p", st.p[i], ref.params[i]), ("m", st.s1[i], ref.m[i]),
                                        ("v", st.s2[i], ref.v[i])):
                    got = host(got)
                    scale_ = float(np.max(np.abs(want))) or 1.0
                    err = np.max(np.abs(got.astype(np.float64) - want) / (np.abs(want) + scale_))
                    worst = max(worst, float(err))
                    assert np.array_equal(got, want), f"step {t} {kind} {name} differs from the host loop"
            assert worst <= (1e-6 if t == 1 else 1e-5)
    for i in range(len(names)):
        want = st.p[i].to(torch.bfloat16).view(torch.int16)
        assert torch.equal(st.shadow[i].view(torch.int16), want), f"shadow {names[i]}"
    plan.close()


def test_llama1b_full_size_properties():
    """1,345,423,360 parameters, one fused step (clip 1.0 + shadow) at full size:
    - the norm equals an independent float64 reduction (torch) within 1e-6 relative;
    - every shadow element is round-to-nearest-even of the GPU's own master (torch's
      conversion, independent of this library) — bit-exact over all 1.3B elements;
    - ALL 219 tensors match the oracle element for element in p, m and v, with the clip
      coefficient derived from the norm (one tensor at a time on the host);
    - gradients are left untouched by the folded clip; two launches were issued."""
    import gograd_b200 as eng
    from gograd_b200 import paramsets, workload
    from gograd_b200.engine import OE_WRITE_SHADOW
    from oracle import oracle

    ps = paramsets.get("llama1b")
    assert ps.numel == paramsets.EXPECTED_NUMEL["llama1b"] and len(ps.params) == 219
    st = workload.materialize(ps, "cuda:0")
    # make the clip trigger: the natural norm is ~36.7 > 1
    plan = eng.Plan(st.descs())
    assert plan.active_elems == ps.numel
    p_before = [t.clone() for t in st.p]          # 5.4 GB on the device; read back one tensor at a time
    g_before = [t.clone() for t in st.g]
    ref_sq = sum(float((g.double() ** 2).sum().item()) for g in st.g)
    hp = ps.hparams
    b1, b2 = workload.bias_corrections(hp["beta1"], hp["beta2"], 1)
    eng.launch_count_reset()
    plan.grad_norm()
    plan.adamw_step(eng.AdamWHParams(hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], b1, b2, ps.max_norm,
                                     OE_WRITE_SHADOW))
    norm, sumsq = plan.read_norm()
    assert eng.launch_count() == 2
    assert abs(sumsq - ref_sq) <= 1e-9 * ref_sq
    assert abs(norm - ref_sq ** 0.5) <= 1e-6 * ref_sq ** 0.5
    for i in range(len(st.p)):
        assert torch.equal(st.shadow[i].view(torch.int16), st.p[i].to(torch.bfloat16).view(torch.int16)), i
    coef = float(oracle.clip_coefficient(norm, ps.max_norm))
    assert coef < 1
    wd = ps.groups[0].weight_decay
    checked = 0
    for i, spec in enumerate(ps.params):
        assert torch.equal(st.g[i], g_before[i]), f"folded clip modified the gradient of {spec.name}"
        p0, g = host(p_before[i]).copy(), host(g_before[i]).copy()
        oracle.scale_(g, coef)
        o = oracle.OracleAdamW([p0], lr=hp["lr"], weight_decay=wd, beta1=hp["beta1"], beta2=hp["beta2"],
                               eps=hp["eps"], max_procs=os.cpu_count() or 1)
        o.step([g])
        assert np.array_equal(host(st.p[i]), o.params[0]), spec.name
        assert np.array_equal(host(st.s1[i]), o.m[0]) and np.array_equal(host(st.s2[i]), o.v[0]), spec.name
        checked += p0.size
    assert checked == ps.numel
    del p_before, g_before
    # linearity of the norm: doubling every gradient doubles it exactly (power of two)
    for g in st.g:
        g.mul_(2.0)
    plan.grad_norm()
    norm2, sumsq2 = plan.read_norm()
    assert sumsq2 == 4.0 * sumsq and norm2 == np.float32(2.0) * np.float32(norm)
    plan.close()


def test_indexing_beyond_2_to_32_elements():
    """Flat shards of the 8B set are longer than 2^32 elements, so the reduce kernel indexes in 64 bits.
    Two emulated ranks with 2^32 + 12,288 + 3 elements each (34 GB on the device): the reduced values
    at sampled positions on both sides of the 2^31 and 2^32 boundaries and at the ragged end, and the
    sum of squares against an independent float64 reduction."""
    import gograd_b200 as eng
    from gograd_b200.engine import OE_PARTIAL_ONLY

    eng.init(0)
    n = (1 << 32) + 12_288 + 3
    free, _ = torch.cuda.mem_get_info()
    if free < 40 * (1 << 30):
        pytest.skip("needs 40 GB of free device memory")
    gen = torch.Generator(device="cuda").manual_seed(9)
    g0 = torch.empty(n, dtype=torch.float32, device="cuda").normal_(0, 1e-3, generator=gen)
    g1 = torch.empty(n, dtype=torch.float32, device="cuda").normal_(0, 1e-3, generator=gen)
    windows = [(0, 4096), ((1 << 31) - 2048, (1 << 31) + 2048), ((1 << 32) - 2048, (1 << 32) + 2048), (n - 5000, n)]
    want = [((g0[a:b] + g1[a:b]) * 0.5).cpu() for a, b in windows]
    want_sq = 0.0
    step = 1 << 28
    for a in range(0, n, step):
        want_sq += float(((g0[a:a + step] + g1[a:a + step]) * 0.5).double().pow(2).sum().item())
    dummy = torch.zeros(8, device="cuda")
    plan = eng.Plan([eng.TensorDesc(dummy, dummy)])
    plan.peer_reduce_grads([g0.data_ptr(), g1.data_ptr()], 0, n, g0.data_ptr(), 0.5, OE_PARTIAL_ONLY)  # in place
    _, got_sq = plan.read_norm()
    assert abs(got_sq - want_sq) <= 1e-10 * want_sq
    for (a, b), w in zip(windows, want):
        assert torch.equal(g0[a:b].cpu(), w), (a, b)
    plan.close()
    del g0, g1
    torch.cuda.empty_cache()
    # the plan-based kernels take one tensor of more than 2^31 elements (a single descriptor)
    m_elems = (1 << 31) + 4096 + 1
    p = torch.full((m_elems,), 0.5, dtype=torch.float32, device="cuda")
    g = torch.full((m_elems,), 2.0, dtype=torch.float32, device="cuda")
    g[-1] = 3.0
    plan = eng.Plan([eng.TensorDesc(p, g)])
    plan.grad_norm()
    norm, sumsq = plan.read_norm()
    assert sumsq == 4.0 * (m_elems - 1) + 9.0
    plan.sgd_step(eng.SGDHParams(0.125))
    torch.cuda.synchronize()
    assert float(p[0].item()) == 0.25 and float(p[(1 << 31) + 5].item()) == 0.25 and float(p[-1].item()) == 0.125
    assert float(p.min().item()) == 0.125 and float(p.max().item()) == 0.25
    plan.close()
