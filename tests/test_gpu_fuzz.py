"""Seeded randomised comparison of the engine with the oracle: random tensor counts, ragged sizes,
unaligned addresses, absent gradients, groups, clip rules, shadows, flags, work-unit sizes, gradient
scales, host or device step counters and both optimizers.
Every fp32 output must be bit-identical to the oracle's, every shadow equal to RNE of the master."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

SIZES = [1, 2, 3, 4, 5, 7, 8, 63, 64, 65, 1000, 4095, 4096, 4097, 8191, 8193, 12288, 20011]


def _guards_untouched(view):
    """The elements of the allocation around a view still hold what they were created with (zeros)."""
    base = view._base
    if base is None:
        return True
    start = view.storage_offset()
    flat = base.reshape(-1)
    return bool((flat[:start] == 0).all()) and bool((flat[start + view.numel():] == 0).all())


def _slice_with_offset(values, offset):
    """A device tensor whose first element sits `offset` floats past an allocation boundary."""
    backing = torch.zeros(values.size + offset + 4, dtype=torch.float32, device="cuda")
    view = backing[offset:offset + values.size]
    view.copy_(torch.from_numpy(values))
    return view


@pytest.mark.parametrize("seed", range(64))
def test_random_configuration(seed):
    import gograd_b200 as eng
    from gograd_b200.engine import (OE_CLIP_DEVFORM, OE_MAXIMIZE, OE_NESTEROV, OE_WRITE_SHADOW, OE_ZERO_GRAD)
    from gograd_b200.workload import bias_corrections
    from oracle import oracle

    eng.init(0)
    rng = np.random.default_rng(1000 + seed)
    n_tensors = int(rng.integers(1, 7))
    sizes = [int(rng.choice(SIZES)) for _ in range(n_tensors)]
    offsets = [int(rng.choice([0, 0, 0, 1, 2, 3])) for _ in range(n_tensors)]
    scales = [float(rng.choice([1.0, 0.5, 2.0])) for _ in range(n_tensors)]
    decays = [float(rng.choice([0.0, 0.01, 0.1])) for _ in range(n_tensors)]
    use_adamw = bool(rng.integers(0, 2))
    shadow_on = bool(rng.integers(0, 2))
    zero_grad = bool(rng.integers(0, 2))
    clip = float(rng.choice([0.0, 0.05, 1e9]))          # off, triggers, never triggers
    devform = bool(rng.integers(0, 2))
    steps = 3
    extra = np.random.default_rng(5000 + seed)          # drawn apart: the cases above keep their configurations
    grad_scale = float(extra.choice([1.0, 1.0, 0.25, 1.0 / 3.0, 1.0 / 1024.0]))
    unit = int(extra.choice([0, 0, 1024, 2048, 8192]))
    device_counter = bool(extra.integers(0, 2))
    step_dev = torch.zeros(1, dtype=torch.int32, device="cuda")
    host_p = [rng.normal(0, .05, n).astype(np.float32) for n in sizes]
    p = [_slice_with_offset(x, o) for x, o in zip(host_p, offsets)]
    g = [_slice_with_offset(np.zeros(n, np.float32), o) for n, o in zip(sizes, offsets)]
    s1 = [_slice_with_offset(np.zeros(n, np.float32), o) for n, o in zip(sizes, offsets)]
    sh = [torch.zeros(n + 3, dtype=torch.int16, device="cuda")[int(rng.choice([0, 0, 1])):][:n] for n in sizes]
    groups = [oracle.Group(f"g{i}", [i], scales[i], decays[i]) for i in range(n_tensors)]
    if use_adamw:
        beta2 = float(rng.choice([0.95, 0.999]))
        s2 = [_slice_with_offset(np.zeros(n, np.float32), o) for n, o in zip(sizes, offsets)]
        ref = oracle.OracleAdamW([x.copy() for x in host_p], lr=1e-3, groups=groups, beta2=beta2)
    else:
        momentum = float(rng.choice([0.0, 0.9]))
        nesterov = bool(momentum > 0 and rng.integers(0, 2))
        dampening = 0.0 if nesterov else float(rng.choice([0.0, 0.2]))
        maximize = bool(rng.integers(0, 2))
        s2 = [torch.zeros(1, device="cuda") for _ in sizes]
        ref = oracle.OracleSGD([x.copy() for x in host_p], lr=0.05, momentum=momentum, dampening=dampening,
                               nesterov=nesterov, maximize=maximize, groups=groups)
    plan = None
    for t in range(1, steps + 1):
        present = [bool(rng.random() > 0.25) for _ in sizes]
        grads = [rng.normal(0, .02, n).astype(np.float32) if ok else None for n, ok in zip(sizes, present)]
        descs = []
        for i in range(n_tensors):
            if grads[i] is not None:
                g[i].copy_(torch.from_numpy(grads[i]))
            state1 = s1[i] if (use_adamw or momentum > 0) else None
            state2 = s2[i] if (use_adamw or momentum > 0) else None
            descs.append(eng.TensorDesc(p[i], g[i] if present[i] else None, state1, state2,
                                        sh[i] if shadow_on else None, scales[i], decays[i]))
        if plan is None:
            plan = eng.Plan(descs, 0, unit)
            plan.set_grad_scale(grad_scale)
        else:
            plan.update(descs)
        # the oracle reads the gradients at the plan's scale, then clips in place with the rule under test
        clipped = [None if x is None else x.copy() for x in grads]
        for x in clipped:
            if x is not None:
                oracle.scale_(x, grad_scale)
        if clip > 0:
            norm = np.float32(np.sqrt(oracle.sum_squares(clipped)))
            coef = oracle.clip_coefficient(float(norm), clip, devform=devform)
            for x in clipped:
                if x is not None:
                    oracle.scale_(x, float(coef))
        flags = (OE_WRITE_SHADOW if shadow_on else 0) | (OE_ZERO_GRAD if zero_grad else 0) | \
                (OE_CLIP_DEVFORM if devform else 0)
        if clip > 0:
            plan.grad_norm()
        if use_adamw:
            ref.step(clipped)
            b1, b2 = bias_corrections(0.9, beta2, t)
            if device_counter:
                plan.adamw_step(eng.AdamWHParams(1e-3, 0.9, beta2, 1e-8, max_norm=clip, flags=flags,
                                                 step_dev=step_dev.data_ptr()))
            else:
                plan.adamw_step(eng.AdamWHParams(1e-3, 0.9, beta2, 1e-8, b1, b2, clip, flags))
        else:
            ref.step(clipped)
            flags |= (OE_NESTEROV if nesterov else 0) | (OE_MAXIMIZE if maximize else 0)
            plan.sgd_step(eng.SGDHParams(0.05, momentum, dampening, clip, flags,
                                         step_dev=step_dev.data_ptr() if device_counter else 0))
        torch.cuda.synchronize()
        if device_counter:
            assert int(step_dev.item()) == t, "the launch advances the device step counter"
        what = f"seed {seed} step {t}"
        for i in range(n_tensors):
            assert np.array_equal(p[i].cpu().numpy(), ref.params[i]), f"{what}: p[{i}] size {sizes[i]} offset {offsets[i]}"
            if use_adamw:
                assert np.array_equal(s1[i].cpu().numpy(), ref.m[i]) and np.array_equal(s2[i].cpu().numpy(), ref.v[i]), what
            elif momentum > 0:
                if ref.initialized[i]:
                    assert np.array_equal(s1[i].cpu().numpy(), ref.buffers[i]), what
                assert float(s2[i].item()) == float(ref.initialized[i]), what
            if shadow_on and present[i]:
                assert np.array_equal(sh[i].cpu().numpy().view(np.uint16), oracle.f32_to_bf16(ref.params[i])), what
            if present[i]:
                want_g = np.zeros(sizes[i], np.float32) if zero_grad else grads[i]
                assert np.array_equal(g[i].cpu().numpy(), want_g), f"{what}: gradient after the step"
    # canaries: nothing was written outside any tensor, whatever its offset, tail or work-unit size
    for group in (p, g, s1, sh, s2 if use_adamw else []):
        for t in group:
            assert _guards_untouched(t), f"seed {seed}: a kernel wrote outside a tensor"
    plan.close()
