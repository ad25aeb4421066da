"""The allocation-free norm entry point, oe_grad_norm_static.

Some users of this library cannot allocate device memory once their training loop runs:
they reserved the whole GPU for their own arena at start-up, or they cannot take the
device-wide synchronisation that an allocation brings. For them the norm of one gradient
buffer is available without a plan, with its scratch in a fixed __device__ array of the
library. This test calls it through the C ABI twice in a row, on different data of
different lengths (the array is shared and keeps the previous call's contents, so the
second call proves that stale partial sums and the arrival counter do not leak), and
checks each result against the plan-based oe_grad_norm within the 1e-6 relative bound the
other norm tests use. It also checks that an over-long input is refused before any launch.

Collected last on purpose (file name), and self-contained: it passes alone in a fresh
process and after the rest of the suite.
"""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def test_static_norm_matches_plan_norm_twice():
    import gograd_b200 as eng
    from gograd_b200._lib import OE_ERR_LIMIT, lib

    eng.init(0)
    stream = int(torch.cuda.current_stream().cuda_stream)
    out = torch.full((1,), -1.0, dtype=torch.float32, device="cuda")
    rng = np.random.default_rng(42)
    # first a long buffer with a ragged tail, then a short one 4 bytes off a 16-byte boundary, then
    # a buffer longer than the persistent grid's first sweep (148 SMs x 4 CTAs x 65536 elements), and
    # one that crosses several spans on the element-by-element path (base 4 bytes off the boundary)
    for numel, offset, scale in ((3_000_001, 0, 1e-3), (70_001, 1, 5.0), (45_000_003, 0, 2e-3), (400_003, 1, 0.5)):
        host = (rng.standard_normal(numel + offset) * scale).astype(np.float32)
        backing = torch.from_numpy(host).cuda()
        g = backing[offset:]
        p = torch.zeros_like(g)
        plan = eng.Plan([eng.TensorDesc(p, g)])
        plan.grad_norm()
        want, _ = plan.read_norm()
        out.fill_(-1.0)
        rc = lib().oe_grad_norm_static(0, g.data_ptr(), numel, out.data_ptr(), stream)
        assert rc == 0, lib().oe_last_error()
        torch.cuda.synchronize()
        got = float(out.item())
        assert abs(got - want) <= 1e-6 * want, (numel, got, want)
        exact = float(np.sqrt(np.sum(host[offset:].astype(np.float64) ** 2)))
        assert abs(got - exact) <= 1e-6 * exact
        plan.close()
    # beyond 2^28 elements the array's slots each stand for 65536 elements instead of 8192: one buffer
    # on that side of the switch, generated on the device, against the plan norm and torch's float64 sum
    numel = (1 << 28) + 70_001
    g = torch.empty(numel, dtype=torch.float32, device="cuda").normal_(0.0, 1e-3)
    p = torch.zeros(8, device="cuda")
    plan = eng.Plan([eng.TensorDesc(g, g)])
    plan.grad_norm()
    want, _ = plan.read_norm()
    rc = lib().oe_grad_norm_static(0, g.data_ptr(), numel, out.data_ptr(), stream)
    assert rc == 0, lib().oe_last_error()
    torch.cuda.synchronize()
    got = float(out.item())
    exact = 0.0
    for a in range(0, numel, 1 << 26):
        exact += float(g[a:a + (1 << 26)].double().pow(2).sum().item())
    exact = exact ** 0.5
    assert abs(got - want) <= 1e-6 * want and abs(got - exact) <= 1e-6 * exact, (got, want, exact)
    plan.close()
    del g, p
    # an empty buffer has norm 0; the address is not read
    rc = lib().oe_grad_norm_static(0, 0, 0, out.data_ptr(), stream)
    assert rc == 0, lib().oe_last_error()
    torch.cuda.synchronize()
    assert float(out.item()) == 0.0
    # beyond the fixed array's capacity: refused with a message, nothing launched, output untouched
    out.fill_(7.0)
    rc = lib().oe_grad_norm_static(0, out.data_ptr(), (1 << 31) + 1, out.data_ptr(), stream)
    assert rc == OE_ERR_LIMIT
    assert b"maximum" in lib().oe_last_error()
    torch.cuda.synchronize()
    assert float(out.item()) == 7.0
