"""Device-resident synthetic state for a ParamSet (torch is the allocator and the RNG)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .engine import TensorDesc
from .paramsets import ParamSet


@dataclass
class DeviceState:
    ps: ParamSet
    device: torch.device
    p: List[torch.Tensor]
    g: List[Optional[torch.Tensor]]
    s1: List[Optional[torch.Tensor]]   # AdamW m | SGD momentum buffer
    s2: List[Optional[torch.Tensor]]   # AdamW v | SGD init flag (1 float)
    shadow: List[Optional[torch.Tensor]]

    def descs(self) -> List[TensorDesc]:
        out = []
        for i, spec in enumerate(self.ps.params):
            grp = self.ps.group_of(spec.group)
            out.append(TensorDesc(self.p[i], self.g[i], self.s1[i], self.s2[i], self.shadow[i], grp.lr_scale,
                                  grp.weight_decay))
        return out

    @property
    def numel(self) -> int:
        return sum(int(t.numel()) for t in self.p)


def init_weight(spec, gen: torch.Generator, device) -> torch.Tensor:
    n = spec.numel
    if spec.init == "zeros":
        return torch.zeros(n, dtype=torch.float32, device=device)
    if spec.init == "ones":
        return torch.ones(n, dtype=torch.float32, device=device)
    if spec.init == "uniform":
        return (torch.rand(n, dtype=torch.float32, device=device, generator=gen) * 2 - 1) * spec.init_scale
    return torch.randn(n, dtype=torch.float32, device=device, generator=gen) * spec.init_scale


def boosted_indices(ps: ParamSet) -> List[int]:
    """Tensors whose gradients are scaled x100 so that clipping triggers (seeded shuffle)."""
    if ps.boosted_fraction <= 0:
        return []
    k = max(1, round(ps.boosted_fraction * len(ps.params)))
    g = torch.Generator().manual_seed(ps.grad_seed + 1000)
    return sorted(torch.randperm(len(ps.params), generator=g)[:k].tolist())


def fill_grads(state: DeviceState, step: int) -> None:
    """Fresh gradients ~ N(0, grad_std^2) for one step, seeded by (grad_seed, step)."""
    gen = torch.Generator(device=state.device).manual_seed(state.ps.grad_seed * 1_000_003 + step)
    boosted = set(boosted_indices(state.ps))
    for i, g in enumerate(state.g):
        if g is None:
            continue
        g.normal_(0.0, state.ps.grad_std, generator=gen)
        if i in boosted:
            g.mul_(100.0)


def materialize(ps: ParamSet, device="cuda:0", weight_seed: int = 1234, with_grads: bool = True) -> DeviceState:
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(weight_seed)
    p = [init_weight(s, gen, device) for s in ps.params]
    g = [torch.zeros_like(t) if with_grads else None for t in p]
    if ps.optimizer == "adamw":
        s1 = [torch.zeros_like(t) for t in p]
        s2 = [torch.zeros_like(t) for t in p]
    else:
        use_momentum = ps.hparams.get("momentum", 0.0) > 0
        s1 = [torch.zeros_like(t) if use_momentum else None for t in p]
        s2 = [torch.zeros(1, dtype=torch.float32, device=device) if use_momentum else None for t in p]
    shadow = [torch.zeros(t.numel(), dtype=torch.bfloat16, device=device) if ps.bf16_shadow else None for t in p]
    state = DeviceState(ps, device, p, g, s1, s2, shadow)
    if with_grads:
        fill_grads(state, 0)
    return state


def bias_corrections(beta1: float, beta2: float, step: int):
    """float32(1 - pow(float64(beta), float64(step))) with beta first rounded to float32,
    as the optimizer's host code computes it before every step."""
    import numpy as np
    b1, b2 = float(np.float32(beta1)), float(np.float32(beta2))
    return float(np.float32(1.0 - b1 ** step)), float(np.float32(1.0 - b2 ** step))
