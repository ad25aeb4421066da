"""The five synthetic parameter sets the engine is measured and checked on.

Each set is a list of named fp32 tensors with the shapes of a model family (no model
code: the optimizer step only sees flat tensors), the parameter groups, the
hyper-parameters and the gradient distribution. Weights and gradients are seeded
random values of the stated distributions; they stand in for real training state.

    mlp     2-layer MLP, AdamW, 100 steps, no clip, no shadow          203,530 params
    cnn     small CNN, SGD momentum .9 wd 5e-4, 200 steps              114,186 params
    gpt     GPT-style 12x768, AdamW + clip 1.0 + bf16, two groups  109,630,464 params
    llama1b Llama-style 24x2048, AdamW + clip + bf16             1,345,423,360 params
    llama8b Llama-3-8B shapes, sharded AdamW + clip + bf16       8,030,261,248 params
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Tuple


@dataclass
class ParamSpec:
    name: str
    shape: Tuple[int, ...]
    group: str = "default"
    init: str = "normal"      # "normal" | "uniform" | "zeros" | "ones"
    init_scale: float = 0.02  # std for normal, bound for uniform

    @property
    def numel(self) -> int:
        return int(math.prod(self.shape))


@dataclass
class GroupSpec:
    name: str
    lr_scale: float = 1.0
    weight_decay: float = 0.0


@dataclass
class ParamSet:
    key: str
    title: str
    optimizer: str                     # "adamw" | "sgd"
    params: List[ParamSpec]
    groups: List[GroupSpec]
    hparams: Dict[str, float]
    grad_std: float
    grad_seed: int
    steps: int
    max_norm: float = 0.0              # 0 = no clipping
    bf16_shadow: bool = False
    boosted_fraction: float = 0.0      # share of tensors whose gradient is scaled x100
    notes: str = ""
    extra: Dict[str, object] = field(default_factory=dict)

    @property
    def numel(self) -> int:
        return sum(p.numel for p in self.params)

    def group_of(self, name: str) -> GroupSpec:
        return next(g for g in self.groups if g.name == name)


def _uniform_fan_in(name, shape, fan_in, group="default"):
    return ParamSpec(name, shape, group, "uniform", 1.0 / math.sqrt(fan_in))


def mlp() -> ParamSet:
    params = [
        _uniform_fan_in("fc1.weight", (784, 256), 784),
        ParamSpec("fc1.bias", (256,), init="zeros"),
        _uniform_fan_in("fc2.weight", (256, 10), 256),
        ParamSpec("fc2.bias", (10,), init="zeros"),
    ]
    return ParamSet("mlp", "AdamW on a 2-layer MLP parameter set", "adamw", params,
                    [GroupSpec("default", 1.0, 0.01)],
                    dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8), grad_std=0.01, grad_seed=0, steps=100)


def cnn() -> ParamSet:
    params = []
    cin = 3
    for i, cout in enumerate((32, 64, 128)):
        fan_in = cin * 9
        params.append(_uniform_fan_in(f"conv{i + 1}.weight", (cout, cin, 3, 3), fan_in))
        params.append(_uniform_fan_in(f"conv{i + 1}.bias", (cout,), fan_in))
        params.append(ParamSpec(f"bn{i + 1}.gamma", (cout,), init="ones"))
        params.append(ParamSpec(f"bn{i + 1}.beta", (cout,), init="zeros"))
        cin = cout
    params.append(_uniform_fan_in("fc.weight", (10, 2048), 2048))
    params.append(_uniform_fan_in("fc.bias", (10,), 2048))
    return ParamSet("cnn", "SGD with momentum over a small CNN parameter set", "sgd", params,
                    [GroupSpec("default", 1.0, 5e-4)],
                    dict(lr=0.05, momentum=0.9, dampening=0.0, nesterov=0, maximize=0),
                    grad_std=0.02, grad_seed=1, steps=200)


def gpt() -> ParamSet:
    d, layers, ffn, vocab = 768, 12, 3072, 32000
    params = [ParamSpec("embedding.weight", (vocab, d), "decay")]  # tied: one tensor serves both ends
    for l in range(layers):
        pre = f"layers.{l}."
        params += [
            ParamSpec(pre + "attn.qkv.weight", (3 * d, d), "decay"), ParamSpec(pre + "attn.qkv.bias", (3 * d,), "no_decay", "zeros"),
            ParamSpec(pre + "attn.out.weight", (d, d), "decay"), ParamSpec(pre + "attn.out.bias", (d,), "no_decay", "zeros"),
            ParamSpec(pre + "ln1.gamma", (d,), "no_decay", "ones"), ParamSpec(pre + "ln1.beta", (d,), "no_decay", "zeros"),
            ParamSpec(pre + "mlp.fc1.weight", (ffn, d), "decay"), ParamSpec(pre + "mlp.fc1.bias", (ffn,), "no_decay", "zeros"),
            ParamSpec(pre + "mlp.fc2.weight", (d, ffn), "decay"), ParamSpec(pre + "mlp.fc2.bias", (d,), "no_decay", "zeros"),
            ParamSpec(pre + "ln2.gamma", (d,), "no_decay", "ones"), ParamSpec(pre + "ln2.beta", (d,), "no_decay", "zeros"),
        ]
    return ParamSet("gpt", "AdamW + clip + bf16 shadow over a GPT-style parameter set", "adamw", params,
                    [GroupSpec("decay", 1.0, 0.1), GroupSpec("no_decay", 1.0, 0.0)],
                    dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8), grad_std=0.01, grad_seed=2, steps=50,
                    max_norm=1.0, bf16_shadow=True, boosted_fraction=0.02,
                    notes="tied embedding; 109,630,464 parameters from the listed tensors")


def gpt_sgd() -> ParamSet:
    """The GPT-style tensors under SGD with momentum: a mid-size streaming case of the SGD kernel
    (larger than L2, small enough to profile), not one of the reference's configurations."""
    base = gpt()
    return ParamSet("gpt_sgd", "SGD with momentum over the GPT-style parameter set", "sgd", base.params,
                    [GroupSpec("decay", 1.0, 5e-4), GroupSpec("no_decay", 1.0, 0.0)],
                    dict(lr=0.05, momentum=0.9, dampening=0.0, nesterov=0, maximize=0),
                    grad_std=0.01, grad_seed=5, steps=50)


def _llama(key, title, d, layers, kv_dim, ffn, vocab, seed, steps, beta2):
    params = [ParamSpec("embed_tokens.weight", (vocab, d))]
    for l in range(layers):
        pre = f"layers.{l}."
        params += [
            ParamSpec(pre + "attn.q.weight", (d, d)), ParamSpec(pre + "attn.k.weight", (kv_dim, d)),
            ParamSpec(pre + "attn.v.weight", (kv_dim, d)), ParamSpec(pre + "attn.o.weight", (d, d)),
            ParamSpec(pre + "mlp.gate.weight", (ffn, d)), ParamSpec(pre + "mlp.up.weight", (ffn, d)),
            ParamSpec(pre + "mlp.down.weight", (d, ffn)),
            ParamSpec(pre + "input_norm.weight", (d,), init="ones"), ParamSpec(pre + "post_norm.weight", (d,), init="ones"),
        ]
    params += [ParamSpec("norm.weight", (d,), init="ones"), ParamSpec("lm_head.weight", (vocab, d))]
    return ParamSet(key, title, "adamw", params, [GroupSpec("default", 1.0, 0.1)],
                    dict(lr=1e-4, beta1=0.9, beta2=beta2, eps=1e-8), grad_std=1e-3, grad_seed=seed, steps=steps,
                    max_norm=1.0, bf16_shadow=True, notes="untied embedding and lm_head plus the final norm")


def llama1b() -> ParamSet:
    return _llama("llama1b", "AdamW + clip + bf16 shadow over a Llama-style 1.3B parameter set",
                  2048, 24, 2048, 5504, 32000, seed=3, steps=20, beta2=0.999)


def llama8b() -> ParamSet:
    return _llama("llama8b", "Sharded AdamW + clip + bf16 shadow over a Llama-3-8B-shaped parameter set",
                  4096, 32, 1024, 14336, 128256, seed=4, steps=10, beta2=0.95)


REGISTRY = {"mlp": mlp, "cnn": cnn, "gpt": gpt, "gpt_sgd": gpt_sgd, "llama1b": llama1b, "llama8b": llama8b}
EXPECTED_NUMEL = {"mlp": 203_530, "cnn": 114_186, "gpt": 109_630_464, "gpt_sgd": 109_630_464, "llama1b": 1_345_423_360,
                  "llama8b": 8_030_261_248}


def get(key: str) -> ParamSet:
    return REGISTRY[key]()


def scaled(ps: ParamSet, max_numel: int) -> ParamSet:
    """The leading tensors of a set up to max_numel elements (always at least one tensor):
    a bounded sample with the same tensor shapes, used for CPU timing and small GPU cases."""
    keep, total = [], 0
    for p in ps.params:
        if keep and total + p.numel > max_numel:
            break
        keep.append(p)
        total += p.numel
    out = ParamSet(**{**ps.__dict__})
    out.params = keep
    return out
