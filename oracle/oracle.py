"""ctypes front-end of the CPU oracle (test infrastructure, never shipped).

The arithmetic lives in ``optim_oracle.c``; this module only carries the host-side
control flow of the reference's CPU optimizers — which parameters are skipped,
when the step counter moves, how groups scale the rate — so that a test can drive
the oracle the way the reference's own tests drive ``AdamW``/``SGD``:

* ``OracleAdamW.step``      follows ``AdamW.Step``      (autograd/nn.go:492-531)
* ``OracleSGD.step``        follows ``SGD.Step``        (autograd/sgd.go:178-225)
* ``clip_grad_norm``        follows ``ClipGradNorm``    (autograd/nn.go:318-333)
* ``f32_to_bf16``           follows ``f32_to_bf16``     (autograd/cuda_kernels.go:86)

Only tests, the smoke check and the benchmark's CPU-baseline leg import this.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboptim_oracle.so")


def build(force: bool = False) -> str:
    """Compile the C restatement with the committed Makefile; returns the library path."""
    src = os.path.join(_HERE, "optim_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True, stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None
_f32p = C.POINTER(C.c_float)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        f, sz, i, i64 = C.c_float, C.c_size_t, C.c_int, C.c_int64
        _lib.oracle_bias_corrections.argtypes = [f, f, i64, _f32p, _f32p]
        _lib.oracle_normalize_lr_scale.argtypes = [f]
        _lib.oracle_normalize_lr_scale.restype = f
        _lib.oracle_adamw_group_scale.argtypes = [f, f, f, _f32p, _f32p]
        _lib.oracle_sgd_group_scale.argtypes = [f, f, f, _f32p, _f32p]
        _lib.oracle_adamw_update.argtypes = [_f32p, _f32p, _f32p, _f32p, sz, f, f, f, f, f, f, f]
        _lib.oracle_adamw_update_parallel.argtypes = [_f32p, _f32p, _f32p, _f32p, sz, f, f, f, f, f, f, f, i]
        _lib.oracle_adamw_update_devform.argtypes = [_f32p, _f32p, _f32p, _f32p, sz, f, f, f, f, f, f, f, f]
        _lib.oracle_parallel_workers.argtypes = [sz, i]
        _lib.oracle_parallel_workers.restype = i
        _lib.oracle_sgd_update.argtypes = [_f32p, _f32p, _f32p, sz, i, f, f, f, f, i, i]
        _lib.oracle_sum_squares.argtypes = [C.POINTER(_f32p), C.POINTER(sz), sz]
        _lib.oracle_sum_squares.restype = C.c_double
        _lib.oracle_clip_coefficient.argtypes = [f, f]
        _lib.oracle_clip_coefficient.restype = f
        _lib.oracle_clip_coefficient_devform.argtypes = [f, f]
        _lib.oracle_clip_coefficient_devform.restype = f
        _lib.oracle_clip_grad_norm.argtypes = [C.POINTER(_f32p), C.POINTER(sz), sz, f, _f32p]
        _lib.oracle_clip_grad_norm.restype = f
        _lib.oracle_scale.argtypes = [_f32p, sz, f]
        _lib.oracle_f32_to_bf16.argtypes = [_f32p, C.POINTER(C.c_uint16), sz, i]
        _lib.oracle_f32_to_bf16_one.argtypes = [f, i]
        _lib.oracle_f32_to_bf16_one.restype = C.c_uint16
        _lib.oracle_first_invalid_moment.argtypes = [_f32p, _f32p, sz]
        _lib.oracle_first_invalid_moment.restype = sz
    return _lib


def _ptr(a: Optional[np.ndarray]):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"], "oracle arrays are contiguous float32"
    return a.ctypes.data_as(_f32p)


def bias_corrections(beta1: float, beta2: float, t: int):
    a, b = C.c_float(), C.c_float()
    lib().oracle_bias_corrections(beta1, beta2, t, C.byref(a), C.byref(b))
    return np.float32(a.value), np.float32(b.value)


@dataclass
class Group:
    """One resolved parameter group (autograd/param_groups.go:30-35)."""
    name: str
    indexes: List[int]
    lr_scale: float = 1.0
    weight_decay: float = 0.0


def resolve_groups(n_params: int, groups: Optional[Sequence[Group]], base_decay: float = 0.0):
    """Owner index per parameter; no groups = one default group (param_groups.go:104-111)."""
    if not groups:
        return [Group("default", list(range(n_params)), 1.0, base_decay)], [0] * n_params
    owner = [-1] * n_params
    out = []
    for gi, g in enumerate(groups):
        scale = float(lib().oracle_normalize_lr_scale(g.lr_scale))
        out.append(Group(g.name, list(g.indexes), scale, g.weight_decay))
        for i in g.indexes:
            assert owner[i] < 0, "parameter in two groups"
            owner[i] = gi
    assert all(o >= 0 for o in owner), "parameter in no group"
    return out, owner


@dataclass
class OracleAdamW:
    """Host control flow of AdamW.Step, CPU branch (autograd/nn.go:487-531)."""
    params: List[np.ndarray]
    lr: float
    weight_decay: float = 0.0
    groups: Optional[Sequence[Group]] = None
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    max_procs: int = 1
    step_count: int = 0
    m: List[np.ndarray] = field(default_factory=list)
    v: List[np.ndarray] = field(default_factory=list)

    def __post_init__(self):
        self._groups, self._owner = resolve_groups(len(self.params), self.groups, self.weight_decay)
        if not self.m:
            self.m = [np.zeros(p.size, np.float32) for p in self.params]
            self.v = [np.zeros(p.size, np.float32) for p in self.params]

    def group_scale(self, n: int):
        g = self._groups[self._owner[n]]
        s, d = C.c_float(), C.c_float()
        lib().oracle_adamw_group_scale(self.lr, g.lr_scale, g.weight_decay, C.byref(s), C.byref(d))
        return s.value, d.value

    def step(self, grads: Sequence[Optional[np.ndarray]]):
        """grads[i] None or empty = the parameter is skipped; the counter is shared."""
        self.step_count += 1
        a, b = C.c_float(), C.c_float()
        lib().oracle_bias_corrections(self.beta1, self.beta2, self.step_count, C.byref(a), C.byref(b))
        for n, p in enumerate(self.params):
            g = grads[n]
            if g is None or g.size == 0:
                continue
            assert g.size == p.size
            step, decay = self.group_scale(n)
            lib().oracle_adamw_update_parallel(_ptr(p.reshape(-1)), _ptr(g.reshape(-1)), _ptr(self.m[n]),
                                               _ptr(self.v[n]), p.size, self.beta1, self.beta2, self.eps, step,
                                               decay, a.value, b.value, self.max_procs)


@dataclass
class OracleSGD:
    """Host control flow of SGD.Step, CPU loop (autograd/sgd.go:178-225)."""
    params: List[np.ndarray]
    lr: float
    momentum: float = 0.0
    dampening: float = 0.0
    weight_decay: float = 0.0
    nesterov: bool = False
    maximize: bool = False
    groups: Optional[Sequence[Group]] = None
    step_count: int = 0

    def __post_init__(self):
        self._groups, self._owner = resolve_groups(len(self.params), self.groups, self.weight_decay)
        self.buffers: List[Optional[np.ndarray]] = [None] * len(self.params)
        self.initialized = [False] * len(self.params)

    def group_scale(self, n: int):
        g = self._groups[self._owner[n]]
        s, d = C.c_float(), C.c_float()
        lib().oracle_sgd_group_scale(self.lr, g.lr_scale, g.weight_decay, C.byref(s), C.byref(d))
        return s.value, d.value

    def step(self, grads: Sequence[Optional[np.ndarray]]):
        """grads[i] None = skipped and left uninitialised; an all-zero gradient updates."""
        self.step_count += 1
        for n, p in enumerate(self.params):
            g = grads[n]
            if g is None:
                continue
            assert g.size == p.size
            first = not self.initialized[n]
            lr, decay = self.group_scale(n)
            if self.momentum > 0 and first:
                self.buffers[n] = np.zeros(p.size, np.float32)
            lib().oracle_sgd_update(_ptr(p.reshape(-1)), _ptr(g.reshape(-1)), _ptr(self.buffers[n]), p.size,
                                    int(first), lr, self.momentum, self.dampening, decay, int(self.nesterov),
                                    int(self.maximize))
            if self.momentum > 0:
                self.initialized[n] = True


def _grad_table(grads: Sequence[Optional[np.ndarray]]):
    present = [g.reshape(-1) for g in grads if g is not None and g.size > 0]
    ptrs = (_f32p * max(len(present), 1))(*[_ptr(g) for g in present])
    sizes = (C.c_size_t * max(len(present), 1))(*[g.size for g in present])
    return present, ptrs, sizes


def sum_squares(grads: Sequence[Optional[np.ndarray]]) -> float:
    present, ptrs, sizes = _grad_table(grads)
    return float(lib().oracle_sum_squares(ptrs, sizes, len(present)))


def clip_grad_norm(grads: Sequence[Optional[np.ndarray]], max_norm: float):
    """In-place clip; returns (pre-clip norm as float32, scale applied)."""
    present, ptrs, sizes = _grad_table(grads)
    scale = C.c_float(1.0)
    norm = lib().oracle_clip_grad_norm(ptrs, sizes, len(present), max_norm, C.byref(scale))
    return np.float32(norm), np.float32(scale.value)


def clip_coefficient(norm: float, max_norm: float, devform: bool = False) -> np.float32:
    fn = lib().oracle_clip_coefficient_devform if devform else lib().oracle_clip_coefficient
    return np.float32(fn(norm, max_norm))


def scale_(g: np.ndarray, scale: float) -> None:
    lib().oracle_scale(_ptr(g.reshape(-1)), g.size, scale)


def f32_to_bf16(x: np.ndarray, nan_canonical: bool = True) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    y = np.empty(x.size, np.uint16)
    lib().oracle_f32_to_bf16(_ptr(x), y.ctypes.data_as(C.POINTER(C.c_uint16)), x.size, int(nan_canonical))
    return y


def adamw_update_devform(p, g, m, v, norm, b1, b2, step_over_bc1, bc2, decay, eps, max_norm):
    lib().oracle_adamw_update_devform(_ptr(p), _ptr(g), _ptr(m), _ptr(v), p.size, norm, b1, b2, step_over_bc1,
                                      bc2, decay, eps, max_norm)


def first_invalid_moment(m: np.ndarray, v: np.ndarray) -> int:
    return int(lib().oracle_first_invalid_moment(_ptr(m), _ptr(v), m.size))
