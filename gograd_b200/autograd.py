"""ctypes binding of libgograd_host.so: the C++ host mirror of gograd's optimizer surface.

Names follow the reference (``NewAdamW``, ``NewSGDGroups``, ``ClipGradNorm``, ...). All logic
lives in C++ (gograd_b200/csrc/host); this file only marshals arguments. Errors — the
mirror's counterpart of a Go error value or panic — raise ``HostError``.
"""
from __future__ import annotations

import ctypes as C
import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libgograd_host.so")
_lib = None
_f32p = C.POINTER(C.c_float)


class HostError(RuntimeError):
    pass


class _SGDOptions(C.Structure):
    _fields_ = [("lr", C.c_float), ("momentum", C.c_float), ("dampening", C.c_float), ("weight_decay", C.c_float),
                ("nesterov", C.c_int32), ("maximize", C.c_int32)]


class _OneCycle(C.Structure):
    _fields_ = [("max_lr", C.c_double), ("pct_start", C.c_double), ("div_factor", C.c_double),
                ("final_div_factor", C.c_double), ("total", C.c_int32), ("step_count", C.c_int32)]


class _Accumulator(C.Structure):
    _fields_ = [("groups", C.c_int32), ("pending", C.c_int32)]


class _Groups(C.Structure):
    _fields_ = [("n_groups", C.c_int32), ("group_names", C.POINTER(C.c_char_p)), ("offsets", C.POINTER(C.c_int32)),
                ("members", C.POINTER(C.c_int32)), ("lr_scales", _f32p), ("decays", _f32p)]


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `make -C gograd_b200/csrc`")
        from . import _lib as engine_lib
        engine_lib.lib()  # liboptengine.so first (the host library links against it)
        h = C.CDLL(LIB_PATH)
        h.gg_last_error.restype = C.c_char_p
        h.gg_tensor_numel.restype = C.c_int64
        h.gg_opt_step_count.restype = C.c_int64
        h.gg_tensor_address.restype = C.c_uint64
        h.gg_tensor_shadow_lease.restype = C.c_uint64
        h.gg_tensor_shadow_release.restype = None
        h.gg_tensor_shadow_release.argtypes = [C.c_void_p, C.c_uint64]
        h.gg_tensor_free.restype = None
        h.gg_opt_free.restype = None
        h.gg_release_clip_state.restype = None
        h.gg_accumulator_reset.restype = None
        h.gg_state_stream_abort.restype = None
        h.gg_state_stream_abort.argtypes = [C.c_void_p]
        h.gg_state_stream_finish.argtypes = [C.c_void_p]
        h.gg_state_stream_next.argtypes = [C.c_void_p, C.c_char_p, C.c_int32, C.POINTER(C.c_int64)]
        h.gg_state_stream_append.argtypes = [C.c_void_p, C.c_char_p, _f32p, C.c_int64]
        _lib = h
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise HostError(lib().gg_last_error().decode("utf-8", "replace"))


def _f(x: float):
    return C.byref(C.c_float(x))


class Tensor:
    """A contiguous float32 CUDA leaf (autograd.Tensor as the optimizer path sees it)."""

    def __init__(self, values, shape: Optional[Sequence[int]] = None, device: int = 0, requires_grad: bool = True):
        v = np.ascontiguousarray(values, np.float32).reshape(-1)
        shape = list(shape) if shape is not None else [v.size]
        self.shape = shape
        self._h = C.c_void_p()
        arr = (C.c_int32 * max(len(shape), 1))(*shape)
        _check(lib().gg_tensor_new(v.ctypes.data_as(_f32p), arr, len(shape), device, int(requires_grad), C.byref(self._h)))

    @property
    def numel(self) -> int:
        return int(lib().gg_tensor_numel(self._h))

    def to_host(self) -> np.ndarray:
        out = np.empty(self.numel, np.float32)
        _check(lib().gg_tensor_to_host(self._h, out.ctypes.data_as(C.c_void_p)))
        return out

    def copy_from_host(self, values) -> None:
        v = np.ascontiguousarray(values, np.float32).reshape(-1)
        assert v.size == self.numel
        _check(lib().gg_tensor_copy_from_host(self._h, v.ctypes.data_as(C.c_void_p)))

    @property
    def has_grad(self) -> bool:
        return bool(lib().gg_tensor_has_grad(self._h))

    @property
    def grad_known_zero(self) -> bool:
        return bool(lib().gg_tensor_grad_known_zero(self._h))

    def set_grad(self, values) -> None:
        """None makes the gradient absent (a nil gradBuf)."""
        if values is None:
            _check(lib().gg_tensor_set_grad(self._h, None))
            return
        v = np.ascontiguousarray(values, np.float32).reshape(-1)
        assert v.size == self.numel
        _check(lib().gg_tensor_set_grad(self._h, v.ctypes.data_as(C.c_void_p)))

    def ensure_grad(self) -> None:
        _check(lib().gg_tensor_ensure_grad(self._h))

    def grad_to_host(self) -> np.ndarray:
        out = np.empty(self.numel, np.float32)
        _check(lib().gg_tensor_grad_to_host(self._h, out.ctypes.data_as(C.c_void_p)))
        return out

    def shadow_to_host(self) -> np.ndarray:
        out = np.empty(self.numel, np.uint16)
        _check(lib().gg_tensor_shadow_to_host(self._h, out.ctypes.data_as(C.c_void_p)))
        return out

    @property
    def shadow_current(self) -> bool:
        return bool(lib().gg_tensor_shadow_current(self._h))

    def address(self, which: int = 0) -> int:
        return int(lib().gg_tensor_address(self._h, which))

    def shadow_lease(self) -> int:
        """Takes a lease on the current bf16 shadow and returns its device address."""
        return int(lib().gg_tensor_shadow_lease(self._h))

    def shadow_release(self, address: int) -> None:
        lib().gg_tensor_shadow_release(self._h, address)

    @property
    def leased_shadows(self) -> int:
        return int(lib().gg_tensor_leased_shadows(self._h))

    def close(self) -> None:
        if self._h:
            lib().gg_tensor_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


@dataclass
class Parameter:
    Name: str
    Value: Optional[Tensor]


@dataclass
class ParameterGroupSpec:
    Name: str
    Params: List[Parameter]
    LRScale: float = 0.0
    WeightDecay: float = 0.0


@dataclass
class SGDOptions:
    LR: float = 0.0
    Momentum: float = 0.0
    Dampening: float = 0.0
    WeightDecay: float = 0.0
    Nesterov: bool = False
    Maximize: bool = False

    def to_c(self) -> _SGDOptions:
        return _SGDOptions(self.LR, self.Momentum, self.Dampening, self.WeightDecay, int(self.Nesterov), int(self.Maximize))


def _param_arrays(params: Sequence[Parameter]):
    n = len(params)
    names = (C.c_char_p * max(n, 1))(*[p.Name.encode() for p in params])
    handles = (C.c_void_p * max(n, 1))(*[(p.Value._h if p.Value is not None else None) for p in params])
    return names, handles, n


def _groups_struct(params: Sequence[Parameter], specs: Sequence[ParameterGroupSpec]):
    index_of = {id(p.Value): i for i, p in enumerate(params) if p.Value is not None}
    names = (C.c_char_p * max(len(specs), 1))(*[s.Name.encode() for s in specs])
    offsets, members = [0], []
    for s in specs:
        for p in s.Params:
            members.append(index_of.get(id(p.Value), -1))  # -1: a tensor the optimizer does not own
        offsets.append(len(members))
    off = (C.c_int32 * len(offsets))(*offsets)
    mem = (C.c_int32 * max(len(members), 1))(*members)
    scales = (C.c_float * max(len(specs), 1))(*[s.LRScale for s in specs])
    decays = (C.c_float * max(len(specs), 1))(*[s.WeightDecay for s in specs])
    g = _Groups(len(specs), names, off, mem, scales, decays)
    g._keep = (names, off, mem, scales, decays)
    return g


class _Optimizer:
    def __init__(self, handle, params):
        self._h = handle
        self.Params = list(params)

    def Step(self) -> None:
        _check(lib().gg_opt_step(self._h))

    def StepClipped(self, max_norm: float) -> None:
        _check(lib().gg_opt_step_clipped(self._h, _f(max_norm)))

    def LastGradNorm(self) -> float:
        out = C.c_float()
        _check(lib().gg_opt_last_norm(self._h, C.byref(out)))
        return out.value

    def ZeroGrad(self) -> None:
        _check(lib().gg_opt_zero_grad(self._h))

    def LearningRate(self) -> float:
        out = C.c_float()
        _check(lib().gg_opt_get_lr(self._h, C.byref(out)))
        return out.value

    def SetLearningRate(self, lr: float) -> None:
        _check(lib().gg_opt_set_lr(self._h, _f(lr)))

    @property
    def StepCount(self) -> int:
        return int(lib().gg_opt_step_count(self._h))

    def SetEngine(self, write_shadow: bool = False, clip_devform: bool = False) -> None:
        _check(lib().gg_opt_set_engine(self._h, int(write_shadow), int(clip_devform)))

    def SetZeroGradInStep(self, on: bool = True) -> None:
        """AdamW only: Step stores zeros over the gradients it reads; ZeroGrad then has nothing to launch."""
        _check(lib().gg_opt_set_zero_grad_in_step(self._h, int(on)))

    def SetGradScale(self, scale: float) -> None:
        """Step and StepClipped read every gradient element as float32(g * scale) from now on."""
        _check(lib().gg_opt_set_grad_scale(self._h, _f(scale)))

    def groupScale(self, index: int):
        a, b = C.c_float(), C.c_float()
        _check(lib().gg_opt_group_scale(self._h, index, C.byref(a), C.byref(b)))
        return np.float32(a.value), np.float32(b.value)

    def _state(self, index: int, which: int):
        n = self.Params[index].Value.numel
        out = np.zeros(n, np.float32)
        flag = C.c_int32()
        _check(lib().gg_opt_state(self._h, index, which, out.ctypes.data_as(_f32p), C.byref(flag)))
        return out, bool(flag.value)

    def SaveSafeTensors(self, path: str) -> None:
        _check(lib().gg_opt_save(self._h, path.encode()))

    def LoadSafeTensors(self, path: str) -> None:
        _check(lib().gg_opt_load(self._h, path.encode()))

    def Close(self) -> None:
        _check(lib().gg_opt_close(self._h))

    def __del__(self):
        try:
            if self._h:
                lib().gg_opt_free(self._h)
                self._h = None
        except Exception:
            pass


class AdamW(_Optimizer):
    def M(self, index: int) -> np.ndarray:
        return self._state(index, 0)[0]

    def V(self, index: int) -> np.ndarray:
        return self._state(index, 1)[0]

    def SetConfig(self, beta1: Optional[float] = None, beta2: Optional[float] = None, eps: Optional[float] = None):
        _check(lib().gg_adamw_set_config(self._h, None if beta1 is None else _f(beta1),
                                         None if beta2 is None else _f(beta2), None if eps is None else _f(eps)))

    def PrepareGraph(self) -> None:
        _check(lib().gg_adamw_prepare_graph(self._h))

    def StepCaptured(self) -> None:
        _check(lib().gg_adamw_step_captured(self._h))

    def GraphStepCount(self) -> int:
        out = C.c_int32()
        _check(lib().gg_adamw_graph_step_count(self._h, C.byref(out)))
        return out.value


class SGD(_Optimizer):
    def Buffer(self, index: int):
        """(momentum buffer, initialised flag) of one parameter."""
        return self._state(index, 2)

    def PrepareGraph(self) -> None:
        _check(lib().gg_opt_prepare_graph(self._h))

    def StepCaptured(self) -> None:
        _check(lib().gg_opt_step_captured(self._h))

    def GraphStepCount(self) -> int:
        out = C.c_int32()
        _check(lib().gg_opt_graph_step_count(self._h, C.byref(out)))
        return out.value


def NewAdamW(params: Sequence[Parameter], lr: float, decay: float) -> AdamW:
    names, handles, n = _param_arrays(params)
    h = C.c_void_p()
    _check(lib().gg_adamw_new(names, handles, n, _f(lr), _f(decay), C.byref(h)))
    return AdamW(h, params)


def NewAdamWGroups(params: Sequence[Parameter], lr: float, specs: Sequence[ParameterGroupSpec]) -> AdamW:
    names, handles, n = _param_arrays(params)
    g = _groups_struct(params, specs)
    h = C.c_void_p()
    _check(lib().gg_adamw_new_groups(names, handles, n, _f(lr), C.byref(g), C.byref(h)))
    return AdamW(h, params)


def NewSGD(params: Sequence[Parameter], options: SGDOptions) -> SGD:
    names, handles, n = _param_arrays(params)
    o = options.to_c()
    h = C.c_void_p()
    _check(lib().gg_sgd_new(names, handles, n, C.byref(o), C.byref(h)))
    return SGD(h, params)


def NewSGDGroups(params: Sequence[Parameter], options: SGDOptions, specs: Sequence[ParameterGroupSpec]) -> SGD:
    names, handles, n = _param_arrays(params)
    g = _groups_struct(params, specs)
    o = options.to_c()
    h = C.c_void_p()
    _check(lib().gg_sgd_new_groups(names, handles, n, C.byref(o), C.byref(g), C.byref(h)))
    return SGD(h, params)


def PartitionParameters(params: Sequence[Parameter], assign) -> List[ParameterGroupSpec]:
    """One spec per label returned by assign(name), in order of first appearance."""
    names, handles, n = _param_arrays(params)
    labels = (C.c_char_p * max(n, 1))(*[(assign(p.Name) or "").encode() for p in params])
    buf = C.create_string_buffer(1 << 16)
    _check(lib().gg_partition_parameters(names, handles, labels, n, buf, len(buf)))
    by_name = {p.Name: p for p in params}
    return [ParameterGroupSpec(g["Name"], [by_name[x] for x in g["Params"]]) for g in json.loads(buf.value.decode())]


def ClipGradNorm(params: Sequence[Parameter], max_norm: float) -> float:
    """Scales the present gradients in place on the device; returns NaN like the reference
    (the norm stays on the device, read it with GradientNormToHost)."""
    handles = (C.c_void_p * max(len(params), 1))(*[p.Value._h for p in params])
    _check(lib().gg_clip_grad_norm(handles, len(params), _f(max_norm)))
    return float("nan")


def GradientNormToHost() -> float:
    out = C.c_float()
    _check(lib().gg_gradient_norm_to_host(C.byref(out)))
    return out.value


def ReleaseClipState() -> None:
    lib().gg_release_clip_state()


class GradAccumulator:
    """The bookkeeping of autograd.GradAccumulator (autograd/accumulate.go:15-71)."""

    def __init__(self, groups: int):
        self._a = _Accumulator()
        _check(lib().gg_accumulator_new(groups, C.byref(self._a)))

    def MicroBatch(self):
        """What Backward does around the differentiation: (seed 1/groups, group complete?)."""
        seed, done = C.c_float(), C.c_int32()
        _check(lib().gg_accumulator_micro_batch(C.byref(self._a), C.byref(seed), C.byref(done)))
        return np.float32(seed.value), bool(done.value)

    def Pending(self) -> int:
        return self._a.pending

    def Groups(self) -> int:
        return self._a.groups

    def Reset(self) -> None:
        lib().gg_accumulator_reset(C.byref(self._a))


class _TrainingLoop(C.Structure):
    NEXT = C.CFUNCTYPE(C.c_int, C.c_void_p)
    POSITION = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_char), C.c_int32, C.POINTER(C.c_int32))
    STEP = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_double))
    REPORT = C.CFUNCTYPE(None, C.c_void_p, C.c_int32, C.POINTER(C.c_double))
    SAVE = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_char), C.c_int32)
    _fields_ = [("user", C.c_void_p), ("next", NEXT), ("next_epoch", NEXT), ("position", POSITION), ("step", STEP),
                ("report", REPORT), ("save", SAVE), ("optimizer", C.c_void_p), ("schedule", C.c_void_p),
                ("updates", C.c_int32), ("applied", C.c_int32), ("accumulate", C.c_int32), ("log_every", C.c_int32)]


class LoopCancelled(Exception):
    """Raise from a reader or a step to stop the run the way a cancelled context does."""


class LoopStopped(HostError):
    """TrainingLoop.Run ended on a cancellation (after Save has run)."""


class TrainingLoop:
    """autograd.TrainingLoop (autograd/training_loop.go:53-214) over the host library.

    reader: object with next() -> batch (raise StopIteration at the end of an epoch) and next_epoch();
    sampler: object with marshal() -> bytes, or None; step(batch, seed) -> loss, back-propagating with
    the seed 1/accumulate; report(update, loss) and save(savepoint: Optional[bytes]) are optional.
    Exceptions of the callbacks end the run; LoopCancelled is the cancellation."""

    END_OF_EPOCH, CANCELLED, FAILED = 1, 2, 3

    def __init__(self, reader, optimizer, step, sampler=None, schedule: Optional["OneCycle"] = None, updates: int = 0,
                 applied: int = 0, accumulate: int = 0, log_every: int = 0, report=None, save=None):
        self.reader, self.optimizer, self.step, self.sampler, self.schedule = reader, optimizer, step, sampler, schedule
        self.Updates, self.Applied, self.Accumulate, self.LogEvery = updates, applied, accumulate, log_every
        self.report, self.save = report, save
        self._batch = None

    def _guard(self, fn, cancelled=2, failed=3):
        try:
            return fn() or 0
        except LoopCancelled as e:
            lib().gg_loop_set_error((str(e) or "context canceled").encode())
            return cancelled
        except Exception as e:  # any other error ends the run and is reported by it
            lib().gg_loop_set_error(f"{type(e).__name__}: {e}".encode())
            return failed

    def Run(self) -> None:
        T = _TrainingLoop

        def do_next(_user):
            def body():
                try:
                    self._batch = self.reader.next()
                except StopIteration:
                    return self.END_OF_EPOCH
            return self._guard(body)

        def do_next_epoch(_user):
            return self._guard(lambda: self.reader.next_epoch(), failed=1, cancelled=1)

        def do_position(_user, out, capacity, length):
            def body():
                payload = bytes(self.sampler.marshal())
                if len(payload) > capacity:
                    raise ValueError("sampler position too large")
                C.memmove(out, payload, len(payload))
                length[0] = len(payload)
            return self._guard(body, failed=1, cancelled=1)

        def do_step(_user, seed, loss):
            def body():
                loss[0] = float(self.step(self._batch, np.float32(seed[0])))
            return self._guard(body)

        def do_report(_user, update, loss):
            self.report(update, loss[0])

        def do_save(_user, savepoint, length):
            return self._guard(lambda: self.save(C.string_at(savepoint, length) if savepoint else None), failed=1,
                               cancelled=1)

        keep = [T.NEXT(do_next) if self.reader is not None else T.NEXT(),
                T.NEXT(do_next_epoch) if self.reader is not None else T.NEXT(),
                T.POSITION(do_position) if self.sampler is not None else T.POSITION(),
                T.STEP(do_step) if self.step is not None else T.STEP(),
                T.REPORT(do_report) if self.report is not None else T.REPORT(),
                T.SAVE(do_save) if self.save is not None else T.SAVE()]
        c = T(None, *keep, self.optimizer._h if self.optimizer is not None else None,
              C.cast(C.pointer(self.schedule._c), C.c_void_p) if self.schedule is not None else None,
              self.Updates, self.Applied, self.Accumulate, self.LogEvery)
        rc = lib().gg_training_loop_run(C.byref(c))
        self.Applied = c.applied
        if rc == self.CANCELLED:
            raise LoopStopped(lib().gg_last_error().decode("utf-8", "replace"))
        _check(rc)


class OneCycle:
    def __init__(self, max_lr: float, total: int, pct_start: float):
        self._c = _OneCycle()
        _check(lib().gg_onecycle_new(C.byref(C.c_double(max_lr)), total, C.byref(C.c_double(pct_start)), C.byref(self._c)))

    @property
    def StepCount(self) -> int:
        return self._c.step_count

    @StepCount.setter
    def StepCount(self, v: int) -> None:
        self._c.step_count = v

    def LR(self) -> float:
        out = C.c_double()
        _check(lib().gg_onecycle_lr(C.byref(self._c), C.byref(out)))
        return out.value

    def Step(self, optimizer: _Optimizer) -> None:
        _check(lib().gg_onecycle_step(C.byref(self._c), optimizer._h))

    def fields(self):
        c = self._c
        return (c.max_lr, c.pct_start, c.div_factor, c.final_div_factor, c.total, c.step_count)


def SaveTrainingCheckpoint(path: str, model: Sequence[Parameter], optimizer: _Optimizer, scheduler: OneCycle,
                           metadata: Optional[Dict[str, str]] = None) -> None:
    names, handles, n = _param_arrays(model)
    metadata = metadata or {}
    keys = (C.c_char_p * max(len(metadata), 1))(*[k.encode() for k in metadata])
    vals = (C.c_char_p * max(len(metadata), 1))(*[v.encode() for v in metadata.values()])
    _check(lib().gg_save_training_checkpoint(path.encode(), names, handles, n, optimizer._h, C.byref(scheduler._c),
                                             keys, vals, len(metadata)))


def LoadTrainingCheckpoint(path: str, model: Sequence[Parameter], optimizer: _Optimizer, scheduler: OneCycle) -> Dict[str, str]:
    names, handles, n = _param_arrays(model)
    buf = C.create_string_buffer(1 << 16)
    _check(lib().gg_load_training_checkpoint(path.encode(), names, handles, n, optimizer._h, C.byref(scheduler._c), buf,
                                             len(buf)))
    return json.loads(buf.value.decode() or "{}")


def safetensors_write(path: str, entries: Dict[str, np.ndarray], metadata: Optional[Dict[str, str]]) -> None:
    """Host-only: writes float32 entries in the reference's container layout."""
    names = list(entries)
    arrays = [np.require(entries[k], np.float32, "C") for k in names]
    c_names = (C.c_char_p * max(len(names), 1))(*[k.encode() for k in names])
    c_data = (_f32p * max(len(names), 1))(*[a.ctypes.data_as(_f32p) for a in arrays])
    shapes, offsets = [], [0]
    for a in arrays:
        shapes += list(a.shape)
        offsets.append(len(shapes))
    c_shapes = (C.c_int32 * max(len(shapes), 1))(*shapes)
    c_off = (C.c_int32 * len(offsets))(*offsets)
    md = metadata or {}
    keys = (C.c_char_p * max(len(md), 1))(*[k.encode() for k in md])
    vals = (C.c_char_p * max(len(md), 1))(*[v.encode() for v in md.values()])
    _check(lib().gg_safetensors_write(path.encode(), c_names, c_data, c_shapes, c_off, len(names), keys, vals,
                                      len(md) if metadata is not None else -1))


def safetensors_describe(path: str) -> dict:
    buf = C.create_string_buffer(1 << 20)
    _check(lib().gg_safetensors_describe(path.encode(), buf, len(buf)))
    return json.loads(buf.value.decode())


class _AdamWConfig(C.Structure):
    _fields_ = [("step_count", C.c_int32), ("lr", C.c_float), ("weight_decay", C.c_float), ("beta1", C.c_float),
                ("beta2", C.c_float), ("eps", C.c_float)]


def _state_c_args(names, shapes, step_count, lr, weight_decay, beta1, beta2, eps, groups):
    """The flat C arguments both state writers share; the returned tuple keeps every array alive."""
    n = len(names)
    c_names = (C.c_char_p * max(n, 1))(*[x.encode() for x in names])
    flat, offsets = [], [0]
    for sh in shapes:
        flat += list(sh)
        offsets.append(len(flat))
    c_shapes = (C.c_int32 * max(len(flat), 1))(*flat)
    c_off = (C.c_int32 * len(offsets))(*offsets)
    cfg = _AdamWConfig(step_count, lr, weight_decay, beta1, beta2, eps)
    g_names = (C.c_char_p * max(len(groups), 1))(*[g[0].encode() for g in groups])
    g_off, g_mem = [0], []
    for g in groups:
        g_mem += list(g[1])
        g_off.append(len(g_mem))
    c_goff = (C.c_int32 * len(g_off))(*g_off)
    c_gmem = (C.c_int32 * max(len(g_mem), 1))(*g_mem)
    c_scales = (C.c_float * max(len(groups), 1))(*[g[2] for g in groups])
    c_decays = (C.c_float * max(len(groups), 1))(*[g[3] for g in groups])
    gs = _Groups(len(groups), g_names, c_goff, c_gmem, c_scales, c_decays)
    return n, c_names, c_shapes, c_off, cfg, gs, (g_names, c_goff, c_gmem, c_scales, c_decays)


def adamw_state_write(path: str, names: Sequence[str], shapes: Sequence[Sequence[int]], m: Sequence[np.ndarray],
                      v: Sequence[np.ndarray], step_count: int, lr: float, weight_decay: float, beta1: float,
                      beta2: float, eps: float, groups: Sequence[tuple]) -> None:
    """Host-only: writes a "gograd-adamw" state file from gathered moments.
    groups: (name, member indexes, lr_scale, weight_decay) per group."""
    n, c_names, c_shapes, c_off, cfg, gs, _keep = _state_c_args(names, shapes, step_count, lr, weight_decay, beta1,
                                                                beta2, eps, groups)
    ms = [np.require(x, np.float32, "C") for x in m]
    vs = [np.require(x, np.float32, "C") for x in v]
    c_m = (_f32p * max(n, 1))(*[x.ctypes.data_as(_f32p) for x in ms])
    c_v = (_f32p * max(n, 1))(*[x.ctypes.data_as(_f32p) for x in vs])
    _check(lib().gg_adamw_state_write(path.encode(), n, c_names, c_shapes, c_off, c_m, c_v, C.byref(cfg), C.byref(gs)))


class _SGDConfig(C.Structure):
    _fields_ = [("step_count", C.c_int32), ("lr", C.c_float), ("momentum", C.c_float), ("dampening", C.c_float),
                ("weight_decay", C.c_float), ("nesterov", C.c_int32), ("maximize", C.c_int32)]


class _StateStream:
    """Common part of the streamed state writers: values arrive entry by entry in file order."""
    _h = None

    def next(self):
        """(entry name, values still missing) of the entry the file wants next; None at the end."""
        buf = C.create_string_buffer(64)
        remaining = C.c_int64()
        _check(lib().gg_state_stream_next(self._h, buf, len(buf), C.byref(remaining)))
        name = buf.value.decode()
        return (name, remaining.value) if name else None

    def append(self, entry: str, values: np.ndarray) -> None:
        v = np.require(values, np.float32, "C").reshape(-1)
        _check(lib().gg_state_stream_append(self._h, entry.encode(), v.ctypes.data_as(_f32p), C.c_int64(v.size)))

    def finish(self) -> None:
        h, self._h = self._h, None
        _check(lib().gg_state_stream_finish(h))

    def abort(self) -> None:
        if self._h:
            h, self._h = self._h, None
            lib().gg_state_stream_abort(h)

    def __del__(self):
        try:
            self.abort()
        except Exception:
            pass


class SGDStateStream(_StateStream):
    """A "gograd-sgd" state file (autograd/sgd_state.go:150-194) written front to back: one entry
    buffer.<i> per parameter whose momentum buffer is initialised; flags, options and groups in the
    metadata. groups: (name, member indexes, lr_scale, weight_decay) per group."""

    def __init__(self, path: str, names: Sequence[str], shapes: Sequence[Sequence[int]], step_count: int, lr: float,
                 momentum: float, dampening: float, weight_decay: float, nesterov: bool, maximize: bool,
                 initialized: Sequence[bool], groups: Sequence[tuple]):
        n, c_names, c_shapes, c_off, _cfg, gs, _keep = _state_c_args(names, shapes, step_count, lr, weight_decay, 0.0,
                                                                     0.0, 0.0, groups)
        cfg = _SGDConfig(step_count, lr, momentum, dampening, weight_decay, int(nesterov), int(maximize))
        flags = (C.c_uint8 * max(n, 1))(*[1 if b else 0 for b in initialized])
        self._h = C.c_void_p()
        _check(lib().gg_sgd_state_stream_begin(path.encode(), n, c_names, c_shapes, c_off, C.byref(cfg), flags,
                                               C.byref(gs), C.byref(self._h)))


class AdamWStateStream(_StateStream):
    """The same "gograd-adamw" file written front to back without holding the moments: the file's
    layout is fixed by names, shapes, configuration and groups; the values then arrive entry by
    entry in the order the file stores them, an entry possibly in consecutive pieces."""

    def __init__(self, path: str, names: Sequence[str], shapes: Sequence[Sequence[int]], step_count: int, lr: float,
                 weight_decay: float, beta1: float, beta2: float, eps: float, groups: Sequence[tuple]):
        n, c_names, c_shapes, c_off, cfg, gs, _keep = _state_c_args(names, shapes, step_count, lr, weight_decay, beta1,
                                                                    beta2, eps, groups)
        self._h = C.c_void_p()
        _check(lib().gg_adamw_state_stream_begin(path.encode(), n, c_names, c_shapes, c_off, C.byref(cfg), C.byref(gs),
                                                 C.byref(self._h)))
