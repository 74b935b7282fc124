"""Public objects of the ``orchestra`` package.

Same import paths, class names, signatures, defaults and error types as the reference's Python
module (orchestra-py/src/{arch,activations,initialization,datasets,optimizers,loss_fns,sync,store,
serializer,training,session}.rs). Each object is a thin description that serialises to the
``model.json`` / ``training.json`` schema; parsing, validation and planning happen in the C++ core
(``orchestra._orchestra``), the run itself in ``oxidized_neural_orchestra_b200.runtime``.
"""
from __future__ import annotations

import json
import math
import os
from typing import Any, Sequence


def _positive_int(v: Any, name: str) -> int:
    if isinstance(v, bool) or not isinstance(v, int):
        raise TypeError(f"{name} must be an integer")
    if v <= 0:
        raise ValueError(f"{name} must be greater than 0")
    return v


def _float(v: Any, name: str) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise TypeError(f"{name} must be a number")
    return float(v)


# ---------------------------------------------------------------------------------------------
# activations (orchestra-py/src/activations.rs:6-86) + the additive GELU
# ---------------------------------------------------------------------------------------------
class _Act:
    def to_config(self):
        raise NotImplementedError

    def __repr__(self):
        return f"{type(self).__name__}({', '.join(f'{k}={v}' for k, v in vars(self).items())})"


class Sigmoid(_Act):
    def __init__(self, amp: float = 1.0):
        self.amp = _float(amp, "amp")

    def to_config(self):
        return {"sigmoid": {"amp": self.amp}}


class Tanh(_Act):
    def __init__(self, amp: float = 1.0):
        self.amp = _float(amp, "amp")

    def to_config(self):
        return {"tanh": {"amp": self.amp}}


class ReLU(_Act):
    def __init__(self, slope: float):
        self.slope = _float(slope, "slope")

    def to_config(self):
        return {"relu": {"slope": self.slope}}


class Softmax(_Act):
    def to_config(self):
        return "softmax"


class GELU(_Act):
    """Exact (erf) GELU. Not part of the reference's activation set; additive on this runtime."""

    def to_config(self):
        return "gelu"


# ---------------------------------------------------------------------------------------------
# initialisers (orchestra-py/src/initialization.rs:12-186)
# ---------------------------------------------------------------------------------------------
class _Init:
    _tag = ""

    def to_config(self):
        return self._tag

    def __repr__(self):
        return f"{type(self).__name__}()"


class Kaiming(_Init):
    _tag = "kaiming"


class Xavier(_Init):
    _tag = "xavier"


class Lecun(_Init):
    _tag = "lecun"


class XavierUniform(_Init):
    _tag = "xavier_uniform"


class LecunUniform(_Init):
    _tag = "lecun_uniform"


class Const(_Init):
    def __init__(self, value: float):
        self.value = _float(value, "value")

    def to_config(self):
        return {"const": {"value": self.value}}


class Uniform(_Init):
    def __init__(self, low: float, high: float):
        self.low, self.high = _float(low, "low"), _float(high, "high")

    def to_config(self):
        return {"uniform": {"low": self.low, "high": self.high}}


class UniformInclusive(_Init):
    def __init__(self, low: float, high: float):
        self.low, self.high = _float(low, "low"), _float(high, "high")

    def to_config(self):
        return {"uniform_inclusive": {"low": self.low, "high": self.high}}


class Normal(_Init):
    def __init__(self, mean: float, std_dev: float):
        self.mean, self.std_dev = _float(mean, "mean"), _float(std_dev, "std_dev")

    def to_config(self):
        return {"normal": {"mean": self.mean, "std_dev": self.std_dev}}


def _init_cfg(init: Any):
    if not isinstance(init, _Init):
        raise TypeError("init must be a parameter initializer")
    return init.to_config()


def _act_cfg(act_fn: Any):
    if act_fn is None:
        return None
    if not isinstance(act_fn, _Act):
        raise TypeError("act_fn must be an activation function (Sigmoid, Tanh, ReLU, Softmax) or None")
    return act_fn.to_config()


def _triple(v: Any, name: str) -> list[int]:
    if not isinstance(v, (tuple, list)) or len(v) != 3:
        raise TypeError(f"{name} must be a tuple of three integers")
    out = []
    for x in v:
        if isinstance(x, bool) or not isinstance(x, int):
            raise TypeError(f"{name} must be a tuple of three integers")
        if x <= 0:
            raise ValueError(f"{name} must be > 0")
        out.append(x)
    return out


# ---------------------------------------------------------------------------------------------
# layers (orchestra-py/src/arch.rs:99-340)
# ---------------------------------------------------------------------------------------------
class Dense:
    def __init__(self, output_size: int, init, act_fn=None):
        self.output_size = _positive_int(output_size, "output_size")
        self._init, self._act = _init_cfg(init), _act_cfg(act_fn)

    def to_config(self):
        return {"dense": {"output_size": self.output_size, "init": self._init, "act_fn": self._act}}


class Conv2d:
    def __init__(self, input_dim, kernel_dim, stride: int, padding: int, init, act_fn=None):
        self.input_dim, self.kernel_dim = _triple(input_dim, "input_dim"), _triple(kernel_dim, "kernel_dim")
        if isinstance(stride, bool) or not isinstance(stride, int) or isinstance(padding, bool) or not isinstance(padding, int):
            raise TypeError("stride and padding must be integers")
        if stride <= 0:
            raise ValueError("stride must be > 0")
        if padding < 0:
            raise ValueError("padding must be >= 0")
        self.stride, self.padding = stride, padding
        self._init, self._act = _init_cfg(init), _act_cfg(act_fn)

    def to_config(self):
        return {"conv": {"input_dim": self.input_dim, "kernel_dim": self.kernel_dim, "stride": self.stride,
                         "padding": self.padding, "init": self._init, "act_fn": self._act}}


class MaxPooling:
    def __init__(self, input_dim, filter_size: int, stride: int, padding: int, act_fn=None):
        self.input_dim = _triple(input_dim, "input_dim")
        for v, n in ((filter_size, "filter_size"), (stride, "stride")):
            if isinstance(v, bool) or not isinstance(v, int):
                raise TypeError(f"{n} must be an integer")
            if v <= 0:
                raise ValueError(f"{n} must be > 0")
        if isinstance(padding, bool) or not isinstance(padding, int):
            raise TypeError("padding must be an integer")
        if padding < 0:
            raise ValueError("padding must be >= 0")
        self.filter_size, self.stride, self.padding = filter_size, stride, padding
        self._act = _act_cfg(act_fn)

    def to_config(self):
        return {"max_pooling": {"input_dim": self.input_dim, "filter_size": self.filter_size,
                                "stride": self.stride, "padding": self.padding, "act_fn": self._act}}


class Sequential:
    def __init__(self, layers: Sequence[Any]):
        layers = list(layers)
        if not layers:
            raise ValueError("model must have at least one layer")
        for l in layers:
            if not isinstance(l, (Dense, Conv2d, MaxPooling)):
                raise TypeError("layers must be Dense, Conv2d or MaxPooling instances")
        self.layers = layers

    def to_config(self) -> dict:
        return {"layers": [l.to_config() for l in self.layers]}

    def to_json(self) -> str:
        return json.dumps(self.to_config())


# ---------------------------------------------------------------------------------------------
# datasets (orchestra-py/src/datasets.rs:23-115)
# ---------------------------------------------------------------------------------------------
class InlineDataset:
    def __init__(self, samples, labels, x_size: int, y_size: int):
        self.x_size, self.y_size = _positive_int(x_size, "x_size"), _positive_int(y_size, "y_size")
        import numpy as np

        self.samples = np.ascontiguousarray(np.asarray(samples, dtype=np.float32).reshape(-1))
        self.labels = np.ascontiguousarray(np.asarray(labels, dtype=np.float32).reshape(-1))

    def to_config(self, with_data: bool = True):
        src = {"samples": self.samples.tolist() if with_data else [], "labels": self.labels.tolist() if with_data else []}
        return {"src": {"inline": src}, "x_size": self.x_size, "y_size": self.y_size}


class LocalDataset:
    def __init__(self, samples_path: str, labels_path: str, x_size: int, y_size: int):
        self.x_size, self.y_size = _positive_int(x_size, "x_size"), _positive_int(y_size, "y_size")
        self.samples_path, self.labels_path = os.fspath(samples_path), os.fspath(labels_path)
        if not os.path.isfile(self.samples_path):
            raise ValueError(f"samples_path does not exist: {self.samples_path}")
        if not os.path.isfile(self.labels_path):
            raise ValueError(f"labels_path does not exist: {self.labels_path}")

    def to_config(self, with_data: bool = True):
        return {"src": {"local": {"samples_path": self.samples_path, "labels_path": self.labels_path}},
                "x_size": self.x_size, "y_size": self.y_size}


# ---------------------------------------------------------------------------------------------
# optimizers / losses / sync / store / serializer
# ---------------------------------------------------------------------------------------------
def _pos(v, name):
    v = _float(v, name)
    if not (v > 0.0) or not math.isfinite(v):
        raise ValueError(f"{name} must be a positive number")
    return v


def _unit(v, name):
    v = _float(v, name)
    if not (0.0 <= v <= 1.0):
        raise ValueError(f"{name} must be between 0.0 and 1.0")
    return v


class GradientDescent:
    def __init__(self, lr: float):
        self.lr = _float(lr, "lr")

    def to_config(self):
        return {"gradient_descent": {"lr": _pos(self.lr, "lr")}}


class GradientDescentWithMomentum:
    def __init__(self, lr: float, mu: float):
        self.lr, self.mu = _float(lr, "lr"), _float(mu, "mu")

    def to_config(self):
        return {"gradient_descent_with_momentum": {"lr": _pos(self.lr, "lr"), "mu": _unit(self.mu, "mu")}}


class Adam:
    def __init__(self, lr: float, b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8):
        self.lr, self.b1, self.b2, self.eps = _float(lr, "lr"), _float(b1, "b1"), _float(b2, "b2"), _float(eps, "eps")

    def to_config(self):
        return {"adam": {"lr": _pos(self.lr, "lr"), "b1": _unit(self.b1, "b1"), "b2": _unit(self.b2, "b2"),
                         "eps": _pos(self.eps, "eps")}}


class Mse:
    def to_config(self):
        return "mse"


class CrossEntropy:
    def to_config(self):
        return "cross_entropy"


class BarrierSync:
    def to_config(self):
        return "barrier"


class NonBlockingSync:
    def to_config(self):
        return "non_blocking"


class BlockingStore:
    def to_config(self):
        return "blocking"


class WildStore:
    def to_config(self):
        return "wild"


class BaseSerializer:
    def to_config(self):
        return "base"


class SparseSerializer:
    def __init__(self, r: float):
        self.r = _float(r, "r")

    def to_config(self):
        return {"sparse_capable": {"r": _unit(self.r, "r")}}
