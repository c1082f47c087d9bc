"""Declarative call constraints (device, dtype, shape, compute capability).

Interface-compatible with the reference's comfy_kitchen/constraints.py: the same
rule and result classes, the same ``validate_function_call`` entry point.  A
backend publishes one ``FunctionConstraints`` per function; the registry checks a
call's keyword arguments against it before dispatching.
"""
from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass, field

import torch

__all__ = [
    "DivisibleBy", "ExactDims", "FunctionConstraints", "MinDims", "ParamConstraint", "ShapeRule",
    "ValidationResult", "validate_function_call", "validate_param",
]


class ShapeRule:
    """A predicate on a tensor's shape."""

    def check(self, tensor: torch.Tensor) -> bool:  # pragma: no cover - interface
        raise NotImplementedError

    def describe(self) -> str:  # pragma: no cover - interface
        raise NotImplementedError


@dataclass(frozen=True)
class DivisibleBy(ShapeRule):
    dim: int
    factor: int

    def check(self, tensor: torch.Tensor) -> bool:
        return tensor.dim() > self.dim and tensor.shape[self.dim] % self.factor == 0

    def describe(self) -> str:
        return f"dim[{self.dim}] divisible by {self.factor}"


@dataclass(frozen=True)
class MinDims(ShapeRule):
    ndim: int

    def check(self, tensor: torch.Tensor) -> bool:
        return tensor.dim() >= self.ndim

    def describe(self) -> str:
        return f"at least {self.ndim}D"


@dataclass(frozen=True)
class ExactDims(ShapeRule):
    ndim: int

    def check(self, tensor: torch.Tensor) -> bool:
        return tensor.dim() == self.ndim

    def describe(self) -> str:
        return f"exactly {self.ndim}D"


@dataclass(frozen=True)
class ParamConstraint:
    """What one keyword argument may be.  ``None`` fields mean "anything"
    (``devices=None`` defers to the function's ``default_devices``)."""

    dtypes: frozenset | None = None
    devices: frozenset | None = None
    shape_rules: tuple = ()

    def check_dtype(self, value) -> bool:
        if self.dtypes is None:
            return True
        if isinstance(value, torch.Tensor):
            return value.dtype in self.dtypes
        return value in self.dtypes or type(value) in self.dtypes  # a dtype argument, or a plain Python value

    def check_device(self, tensor: torch.Tensor, default_devices: frozenset) -> bool:
        allowed = default_devices if self.devices is None else self.devices
        return "*" in allowed or tensor.device.type in allowed

    def check_shape(self, tensor: torch.Tensor) -> bool:
        return all(rule.check(tensor) for rule in self.shape_rules)


@dataclass(frozen=True)
class FunctionConstraints:
    params: dict = field(default_factory=dict)
    default_devices: frozenset = field(default_factory=lambda: frozenset({"cuda", "cpu"}))
    min_compute_capability: tuple | None = None

    def __hash__(self) -> int:
        return hash((tuple(sorted(self.params.items(), key=lambda kv: kv[0])), self.default_devices,
                     self.min_compute_capability))


@dataclass
class ValidationResult:
    success: bool
    failed_param: str | None = None
    failure_reason: str | None = None

    @staticmethod
    def ok() -> "ValidationResult":
        return ValidationResult(True)

    @staticmethod
    def fail(param: str, reason: str) -> "ValidationResult":
        return ValidationResult(False, param, reason)


def validate_param(name: str, value, constraint: ParamConstraint, default_devices: frozenset) -> ValidationResult:
    if value is None:
        return ValidationResult.ok()
    if not constraint.check_dtype(value):
        shown = value.dtype if isinstance(value, torch.Tensor) else value
        return ValidationResult.fail(name, f"dtype {shown} not in {set(constraint.dtypes)}")
    if not isinstance(value, torch.Tensor):
        return ValidationResult.ok()
    if not constraint.check_device(value, default_devices):
        allowed = default_devices if constraint.devices is None else constraint.devices
        return ValidationResult.fail(name, f"device {value.device.type} not in {set(allowed)}")
    for rule in constraint.shape_rules:
        if not rule.check(value):
            return ValidationResult.fail(name, f"shape {list(value.shape)} fails: {rule.describe()}")
    return ValidationResult.ok()


def validate_function_call(constraints: FunctionConstraints, kwargs: Mapping,
                           compute_capability: tuple | None = None) -> ValidationResult:
    need = constraints.min_compute_capability
    if need is not None:
        if compute_capability is None:
            return ValidationResult.fail("__hardware__", "CUDA compute capability required but not available")
        if tuple(compute_capability) < tuple(need):
            have = ".".join(map(str, compute_capability))
            return ValidationResult.fail("__hardware__", f"compute capability {have} < required {need[0]}.{need[1]}")
    for pname, pc in constraints.params.items():
        res = validate_param(pname, kwargs.get(pname), pc, constraints.default_devices)
        if not res.success:
            return res
    return ValidationResult.ok()
