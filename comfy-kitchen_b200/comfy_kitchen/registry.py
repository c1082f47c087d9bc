"""Backend registry.

Same public surface as the reference's comfy_kitchen/registry.py (``register``,
``get_implementation``, ``use_backend``, ``list_backends`` ...), but this build ships
exactly one compute backend, ``cuda`` (hand-written sm_100a kernels); the default
priority list therefore contains only it.  Other names can still be registered by a
caller (the tests register the CPU oracle as ``eager``) and reached through
``use_backend`` or an explicit ``backend=`` argument; they are never picked
automatically, so a CPU tensor raises ``NoCapableBackendError`` instead of silently
running somewhere else.
"""
from __future__ import annotations

import logging
import threading
from collections.abc import Callable, Mapping
from contextlib import contextmanager
from typing import Any

import torch

from .constraints import FunctionConstraints, ValidationResult, validate_function_call
from .exceptions import BackendNotFoundError, BackendNotImplementedError, NoCapableBackendError

logger = logging.getLogger("comfy_kitchen.dispatch")

KNOWN_BACKENDS = ("cuda", "triton", "eager")  # names the reference reports in list_backends()


class BackendRegistry:
    def __init__(self):
        self._backends: dict[str, Any] = {}
        self._capabilities: dict[str, set[str]] = {}
        self._constraints: dict[tuple[str, str], FunctionConstraints] = {}
        self._priority: list[str] = ["cuda"]
        self._disabled: set[str] = set()
        self._unavailable: dict[str, str] = {}
        self._lock = threading.Lock()
        self._tls = threading.local()
        self._cc: tuple[int, int] | None | bool = False  # False = not looked up yet

    # ------------------------------------------------------------------ hardware
    @property
    def _compute_capability(self) -> tuple[int, int] | None:
        if self._cc is False:
            cc = None
            if torch.cuda.is_available():
                try:
                    p = torch.cuda.get_device_properties(torch.cuda.current_device())
                    cc = (p.major, p.minor)
                except Exception:  # pragma: no cover - driver trouble
                    cc = None
            self._cc = cc
        return self._cc

    # ------------------------------------------------------------------ registration
    def register(self, name: str, module, capabilities: dict[str, FunctionConstraints]):
        with self._lock:
            self._backends[name] = module
            self._capabilities[name] = set(capabilities)
            for func, cons in capabilities.items():
                self._constraints[(name, func)] = cons
            self._unavailable.pop(name, None)

    def get_constraints(self, backend_name: str, func_name: str) -> FunctionConstraints | None:
        return self._constraints.get((backend_name, func_name))

    def mark_unavailable(self, name: str, reason: str):
        with self._lock:
            self._unavailable[name] = reason

    def disable(self, backend_name: str):
        with self._lock:
            self._disabled.add(backend_name)

    def enable(self, backend_name: str):
        with self._lock:
            self._disabled.discard(backend_name)

    def set_priority(self, priority_list: list[str]):
        with self._lock:
            self._priority = list(priority_list)

    def is_available(self, backend_name: str) -> bool:
        return backend_name in self._backends and backend_name not in self._disabled

    def list_backends(self) -> dict:
        names = set(KNOWN_BACKENDS) | set(self._priority) | set(self._backends) | set(self._unavailable)
        return {
            n: {
                "available": n in self._backends,
                "disabled": n in self._disabled,
                "unavailable_reason": self._unavailable.get(n),
                "capabilities": sorted(self._capabilities.get(n, ())),
            }
            for n in names
        }

    # ------------------------------------------------------------------ selection
    def validate_backend_for_call(self, backend_name: str, func_name: str, kwargs: Mapping[str, Any]) -> ValidationResult:
        if not self.is_available(backend_name):
            return ValidationResult.fail("__backend__", self._unavailable.get(backend_name, "not available"))
        if func_name not in self._capabilities.get(backend_name, ()):
            return ValidationResult.fail("__function__", "not implemented")
        cons = self._constraints.get((backend_name, func_name))
        if cons is None:
            return ValidationResult.ok()
        return validate_function_call(cons, kwargs, compute_capability=self._compute_capability)

    def _try(self, name: str, func_name: str, kwargs, failures: dict[str, str]) -> bool:
        if not self.is_available(name):
            failures[name] = "not available"
            return False
        if func_name not in self._capabilities.get(name, ()):
            failures[name] = "not implemented"
            return False
        if kwargs:
            res = self.validate_backend_for_call(name, func_name, kwargs)
            if not res.success:
                failures[name] = f"{res.failed_param}: {res.failure_reason}"
                return False
        return True

    def get_capable_backend(self, func_name: str, kwargs: Mapping[str, Any] | None = None) -> str:
        failures: dict[str, str] = {}
        override = getattr(self._tls, "backend_override", None)
        candidates = ([override] if override else []) + [n for n in self._priority if n != override]
        for name in candidates:
            if name != override and (not self.is_available(name) or func_name not in self._capabilities.get(name, ())):
                continue  # silently skip what is simply absent from the automatic list
            if self._try(name, func_name, kwargs, failures):
                logger.debug("Backend %s selected for %s%s", name, func_name, " (override)" if name == override else "")
                return name
        raise NoCapableBackendError(func_name, failures)

    def get_implementation(self, func_name: str, backend: str | None = None,
                           kwargs: Mapping[str, Any] | None = None) -> Callable:
        if backend:
            if backend not in self._backends:
                raise BackendNotFoundError(backend, self._unavailable.get(backend, "not registered"))
            if backend in self._disabled:
                raise BackendNotFoundError(backend, "disabled")
            if func_name not in self._capabilities.get(backend, ()):
                raise BackendNotImplementedError(backend, func_name)
            if kwargs:
                res = self.validate_backend_for_call(backend, func_name, kwargs)
                if not res.success:
                    raise NoCapableBackendError(func_name, {backend: f"{res.failed_param}: {res.failure_reason}"})
            return getattr(self._backends[backend], func_name)
        return getattr(self._backends[self.get_capable_backend(func_name, kwargs)], func_name)

    @contextmanager
    def use_backend(self, backend_name: str):
        if not self.is_available(backend_name):
            if backend_name in self._unavailable:
                raise BackendNotFoundError(backend_name, self._unavailable[backend_name])
            raise BackendNotFoundError(backend_name, "disabled" if backend_name in self._disabled else "not registered")
        previous = getattr(self._tls, "backend_override", None)
        self._tls.backend_override = backend_name
        try:
            yield
        finally:
            if previous is None:
                del self._tls.backend_override
            else:
                self._tls.backend_override = previous


registry = BackendRegistry()
