"""Errors raised by backend selection (same classes and attributes as the reference's
comfy_kitchen/exceptions.py, so ``except`` clauses written against it keep working)."""


class BackendError(RuntimeError):
    """Root of the backend-selection errors."""


class BackendNotFoundError(BackendError):
    def __init__(self, backend_name: str, reason: str | None = None):
        self.backend_name = backend_name
        text = f"Backend '{backend_name}' is not available"
        super().__init__(f"{text}: {reason}" if reason else text)


class BackendNotImplementedError(BackendError):
    def __init__(self, backend_name: str, func_name: str):
        self.backend_name = backend_name
        self.func_name = func_name
        super().__init__(f"Backend '{backend_name}' does not implement '{func_name}'")


class NoCapableBackendError(BackendError):
    """No registered backend accepts the call (device, dtype, shape or hardware constraint)."""

    def __init__(self, func_name: str, failures: dict[str, str]):
        self.func_name = func_name
        self.failures = failures
        if failures:
            why = "; ".join(f"{k}: {v}" for k, v in failures.items())
            super().__init__(f"No backend can handle '{func_name}': {why}")
        else:
            super().__init__(f"No backend available for '{func_name}'")
