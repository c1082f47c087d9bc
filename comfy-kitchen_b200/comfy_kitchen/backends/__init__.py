"""Backend registration.  One backend ships: ``cuda``.  ``triton`` is reported as not built so tools
that list backends still see the name."""
from __future__ import annotations

from comfy_kitchen.registry import registry


def register_backends() -> None:
    registry.mark_unavailable("triton", "not built: this package contains sm_100a CUDA kernels only")
    try:
        from . import cuda as cuda_backend
    except Exception as e:  # library missing or unloadable: nothing can run, say why
        registry.mark_unavailable("cuda", f"{type(e).__name__}: {e}")
        return
    registry.register("cuda", cuda_backend, cuda_backend.build_constraints())
