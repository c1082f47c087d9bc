"""comfy_kitchen, B200 build: the quantized-linear hot path on hand-written sm_100a kernels.

Public names follow the reference package (comfy_kitchen/__init__.py:28-72).
"""
__version__ = "0.2.18+b200"
