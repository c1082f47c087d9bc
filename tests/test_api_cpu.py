"""CPU-side checks: the shared library loads and exports the declared C ABI, the registry and the
constraint system behave like the reference's, and the QuantizedTensor bookkeeping (shapes,
padding, transposes, serialisation, dispatch order) is right.  The layout tests run on CPU by
registering the CPU oracle under the backend name ``eager`` and selecting it explicitly — the
package itself never does that."""
import ctypes
import os

import pytest
import torch

import comfy_kitchen as ck
from comfy_kitchen import _native
from comfy_kitchen.constraints import (DivisibleBy, ExactDims, FunctionConstraints, MinDims, ParamConstraint,
                                       validate_function_call)
from comfy_kitchen.registry import registry
from comfy_kitchen.tensor import QuantizedTensor, TensorCoreFP8Layout, TensorCoreMXFP8Layout, TensorCoreNVFP4Layout


# ------------------------------------------------------------------ the C ABI


def test_library_exports_every_declared_symbol():
    import __graft_entry__ as entry

    declared = entry.declared_symbols()
    assert len(declared) >= 19
    lib = ctypes.CDLL(_native.LIB_PATH)
    missing = [s for s in declared if not hasattr(lib, s)]
    assert not missing, missing
    # and the Python binding covers the same set
    bound = set(_native.SIGNATURES) | set(_native._RESTYPES)
    assert set(declared) <= bound, sorted(set(declared) - bound)


def test_header_is_valid_c_and_cxx():
    """The boundary header must compile by itself in both languages (every csrc/*.cu also includes it through
    ck_common.cuh, so a definition that drifts from its declaration fails the build)."""
    import os
    import shutil
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = os.path.join(root, "include", "comfy_kitchen_b200.h")
    for cmd in (["gcc", "-std=c11", "-Wall", "-Werror", "-fsyntax-only", "-x", "c", header],
                ["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-x", "c++", header]):
        if shutil.which(cmd[0]) is None:
            pytest.skip(f"{cmd[0]} not installed")
        r = subprocess.run(cmd, capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
    common = open(os.path.join(root, "comfy-kitchen_b200", "csrc", "ck_common.cuh")).read()
    assert '#include "comfy_kitchen_b200.h"' in common
    for name in os.listdir(os.path.join(root, "comfy-kitchen_b200", "csrc")):
        if name.endswith(".cu"):
            assert '#include "ck_common.cuh"' in open(os.path.join(root, "comfy-kitchen_b200", "csrc", name)).read(), name


def test_argument_errors_come_back_as_status_and_message():
    lib = _native.load()
    assert lib.ck_abi_version() == 1
    rc = lib.launch_quantize_nvfp4_kernel(None, None, None, None, 16, 16, 16, 16, 0.0, 2, True, None)
    assert rc == -4 and b"null pointer" in lib.ck_last_error()
    with pytest.raises(RuntimeError, match="unknown option"):
        _native.call("ck_set_option", b"no_such_option", 1)


def test_every_documented_option_is_accepted():
    """The option names listed in csrc/ck_options.h (and the public one) are the ones ck_set_option knows."""
    import re

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "comfy-kitchen_b200", "csrc", "ck_options.h")).read()
    names = re.findall(r'^//   "([a-z_]+)"', text, flags=re.M)
    assert len(names) >= 8 and "qk_heads_per_warp" in names
    defaults = {"norm_cache": -1, "gelu_table_min": 8 << 20, "gemm_map_cache": 1}
    for name in names + ["nvfp4_exact_div"]:
        _native.call("ck_set_option", name.encode(), defaults.get(name, 0))   # (sets the default back)


# ------------------------------------------------------------------ registry


@pytest.fixture()
def eager():
    """The CPU oracle registered as backend 'eager' for the duration of a test."""
    from oracle import ck_oracle

    names = ["quantize_per_tensor_fp8", "dequantize_per_tensor_fp8", "quantize_nvfp4", "dequantize_nvfp4",
             "scaled_mm_nvfp4", "quantize_mxfp8", "dequantize_mxfp8", "scaled_mm_mxfp8", "apply_rope", "apply_rope1",
             "apply_rope_split_half", "apply_rope_split_half1", "adaln"]
    cpu = FunctionConstraints(default_devices=frozenset({"cpu"}))
    registry.register("eager", ck_oracle, {n: cpu for n in names})
    try:
        yield ck_oracle
    finally:
        with registry._lock:
            registry._backends.pop("eager", None)
            registry._capabilities.pop("eager", None)


def test_backend_listing_and_single_backend_policy():
    info = ck.list_backends()
    assert {"cuda", "triton", "eager"} <= set(info)
    assert info["cuda"]["available"] and "scaled_mm_nvfp4" in info["cuda"]["capabilities"]
    assert not info["triton"]["available"] and "not built" in info["triton"]["unavailable_reason"]
    assert registry._priority == ["cuda"]


def test_cpu_tensors_are_refused_not_rerouted(eager):
    x = torch.randn(16, 32).bfloat16()
    with pytest.raises(ck.NoCapableBackendError) as e:
        ck.quantize_nvfp4(x, torch.tensor(0.01))
    assert "cuda" in e.value.failures and e.value.func_name == "quantize_nvfp4"
    # explicit selection reaches the oracle
    with ck.use_backend("eager"):
        q, sf = ck.quantize_nvfp4(x, torch.tensor(0.01))
    assert q.shape == (16, 16) and sf.shape == (128, 4)


def test_use_backend_errors():
    with pytest.raises(ck.BackendNotFoundError):
        with ck.use_backend("triton"):
            pass
    with pytest.raises(ck.BackendNotFoundError):
        with ck.use_backend("nope"):
            pass
    with pytest.raises(ck.BackendNotImplementedError):
        registry.get_implementation("no_such_function", backend="cuda")
    ck.disable_backend("cuda")
    try:
        with pytest.raises(ck.BackendNotFoundError):
            registry.get_implementation("adaln", backend="cuda")
    finally:
        ck.enable_backend("cuda")


def test_nested_override_restores(eager):
    with ck.use_backend("eager"):
        with ck.use_backend("eager"):
            pass
        assert registry._tls.backend_override == "eager"
    assert getattr(registry._tls, "backend_override", None) is None


# ------------------------------------------------------------------ constraints


def test_constraint_rules():
    t = torch.zeros(4, 48)
    assert DivisibleBy(1, 16).check(t) and not DivisibleBy(1, 32).check(t) and not DivisibleBy(2, 2).check(t)
    assert ExactDims(2).check(t) and not ExactDims(3).check(t) and MinDims(2).check(t) and not MinDims(3).check(t)
    fc = FunctionConstraints(
        params={"x": ParamConstraint(dtypes=frozenset({torch.bfloat16}), shape_rules=(ExactDims(2), DivisibleBy(1, 16))),
                "output_type": ParamConstraint(dtypes=frozenset({torch.float8_e4m3fn}))},
        default_devices=frozenset({"cuda"}), min_compute_capability=(10, 0))
    r = validate_function_call(fc, {"x": t.bfloat16()}, compute_capability=None)
    assert not r.success and r.failed_param == "__hardware__"
    r = validate_function_call(fc, {"x": t.bfloat16()}, compute_capability=(9, 0))
    assert not r.success and "9.0" in r.failure_reason
    r = validate_function_call(fc, {"x": t.bfloat16()}, compute_capability=(10, 0))
    assert not r.success and r.failed_param == "x" and "device" in r.failure_reason
    fc_cpu = FunctionConstraints(params=fc.params, default_devices=frozenset({"*"}))
    assert validate_function_call(fc_cpu, {"x": t.bfloat16(), "output_type": torch.float8_e4m3fn}).success
    assert validate_function_call(fc_cpu, {"x": t}).failed_param == "x"  # dtype
    assert validate_function_call(fc_cpu, {"x": torch.zeros(4, 40).bfloat16()}).failure_reason.endswith("divisible by 16")
    assert validate_function_call(fc_cpu, {"x": None, "output_type": torch.float8_e5m2}).failed_param == "output_type"
    assert hash(fc) == hash(FunctionConstraints(params=dict(fc.params), default_devices=fc.default_devices,
                                                min_compute_capability=(10, 0)))


# ------------------------------------------------------------------ QuantizedTensor on the oracle


def test_nvfp4_layout_padding_and_serialisation(eager):
    x = torch.randn(129, 130).bfloat16()
    with ck.use_backend("eager"):
        qt = QuantizedTensor.from_float(x, "TensorCoreNVFP4Layout")
        assert tuple(qt.shape) == (129, 130) and qt.dtype == torch.bfloat16
        assert qt.storage_shape == (144, 72) and qt.padded_shape == (144, 144) and qt.is_padded
        assert qt.storage_dtype == torch.uint8 and qt.nbytes == 144 * 72
        assert qt._params.block_scale.shape == (256, 12) and qt._params.block_scale.dtype == torch.float8_e4m3fn
        d = qt.dequantize()
        assert tuple(d.shape) == (129, 130)
        assert (d.float() - x.float()).abs().max() < 0.6 * x.float().abs().max() / 6 + 0.3
        sd = qt.state_dict("layer.weight")
        assert set(sd) == {"layer.weight", "layer.weight_scale", "layer.weight_scale_2"}
        assert sd["layer.weight_scale_2"].dtype == torch.float32
        # a given scale is honoured, "recalculate" recomputes
        q2 = QuantizedTensor.from_float(x, "TensorCoreNVFP4Layout", scale=0.01)
        assert float(q2._params.scale) == pytest.approx(0.01)
    assert TensorCoreNVFP4Layout.get_storage_shape((129, 130)) == (144, 72)
    with pytest.raises(ValueError):
        TensorCoreNVFP4Layout.quantize(torch.randn(2, 3, 4))


def test_transpose_is_a_flag_and_mm_orientation(eager):
    x, w = torch.randn(48, 64).bfloat16(), (0.05 * torch.randn(80, 64)).bfloat16()
    with ck.use_backend("eager"):
        for name in ("TensorCoreNVFP4Layout", "TensorCoreMXFP8Layout"):
            qx, qw = QuantizedTensor.from_float(x, name), QuantizedTensor.from_float(w, name)
            wt = qw.t()
            assert tuple(wt.shape) == (64, 80) and wt._params.transposed and wt._qdata is qw._qdata
            assert not wt.t()._params.transposed
            assert torch.equal(wt.dequantize(), qw.dequantize().t())
            ref = torch.nn.functional.linear(qx.dequantize(), qw.dequantize())
            y_lin = torch.nn.functional.linear(qx, qw)
            y_mm = torch.mm(qx, wt)
            y_add = torch.addmm(torch.zeros(80).bfloat16(), qx, wt)
            for y in (y_lin, y_mm, y_add):
                assert tuple(y.shape) == (48, 80) and y.dtype == torch.bfloat16
                assert (y.float() - ref.float()).abs().max() <= 0.05 * ref.float().abs().max() + 0.05
            # orientations the kernels do not cover fall back to the dequantized op, bit for bit
            qb = QuantizedTensor.from_float(w.t().contiguous(), name)  # [64, 80] stored untransposed
            assert torch.equal(torch.mm(qx, qb), torch.mm(qx.dequantize(), qb.dequantize()))
            qxt = QuantizedTensor.from_float(x.t().contiguous(), name).t()  # logically [48, 64], stored transposed
            assert torch.equal(torch.mm(qxt, wt), torch.mm(qxt.dequantize(), wt.dequantize()))


def test_padded_linear_is_cropped(eager):
    x, w = torch.randn(49, 81).bfloat16(), (0.05 * torch.randn(113, 81)).bfloat16()
    with ck.use_backend("eager"):
        for name in ("TensorCoreNVFP4Layout", "TensorCoreMXFP8Layout"):
            y = torch.nn.functional.linear(QuantizedTensor.from_float(x, name), QuantizedTensor.from_float(w, name))
            assert tuple(y.shape) == (49, 113)


def test_generic_tensor_ops(eager):
    x = torch.randn(32, 64).bfloat16()
    with ck.use_backend("eager"):
        qt = QuantizedTensor.from_float(x, "TensorCoreFP8Layout")
        assert qt.storage_dtype == torch.float8_e4m3fn and set(qt.state_dict("w")) == {"w", "w_scale"}
        c = qt.clone()
        assert c._qdata.data_ptr() != qt._qdata.data_ptr() and torch.equal(c.dequantize(), qt.dequantize())
        assert qt.detach()._layout_cls == "TensorCoreFP8Layout"
        f = qt.to(torch.float16)
        assert f.dtype == torch.float16 and torch.equal(f._qdata.view(torch.uint8), qt._qdata.view(torch.uint8)) and f.dequantize().dtype == torch.float16
        assert qt.to(torch.bfloat16) is qt
        e = torch.empty_like(qt)
        assert isinstance(e, QuantizedTensor) and e.storage_shape == qt.storage_shape
        e.copy_(qt)
        assert torch.equal(e.dequantize(), qt.dequantize())
        with pytest.raises(TypeError):
            e.copy_(x)
        with pytest.raises(TypeError):
            e.copy_(QuantizedTensor.from_float(x, "TensorCoreMXFP8Layout"))
        # FP8 shape ops stay quantized
        v = qt.view(64, 32)
        assert isinstance(v, QuantizedTensor) and tuple(v.shape) == (64, 32)
        assert isinstance(qt.t(), QuantizedTensor) and tuple(qt.t().shape) == (64, 32)
        # anything without a handler dequantizes
        assert torch.equal(qt + 1, qt.dequantize() + 1)
        # block formats do not keep views quantized
        q4 = QuantizedTensor.from_float(x, "TensorCoreNVFP4Layout")
        assert not isinstance(q4.reshape(64, 32), QuantizedTensor)


def test_flatten_roundtrip(eager):
    x = torch.randn(32, 64).bfloat16()
    with ck.use_backend("eager"):
        for name in ("TensorCoreFP8Layout", "TensorCoreNVFP4Layout", "TensorCoreMXFP8Layout"):
            qt = QuantizedTensor.from_float(x, name)
            inner, ctx = qt.__tensor_flatten__()
            assert inner[0] == "_qdata" and ctx["layout_cls"] == name
            tensors = {n: getattr(qt, n) for n in inner}
            back = QuantizedTensor.__tensor_unflatten__(tensors, ctx, qt.shape, None)
            assert torch.equal(back.dequantize(), qt.dequantize()) and back._params.orig_shape == (32, 64)
            new = qt.requantize_from_float(x * 2)
            assert new._layout_cls == name


def test_layout_requirements():
    req = TensorCoreNVFP4Layout.get_requirements()
    assert req["layout"] == "TensorCoreNVFP4Layout" and req["min_sm_version"] == (10, 0)
    assert TensorCoreFP8Layout.MIN_SM_VERSION == (8, 9) and TensorCoreMXFP8Layout.MIN_SM_VERSION == (10, 0)
    assert TensorCoreMXFP8Layout.get_padded_shape((65, 96)) == (96, 96)
