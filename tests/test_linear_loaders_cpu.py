"""Checkpoint loading in the reference's key contract (samples/nvfp4_linear.py:39-80) and its tensor-parallel
variant, on CPU with the oracle registered as backend 'eager'."""
import pytest
import torch

import comfy_kitchen as ck
from comfy_kitchen.constraints import FunctionConstraints
from comfy_kitchen.linear import MXFP8Linear, NVFP4Linear, patch_model_with_mxfp8
from comfy_kitchen.registry import registry
from comfy_kitchen.sharding import take_ranges
from comfy_kitchen.tensor import QuantizedTensor


@pytest.fixture()
def eager():
    from oracle import ck_oracle

    names = ["quantize_nvfp4", "dequantize_nvfp4", "quantize_mxfp8", "dequantize_mxfp8", "scaled_mm_nvfp4", "scaled_mm_mxfp8"]
    cpu = FunctionConstraints(default_devices=frozenset({"cpu"}))
    registry.register("eager", ck_oracle, {n: cpu for n in names})
    try:
        with ck.use_backend("eager"):
            yield ck_oracle
    finally:
        with registry._lock:
            registry._backends.pop("eager", None)
            registry._capabilities.pop("eager", None)


def _checkpoint(orc, n, k, seed=0, input_scale=True):
    g = torch.Generator().manual_seed(seed)
    w = (0.02 * torch.randn(n, k, generator=g)).bfloat16()
    ts = (w.float().abs().max() / (6 * 448)).float().reshape(1)
    q, sf = orc.quantize_nvfp4(w, ts)
    sd = {"weight": q, "weight_scale": sf.view(torch.uint8), "weight_scale_2": ts,
          "bias": (0.02 * torch.randn(n, generator=g)).bfloat16()}
    if input_scale:
        sd["input_scale"] = torch.tensor([4.5 / (6 * 448)])
    return w, sd


def test_nvfp4_linear_loads_the_key_contract_and_runs(eager):
    n, k = 256, 512
    w, sd = _checkpoint(eager, n, k)
    m = NVFP4Linear(k, n, bias=True)
    missing, unexpected = m.load_state_dict(dict(sd))
    assert not missing and not unexpected
    assert isinstance(m.weight.data, QuantizedTensor) or isinstance(m.weight, QuantizedTensor)
    x = torch.randn(64, k, generator=torch.Generator().manual_seed(1)).bfloat16()
    y = m(x)
    qx, sx = eager.quantize_nvfp4(x, sd["input_scale"])
    want = eager.scaled_mm_nvfp4(qx, sd["weight"], sd["input_scale"], sd["weight_scale_2"], sx,
                                 sd["weight_scale"].view(torch.float8_e4m3fn), bias=sd["bias"], out_dtype=torch.bfloat16)
    assert torch.equal(y, want)
    # what it saves is what it loaded
    out = m.state_dict()
    for key in ("weight", "weight_scale", "weight_scale_2", "bias", "input_scale"):
        assert key in out, key
    assert torch.equal(out["weight"], sd["weight"])
    assert torch.equal(out["weight_scale"].view(torch.uint8), sd["weight_scale"])
    # without input_scale the layer quantizes dynamically and reports the key as missing, like the reference's sample
    w2, sd2 = _checkpoint(eager, n, k, input_scale=False)
    m2 = NVFP4Linear(k, n, bias=True)
    missing, _ = m2.load_state_dict(dict(sd2), strict=False)
    assert missing == ["input_scale"] and m2.input_scale is None
    assert m2(x).shape == (64, n)


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_shards_equal_quantizing_the_slice(eager, world):
    n, k = 512, 1024
    w, sd = _checkpoint(eager, n, k, seed=3)
    ts = sd["weight_scale_2"]
    x = torch.randn(32, k, generator=torch.Generator().manual_seed(2)).bfloat16()
    full = NVFP4Linear(k, n)
    full.load_state_dict(dict(sd))
    y_full = full(x).float()
    partial_sum, cols = torch.zeros(32, n), []
    for rank in range(world):
        col = NVFP4Linear(k, n, parallel="column", rank=rank, world=world)
        col.load_state_dict(dict(sd))
        lo, hi = rank * n // world, (rank + 1) * n // world
        q_ref, sf_ref = eager.quantize_nvfp4(w[lo:hi].contiguous(), ts)
        assert torch.equal(col.weight._qdata, q_ref)
        assert torch.equal(col.weight._params.block_scale.view(torch.uint8), sf_ref.view(torch.uint8))
        assert torch.equal(col.bias.data, sd["bias"][lo:hi])
        cols.append(col(x))
        row = NVFP4Linear(k, n, parallel="row", rank=rank, world=world)
        row.load_state_dict(dict(sd))
        lo, hi = rank * k // world, (rank + 1) * k // world
        q_ref, sf_ref = eager.quantize_nvfp4(w[:, lo:hi].contiguous(), ts)
        assert torch.equal(row.weight._qdata, q_ref)
        assert torch.equal(row.weight._params.block_scale.view(torch.uint8), sf_ref.view(torch.uint8))
        assert (row.bias is not None) == (rank == 0)
        xq = QuantizedTensor.from_float(x[:, lo:hi].contiguous(), "TensorCoreNVFP4Layout", scale=sd["input_scale"])
        partial_sum += row(xq).float()
    assert torch.equal(torch.cat(cols, dim=1).float(), y_full)       # column shards: the same numbers, split
    assert (partial_sum - y_full).abs().max() <= 2e-2 * y_full.abs().max()   # row shards: summation order and bf16 partials


def test_take_ranges_for_fused_qkv_and_fused_second_linear(eager):
    h, heads, hd = 512, 4, 128
    g = torch.Generator().manual_seed(5)
    w = (0.02 * torch.randn(3 * h, h, generator=g)).bfloat16()
    full = QuantizedTensor.from_float(w, "TensorCoreNVFP4Layout")
    ts = full._params.scale
    # rank 1 of 2 keeps heads 2..3 of q, k and v
    ranges = [(part * h + 2 * hd, part * h + 4 * hd) for part in range(3)]
    shard = take_ranges(full, 0, ranges)
    rows = torch.cat([torch.arange(lo, hi) for lo, hi in ranges])
    q_ref, sf_ref = eager.quantize_nvfp4(w[rows].contiguous(), ts)
    assert torch.equal(shard._qdata, q_ref)
    assert torch.equal(shard._params.block_scale.view(torch.uint8), sf_ref.view(torch.uint8))
    # columns: [attention 512 | mlp 2048] -> this rank's attention columns and MLP columns
    w2 = (0.02 * torch.randn(256, h + 4 * h, generator=g)).bfloat16()
    full2 = QuantizedTensor.from_float(w2, "TensorCoreNVFP4Layout")
    cr = [(256, 512), (h + 1024, h + 2048)]
    shard2 = take_ranges(full2, 1, cr)
    cols = torch.cat([torch.arange(lo, hi) for lo, hi in cr])
    q_ref, sf_ref = eager.quantize_nvfp4(w2[:, cols].contiguous(), full2._params.scale)
    assert torch.equal(shard2._qdata, q_ref)
    assert torch.equal(shard2._params.block_scale.view(torch.uint8), sf_ref.view(torch.uint8))
    with pytest.raises(ValueError):
        take_ranges(full, 0, [(64, 256)])


def test_mxfp8_patcher(eager):
    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(128, 256).bfloat16()
            self.small = torch.nn.Linear(16, 16).bfloat16()
            self.skip_me = torch.nn.Linear(128, 128).bfloat16()

    model = Tiny()
    w = model.a.weight.data.clone()
    # (the patcher quantizes on the device in the product; here the CPU oracle stands in, so keep tensors where they are)
    model, n = patch_model_with_mxfp8_cpu(model)
    assert n == 1 and isinstance(model.a, MXFP8Linear) and isinstance(model.small, torch.nn.Linear)
    x = torch.randn(2, 8, 128).bfloat16()
    y = model.a(x)
    q, s = eager.quantize_mxfp8(w)
    ref = torch.nn.functional.linear(x.float(), eager.dequantize_mxfp8(q, s, torch.float32), model.a.bias.float())
    assert y.shape == (2, 8, 256)
    assert (y.float() - ref).abs().max() <= 0.1 * ref.abs().max()


def patch_model_with_mxfp8_cpu(model):
    """patch_model_with_mxfp8 with the device move disabled (MXFP8Linear.from_linear(device=...) moves to CUDA)."""
    orig = MXFP8Linear.from_linear.__func__
    try:
        MXFP8Linear.from_linear = classmethod(lambda cls, linear, device="cpu": cls(
            linear.in_features, linear.out_features, linear.bias,
            QuantizedTensor.from_float(linear.weight.data, "TensorCoreMXFP8Layout"), linear.weight.dtype))
        return patch_model_with_mxfp8(model, min_features=64, skip_names=["skip_me"])
    finally:
        MXFP8Linear.from_linear = classmethod(orig)
