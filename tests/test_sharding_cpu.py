"""Tensor-parallel slicing of quantized weights: a shard cut out of a quantized checkpoint equals quantizing
the sliced float weight with the same per-tensor scale, byte for byte (CPU, oracle registered as 'eager')."""
import pytest
import torch

import comfy_kitchen as ck
from comfy_kitchen.constraints import FunctionConstraints
from comfy_kitchen.registry import registry
from comfy_kitchen.sharding import shard_linear_state, shard_quantized, slice_tiled_scales
from comfy_kitchen.tensor import QuantizedTensor


@pytest.fixture()
def eager():
    from oracle import ck_oracle

    names = ["quantize_nvfp4", "dequantize_nvfp4", "quantize_mxfp8", "dequantize_mxfp8"]
    cpu = FunctionConstraints(default_devices=frozenset({"cpu"}))
    registry.register("eager", ck_oracle, {n: cpu for n in names})
    try:
        with ck.use_backend("eager"):
            yield ck_oracle
    finally:
        with registry._lock:
            registry._backends.pop("eager", None)
            registry._capabilities.pop("eager", None)


def _weight(n, k, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (0.02 * torch.randn(n, k, generator=g)).bfloat16()


@pytest.mark.parametrize("layout", ["TensorCoreNVFP4Layout", "TensorCoreMXFP8Layout"])
@pytest.mark.parametrize("dim,world", [(0, 2), (0, 3), (1, 2), (1, 4)])
def test_shard_equals_quantizing_the_slice(eager, layout, dim, world):
    n, k = 768, 512
    w = _weight(n, k)
    full = QuantizedTensor.from_float(w, layout)
    size = (n, k)[dim] // world
    for rank in range(world):
        shard = shard_quantized(full, dim, rank, world)
        piece = w[rank * size:(rank + 1) * size] if dim == 0 else w[:, rank * size:(rank + 1) * size]
        kwargs = {"scale": full._params.scale} if layout == "TensorCoreNVFP4Layout" else {}
        want = QuantizedTensor.from_float(piece.contiguous(), layout, **kwargs)
        assert shard.shape == want.shape
        assert torch.equal(shard._qdata.view(torch.uint8), want._qdata.view(torch.uint8))
        a = getattr(shard._params, "block_scale", shard._params.scale)
        b = getattr(want._params, "block_scale", want._params.scale)
        assert a.shape == b.shape and torch.equal(a.view(torch.uint8), b.view(torch.uint8))
        torch.testing.assert_close(shard.dequantize().float(), want.dequantize().float(), rtol=0, atol=0)


def test_boundaries_must_sit_on_scale_tiles(eager):
    full = QuantizedTensor.from_float(_weight(384, 512), "TensorCoreNVFP4Layout")
    with pytest.raises(ValueError, match="multiples of 128"):
        shard_quantized(full, 0, 1, 4)        # 96-row shards cut through a 128-row scale tile
    with pytest.raises(ValueError, match="multiples of 64"):
        shard_quantized(full, 1, 1, 16)       # 32-column shards cut through a 4-column scale tile
    with pytest.raises(ValueError, match="does not split"):
        shard_quantized(full, 0, 0, 5)


def test_ragged_tail_of_tiled_scales_is_zeroed():
    s = torch.arange(256 * 8, dtype=torch.int64).remainder(251).add(1).to(torch.uint8).reshape(256, 8)
    out = slice_tiled_scales(s, (128, 200), (4, 6))
    assert out.shape == (128, 4)
    from oracle import ck_oracle as orc
    # positions of (row, col) in the tiled buffer: compare with the oracle's de-tiling of both buffers
    logical_full = orc.from_blocked(s, 256, 8)
    logical_part = orc.from_blocked(out, 128, 4)
    assert torch.equal(logical_part[:72, :2], logical_full[128:200, 4:6])
    assert logical_part[72:].abs().sum() == 0 and logical_part[:, 2:].abs().sum() == 0


def test_linear_state_column_and_row_parallel(eager):
    n, k = 256, 256
    w = _weight(n, k, seed=3)
    full = QuantizedTensor.from_float(w, "TensorCoreNVFP4Layout")
    state = {"l.weight": full._qdata, "l.weight_scale": full._params.block_scale.view(torch.uint8),
             "l.weight_scale_2": full._params.scale, "l.bias": torch.arange(n, dtype=torch.float32),
             "l.input_scale": torch.tensor(0.01)}
    col = [shard_linear_state(state, "l.", "column", r, 2) for r in range(2)]
    row = [shard_linear_state(state, "l.", "row", r, 2) for r in range(2)]
    assert [tuple(c["weight"].shape) for c in col] == [(128, 256)] * 2
    assert [tuple(r["weight"].shape) for r in row] == [(256, 128)] * 2
    assert torch.equal(torch.cat([c["bias"] for c in col]), state["l.bias"])
    assert row[0]["bias"] is state["l.bias"] and row[1]["bias"] is None
    deq = full.dequantize().float()
    torch.testing.assert_close(torch.cat([c["weight"].dequantize().float() for c in col], 0), deq, rtol=0, atol=0)
    torch.testing.assert_close(torch.cat([r["weight"].dequantize().float() for r in row], 1), deq, rtol=0, atol=0)
    # x @ W^T == sum over ranks of x[:, shard] @ W[:, shard]^T  (what the all-reduce adds up)
    x = torch.randn(8, k)
    parts = sum(x[:, r * 128:(r + 1) * 128] @ row[r]["weight"].dequantize().float().t() for r in range(2))
    torch.testing.assert_close(parts, x @ deq.t(), rtol=1e-5, atol=1e-5)
