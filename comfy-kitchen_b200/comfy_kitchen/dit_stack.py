"""Synthetic Flux-like DiT stack on the quantized-linear path, with Megatron tensor parallelism.

The reference ships kernels and tensor wrappers but no model; this module is the workload its
NVFP4 path is aimed at (an MMDiT with double-stream and single-stream blocks), built only from
the package's own operators so that one forward exercises every kernel of the path:

    LayerNorm + AdaLN modulation -> NVFP4   adaln_quantize_nvfp4      (fused front end)
    block-scaled GEMM, alpha and bias fused  scaled_mm_nvfp4
    per-head RMSNorm of q and k, rotary      qk_norm_rope              (fused, writes the attention layout)
    embedding, q/k/v relayout
    activation re-quantisation               quantize_nvfp4_gather     (reads attention's layout / a column
                                                                       slice in place, GELU fused)

Attention itself is torch's scaled_dot_product_attention in bf16.

Tensor parallelism (world size t, one process per GPU): attention heads and MLP columns are split
across ranks.  The first GEMM of each half-block is column-parallel (no exchange), the second is
row-parallel and ends in one all-reduce(sum) of the [tokens, hidden] partial result over the
process group (NCCL on GPUs, gloo in the CPU tests).  A forward of the full model issues
2 * n_double + n_single all-reduces (76 for 19 + 38 blocks).  Weights are quantised after slicing,
with the per-tensor scale taken from the unsliced weight, so every rank's shard decodes to the
same values as the corresponding part of the full weight.  K-shards are multiples of 64 elements
and N-shards multiples of 128 rows for the configurations used (hidden 3072, t <= 8), which keeps
whole 128x4 scale tiles on one rank.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

F4_MAX = 6.0
E4M3_MAX = 448.0


@dataclass
class DiTConfig:
    hidden: int = 3072
    heads: int = 24
    head_dim: int = 128
    mlp_ratio: int = 4
    n_double: int = 19
    n_single: int = 38
    txt_tokens: int = 512
    img_grid: tuple[int, int] = (64, 64)
    axes_dim: tuple[int, int, int] = (16, 56, 56)
    theta: float = 10000.0
    eps: float = 1e-6
    seed: int = 0
    weight_std: float = 0.02
    init_device: str = ""   # where the random weights are drawn ("" = the stack's device); "cpu" gives the
                            # same weights on any device, at the cost of a slow start for the full model

    @property
    def img_tokens(self) -> int:
        return self.img_grid[0] * self.img_grid[1]

    @property
    def tokens(self) -> int:
        return self.txt_tokens + self.img_tokens

    @property
    def mlp_hidden(self) -> int:
        return self.mlp_ratio * self.hidden

    def validate(self, world: int) -> None:
        assert self.hidden == self.heads * self.head_dim, "hidden must equal heads * head_dim"
        assert sum(self.axes_dim) == self.head_dim, "rope axes must add up to head_dim"
        assert self.heads % world == 0, f"{self.heads} heads do not split over {world} ranks"
        assert self.mlp_hidden % world == 0
        assert (self.hidden // world) % 64 == 0 and (self.mlp_hidden // world) % 64 == 0, \
            "K-shards must be multiples of 64 elements (one scale tile)"


class TensorParallel:
    """Rank bookkeeping and the one collective the stack needs."""

    def __init__(self, group=None, single: bool = False):
        """``single=True`` gives a one-rank instance even inside an initialised process group (a measurement
        that one rank makes on its own must not enter collectives the other ranks never join)."""
        import torch.distributed as dist

        self._dist = dist
        if not single and dist.is_available() and dist.is_initialized():
            self.group = group
            self.rank = dist.get_rank(group)
            self.world = dist.get_world_size(group)
        else:
            self.group, self.rank, self.world = None, 0, 1
        self.all_reduce_calls = 0
        self.on_all_reduce = None   # set while a forward is being recorded in segments (DiTStack.capture_segments)

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        self.all_reduce_calls += 1
        if self.on_all_reduce is not None:
            return self.on_all_reduce(t)
        if self.world > 1:
            self._dist.all_reduce(t, op=self._dist.ReduceOp.SUM, group=self.group)
        return t

    def all_reduce_max(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            self._dist.all_reduce(t, op=self._dist.ReduceOp.MAX, group=self.group)
        return t


def rope_freqs(cfg: DiTConfig, device, dtype=torch.float32) -> torch.Tensor:
    """[1, 1, tokens, head_dim/2, 2, 2] rotation matrices [[cos, -sin], [sin, cos]].

    Position ids: text tokens (0, 0, 0), image tokens (0, row, col) on the image grid; pair i of
    axis a (axes_dim[a] / 2 pairs) turns by pos_a * theta^(-2i / axes_dim[a]).
    """
    gh, gw = cfg.img_grid
    ids = torch.zeros(cfg.tokens, 3, dtype=torch.float64)
    rows = torch.arange(gh, dtype=torch.float64).repeat_interleave(gw)
    cols = torch.arange(gw, dtype=torch.float64).repeat(gh)
    ids[cfg.txt_tokens:, 1] = rows
    ids[cfg.txt_tokens:, 2] = cols
    parts = []
    for a, d in enumerate(cfg.axes_dim):
        omega = cfg.theta ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)
        parts.append(ids[:, a:a + 1] * omega[None, :])
    ang = torch.cat(parts, dim=1)  # [tokens, head_dim / 2]
    cos, sin = ang.cos(), ang.sin()
    m = torch.stack([torch.stack([cos, -sin], dim=-1), torch.stack([sin, cos], dim=-1)], dim=-2)
    return m.to(dtype)[None, None].contiguous().to(device)


class QuantLinear:
    """One NVFP4 weight shard: packed codes [N, K/2], tiled E4M3 block scales, fp32 tensor scale."""

    def __init__(self, ops, w: torch.Tensor, tensor_scale: torch.Tensor, bias: torch.Tensor | None):
        self.ops = ops
        self.n, self.k = w.shape
        self.tensor_scale = tensor_scale.float().reshape(())
        self.qdata, self.block_scales = ops.quantize_nvfp4(w.contiguous(), self.tensor_scale)
        self.bias = bias

    @classmethod
    def from_shard(cls, ops, shard, bias: torch.Tensor | None) -> "QuantLinear":
        """From a QuantizedTensor cut out of a checkpoint (comfy_kitchen/sharding.py): nothing is re-quantized."""
        self = cls.__new__(cls)
        self.ops = ops
        self.n, self.k = shard._params.orig_shape
        self.tensor_scale = shard._params.scale.float().reshape(())
        self.qdata, self.block_scales = shard._qdata, shard._params.block_scale
        self.bias = bias
        return self

    def _alpha_for(self, act_scale: torch.Tensor) -> torch.Tensor:
        """act_scale * weight scale as a device scalar.  Static activation scales are the same tensor objects call
        after call, so the product is kept per scale tensor (a one-element multiply per GEMM was 228 launches and
        0.4 ms of a forward); a tensor that was modified in place since, or a new one, is multiplied again."""
        cache = self.__dict__.setdefault("_alphas", {})
        hit = cache.get(id(act_scale))
        if hit is not None and hit[0] is act_scale and hit[2] == act_scale._version:
            return hit[1]
        alpha = (act_scale * self.tensor_scale).reshape(1)
        capturing = act_scale.is_cuda and torch.cuda.is_current_stream_capturing()
        # (a tensor made during capture belongs to that graph; entries are never dropped, because a captured graph
        # may hold the address of a kept product: past a handful, further scales are simply not kept)
        if not capturing and (id(act_scale) in cache or len(cache) < 8):
            cache[id(act_scale)] = (act_scale, alpha, act_scale._version)
        return alpha

    def __call__(self, qx: torch.Tensor, sx: torch.Tensor, act_scale: torch.Tensor, out=None, residual=None, gate=None,
                 scatter=None) -> torch.Tensor:
        alpha = self._alpha_for(act_scale)
        extra = {} if residual is None else {"residual": residual, "gate": gate}
        if scatter is not None:
            extra["scatter"] = scatter
        return self.ops.scaled_mm_nvfp4(qx, self.qdata, act_scale, self.tensor_scale, sx, self.block_scales,
                                        bias=self.bias, out_dtype=torch.bfloat16, alpha=alpha, out=out, **extra)


def _weight_scale(w: torch.Tensor) -> torch.Tensor:
    return (w.float().abs().max() / (F4_MAX * E4M3_MAX)).reshape(())


@dataclass
class _Sites:
    """Per-tensor activation scales, one per quantisation site, keyed by name."""
    static: dict = field(default_factory=dict)
    observed: dict = field(default_factory=dict)
    recording: bool = False


class DiTStack:
    """The stack's weights for one rank and its forward pass.

    ops: a module or object with the package's operator names (default: the CUDA backend).
    """

    def __init__(self, cfg: DiTConfig, device, tp: TensorParallel | None = None, ops=None, state: dict | None = None):
        """``state``: a checkpoint of the whole (unsharded) model in the reference's key contract, as
        ``make_checkpoint`` writes it; each rank then cuts its shards out of the packed codes and tiled scales
        (no re-quantization).  Without it the weights are drawn and quantized here."""
        self._state = state
        if ops is None:
            from comfy_kitchen.backends import cuda as ops  # raises if the native library is missing
        self.cfg, self.ops, self.device = cfg, ops, torch.device(device)
        self.tp = tp or TensorParallel()
        cfg.validate(self.tp.world)
        self.sites = _Sites()
        self.exchange = None   # PeerExchange once enable_peer_exchange() has run (CUDA only)
        # the GEMM kernel can apply x += gate * y in its epilogue (CUDA backend; the CPU operator sets used by
        # the tests have no such argument)
        self.fuse_residual_in_gemm = self.device.type == "cuda" and hasattr(ops, "launch_residual_supported")
        self._xbuf = None      # the residual stream [tokens, hidden], text tokens first; updated in place
        # Sequence-parallel front end (needs the peer exchange): each rank keeps the residual stream, and runs the
        # norm -> quantize in front of the column-parallel GEMMs, for its own rows only; the quantized rows are
        # then gathered.  Switched on by enable_sequence_parallel() after calibrate().
        self.sequence_parallel = False
        self._mods = None   # all blocks' modulation vectors during a forward
        self.heads_local = cfg.heads // self.tp.world
        self.freqs = rope_freqs(cfg, self.device)
        self.double = [self._make_double(i) for i in range(cfg.n_double)]
        self.single = [self._make_single(i) for i in range(cfg.n_single)]
        self._pack_modulation()
        self._state = None

    # ------------------------------------------------------------------ weights

    def _randn(self, shape, layer: int, name: str, std: float) -> torch.Tensor:
        dev = torch.device(self.cfg.init_device) if self.cfg.init_device else self.device
        g = torch.Generator(device=dev)
        g.manual_seed((self.cfg.seed * 1_000_003 + layer * 101 + sum(map(ord, name))) & 0x7FFFFFFF)
        return (std * torch.randn(shape, generator=g, device=dev, dtype=torch.float32)).bfloat16().to(self.device)

    def _head_range(self) -> tuple[int, int]:
        """This rank's heads as a row range inside one of q / k / v (each heads * head_dim rows)."""
        hd = self.cfg.head_dim
        lo = self.tp.rank * self.heads_local * hd
        return lo, lo + self.heads_local * hd

    def _qkv_ranges(self) -> list[tuple[int, int]]:
        h = self.cfg.hidden
        lo, hi = self._head_range()
        return [(lo, hi), (h + lo, h + hi), (2 * h + lo, 2 * h + hi)]

    def _mlp_range(self, base: int = 0) -> tuple[int, int]:
        n = self.cfg.mlp_hidden // self.tp.world
        return base + self.tp.rank * n, base + (self.tp.rank + 1) * n

    def _index(self, ranges) -> torch.Tensor:
        return torch.cat([torch.arange(lo, hi, device=self.device) for lo, hi in ranges])

    def _linear(self, name: str, layer: int, shape, rows=None, cols=None, row_parallel=False) -> QuantLinear:
        """One quantized linear of this rank: the shard [rows (ranges) x cols (ranges)] of the full weight `name`
        of block `layer` ([N, K] = shape).  From the checkpoint when there is one, else drawn and quantized here
        with the per-tensor scale of the unsliced weight."""
        c = self.cfg
        key = f"{layer}.{name}."
        if self._state is not None:
            from comfy_kitchen.sharding import take_ranges
            from comfy_kitchen.tensor import QuantizedTensor, TensorCoreNVFP4Layout

            st = self._state
            params = TensorCoreNVFP4Layout.Params(scale=st[key + "weight_scale_2"].to(self.device), orig_dtype=torch.bfloat16,
                                                  orig_shape=tuple(shape),
                                                  block_scale=st[key + "weight_scale"].to(self.device).view(torch.float8_e4m3fn))
            qt = QuantizedTensor(st[key + "weight"].to(self.device), "TensorCoreNVFP4Layout", params)
            if rows is not None:
                qt = take_ranges(qt, 0, rows)
            if cols is not None:
                qt = take_ranges(qt, 1, cols)
            bias_full = st[key + "bias"].to(self.device)
        else:
            w_full = self._randn(shape, layer, name, c.weight_std)
            bias_full = self._randn((shape[0],), layer, name + "_b", c.weight_std)
            ts = _weight_scale(w_full)
            w = w_full
            if rows is not None:
                w = w[self._index(rows)]
            if cols is not None:
                w = w[:, self._index(cols)]
            qt = None
        if row_parallel:  # the partial results are summed: the bias goes in once
            bias = bias_full if self.tp.rank == 0 else None
        else:
            bias = bias_full[self._index(rows)] if rows is not None else bias_full
        bias = None if bias is None else bias.float().contiguous()
        if qt is not None:
            return QuantLinear.from_shard(self.ops, qt, bias)
        return QuantLinear(self.ops, w, ts, bias)

    def _mod(self, layer: int, n: int):
        if self._state is not None:
            return self._state[f"{layer}.mod_w"].to(self.device), self._state[f"{layer}.mod_b"].to(self.device)
        h = self.cfg.hidden
        return self._randn((n * h, h), layer, "mod_w", self.cfg.weight_std), self._randn((n * h,), layer, "mod_b", self.cfg.weight_std)

    def _make_double(self, i: int) -> dict:
        c, blk = self.cfg, {}
        h, hd = c.hidden, c.head_dim
        for s in ("img", "txt"):
            L = 1000 + 2 * i + (s == "txt")
            p = {}
            p["mod_w"], p["mod_b"] = self._mod(L, 6)
            p["qkv"] = self._linear("qkv", L, (3 * h, h), rows=self._qkv_ranges())
            p["q_norm"] = torch.ones(hd, device=self.device, dtype=torch.bfloat16)
            p["k_norm"] = torch.ones(hd, device=self.device, dtype=torch.bfloat16)
            p["proj"] = self._linear("proj", L, (h, h), cols=[self._head_range()], row_parallel=True)
            p["up"] = self._linear("up", L, (c.mlp_hidden, h), rows=[self._mlp_range()])
            p["down"] = self._linear("down", L, (h, c.mlp_hidden), cols=[self._mlp_range()], row_parallel=True)
            blk[s] = p
        return blk

    def _make_single(self, i: int) -> dict:
        c = self.cfg
        h = c.hidden
        L = 5000 + i
        p = {}
        p["mod_w"], p["mod_b"] = self._mod(L, 3)
        # linear1 rows: [q | k | v | mlp]; this rank keeps its heads of q, k, v and its slice of the MLP
        p["linear1"] = self._linear("linear1", L, (3 * h + c.mlp_hidden, h), rows=self._qkv_ranges() + [self._mlp_range(3 * h)])
        p["q_norm"] = torch.ones(c.head_dim, device=self.device, dtype=torch.bfloat16)
        p["k_norm"] = torch.ones(c.head_dim, device=self.device, dtype=torch.bfloat16)
        # linear2 columns: [attention output | MLP activations], sliced the same way
        p["linear2"] = self._linear("linear2", L, (h, h + c.mlp_hidden), cols=[self._head_range(), self._mlp_range(h)],
                                    row_parallel=True)
        return p

    def _pack_modulation(self) -> None:
        """Every block's modulation is a linear of the same conditioning vector: stack all of them into one
        weight so that a forward computes them with one matrix-vector product instead of one per block."""
        owners = [blk[s] for blk in self.double for s in ("img", "txt")] + list(self.single)
        if not owners:
            self.mod_w = self.mod_b = None
            return
        self.mod_w = torch.cat([p["mod_w"] for p in owners])
        self.mod_b = torch.cat([p["mod_b"] for p in owners])
        off = 0
        for p in owners:
            n = p["mod_w"].shape[0]
            p["mod_slice"] = (off, off + n)
            p["mod_w"], p["mod_b"] = self.mod_w[off:off + n], self.mod_b[off:off + n]   # views: no second copy
            off += n

    # ------------------------------------------------------------------ activation scales

    def _act_scale(self, site: str, x: torch.Tensor | None = None, amax: torch.Tensor | None = None) -> torch.Tensor:
        """Static scale when calibrated; otherwise amax / (6 * 448) of this call's tensor."""
        st = self.sites
        if not st.recording and site in st.static:
            return st.static[site]
        if amax is None:
            amax = x.float().abs().max()
        amax = amax.reshape(())
        if st.recording:
            prev = st.observed.get(site)
            st.observed[site] = amax if prev is None else torch.maximum(prev, amax)
        return torch.clamp(amax, min=1e-12) / (F4_MAX * E4M3_MAX)

    @torch.no_grad()
    def calibrate(self, img: torch.Tensor, txt: torch.Tensor, vec: torch.Tensor, margin: float = 1.0) -> None:
        """One forward with per-call scales; the observed maxima (over ranks too) become static scales."""
        self.sites.recording, self.sites.observed = True, {}
        try:
            self.forward(img, txt, vec)
        finally:
            self.sites.recording = False
        names = sorted(self.sites.observed)
        if names:
            packed = torch.stack([self.sites.observed[n].float() for n in names])
            self.tp.all_reduce_max(packed)
            for n, a in zip(names, packed):
                self.sites.static[n] = (torch.clamp(a * margin, min=1e-12) / (F4_MAX * E4M3_MAX)).reshape(())

    # ------------------------------------------------------------------ pieces of the forward

    def _modulation(self, p: dict, vec: torch.Tensor, n: int):
        """This block's (shift, scale, gate, ...) vectors, each [1, hidden], replicated on every rank."""
        if self._mods is not None:
            lo, hi = p["mod_slice"]
            return self._mods[:, lo:hi].chunk(n, dim=-1)
        return F.linear(F.silu(vec), p["mod_w"], p["mod_b"]).chunk(n, dim=-1)

    def _norm_quant(self, site: str, x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor):
        """LayerNorm + modulation + NVFP4 quantise in one kernel.  Without a static scale the maximum comes
        from the standalone AdaLN kernel first (calibration only)."""
        if self.sites.recording or site not in self.sites.static:
            y = self.ops.adaln(x[None], scale, shift, self.cfg.eps)
            g = self._act_scale(site, y)
        else:
            g = self.sites.static[site]
        qx, sx = self.ops.adaln_quantize_nvfp4(x[None], scale, shift, g, self.cfg.eps)
        return qx, sx, g

    def _front_end(self, parts):
        """Norm + modulation + NVFP4 for consecutive row ranges of the residual stream.
        parts: (site, row_begin, row_end, scale, shift) per range, in row order, covering the stream.
        Returns (qx, sx, g) per part.  Replicated form: one fused kernel per part over all its rows.
        Sequence-parallel form: each rank runs the kernel on its rows of each part, writing into the shared
        activation buffers, and one gather distributes all ranks' rows before the GEMMs read them."""
        if not self.sequence_parallel:
            return [self._norm_quant(site, self._xbuf[a:b], scale, shift) for site, a, b, scale, shift in parts]
        ex, out = self.exchange, []
        for site, a, b, scale, shift in parts:
            g = self.sites.static[site]
            qx, sx = ex.qx[a:b], ex.sx[a:(b + 127) // 128 * 128]      # this part's rows of the shared buffers
            lo, hi = max(ex.row_lo, a), min(ex.row_hi, b)
            if lo < hi:
                self.ops.adaln_quantize_nvfp4_rows(self._xbuf[a:b][None], scale, shift, g, qx, sx, lo - a, hi - a, self.cfg.eps)
            out.append((qx, sx.view(torch.float8_e4m3fn), g))
        ex.gather_quantized()
        return out

    def _quant(self, site: str, segments):
        """NVFP4 of the column concatenation of the segments ((tensor, activation) pairs: see
        quantize_nvfp4_gather), read in place.  Without a static scale the maximum is taken from the
        materialised activation first (calibration only)."""
        if self.sites.recording or site not in self.sites.static:
            cols = []
            for t, act in segments:
                m = t if t.dim() == 2 else t.permute(1, 0, 2).reshape(t.shape[1], -1)
                cols.append(F.gelu(m, approximate="tanh") if act == "gelu_tanh" else m)
            g = self._act_scale(site, amax=torch.stack([c.float().abs().max() for c in cols]).max())
        else:
            g = self.sites.static[site]
        qx, sx = self.ops.quantize_nvfp4_gather(segments, g)
        return qx, sx, g

    def _attend(self, parts) -> torch.Tensor:
        """parts: (qkv [tokens_i, >= 3*heads_local*head_dim], q_norm, k_norm) per segment of the joint sequence, in
        token order.  One fused kernel per segment normalises q and k per head, applies the rotary embedding and
        writes q, k, v in the layout attention reads; returns the attention output [tokens, heads_local*head_dim]."""
        c, hl = self.cfg, self.heads_local
        total = sum(x[0].shape[0] for x in parts)
        freqs = self.freqs if total == c.tokens else self.freqs[:, :, :total].contiguous()
        q = k = v = None
        off = 0
        for qkv, q_w, k_w in parts:
            q, k, v = self.ops.qk_norm_rope(qkv, q_w, k_w, freqs, hl, q, k, v, off, c.eps)
            off += qkv.shape[0]
        return F.scaled_dot_product_attention(q, k, v)[0]   # [heads_local, tokens, head_dim]; the quantizer reads it in place

    def enable_peer_exchange(self, mode: str | None = None) -> None:
        """Replace "NCCL all-reduce, then residual update" by the fused exchange kernel over peer memory
        (comfy_kitchen/tp_exchange.py).  Every rank must call this at the same point.  The residual stream then
        lives in the exchange's shared buffer."""
        from comfy_kitchen.tp_exchange import PeerExchange

        assert self.device.type == "cuda"
        n_mod = 0 if self.mod_w is None else self.mod_w.shape[0]
        self.exchange = PeerExchange(self.tp.group, self.device, self.cfg.tokens, self.cfg.hidden, torch.bfloat16, mode,
                                     extra_bytes=2 * n_mod)
        self._xbuf = self.exchange.residual
        # The blocks' modulation vectors are one matrix-vector product over 6.5 GB of weights per forward (1 ms):
        # with several ranks each keeps and multiplies only its share of the rows, and the shares are gathered.
        self._mod_rows = None
        if self.tp.world > 1 and n_mod and n_mod % (8 * self.tp.world) == 0:
            per = n_mod // self.tp.world
            lo = self.tp.rank * per
            self._mod_rows = (lo, lo + per)
            self._mod_w_shard = self.mod_w[lo:lo + per].clone()
            self._mod_b_shard = self.mod_b[lo:lo + per].clone()
            for p_ in [blk[s] for blk in self.double for s in ("img", "txt")] + list(self.single):
                p_.pop("mod_w", None), p_.pop("mod_b", None)     # (views of the full matrix)
            self.mod_w = self.mod_b = None
            self._n_mod = n_mod

    def enable_sequence_parallel(self) -> None:
        """From now on every rank updates and normalises only its rows of the residual stream (whole 128-row scale
        tiles, PeerExchange.row_bounds) and the ranks exchange the NVFP4 activation (0.56 bytes per element) instead
        of the bf16 residual.  Needs static activation scales (calibrate() runs in the replicated form, where every
        rank sees whole tensors) and a text length that is a multiple of 128 rows."""
        assert self.exchange is not None, "enable_peer_exchange() first"
        assert self.sites.static, "calibrate() first: the sequence-parallel front end needs static activation scales"
        assert self.cfg.txt_tokens % 128 == 0, "text tokens must fill whole 128-row scale tiles"
        self.sequence_parallel = True

    def try_enable_peer_exchange(self, mode: str | None = None) -> str | None:
        """enable_peer_exchange() with agreement between the ranks: the exchange is kept only if every rank
        could set it up; otherwise every rank stays on the NCCL path.  Returns None on success, else why not."""
        err = None
        try:
            self.enable_peer_exchange(mode)
        except Exception as e:  # noqa: BLE001 - any failure means "use the NCCL path"
            err = f"{type(e).__name__}: {e}"
        if self.tp.world > 1:
            ok = torch.tensor([0.0 if err else 1.0], device=self.device)
            self.tp._dist.all_reduce(ok, op=self.tp._dist.ReduceOp.MIN, group=self.tp.group)
            if float(ok.item()) < 1.0 and err is None:
                err = "another rank could not set the exchange up"
        if err:
            self.exchange, self._xbuf = None, None
        return err

    def _residual(self, rows: int) -> torch.Tensor:
        if self._xbuf is None or self._xbuf.shape[0] != rows:
            assert self.exchange is None, "the exchange buffers are sized for the configured token count"
            self._xbuf = torch.empty((rows, self.cfg.hidden), device=self.device, dtype=torch.bfloat16)
        return self._xbuf

    def _row_parallel_update(self, linears, inputs, sites, gates) -> None:
        """Row-parallel GEMMs of consecutive token ranges of the residual stream, the sum of their partial
        results over the ranks, and  x += gate * y  on the residual stream (one gate per range).
        inputs: per range the list of (tensor, activation) segments that make up the GEMM's input columns."""
        rows = [segs[0][0].shape[-2] for segs in inputs]
        x = self._xbuf
        assert sum(rows) == x.shape[0]
        fused = self.exchange is not None
        if self.tp.world == 1 and self.fuse_residual_in_gemm and self.tp.on_all_reduce is None:
            # one rank: nothing to sum, so the GEMM's epilogue applies the residual update itself, in place
            self.tp.all_reduce_calls += 1
            off = 0
            for lin, segs, site, r, gate in zip(linears, inputs, sites, rows, gates):
                qx, sx, g = self._quant(site, segs)
                lin(qx, sx, g, out=x[off:off + r], residual=x[off:off + r], gate=gate)
                off += r
            return
        if fused and self.sequence_parallel:
            # the GEMMs' epilogues deliver each tile row to the rank that owns it (reduce-scatter over NVLink while
            # the main loop runs); the owner then sums its slabs from local memory and updates its residual rows
            self.tp.all_reduce_calls += 1
            off = 0
            for lin, segs, site, r in zip(linears, inputs, sites, rows):
                qx, sx, g = self._quant(site, segs)
                lin(qx, sx, g, scatter=self.exchange.scatter_args(off))
                off += r
            two = len(gates) > 1
            self.exchange.reduce_rows(gates[0], gates[1] if two else None, rows[0] if two else 0, scattered=True)
            return
        y = self.exchange.partial if fused else torch.empty_like(x)
        off = 0
        for lin, segs, site, r in zip(linears, inputs, sites, rows):
            qx, sx, g = self._quant(site, segs)
            lin(qx, sx, g, out=y[off:off + r])
            off += r
        if fused:
            self.tp.all_reduce_calls += 1
            two = len(gates) > 1
            if self.sequence_parallel:   # (not reached: kept for a sequence-parallel run without the scattered GEMM)
                self.exchange.reduce_rows(gates[0], gates[1] if two else None, rows[0] if two else 0)
            else:
                self.exchange.exchange(gates[0], gates[1] if two else None, rows[0] if two else 0)
            return
        y = self.tp.all_reduce_sum(y)
        off = 0
        for gate, r in zip(gates, rows):
            x[off:off + r].addcmul_(gate, y[off:off + r])
            off += r

    def _double_block(self, i: int, vec: torch.Tensor) -> None:
        blk, tt = self.double[i], self._tt
        order = ("txt", "img")   # token order of the residual stream
        mods = {s: self._modulation(blk[s], vec, 6) for s in order}
        total = self._xbuf.shape[0]
        span = {"txt": (0, tt), "img": (tt, total)}
        acts = self._front_end([(f"d{i}.{s}.attn_in", *span[s], mods[s][1], mods[s][0]) for s in order])
        parts = []
        for s, (qx, sx, g) in zip(order, acts):
            parts.append((blk[s]["qkv"](qx, sx, g), blk[s]["q_norm"], blk[s]["k_norm"]))
        o = self._attend(parts)
        self._row_parallel_update([blk[s]["proj"] for s in order], [[(o[:, :tt], None)], [(o[:, tt:], None)]],
                                  [f"d{i}.{s}.attn_out" for s in order], [mods[s][2] for s in order])
        acts = self._front_end([(f"d{i}.{s}.mlp_in", *span[s], mods[s][4], mods[s][3]) for s in order])
        mids = []
        for s, (qx, sx, g) in zip(order, acts):
            mids.append([(blk[s]["up"](qx, sx, g), "gelu_tanh")])   # GELU happens inside the quantizer
        self._row_parallel_update([blk[s]["down"] for s in order], mids, [f"d{i}.{s}.mlp_mid" for s in order],
                                  [mods[s][5] for s in order])

    def _single_block(self, i: int, vec: torch.Tensor) -> None:
        p, c, hl = self.single[i], self.cfg, self.heads_local
        shift, scale, gate = self._modulation(p, vec, 3)
        (qx, sx, g), = self._front_end([(f"s{i}.in", 0, self._xbuf.shape[0], scale, shift)])
        h1 = p["linear1"](qx, sx, g)   # [tokens, q | k | v | mlp]: the fused kernel reads the first part in place
        n_qkv = 3 * hl * c.head_dim
        o = self._attend([(h1, p["q_norm"], p["k_norm"])])
        # linear2's input columns: [attention output | GELU(mlp part of h1)], both read where they are
        self._row_parallel_update([p["linear2"]], [[(o, None), (h1[:, n_qkv:], "gelu_tanh")]], [f"s{i}.mid"], [gate])

    @torch.no_grad()
    def forward(self, img: torch.Tensor, txt: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
        """img [img_tokens, hidden], txt [txt_tokens, hidden], vec [1, hidden] (bf16) -> [tokens, hidden],
        text tokens first.  Every rank receives the same inputs and returns the same (replicated) output."""
        if getattr(self, "_mod_rows", None) is not None:
            lo, hi = self._mod_rows
            mods = self.exchange.extra[:2 * self._n_mod].view(torch.bfloat16)
            mods[lo:hi].copy_(F.linear(F.silu(vec), self._mod_w_shard, self._mod_b_shard)[0])
            self.exchange.gather_extra(2 * lo, 2 * hi)
            self._mods = mods[None]
        else:
            self._mods = F.linear(F.silu(vec), self.mod_w, self.mod_b) if self.mod_w is not None else None
        tt = self._tt = txt.shape[0]
        x = self._residual(tt + img.shape[0])
        x[:tt].copy_(txt)
        x[tt:].copy_(img)
        try:
            for i in range(self.cfg.n_double):
                self._double_block(i, vec)
            for i in range(self.cfg.n_single):
                self._single_block(i, vec)
            if self.sequence_parallel:
                self.exchange.gather_residual()   # every rank ends with the whole stream again
        finally:
            self._mods = None
        return x.clone()   # the residual buffer is reused by the next forward

    __call__ = forward

    def capture(self, img: torch.Tensor, txt: torch.Tensor, vec: torch.Tensor):
        """Record one forward into a CUDA graph and return ``replay(img, txt, vec) -> out``.

        The forward is ~40 small launches per block; replaying a graph removes their host cost.  Needs static
        activation scales (call calibrate() first) so that no value-dependent host work is left in the forward.
        Inputs are copied into the graph's own buffers; the returned tensor is the graph's output buffer
        (overwritten by the next replay).  On several ranks this needs the peer exchange
        (enable_peer_exchange()): its kernels are ordinary launches and are recorded like any other, whereas a
        forward that ends its row-parallel GEMMs with NCCL calls is recorded in segments (capture_segments()).
        Every rank must capture, and later replay, in step.
        """
        assert self.tp.world == 1 or self.exchange is not None, \
            "several ranks: enable_peer_exchange() first, or use capture_segments()"
        assert self.device.type == "cuda", "graph capture needs a CUDA device"
        assert self.sites.static, "calibrate() first: capture needs static activation scales"
        bufs = [img.clone(), txt.clone(), vec.clone()]
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):  # warm up on the capture stream: lazy initialisation must not be recorded
                self.forward(*bufs)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
            out = self.forward(*bufs)

        torch.cuda.current_stream(self.device).wait_stream(side)
        if self.tp.world > 1:
            # no rank replays (and waits in an exchange kernel) while another is still recording
            torch.cuda.synchronize(self.device)
            self.tp._dist.barrier(group=self.tp.group)

        def replay(img_, txt_, vec_):
            bufs[0].copy_(img_, non_blocking=True)
            bufs[1].copy_(txt_, non_blocking=True)
            bufs[2].copy_(vec_, non_blocking=True)
            graph.replay()
            return out

        replay.graph = graph
        return replay

    def capture_best(self, img: torch.Tensor, txt: torch.Tensor, vec: torch.Tensor):
        """(replay, description): one graph per forward where that is possible (one rank, or the peer exchange
        is on), else the chain of graphs between NCCL all-reduces."""
        if self.tp.world == 1:
            return self.capture(img, txt, vec), "one CUDA graph per forward"
        if self.exchange is not None:
            how = ("sequence parallel: row-parallel GEMMs scatter their tile rows to the owning ranks, each rank sums and "
                   "normalises its rows, NVFP4 rows gathered"
                   if self.sequence_parallel else "fused all-reduce + residual kernels")
            return self.capture(img, txt, vec), "one CUDA graph per forward, exchange over peer memory inside (" + how + ")"
        return self.capture_segments(img, txt, vec), "CUDA graphs between NCCL all-reduces"

    @torch.no_grad()
    def exchange_report(self, img: torch.Tensor, txt: torch.Tensor, vec: torch.Tensor, iters: int = 20) -> dict:
        """Stand-alone timings (device events, every rank in step) of the two parts of a forward that do not
        shrink with the rank count: the exchange after every row-parallel GEMM, and the norm -> quantize front
        end that every rank runs on the whole sequence.  Multiplied out to one forward."""
        n = self.expected_all_reduces()
        x = self._residual(self.cfg.tokens)
        gate = torch.zeros(self.cfg.hidden, device=self.device, dtype=torch.bfloat16)

        def timed(fn):
            for _ in range(3):
                fn()
            torch.cuda.synchronize(self.device)
            if self.tp.world > 1:
                self.tp._dist.barrier(group=self.tp.group)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                fn()
            b.record()
            torch.cuda.synchronize(self.device)
            t = torch.tensor([a.elapsed_time(b) / iters], device=self.device, dtype=torch.float64)
            if self.tp.world > 1:
                self.tp._dist.all_reduce(t, op=self.tp._dist.ReduceOp.MAX, group=self.tp.group)
            return float(t.item())

        if self.exchange is not None and self.sequence_parallel:
            ex = self.exchange
            scale0 = torch.zeros(1, 1, self.cfg.hidden, device=self.device, dtype=torch.bfloat16)
            g0 = torch.ones((), device=self.device)

            def sp_step():
                ex.reduce_rows(gate)
                if ex.row_lo < ex.row_hi:
                    self.ops.adaln_quantize_nvfp4_rows(x[None], scale0, scale0, g0, ex.qx, ex.sx, ex.row_lo, ex.row_hi, self.cfg.eps)
                ex.gather_quantized()
            per = timed(sp_step)
            per_reduce = timed(lambda: ex.reduce_rows(gate))
            per_gather = timed(ex.gather_quantized)
            return {"all_reduce_ms": round(per * n, 3), "all_reduce_us_each": round(per * 1e3, 1),
                    "all_reduce_how": "sequence parallel: reduce of the rank's rows over peer loads + norm -> NVFP4 of those rows + "
                                      "gather of the quantized rows (peer stores)",
                    "reduce_rows_us_each": round(per_reduce * 1e3, 1), "gather_quantized_us_each": round(per_gather * 1e3, 1),
                    "all_reduce_bytes_each": int(x.numel() * 2), "elementwise_ms": 0.0,
                    "elementwise_what": "the norm -> NVFP4 front end runs on each rank's rows only (inside all_reduce_ms)"}
        if self.exchange is not None:
            per = timed(lambda: self.exchange.exchange(gate))
            what = ("fused all-reduce + residual kernel, " +
                    ("NVLink-switch reduction and broadcast (multimem)" if self.exchange.multimem else "peer loads and stores"))
        else:
            y = torch.zeros_like(x)

            def nccl():
                self.tp.all_reduce_sum(y)
                x.addcmul_(gate, y)
            per = timed(nccl)
            what = "NCCL all-reduce + addcmul"
        scale = torch.zeros(1, 1, self.cfg.hidden, device=self.device, dtype=torch.bfloat16)
        g = torch.ones((), device=self.device)
        per_norm = timed(lambda: self.ops.adaln_quantize_nvfp4(x[None], scale, scale, g, self.cfg.eps))
        return {"all_reduce_ms": round(per * n, 3), "all_reduce_us_each": round(per * 1e3, 1), "all_reduce_how": what,
                "all_reduce_bytes_each": int(x.numel() * 2),
                "elementwise_ms": round(per_norm * n, 3),
                "elementwise_what": f"norm -> NVFP4 of the whole sequence, {n} per forward, done in full on every rank"}

    def capture_segments(self, img: torch.Tensor, txt: torch.Tensor, vec: torch.Tensor):
        """Tensor-parallel variant of capture(): the forward is recorded as a chain of CUDA graphs that ends at
        every all-reduce; ``replay`` launches graph, all-reduce, graph, ... so the collectives stay ordinary NCCL
        calls between graph launches and the host issues ~2 calls per all-reduce instead of ~40 per block.
        All graphs share one memory pool and are replayed in the order they were captured.  Every rank must
        call this, and later ``replay``, in step.  Also valid on a single rank (the all-reduces are no-ops)."""
        assert self.device.type == "cuda", "graph capture needs a CUDA device"
        assert self.sites.static, "calibrate() first: capture needs static activation scales"
        bufs = [img.clone(), txt.clone(), vec.clone()]
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):   # warm up (with real all-reduces) on the capture stream
                self.forward(*bufs)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        if self.tp.world > 1:
            self.tp._dist.barrier(group=self.tp.group)   # no collective in flight while captures are open
            torch.cuda.synchronize(self.device)
        pool = torch.cuda.graph_pool_handle()
        graphs, reduces = [], []
        current = [None]

        def begin():
            g = torch.cuda.CUDAGraph()
            g.capture_begin(pool=pool, capture_error_mode="thread_local")
            current[0] = g

        def split(t: torch.Tensor) -> torch.Tensor:
            current[0].capture_end()
            graphs.append(current[0])
            reduces.append(t)
            begin()
            return t

        with torch.cuda.stream(side):
            self.tp.on_all_reduce = split
            try:
                begin()
                out = self.forward(*bufs)
                current[0].capture_end()
                graphs.append(current[0])
            finally:
                self.tp.on_all_reduce = None
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        tp = self.tp

        def replay(img_, txt_, vec_):
            bufs[0].copy_(img_, non_blocking=True)
            bufs[1].copy_(txt_, non_blocking=True)
            bufs[2].copy_(vec_, non_blocking=True)
            for k, g in enumerate(graphs):
                g.replay()
                if k < len(reduces) and tp.world > 1:
                    tp._dist.all_reduce(reduces[k], op=tp._dist.ReduceOp.SUM, group=tp.group)
            return out

        replay.graphs = graphs
        return replay

    def expected_all_reduces(self) -> int:
        return 2 * self.cfg.n_double + self.cfg.n_single


def make_checkpoint(cfg: DiTConfig, device, ops=None) -> dict:
    """The whole synthetic model as a checkpoint in the reference's key contract (samples/nvfp4_linear.py:39-80):
    per linear ``<layer>.<name>.weight`` (packed NVFP4 codes [N, K/2]), ``.weight_scale`` (tiled E4M3 block scales
    as uint8), ``.weight_scale_2`` (fp32 per-tensor scale), ``.bias``; per block ``<layer>.mod_w`` / ``.mod_b``.
    Every weight is quantized as a whole, on ``device``, from the same random draws DiTStack makes itself, so a
    stack built from this checkpoint on any number of ranks equals one built directly."""
    one = DiTStack.__new__(DiTStack)
    if ops is None:
        from comfy_kitchen.backends import cuda as ops
    one.cfg, one.ops, one.device, one._state = cfg, ops, torch.device(device), None
    h, m = cfg.hidden, cfg.mlp_hidden
    out = {}

    def put(layer, name, shape):
        w = one._randn(shape, layer, name, cfg.weight_std)
        ts = _weight_scale(w).float().reshape(1)
        q, sf = ops.quantize_nvfp4(w.contiguous(), ts)
        key = f"{layer}.{name}."
        out[key + "weight"], out[key + "weight_scale"], out[key + "weight_scale_2"] = q, sf.view(torch.uint8), ts
        out[key + "bias"] = one._randn((shape[0],), layer, name + "_b", cfg.weight_std)

    for i in range(cfg.n_double):
        for s in ("img", "txt"):
            layer = 1000 + 2 * i + (s == "txt")
            out[f"{layer}.mod_w"] = one._randn((6 * h, h), layer, "mod_w", cfg.weight_std)
            out[f"{layer}.mod_b"] = one._randn((6 * h,), layer, "mod_b", cfg.weight_std)
            for name, shape in (("qkv", (3 * h, h)), ("proj", (h, h)), ("up", (m, h)), ("down", (h, m))):
                put(layer, name, shape)
    for i in range(cfg.n_single):
        layer = 5000 + i
        out[f"{layer}.mod_w"] = one._randn((3 * h, h), layer, "mod_w", cfg.weight_std)
        out[f"{layer}.mod_b"] = one._randn((3 * h,), layer, "mod_b", cfg.weight_std)
        put(layer, "linear1", (3 * h + m, h))
        put(layer, "linear2", (h, h + m))
    return out


def gemm_flops_per_forward(cfg: DiTConfig) -> float:
    """Multiply-add work of the quantized linears of one forward, in flop (2 per multiply-add)."""
    h, m = cfg.hidden, cfg.mlp_hidden
    per_token_double = 2 * (3 * h * h + h * h + 2 * h * m)      # qkv, proj, up, down per stream token
    per_token_single = 2 * ((3 * h + m) * h + (h + m) * h)       # linear1, linear2
    return float(cfg.tokens) * (cfg.n_double * per_token_double + cfg.n_single * per_token_single)


def attention_flops_per_forward(cfg: DiTConfig) -> float:
    return 4.0 * cfg.tokens * cfg.tokens * cfg.hidden * (cfg.n_double + cfg.n_single)


def reference_forward(stack: DiTStack, img: torch.Tensor, txt: torch.Tensor, vec: torch.Tensor, dequant) -> torch.Tensor:
    """The same graph with every quantized linear replaced by bf16 F.linear on the dequantized weight shard
    (dequant(qdata, tensor_scale, block_scales) -> bf16 [N, K]) and unquantised activations.  World size 1 only;
    the tests use it to bound the quantisation error of the stack."""
    assert stack.tp.world == 1
    c, ops = stack.cfg, stack.ops

    def lin(q: QuantLinear, x):
        w = dequant(q.qdata, q.tensor_scale, q.block_scales)
        return F.linear(x, w, None if q.bias is None else q.bias.to(x.dtype))

    def ln_mod(x, scale, shift):
        return (F.layer_norm(x.float(), (c.hidden,), eps=c.eps) * (1 + scale.float()) + shift.float()).to(x.dtype)

    def heads(t3):
        t = t3.shape[0]
        return t3.view(t, 3, c.heads, c.head_dim).unbind(1)

    def rope(x):  # x [1, heads, tokens, head_dim]
        f = stack.freqs[:, :, :x.shape[2]].to(torch.float32)
        xp = x.float().reshape(*x.shape[:-1], -1, 1, 2)
        return (f[..., 0] * xp[..., 0] + f[..., 1] * xp[..., 1]).reshape(x.shape).to(x.dtype)

    def rms(x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + c.eps) * w.float()).to(x.dtype)

    def attend(q, k, v):
        q = rope(q.permute(1, 0, 2)[None])
        k = rope(k.permute(1, 0, 2)[None])
        o = F.scaled_dot_product_attention(q, k, v.permute(1, 0, 2)[None])
        return o[0].permute(1, 0, 2).reshape(q.shape[2], c.hidden)

    tt = c.txt_tokens
    for i in range(c.n_double):
        blk = stack.double[i]
        xs = {"img": img, "txt": txt}
        mods = {s: stack._modulation(blk[s], vec, 6) for s in xs}
        qs, ks, vs = [], [], []
        for s in ("txt", "img"):
            q, k, v = heads(lin(blk[s]["qkv"], ln_mod(xs[s], mods[s][1], mods[s][0])))
            qs.append(rms(q, blk[s]["q_norm"])); ks.append(rms(k, blk[s]["k_norm"])); vs.append(v)
        o = attend(torch.cat(qs), torch.cat(ks), torch.cat(vs))
        for s, osl in (("txt", o[:tt]), ("img", o[tt:])):
            xs[s] = torch.addcmul(xs[s], mods[s][2], lin(blk[s]["proj"], osl))
            hmid = F.gelu(lin(blk[s]["up"], ln_mod(xs[s], mods[s][4], mods[s][3])), approximate="tanh")
            xs[s] = torch.addcmul(xs[s], mods[s][5], lin(blk[s]["down"], hmid))
        img, txt = xs["img"], xs["txt"]
    x = torch.cat([txt, img])
    for i in range(c.n_single):
        p = stack.single[i]
        shift, scale, gate = stack._modulation(p, vec, 3)
        h1 = lin(p["linear1"], ln_mod(x, scale, shift))
        q, k, v = heads(h1[:, :3 * c.hidden].contiguous())
        o = attend(rms(q, p["q_norm"]), rms(k, p["k_norm"]), v)
        mid = torch.cat([o, F.gelu(h1[:, 3 * c.hidden:], approximate="tanh")], dim=1)
        x = torch.addcmul(x, gate, lin(p["linear2"], mid))
    return x
