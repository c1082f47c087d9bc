"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the NVFP4 linear sweep of the Flux-like MMDiT shapes): for token counts
M = 4608 x {1, 2, 4} and layers (N, K) in {(9216,3072) QKV, (3072,3072) proj,
(12288,3072) MLP-up, (3072,12288) MLP-down}, one "linear" = activation front end
(fused LayerNorm+AdaLN -> NVFP4 quantize for the K=3072 layers, whose input is the
hidden state; plain NVFP4 quantize for MLP-down, whose input is the MLP activation)
followed by the NVFP4 block-scaled GEMM with fp32 bias and bf16 output.  One step =
all 12 linears.  Synthetic data: activations N(0,1), weights N(0,0.02), modulation
N(0,0.1), fixed seeds; weights are quantized once outside the timed region, as in
inference.

Printed JSON (one line, rank 0):
  value     TFLOP/s of the whole job (2*M*N*K per linear), inputs resident in HBM
  e2e       the same metric with the activations starting in pinned host memory and the
            outputs read back to the host inside the timed region (copies and kernels overlap on three streams)
  roofline  the NVFP4 GEMM kernel against the tensor peak (4 x the measured sustained bf16 GEMM rate: dense FP4 is
            4 x dense bf16 on this part)
  cpu_baseline  the CPU oracle (a port of the reference's eager arithmetic) on a bounded sample
  quantizers    GB/s of the memory-bound kernels at the largest sweep shape
With --impl reference the CPU oracle is what is timed (the reference's own path for this
workload runs on the host cores; it cannot execute block-scaled GEMMs on a CPU, so the
GEMM there is dequantize -> fp32 matmul, as the reference's tests do).

N > 1 (torchrun): every rank runs the same sweep on its own tokens (the linears are
independent per token: no collective in the data path); value = N x per-rank work / max time.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "comfy-kitchen_b200"), ROOT):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

LAYERS = [("qkv", 9216, 3072), ("proj", 3072, 3072), ("mlp_up", 12288, 3072), ("mlp_down", 3072, 12288)]
BATCHES = [1, 2, 4]
TOKENS = 4608
HIDDEN = 3072


def step_flops() -> float:
    return float(sum(2.0 * TOKENS * b * n * k for b in BATCHES for _, n, k in LAYERS))


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "_source": "fallback"}


def gemm_traffic() -> dict:
    """DRAM bytes of one GEMM launch as ncu counted them, read from the committed capture summary (lines
    `dram_read_bytes:`, `dram_write_bytes:`, `captured:` of the profile file), never a literal here."""
    import re

    path = os.path.join(ROOT, "profiles", "gemm_blockscaled_nvfp4_4608x9216x3072.md")
    try:
        text = open(path).read()
        rd = float(re.search(r"^dram_read_bytes:\s*([0-9.eE+]+)", text, re.M).group(1))
        wr = float(re.search(r"^dram_write_bytes:\s*([0-9.eE+]+)", text, re.M).group(1))
        cap = re.search(r"^captured:\s*(.+)$", text, re.M)
        return {"traffic": rd + wr, "traffic_case": "M4608 N9216 K3072, one launch: "
                f"{rd / 1e6:.1f} MB read, {wr / 1e6:.1f} MB written (algorithmic: 23.9 MB operands + scales, 84.9 MB output)",
                "traffic_source": "profiles/" + os.path.basename(path) + (f" ({cap.group(1).strip()})" if cap else "")}
    except (OSError, AttributeError, ValueError):
        return {"traffic": None, "traffic_source": "no capture summary found"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        clocks, mx, reasons = [], None, set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        # the median of the upper half: samples taken under load (idle samples sit at the floor)
        load = clocks[len(clocks) // 2:] if clocks else []
        return {"sm_mhz": load[len(load) // 2] if load else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clocks)}


# ----------------------------------------------------------------------------- our arm


class Workload:
    """Device-resident tensors of the sweep plus the pinned host copies for the e2e leg."""

    def __init__(self, device, seed: int):
        from comfy_kitchen.backends import cuda as ck

        self.ck = ck
        self.device = device
        g = torch.Generator(device=device).manual_seed(seed)
        self.weights = {}
        for name, n, k in LAYERS:
            w = (0.02 * torch.randn(n, k, device=device, generator=g)).bfloat16()
            gw = (w.float().abs().max() / (6 * 448)).float().reshape(1)
            qw, sw = ck.quantize_nvfp4(w, gw)
            bias = (0.02 * torch.randn(n, device=device, generator=g)).float()
            self.weights[name] = (qw, sw, gw, bias)
            del w
        self.acts = {}
        for b in BATCHES:
            x = torch.randn(b, TOKENS, HIDDEN, device=device, generator=g).bfloat16()
            shift = (0.1 * torch.randn(b, 1, HIDDEN, device=device, generator=g)).bfloat16()
            scale = (0.1 * torch.randn(b, 1, HIDDEN, device=device, generator=g)).bfloat16()
            h = torch.randn(b * TOKENS, 4 * HIDDEN, device=device, generator=g).bfloat16()
            # static per-tensor activation scales (calibrated once, like input_scale of a checkpoint)
            y = ck.adaln(x, scale, shift, 1e-6)
            gx = (y.float().abs().max() / (6 * 448)).float().reshape(1)
            gh = (h.float().abs().max() / (6 * 448)).float().reshape(1)
            del y
            self.acts[b] = (x, shift, scale, h, gx, gh)
        self.alphas = {(b, name): self.acts[b][4 if k == HIDDEN else 5] * self.weights[name][2]
                       for b in BATCHES for name, _, k in LAYERS}
        self.gemm_events: list[tuple[torch.cuda.Event, torch.cuda.Event, float]] = []
        self.gemm_keys: list[str] = []

    def linear(self, b: int, name: str, x, shift, scale, h, gx, gh, record: bool):
        ck = self.ck
        qw, sw, gw, bias = self.weights[name]
        n, k = qw.shape[0], qw.shape[1] * 2
        if k == HIDDEN:
            qa, sa = ck.adaln_quantize_nvfp4(x, scale, shift, gx, 1e-6)
            ga = gx
        else:
            qa, sa = ck.quantize_nvfp4(h, gh)
            ga = gh
        if record:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        out = ck.scaled_mm_nvfp4(qa, qw, ga, gw, sa, sw, bias=bias, out_dtype=torch.bfloat16, alpha=self.alphas[(b, name)])
        if record:
            e1.record()
            self.gemm_events.append((e0, e1, 2.0 * TOKENS * b * n * k))
            self.gemm_keys.append(f"{TOKENS * b}x{n}x{k}")
        return out

    def step(self, record: bool = False):
        outs = None
        for b in BATCHES:
            x, shift, scale, h, gx, gh = self.acts[b]
            for name, _, _ in LAYERS:
                outs = self.linear(b, name, x, shift, scale, h, gx, gh, record)
        return outs

    # ---- e2e: activations start in pinned host memory, outputs end there
    def make_host(self):
        self.host_in, self.host_out = {}, {}
        for b in BATCHES:
            x, shift, scale, h, gx, gh = self.acts[b]
            self.host_in[b] = (x.cpu().pin_memory(), h.cpu().pin_memory())
            self.host_out[b] = {name: torch.empty(b * TOKENS, n, dtype=torch.bfloat16).pin_memory() for name, n, _ in LAYERS}
        h2d = sum(3 * xi.numel() * 2 + hi.numel() * 2 for xi, hi in self.host_in.values())
        d2h = sum(t.numel() * 2 for d in self.host_out.values() for t in d.values())
        return h2d, d2h

    def step_e2e(self):
        """Every linear is an independent call whose input crosses the bus and whose output goes back.  Three
        streams (host-to-device copies, kernels, device-to-host copies) chained by events, so the copy of the
        next input and of the previous output overlap the kernels of the current linear."""
        if not hasattr(self, "s_in"):
            self.s_in, self.s_out = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)
        cur = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(cur)
        for b in BATCHES:
            _, shift, scale, _, gx, gh = self.acts[b]
            hx, hh = self.host_in[b]
            for name, _, k in LAYERS:
                with torch.cuda.stream(self.s_in):
                    dev_in = (hx if k == HIDDEN else hh).to(self.device, non_blocking=True)
                    ready = torch.cuda.Event()
                    ready.record(self.s_in)
                cur.wait_event(ready)
                dev_in.record_stream(cur)
                if k == HIDDEN:
                    out = self.linear(b, name, dev_in, shift, scale, None, gx, gh, False)
                else:
                    out = self.linear(b, name, None, shift, scale, dev_in, gx, gh, False)
                done = torch.cuda.Event()
                done.record(cur)
                self.s_out.wait_event(done)
                with torch.cuda.stream(self.s_out):
                    self.host_out[b][name].copy_(out, non_blocking=True)
                out.record_stream(self.s_out)
        cur.wait_stream(self.s_out)


SWEEP_M = (1024, 4608, 18432, 65536)
SWEEP_K = (3072, 12288)


class _GraphLoop:
    """A list of launches recorded once into a CUDA graph, so that replaying them costs no host time per launch
    (a Python call into the library takes longer than the small kernels run)."""

    def __init__(self, fns, device):
        self.n = len(fns)
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for f in fns:   # warm up on the capture stream: lazy initialisation must not be recorded
                f()
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=side):
            for f in fns:
                f()
        torch.cuda.current_stream(device).wait_stream(side)
        self.graph.replay()
        torch.cuda.synchronize(device)

    def seconds_per_launch(self, reps: int) -> float:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            self.graph.replay()
        b.record()
        b.synchronize()
        return a.elapsed_time(b) / (reps * self.n) * 1e-3


def _rotating_time(make_fn, n_sets: int, iters: int) -> float:
    """Seconds per launch: one launch per tensor set, recorded into a CUDA graph and replayed back to back; the
    sets together exceed L2, so no launch finds its input there."""
    loop = _GraphLoop([make_fn(i) for i in range(n_sets)], torch.cuda.current_device())
    return loop.seconds_per_launch(max(2, iters // n_sets))


def quantizer_sweep(device, hbm_gbs: float) -> dict:
    """The memory-bound kernels on every shape of the sweep (M in SWEEP_M, K in SWEEP_K, bf16): GB/s =
    algorithmic bytes / time per launch and the fraction of the measured copy bandwidth.  Launches run back to
    back over rotating tensor sets larger than L2 (300 MB per op at least)."""
    from comfy_kitchen.backends import cuda as ck

    g = torch.Generator(device=device).manual_seed(1)
    rows = []
    for M in SWEEP_M:
        for K in SWEEP_K:
            n = M * K
            n_sets = max(1, min(16, -(-(300 << 20) // (2 * n))))
            iters = max(3 * n_sets, 6)
            xs = []
            for _ in range(n_sets):
                x = torch.randn(M, K, device=device, generator=g)
                x = torch.where(torch.rand(M, K, device=device, generator=g) < 0.001, 50.0 * x, x).bfloat16()
                xs.append(x)
            amax = max(float(x.float().abs().max()) for x in xs)
            g4 = torch.tensor([amax / (6 * 448)], device=device)
            s8 = torch.tensor([amax / 448], device=device)
            res = {}
            res["quantize_nvfp4"] = 2.5625 * n / _rotating_time(lambda i: (lambda: ck.quantize_nvfp4(xs[i], g4)), n_sets, iters)
            q4 = [ck.quantize_nvfp4(x, g4) for x in xs]
            res["dequantize_nvfp4"] = 2.5625 * n / _rotating_time(lambda i: (lambda: ck.dequantize_nvfp4(q4[i][0], g4, q4[i][1])), n_sets, iters)
            del q4
            res["quantize_mxfp8"] = 3.03125 * n / _rotating_time(lambda i: (lambda: ck.quantize_mxfp8(xs[i])), n_sets, iters)
            q8 = [ck.quantize_mxfp8(x) for x in xs]
            res["dequantize_mxfp8"] = 3.03125 * n / _rotating_time(lambda i: (lambda: ck.dequantize_mxfp8(q8[i][0], q8[i][1])), n_sets, iters)
            del q8
            res["quantize_fp8"] = 3.0 * n / _rotating_time(lambda i: (lambda: ck.quantize_per_tensor_fp8(xs[i], s8)), n_sets, iters)
            qf = [ck.quantize_per_tensor_fp8(x, s8) for x in xs]
            res["dequantize_fp8"] = 3.0 * n / _rotating_time(lambda i: (lambda: ck.dequantize_per_tensor_fp8(qf[i], s8)), n_sets, iters)
            del qf, xs
            rows.append({"shape": [M, K], "sets": n_sets,
                         **{k: {"gbs": round(v / 1e9, 0), "frac": round(v / 1e9 / hbm_gbs, 3)} for k, v in res.items()}})
    return {"unit": "GB/s", "hbm_peak": hbm_gbs, "l2": "rotating tensor sets larger than L2", "shapes": rows}


def front_end_and_rope(device, hbm_gbs: float) -> dict:
    """The fused LayerNorm+AdaLN -> NVFP4 front end on the three token counts of the GEMM sweep (rows of 3072) and
    RoPE on q, k [B, 24, 4608, 128] with an fp32 table, B = 1, 2, 4: GB/s of algorithmic bytes and the fraction of
    the measured copy bandwidth; rotating tensor sets larger than L2."""
    from comfy_kitchen.backends import cuda as ck

    g = torch.Generator(device=device).manual_seed(2)
    out = {"unit": "GB/s", "hbm_peak": hbm_gbs, "adaln_quantize_nvfp4": [], "rope": []}
    for bsz in BATCHES:
        M = TOKENS * bsz
        n_sets = max(2, min(16, -(-(300 << 20) // (2 * M * HIDDEN))))
        xs = [torch.randn(bsz, TOKENS, HIDDEN, device=device, generator=g).bfloat16() for _ in range(n_sets)]
        sc = (0.1 * torch.randn(bsz, 1, HIDDEN, device=device, generator=g)).bfloat16()
        sh = (0.1 * torch.randn(bsz, 1, HIDDEN, device=device, generator=g)).bfloat16()
        gx = torch.tensor([6.0 / (6 * 448)], device=device)
        t = _rotating_time(lambda i: (lambda: ck.adaln_quantize_nvfp4(xs[i], sc, sh, gx, 1e-6)), n_sets, 4 * n_sets)
        by = 2.5625 * M * HIDDEN + 4.0 * bsz * HIDDEN
        out["adaln_quantize_nvfp4"].append({"shape": [M, HIDDEN], "us": round(t * 1e6, 1), "gbs": round(by / t / 1e9, 0),
                                            "frac": round(by / t / 1e9 / hbm_gbs, 3)})
        del xs
        n_sets = max(2, -(-(300 << 20) // (4 * bsz * 24 * TOKENS * 128)))
        qs = [torch.randn(bsz, 24, TOKENS, 128, device=device, generator=g).bfloat16() for _ in range(n_sets)]
        ks = [torch.randn(bsz, 24, TOKENS, 128, device=device, generator=g).bfloat16() for _ in range(n_sets)]
        fr = torch.randn(bsz, 1, TOKENS, 64, 2, 2, device=device, generator=g)
        t = _rotating_time(lambda i: (lambda: ck.apply_rope(qs[i], ks[i], fr)), n_sets, 4 * n_sets)
        by = 8.0 * qs[0].numel() + 4.0 * fr.numel()
        out["rope"].append({"shape": list(qs[0].shape), "us": round(t * 1e6, 1), "gbs": round(by / t / 1e9, 0),
                            "frac": round(by / t / 1e9 / hbm_gbs, 3)})
        del qs, ks
    return out


def host_overhead(device, calls: int = 3000) -> dict:
    """Host microseconds per call on tiny tensors (the GPU keeps up, so wall time is host time): the public API
    as it is (dispatcher bypassed for plain eager tensors), the same call forced through torch's custom-op
    dispatcher (what every call cost before, and what the reference's call path pays:
    comfy_kitchen/registry.py:180-233 plus torch.library), the backend function alone, and the GEMM launcher
    with and without its cache of encoded tensor maps."""
    import comfy_kitchen as ckp
    from comfy_kitchen.backends import cuda as ck

    x = torch.randn(128, 256, device=device).bfloat16()
    g = torch.tensor([0.01], device=device)

    def per_call(fn):
        for _ in range(50):
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(calls):
            fn()
        dt = time.perf_counter() - t0
        torch.cuda.synchronize()
        return round(dt / calls * 1e6, 1)

    out = {"unit": "us per call (host)", "calls": calls}
    out["quantize_nvfp4_public_api"] = per_call(lambda: ckp.quantize_nvfp4(x, g))
    out["quantize_nvfp4_through_dispatcher"] = per_call(lambda: torch.ops.comfy_kitchen.quantize_nvfp4(x, g, 0.0, False, True))
    out["quantize_nvfp4_backend_function"] = per_call(lambda: ck.quantize_nvfp4(x, g))
    qx, sx = ck.quantize_nvfp4(x, g)
    w = torch.randn(256, 256, device=device).bfloat16()
    qw, sw = ck.quantize_nvfp4(w, g)
    alpha = g * g
    y = torch.empty(128, 256, device=device, dtype=torch.bfloat16)
    gemm = lambda: ck.scaled_mm_nvfp4(qx, qw, g, g, sx, sw, out_dtype=torch.bfloat16, alpha=alpha, out=y)  # noqa: E731
    out["scaled_mm_nvfp4_backend_function"] = per_call(gemm)
    ck.set_option("gemm_map_cache", 0)
    try:
        out["scaled_mm_nvfp4_backend_function_no_map_cache"] = per_call(gemm)
    finally:
        ck.set_option("gemm_map_cache", 1)
    return out


def _library_scaled_mm(kind: str, qa, qb, sa, sb, ga, gb, bias):
    """The reference's eager path for the block-scaled GEMMs on a CUDA device: torch's scaled_mm, i.e. the
    cuBLASLt kernel (comfy_kitchen/backends/eager/quantization.py:224-248 and :369-404 through
    comfy_kitchen/scaled_mm_v2.py:38-74).  Operands are this GPU's own memory."""
    from comfy_kitchen.scaled_mm_v2 import ScalingType, SwizzleType, scaled_mm_v2

    if kind == "nvfp4":
        return scaled_mm_v2(
            qa.view(torch.float4_e2m1fn_x2), qb.view(torch.float4_e2m1fn_x2).t(),
            scale_a=[sa.view(-1), ga], scale_b=[sb.view(-1), gb], bias=bias, out_dtype=torch.bfloat16,
            scale_recipe_a=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
            scale_recipe_b=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
            swizzle_a=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
            swizzle_b=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE])
    return scaled_mm_v2(qa, qb.t(), scale_a=sa, scale_b=sb, bias=bias, out_dtype=torch.bfloat16,
                        scale_recipe_a=ScalingType.BlockWise1x32, scale_recipe_b=ScalingType.BlockWise1x32,
                        swizzle_a=SwizzleType.SWIZZLE_32_4_4, swizzle_b=SwizzleType.SWIZZLE_32_4_4)


def gemm_vs_library(device, kinds=("nvfp4", "mxfp8"), rounds: int = 5) -> dict:
    """Our block-scaled GEMMs beside the library's (cuBLASLt through torch's scaled_mm, the reference's eager
    call) on the twelve sweep shapes, same process, same operands.  Per shape and implementation the launches over
    rotating operand sets (together larger than L2, at least two) are recorded into a CUDA graph; the two graphs
    are replayed in turn, ours / library / ours / ..., so that clock drift under the power cap hits both alike,
    and the median round counts.  Reports TFLOP/s per shape and the ratio ours / library."""
    from comfy_kitchen.backends import cuda as ck

    g = torch.Generator(device=device).manual_seed(7)
    out = {}
    for kind in kinds:
        rows, lib_note = [], None
        for bsz in BATCHES:
            for name, n, k in LAYERS:
                m = TOKENS * bsz
                set_bytes = m * k // (2 if kind == "nvfp4" else 1) + n * k // (2 if kind == "nvfp4" else 1) + 2 * m * n
                n_sets = max(2, min(8, -(-(300 << 20) // set_bytes)))
                ours, lib = [], []
                diff = None
                for i in range(n_sets):
                    x = torch.randn(m, k, device=device, generator=g).bfloat16()
                    w = (0.02 * torch.randn(n, k, device=device, generator=g)).bfloat16()
                    bias16 = (0.02 * torch.randn(n, device=device, generator=g)).bfloat16()
                    if kind == "nvfp4":
                        gx = (x.float().abs().max() / (6 * 448)).float().reshape(1)
                        gw = (w.float().abs().max() / (6 * 448)).float().reshape(1)
                        qx, sx = ck.quantize_nvfp4(x, gx)
                        qw, sw = ck.quantize_nvfp4(w, gw)
                        alpha = gx * gw
                        ours.append(lambda qx=qx, qw=qw, gx=gx, gw=gw, sx=sx, sw=sw, b=bias16, al=alpha:
                                    ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, bias=b, out_dtype=torch.bfloat16, alpha=al))
                    else:
                        gx = gw = None
                        qx, sx = ck.quantize_mxfp8(x)
                        qw, sw = ck.quantize_mxfp8(w)
                        ours.append(lambda qx=qx, qw=qw, sx=sx, sw=sw, b=bias16:
                                    ck.scaled_mm_mxfp8(qx, qw, sx, sw, bias=b, out_dtype=torch.bfloat16))
                    lib.append(lambda qx=qx, qw=qw, sx=sx, sw=sw, gx=gx, gw=gw, b=bias16:
                               _library_scaled_mm(kind, qx, qw, sx, sw, gx, gw, b))
                    del x, w
                try:
                    y, y_lib = ours[0](), lib[0]()
                    torch.cuda.synchronize()
                    diff = (y.float() - y_lib.float()).abs().max().item() / max(y_lib.float().abs().max().item(), 1e-30)
                    loop_lib = _GraphLoop(lib, device)
                except Exception as e:  # the library leg is a comparison, not the product: report and go on
                    loop_lib, lib_note = None, f"{type(e).__name__}: {str(e)[:160]}"
                loop_ours = _GraphLoop(ours, device)
                reps = max(2, 16 // n_sets)
                t_o, t_l = [], []
                for _ in range(rounds):
                    t_o.append(loop_ours.seconds_per_launch(reps))
                    if loop_lib:
                        t_l.append(loop_lib.seconds_per_launch(reps))
                t_o.sort()
                t_l.sort()
                fl = 2.0 * m * n * k / 1e12
                row = {"shape": [m, n, k], "sets": n_sets, "ours_tflops": round(fl / t_o[len(t_o) // 2], 0)}
                if loop_lib:
                    row["library_tflops"] = round(fl / t_l[len(t_l) // 2], 0)
                    row["ratio"] = round(t_l[len(t_l) // 2] / t_o[len(t_o) // 2], 3)
                    row["max_abs_diff_over_max"] = round(diff, 5)
                rows.append(row)
                del ours, lib, loop_ours, loop_lib
        ratios = [r["ratio"] for r in rows if "ratio" in r]
        out[kind] = {"shapes": rows, "library": "cuBLASLt via torch scaled_mm (the reference's eager call), bf16 bias",
                     "timing": f"median of {rounds} rounds, each a CUDA graph of launches over rotating operand sets larger "
                               "than L2, ours and the library's graph replayed in turn"}
        if ratios:
            prod = 1.0
            for r in ratios:
                prod *= r
            out[kind]["ratio_geomean"] = round(prod ** (1.0 / len(ratios)), 3)
            out[kind]["ratio_min"] = min(ratios)
        if lib_note:
            out[kind]["library_error"] = lib_note
    return out


# ----------------------------------------------------------------------------- CPU arm


def cpu_sample_step(rows: int, threads: int) -> tuple[float, float]:
    """One pass of the same 4 layers on `rows` tokens with the CPU oracle; returns (seconds, flops)."""
    from oracle import ck_oracle as orc

    orc.set_threads(threads)
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, rows, HIDDEN, generator=g).bfloat16()
    shift = (0.1 * torch.randn(1, 1, HIDDEN, generator=g)).bfloat16()
    scale = (0.1 * torch.randn(1, 1, HIDDEN, generator=g)).bfloat16()
    h = torch.randn(rows, 4 * HIDDEN, generator=g).bfloat16()
    cache = getattr(cpu_sample_step, "_w", None)
    if cache is None:
        cache = {}
        for name, n, k in LAYERS:
            w = (0.02 * torch.randn(n, k, generator=g)).bfloat16()
            gw = (w.float().abs().max() / (6 * 448)).float()
            qw, sw = orc.quantize_nvfp4(w, gw)
            cache[name] = (qw, sw, gw, (0.02 * torch.randn(n, generator=g)).float())
        cpu_sample_step._w = cache
    gx, gh = torch.tensor(0.002), torch.tensor(0.002)
    t0 = time.perf_counter()
    flops = 0.0
    for name, n, k in LAYERS:
        qw, sw, gw, bias = cache[name]
        if k == HIDDEN:
            y = orc.adaln(x, scale, shift, 1e-6).reshape(rows, HIDDEN)
            qa, sa = orc.quantize_nvfp4(y, gx)
            ga = gx
        else:
            qa, sa = orc.quantize_nvfp4(h, gh)
            ga = gh
        orc.scaled_mm_nvfp4(qa, qw, ga, gw, sa, sw, bias=bias, out_dtype=torch.bfloat16)
        flops += 2.0 * rows * n * k
    return time.perf_counter() - t0, flops


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows = 512
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_sample_step(rows, threads)
    t_total, f_total = 0.0, 0.0
    for _ in range(args.steps):
        t, f = cpu_sample_step(rows, threads)
        t_total += t
        f_total += f
    value = f_total / t_total / 1e12
    sample = f"{rows} tokens x 4 layers per step (of 32256 tokens x 4 layers), CPU oracle, dequantize->fp32 matmul"
    line = {
        "impl": "reference", "metric": "nvfp4_linear_throughput", "value": round(value, 4), "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(t_total / args.steps * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x e4m3 block scales), fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": "NVFP4 linear sweep, Flux-like MMDiT shapes (configs[2])", "tokens": [TOKENS * b for b in BATCHES],
                   "layers": [[n, k] for _, n, k in LAYERS], "l2": "inputs larger than L2"},
        "cpu_baseline": {"value": round(value, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 4), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def max_over_ranks(elapsed_ms: float, dist, device) -> float:
    """The slowest rank's device time: what a multi-GPU number is quoted on."""
    if dist is None:
        return float(elapsed_ms)
    t = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def job_throughput(world: int, flops_per_rank_step: float, steps: int, elapsed_ms: float) -> float:
    """Whole-job TFLOP/s when every rank does `flops_per_rank_step` per step (token-sharded, weak scaling)."""
    return world * flops_per_rank_step * steps / (elapsed_ms * 1e-3) / 1e12


def run_case(args) -> None:
    """One kernel on one shape, timed with CUDA events (small, self-contained: what the ncu captures run)."""
    from comfy_kitchen.backends import cuda as ck

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    M, N, K = args.m, args.n, args.k
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(M, K, device=dev, generator=g).bfloat16()
    gx = (x.float().abs().max() / (6 * 448)).float().reshape(1)
    work, unit = None, "GB/s"
    if args.case in ("gemm_nvfp4", "gemm_mxfp8"):
        w = (0.02 * torch.randn(N, K, device=dev, generator=g)).bfloat16()
        bias = (0.02 * torch.randn(N, device=dev, generator=g)).float()
        work, unit = 2.0 * M * N * K / 1e3, "TFLOP/s"
        if args.case == "gemm_nvfp4":
            gw = (w.float().abs().max() / (6 * 448)).float().reshape(1)
            qx, sx = ck.quantize_nvfp4(x, gx)
            qw, sw = ck.quantize_nvfp4(w, gw)
            alpha = gx * gw
            fn = lambda: ck.scaled_mm_nvfp4(qx, qw, gx, gw, sx, sw, bias=bias, out_dtype=torch.bfloat16, alpha=alpha)  # noqa: E731
        else:
            qx, sx = ck.quantize_mxfp8(x)
            qw, sw = ck.quantize_mxfp8(w)
            fn = lambda: ck.scaled_mm_mxfp8(qx, qw, sx, sw, bias=bias, out_dtype=torch.bfloat16)  # noqa: E731
    elif args.case == "quantize_nvfp4":
        work, fn = 2.5625 * M * K, (lambda: ck.quantize_nvfp4(x, gx))
    elif args.case == "dequantize_nvfp4":
        q, sf = ck.quantize_nvfp4(x, gx)
        work, fn = 2.5625 * M * K, (lambda: ck.dequantize_nvfp4(q, gx, sf))
    elif args.case == "quantize_mxfp8":
        work, fn = 3.03125 * M * K, (lambda: ck.quantize_mxfp8(x))
    elif args.case == "quantize_fp8":
        s8 = gx * 6
        work, fn = 3.0 * M * K, (lambda: ck.quantize_per_tensor_fp8(x, s8))
    elif args.case == "adaln_quantize_nvfp4":
        xs = x.view(1, M, K)
        sc = (0.1 * torch.randn(1, 1, K, device=dev, generator=g)).bfloat16()
        sh = (0.1 * torch.randn(1, 1, K, device=dev, generator=g)).bfloat16()
        work, fn = 2.5625 * M * K, (lambda: ck.adaln_quantize_nvfp4(xs, sc, sh, gx, 1e-6))
    elif args.case == "adaln":
        xs = x.view(1, M, K)
        sc = (0.1 * torch.randn(1, 1, K, device=dev, generator=g)).bfloat16()
        sh = (0.1 * torch.randn(1, 1, K, device=dev, generator=g)).bfloat16()
        work, fn = 4.0 * M * K, (lambda: ck.adaln(xs, sc, sh, 1e-6))
    elif args.case == "rope":
        q = torch.randn(M // 4608 or 1, 24, 4608, 128, device=dev, generator=g).bfloat16()
        k = torch.randn_like(q)
        fr = torch.randn(q.shape[0], 1, 4608, 64, 2, 2, device=dev, generator=g)
        work, fn = 8.0 * q.numel() + 4.0 * fr.numel(), (lambda: ck.apply_rope(q, k, fr))
    elif args.case == "qk_norm_rope":
        # --m tokens, --n heads: the QKV GEMM's output [tokens, 3 * heads * 128] -> q, k, v [1, heads, tokens, 128]
        heads = N if N <= 128 else 24
        qkv = torch.randn(M, 3 * heads * 128, device=dev, generator=g).bfloat16()
        qw = (1 + 0.1 * torch.randn(128, device=dev, generator=g)).bfloat16()
        kw = (1 + 0.1 * torch.randn(128, device=dev, generator=g)).bfloat16()
        fr = torch.randn(1, 1, M, 64, 2, 2, device=dev, generator=g)
        outs = [torch.empty(1, heads, M, 128, device=dev, dtype=torch.bfloat16) for _ in range(3)]
        work = 2.0 * 2 * 3 * M * heads * 128 + 4.0 * fr.numel()
        fn = lambda: ck.qk_norm_rope(qkv, qw, kw, fr, heads, q_out=outs[0], k_out=outs[1], v_out=outs[2])  # noqa: E731
    elif args.case == "quantize_nvfp4_gather":
        # the input of a single block's second linear: attention output [24, tokens, 128] | GELU(MLP) [tokens, 12288]
        att = torch.randn(24, M, 128, device=dev, generator=g).bfloat16()
        mlp = torch.randn(M, 12288, device=dev, generator=g).bfloat16()
        g4 = torch.tensor([4.0 / (6 * 448)], device=dev)
        work = 2.5625 * M * (3072 + 12288)
        fn = lambda: ck.quantize_nvfp4_gather([(att, None), (mlp, "gelu_tanh")], g4)  # noqa: E731
    else:
        raise SystemExit(f"unknown --case {args.case}")
    for _ in range(max(1, args.warmup)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"case": args.case, "shape": [M, N, K], "ms": round(ms, 4), "value": round(work / ms / 1e6, 1), "unit": unit}))


# ----------------------------------------------------------------------------- DiT stack (tensor parallel)


def dit_forward_ms(device, steps: int = 3) -> dict:
    """ms per forward of the full synthetic stack on one GPU (one CUDA graph per forward), for the default line."""
    from comfy_kitchen.dit_stack import DiTConfig, DiTStack, TensorParallel, gemm_flops_per_forward

    cfg = DiTConfig()
    stack = DiTStack(cfg, device, tp=TensorParallel(single=True))   # rank 0 measures this alone
    g = torch.Generator().manual_seed(11)
    img = torch.randn(cfg.img_tokens, cfg.hidden, generator=g).bfloat16().to(device)
    txt = torch.randn(cfg.txt_tokens, cfg.hidden, generator=g).bfloat16().to(device)
    vec = torch.randn(1, cfg.hidden, generator=g).bfloat16().to(device)
    stack.calibrate(img, txt, vec)
    run = stack.capture(img, txt, vec)
    for _ in range(3):
        run(img, txt, vec)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run(img, txt, vec)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"ms_per_forward": round(ms, 2), "tp": 1, "blocks": [cfg.n_double, cfg.n_single], "tokens": cfg.tokens,
            "linear_tflops": round(gemm_flops_per_forward(cfg) / (ms * 1e-3) / 1e12, 1), "launch": "CUDA graph"}


def dit_tp_leg(args, dist, device, rank: int, world: int) -> dict:
    """The tensor-parallel DiT stack over all ranks of the live process group: ms per forward (device events,
    slowest rank), how it was launched, the time inside the all-reduce steps and the per-forward cost of the
    work that every rank still does in full (norm -> quantize of the whole sequence)."""
    from comfy_kitchen.dit_stack import DiTConfig, DiTStack, TensorParallel, gemm_flops_per_forward

    cfg = DiTConfig()
    stack = DiTStack(cfg, device, tp=TensorParallel())
    g = torch.Generator().manual_seed(11)   # the same inputs on every rank
    img = torch.randn(cfg.img_tokens, cfg.hidden, generator=g).bfloat16().to(device)
    txt = torch.randn(cfg.txt_tokens, cfg.hidden, generator=g).bfloat16().to(device)
    vec = torch.randn(1, cfg.hidden, generator=g).bfloat16().to(device)
    why_not = None if args.nccl else stack.try_enable_peer_exchange()
    stack.calibrate(img, txt, vec)
    steps = max(3, min(args.steps, 10))

    def timed_forward():
        run, how = stack.capture_best(img, txt, vec)
        for _ in range(3):
            y = run(img, txt, vec)
        torch.cuda.synchronize()
        # (the status words are read and cleared here: a wait that ran out while the ranks were still starting up
        # at different times says nothing about the timed forwards)
        if stack.exchange is not None:
            stack.exchange.status()
        stack.ops.gemm_device_status()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            y = run(img, txt, vec)
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        return max_over_ranks(e0.elapsed_time(e1), dist, device) / steps, how, y

    def checked(out) -> str:
        """'' when this rank's forward looks sound, else what is wrong (device status words, non-finite output)."""
        if stack.ops.gemm_device_status() != 0:
            return "GEMM kernel reported a device-side timeout"
        if stack.exchange is not None and stack.exchange.status() != 0:
            return "the exchange kernel timed out waiting for a peer"
        if not bool(torch.isfinite(out.float()).all()):
            return "non-finite output"
        return ""

    def all_ranks_agree(problem: str) -> bool:
        """Every rank learns whether any rank found a problem, so that all of them go on, or stop, together (a rank
        that raised alone would leave the others waiting in the next collective)."""
        t = torch.tensor([0 if problem else 1], device=device, dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    # The form with the replicated front end first (every rank normalises and quantizes the whole sequence), then,
    # where the peer exchange is available, the sequence-parallel form; the line carries both and the faster one
    # as ms_per_forward.
    ms, launch, out = timed_forward()
    problem = checked(out)
    if not all_ranks_agree(problem):
        raise RuntimeError("tensor-parallel forward (replicated front end): " + (problem or "a problem on another rank"))
    forms = {"replicated_front_end_ms": round(ms, 2)}
    front_end = "replicated"
    res_report = {}
    if world <= 4:
        # Stand-alone timings of the exchange and of the replicated front end (they contain collectives of their own;
        # run on up to four ranks, where this build was checked).
        try:
            res_report = stack.exchange_report(img, txt, vec)
        except Exception as e:  # noqa: BLE001 - the forward's figures stand without it
            res_report = {"exchange_report_error": f"{type(e).__name__}: {str(e)[:200]}"}
    else:
        res_report = {"exchange_report": "not taken above four ranks"}
    if stack.exchange is not None and not args.no_sp:
        stack.enable_sequence_parallel()
        ms_sp, launch_sp, out_sp = timed_forward()
        problem = checked(out_sp)
        if all_ranks_agree(problem):
            forms["sequence_parallel_ms"] = round(ms_sp, 2)
            if ms_sp <= ms:
                ms, launch, out, front_end = ms_sp, launch_sp, out_sp, "sequence parallel"
        else:
            forms["sequence_parallel_error"] = problem or "a problem on another rank"
    res = {"tp": world, "ms_per_forward": round(ms, 2), "front_end": front_end, **forms, "launch": launch, "steps": steps,
           "blocks": [cfg.n_double, cfg.n_single], "tokens": cfg.tokens,
           "all_reduces_per_forward": stack.expected_all_reduces(),
           "linear_tflops": round(gemm_flops_per_forward(cfg) / (ms * 1e-3) / 1e12, 1)}
    res.update(res_report)
    if why_not:
        res["peer_exchange_unavailable"] = why_not[:200]
    del stack
    torch.cuda.empty_cache()
    return res


def run_dit(args) -> None:
    """One step = one forward of the synthetic Flux-like stack (19 double + 38 single blocks unless --dit-blocks
    says otherwise) on 4608 tokens, tensor-parallel over the N ranks (strong scaling: the work is fixed)."""
    from comfy_kitchen.dit_stack import (DiTConfig, DiTStack, TensorParallel, attention_flops_per_forward,
                                         gemm_flops_per_forward)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product path has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist  # type: ignore[no-redef]

        dist.init_process_group("nccl", device_id=device, timeout=__import__("datetime").timedelta(seconds=300))
    nd, ns = (int(v) for v in args.dit_blocks.split(","))
    cfg = DiTConfig(n_double=nd, n_single=ns)
    stack = DiTStack(cfg, device, tp=TensorParallel())
    why_not = None
    if world > 1 and not args.nccl:
        why_not = stack.try_enable_peer_exchange()
    g = torch.Generator().manual_seed(11)  # the same inputs on every rank
    host = [torch.randn(cfg.img_tokens, cfg.hidden, generator=g).bfloat16().pin_memory(),
            torch.randn(cfg.txt_tokens, cfg.hidden, generator=g).bfloat16().pin_memory(),
            torch.randn(1, cfg.hidden, generator=g).bfloat16().pin_memory()]
    img, txt, vec = (t.to(device) for t in host)
    stack.calibrate(img, txt, vec)
    if stack.exchange is not None and not args.no_sp:
        stack.enable_sequence_parallel()
    eager = args.no_graph
    # one graph on a single rank; with tensor parallelism a chain of graphs with the all-reduces between them
    run, how = (stack.forward, "eager") if eager else stack.capture_best(img, txt, vec)
    for _ in range(max(args.warmup, 3)):
        out = run(img, txt, vec)
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = run(img, txt, vec)
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    elapsed_ms = max_over_ranks(e0.elapsed_time(e1), dist, device)
    assert stack.ops.gemm_device_status() == 0, "GEMM kernel reported a device-side timeout"
    assert torch.isfinite(out.float()).all(), "non-finite output"
    ms = elapsed_ms / args.steps
    # end to end: inputs from pinned host memory, output back to the host, wall clock
    host_out = torch.empty(cfg.tokens, cfg.hidden, dtype=torch.bfloat16).pin_memory()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    n_e2e = max(1, min(args.steps, 3))
    for _ in range(n_e2e):
        d = [t.to(device, non_blocking=True) for t in host]
        host_out.copy_(run(*d), non_blocking=True)
        torch.cuda.synchronize()
    t_e2e = (time.perf_counter() - t0) / n_e2e * 1e3
    t_e2e = max_over_ranks(t_e2e, dist, device)
    if rank == 0:
        gf, af = gemm_flops_per_forward(cfg), attention_flops_per_forward(cfg)
        print(json.dumps({
            "metric": "dit_stack_forward_ms", "value": round(ms, 3), "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 3), "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "nvfp4 linears (fp32 accumulate), bf16 attention", "data": "synthetic",
            "config": {"workload": "synthetic Flux-like DiT stack (configs[4])", "double_blocks": nd, "single_blocks": ns,
                       "tokens": cfg.tokens, "hidden": cfg.hidden, "parallelism": f"tp{world}",
                       "all_reduces_per_forward": stack.expected_all_reduces(),
                       "launch": how, "peer_exchange_unavailable": why_not,
                       "l2": "weights (6 GB per rank at tp1) larger than L2"},
            "linear_tflops": round(gf / (ms * 1e-3) / 1e12, 1), "attention_tflop_per_forward": round(af / 1e12, 2),
            "e2e": {"value": round(t_e2e, 3), "unit": "ms", "h2d_bytes_per_step": int(sum(t.numel() * 2 for t in host)),
                    "d2h_bytes_per_step": int(host_out.numel() * 2)},
            "clocks": clocks,
        }))
    if dist is not None:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------- main


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--min-seconds", type=float, default=2.0,
                    help="the timed region repeats the K steps until it is at least this long")
    ap.add_argument("--no-extras", action="store_true", help="skip the quantizer sweep, e2e and CPU legs")
    ap.add_argument("--case", default=None,
                    help="run one kernel instead of the sweep (for profiling): gemm_nvfp4, gemm_mxfp8, quantize_nvfp4, "
                         "dequantize_nvfp4, quantize_mxfp8, quantize_fp8, adaln, adaln_quantize_nvfp4, rope, qk_norm_rope, "
                         "quantize_nvfp4_gather")
    ap.add_argument("--workload", default="linear", choices=["linear", "dit"],
                    help="linear: the NVFP4 linear sweep (default); dit: the tensor-parallel DiT stack, ms per forward")
    ap.add_argument("--dit-blocks", default="19,38", help="double,single block counts for --workload dit")
    ap.add_argument("--no-dit", action="store_true", help="skip the DiT-stack leg of the default line")
    ap.add_argument("--nccl", action="store_true",
                    help="tensor-parallel DiT stack: NCCL all-reduce + addcmul instead of the fused peer-memory exchange kernel")
    ap.add_argument("--no-sp", action="store_true",
                    help="tensor-parallel DiT stack with the peer exchange: keep the norm -> quantize front end replicated "
                         "on every rank instead of sequence-parallel")
    ap.add_argument("--no-graph", action="store_true", help="--workload dit: launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--m", type=int, default=9216)
    ap.add_argument("--n", type=int, default=9216)
    ap.add_argument("--k", type=int, default=3072)
    args = ap.parse_args()
    if args.case:
        run_case(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload == "dit":
        run_dit(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product path has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist  # type: ignore[no-redef]

        dist.init_process_group("nccl", device_id=device, timeout=__import__("datetime").timedelta(seconds=300))

    wl = Workload(device, seed=1000 + rank)
    for _ in range(args.warmup):
        wl.step()
    torch.cuda.synchronize()
    # One "repeat" = the K steps asked for.  The timed region loops whole repeats until it is at least
    # --min-seconds long, so that the GPU settles at the clock it can hold under its power cap and the clock
    # sampler sees many samples; every rank uses the same repeat count (the slowest rank's estimate).
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    wl.step()
    e1.record()
    torch.cuda.synchronize()
    est_ms = max_over_ranks(e0.elapsed_time(e1), dist, device)
    repeats = max(1, int(-(-args.min_seconds * 1e3 // (est_ms * args.steps))))
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(repeats * args.steps):
        wl.step()
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    elapsed_ms = max_over_ranks(e0.elapsed_time(e1), dist, device)
    assert wl.ck.gemm_device_status() == 0, "GEMM kernel reported a device-side timeout"
    flops = step_flops()
    timed_steps = repeats * args.steps
    value = job_throughput(world, flops, timed_steps, elapsed_ms)

    # Second pass, straight after the first so that the clocks are the same: the same steps with an event pair
    # around every GEMM launch (kept out of the headline loop); gives the GEMM kernel's share and rate.
    n2 = max(1, timed_steps // 2)
    for _ in range(n2):
        wl.step(record=True)
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    gemm_ms = sum(a.elapsed_time(b) for a, b, _ in wl.gemm_events)
    gemm_flops = sum(f for _, _, f in wl.gemm_events)
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12
    per_shape = {}
    for a, b, f, key in ((a, b, f, k) for (a, b, f), k in zip(wl.gemm_events, wl.gemm_keys)):
        t, fl = per_shape.get(key, (0.0, 0.0))
        per_shape[key] = (t + a.elapsed_time(b), fl + f)
    peaks = measured_peaks()
    # Dense FP4 peak = 4 x dense bf16 peak on this part (9 vs 2.25 PFLOP/s nominal).  The timed region is seconds
    # long and runs under the power cap, so the denominator is 4 x the sustained cuBLAS bf16 rate; the fraction
    # of 4 x the burst rate and of the nominal figure are given beside it.
    peak = 4.0 * float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
    peak_burst = 4.0 * float(peaks["bf16_tflops"])
    sm_mhz = (clocks or {}).get("sm_mhz")

    line = {
        "metric": "nvfp4_linear_throughput", "value": round(value, 1), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(elapsed_ms / timed_steps, 3),
        "repeats": repeats, "timed_steps": timed_steps, "timed_region_s": round(elapsed_ms * 1e-3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "nvfp4 (e2m1 x e4m3 block scales), fp32 accumulate", "data": "synthetic",
        "config": {"workload": "NVFP4 linear sweep, Flux-like MMDiT shapes (configs[2]): fused LN+AdaLN->NVFP4 quantize, "
                               "NVFP4 GEMM + fp32 bias -> bf16", "tokens": [TOKENS * b for b in BATCHES],
                   "layers": [[n, k] for _, n, k in LAYERS], "l2": "inputs larger than L2 (1.9 GB of outputs per step)",
                   "parallelism": f"tokens x{world}" if world > 1 else "single GPU",
                   "timed_region": f"{repeats} x {args.steps} steps back to back (>= {args.min_seconds} s)"},
        "gpu_launches": 24 * timed_steps,
        "clocks": clocks,
        "ms_per_step_x_sm_mhz": round(elapsed_ms / timed_steps * sm_mhz, 1) if sm_mhz else None,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": round(peak, 1), "unit": "TFLOP/s",
                     "frac": round(achieved / peak, 4), "frac_of_4x_burst_bf16": round(achieved / peak_burst, 4),
                     "frac_of_nominal_dense_fp4": round(achieved / 9000.0, 4),
                     "kernel": "gemm_blockscaled_kernel<fp4>",
                     "peak_source": f"4 x bf16_tflops_sustained ({peaks['_source']}): the region is seconds long under the power cap",
                     "gemm_share_of_step": round(gemm_ms / n2 / (elapsed_ms / timed_steps), 3),
                     "per_shape_tflops": {k: round(fl / (t * 1e-3) / 1e12, 0) for k, (t, fl) in per_shape.items()},
                     **gemm_traffic()},
    }

    # ---- e2e through the public API with host buffers, on every rank at once (they share the host's memory
    # and PCIe paths, as a real multi-GPU job would): wall clock between barriers, slowest rank.
    if not args.no_extras:
        h2d, d2h = wl.make_host()
        wl.step_e2e()
        torch.cuda.synchronize()
        n_e2e = max(1, min(args.steps, 3))
        if dist is not None:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            wl.step_e2e()
        torch.cuda.synchronize()
        t_e2e = max_over_ranks((time.perf_counter() - t0) / n_e2e * 1e3, dist, device) * 1e-3
        line["e2e"] = {"value": round(world * flops / t_e2e / 1e12, 2), "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d) * world,
                       "d2h_bytes_per_step": int(d2h) * world, "steps": n_e2e}
        del wl.host_in, wl.host_out
    # ---- N > 1: the tensor-parallel DiT stack of configs[4] over all ranks (strong scaling), while the group is alive
    if dist is not None and not args.no_dit and not args.no_extras:
        try:
            line["dit_stack"] = dit_tp_leg(args, dist, device, rank, world)
        except Exception as e:  # noqa: BLE001 - the contract line must still be printed; the failure is reported in it
            line["dit_stack"] = {"tp": world, "error": f"{type(e).__name__}: {str(e)[:300]}"}
    # The legs below are single-GPU measurements that rank 0 makes alone: the process group goes first, so that
    # nothing in them can wait for a rank that has already left.
    if dist is not None:
        dist.destroy_process_group()
        dist = None
    if rank == 0 and world > 1 and isinstance(line.get("dit_stack"), dict):
        one = dit_forward_ms(device, steps=3)
        d = line["dit_stack"]
        d["tp1_ms_same_run"] = one["ms_per_forward"]
        d["strong_scaling_eff"] = round(one["ms_per_forward"] / (world * d["ms_per_forward"]), 3)
    if rank == 0 and not args.no_extras and world == 1:
        # (single-GPU measurements: made once, in the N = 1 line)
        # ---- memory-bound kernels on every shape of the sweep (configs[1])
        line["quantizers"] = quantizer_sweep(device, float(peaks["hbm_gbs"]))
        # ---- the fused front end and RoPE at their config shapes
        line["front_end_rope"] = front_end_and_rope(device, float(peaks["hbm_gbs"]))
        # ---- ours beside the library's kernel (cuBLASLt), NVFP4 and MXFP8, all twelve shapes
        vs = gemm_vs_library(device)
        line["roofline"]["vs_library"] = vs["nvfp4"].get("ratio_geomean")
        line["roofline"]["vs_library_min"] = vs["nvfp4"].get("ratio_min")
        line["gemm_vs_library"] = vs
        # ---- host cost of a call (dispatch overhead)
        line["host_overhead"] = host_overhead(device)
        # ---- the DiT stack of configs[4] on this GPU (tp1; `--workload dit` runs it tensor-parallel)
        if not args.no_dit:
            line["dit_stack"] = dit_forward_ms(device, steps=3)
        # ---- CPU oracle on a bounded sample
        threads = os.cpu_count() or 1
        cpu_sample_step(512, threads)
        t_cpu, f_cpu = cpu_sample_step(512, threads)
        line["cpu_baseline"] = {"value": round(f_cpu / t_cpu / 1e12, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                "sample": "512 tokens x 4 layers (of 32256 tokens x 4 layers), CPU oracle, dequantize->fp32 matmul"}
    if rank == 0:
        line.setdefault("e2e", None)
        print(json.dumps(line))


if __name__ == "__main__":
    main()
