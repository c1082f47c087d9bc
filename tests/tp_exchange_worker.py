"""One rank of the multi-GPU exchange test (see tests/test_gpu_tp_exchange.py); run under torch.distributed.run."""
import datetime
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "comfy-kitchen_b200"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    from comfy_kitchen.dit_stack import DiTConfig, DiTStack, TensorParallel
    from comfy_kitchen.tp_exchange import PeerExchange

    # ---- the kernel against an all-gather + fp32 sum + addcmul: plain peer loads, then the NVLink-switch path
    rows, cols, split = 1000, 3072, 256
    for multimem in ("0", "1"):
        os.environ["CK_TP_MULTIMEM"] = multimem
        ex = PeerExchange(None, dev, rows, cols, torch.bfloat16)
        if multimem == "1" and not ex.multimem:
            print(f"[rank {rank}] no multicast address on this allocation: switch path not exercised", flush=True)
            continue
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        gs = torch.Generator(device=dev).manual_seed(7)      # the same on every rank
        x0 = torch.randn(rows, cols, device=dev, generator=gs).bfloat16()
        g0 = torch.randn(cols, device=dev, generator=gs).bfloat16()
        g1 = torch.randn(cols, device=dev, generator=gs).bfloat16()
        ex.residual.copy_(x0)
        torch.cuda.synchronize()
        dist.barrier()
        want = x0.clone()
        for it in range(3):
            part = torch.randn(rows, cols, device=dev, generator=g).bfloat16()
            ex.partial.copy_(part)
            ex.exchange(g0, g1, split)
            # reference: fp32 sum over the ranks in rank order, rounded once, then addcmul
            allp = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(allp, part)
            s = torch.zeros(rows, cols, device=dev)
            for t in allp:
                s += t.float()
            y = s.bfloat16()
            want[:split] = torch.addcmul(want[:split], g0, y[:split])
            want[split:] = torch.addcmul(want[split:], g1, y[split:])
            if not ex.multimem:
                assert torch.equal(ex.residual, want), f"rank {rank} call {it}: residual differs"
            else:
                # the switch forms and rounds the sum its own way (measured: many elements differ from the ordered
                # fp32 sum rounded to nearest, each by one bf16 step of y): a tolerance, not equality
                diff = (ex.residual.float() - want.float()).abs()
                assert diff.max() <= 2.0 ** -6 * want.float().abs().max(), f"rank {rank} call {it}: {diff.max().item()}"
                want = ex.residual.clone()
        # all ranks hold the same bits
        mine = ex.residual.clone()
        ref = mine.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(mine, ref)
        assert ex.status() == 0
        print(f"[rank {rank}] exchange kernel ok ({'NVLink-switch multimem' if ex.multimem else 'peer loads'})", flush=True)
        del ex
    os.environ.pop("CK_TP_MULTIMEM", None)

    # ---- the stack: peer-exchange forward (eager and one graph) against the NCCL forward
    cfg = DiTConfig(n_double=2, n_single=2, txt_tokens=128, img_grid=(16, 24))
    g = torch.Generator().manual_seed(3)
    img = torch.randn(cfg.img_tokens, cfg.hidden, generator=g).bfloat16().to(dev)
    txt = torch.randn(cfg.txt_tokens, cfg.hidden, generator=g).bfloat16().to(dev)
    vec = torch.randn(1, cfg.hidden, generator=g).bfloat16().to(dev)
    base = DiTStack(cfg, dev, tp=TensorParallel())
    base.calibrate(img, txt, vec)
    y_nccl = base.forward(img, txt, vec)
    fused = DiTStack(cfg, dev, tp=TensorParallel())
    why = fused.try_enable_peer_exchange()
    assert why is None, why
    fused.sites.static = dict(base.sites.static)
    y_eager = fused.forward(img, txt, vec)
    rel = ((y_eager.float() - y_nccl.float()).norm() / y_nccl.float().norm()).item()
    assert rel < 2e-2, rel      # NCCL sums in another order and precision: tolerance, not equality
    run, how = fused.capture_best(img, txt, vec)
    assert "one CUDA graph" in how
    for _ in range(2):
        y_graph = run(img, txt, vec)
    torch.cuda.synchronize()
    assert torch.equal(y_graph, y_eager), "graph replay differs from the eager forward"
    # sequence-parallel front end: every rank normalises and quantizes only its rows and the ranks exchange the
    # NVFP4 activation; the arithmetic per element is unchanged, so the output must be bit-identical
    fused.enable_sequence_parallel()
    y_sp = fused.forward(img, txt, vec)
    # the same arithmetic per element, except that the norm kernel may split a row's statistics over a different
    # number of warps when it is given fewer rows (one rounding step of an activation here and there)
    rel_sp = ((y_sp.float() - y_eager.float()).norm() / y_eager.float().norm()).item()
    assert rel_sp < 1e-2, rel_sp
    run_sp, how_sp = fused.capture_best(img, txt, vec)
    for _ in range(2):
        y_sp_graph = run_sp(img, txt, vec)
    torch.cuda.synchronize()
    assert torch.equal(y_sp_graph, y_sp), "sequence-parallel graph replay differs from its eager forward"
    assert fused.exchange.status() == 0
    assert fused.ops.gemm_device_status() == 0
    assert fused.ops.norm_device_status() == 0
    # a split in which one rank's rows are exactly the text tokens (what eight ranks give on the full model): that rank
    # has no image rows to normalise and receives no image tile rows from the scattered GEMMs
    cfg2 = DiTConfig(n_double=2, n_single=1, txt_tokens=128 * (world - 1) if world > 1 else 128, img_grid=(8, 16 * max(world - 1, 1)))
    img2 = torch.randn(cfg2.img_tokens, cfg2.hidden, generator=g).bfloat16().to(dev)
    txt2 = torch.randn(cfg2.txt_tokens, cfg2.hidden, generator=g).bfloat16().to(dev)
    st2 = DiTStack(cfg2, dev, tp=TensorParallel())
    assert st2.try_enable_peer_exchange() is None
    if world == 2:
        assert st2.exchange.row_bounds == [0, cfg2.txt_tokens, cfg2.tokens], st2.exchange.row_bounds
    st2.calibrate(img2, txt2, vec)
    y_rep = st2.forward(img2, txt2, vec)
    st2.enable_sequence_parallel()
    y_sp2 = st2.forward(img2, txt2, vec)
    rel2 = ((y_sp2.float() - y_rep.float()).norm() / y_rep.float().norm()).item()
    assert rel2 < 1e-2, rel2
    assert st2.exchange.status() == 0 and st2.ops.gemm_device_status() == 0
    dist.barrier()
    if rank == 0:
        print(f"stack: fused vs NCCL relative difference {rel:.2e}; {how}")
        print("TP_EXCHANGE_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
