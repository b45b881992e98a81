"""Worker of tests/test_gpu_multi.py: launched by torch.distributed.run, one rank per GPU.  Compares the
expert-parallel fused MoE (token-sharded all-to-all mode and replicated all-reduce mode) and the row-sharded dense
layer with the single-GPU result computed on the same rank."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import muxi_native_layout_kernels_b200 as mlk  # noqa: E402
from muxi_native_layout_kernels_b200 import parallel  # noqa: E402
from muxi_native_layout_kernels_b200.muxi_moe_planC import fused_moe  # noqa: E402


def _peer_reduce_cases(parallel, red, x, w1l, w2l, logits, topk, kw, full, close, world):
    import muxi_native_layout_kernels_b200 as mlk
    res = {}
    y1 = parallel.fused_moe_ep_replicated(x, w1l, w2l, logits, topk, True, reducer=red, **kw).clone()
    y2 = parallel.fused_moe_ep_replicated(x, w1l, w2l, logits, topk, True, reducer=red, **kw).clone()
    res["replicated peer-memory reduce"] = close(y1, full)
    gathered = [torch.empty_like(y1) for _ in range(world)]
    dist.all_gather(gathered, y1)
    same = torch.equal(y1, y2) and all(torch.equal(gathered[0], t) for t in gathered)
    res["peer-memory reduce deterministic"] = (same, 0.0)
    xr, lr = x.clone(), logits.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        parallel.fused_moe_ep_replicated(xr, w1l, w2l, lr, topk, True, reducer=red, **kw)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            yr = parallel.fused_moe_ep_replicated(xr, w1l, w2l, lr, topk, True, reducer=red, **kw)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    res["peer-memory reduce graph"] = (torch.equal(yr, y1), 0.0)
    del graph
    # both forms of the kernel on their own (one pass with (value, epoch) pairs for small shares, reduce-scatter +
    # all-gather for large ones) against the shares gathered with NCCL and added in rank order: bit-equal, three calls
    rank = dist.get_rank()
    for tokens, hidden in ((5, 256), (640, 512)):
        r2 = parallel.PeerReducer(tokens, hidden, torch.bfloat16)
        good = True
        for call in range(3):
            gen = torch.Generator(device=x.device).manual_seed(1000 * call + rank)
            r2.share.copy_(torch.randn(tokens, hidden, generator=gen, device=x.device) * 50)
            got = r2.reduce().clone()
            parts = [torch.empty_like(r2.share) for _ in range(world)]
            dist.all_gather(parts, r2.share)
            want = parts[0].clone()
            for pt in parts[1:]:
                want += pt
            good = good and torch.equal(got, want.to(torch.bfloat16))
        res[f"peer-memory reduce alone [{tokens}, {hidden}]"] = (good, 0.0)
        del r2
    assert mlk.kernel_status() == 0
    return res


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    g = torch.Generator().manual_seed(77)
    ok = True
    for (E, topk, H, I, T, fp8) in [(16, 4, 256, 128, 24, False), (32, 8, 256, 128, 40, True)]:
        x = torch.randn(world * T, H, generator=g).to(torch.bfloat16).to(dev)
        logits = torch.randn(world * T, E, generator=g).to(torch.bfloat16).to(dev)
        if fp8:
            w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.25).to(torch.float8_e4m3fn).to(dev)
            w2 = (torch.randn(E, H, I, generator=g) * 0.25).to(torch.float8_e4m3fn).to(dev)
        else:
            w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16).to(dev)
            w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        w1a, w2a = mlk.layoutA(w1), mlk.layoutA(w2)
        kw = dict(soft_fp8=True, block_shape=[128, 128]) if fp8 else {}
        full = fused_moe(x, w1a, w2a, logits, topk, True, **kw).float()
        el = E // world
        w1l, w2l = w1a[rank * el:(rank + 1) * el].contiguous(), w2a[rank * el:(rank + 1) * el].contiguous()
        xs, ls = x[rank * T:(rank + 1) * T].contiguous(), logits[rank * T:(rank + 1) * T].contiguous()
        want = full[rank * T:(rank + 1) * T]
        scale = max(1.0, float(full.pow(2).mean().sqrt()))

        def close(got, ref):
            d = (got.float() - ref).abs()
            return bool((d <= 1e-2 * scale + 1e-2 * ref.abs()).all()), float(d.max())

        res = {}
        res["all_to_all"] = close(parallel.fused_moe_ep(xs, w1l, w2l, ls, topk, True, soft_fp8=fp8), want)
        res["gather"] = close(parallel.fused_moe_ep(xs, w1l, w2l, ls, topk, True, soft_fp8=fp8, exchange="gather"), want)
        res["replicated fp32"] = close(parallel.fused_moe_ep_replicated(x, w1l, w2l, logits, topk, True, **kw), full)
        res["replicated bf16"] = close(parallel.fused_moe_ep_replicated(x, w1l, w2l, logits, topk, True,
                                                                        reduce_dtype=torch.bfloat16, **kw), full)
        # the same with the shares added over peer memory (one kernel per rank, no NCCL call); twice in a row (epochs),
        # bit-equal on all ranks and between the calls, then inside a CUDA graph
        try:
            red = parallel.PeerReducer(x.shape[0], H, torch.bfloat16)
        except Exception as e:      # no peer-mappable memory on this machine: every rank fails alike
            red = None
            print(f"rank {rank} peer-memory reduce not run: {type(e).__name__}: {e}", flush=True)
        if red is not None:
            res.update(_peer_reduce_cases(parallel, red, x, w1l, w2l, logits, topk, kw, full, close, world))
        # the static-shape modes inside a CUDA graph (collectives included), replayed on new inputs
        xg, lg = xs.clone(), ls.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            parallel.fused_moe_ep(xg, w1l, w2l, lg, topk, True, soft_fp8=fp8, exchange="gather")
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                yg = parallel.fused_moe_ep(xg, w1l, w2l, lg, topk, True, soft_fp8=fp8, exchange="gather")
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        torch.cuda.synchronize()
        res["gather graph"] = close(yg, want)
        del graph
        for name, (good, dmax) in res.items():
            print(f"rank {rank} E={E} fp8={fp8} {name}: max diff {dmax:.4g} ok={good}", flush=True)
            ok = ok and good
    # dense: row shard, then all-gather of the output columns
    W = (torch.randn(1024, 512, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    X = torch.randn(8, 512, generator=g).to(torch.bfloat16).to(dev)
    y_full = mlk.gemm_layoutA(mlk.layoutA(W), X)
    y_loc = mlk.gemm_layoutA(mlk.layoutA(parallel.shard_rows(W, rank, world)), X)
    ok3 = torch.equal(parallel.all_gather_columns(y_loc), y_full)
    print(f"rank {rank} dense row shard ok={ok3}", flush=True)
    ok = ok and ok3
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
