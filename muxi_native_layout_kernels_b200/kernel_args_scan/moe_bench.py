"""Times the fused MoE layer (router + alignment + expert compute + combine) on one GPU.

    python -m muxi_native_layout_kernels_b200.kernel_args_scan.moe_bench [--config mixtral|fine|both] [--tokens 1,16]
           [--iters 20] [--json]

mixtral: E=8, top-2, H=4096, I=14336, bf16 weights ~ N(0, 0.02^2), seed 3.
fine:    E=128, top-8, H=2048, I=768, e4m3 weights (N(0,1)*0.5 cast, repacked), seed 4.
Role of the reference's benchmark_and_test/benchmark_muxi_moe.py.  Every iteration uses a different activation
batch (8 batches are cycled), so different experts are hit; the layer is captured in a CUDA graph per batch and the
replays are timed with CUDA events (us_graph), next to the eager Python call (us_eager, includes host overhead).
Algorithmic bytes = distinct experts selected x 3*I*H*weight bytes + 4*T*H + 2*T*E.
"""
from __future__ import annotations

import argparse
import json

import torch

import muxi_native_layout_kernels_b200 as mlk
from muxi_native_layout_kernels_b200.muxi_moe_planC import fused_moe

CONFIGS = {
    "mixtral": dict(E=8, topk=2, H=4096, I=14336, fp8=False, seed=3, tokens=[1, 16, 64, 256]),
    "fine": dict(E=128, topk=8, H=2048, I=768, fp8=True, seed=4, tokens=[1, 32, 128, 512]),
}
NBATCH = 8


def build(cfg, dev):
    g = torch.Generator(device=dev).manual_seed(cfg["seed"])
    E, H, I = cfg["E"], cfg["H"], cfg["I"]
    if cfg["fp8"]:
        w1 = (torch.randn(E, 2 * I, H, generator=g, device=dev) * 0.5).to(torch.float8_e4m3fn)
        w2 = (torch.randn(E, H, I, generator=g, device=dev) * 0.5).to(torch.float8_e4m3fn)
        w1 = mlk.fp8_weight_repack(mlk.layoutA(w1))
        w2 = mlk.fp8_weight_repack(mlk.layoutA(w2))
    else:
        w1 = mlk.layoutA((torch.randn(E, 2 * I, H, generator=g, device=dev) * 0.02).to(torch.bfloat16))
        w2 = mlk.layoutA((torch.randn(E, H, I, generator=g, device=dev) * 0.02).to(torch.bfloat16))
    wg = (torch.randn(E, H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    return w1, w2, wg, g


def run_case(cfg, T, w1, w2, wg, g, dev, iters, scales=False, peak=6450.0):
    E, H, I, topk, fp8 = cfg["E"], cfg["H"], cfg["I"], cfg["topk"], cfg["fp8"]
    xs = [torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16) for _ in range(NBATCH)]
    logits = [(x.float() @ wg.float().t()).to(torch.bfloat16) for x in xs]
    kw = dict(block_shape=[128, 128], soft_fp8=True, fp8_repacked=True) if fp8 else {}
    if fp8 and scales:
        # block-scale tensors as the reference's interface wants them (all ones: the weights are synthetic)
        kw.update(w1_scale=torch.ones(E, 2 * I // 128, H // 128, device=dev),
                  w2_scale=torch.ones(E, H // 128, I // 128, device=dev))

    def call(i):
        return fused_moe(xs[i], w1, w2, logits[i], topk, True, **kw)

    for i in range(NBATCH):
        call(i)
    torch.cuda.synchronize()
    distinct = sum(int(torch.topk(torch.softmax(l.float(), -1), topk, dim=-1)[1].unique().numel()) for l in logits) / NBATCH
    nbytes = distinct * 3 * I * H * (1 if fp8 else 2) + 4 * T * H + 2 * T * E
    # eager
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for it in range(iters):
        call(it % NBATCH)
    e1.record()
    torch.cuda.synchronize()
    us_eager = e0.elapsed_time(e1) * 1e3 / iters
    # graph: one graph holding all NBATCH layers back to back
    graph = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(graph, stream=s):
            for i in range(NBATCH):
                call(i)
    torch.cuda.current_stream().wait_stream(s)
    graph.replay()
    torch.cuda.synchronize()
    reps = max(1, iters // NBATCH)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us_graph = e0.elapsed_time(e1) * 1e3 / (reps * NBATCH)
    gbs = nbytes / us_graph / 1e3
    return {"T": T, "experts_hit": distinct, "us_graph": round(us_graph, 2), "us_eager": round(us_eager, 2),
            "algorithmic_mb": round(nbytes / 1e6, 1), "gbs": round(gbs, 1), "frac_measured": round(gbs / peak, 3),
            "frac_nominal_8TBs": round(gbs / 8000.0, 3)}


def run(config="both", tokens=None, iters=24, dev=None, scales=False, peak=6450.0):
    dev = dev or torch.device("cuda")
    mlk.set_static_weights(True)
    out = {}
    for name in (["mixtral", "fine"] if config == "both" else [config]):
        cfg = CONFIGS[name]
        w1, w2, wg, g = build(cfg, dev)
        out[name] = [run_case(cfg, T, w1, w2, wg, g, dev, iters, scales, peak) for T in (tokens or cfg["tokens"])]
        del w1, w2
        torch.cuda.empty_cache()
    return out


def _close(got, want):
    want = want.float()
    scale = max(1.0, float(want.pow(2).mean().sqrt()))
    return bool(((got.float() - want).abs() <= 1e-2 * scale + 1e-2 * want.abs()).all())


def _time_ep(call, iters, graphs, dev):
    """us per call: eager (host launch overhead included) and, if asked for and possible, as CUDA-graph replays of
    NBATCH calls; max over ranks."""
    import torch.distributed as dist
    for i in range(NBATCH):
        call(i)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for it in range(iters):
        call(it % NBATCH)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out = {"us_eager": round(float(t[0]), 2)}
    if graphs:
        graph = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            call(0)
            with torch.cuda.graph(graph, stream=s):
                for i in range(NBATCH):
                    call(i)
        torch.cuda.current_stream().wait_stream(s)
        graph.replay()
        torch.cuda.synchronize()
        dist.barrier()
        reps = max(1, iters // NBATCH)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (reps * NBATCH)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out["us_graph"] = round(float(t[0]), 2)
        del graph
    return out


def run_ep(config, rank, world, tokens=None, iters=24, dev=None, graphs=False):
    """Expert-parallel layer on `world` ranks (one process per GPU, torch.distributed initialised), both modes of
    parallel.py, on identical seeded weights: every rank generates the full expert weights from the same seed, keeps
    its E / world experts and checks its output of one batch against the single-GPU layer it computes from the full
    weights (parity_ok).
      replicated   tokens and router logits on every rank, each rank adds its experts' share (experts_map), NCCL
                   all-reduce of the shares; us_eager and us_graph
      replicated_peer_reduce   the same with the shares added by one kernel per rank over peer memory
                   (parallel.PeerReducer) instead of the all-reduce and the cast
      all_to_all   tokens sharded T / world per rank, NCCL all-to-all dispatch of exactly the routed rows, local
                   experts, all-to-all combine of the fp32 rows; us_eager only (the split sizes cost a host copy)
      gather_reduce_scatter  tokens sharded, static shapes: all-gather of tokens and logits, local share, reduce-scatter
                   of the fp32 shares; us_eager and us_graph
    Times are CUDA events around the calls after a barrier, max over ranks."""
    import torch.distributed as dist

    from muxi_native_layout_kernels_b200.parallel import PeerReducer, fused_moe_ep, fused_moe_ep_replicated
    dev = dev or torch.device("cuda")
    mlk.set_static_weights(True)
    out = {}
    for name in (["mixtral", "fine"] if config == "both" else [config]):
        cfg = dict(CONFIGS[name])
        E, H, I, topk, fp8 = cfg["E"], cfg["H"], cfg["I"], cfg["topk"], cfg["fp8"]
        if E % world != 0:
            continue
        w1, w2, wg, g = build(cfg, dev)                     # same seed, same bytes on every rank
        el = E // world
        w1l, w2l = w1[rank * el:(rank + 1) * el].contiguous(), w2[rank * el:(rank + 1) * el].contiguous()
        kw = dict(block_shape=[128, 128], soft_fp8=True, fp8_repacked=True) if fp8 else {}
        kw_ep = dict(soft_fp8=True, fp8_repacked=True) if fp8 else {}
        rows = []
        for T in (tokens or cfg["tokens"]):
            xs = [torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16) for _ in range(NBATCH)]
            logits = [(x.float() @ wg.float().t()).to(torch.bfloat16) for x in xs]
            want = fused_moe(xs[0], w1, w2, logits[0], topk, True, **kw)
            row = {"T": T, "experts_per_rank": el}
            got = fused_moe_ep_replicated(xs[0], w1l, w2l, logits[0], topk, True, **kw)
            rep = _time_ep(lambda i: fused_moe_ep_replicated(xs[i], w1l, w2l, logits[i], topk, True, **kw), iters, graphs, dev)
            rep["parity_ok"] = _close(got, want)
            row["replicated"] = rep
            # the same with the shares added over peer memory by one kernel per rank instead of the all-reduce
            try:
                red = PeerReducer(T, H, torch.bfloat16)
            except Exception as e:          # no peer-mappable memory on this machine (every rank fails alike)
                red = None
                row["replicated_peer_reduce"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
            if red is not None:
                got = fused_moe_ep_replicated(xs[0], w1l, w2l, logits[0], topk, True, reducer=red, **kw).clone()
                pr = _time_ep(lambda i: fused_moe_ep_replicated(xs[i], w1l, w2l, logits[i], topk, True, reducer=red, **kw),
                              iters, graphs, dev)
                pr["parity_ok"] = _close(got, want)
                row["replicated_peer_reduce"] = pr
                del red
            if T % world == 0:
                tl = T // world
                xl = [x[rank * tl:(rank + 1) * tl].contiguous() for x in xs]
                ll = [l[rank * tl:(rank + 1) * tl].contiguous() for l in logits]
                got = fused_moe_ep(xl[0], w1l, w2l, ll[0], topk, True, **kw_ep)
                # exact split sizes need one device -> host copy per call: eager only
                a2a = _time_ep(lambda i: fused_moe_ep(xl[i], w1l, w2l, ll[i], topk, True, **kw_ep), iters, False, dev)
                a2a["parity_ok"] = _close(got, want[rank * tl:(rank + 1) * tl])
                a2a["tokens_per_rank"] = tl
                row["all_to_all"] = a2a
                got = fused_moe_ep(xl[0], w1l, w2l, ll[0], topk, True, exchange="gather", **kw_ep)
                gat = _time_ep(lambda i: fused_moe_ep(xl[i], w1l, w2l, ll[i], topk, True, exchange="gather", **kw_ep), iters, graphs, dev)
                gat["parity_ok"] = _close(got, want[rank * tl:(rank + 1) * tl])
                gat["tokens_per_rank"] = tl
                row["gather_reduce_scatter"] = gat
            modes = [m for m in ("replicated", "replicated_peer_reduce", "all_to_all", "gather_reduce_scatter")
                     if m in row and "parity_ok" in row[m]]
            flags = torch.tensor([int(row[m]["parity_ok"]) for m in modes], device=dev)
            dist.all_reduce(flags, op=dist.ReduceOp.MIN)
            for m, f in zip(modes, flags.tolist()):
                row[m]["parity_ok"] = bool(f)
            rows.append(row)
        out[name] = rows
        del w1, w2, w1l, w2l
        torch.cuda.empty_cache()
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="both", choices=["mixtral", "fine", "both"])
    ap.add_argument("--tokens", default=None)
    ap.add_argument("--iters", type=int, default=24)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--scales", action="store_true", help="e4m3 configs: pass block-scale tensors (all ones)")
    a = ap.parse_args()
    res = run(a.config, [int(t) for t in a.tokens.split(",")] if a.tokens else None, a.iters, scales=a.scales)
    if a.json:
        print(json.dumps(res))
    else:
        for name, rows in res.items():
            for r in rows:
                print(name, r, flush=True)
