"""Benchmark of the weight-streaming hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (config.workload = "narrow_gemm_bf16_llama8b"): one step is one pass over the narrow-GEMM grid
tokens in {1,2,4,8,16,32,64} x (N,K) in {(4096,4096),(14336,4096),(4096,14336)}, bf16, native-layout weights,
row-major activations (gemm_layoutA) -- 21 kernel launches.  Cases are ordered so that the same weight matrix is
never used twice in a row: 235-268 MB of other weights stream between two uses, more than the 126 MB L2, so every
launch reads its weights from HBM.  metric = algorithmic bytes of the step / device time of the step.
At N > 1 every weight matrix is sharded over its output rows (rank g owns rows [g*N/G, (g+1)*N/G)), activations are
replicated, no collective runs in the data path; total work is fixed, hence "scaling": "strong".

value      device-resident inputs; the step is captured once in a CUDA graph and replayed K times (launch overhead
           of the Python host does not enter), timed with CUDA events, max over ranks.
e2e        the same step through the public Python API with HOST inputs: the activations of every case are copied
           from pinned host memory, the case runs, and its result is copied back to pinned host memory, as a
           copy / compute / copy pipeline inside the step; weights stay resident (they are model state, prepacked
           once offline).
roofline   HBM; achieved = algorithmic bytes per launch / average launch duration over the timed region.
cpu_baseline / --impl reference: the reference's torch formulation of the same math on the host cores
           ((X.float() @ W.float().T).to(bf16), the expected-value path of its benchmarks), all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

TOKENS = [1, 2, 4, 8, 16, 32, 64]
SHAPES = [(4096, 4096), (14336, 4096), (4096, 14336)]
# end-to-end pipeline: execution order of the token counts (small transfers first and last, large ones in the middle),
# the token count the second host -> device copy begins with, and the token counts whose three results share one
# device -> host dependency (chosen by measurement: 408 us per step against 449 us for the plain order with one
# event per tensor, 367 us with everything resident)
E2E_TOKEN_ORDER = [1, 2, 4, 64, 32, 16, 8]
E2E_SECOND_COPY_FROM = 64
E2E_GROUPED_OUT = (1, 2, 4)
# dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes, ncu captures of the dense kernels on the
# 117.4 MB weights: CUDA-core n=1 123.4/117.5, tcgen05 cluster n=16 121.6/118.0, n=64 122.9/119.8
NCU_TRAFFIC_RATIO = 1.03
NOMINAL_HBM_GBS = 8000.0


def algorithmic_bytes(n_tok: int, N: int, K: int, wbytes: int = 2) -> int:
    """The reference's own traffic formula (benchmark_and_test/gemv_benchmark.py:111): weights + activations in + out."""
    return N * K * wbytes + 2 * (n_tok * K + n_tok * N)


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def measured_tensor_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"])
        except Exception:
            pass
    return 1590.0


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
                for n_, v in zip(names, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n_)
            except Exception:
                continue
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def case_order():
    return [(n, N, K) for n in TOKENS for (N, K) in SHAPES]


# ------------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's torch math on the host cores
# ------------------------------------------------------------------------------------------------------

def cpu_pass(weights, acts):
    from oracle import dense as odense
    out = None
    for (n, N, K) in case_order():
        out = odense.gemm_ref(acts[(n, K)], weights[(N, K)])
    return out


def cpu_inputs():
    g = torch.Generator().manual_seed(1)
    weights = {s: (torch.randn(s[0], s[1], generator=g) * 0.02).to(torch.bfloat16) for s in SHAPES}
    acts = {(n, K): torch.randn(n, K, generator=g).to(torch.bfloat16) for n in TOKENS for K in (4096, 14336)}
    return weights, acts


def time_cpu(passes: int, warm: int = 1):
    torch.set_num_threads(os.cpu_count() or 1)
    weights, acts = cpu_inputs()
    for _ in range(warm):
        cpu_pass(weights, acts)
    t0 = time.perf_counter()
    for _ in range(passes):
        cpu_pass(weights, acts)
    dt = (time.perf_counter() - t0) / passes
    total = sum(algorithmic_bytes(n, N, K) for (n, N, K) in case_order())
    return total / dt / 1e9, dt


def time_cpu_moe():
    """The oracle's fused MoE (the reference's torch formulation, muxi_layout_kernels/utils.py:131-244) on the host
    cores, one run each of the two MoE configurations at their largest token count; weights seeded as in
    kernel_args_scan/moe_bench.py but generated on the host."""
    from oracle import moe as omoe
    torch.set_num_threads(os.cpu_count() or 1)
    out = []
    for name, (E, topk, H, I, fp8, seed, T) in {"C4 mixtral bf16": (8, 2, 4096, 14336, False, 3, 256),
                                              "C5 fine-grained e4m3": (128, 8, 2048, 768, True, 4, 512)}.items():
        g = torch.Generator().manual_seed(seed)
        # timing only: one seeded expert, repeated for every expert (generating 1.4 G random weights on the host would
        # take longer than the layer itself)
        wdt, std = (torch.float8_e4m3fn, 0.5) if fp8 else (torch.bfloat16, 0.02)
        w1 = (torch.randn(2 * I, H, generator=g) * std).to(wdt).unsqueeze(0).repeat(E, 1, 1)
        w2 = (torch.randn(H, I, generator=g) * std).to(wdt).unsqueeze(0).repeat(E, 1, 1)
        wg = (torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16)
        x = torch.randn(T, H, generator=g).to(torch.bfloat16)
        logits = (x.float() @ wg.float().t()).to(torch.bfloat16)
        t0 = time.perf_counter()
        omoe.fused_moe_ref(x, w1, w2, logits, topk, True)
        dt = time.perf_counter() - t0
        out.append({"config": name, "T": T, "us": round(dt * 1e6, 1), "cores": os.cpu_count(), "kind": "port",
                    "sample": "one run of the whole layer (router + experts), torch on all host threads; one seeded expert's weights repeated for all experts"})
        del w1, w2
    return out


def step_config(world: int) -> dict:
    """The workload both arms are timed on (their JSON lines carry the same `config`): the 21-case narrow-GEMM grid,
    weights sharded over their rows at N > 1, with the note on what sits between two uses of one weight matrix."""
    per_rank_weights = sum(N // world * K * 2 for (N, K) in SHAPES)
    between = per_rank_weights - max(N // world * K * 2 for (N, K) in SHAPES)
    l2_note = (f"consecutive launches use different weight matrices; {between / 1e6:.0f} MB of other weights stream between "
               f"two uses of one matrix (L2 is 126 MB)" + ("" if between > 126e6 else
               ": at this shard size the weights are partly L2-resident, so the value is not a pure HBM figure"))
    return {"workload": "narrow_gemm_bf16_llama8b", "tokens": TOKENS, "shapes": SHAPES, "variant": "gemm_layoutA",
            "launches_per_step": len(case_order()), "sharding": f"rows/{world}", "static_weights": True, "l2": l2_note}


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    gbs, dt = time_cpu(max(1, args.steps), warm=min(1, args.warmup))
    line = {
        "impl": "reference", "metric": "narrow_gemm_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": step_config(world),
        "implementation": "the reference's math for this path (fp32 matmul of the bf16 operands, rounded once) in torch on all "
                          "host threads, unsharded, on rank 0",
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
                         "sample": f"{max(1, args.steps)} full passes over the 21-case grid (whole workload, all host threads)"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------------

def run_ours(args):
    import torch.distributed as dist

    import muxi_native_layout_kernels_b200 as mlk

    rank, world, local = dist_env()
    assert torch.cuda.is_available(), "bench.py needs a CUDA device for --impl ours"
    mlk.set_static_weights(True)   # weights are prepacked once below and only read afterwards
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # inputs: seeded on the CPU, identical on every rank; each rank keeps its row shard of every weight matrix
    g = torch.Generator().manual_seed(1)
    weights, host_acts = {}, {}
    for (N, K) in SHAPES:
        W = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
        rows = N // world
        assert rows % 128 == 0, "row shard must stay a multiple of 128"
        weights[(N, K)] = mlk.layoutA(W[rank * rows:(rank + 1) * rows].contiguous().to(dev))
    for n in TOKENS:
        for K in (4096, 14336):
            host_acts[(n, K)] = torch.randn(n, K, generator=g).to(torch.bfloat16).pin_memory()
    dev_acts = {k: v.to(dev) for k, v in host_acts.items()}
    # end-to-end buffers: the step's activations in one pinned host buffer (laid out in the order the pipeline below
    # needs them) with a device copy, and one pinned host buffer that receives the step's 21 results
    e2e_tokens = E2E_TOKEN_ORDER
    in_off, off = {}, 0
    for n in e2e_tokens:
        for K in (4096, 14336):
            in_off[(n, K)] = off
            off += host_acts[(n, K)].numel()
    host_in = torch.empty(off, dtype=torch.bfloat16).pin_memory()
    for key, o in in_off.items():
        host_in[o:o + host_acts[key].numel()].copy_(host_acts[key].reshape(-1))
    dev_in = torch.empty(off, dtype=torch.bfloat16, device=dev)
    dev_in_view = {key: dev_in[o:o + host_acts[key].numel()].view(host_acts[key].shape) for key, o in in_off.items()}
    split = in_off[(E2E_SECOND_COPY_FROM, 4096)]       # first H2D copy: the small token counts; second: the rest
    order = case_order()
    e2e_order = [(n, N, K) for n in e2e_tokens for (N, K) in SHAPES]
    out_off, off = {}, 0
    for (n, N, K) in e2e_order:
        out_off[(n, N, K)] = off
        off += n * (N // world)
    host_out = torch.empty(off, dtype=torch.bfloat16).pin_memory()
    step_bytes_total = sum(algorithmic_bytes(n, N, K) for (n, N, K) in order)

    def step_device():
        out = None
        for (n, N, K) in order:
            out = mlk.gemm_layoutA(weights[(N, K)], dev_acts[(n, K)])
        return out

    # End-to-end step as a three-stage pipeline over the same 21 cases: the activations go host -> device on a copy
    # stream in two copies (the token counts that run first, then the rest), the cases run on the compute stream as
    # their activations arrive, and the results go device -> host on a second copy stream while later cases compute.
    # The cases with the large transfers run in the middle of the step, so that only the first small copy in and the
    # last small copies out are not hidden.  The step begins with nothing of its inputs on the device and ends when
    # the last result is in host memory.  Every cross-stream dependency costs a few microseconds (a kernel that waits
    # for an event cannot overlap its predecessor's tail), hence two input events and one output event per case or,
    # for the smallest cases, per token count.
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def step_e2e():
        cur = torch.cuda.current_stream()
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        with torch.cuda.stream(s_in):
            dev_in[:split].copy_(host_in[:split], non_blocking=True)
            first = torch.cuda.Event()
            first.record(s_in)
            dev_in[split:].copy_(host_in[split:], non_blocking=True)
            second = torch.cuda.Event()
            second.record(s_in)
        keep, pending = [], []

        def copy_out():
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for o, c in pending:
                    host_out[o:o + c.numel()].view(c.shape).copy_(c, non_blocking=True)
            pending.clear()

        for n in e2e_tokens:
            if n == e2e_tokens[0]:
                cur.wait_event(first)
            if n == E2E_SECOND_COPY_FROM:
                cur.wait_event(second)
            for (N, K) in SHAPES:
                c = mlk.gemm_layoutA(weights[(N, K)], dev_in_view[(n, K)])
                keep.append(c)      # read by the copy stream: no reuse of the buffer inside the step
                pending.append((out_off[(n, N, K)], c))
                if n not in E2E_GROUPED_OUT:
                    copy_out()
            if pending:
                copy_out()
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
        return keep

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step_device()
    torch.cuda.synchronize()

    # capture one step, replay it K times
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step_device()
        with torch.cuda.graph(graph, stream=side):
            step_device()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        graph.replay()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)

    # end-to-end through the public API with host buffers: every case copies its activations from pinned host memory,
    # runs, and copies its result back to pinned host memory, all inside the timed region.  Timed twice: as eager
    # Python calls (host submission cost included) and as a CUDA graph of the same calls and copies (what a serving
    # loop with static buffers replays); the graph number is the one reported as e2e.
    for _ in range(2):
        step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_e2e()
    e1.record()
    barrier()
    ms_e2e_eager = e0.elapsed_time(e1)
    graph_e2e = torch.cuda.CUDAGraph()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step_e2e()
        with torch.cuda.graph(graph_e2e, stream=side):
            step_e2e()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        graph_e2e.replay()
    barrier()
    e0.record()
    for _ in range(args.steps):
        graph_e2e.replay()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None

    if world > 1:
        t = torch.tensor([ms, ms_e2e, ms_e2e_eager], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e, ms_e2e_eager = float(t[0]), float(t[1]), float(t[2])

    peak, peak_kind = measured_peak()
    # every BASELINE configuration that is not the headline step, one row per (operator, dtype, shape, tokens): each
    # rank times its own row shards, the row's time is the max over ranks
    per_config = None
    if not args.no_per_config:
        from muxi_native_layout_kernels_b200.kernel_args_scan import dense_bench
        try:
            per_config = dense_bench.run(dev, peak, rank, world, tensor_peak=measured_tensor_peak())
            if world > 1:
                t = torch.tensor([r["us"] for r in per_config], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                for r, us in zip(per_config, t.tolist()):
                    if r["config"] == "F3":
                        tf = 2.0 * r["N"] * world * r["tokens"] * r["K"] / us / 1e6
                        r.update(N=r["N"] * world, us=round(us, 2), tflops=round(tf, 1),
                                 frac_measured_tensor=round(tf / world / measured_tensor_peak(), 3))
                        continue
                    # whole-job figures: all ranks' bytes over the slowest rank's time; fractions per GPU
                    wb = 1 if r["dtype"] == "e4m3" else 2
                    nbytes = r["N"] * world * r["K"] * wb + 2 * r["tokens"] * (r["K"] + r["N"] * world)
                    r.update(N=r["N"] * world, us=round(us, 2), gbs=round(nbytes / us / 1e3, 1),
                             frac_measured=round(nbytes / us / 1e3 / world / peak, 3),
                             frac_nominal_8TBs=round(nbytes / us / 1e3 / world / NOMINAL_HBM_GBS, 3))
        except Exception as exc:       # the headline line must still be printed
            per_config = {"error": repr(exc)[:300]}

    moe_ep = None
    if world > 1 and not args.no_moe:
        # every rank takes part (collectives inside); rank 0 reports
        from muxi_native_layout_kernels_b200.kernel_args_scan import moe_bench
        try:
            moe_ep = moe_bench.run_ep("both", rank, world, None, 24, dev, graphs=True)
        except Exception as exc:       # the dense line must still be printed
            moe_ep = {"error": repr(exc)[:300]}

    if rank == 0:
        ms_step = ms / args.steps
        value = step_bytes_total / (ms_step * 1e-3) / 1e9
        e2e_value = step_bytes_total / (ms_e2e / args.steps * 1e-3) / 1e9
        per_rank_bytes = sum(algorithmic_bytes(n, N // world, K) for (n, N, K) in order)
        achieved = per_rank_bytes / (ms_step * 1e-3) / 1e9
        line = {
            "metric": "narrow_gemm_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": step_config(world),
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "GB/s", "mode": "CUDA graph of one step, a three-stage pipeline: the activations host -> device in two copies on a copy stream, the 21 public API calls on the compute stream as their inputs arrive (token counts in the order 1, 2, 4, 64, 32, 16, 8), every result device -> host on a second copy stream; the step ends when the last result is in host memory",
                    "eager_value": step_bytes_total / (ms_e2e_eager / args.steps * 1e-3) / 1e9,
                    "h2d_bytes_per_step": host_in.numel() * 2, "d2h_bytes_per_step": host_out.numel() * 2},
            "gpu_launches": len(order) * args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                         "traffic": NCU_TRAFFIC_RATIO * per_rank_bytes / len(order),
                         "traffic_source": "average bytes per launch = algorithmic bytes x 1.03, the dram read+write / "
                                           "algorithmic ratio ncu measured on the dense kernels (profiles/dense_kernels_bf16.md)",
                         "peak_source": f"of {peak_kind}",
                         "kernel": "dense_umma_kernel (17 launches) / gemv_simt_kernel (3) / dense_mma_kernel (1-2), averaged"},
        }
        if per_config is not None:
            line["per_config"] = per_config
        if world == 1 and not args.no_moe:
            # second half of the metric: fused-MoE layer time (router + alignment + experts + combine), CUDA-graph
            # replay over 8 different activation batches, see kernel_args_scan/moe_bench.py
            from muxi_native_layout_kernels_b200.kernel_args_scan import moe_bench
            line["moe_layer_us"] = moe_bench.run("both", None, 24, dev, peak=peak)
        if world > 1 and not args.no_moe:
            line["moe_layer_us"] = moe_ep
            line["moe_layer_mode"] = (f"expert parallel over {world} GPUs, E/{world} experts per rank, the modes of parallel.py on identical "
                                      "seeded weights: replicated (tokens on every rank, experts_map, NCCL all-reduce of the fp32 shares), replicated_peer_reduce "
                                      "(the same, shares added over NVLink peer memory by one kernel per rank, no NCCL call), "
                                      "all_to_all (tokens sharded, NCCL all-to-all dispatch of the routed rows and combine of fp32 rows) and "
                                      "gather_reduce_scatter (tokens sharded, all-gather + local share + reduce-scatter, static shapes); parity_ok = every rank's output "
                                      "of one batch equals the single-GPU layer within |d| <= 1e-2 max(1, rms) + 1e-2 |want|; "
                                      "us_eager = eager calls (host launch overhead included), us_graph = CUDA-graph replays; max over ranks")
        if world == 1 and not args.no_cpu:
            gbs, dt = time_cpu(passes=args.cpu_passes)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
                                    "sample": f"{args.cpu_passes} full passes over the 21-case grid, torch fp32 matmul, all host threads"}
            if not args.no_moe:
                line["cpu_baseline"]["moe_layer_us"] = time_cpu_moe()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--cpu-passes", type=int, default=5)
    ap.add_argument("--no-moe", action="store_true", help="skip the fused-MoE layer timings")
    ap.add_argument("--no-per-config", action="store_true", help="skip the per-configuration table (C1, C2 variants, C3)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
