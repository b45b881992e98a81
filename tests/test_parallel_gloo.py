"""Multi-process (gloo, CPU, world size 2) tests of the sharding logic: the expert-parallel exchange plan with both
all-to-alls, and the row sharding of dense layers.  The expert arithmetic is done by the CPU oracle here; the GPU
tests cover the kernels themselves."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

from muxi_native_layout_kernels_b200 import parallel
from oracle import dense as odense
from oracle import moe as omoe

WORLD = 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs():
    g = torch.Generator().manual_seed(900)
    E, topk, H, I, T = 8, 3, 64, 32, 10           # T tokens per rank
    x = torch.randn(WORLD * T, H, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.1).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.1).to(torch.bfloat16)
    logits = torch.randn(WORLD * T, E, generator=g).to(torch.bfloat16)
    return E, topk, H, I, T, x, w1, w2, logits


def _worker(rank, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        torch.set_num_threads(1)
        E, topk, H, I, T, x, w1, w2, logits = _inputs()
        e_local = E // WORLD
        xs, ls = x[rank * T:(rank + 1) * T], logits[rank * T:(rank + 1) * T]
        ids, wts, _ = omoe.router_ref(ls, topk)
        wts = omoe.renormalize_ref(wts).to(x.dtype)
        w1l, w2l = w1[rank * e_local:(rank + 1) * e_local], w2[rank * e_local:(rank + 1) * e_local]

        def experts_fn(rows, local_expert, weight):
            y = torch.zeros(rows.shape, dtype=torch.float32)
            for r in range(rows.shape[0]):
                e = int(local_expert[r])
                h = w1l[e].float() @ rows[r].float()
                a = (F.silu(h[:I]) * h[I:]).to(x.dtype).float()        # the kernels round the activation once
                y[r] = float(weight[r]) * (w2l[e].float() @ a)
            return y                                                   # fp32 rows travel back

        gather_fn = lambda t, idx: t[idx.long()]

        def combine_fn(rows, slot_to_row, T_, topk_):
            assert rows.dtype == torch.float32
            return rows[slot_to_row.long()].view(T_, topk_, -1).sum(1).to(x.dtype)

        y = parallel.moe_exchange(xs, ids.to(torch.int32), wts, e_local, experts_fn, gather_fn, combine_fn)
        y32 = omoe.experts_ref(xs, w1, w2, ids, wts, compute_dtype=torch.float32)
        rep = odense.error_report(y, y32, atol=2e-2, rtol=2e-2)
        # dense row sharding: the two shards' outputs are the two column halves of the full product
        W = w1[0]
        Xd = x[:4]
        y_loc = odense.gemm_ref(Xd, parallel.shard_rows(W, rank, WORLD, multiple=16))
        y_all = parallel.all_gather_columns(y_loc)
        dense_ok = torch.equal(y_all, odense.gemm_ref(Xd, W))
        plan = parallel.plan_dispatch(ids.to(torch.int32), e_local, WORLD)
        plan_ok = (int(plan.send_counts.sum()) == T * topk and
                   bool((plan.send_slot.long()[plan.slot_to_row.long()] == torch.arange(T * topk)).all()) and
                   bool((plan.send_expert >= 0).all()) and bool((plan.send_expert < e_local).all()))
        out.put((rank, rep, dense_ok, plan_ok))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_exchange_and_row_sharding_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in range(WORLD)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, rep, dense_ok, plan_ok in results:
        assert rep["ok"], (rank, rep)
        assert dense_ok and plan_ok, (rank, dense_ok, plan_ok)


def test_plan_dispatch_single_process():
    ids = torch.tensor([[0, 5], [7, 1], [2, 3]], dtype=torch.int32)
    plan = parallel.plan_dispatch(ids, experts_per_rank=4, world=2)
    assert plan.send_counts.tolist() == [4, 2]
    assert plan.send_slot.tolist() == [0, 3, 4, 5, 1, 2]          # stable inside a destination
    assert plan.send_token.tolist() == [0, 1, 2, 2, 0, 1]
    assert plan.send_expert.tolist() == [0, 1, 2, 3, 1, 3]
    assert plan.slot_to_row.tolist() == [0, 4, 5, 1, 2, 3]


def test_packed_dispatch_rows_round_trip():
    g = torch.Generator().manual_seed(5)
    rows = torch.randn(7, 64, generator=g).to(torch.bfloat16)
    expert = torch.arange(7, dtype=torch.int32) * 3 - 2
    weight = torch.rand(7, generator=g).to(torch.bfloat16)
    buf = parallel.pack_rows(rows, expert, weight)
    assert buf.shape == (7, 2 * 64 + 16) and buf.dtype == torch.uint8
    r2, e2, w2 = parallel.unpack_rows(buf, 64, torch.bfloat16)
    assert torch.equal(r2, rows) and torch.equal(e2, expert) and torch.equal(w2, weight.float())


def test_shard_rows_rejects_uneven_split():
    import pytest
    with pytest.raises(ValueError):
        parallel.shard_rows(torch.zeros(384, 8), 0, 2, multiple=128)
