"""Sharding of the weight-streaming path over the GPUs of one node (one process per GPU, torch.distributed).

The reference is single-GPU; its only hook is ``experts_map`` (csrc/moe_kernels/moe_align_tokens.h:46-49).  Two
natural partitions exist and both are provided here:

* dense layers: output features are independent, and layout A is row-group major, so rank g simply owns the weight
  rows ``[g*m/G, (g+1)*m/G)``; activations are replicated and no collective is needed (``all_gather_columns`` is
  there for callers that want the full ``y`` on every rank).
* fused MoE, expert parallel: rank g owns experts ``[g*E/G, (g+1)*E/G)``.
  - ``fused_moe_ep_replicated``: tokens replicated, every rank computes its experts' share through ``experts_map``
    and the shares are all-reduced (what the reference's hook supports).
  - ``fused_moe_ep``: tokens sharded; the router runs locally, every routed (token, slot) row travels to the rank
    that owns its expert (all-to-all), is processed there as a one-expert token, travels back (all-to-all) and the
    source rank adds each token's top-k rows in fp32 in a fixed order.

The exchange plan (who sends how many rows to whom, and where returned rows belong) is plain integer tensor
arithmetic and is kept separate from the device work (``plan_dispatch``) so that it runs -- and is tested -- on CPU
tensors with the gloo backend as well.  All NCCL traffic lands in this GPU's own memory before any kernel reads it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional

import torch
import torch.distributed as dist


# ---------------------------------------------------------------------------------------------------------
# dense layers
# ---------------------------------------------------------------------------------------------------------

def shard_rows(W: torch.Tensor, rank: int, world: int, multiple: int = 128) -> torch.Tensor:
    """Rows ``[rank*m/world, (rank+1)*m/world)`` of ``W[m,k]`` (contiguous).  The shard height must stay a multiple
    of ``multiple`` (128 for the GEMM entry points, 16 for GeMV)."""
    m = W.shape[0]
    if m % world != 0 or (m // world) % multiple != 0:
        raise ValueError(f"{m} rows cannot be split over {world} ranks in multiples of {multiple}")
    rows = m // world
    return W[rank * rows:(rank + 1) * rows].contiguous()


def all_gather_columns(y_local: torch.Tensor, group=None) -> torch.Tensor:
    """``y_local[n, m/G]`` of every rank -> ``y[n, m]`` on every rank (optional; the sharded layer itself needs no
    collective)."""
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    parts = [torch.empty_like(y_local) for _ in range(world)]
    dist.all_gather(parts, y_local.contiguous(), group=group)
    return torch.cat(parts, dim=-1)


# ---------------------------------------------------------------------------------------------------------
# expert-parallel exchange plan (device independent)
# ---------------------------------------------------------------------------------------------------------

@dataclass
class DispatchPlan:
    send_slot: torch.Tensor      # int32 [n_send]: flat slot (token*topk + j) of every row sent, grouped by destination
    send_token: torch.Tensor     # int32 [n_send]: source token of every row sent
    send_expert: torch.Tensor    # int32 [n_send]: expert id local to the destination rank
    send_counts: torch.Tensor    # int64 [world]: rows sent to each rank (same device as the routing)
    slot_to_row: torch.Tensor    # int32 [T*topk]: position of slot in the send order (= in the returned rows)


def plan_dispatch(topk_ids: torch.Tensor, experts_per_rank: int, world: int) -> DispatchPlan:
    """Groups the routed slots of this rank by destination rank (stable: ascending slot inside a destination).
    Pure tensor arithmetic on the device of ``topk_ids``: nothing is copied to the host here."""
    T, topk = topk_ids.shape
    flat = topk_ids.reshape(-1).to(torch.int64)
    dest = torch.div(flat, experts_per_rank, rounding_mode="floor")
    order = torch.sort(dest, stable=True)[1]
    counts = torch.bincount(dest, minlength=world)[:world]
    slot_to_row = torch.empty_like(order)
    slot_to_row[order] = torch.arange(order.numel(), device=order.device)
    return DispatchPlan(
        send_slot=order.to(torch.int32),
        send_token=torch.div(order, topk, rounding_mode="floor").to(torch.int32),
        send_expert=(flat[order] - dest[order] * experts_per_rank).to(torch.int32),
        send_counts=counts,
        slot_to_row=slot_to_row.to(torch.int32),
    )


def exchange_counts(send_counts: torch.Tensor, group=None):
    """All-to-all of the per-destination row counts, then ONE device -> host copy of both count vectors (the split
    sizes of the row exchange have to be host integers).  Returns (send_counts, recv_counts) as lists."""
    world = dist.get_world_size(group)
    s = send_counts.to(torch.int64)
    r = torch.empty(world, dtype=torch.int64, device=s.device)
    dist.all_to_all_single(r, s, group=group)
    both = torch.cat([s, r]).tolist()
    return [int(v) for v in both[:world]], [int(v) for v in both[world:]]


def _a2a(send: torch.Tensor, send_counts: List[int], recv_counts: List[int], group=None) -> torch.Tensor:
    recv = torch.empty((sum(recv_counts),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    dist.all_to_all_single(recv, send.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    return recv


# every routed row travels with its routing: [H activations | local expert id (int32) | routing weight (fp32)], padded
# to a multiple of 16 bytes, so that the dispatch is one all-to-all
_HEADER_BYTES = 16


def pack_rows(rows: torch.Tensor, expert: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """[R, H] 16-bit rows + int32 expert ids + weights -> uint8 [R, 2 H + 16]."""
    R, H = rows.shape
    buf = torch.empty(R, 2 * H + _HEADER_BYTES, dtype=torch.uint8, device=rows.device)
    buf[:, :2 * H] = rows.contiguous().view(torch.uint8).view(R, 2 * H)
    head = torch.zeros(R, 4, dtype=torch.int32, device=rows.device)
    head[:, 0] = expert
    head[:, 1] = weight.float().view(torch.int32)
    buf[:, 2 * H:] = head.view(torch.uint8).view(R, _HEADER_BYTES)
    return buf


def unpack_rows(buf: torch.Tensor, H: int, dtype: torch.dtype):
    R = buf.shape[0]
    rows = buf[:, :2 * H].contiguous().view(dtype).view(R, H)
    head = buf[:, 2 * H:].contiguous().view(torch.int32).view(R, 4)
    return rows, head[:, 0].contiguous(), head[:, 1].contiguous().view(torch.float32)


def moe_exchange(
    x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, experts_per_rank: int,
    experts_fn: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor],
    gather_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
    combine_fn: Callable[[torch.Tensor, torch.Tensor, int, int], torch.Tensor],
    group=None,
) -> torch.Tensor:
    """Dispatch -> local expert compute -> combine for this rank's tokens: two all-to-alls of rows (one packed buffer
    each way) after one small all-to-all of the counts and one device -> host copy.

    experts_fn(rows [R,H], local_expert [R] int32, weight [R] fp32) -> weighted outputs [R,H] in fp32
    gather_fn(x [T,H], token_index [R] int32) -> rows [R,H]
    combine_fn(rows [R,H] fp32, slot_to_row [T*topk] int32, T, topk) -> y [T,H] in x.dtype
    """
    world = dist.get_world_size(group)
    T, topk = topk_ids.shape
    H = x.shape[1]
    plan = plan_dispatch(topk_ids, experts_per_rank, world)
    send_counts, recv_counts = exchange_counts(plan.send_counts, group)
    rows = gather_fn(x, plan.send_token)
    w_send = topk_weights.reshape(-1)[plan.send_slot.long()]
    packed_in = _a2a(pack_rows(rows, plan.send_expert, w_send), send_counts, recv_counts, group)
    rows_in, e_in, w_in = unpack_rows(packed_in, H, x.dtype)
    out_rows = experts_fn(rows_in, e_in, w_in)
    back = _a2a(out_rows, recv_counts, send_counts, group)
    return combine_fn(back, plan.slot_to_row, T, topk)


# ---------------------------------------------------------------------------------------------------------
# GPU entry points
# ---------------------------------------------------------------------------------------------------------

def _gpu_gather(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    from ._lib import check, lib
    out = torch.empty((idx.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    check(lib.mlk_moe_gather_rows(x.data_ptr(), idx.data_ptr(), out.data_ptr(), idx.numel(), x.shape[1], x.shape[0],
                                  torch.cuda.current_stream(x.device).cuda_stream))
    return out


def _gpu_combine(rows: torch.Tensor, slot_to_row: torch.Tensor, T: int, topk: int, out_dtype=torch.bfloat16) -> torch.Tensor:
    """y[t] = round(sum_j rows[slot_to_row[t * topk + j]]), j ascending, fp32 rows: the single-GPU combine."""
    from ._lib import check, lib
    H = rows.shape[1]
    y = torch.empty((T, H), dtype=out_dtype, device=rows.device)
    code = (1 if out_dtype == torch.float16 else 0) + (2 if rows.dtype == torch.float32 else 0)
    check(lib.mlk_moe_unpermute_sum(rows.data_ptr() if rows.numel() else None, slot_to_row.data_ptr(), y.data_ptr(), T,
                                    topk, H, rows.shape[0], code, torch.cuda.current_stream(rows.device).cuda_stream))
    return y


def _expert_map(E: int, e_local: int, rank: int, device) -> torch.Tensor:
    emap = torch.full((E,), -1, dtype=torch.int32, device=device)
    emap[rank * e_local:(rank + 1) * e_local] = torch.arange(e_local, dtype=torch.int32, device=device)
    return emap


_MAPS = {}


def _cached_expert_map(E: int, e_local: int, rank: int, device) -> torch.Tensor:
    key = (E, e_local, rank, str(device))
    m = _MAPS.get(key)
    if m is None:
        m = _MAPS[key] = _expert_map(E, e_local, rank, device)
    return m


def fused_moe_ep(
    hidden_states: torch.Tensor, w1_local: torch.Tensor, w2_local: torch.Tensor, gating_output: torch.Tensor,
    topk: int, renormalize: bool, group=None, score_func: str = "softmax", num_expert_group: int = 1,
    topk_group: int = 1, gating_bias: Optional[torch.Tensor] = None, w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None, soft_fp8: bool = False, fp8_repacked: bool = False,
    exchange: str = "all_to_all",
) -> torch.Tensor:
    """Expert-parallel fused MoE for this rank's tokens ``hidden_states [T_local, H]``; ``w1_local [E/G, 2I, H]`` and
    ``w2_local [E/G, H, I]`` hold this rank's experts in layout A; ``gating_output [T_local, E]`` covers all experts.

    exchange="all_to_all": the router runs locally, every routed (token, slot) row travels to the rank that owns its
      expert with exactly the rows that are routed there (NCCL all-to-all with split sizes, which costs one
      device -> host copy of the counts per call: not capturable in a CUDA graph), is weighted there and comes back
      in fp32; the source rank adds each token's top-k rows in slot order and rounds once -- the arithmetic of the
      single-GPU layer.
    exchange="gather": static shapes, capturable.  Tokens and logits are all-gathered (every rank needs T_local equal),
      every rank computes the fp32 share of its experts for all tokens (``experts_map``) and a reduce-scatter hands
      each rank the sum for its own tokens.  With top-k of the order of the rank count nearly every token visits
      every rank anyway, and a fixed-capacity all-to-all would move the same bytes."""
    from . import ext
    T, H = hidden_states.shape
    E = gating_output.shape[1]
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    e_local = w1_local.shape[0]
    if e_local * world != E:
        raise ValueError(f"{E} experts over {world} ranks need {E // max(world, 1)} local experts, got {e_local}")
    dev = hidden_states.device
    if exchange == "gather":
        from .muxi_moe_planC import fused_moe
        x_all = torch.empty((world * T, H), dtype=hidden_states.dtype, device=dev)
        l_all = torch.empty((world * T, E), dtype=gating_output.dtype, device=dev)
        dist.all_gather_into_tensor(x_all, hidden_states.contiguous(), group=group)
        dist.all_gather_into_tensor(l_all, gating_output.contiguous(), group=group)
        kw = dict(w1_scale=w1_scale, w2_scale=w2_scale, block_shape=[128, 128], soft_fp8=True, fp8_repacked=fp8_repacked) if soft_fp8 else {}
        share = fused_moe(x_all, w1_local, w2_local, l_all, topk, renormalize, use_grouped_topk=num_expert_group != 1,
                          num_expert_group=num_expert_group, topk_group=topk_group, gating_bias=gating_bias,
                          score_func=score_func, experts_map=_cached_expert_map(E, e_local, rank, dev),
                          out_dtype=torch.float32, **kw)
        mine = torch.empty((T, H), dtype=torch.float32, device=dev)
        dist.reduce_scatter_tensor(mine, share, group=group)
        return mine.to(hidden_states.dtype)
    if exchange != "all_to_all":
        raise ValueError("exchange must be 'all_to_all' or 'gather'")
    ids = torch.empty(T, topk, dtype=torch.int32, device=dev)
    wts = torch.empty(T, topk, dtype=hidden_states.dtype, device=dev)
    ext.fused_routing_gate(gating_output, 0 if score_func == "softmax" else 1, T, H, num_expert_group, topk_group, ids,
                           wts, topk, gating_bias, renormalize=bool(renormalize))

    def experts_fn(rows, local_expert, weight):
        R = rows.shape[0]
        y = torch.zeros((R, H), dtype=torch.float32, device=dev)
        if R == 0:
            return y
        m1 = w1_local.shape[1]
        n_pad = R + e_local * 15
        sorted_ids = torch.empty((n_pad,), dtype=torch.int32, device=dev)
        cumsum = torch.empty(e_local + 1, dtype=torch.int32, device=dev)
        nblk = torch.empty(1, dtype=torch.int32, device=dev)
        blk = torch.empty((n_pad + 15) // 16, dtype=torch.int32, device=dev)
        C = torch.empty(m1 * R, dtype=rows.dtype, device=dev)
        args = (w1_local, w2_local, rows, R, e_local, 1, local_expert.view(R, 1).contiguous(),
                weight.to(rows.dtype).view(R, 1).contiguous(), sorted_ids, cumsum, nblk, blk, C, y)
        if soft_fp8:
            ext.fused_experts_compute(*args, w1_scale, w2_scale, [128, 128], True, fp8_repacked=fp8_repacked)
        else:
            ext.fused_experts_compute(*args)
        return y

    return moe_exchange(hidden_states, ids, wts, e_local, experts_fn, _gpu_gather,
                        lambda rows, s2r, T_, k_: _gpu_combine(rows, s2r, T_, k_, hidden_states.dtype), group)


class PeerReducer:
    """Buffers and launch of the expert-parallel combine over peer memory (``mlk_ep_reduce_shares``): every rank's fp32
    share ``[tokens, hidden]``, every rank's 16-bit output and a flag block, allocated as symmetric memory so that each
    rank holds pointers to all of them.  One kernel per rank adds the shares of the rows it owns in rank order, rounds
    once and stores the rows into every rank's output: a reduce-scatter and an all-gather in one pass over NVLink, no
    NCCL call, capturable in a CUDA graph.  All ranks must construct it collectively and call ``reduce`` in step."""

    def __init__(self, tokens: int, hidden: int, dtype: torch.dtype = torch.bfloat16, group=None, device=None):
        import torch.distributed._symmetric_memory as symm
        from ._lib import lib
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.tokens, self.hidden, self.dtype = tokens, hidden, dtype
        self.share = symm.empty((tokens, hidden), dtype=torch.float32, device=device)
        self.out = symm.empty((tokens, hidden), dtype=dtype, device=device)
        self.flags = symm.empty((int(lib.mlk_ep_reduce_flag_bytes()) // 4,), dtype=torch.int32, device=device)
        self.flags.zero_()
        # decode batches: receive buffer of the one-pass form (every rank's share arrives here as (value, epoch) pairs)
        recv_bytes = int(lib.mlk_ep_reduce_recv_bytes(self.world, tokens, hidden))
        self.recv = symm.empty((max(recv_bytes, 16) // 4,), dtype=torch.int32, device=device) if recv_bytes else None
        if self.recv is not None:
            self.recv.zero_()
        self._handles = [symm.rendezvous(t, group) for t in (self.share, self.out, self.flags)]
        self._recv_handle = symm.rendezvous(self.recv, group) if self.recv is not None else None
        torch.cuda.synchronize(device)
        dist.barrier(group)              # every rank's flag block is zero before anybody's first launch

    def reduce(self) -> torch.Tensor:
        """Adds the ranks' ``share`` buffers; returns ``out`` (the same tensor every call)."""
        from . import ext
        from ._lib import check, lib
        hs, ho, hf = self._handles
        check(lib.mlk_ep_reduce_shares(hs.buffer_ptrs_dev, ho.buffer_ptrs_dev, hf.buffer_ptrs_dev,
                                       self._recv_handle.buffer_ptrs_dev if self._recv_handle is not None else None,
                                       self.rank, self.world,
                                       self.tokens, self.hidden, 1 if self.dtype == torch.float16 else 0,
                                       ext._status_ptr(self.share), ext._stream(self.share)))
        return self.out


def fused_moe_ep_replicated(hidden_states, w1_local, w2_local, gating_output, topk, renormalize, group=None,
                            reduce_dtype: torch.dtype = torch.float32, reducer: Optional[PeerReducer] = None, **kw):
    """Tokens replicated on every rank; each rank adds its experts' share (``experts_map``) and the shares are summed
    with an all-reduce.  This is the expert-parallel mode the reference's ``experts_map`` hook was made for
    (csrc/moe_kernels/moe_align_tokens.h:44-49).  The shares leave the layer as un-rounded fp32 sums and are reduced in
    fp32 (one rounding at the end, as on one GPU); ``reduce_dtype=torch.bfloat16`` halves the all-reduce traffic at
    the price of one rounding per rank.  ``reducer`` (a ``PeerReducer`` for this token count) replaces the all-reduce and
    the cast by one peer-memory kernel per rank."""
    from .muxi_moe_planC import fused_moe
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    E = gating_output.shape[1]
    e_local = w1_local.shape[0]
    emap = _cached_expert_map(E, e_local, rank, hidden_states.device)
    if world == 1:
        return fused_moe(hidden_states, w1_local, w2_local, gating_output, topk, renormalize, experts_map=emap, **kw)
    if reducer is not None:
        # shares straight into peer-readable memory, one kernel per rank adds them over NVLink (fp32, rank order, one
        # rounding); the returned tensor is the reducer's output buffer
        fused_moe(hidden_states, w1_local, w2_local, gating_output, topk, renormalize, experts_map=emap,
                  out_dtype=torch.float32, out=reducer.share, **kw)
        return reducer.reduce()
    if reduce_dtype == torch.float32:
        share = fused_moe(hidden_states, w1_local, w2_local, gating_output, topk, renormalize, experts_map=emap,
                          out_dtype=torch.float32, **kw)
        dist.all_reduce(share, group=group)
        return share.to(hidden_states.dtype)
    share = fused_moe(hidden_states, w1_local, w2_local, gating_output, topk, renormalize, experts_map=emap, **kw)
    dist.all_reduce(share, group=group)
    return share
