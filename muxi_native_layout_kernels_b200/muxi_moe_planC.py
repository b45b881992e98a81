"""Fused MoE layer, "plan C": router -> renormalise -> expert compute, with no host synchronisation.

Same signature and semantics as the reference's ``muxi_layout_kernels.muxi_moe_planC.fused_moe``
(muxi_layout_kernels/muxi_moe_planC.py:6-149); the reference's MetaX tile arguments are accepted and, apart from
``APerWarp``, ignored.  Differences a caller can rely on:
  * the router accepts any group configuration with ``num_experts % num_expert_group == 0`` (the reference
    kernel only 8 groups / 4 kept / top-8);
  * ``w1_scale``/``w2_scale`` may be ``None`` with ``soft_fp8=True`` (unit scales);
  * each token's expert outputs are summed in fp32 in a fixed order and rounded once (``deterministic=True``,
    the default); ``deterministic=False`` accumulates into ``y`` with 16-bit atomics like the reference;
  * the launch sequence is 5 kernels (router, alignment, GEMM1+SiLU, GEMM2, combine) instead of 6.
"""
from __future__ import annotations

from typing import List, Optional

import torch

import csv
from pathlib import Path

from . import ext

# Launch arguments of the expert-compute kernels, tuned offline by kernel_args_scan/moe_scan.py (the reference tunes
# its MoE tile arguments with kernel_args_scan/muxi_moe_args_scan.py and bakes them into this function's defaults).
# Key: (experts, topk, hidden, intermediate, fp8) -> [(tokens, (six ints))] sorted by tokens; the row with the
# smallest tokens >= the batch is used.  A missing key means automatic choice inside the library.
_MOE_TABLE_FILE = Path(__file__).resolve().parent / "moe_dispatch_arg.csv"
_MOE_TABLE = None


# Opt-in NVTX ranges around the stages of one layer call ("planC.router", "planC.experts"), for timelines taken with a
# system profiler; off by default (a range costs host time on every call).
_NVTX = False


def set_nvtx(enabled: bool) -> None:
    global _NVTX
    _NVTX = bool(enabled)


class _Range:
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if _NVTX:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if _NVTX:
            torch.cuda.nvtx.range_pop()
        return False


def _moe_table():
    global _MOE_TABLE
    if _MOE_TABLE is None:
        table = {}
        if _MOE_TABLE_FILE.exists():
            with open(_MOE_TABLE_FILE) as f:
                rows = csv.reader(f)
                next(rows, None)
                for r in rows:
                    if len(r) != 12:
                        continue
                    v = [int(x) for x in r]
                    table.setdefault(tuple(v[:5]), []).append((v[5], tuple(v[6:])))
            for rows_ in table.values():
                rows_.sort()
        _MOE_TABLE = table
    return _MOE_TABLE


def lookup_moe_args(E: int, topk: int, H: int, I: int, fp8: bool, T: int, allow_decode: bool = True):
    """Row of the smallest tabulated token count >= T (the last row beyond the table).  allow_decode=False skips rows
    of the single-kernel decode path (tuning values >= 300), which takes at most 8 tokens and 64 routed slots."""
    rows = _moe_table().get((E, topk, H, I, int(fp8)))
    if not rows:
        return None
    usable = [(t, args) for t, args in rows if allow_decode or args[1] < 300]
    if not usable:
        return None
    for t, args in usable:
        if t >= T:
            return args
    return usable[-1][1]


def fused_moe(
    hidden_states: torch.Tensor,  # [batch_size, hidden_size]
    w1: torch.Tensor,             # [E, 2I, H], every expert in layout A (gate rows first, then up rows)
    w2: torch.Tensor,             # [E, H, I],  every expert in layout A
    gating_output: torch.Tensor,  # [batch_size, num_experts] router logits
    topk: int,
    renormalize: bool,
    use_grouped_topk: bool = False,
    num_expert_group: Optional[int] = None,
    topk_group: Optional[int] = None,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[List[int]] = None,
    gating_bias: Optional[torch.Tensor] = None,
    score_func: str = "softmax",
    soft_fp8: bool = False,
    APerWarp: int = 2,
    splitK: int = 3,
    tile_m_2: int = 128,
    tile_n_2: int = 16,
    tile_k_2: int = 128,
    block_dim_x_gemm: int = 256,
    experts_map: Optional[torch.Tensor] = None,
    fp8_repacked: bool = False,
    deterministic: bool = True,
    tune=None,
    gate_weight: Optional[torch.Tensor] = None,
    out_dtype: Optional[torch.dtype] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    # gate_weight [E, H] (extension): the router GEMM runs fused with the routing kernel and `gating_output` is not
    # read (pass None)
    assert gate_weight is not None or hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    if num_expert_group is None:
        num_expert_group = 1
    if topk_group is None:
        topk_group = 1
    if not use_grouped_topk and num_expert_group != 1:
        raise ValueError("When use_grouped_topk is False, num_expert_group must be 1.")

    shape = hidden_states.size()
    B, H = hidden_states.shape
    num_experts = gate_weight.shape[0] if gate_weight is not None else gating_output.shape[1]
    dev = hidden_states.device

    if score_func == "softmax":
        score_fun = 0
    elif score_func == "sigmoid":
        score_fun = 1
    else:
        raise ValueError("Unsupported scoring function")

    # 1. router
    topk_ids = torch.empty(B, topk, dtype=torch.int32, device=dev)
    topk_weights = torch.empty(B, topk, dtype=hidden_states.dtype, device=dev)
    e1, m1, k1 = w1.shape
    e2, m2, k2 = w2.shape
    if tune is None:
        # with an experts_map (expert parallelism) this rank sees e1 of the num_experts experts and, on average, that
        # share of the routed slots: the expert GEMMs have the work items of a layer with e1 experts and
        # B * e1 / num_experts tokens, and that row applies
        t_eff = B if experts_map is None else max(1, -(-B * e1 // num_experts))
        decode_ok = B <= 8 and B * topk <= 64
        tune = lookup_moe_args(e1, topk, H, k2, soft_fp8, t_eff, decode_ok)
        if tune is None and experts_map is not None:
            tune = lookup_moe_args(num_experts, topk, H, k2, soft_fp8, B, decode_ok)   # no row for the local count: the full layer's
    # decode batches tuned for the single-kernel path: the routing runs inside the expert-compute call (one launch
    # for the whole layer); otherwise the router kernel comes first
    routing = None
    if gate_weight is None and tune is not None and len(tune) == 6 and tune[1] >= 300 and tune[4] >= 300 and B <= 8 and B * topk <= 64 \
            and num_experts <= 256:
        routing = (gating_output, score_fun, num_expert_group, topk_group, gating_bias, bool(renormalize))
    # renormalisation (reference: two torch ops, muxi_moe_planC.py:69-70) happens inside the router kernel, with the
    # same roundings
    elif gate_weight is not None:
        with _Range("planC.router"):
            ext.fused_router_gemm_gate(hidden_states, gate_weight, score_fun, num_expert_group, topk_group, topk_ids,
                                       topk_weights, topk, gating_bias, renormalize=bool(renormalize))
    else:
        with _Range("planC.router"):
            ext.fused_routing_gate(gating_output, score_fun, B, H, num_expert_group, topk_group, topk_ids, topk_weights,
                                   topk, gating_bias, renormalize=bool(renormalize))

    # 2. experts
    assert e1 == e2
    assert k1 == m2
    micro_batchsize = 16
    max_num_tokens_padded = topk * B + num_experts * (micro_batchsize - 1)
    # the alignment kernel writes the sentinel itself: no fill kernel needed
    sorted_token_ids = torch.empty((max_num_tokens_padded,), dtype=torch.int32, device=dev)
    cumsum_buffer = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    padded_num_experts = torch.empty(1, dtype=torch.int32, device=dev)
    experts_ids = torch.empty((max_num_tokens_padded + micro_batchsize - 1) // micro_batchsize, dtype=torch.int32,
                              device=dev)
    # workspace: the fused GEMM1 epilogue writes [B*topk, I] activations into the first half; the second half
    # holds the expert work list.  Nothing in it has to be zero.
    C = torch.empty(topk * m1 * B, dtype=hidden_states.dtype, device=dev)
    # the fixed-order combine writes every element of y; the atomic variant accumulates into zeros
    # out_dtype=torch.float32 (extension, deterministic only): the sums over this rank's experts un-rounded, for callers
    # that add the shares of several ranks before the one rounding
    # out (extension): the tensor the result is written to (e.g. a buffer other GPUs can read), contiguous, of the
    # result's shape and dtype
    if out_dtype is not None and out_dtype != hidden_states.dtype:
        if out_dtype != torch.float32 or not deterministic:
            raise ValueError("out_dtype must be the activation dtype or torch.float32 (with deterministic=True)")
        y = torch.empty(hidden_states.shape, dtype=torch.float32, device=dev) if out is None else out
    elif out is not None:
        y = out if deterministic else out.zero_()
    else:
        y = torch.empty_like(hidden_states) if deterministic else torch.zeros_like(hidden_states)
    if out is not None and (out.shape != hidden_states.shape or not out.is_contiguous() or
                            out.dtype != (out_dtype or hidden_states.dtype)):
        raise ValueError("out must be contiguous with the result's shape and dtype")

    if experts_map is not None and experts_map.dtype != torch.int:
        experts_map = experts_map.to(torch.int)
    with _Range("planC.experts" if routing is None else "planC.router+experts"):
        _experts(soft_fp8, w1, w2, hidden_states, B, e1, topk, topk_ids, topk_weights, sorted_token_ids, cumsum_buffer,
                 padded_num_experts, experts_ids, C, y, w1_scale, w2_scale, block_shape, experts_map, fp8_repacked,
                 deterministic, tune, routing, APerWarp, splitK, tile_m_2, tile_n_2, tile_k_2, block_dim_x_gemm)
    return y.view(shape)


def _experts(soft_fp8, w1, w2, hidden_states, B, e1, topk, topk_ids, topk_weights, sorted_token_ids, cumsum_buffer,
             padded_num_experts, experts_ids, C, y, w1_scale, w2_scale, block_shape, experts_map, fp8_repacked,
             deterministic, tune, routing, APerWarp, splitK, tile_m_2, tile_n_2, tile_k_2, block_dim_x_gemm):
    if soft_fp8:
        ext.fused_experts_compute(w1, w2, hidden_states, B, e1, topk, topk_ids, topk_weights, sorted_token_ids,
                                  cumsum_buffer, padded_num_experts, experts_ids, C, y, w1_scale, w2_scale,
                                  block_shape if block_shape is not None else [128, 128], soft_fp8,
                                  experts_map=experts_map, fp8_repacked=fp8_repacked, deterministic=deterministic,
                                  tune=tune, routing=routing)
    else:
        ext.fused_experts_compute(w1, w2, hidden_states, B, e1, topk, topk_ids, topk_weights, sorted_token_ids,
                                  cumsum_buffer, padded_num_experts, experts_ids, C, y, APerWarp=APerWarp,
                                  splitK=splitK, tile_m_2=tile_m_2, tile_n_2=tile_n_2, tile_k_2=tile_k_2,
                                  block_dim_x_gemm=block_dim_x_gemm, experts_map=experts_map,
                                  deterministic=deterministic, tune=tune, routing=routing)


class GraphedFusedMoE:
    """``fused_moe`` for a fixed token count, captured once in a CUDA graph.

    The eager call spends more time in Python, the allocator and the launches (eight ``torch.empty`` and five to six
    kernel launches) than the GPU spends on the layer when the batch is small.  This object owns static input, routing and
    workspace buffers, captures the layer's launches once, and replays them: ``layer(hidden_states, gating_output)``
    copies the two inputs into the static buffers, replays the graph on the current stream and returns the static
    output tensor (valid until the next call; clone it to keep it).  Weights, scales, bias and the expert map are
    captured by address: update them in place.  The reference has no counterpart (its planC is eager only).
    """

    def __init__(self, w1, w2, tokens: int, num_experts: int, topk: int, renormalize: bool, dtype=torch.bfloat16, **kwargs):
        dev = w1.device
        H = w1.shape[2]
        self.x = torch.zeros(tokens, H, dtype=dtype, device=dev)
        self.logits = torch.zeros(tokens, num_experts, dtype=dtype, device=dev)
        self._args = (w1, w2, topk, renormalize, kwargs)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):                      # warm-up: table loading, attribute setting, allocator growth
                fused_moe(self.x, w1, w2, self.logits, topk, renormalize, **kwargs)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self.y = fused_moe(self.x, w1, w2, self.logits, topk, renormalize, **kwargs)
        torch.cuda.current_stream(dev).wait_stream(side)

    def __call__(self, hidden_states: torch.Tensor, gating_output: torch.Tensor) -> torch.Tensor:
        if hidden_states.shape != self.x.shape or gating_output.shape != self.logits.shape:
            raise ValueError(f"captured for {tuple(self.x.shape)} tokens x hidden and {tuple(self.logits.shape)} logits")
        self.x.copy_(hidden_states)
        self.logits.copy_(gating_output)
        self.graph.replay()
        return self.y
