"""Torch-level helpers the reference package exposes next to its kernels (muxi_layout_kernels/utils.py).

``fused_moe`` is the dense, per-expert torch formulation of the MoE layer that the reference's tests compare the
fused kernels with (utils.py:131-244); ``scale_tensor`` / ``scale_whole_tensor`` expand 128x128 block scales
(utils.py:7-25).  None of this is used by the CUDA path of this package; it exists so that code written against
the reference package (its tests, its benchmarks) keeps importing and running.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

_BLOCK = 128


def scale_tensor(weight: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """``weight[m,k]`` times the per-128x128-block factor ``scale[ceil(m/128), ceil(k/128)]``, in weight's dtype."""
    m, k = weight.shape
    full = scale.repeat_interleave(_BLOCK, dim=0)[:m].repeat_interleave(_BLOCK, dim=1)[:, :k]
    # the reference multiplies block by block with a 0-dim fp32 factor: fp32 product, one rounding
    return (weight.to(torch.float32) * full.to(torch.float32)).to(weight.dtype)


def scale_whole_tensor(weight: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Per-expert ``scale_tensor`` of ``weight[E,m,k]`` after converting it to bf16."""
    w = weight.to(torch.bfloat16)
    return torch.stack([scale_tensor(w[e], scale[e]) for e in range(w.shape[0])])


def _route(gating_output, topk, num_expert_group, topk_group, renormalize, bias, score_func, dtype):
    if score_func == "softmax":
        scores = torch.softmax(gating_output, dim=-1, dtype=dtype)
    elif score_func == "sigmoid":
        scores = torch.sigmoid(gating_output)
    else:
        raise ValueError("Unsupported scoring function")
    sel = scores if bias is None else scores + bias.unsqueeze(0)
    T = sel.shape[0]
    grouped = sel.view(T, num_expert_group, -1)
    group_scores = grouped.max(dim=-1).values if bias is None else grouped.topk(2, dim=-1)[0].sum(dim=-1)
    keep = torch.topk(group_scores, k=topk_group, dim=-1, sorted=False)[1]
    gmask = torch.zeros_like(group_scores).scatter_(1, keep, 1)
    emask = gmask.unsqueeze(-1).expand(T, num_expert_group, sel.shape[-1] // num_expert_group).reshape(T, -1)
    masked = sel.masked_fill(~emask.bool(), 0.0)
    ids = torch.topk(masked, k=topk, dim=-1, sorted=False)[1]
    weights = scores.gather(1, ids)     # un-biased scores are the routing weights
    if renormalize:
        weights = weights / weights.sum(dim=-1, keepdim=True)
    return ids, weights.to(dtype)


def fused_moe(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    gating_output: torch.Tensor,
    topk: int,
    num_expert_group: int = 0,
    topk_group: int = 1,
    global_num_experts: int = 1,
    expert_map: Optional[torch.Tensor] = None,
    renormalize: bool = False,
    e_score_correction_bias: Optional[torch.Tensor] = None,
    score_func: str = "softmax",
) -> torch.Tensor:
    """Dense-loop MoE on *un-permuted* weights ``w1 [E,2I,H]`` (gate rows then up rows) and ``w2 [E,H,I]``.
    Every expert processes every token; tokens not routed to it get weight 0.  All arithmetic runs in the dtype
    of ``hidden_states``, as in the reference."""
    orig_shape = hidden_states.shape
    H = hidden_states.shape[-1]
    dtype = hidden_states.dtype
    x = hidden_states.reshape(-1, H)
    logits = gating_output.reshape(x.shape[0], global_num_experts)
    groups = num_expert_group if num_expert_group else 1
    ids, weights = _route(logits, topk, groups, topk_group, renormalize, e_score_correction_bias, score_func, dtype)
    if expert_map is not None:
        ids = expert_map[ids]
    I = w2.shape[-1]
    out = None
    for e in range(w1.shape[0]):
        w_e = (weights * (ids == e)).sum(dim=-1, keepdim=True)
        h = F.linear(x, w1[e])
        h = h[:, I:] * F.silu(h[:, :I])
        contrib = F.linear(h, w2[e]) * w_e
        out = contrib if out is None else out + contrib
    return out.view(orig_shape)
