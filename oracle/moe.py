"""TEST INFRASTRUCTURE -- CPU oracle for the fused MoE (router, token alignment, expert compute).

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline leg may import this package.

Restates, with torch on CPU:
  * the router of the reference's torch path (muxi_layout_kernels/utils.py:160-216) with the tie rule of its
    device kernel ("lower id wins", csrc/moe_kernels/fused_topK.h:255-262) -- torch.topk leaves ties unspecified;
  * the alignment contract of csrc/moe_kernels/moe_align_tokens.h:9-94 and moe_align_tokens.cu:5-21;
  * the dense per-expert loop of utils.py:217-244, in the activation dtype (five 16-bit roundings per token and a
    16-bit running sum over experts), plus an fp32 evaluation of the same math with the same routing decisions.
Pinned against outputs of the imported reference functions: tests/golden/make_golden.py -> tests/golden/moe_*.pt.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------------------------------------------
# router
# ---------------------------------------------------------------------------------------------------

def _topk_lower_id_wins(values: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest entries per row; among equal values the lower index is taken first."""
    order = torch.sort(values.to(torch.float32), dim=-1, descending=True, stable=True)[1]
    return order[:, :k]


def router_ref(logits: torch.Tensor, topk: int, num_expert_group: int = 1, topk_group: int = 1,
               bias: Optional[torch.Tensor] = None, score_func: str = "softmax") -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (ids int64 [T,topk] in selection order, weights [T,topk] in logits' dtype, masked selection scores
    [T,E]).  No renormalisation here (the caller does it, muxi_moe_planC.py:69-70)."""
    dtype = logits.dtype
    if score_func == "softmax":
        scores = torch.softmax(logits, dim=-1, dtype=dtype)          # utils.py:164
    elif score_func == "sigmoid":
        scores = torch.sigmoid(logits)                               # utils.py:166
    else:
        raise ValueError(score_func)
    sel = scores if bias is None else scores + bias.unsqueeze(0)    # utils.py:167-171
    T, E = sel.shape
    G = num_expert_group
    grouped = sel.view(T, G, E // G)
    if bias is None:
        gscore = grouped.max(dim=-1).values                          # utils.py:178-180
    elif E // G >= 2:
        gscore = grouped.topk(2, dim=-1)[0].sum(dim=-1)              # utils.py:174-176
    else:
        gscore = grouped[..., 0]
    keep = _topk_lower_id_wins(gscore, topk_group)                   # utils.py:184-185 + kernel tie rule
    gmask = torch.zeros(T, G, dtype=torch.bool).scatter_(1, keep, True)
    emask = gmask.unsqueeze(-1).expand(T, G, E // G).reshape(T, E)
    masked = sel.masked_fill(~emask, 0.0)                            # utils.py:196
    ids = _topk_lower_id_wins(masked, topk)                          # utils.py:198-210 + kernel tie rule
    weights = scores.gather(1, ids)                                  # un-biased scores (utils.py:201)
    return ids, weights, masked


def renormalize_ref(weights: torch.Tensor) -> torch.Tensor:
    return weights / weights.sum(dim=-1, keepdim=True)


def compare_topk(ids_got: torch.Tensor, ids_ref: torch.Tensor, masked: torch.Tensor) -> dict:
    """Tie-aware comparison of selected expert sets.  A row counts as a mismatch only if the sets differ AND the
    difference cannot be explained by equal selection scores at the cut (k-th and (k+1)-th oracle scores equal,
    and every disputed expert carries exactly that score)."""
    T, k = ids_ref.shape
    got = torch.sort(ids_got.to(torch.int64), dim=-1)[0]
    ref = torch.sort(ids_ref.to(torch.int64), dim=-1)[0]
    exact = (got == ref).all(dim=-1)
    ties = 0
    bad = 0
    m = masked.to(torch.float32)
    for t in torch.nonzero(~exact).flatten().tolist():
        g, r = set(got[t].tolist()), set(ref[t].tolist())
        cut = torch.sort(m[t], descending=True)[0][k - 1].item()
        disputed = (g ^ r)
        if len(g) == k and all(m[t, e].item() == cut for e in disputed):
            ties += 1
        else:
            bad += 1
    return {"rows": T, "exact": int(exact.sum()), "tie_rows": ties, "mismatch_rows": bad}


# ---------------------------------------------------------------------------------------------------
# alignment contract
# ---------------------------------------------------------------------------------------------------

def align_ref(topk_ids: torch.Tensor, num_experts: int, mbs: int = 16, experts_map: Optional[torch.Tensor] = None) -> dict:
    """Expected outputs of the alignment op, as far as they are determined (order inside an expert is not)."""
    flat = topk_ids.flatten().to(torch.int64)
    if experts_map is not None:
        flat = experts_map.to(torch.int64)[flat]
    numel = flat.numel()
    counts = torch.zeros(num_experts, dtype=torch.int64)
    valid = flat >= 0
    counts.scatter_add_(0, flat[valid], torch.ones(int(valid.sum()), dtype=torch.int64))
    padded = (counts + mbs - 1) // mbs * mbs
    ends = torch.cumsum(padded, 0)
    starts = ends - padded
    block_expert = torch.repeat_interleave(torch.arange(num_experts), padded // mbs)
    slots_of = [torch.nonzero(flat == e).flatten() for e in range(num_experts)]
    return {"counts": counts, "starts": starts, "padded_total": int(ends[-1]) if num_experts else 0,
            "num_blocks": int(ends[-1]) // mbs if num_experts else 0, "block_expert": block_expert,
            "slots_of": slots_of, "sentinel": numel, "cumsum_after": torch.cat([starts + counts, ends[-1:]])}


# ---------------------------------------------------------------------------------------------------
# expert compute
# ---------------------------------------------------------------------------------------------------

def experts_ref(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                compute_dtype: Optional[torch.dtype] = None, dense: bool = False) -> torch.Tensor:
    """y[t] = sum over experts e (ascending) of weight(t,e) * W2_e (up * silu(gate)),  [gate; up] = W1_e x[t].

    compute_dtype None  -> the reference's arithmetic: everything in x.dtype (utils.py:231-242).
    dense False         -> only the tokens routed to an expert are evaluated.  A token that is not routed to e
                           receives the exact addend 0 in the reference's loop, so this is the same sum; the CPU
                           GEMM may order its fp32 partial sums differently for a different row count, which is
                           why the golden-vector pin uses dense=True (every expert sees every token).
    compute_dtype fp32  -> same routing decisions, fp32 arithmetic, no intermediate rounding.
    w1 [E,2I,H] and w2 [E,H,I] are un-permuted; a 1-byte dtype is converted exactly to bf16 first."""
    dt = compute_dtype or x.dtype
    T, H = x.shape
    I = w2.shape[-1]
    xx = x.to(dt)
    ww = weights.to(dt)
    out = torch.zeros(T, H, dtype=dt)
    seen = torch.zeros(T, dtype=torch.bool)
    for e in range(w1.shape[0]):
        hit = (ids == e)
        rows = torch.arange(T) if dense else torch.nonzero(hit.any(dim=-1)).flatten()
        if rows.numel() == 0:
            continue
        w_e = (ww[rows] * hit[rows]).sum(dim=-1, keepdim=True)
        w1e = w1[e].to(torch.bfloat16).to(dt) if w1.element_size() == 1 else w1[e].to(dt)
        w2e = w2[e].to(torch.bfloat16).to(dt) if w2.element_size() == 1 else w2[e].to(dt)
        h = F.linear(xx[rows], w1e)
        h = h[:, I:] * F.silu(h[:, :I])
        contrib = F.linear(h, w2e) * w_e
        first = ~seen[rows]
        # the reference starts its running sum with the first expert's term (no 0 + term rounding difference
        # exists: 0 + v == v exactly), so plain accumulation reproduces it
        out[rows] = torch.where(first.unsqueeze(-1), contrib, out[rows] + contrib)
        seen[rows] = True
    return out


def fused_moe_ref(x, w1, w2, logits, topk, renormalize=True, num_expert_group=1, topk_group=1, bias=None,
                  score_func="softmax", compute_dtype=None, dense=False):
    """Router + renormalise + experts; returns (y, ids, weights, masked)."""
    ids, weights, masked = router_ref(logits, topk, num_expert_group, topk_group, bias, score_func)
    if renormalize:
        weights = renormalize_ref(weights)
    weights = weights.to(x.dtype)
    y = experts_ref(x, w1, w2, ids, weights, compute_dtype, dense)
    return y, ids, weights, masked
