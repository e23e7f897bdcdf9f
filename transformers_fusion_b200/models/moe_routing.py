"""Routing rules of the mixture-of-experts variants that are not plain top-k, and the expert-capacity policies.

Every rule turns the router logits [T, E] into a *selection*: a boolean matrix ``sel`` [T, E] (which experts serve which
token).  The expert path itself stays the fused one (``ops.moe.moe_ffn``: soft-max + top-k + grouped GEMMs on the device):
the selection is handed to it as masked logits (unselected experts at -1e4, so the soft-max runs over the selected experts
only and the top-k picks exactly them), plus a per-token ``covered`` flag that zeroes the output of tokens no expert serves
and, for the pass-through policy, the gate mass that bypasses the experts.

  expert_choice     every expert takes its C best tokens, C = capacity_factor * T / E (a token may get 0..k experts)
  hierarchical      experts in G groups: the best ``top_groups`` groups by group score, then the best expert(s) in each
  base_layer        balanced assignment: every expert gets the same number of tokens (greedy auction over the scores)
  capacity policies after top-k: FIXED re-routes (token, expert) pairs beyond an expert's capacity to the token's
                    next-best expert, TOKEN_DROP removes them, TOKEN_PASS removes them and lets that share of the token
                    pass through unchanged

Reference counterparts: ExpertChoiceMoE / HierarchicalMoE / BaseLayerMoE and CapacityStrategy
(include/quant/moe_variants.h:19-123, src/model/moe_advanced_support.cpp:158-330, 646-700; compute_capacity :183, :296)."""
from __future__ import annotations

import math

import torch

MASKED = -1.0e4


def expert_choice_capacity(T: int, E: int, capacity_factor: float) -> int:
    """Tokens per expert (reference ExpertChoiceMoE::compute_capacity)."""
    return max(1, int(capacity_factor * T / E))


def expert_choice(logits: torch.Tensor, capacity_factor: float, max_per_token: int):
    """sel [T, E]: token t is among expert e's top-C tokens by router probability; a token keeps at most
    ``max_per_token`` of the experts that chose it (its best ones)."""
    T, E = logits.shape
    probs = torch.softmax(logits.float(), -1)
    C = min(T, expert_choice_capacity(T, E, capacity_factor))
    top_t = torch.topk(probs, C, dim=0).indices                       # [C, E]: the tokens each expert takes
    sel = torch.zeros((T, E), dtype=torch.bool, device=logits.device)
    sel.scatter_(0, top_t, True)
    if max_per_token < E:
        keep = torch.topk(torch.where(sel, probs, torch.full_like(probs, -1.0)), max_per_token, dim=1).indices
        cap = torch.zeros_like(sel)
        cap.scatter_(1, keep, True)
        sel &= cap
    return sel


def hierarchical(logits: torch.Tensor, num_groups: int, top_groups: int, top_per_group: int = 1):
    """sel [T, E] with E = num_groups * experts_per_group: group score = log-sum-exp of its experts' logits; the best
    ``top_groups`` groups are kept and inside each the best ``top_per_group`` experts."""
    T, E = logits.shape
    assert E % num_groups == 0, "experts must divide into the groups"
    per = E // num_groups
    z = logits.float().view(T, num_groups, per)
    gscore = torch.logsumexp(z, -1)                                   # [T, G]
    gsel = torch.zeros((T, num_groups), dtype=torch.bool, device=logits.device)
    gsel.scatter_(1, torch.topk(gscore, min(top_groups, num_groups), dim=1).indices, True)
    esel = torch.zeros((T, num_groups, per), dtype=torch.bool, device=logits.device)
    esel.scatter_(2, torch.topk(z, min(top_per_group, per), dim=2).indices, True)
    return (esel & gsel[:, :, None]).view(T, E)


def base_layer(logits: torch.Tensor):
    """Balanced one-expert-per-token assignment: every expert serves ceil(T / E) tokens at most.  Greedy auction: in each
    round every unassigned token bids for its best expert that still has room and each expert takes its highest bids."""
    T, E = logits.shape
    cap = math.ceil(T / E)
    score = logits.float().clone()
    assign = torch.full((T,), -1, dtype=torch.long, device=logits.device)
    room = torch.full((E,), cap, dtype=torch.long, device=logits.device)
    for _ in range(E):
        free = assign < 0
        if not bool(free.any()):
            break
        s = torch.where((room > 0)[None, :], score, torch.full_like(score, -float("inf")))
        bid = s.argmax(-1)                                            # [T]
        val = s.gather(1, bid[:, None])[:, 0]
        val = torch.where(free, val, torch.full_like(val, -float("inf")))
        # per expert: accept the best `room` bidders
        order = torch.argsort(val, descending=True)
        e_sorted = bid[order]
        ok_sorted = torch.isfinite(val[order])
        rank_in_e = torch.zeros(T, dtype=torch.long, device=logits.device)
        onehot = torch.nn.functional.one_hot(e_sorted, E) * ok_sorted[:, None]
        rank_in_e = (onehot.cumsum(0) * onehot).sum(-1) - 1          # position of each bidder in its expert's queue
        take = ok_sorted & (rank_in_e < room[e_sorted])
        tok = order[take]
        assign[tok] = e_sorted[take]
        room -= torch.bincount(e_sorted[take], minlength=E)
    sel = torch.zeros((T, E), dtype=torch.bool, device=logits.device)
    sel[torch.arange(T, device=logits.device)[assign >= 0], assign[assign >= 0]] = True
    return sel


def capacity_limit(T: int, E: int, k: int, capacity_factor: float) -> int:
    return max(1, int(math.ceil(capacity_factor * T * k / E)))


def apply_capacity(logits: torch.Tensor, k: int, capacity_factor: float, policy: str):
    """Top-k selection under a per-expert capacity.  Returns (sel [T, E], passthrough [T]): ``passthrough`` is the share of
    each token's gate mass that bypasses the experts (TOKEN_PASS; zeros for the other policies).  Within an expert, pairs
    are kept in order of gate weight."""
    T, E = logits.shape
    policy = policy.lower()
    probs = torch.softmax(logits.float(), -1)
    w, idx = torch.topk(probs, k, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    cap = capacity_limit(T, E, k, capacity_factor)

    def overflow(idx_, w_):
        """keep [T, k]: the pair is among the `cap` heaviest pairs of its expert."""
        flat_e, flat_w = idx_.reshape(-1), w_.reshape(-1)
        order = torch.argsort(flat_w, descending=True, stable=True)
        onehot = torch.nn.functional.one_hot(flat_e[order], E)
        pos = (onehot.cumsum(0) * onehot).sum(-1) - 1
        keep = torch.empty_like(pos, dtype=torch.bool)
        keep[order] = pos < cap
        return keep.view_as(idx_)
    keep = overflow(idx, w)
    sel = torch.zeros((T, E), dtype=torch.bool, device=logits.device)
    sel.scatter_(1, idx, keep)
    passthrough = torch.zeros(T, dtype=torch.float32, device=logits.device)
    if policy == "fixed":
        # one round of re-routing: a token that lost a pair takes its best expert among those with room left
        counts = sel.sum(0)
        lost = (~keep).sum(-1)
        room = (cap - counts).clamp(min=0)
        cand = torch.where(sel | (room == 0)[None, :], torch.full_like(probs, -1.0), probs)
        extra = torch.topk(cand, k, dim=-1)
        for j in range(k):
            want = (lost > j) & (extra.values[:, j] > 0)
            e_j = extra.indices[:, j]
            # respect the remaining room in token order
            onehot = torch.nn.functional.one_hot(e_j, E) * want[:, None]
            pos = (onehot.cumsum(0) * onehot).sum(-1) - 1
            ok = want & (pos < room[e_j])
            sel[torch.arange(T, device=logits.device)[ok], e_j[ok]] = True
            room = room - torch.bincount(e_j[ok], minlength=E)
    elif policy == "token_pass":
        passthrough = (w * (~keep)).sum(-1)
    elif policy != "token_drop":
        raise ValueError(f"unknown capacity policy '{policy}' (fixed | token_drop | token_pass)")
    return sel, passthrough


def masked_logits(logits: torch.Tensor, sel: torch.Tensor):
    """(logits with unselected experts at MASKED, covered [T] bool).  Gradients reach the router through the selected
    entries only, exactly as through a top-k."""
    return torch.where(sel, logits, torch.full_like(logits, MASKED)), sel.any(-1)
