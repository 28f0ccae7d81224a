"""CPU oracle of expert-parallel routing, dedup, inverse routes and combine.

Everything here runs on CPU tensors for ALL ranks of a group at once, so it is
both the semantic reference the device kernels are diffed against bit for bit
and the planner of the host-staged transport. It states the same contract as
the reference's pure-Python planner (ep_xpress/routing.py:45-164) and combine
oracle (benchmarks/replay.py:74-85), written as vectorised tensor code:

* ``-1`` marks a dropped slot; a row of only ``-1`` is a padding token that is
  sent nowhere and combines to a zero row at its source position;
* weights paired with ``-1`` are ignored and canonicalised to 0 (even NaN/Inf),
  active weights must be finite, an expert may appear once per token;
* ONE row per (token, destination rank), however many of the token's experts
  live there; destination rows are ordered by (source rank, token);
* local expert ids count the owner's experts in order of appearance in
  ``expert_to_rank``; weights of all active slots travel unscaled.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch

MAX_WORLD = 63


@dataclass
class RankRoutes:
    """What one destination rank receives, in (source rank, token) order."""
    source_rank: torch.Tensor   # int64 [rows]
    source_token: torch.Tensor  # int64 [rows]
    local_ids: torch.Tensor     # int64 [rows, topk]   -1 where the expert lives elsewhere
    weights: torch.Tensor       # float32 [rows, topk] active weights, 0 for dropped slots

    @property
    def rows(self) -> int:
        return int(self.source_rank.numel())

    @property
    def inverse(self) -> torch.Tensor:
        return torch.stack([self.source_rank, self.source_token], dim=1)


@dataclass
class RoutePlan:
    world_size: int
    topk: int
    expert_to_rank: List[int]
    expert_local: List[int]
    token_counts: List[int]
    dest_masks: List[torch.Tensor]      # per source rank: int64 [tokens] bit d set <=> a row goes to rank d
    dest_rows: List[torch.Tensor]       # per source rank: int64 [tokens, world] row index at rank d or -1
    received: List[RankRoutes]          # per destination rank

    def remote_masks(self):
        """Destination masks without the source's own bit (what crosses the interconnect)."""
        return [mask & ~(1 << rank) for rank, mask in enumerate(self.dest_masks)]


def expert_local_ids(expert_to_rank: Sequence[int], world_size: int) -> List[int]:
    seen = [0] * world_size
    local = []
    for owner in expert_to_rank:
        local.append(seen[owner])
        seen[owner] += 1
    return local


def _as_owner_list(expert_to_rank, world_size):
    owners = [int(owner) for owner in (expert_to_rank.tolist() if isinstance(expert_to_rank, torch.Tensor)
                                       else expert_to_rank)]
    if not owners:
        raise ValueError("expert_to_rank must contain at least one expert")
    if any(isinstance(o, bool) or o < 0 or o >= world_size for o in owners):
        raise ValueError("expert owner is outside the supported range")
    return owners


def plan_routes(ids_by_rank, weights_by_rank, expert_to_rank, world_size: int, topk: int) -> RoutePlan:
    """Validate every rank's router output, then build the group-wide plan."""
    if isinstance(world_size, bool) or not isinstance(world_size, int) or not 1 <= world_size <= MAX_WORLD:
        raise ValueError("world_size is outside the supported range")
    if isinstance(topk, bool) or not isinstance(topk, int) or topk < 1:
        raise ValueError("topk is outside the supported range")
    if len(ids_by_rank) != world_size or len(weights_by_rank) != world_size:
        raise ValueError("ids_by_rank and weights_by_rank must contain one entry per rank")
    owners = _as_owner_list(expert_to_rank, world_size)
    num_experts = len(owners)
    local_of = expert_local_ids(owners, world_size)
    owner_t = torch.tensor(owners, dtype=torch.int64)
    local_t = torch.tensor(local_of, dtype=torch.int64)

    cleaned = []
    for source in range(world_size):
        ids = torch.as_tensor(ids_by_rank[source]).to(torch.int64).reshape(-1, topk) \
            if torch.as_tensor(ids_by_rank[source]).numel() else torch.zeros((0, topk), dtype=torch.int64)
        raw_w = torch.as_tensor(weights_by_rank[source])
        weights = raw_w.to(torch.float32).reshape(-1, topk) if raw_w.numel() else torch.zeros((0, topk))
        if ids.shape != weights.shape:
            raise ValueError("expert IDs and weights must have equal token counts")
        if ((ids < -1) | (ids >= num_experts)).any():
            raise ValueError("expert ID is outside the supported range")
        active = ids >= 0
        if not torch.isfinite(weights[active]).all():
            bad = (active & ~torch.isfinite(weights)).nonzero()[0].tolist()
            raise ValueError(f"active router weights must be finite real numbers (rank={source}, "
                             f"token={bad[0]}, slot={bad[1]})")
        if ids.shape[0]:
            ordered, _ = torch.sort(torch.where(active, ids, torch.arange(-topk, 0).expand_as(ids)), dim=1)
            if (ordered[:, 1:] == ordered[:, :-1]).any():
                raise ValueError("a token cannot select the same expert twice")
        cleaned.append((ids, torch.where(active, weights, torch.zeros_like(weights))))

    token_counts = [ids.shape[0] for ids, _ in cleaned]
    masks, per_source_hits = [], []
    for ids, _ in cleaned:
        active = ids >= 0
        dest = owner_t[ids.clamp(min=0)]
        # Duplicates collapse (one row per (token, rank)); a dropped slot never hides an active one.
        hit = torch.zeros((ids.shape[0], world_size), dtype=torch.int64).scatter_add_(1, dest, active.to(torch.int64)) > 0
        per_source_hits.append(hit)
        masks.append((hit.to(torch.int64) << torch.arange(world_size)).sum(dim=1))

    received, dest_rows = [], [torch.full((n, world_size), -1, dtype=torch.int64) for n in token_counts]
    for dest in range(world_size):
        src_rank, src_token, rows_ids, rows_w = [], [], [], []
        base = 0
        for source, (ids, weights) in enumerate(cleaned):
            tokens = per_source_hits[source][:, dest].nonzero().flatten()
            dest_rows[source][tokens, dest] = base + torch.arange(tokens.numel())
            base += tokens.numel()
            sel = ids[tokens]
            here = (sel >= 0) & (owner_t[sel.clamp(min=0)] == dest)
            rows_ids.append(torch.where(here, local_t[sel.clamp(min=0)], torch.full_like(sel, -1)))
            rows_w.append(weights[tokens])
            src_rank.append(torch.full((tokens.numel(),), source, dtype=torch.int64))
            src_token.append(tokens)
        received.append(RankRoutes(torch.cat(src_rank), torch.cat(src_token),
                                   torch.cat(rows_ids).reshape(-1, topk), torch.cat(rows_w).reshape(-1, topk)))
    return RoutePlan(world_size, topk, owners, local_of, token_counts, masks, dest_rows, received)


def dispatch_oracle(x_by_rank, plan: RoutePlan):
    """Activation rows every destination rank must receive (BF16, exact copies)."""
    out = []
    for routes in plan.received:
        parts = [x_by_rank[s][routes.source_token[routes.source_rank == s]] for s in range(plan.world_size)]
        hidden = x_by_rank[0].shape[1]
        out.append(torch.cat(parts) if parts else torch.zeros((0, hidden), dtype=torch.bfloat16))
    return out


def scale_expert_oracle(hidden, local_ids, weights, factors=None):
    """Synthetic expert: row * sum_k w_k * factor[local_id_k] over local slots.

    The scale is accumulated in FP32 in slot order with separately rounded
    multiply and add, and the product is rounded once to BF16.
    """
    rows, topk = local_ids.shape
    scale = torch.zeros(rows, dtype=torch.float32)
    for k in range(topk):
        lid = local_ids[:, k]
        here = lid >= 0
        factor = torch.ones(rows) if factors is None else factors[lid.clamp(min=0, max=factors.numel() - 1)]
        term = (weights[:, k].to(torch.float32) * factor.to(torch.float32))
        scale = torch.where(here, scale + term, scale)
    return (hidden.to(torch.float32) * scale[:, None]).to(torch.bfloat16)


def combine_oracle(partials_by_rank, plan: RoutePlan, hidden_size: int, rounding: str = "two_step"):
    """Rank-order FP32 combine of already-weighted BF16 partial rows.

    ``two_step``: remote ranks are summed in ascending rank order in FP32
    starting from +0, rounded to BF16, the local contribution is added and the
    result is rounded again. ``single``: one FP32 sum over all contributing ranks
    (local included) in rank order, one rounding.
    """
    if rounding not in ("two_step", "single"):
        raise ValueError("rounding must be two_step or single")
    outputs = []
    for source in range(plan.world_size):
        tokens = plan.token_counts[source]
        remote = torch.zeros((tokens, hidden_size), dtype=torch.float32)
        local = torch.zeros((tokens, hidden_size), dtype=torch.float32)
        for dest in range(plan.world_size):
            rows = plan.dest_rows[source][:, dest]
            sel = (rows >= 0).nonzero().flatten()
            if not sel.numel():
                continue
            values = partials_by_rank[dest][rows[sel]].to(torch.float32)
            if dest == source and rounding == "two_step":
                local[sel] = values
            else:
                remote[sel] = remote[sel] + values
        if rounding == "two_step":
            out = (remote.to(torch.bfloat16).to(torch.float32) + local).to(torch.bfloat16)
        else:
            out = remote.to(torch.bfloat16)
        outputs.append(out)
    return outputs


def identity_layer_oracle(x, ids, weights, expert_to_rank, rank: int, world_size: int,
                          rounding: str = "two_step"):
    """Output of dispatch -> identity-times-routing-weight expert -> combine for ONE rank's tokens,
    from that rank's own inputs alone (plain PyTorch FP32 on the tensors' device).

    The rows a token sends out come back scaled by the weights of the experts that live on the
    destination rank, so nothing of the other ranks' batches enters a rank's result: every
    destination's partial row is ``bf16(x * scale_r)`` with ``scale_r`` accumulated over the slots
    owned by rank ``r`` in slot order, and the combine adds them in rank order with the
    library's rounding points (see :func:`combine_oracle`). Benchmarks use it to check every step's
    output bit for bit without a group-wide route plan.
    """
    if rounding not in ("two_step", "single"):
        raise ValueError("rounding must be two_step or single")
    device = x.device
    owner = torch.as_tensor(_as_owner_list(expert_to_rank, world_size), dtype=torch.int64, device=device)
    ids = ids.to(torch.int64)
    active = ids >= 0
    dest = torch.where(active, owner[ids.clamp(min=0)], torch.full_like(ids, -1))
    w = torch.where(active, weights.to(torch.float32), torch.zeros_like(weights, dtype=torch.float32))
    xf = x.to(torch.float32)
    remote = torch.zeros_like(xf)
    local = torch.zeros_like(xf)
    for r in range(world_size):
        here = dest == r
        scale = torch.zeros(x.shape[0], dtype=torch.float32, device=device)
        for k in range(ids.shape[1]):
            scale = torch.where(here[:, k], scale + w[:, k], scale)
        partial = (xf * scale[:, None]).to(torch.bfloat16).to(torch.float32)
        partial = torch.where(here.any(dim=1)[:, None], partial, torch.zeros_like(partial))
        if r == rank and rounding == "two_step":
            local = partial
        else:
            remote = remote + partial
    if rounding == "two_step":
        return (remote.to(torch.bfloat16).to(torch.float32) + local).to(torch.bfloat16)
    return remote.to(torch.bfloat16)


def direct_weighted_sum(x_by_rank, ids_by_rank, weights_by_rank, factors_by_expert=None):
    """What a dense MoE with identity-times-factor experts computes, in FP64."""
    outputs = []
    for x, ids, weights in zip(x_by_rank, ids_by_rank, weights_by_rank):
        ids = torch.as_tensor(ids).to(torch.int64)
        w = torch.as_tensor(weights).to(torch.float64)
        if not x.shape[0]:
            outputs.append(x.to(torch.float64))
            continue
        ids, w = ids.reshape(x.shape[0], -1), w.reshape(x.shape[0], -1)
        active = ids >= 0
        factor = torch.ones_like(w) if factors_by_expert is None else factors_by_expert.to(torch.float64)[ids.clamp(min=0)]
        scale = torch.where(active, w * factor, torch.zeros_like(w)).sum(dim=1)
        outputs.append(x.to(torch.float64) * scale[:, None])
    return outputs
