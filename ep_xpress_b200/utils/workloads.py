"""Synthetic router outputs and payloads used by tests and benchmarks.

Behavioural re-creations of the reference's generators: the seven replay route
cases with position-marker payloads (benchmarks/replay.py:19-64), the rotating
communication-benchmark patterns (benchmarks/communication.py:137-150), plus
the DeepSeek-V3-shaped and Zipf-skewed routings the benchmark configs name.
All generators are deterministic in (seed, rank).
"""

from __future__ import annotations

import torch

REPLAY_CASES = ("mixed", "empty", "local", "hotspot", "all_empty", "padding", "all_padding")


def contiguous_expert_map(num_experts: int, world_size: int):
    """Experts in equal contiguous blocks: expert e lives on rank e // (E / W)."""
    if num_experts % world_size:
        raise ValueError("experts must divide evenly across ranks")
    per_rank = num_experts // world_size
    return [e // per_rank for e in range(num_experts)]


def round_robin_expert_map(num_experts: int, world_size: int):
    return [e % world_size for e in range(num_experts)]


def _generator(seed, rank):
    g = torch.Generator()
    g.manual_seed(int(seed) * 1000003 + int(rank) * 7919 + 17)
    return g


def uniform_routing(tokens, num_experts, topk, *, seed=0, rank=0, weights="softmax"):
    """ids uniform without replacement per token; weights softmax or normalised sigmoid."""
    g = _generator(seed, rank)
    scores = torch.rand((tokens, num_experts), generator=g)
    ids = scores.topk(topk, dim=1).indices.to(torch.int64) if tokens else torch.zeros((0, topk), dtype=torch.int64)
    logits = torch.randn((tokens, topk), generator=g)
    if weights == "softmax":
        w = torch.softmax(logits, dim=1)
    elif weights == "sigmoid":
        s = torch.sigmoid(logits)
        w = s / s.sum(dim=1, keepdim=True)
    else:
        raise ValueError("weights must be softmax or sigmoid")
    return ids, w.to(torch.float32)


def zipf_routing(tokens, num_experts, topk, *, exponent=1.2, seed=0, rank=0):
    """Expert popularity ~ Zipf(exponent) under a per-seed permutation, sampled without replacement."""
    g = _generator(seed, rank)
    perm_g = torch.Generator()
    perm_g.manual_seed(int(seed) * 977 + 5)
    popularity = 1.0 / torch.arange(1, num_experts + 1, dtype=torch.float64) ** exponent
    popularity = popularity[torch.randperm(num_experts, generator=perm_g)]
    if tokens == 0:
        return torch.zeros((0, topk), dtype=torch.int64), torch.zeros((0, topk))
    ids = torch.multinomial(popularity.expand(tokens, -1), topk, replacement=False, generator=g)
    logits = torch.randn((tokens, topk), generator=g)
    return ids.to(torch.int64), torch.softmax(logits, dim=1).to(torch.float32)


def gaussian_payload(tokens, hidden, *, seed=0, rank=0):
    g = _generator(seed + 101, rank)
    return torch.randn((tokens, hidden), generator=g).to(torch.bfloat16)


def marker_payload(tokens, hidden, *, rank, iteration=0):
    """Background pattern plus exact BF16 marker columns (rank, token digits, iteration).

    A row delivered to the wrong place cannot pass a bitwise comparison.
    """
    cols = torch.arange(hidden, dtype=torch.float32)
    background = ((cols + 7 * rank) % 29) / 128.0
    x = background.repeat(tokens, 1)
    if hidden >= 8 and tokens:
        t = torch.arange(tokens, dtype=torch.float32)
        x[:, 0] = float(rank)
        x[:, 1] = t % 128
        x[:, 2] = (t // 128) % 128
        x[:, 3] = (t // 16384) % 128
        x[:, 4] = float(iteration % 128)
    return x.to(torch.bfloat16)


def replay_case(case, *, rank, world_size, tokens, topk=4, experts_per_rank=4, iteration=0):
    """Router output of one rank for one of the seven validation route cases."""
    if case not in REPLAY_CASES:
        raise ValueError(f"unknown case {case!r}")
    num_experts = world_size * experts_per_rank
    count = tokens
    if case == "empty":
        count = 0 if rank == world_size - 1 else max(tokens - rank, 0)
    if case == "all_empty":
        count = 0
    ids = torch.full((count, topk), -1, dtype=torch.int64)
    base = torch.tensor([0.5, 0.25, 0.125, 0.125] + [0.0] * max(0, topk - 4))[:topk]
    weights = base.repeat(count, 1).to(torch.float32)
    for t in range(count):
        for slot in range(topk):
            if case == "local":
                owner = rank
            elif case == "hotspot":
                owner = 0
            else:
                owner = (rank + t + slot // 2 + iteration) % world_size
            ids[t, slot] = owner * experts_per_rank + (slot % experts_per_rank)
    if case in ("padding", "all_padding") and count:
        for t in range(count):
            if case == "all_padding" or t % 3 == 0:
                ids[t, :] = -1
                weights[t, :] = float("nan")
            elif t % 3 == 1:
                ids[t, -1] = -1
                weights[t, -1] = float("inf")
    return ids, weights, num_experts


def communication_pattern(step, *, rank, world_size, tokens, num_experts, topk):
    """Rotating patterns: random, hotspot with full dedup, a third of the tokens dropped."""
    g = torch.Generator()
    g.manual_seed(7100 + rank * 37 + step)
    if tokens == 0:
        return torch.zeros((0, topk), dtype=torch.int64), torch.zeros((0, topk))
    ids = torch.stack([torch.randperm(num_experts, generator=g)[:topk] for _ in range(tokens)]).to(torch.int64)
    if step % 4 == 1:
        target = step % world_size
        owned = [e for e in range(num_experts) if e * world_size // num_experts == target][:topk]
        ids[:] = torch.tensor((owned * topk)[:topk])
    elif step % 4 == 2:
        ids[::3] = -1
    weights = torch.full((tokens, topk), 1.0 / topk)
    return ids, weights
