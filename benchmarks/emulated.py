"""Whole-group protocol on ONE GPU: every rank inside single cooperative launches.

    python -m benchmarks.emulated --world 4 --tokens 1024 --hidden 7168 --iterations 5

Peer pointers resolve to the same device, so no NVLink is involved: this measures the
kernels' instruction and local-memory behaviour (and is what `ncu` can capture, since a
multi-rank command must never run under it). Prints device-timed medians per phase.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ep_xpress_b200 import Config, EmulatedGroup  # noqa: E402
from ep_xpress_b200.utils import workloads  # noqa: E402


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--world", type=int, default=4)
    parser.add_argument("--tokens", type=int, default=1024)
    parser.add_argument("--hidden", type=int, default=7168)
    parser.add_argument("--experts", type=int, default=256)
    parser.add_argument("--topk", type=int, default=8)
    parser.add_argument("--iterations", type=int, default=5)
    args = parser.parse_args()
    cfg = Config(hidden_size=args.hidden, topk=args.topk, max_tokens_per_rank=args.tokens, timeout_seconds=10.0,
                 slots=1, workspace_pool_bytes=1 << 20)
    emap = workloads.contiguous_expert_map(args.experts, args.world)
    with EmulatedGroup(args.world, emap, cfg) as group:
        slot = group.create_slot()
        dev = group.device
        batches = []
        for step in range(2):
            xs, ids, ws = [], [], []
            for rank in range(args.world):
                i, w = workloads.uniform_routing(args.tokens, args.experts, args.topk, seed=step, rank=rank,
                                                 weights="sigmoid")
                xs.append(workloads.gaussian_payload(args.tokens, args.hidden, seed=step, rank=rank).to(dev))
                ids.append(i.to(dev))
                ws.append(w.to(dev))
            batches.append((xs, ids, ws))
        times = {"dispatch": [], "expert": [], "combine": []}
        for step in range(args.iterations + 2):
            xs, ids, ws = batches[step % 2]
            marks = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            marks[0].record()
            out = group.dispatch(slot, xs, ids, ws)
            marks[1].record()
            partials = [group.scale_rows(batch) for batch in out]
            marks[2].record()
            group.combine(slot, partials, [args.tokens] * args.world)
            marks[3].record()
            torch.cuda.synchronize()
            if step >= 2:
                for name, (a, b) in {"dispatch": (0, 1), "expert": (1, 2), "combine": (2, 3)}.items():
                    times[name].append(marks[a].elapsed_time(marks[b]) * 1e3)
        assert all(status[0] == 0 for status in group.status())
        print(json.dumps({"world": args.world, "tokens_per_rank": args.tokens, "hidden": args.hidden,
                          "phase_us_p50": {k: statistics.median(v) for k, v in times.items()}}))


if __name__ == "__main__":
    main()
