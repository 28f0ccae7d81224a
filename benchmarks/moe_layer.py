"""Full MoE layer: dispatch -> tcgen05 grouped SwiGLU experts -> combine (the reference measures
this level only inside a serving framework, docs/model-performance.md of the reference).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29503 -m benchmarks.moe_layer --tokens 128 4096 [--baseline]

DeepSeek-V3-shaped layer: hidden 7168, 256 routed experts in contiguous blocks, top-8,
per-expert W1/W3 [7168 x 2048] and W2 [2048 x 7168] BF16 drawn from N(0, 0.02), sigmoid
routing weights normalised to 1. Reports device-timed per-phase medians (max over ranks)
and the experts' achieved FLOP/s against the measured cuBLAS BF16 peak of this pool
(MEASURED_PEAKS.json when present, else the stated fallback). ``--baseline`` adds the
configuration an application would run without this library: two all_to_all_single calls
and a per-expert loop of library GEMMs.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ep_xpress_b200 import Config, Context, get_nccl_comm_handle  # noqa: E402
from ep_xpress_b200.models import SwiGLUMoELayer  # noqa: E402
from ep_xpress_b200.parallel.baseline_nccl import NCCLAllToAllBaseline  # noqa: E402
from ep_xpress_b200.utils import workloads  # noqa: E402


def measured_peak_tflops():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as handle:
            return float(json.load(handle)["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 1400.0, "fallback"


def max_over_ranks(values, world):
    t = torch.tensor(values, dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.cpu().tolist()


def library_experts(rows, meta, w13, w2, topk, owner_base):
    """Baseline runner: per local expert, cuBLAS GEMMs through torch.matmul."""
    ids, weights = meta[:, :topk].to(torch.int64) - owner_base, meta[:, topk:]
    experts, inter = w13.shape[0], w13.shape[1] // 2
    out = torch.zeros(rows.shape, dtype=torch.float32, device=rows.device)
    for e in range(experts):
        hit = (ids == e)
        sel = hit.any(dim=1).nonzero().flatten()
        if not sel.numel():
            continue
        x = rows[sel]
        gu = x @ w13[e].T
        act = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
        y = (act @ w2[e].T).to(torch.float32) * (weights[sel] * hit[sel]).sum(dim=1, keepdim=True)
        out[sel] += y
    return out.to(torch.bfloat16)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--tokens", type=int, nargs="+", default=[128, 4096])
    parser.add_argument("--hidden", type=int, default=7168)
    parser.add_argument("--inter", type=int, default=2048)
    parser.add_argument("--experts", type=int, default=256)
    parser.add_argument("--topk", type=int, default=8)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--samples", type=int, default=10)
    parser.add_argument("--baseline", action="store_true")
    parser.add_argument("--single-cta", action="store_true", help="128-row tiles on single CTAs instead of CTA pairs")
    parser.add_argument("--report", default=None)
    args = parser.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29578")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    local_experts = args.experts // world
    emap = workloads.contiguous_expert_map(args.experts, world)
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    w13 = (torch.randn((local_experts, 2 * args.inter, args.hidden), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    w2 = (torch.randn((local_experts, args.hidden, args.inter), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    peak, peak_source = measured_peak_tflops()
    results = []
    for tokens in args.tokens:
        cfg = Config(hidden_size=args.hidden, topk=args.topk, max_tokens_per_rank=tokens, timeout_seconds=30.0,
                     slots=1)
        ep = Context(get_nccl_comm_handle(dist.group.WORLD), emap, cfg)
        pairs = int(tokens * args.topk * 1.5) + 1024
        layer = SwiGLUMoELayer(ep, w13, w2, max_local_pairs=pairs, pair_ctas=not args.single_cta)
        batches = []
        for step in range(4):
            ids, w = workloads.uniform_routing(tokens, args.experts, args.topk, seed=step, rank=rank, weights="sigmoid")
            batches.append((workloads.gaussian_payload(tokens, args.hidden, seed=step, rank=rank).cuda(), ids.cuda(), w.cuda()))
        timing = []
        for step in range(args.warmup + args.samples):
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            layer(*batches[step % 4], timing=timing if step >= args.warmup else None)
        torch.cuda.synchronize()
        layer.experts.check()
        ep.check()
        phases = {}
        for name, (a, b) in {"dispatch": (0, 1), "experts": (1, 2), "combine": (2, 3), "layer": (0, 3)}.items():
            phases[name] = statistics.median(max_over_ranks([m[a].elapsed_time(m[b]) * 1e3 for m in timing], world))
        sorted_rows = float(layer.experts.counters[1].item())           # tile-padded rows the GEMMs walked
        # Useful work only: (token, slot) pairs whose expert lives on this rank, mean over the batches.
        owner = torch.tensor(emap, device="cuda")
        mine = torch.stack([torch.bincount(owner[ids].flatten(), minlength=world) for _, ids, _ in batches]).sum(0)
        if world > 1:
            dist.all_reduce(mine)
        local_pairs = float(mine[rank].item()) / len(batches)
        flops = local_pairs * 3 * 2 * args.hidden * args.inter
        entry = {"tokens_per_rank": tokens, "phase_us_p50": phases, "sorted_rows_rank0": sorted_rows,
                 "local_pairs_rank0": local_pairs,
                 "expert_tflops": flops / (phases["experts"] * 1e-6) / 1e12,
                 "expert_fraction_of_" + peak_source + "_peak": flops / (phases["experts"] * 1e-6) / 1e12 / peak}
        if args.baseline:
            baseline = NCCLAllToAllBaseline(emap, world)
            samples = []
            for step in range(2 + args.samples):
                x, ids, w = batches[step % 4]
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                rows, meta, route = baseline.dispatch(x, ids, w)
                baseline.combine(library_experts(rows, meta, w13, w2, args.topk, rank * local_experts), route)
                b.record()
                torch.cuda.synchronize()
                if step >= 2:
                    samples.append(a.elapsed_time(b) * 1e3)
            entry["baseline_nccl_library_gemm_layer_us_p50"] = statistics.median(max_over_ranks(samples, world))
        results.append(entry)
        ep.close()
        del layer
        torch.cuda.empty_cache()
    if rank == 0:
        report = {"schema": 1, "world_size": world, "hidden": args.hidden, "inter": args.inter, "experts": args.experts,
                  "topk": args.topk, "cta_pairs": not args.single_cta, "peak_tflops": peak, "peak_source": peak_source, "results": results}
        text = json.dumps(report, indent=1)
        print(text)
        if args.report:
            with open(args.report, "w") as handle:
                handle.write(text)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
