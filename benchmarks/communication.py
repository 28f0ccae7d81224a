"""Communication-only sweep: dispatch and combine latency per MoE layer.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 -m benchmarks.communication --tokens 1 8 64 512 4096 --shape qwen3 --routing zipf

Method (the reference's, benchmarks/communication.py:137-276, applied to the NVLink
transport): the layer (dispatch, synthetic expert, combine) is captured ONCE as a CUDA graph
on a retained workspace and replayed; ``--warmup`` untimed then ``--samples`` timed replays;
route patterns rotate between samples (random, hotspot with full dedup, a third of the
tokens dropped, or uniform / Zipf-skewed); per sample the MAXIMUM over ranks is taken, and
the report gives median / p95 / min / max over samples. Phase times are DEVICE times from the
library's sample ring (earliest CTA start to latest CTA end of the replayed kernel; the layer
is first dispatch CTA to last combine CTA): timing a phase's own graph from the host with
events measures launch latency and the skew of the ranks' hosts - tens of microseconds -
instead of the kernel (``layer_host_us`` keeps that figure for comparison). Payload volume is counted
logically: a (token, remote rank) pair moves ``2 * hidden`` bytes per phase. The roofline
fraction compares the p50 with the time those bytes need over one direction of the rank's
NVLink at the measured peer-copy bandwidth (770 GB/s, 900 nominal).

``--nccl-reference`` also times the two-``all_to_all_single`` baseline
(``ep_xpress_b200.parallel.baseline_nccl``) eagerly on the same inputs.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ep_xpress_b200 import Config, Context, get_nccl_comm_handle  # noqa: E402
from ep_xpress_b200.ops import scale_rows  # noqa: E402
from ep_xpress_b200.parallel.baseline_nccl import NCCLAllToAllBaseline  # noqa: E402
from ep_xpress_b200.utils import workloads  # noqa: E402

SHAPES = {"v3": dict(hidden=7168, experts=256, topk=8), "qwen3": dict(hidden=2048, experts=128, topk=8)}
LINK_GBS_MEASURED = 770.0


def parse_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--shape", choices=sorted(SHAPES), default="v3")
    parser.add_argument("--tokens", type=int, nargs="+", default=[128, 4096])
    parser.add_argument("--routing", choices=("patterns", "uniform", "zipf"), default="uniform")
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--samples", type=int, default=20)
    parser.add_argument("--nccl-reference", action="store_true")
    parser.add_argument("--combine-streaming", choices=("auto", "on", "off"), default="auto")
    parser.add_argument("--items-per-cta", type=int, default=None, help="launch-width policy (see set_tuning)")
    parser.add_argument("--max-ctas", type=int, default=None, help="cap on CTAs per operation")
    parser.add_argument("--report", default=None, help="write the JSON report here (rank 0)")
    return parser.parse_args()


def routes_for(step, routing, rank, world, tokens, shape):
    experts, topk = shape["experts"], shape["topk"]
    if routing == "patterns":
        return workloads.communication_pattern(step, rank=rank, world_size=world, tokens=tokens, num_experts=experts,
                                               topk=topk)
    if routing == "zipf":
        return workloads.zipf_routing(tokens, experts, topk, seed=step, rank=rank)
    return workloads.uniform_routing(tokens, experts, topk, seed=step, rank=rank, weights="sigmoid")


def logical_bytes(ids, owner, rank, hidden):
    """Bytes this rank sends per phase: one row per (token, remote destination rank)."""
    active = ids >= 0
    dest = owner[ids.clamp(min=0)]
    hit = torch.zeros((ids.shape[0], int(owner.max()) + 1), dtype=torch.int32)
    hit.scatter_add_(1, dest, active.to(torch.int32))
    hit = hit > 0
    hit[:, rank] = False
    return int(hit.sum()) * hidden * 2


def summarize(samples):
    ordered = sorted(samples)
    return {"p50": statistics.median(ordered), "p95": ordered[min(len(ordered) - 1, int(0.95 * len(ordered)))],
            "min": ordered[0], "max": ordered[-1]}


def max_over_ranks(values, world):
    t = torch.tensor(values, dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.cpu().tolist()


def run_tokens(ep, args, shape, tokens, rank, world, owner):
    hidden, topk = shape["hidden"], shape["topk"]
    capacity = world * tokens
    workspace = ep.create_workspace(capacity, tokens)
    stream = torch.cuda.Stream()
    static = [torch.zeros((tokens, hidden), dtype=torch.bfloat16, device="cuda"),
              torch.zeros((tokens, topk), dtype=torch.int64, device="cuda"),
              torch.zeros((tokens, topk), dtype=torch.float32, device="cuda")]
    patterns = 8
    inputs, volumes = [], []
    for step in range(patterns):
        ids, w = routes_for(step, args.routing, rank, world, tokens, shape)
        x = workloads.gaussian_payload(tokens, hidden, seed=step, rank=rank)
        inputs.append(tuple(t.cuda() for t in (x, ids, w)))
        volumes.append(logical_bytes(ids, owner, rank, hidden))

    def load(step):
        for dst, src in zip(static, inputs[step % patterns]):
            dst.copy_(src, non_blocking=True)

    state = {}

    def do_dispatch():
        state["batch"] = ep.dispatch_on_stream(*static, stream=stream, workspace=workspace)

    def do_expert():
        state["partial"] = scale_rows(ep, state["batch"], stream=stream)

    def do_combine():
        state["out"] = ep.combine_on_stream(state["partial"], state["batch"].handle, stream=stream)

    def layer():
        do_dispatch(); do_expert(); do_combine()

    with torch.cuda.stream(stream):                      # eager warm-up of the workspace
        load(0)
        layer()
    stream.synchronize()
    ep.prepare_decode_profile(max_samples_per_channel=args.warmup + args.samples, stage="layer")
    ep.prepare_graph_capture()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        layer()
    ep.start_decode_profile()
    host_layer = []
    for step in range(args.warmup + args.samples):
        with torch.cuda.stream(stream):
            load(step)
            ep.prepare_graph_replay(stream)
            stream.synchronize()
            if world > 1:
                dist.barrier()
            marks = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            marks[0].record(stream)
            graph.replay()
            marks[1].record(stream)
        stream.synchronize()
        if step >= args.warmup:
            host_layer.append(marks[0].elapsed_time(marks[1]) * 1e3)
    ring = ep.stop_decode_profile()["stages"]
    first = args.warmup
    dispatch, combine = ring["dispatch"], ring["combine"]
    assert dispatch["samples"] == combine["samples"] == args.warmup + args.samples and not dispatch["dropped_samples"]
    samples = {"dispatch": [ns / 1e3 for ns in dispatch["elapsed_ns"][first:]],
               "combine": [ns / 1e3 for ns in combine["elapsed_ns"][first:]],
               "layer": [(cb + ce - db) / 1e3 for db, cb, ce in zip(dispatch["begin_ns"][first:], combine["begin_ns"][first:],
                                                                   combine["elapsed_ns"][first:])],
               "layer_host": host_layer}
    ep.check()
    result = {"tokens_per_rank": tokens, "capacity": capacity, "ctas": state["batch"].handle._plan.ctas,
              "combine_ctas": state["batch"].handle._plan.combine_ctas}
    for name, values in samples.items():
        result[name + "_us"] = summarize(max_over_ranks(values, world))
    mean_bytes = sum(volumes) / len(volumes)
    worst = max_over_ranks([mean_bytes], world)[0]
    link_us = worst / (LINK_GBS_MEASURED * 1e3)
    result["remote_bytes_per_rank_per_phase"] = worst
    result["link_bound_us_per_phase"] = link_us
    for name in ("dispatch", "combine"):
        p50 = result[name + "_us"]["p50"]
        result[name + "_roofline_fraction_of_measured"] = (link_us / p50) if p50 and world > 1 else None
        result[name + "_logical_gbs_per_rank"] = worst / p50 / 1e3 if p50 else None
    if args.nccl_reference:
        baseline = NCCLAllToAllBaseline(owner.tolist(), world)
        timings = []
        for step in range(3 + args.samples):
            x, ids, w = inputs[step % patterns]
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            rows, _, route = baseline.dispatch(x, ids, w)
            baseline.combine(rows, route)
            b.record()
            torch.cuda.synchronize()
            if step >= 3:
                timings.append(a.elapsed_time(b) * 1e3)
        result["nccl_all_to_all_layer_us"] = summarize(max_over_ranks(timings, world))
    ep.release_workspace(workspace)
    return result


def main():
    args = parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    shape = SHAPES[args.shape]
    emap = workloads.contiguous_expert_map(shape["experts"], world)
    owner = torch.tensor(emap)
    cfg = Config(hidden_size=shape["hidden"], topk=shape["topk"], max_tokens_per_rank=max(args.tokens),
                 timeout_seconds=30.0, slots=1,
                 combine_streaming=args.combine_streaming,
                 workspace_pool_bytes=2 * Config(hidden_size=shape["hidden"], topk=shape["topk"],
                                                 max_tokens_per_rank=max(args.tokens)).nvlink_slot_bytes(world))
    ep = Context(get_nccl_comm_handle(dist.group.WORLD), emap, cfg)
    ep.enable_cuda_graph()
    if args.items_per_cta is not None or args.max_ctas is not None:
        ep.set_tuning(items_per_cta=args.items_per_cta, max_ctas=args.max_ctas)
    report = {"schema": 2, "world_size": world, "shape": args.shape, **shape, "routing": args.routing,
              "combine_streaming": args.combine_streaming, "warmup": args.warmup, "samples": args.samples, "timing": "device sample ring per phase (layer_host_us: CUDA events around the replay), max over ranks per sample",
              "link_gbs_measured": LINK_GBS_MEASURED, "results": []}
    for tokens in args.tokens:
        report["results"].append(run_tokens(ep, args, shape, tokens, rank, world, owner))
    ep.close()
    if rank == 0:
        text = json.dumps(report, indent=1)
        print(text)
        if args.report:
            with open(args.report, "w") as handle:
                handle.write(text)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
