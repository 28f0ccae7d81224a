"""Peer-copy bandwidth between two GPUs of one node: the denominator of the link rooflines.

    python -m benchmarks.peer_copy --bytes 1073741824 --iterations 10

One process drives both devices. The copies are plain `cudaMemcpyPeerAsync` transfers (the
copy engines, no kernel reads a peer's memory), timed with CUDA events on the copying stream.
Prints one JSON line: GB/s for device 0 -> 1, 1 -> 0 and both directions at once (per
direction), next to the nominal 900 GB/s per direction of NVLink 5.
"""

from __future__ import annotations

import argparse
import json
import statistics

import torch


def timed_copy(dst, src, stream, iterations):
    times = []
    with torch.cuda.device(src.device), torch.cuda.stream(stream):
        for step in range(iterations + 3):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            dst.copy_(src, non_blocking=True)
            end.record(stream)
            end.synchronize()
            if step >= 3:
                times.append(begin.elapsed_time(end))
    return statistics.median(times)


def timed_pair(a_dst, a_src, b_dst, b_src, streams, iterations):
    """Both directions in flight together; the slower direction's time counts."""
    times = []
    for step in range(iterations + 3):
        marks = []
        for (dst, src), stream in zip(((a_dst, a_src), (b_dst, b_src)), streams):
            with torch.cuda.device(src.device), torch.cuda.stream(stream):
                begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                begin.record(stream)
                dst.copy_(src, non_blocking=True)
                end.record(stream)
                marks.append((begin, end))
        for _, end in marks:
            end.synchronize()
        if step >= 3:
            times.append(max(b.elapsed_time(e) for b, e in marks))
    return statistics.median(times)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--bytes", type=int, default=1 << 30)
    parser.add_argument("--iterations", type=int, default=10)
    args = parser.parse_args()
    if torch.cuda.device_count() < 2:
        print(json.dumps({"unavailable": "needs two CUDA devices"}))
        return
    d0, d1 = torch.device("cuda", 0), torch.device("cuda", 1)
    if not torch.cuda.can_device_access_peer(0, 1):
        print(json.dumps({"unavailable": "devices 0 and 1 have no peer access"}))
        return
    a0 = torch.empty(args.bytes, dtype=torch.uint8, device=d0).fill_(1)
    b0 = torch.empty(args.bytes, dtype=torch.uint8, device=d0)
    a1 = torch.empty(args.bytes, dtype=torch.uint8, device=d1).fill_(2)
    b1 = torch.empty(args.bytes, dtype=torch.uint8, device=d1)
    s0, s1 = torch.cuda.Stream(d0), torch.cuda.Stream(d1)
    torch.cuda.synchronize(d0)
    torch.cuda.synchronize(d1)
    forward = timed_copy(b1, a0, s0, args.iterations)
    backward = timed_copy(b0, a1, s1, args.iterations)
    both = timed_pair(b1, a0, b0, a1, (s0, s1), args.iterations)
    assert int(b1[-1]) == 1 and int(b0[-1]) == 2
    rate = lambda ms: args.bytes / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": "peer_copy_bandwidth", "unit": "GB/s", "bytes": args.bytes,
                      "device0_to_1": round(rate(forward), 1), "device1_to_0": round(rate(backward), 1),
                      "both_directions_each": round(rate(both), 1), "nominal_per_direction": 900.0,
                      "timing": "CUDA events on the copying stream, median of %d after 3 warm-ups" % args.iterations}))


if __name__ == "__main__":
    main()
