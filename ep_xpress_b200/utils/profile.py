"""Opt-in operation profile: per-CTA records written by profiling specialisations of the kernels.

Nothing is recorded unless a profile was started: ordinary launches run kernel
specialisations that contain no timers at all (the kernels are templates on a
profiling flag, like the reference's ``template<bool Profile>`` kernels,
ep_xpress/csrc/host_sm.cu:85-92). ``start`` preallocates ``int64 [operations, ctas, 24]``
device records under a 64 MiB budget; every eager dispatch/combine takes one slice;
``finish`` does ONE device-to-host copy and one synchronisation. This is the contract
of the reference's operation profile (ep_xpress/host_sm.py:654-807: bounded capture,
dropped-operation count, labels, single readback fence).

One record per CTA (times in ns on the GPU's global timer):

* words 0..7: phase stamps. Dispatch: start, routed, barrier, counts_in, payload_done,
  signalled, padded, done. Combine: start, published (sequential protocol: this CTA's rows are
  out; mailbox protocol: its first pusher is done), peers_ready (sequential: every peer has
  signalled; mailbox: pushers and reducers have joined), reduced; words 4..7 hold pipeline
  cycle counts of the combine's first reduce pipeline instead.
* rows / bytes the CTA stored to other planes, (token, segment) items its reducers issued,
  poll iterations of its bounded waits, the times of its first publication to a peer and of
  the first peer word it saw, the rank's status and the last stamp it reached, the protocol
  it ran, and how long its pushers / its first producer waited.

The report derives DISJOINT per-CTA phases from consecutive stamps; by construction they sum
to the CTA's elapsed time, which :func:`check_invariants` verifies together with the
counter identities (the reference's invariants, tests/test_host_sm_native_cuda.py:276-301).
"""

from __future__ import annotations

import torch

_BUDGET_BYTES = 64 << 20
DISPATCH_PHASES = ("start", "routed", "barrier", "counts_in", "payload_done", "signalled", "padded", "done")
COMBINE_PHASES = ("start", "published", "peers_ready", "reduced")
# combine stamps 4..7 are cycle counts, not times: consumer wait/work, producer wait/work
COMBINE_CYCLES = ("consumer_wait_cycles", "consumer_work_cycles", "producer_wait_cycles", "producer_other_cycles")
# disjoint phases between consecutive stamps
DISPATCH_INTERVALS = ("route", "rank_barrier", "count_exchange", "payload", "signal", "padding", "receive_wait")
COMBINE_INTERVALS = {1: ("push", "signal_wait", "reduce"), 2: ("push", "signal_wait", "reduce"),
                     3: ("push_and_reduce_until_first_pusher_done", "push_and_reduce", "retire")}
COMBINE_PROTOCOLS = {1: "register", 2: "bulk", 3: "mailbox"}
WORDS = {"rows": 8, "bytes": 9, "items": 10, "polls": 11, "first_publish": 12, "first_receive": 13, "status": 14,
         "completion": 15, "mode": 16, "push_wait": 17, "arrival_wait": 18, "store_cycles": 19}


class OperationProfile:
    def __init__(self, context, max_operations=1024):
        if isinstance(max_operations, bool) or not isinstance(max_operations, int) or max_operations < 1:
            raise ValueError("max_operations must be a positive integer")
        self._context = context
        self.stamps = context._core.native.PROFILE_STAMPS
        self.max_ctas = context._core.max_ctas
        if max_operations * self.max_ctas * self.stamps * 8 > _BUDGET_BYTES:
            raise ValueError("the requested profile exceeds the 64 MiB budget; lower max_operations")
        self.max_operations = max_operations
        self.label = None
        self.dropped = 0
        self._records = []
        self._device = torch.zeros((max_operations, self.max_ctas, self.stamps), dtype=torch.int64,
                                   device=context.device)

    def slice_for(self, kind, operation, tag, tokens, capacity, ctas):
        """Counters for the next operation, or None when capturing or full."""
        if torch.cuda.is_current_stream_capturing():
            return None
        if len(self._records) >= self.max_operations:
            self.dropped += 1
            return None
        index = len(self._records)
        self._records.append({"kind": kind, "operation": operation, "tag": tag, "label": self.label,
                              "tokens": tokens, "capacity": capacity, "ctas": ctas})
        return self._device[index]

    def finish(self):
        host = torch.empty(self._device.shape, dtype=torch.int64).pin_memory()
        host.copy_(self._device, non_blocking=True)
        torch.cuda.current_stream(self._context.device).synchronize()
        operations = [summarize(record, host[index, :record["ctas"]]) for index, record in enumerate(self._records)]
        return {"schema": 3, "operations": operations, "dropped_operations": self.dropped,
                "max_operations": self.max_operations, "rank": self._context.rank}


def summarize(record, stamps):
    """Report of one operation from its ``[ctas, words]`` records (a CPU int64 tensor)."""
    kind = record["kind"]
    names = DISPATCH_PHASES if kind == "dispatch" else COMBINE_PHASES
    started = stamps[:, 0][stamps[:, 0] > 0]
    begin = int(started.min()) if started.numel() else 0
    phases = {}
    for column, name in enumerate(names):
        reached = stamps[:, column][stamps[:, column] > 0]
        if reached.numel():
            phases[name] = {"first_ns": int(reached.min()) - begin, "last_ns": int(reached.max()) - begin}
    entry = dict(record)
    if kind == "combine":
        entry["cycles"] = {name: float(stamps[:, 4 + i].double().mean()) for i, name in enumerate(COMBINE_CYCLES)}
        if stamps.shape[1] > WORDS["store_cycles"]:
            entry["cycles"]["consumer_store_cycles"] = float(stamps[:, WORDS["store_cycles"]].double().mean())
    entry["phases"] = phases
    entry["elapsed_ns"] = max((p["last_ns"] for p in phases.values()), default=0)
    wide = stamps.shape[1] > WORDS["arrival_wait"]
    if not wide:
        return entry
    mode = int(stamps[:, WORDS["mode"]].max()) if stamps.shape[0] else 0
    last = len(names) - 1
    complete = (stamps[:, WORDS["completion"]] == last) & (stamps[:, 0] > 0)
    done = stamps[complete]
    if kind == "dispatch":
        intervals = DISPATCH_INTERVALS
        entry["protocol"] = {1: "register", 2: "bulk"}.get(mode, "unknown")
    else:
        intervals = COMBINE_INTERVALS.get(mode, COMBINE_INTERVALS[1])
        entry["protocol"] = COMBINE_PROTOCOLS.get(mode, "unknown")
    per_cta = {}
    if done.shape[0]:
        # A stamp that a CTA's role never wrote (e.g. a mailbox CTA whose pusher found no row)
        # inherits the previous one, so its interval is empty and the sum stays exact.
        filled = done[:, :len(names)].clone()
        for column in range(1, len(names)):
            missing = filled[:, column] == 0
            filled[missing, column] = filled[missing, column - 1]
            behind = filled[:, column] < filled[:, column - 1]        # concurrent roles: clamp to monotone
            filled[behind, column] = filled[behind, column - 1]
        for index, name in enumerate(intervals):
            per_cta[name] = (filled[:, index + 1] - filled[:, index]).tolist()
        entry["cta_elapsed_ns"] = (filled[:, last] - filled[:, 0]).tolist()
    entry["cta_phase_ns"] = per_cta
    entry["complete_ctas"] = int(done.shape[0])
    for name in ("rows", "bytes", "items", "polls", "push_wait", "arrival_wait"):
        entry[name] = int(stamps[:, WORDS[name]].sum())
    for name in ("first_publish", "first_receive"):
        seen = stamps[:, WORDS[name]][stamps[:, WORDS[name]] > 0]
        entry[name + "_ns"] = int(seen.min()) - begin if seen.numel() else None
    entry["status"] = int(stamps[:, WORDS["status"]].max()) if stamps.shape[0] else 0
    entry["completion_phase"] = names[int(stamps[:, WORDS["completion"]].min())] if stamps.shape[0] else None
    return entry


def check_invariants(entry, *, row_bytes=None):
    """Raise ``AssertionError`` unless one operation's report is self-consistent: every CTA reached
    the last phase, its disjoint phases are non-negative and sum to its elapsed time, milestones lie
    inside the operation, and the byte count is the row count times the row size."""
    assert entry["status"] == 0, entry["status"]
    assert entry["complete_ctas"] == entry["ctas"], (entry["complete_ctas"], entry["ctas"])
    assert entry["completion_phase"] == (DISPATCH_PHASES if entry["kind"] == "dispatch" else COMBINE_PHASES)[-1]
    phases = entry["cta_phase_ns"]
    for cta, elapsed in enumerate(entry["cta_elapsed_ns"]):
        parts = [phases[name][cta] for name in phases]
        assert all(part >= 0 for part in parts), parts
        assert sum(parts) == elapsed, (parts, elapsed)
        assert 0 < elapsed <= entry["elapsed_ns"]
    for name in ("first_publish_ns", "first_receive_ns"):
        if entry[name] is not None:
            assert 0 <= entry[name] <= entry["elapsed_ns"], (name, entry[name], entry["elapsed_ns"])
    assert entry["rows"] >= 0 and entry["polls"] >= 0
    if row_bytes is not None:
        assert entry["bytes"] == entry["rows"] * row_bytes, (entry["bytes"], entry["rows"], row_bytes)
