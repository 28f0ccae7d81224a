"""Opt-in operation profile: device-timed dispatch/combine records.

Zero cost when off (nothing is recorded unless a profile was started). While a
profile runs every eager operation is bracketed by CUDA events on its own
stream; ``finish`` performs ONE synchronisation and returns plain records.
This keeps the reference's user-visible contract (bounded capture,
``max_operations``, labels, a single readback fence; ep_xpress/host_sm.py:654-807)
with event timestamps in place of per-CTA counters.
"""

from __future__ import annotations

import torch

_MAX_OPERATIONS = 1 << 16


class OperationProfile:
    def __init__(self, context, max_operations=1024):
        if isinstance(max_operations, bool) or not isinstance(max_operations, int) or \
                not 1 <= max_operations <= _MAX_OPERATIONS:
            raise ValueError(f"max_operations must be an integer in [1, {_MAX_OPERATIONS}]")
        self._context = context
        self.max_operations = max_operations
        self.label = None
        self.dropped = 0
        self._records = []
        self._open = None

    def record(self, kind, handle, tag, stream):
        """Called right AFTER an operation was enqueued on ``stream``."""
        if torch.cuda.is_current_stream_capturing():
            return
        if len(self._records) >= self.max_operations:
            self.dropped += 1
            return
        end = torch.cuda.Event(enable_timing=True)
        end.record(stream)
        self._records.append({"kind": kind, "operation": handle.operation, "tag": tag, "label": self.label,
                              "tokens": handle.local_token_count, "capacity": handle.received_count,
                              "end": end, "stream": stream})

    def mark(self, stream):
        start = torch.cuda.Event(enable_timing=True)
        start.record(stream)
        return start

    def finish(self):
        if self._records:
            self._records[-1]["end"].synchronize()
        first = self._records[0]["end"] if self._records else None
        out = []
        for record in self._records:
            entry = {k: v for k, v in record.items() if k not in ("end", "stream")}
            entry["completed_ms_after_first"] = first.elapsed_time(record["end"]) if record["end"] is not first else 0.0
            out.append(entry)
        return {"schema": 1, "operations": out, "dropped_operations": self.dropped,
                "max_operations": self.max_operations}
