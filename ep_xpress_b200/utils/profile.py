"""Opt-in operation profile: per-CTA phase timestamps written by the kernels.

Nothing is recorded unless a profile was started (the kernels test one null
pointer per phase). ``start`` preallocates ``int64 [operations, ctas, 8]`` device
counters under a 64 MiB budget; every eager dispatch/combine takes one slice and
its thread 0 of each CTA stamps ``%globaltimer`` at the phase boundaries;
``finish`` does ONE device-to-host copy and one synchronisation. This is the
contract of the reference's operation profile (ep_xpress/host_sm.py:654-807:
bounded capture, dropped-operation count, labels, single readback fence) with a
compact stamp record in place of its 43 counters per CTA.

Stamps (ns on the GPU's global timer; 0 = not reached):
  dispatch: start, routed, barrier, counts_in, payload_done, signalled, padded, done
  combine:  start, published, peers_ready, reduced
"""

from __future__ import annotations

import torch

_BUDGET_BYTES = 64 << 20
DISPATCH_PHASES = ("start", "routed", "barrier", "counts_in", "payload_done", "signalled", "padded", "done")
COMBINE_PHASES = ("start", "published", "peers_ready", "reduced")
# combine stamps 4..7 are cycle counts, not times: consumer wait/work, producer wait/work
COMBINE_CYCLES = ("consumer_wait_cycles", "consumer_work_cycles", "producer_wait_cycles", "producer_other_cycles")


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
        operations = []
        for index, record in enumerate(self._records):
            stamps = host[index, :record["ctas"]]
            names = DISPATCH_PHASES if record["kind"] == "dispatch" else COMBINE_PHASES
            begin = int(stamps[:, 0][stamps[:, 0] > 0].min()) if (stamps[:, 0] > 0).any() else 0
            phases = {}
            for column, name in enumerate(names):
                reached = stamps[:, column][stamps[:, column] > 0]
                if reached.numel():
                    phases[name] = {"first_ns": int(reached.min()) - begin, "last_ns": int(reached.max()) - begin}
            entry = dict(record)
            if record["kind"] == "combine":
                entry["cycles"] = {name: float(stamps[:, 4 + i].double().mean()) for i, name in enumerate(COMBINE_CYCLES)}
            entry["phases"] = phases
            entry["elapsed_ns"] = max((p["last_ns"] for p in phases.values()), default=0)
            operations.append(entry)
        return {"schema": 2, "operations": operations, "dropped_operations": self.dropped,
                "max_operations": self.max_operations, "rank": self._context.rank}
