"""Expert-side operators that run between dispatch and combine."""

from __future__ import annotations

import torch


def scale_rows(context, batch, factors=None, out=None, stream=None):
    """Synthetic expert: ``out[row] = bf16(hidden[row] * sum_k w[row,k] * factors[local_ids[row,k]])``.

    Only slots with ``local_ids >= 0`` contribute and only rows below the
    device-side ``valid_count`` are written. ``out`` defaults to the partial plane
    of the batch's slot, which lets combine skip its copy into the heap. This is
    the validation expert of the reference (benchmarks/replay.py:67-71) as one
    fused kernel instead of a chain of tensor ops.
    """
    core = context._core
    if out is None:
        out = context.partial_buffer(batch.handle)
    stream = stream or torch.cuda.current_stream(context.device)
    core.scale_rows(batch.hidden, batch.local_ids, batch.weights, batch.valid_count, factors, out, stream)
    return out
