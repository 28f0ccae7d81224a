"""Grouped SwiGLU expert runner on tcgen05 tensor cores (see csrc/moe_gemm_sm100.cu).

The runner consumes exactly what ``dispatch`` returns - padded ``hidden``,
``local_ids``, ``weights`` and the DEVICE ``valid_count`` - and produces the
rank's already-weighted BF16 partial rows that ``combine`` expects. Nothing is
read back to the host: the number of rows per expert only exists on the GPU.
It replaces the reference adapter's count-aware Triton helpers plus the
framework's Triton GEMM (ep_xpress/adapters/sglang_valid.py:13-255) with
hand-written kernels.

Weights are K-major ("[out_features, in_features]" like ``nn.Linear``):
``w13`` is ``[experts, 2 * inter, hidden]`` with the gate projection in rows
``[0, inter)`` and the up projection in ``[inter, 2 * inter)``; ``w2`` is
``[experts, hidden, inter]``.
"""

from __future__ import annotations

import torch

from .. import native as _native_loader


class GroupedSwiGLU:
    def __init__(self, w13, w2, *, max_rows, topk, max_local_pairs=None, pair_ctas=False, gather_loads=False):
        """``max_local_pairs`` bounds the (row, slot) pairs whose expert lives on this rank.

        ``gather_loads=True``: the first GEMM's TMA producer gathers the activation rows of every
        expert tile straight from the dispatch batch (``tile::gather4``, four rows per copy), so
        no gather launch and no expert-sorted copy of the activations exist. Bit-identical, but
        opt-in: a 128-row operand tile then takes 32 copies of 512 bytes per k-step instead of
        one 16 KB box, and the copy engine's issue rate, not the tensor pipe, bounds the GEMM
        (measured at hidden 7168 / inter 2048, 2 GPUs, 4096 tokens per rank: 7.4 ms against
        3.7 ms with the gather kernel, whose cost is 0.15 ms).


        The default is the worst case (every slot of every row is local). A tighter,
        CPU-known bound saves workspace; exceeding it is reported by :meth:`check`,
        never silently truncated into the output.
        """
        if w13.dim() != 3 or w2.dim() != 3 or w13.dtype != torch.bfloat16 or w2.dtype != torch.bfloat16:
            raise ValueError("w13 and w2 must be BF16 [experts, ., .] tensors")
        experts, two_inter, hidden = w13.shape
        inter = two_inter // 2
        if w2.shape != (experts, hidden, inter) or two_inter % 2:
            raise ValueError("w13 must be [experts, 2 * inter, hidden] and w2 [experts, hidden, inter]")
        if hidden % 256 or inter % 128:
            raise ValueError("hidden must be a multiple of 256 and inter a multiple of 128")
        self.native = _native_loader.load()
        self.w13, self.w2 = w13.contiguous(), w2.contiguous()
        self.experts, self.hidden, self.inter, self.topk, self.max_rows = experts, hidden, inter, topk, max_rows
        self.pair_ctas = bool(pair_ctas)        # GEMMs on clusters of two CTAs (256-row tiles)
        tile = self.native.MOE_TILE_ROWS * (2 if self.pair_ctas else 1)
        worst_rows, _ = self.native.moe_sizes(max_rows, topk, experts, tile)
        if max_local_pairs is None:
            sorted_rows = worst_rows
        else:
            sorted_rows = min(worst_rows, (-(-max_local_pairs // tile) + experts) * tile)
        device = w13.device
        self.sorted_rows = sorted_rows
        self.sorted_row = torch.empty(sorted_rows, dtype=torch.int32, device=device)
        self.sorted_scale = torch.empty(sorted_rows, dtype=torch.float32, device=device)
        self.entry_pos = torch.empty(max_rows * topk, dtype=torch.int32, device=device)
        self.tile_expert = torch.zeros(sorted_rows // tile, dtype=torch.int32, device=device)
        self.counters = torch.zeros(2, dtype=torch.int32, device=device)
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=device)
        self.gather_loads = bool(gather_loads)
        self.sorted_x = None if self.gather_loads else torch.empty((sorted_rows, hidden), dtype=torch.bfloat16,
                                                                   device=device)
        self.act = torch.empty((sorted_rows, inter), dtype=torch.bfloat16, device=device)
        self.y = torch.empty((sorted_rows, hidden), dtype=torch.bfloat16, device=device)
        self.kernel_launches_per_forward = 5 if self.gather_loads else 6

    def forward(self, hidden, local_ids, weights, valid_count, out=None, stream=None):
        rows = hidden.shape[0]
        if rows > self.max_rows:
            raise ValueError("more rows than the runner was created for")
        if out is None:
            out = torch.empty((rows, self.hidden), dtype=torch.bfloat16, device=hidden.device)
        stream = stream or torch.cuda.current_stream(hidden.device)
        if self.gather_loads and (rows == 0 or hidden.data_ptr() % 16):
            raise ValueError("gathered loads need a non-empty, 16-byte aligned activation matrix")
        self.native.moe_forward(hidden, local_ids, weights, valid_count, self.w13, self.w2, out, self.sorted_row,
                                self.sorted_scale, self.entry_pos, self.tile_expert, self.counters, self.error_flag,
                                self.sorted_x, self.act, self.y, stream.cuda_stream, self.pair_ctas)
        return out

    __call__ = forward

    def check(self):
        """Synchronises and raises if a kernel reported a problem."""
        code = int(self.error_flag.item())
        if code == 2:
            raise RuntimeError("more local (row, slot) pairs than max_local_pairs allows; results are incomplete")
        if code:
            raise RuntimeError("the grouped GEMM gave up on a bounded wait")


def swiglu_reference(hidden, local_ids, weights, valid, w13, w2):
    """Plain PyTorch FP32 statement of the runner (same rounding points), for tests."""
    rows, topk = local_ids.shape
    inter = w13.shape[1] // 2
    out = torch.zeros((rows, hidden.shape[1]), dtype=torch.float32, device=hidden.device)
    x = hidden.to(torch.float32)
    for k in range(topk):
        ids = local_ids[:, k]
        for e in ids.unique().tolist():
            if e < 0:
                continue
            sel = ((ids == e) & (torch.arange(rows, device=ids.device) < valid)).nonzero().flatten()
            if not sel.numel():
                continue
            w = w13[e].to(torch.float32)
            gate, up = x[sel] @ w[:inter].T, x[sel] @ w[inter:].T
            act = (torch.nn.functional.silu(gate) * up).to(torch.bfloat16).to(torch.float32)
            y = (act @ w2[e].to(torch.float32).T) * weights[sel, k][:, None]
            out[sel] += y.to(torch.bfloat16).to(torch.float32)
    return out.to(torch.bfloat16)
