"""The allocation-free C entry point of the expert runner against the regular entry point.

Some users of this library cannot allocate device memory where they run the experts
(a serving loop that must not call cudaMalloc, a plugin that only receives raw pointers,
a plain C program). They call ``epx_moe_forward_noalloc`` through its exported C symbol;
its workspace is a fixed array inside the library. This file calls the symbol exactly that
way (ctypes, raw pointers) twice in a row with different problems, so the second call runs
on a workspace that still holds the first call's data, and checks both outputs against
``GroupedSwiGLU`` (caller-allocated workspace).

Collected last on purpose: a run that stops at the first failure has then already run
every other test.
"""

import ctypes

import pytest
import torch

from conftest import gpu_count

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(gpu_count() < 1, reason="needs a CUDA device")]


def library():
    from ep_xpress_b200 import native
    native.load()                                   # libtorch first, then the library itself
    lib = ctypes.CDLL(str(native.library_path()))
    lib.epx_moe_forward_noalloc.restype = ctypes.c_int
    lib.epx_moe_forward_noalloc.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 5 + [ctypes.c_void_p,
                                                                                       ctypes.POINTER(ctypes.c_int)]
    lib.epx_moe_noalloc_scratch_bytes.restype = ctypes.c_ulonglong
    lib.epx_moe_noalloc_last_status.restype = ctypes.c_int
    lib.epx_moe_noalloc_last_status.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int),
                                                ctypes.POINTER(ctypes.c_int)]
    return lib


def problem(rows, topk, experts, hidden, inter, valid, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((rows, hidden), generator=g) * 0.5).to(torch.bfloat16)
    ids = torch.randint(-1, experts, (rows, topk), generator=g)
    for r in range(rows):                            # an expert appears at most once per row
        seen = set()
        for k in range(topk):
            e = int(ids[r, k])
            if e in seen:
                ids[r, k] = -1
            seen.add(e)
    weights = torch.rand((rows, topk), generator=g)
    w13 = (torch.randn((experts, 2 * inter, hidden), generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn((experts, hidden, inter), generator=g) * 0.05).to(torch.bfloat16)
    count = torch.tensor([valid], dtype=torch.int32)
    return [t.cuda() for t in (x, ids, weights, count, w13, w2)]


def call_noalloc(lib, x, ids, weights, count, w13, w2):
    rows, hidden = x.shape
    out = torch.full((rows, hidden), -3.0, dtype=torch.bfloat16, device="cuda")
    cuda_error = ctypes.c_int(0)
    stream = torch.cuda.current_stream().cuda_stream
    code = lib.epx_moe_forward_noalloc(x.data_ptr(), ids.data_ptr(), weights.data_ptr(), count.data_ptr(),
                                       w13.data_ptr(), w2.data_ptr(), out.data_ptr(), rows, ids.shape[1],
                                       w13.shape[0], hidden, w13.shape[1] // 2, stream, ctypes.byref(cuda_error))
    assert code == 0, (code, cuda_error.value)
    status = ctypes.c_int(-1)
    assert lib.epx_moe_noalloc_last_status(stream, ctypes.byref(status), ctypes.byref(cuda_error)) == 0
    assert status.value == 0, "a kernel of the allocation-free call reported a problem"
    torch.cuda.synchronize()
    return out


def test_noalloc_entry_matches_regular_entry_on_two_calls_in_a_row():
    from ep_xpress_b200.ops import GroupedSwiGLU, swiglu_reference
    lib = library()
    assert 0 < lib.epx_moe_noalloc_scratch_bytes() < 8 << 20
    cases = [(150, 4, 3, 512, 256, 150, 11), (90, 2, 2, 256, 128, 61, 12)]
    for rows, topk, experts, hidden, inter, valid, seed in cases:
        x, ids, weights, count, w13, w2 = problem(rows, topk, experts, hidden, inter, valid, seed)
        got = call_noalloc(lib, x, ids, weights, count, w13, w2)
        runner = GroupedSwiGLU(w13, w2, max_rows=rows, topk=topk, pair_ctas=False, gather_loads=False)
        want = torch.full_like(got, -3.0)
        runner(x, ids, weights, count, out=want)
        runner.check()
        # Both entry points run the same kernels in the same order: the outputs are bit-identical,
        # rows at or above valid_count (left at -3) included.
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        reference = swiglu_reference(x, ids, weights, valid, w13, w2)
        torch.testing.assert_close(got[:valid].float(), reference[:valid].float(), rtol=2e-2, atol=2e-2)


def test_noalloc_entry_rejects_problems_beyond_its_fixed_workspace():
    lib = library()
    x, ids, weights, count, w13, w2 = problem(64, 2, 2, 256, 128, 64, 5)
    cuda_error = ctypes.c_int(0)
    args = (x.data_ptr(), ids.data_ptr(), weights.data_ptr(), count.data_ptr(), w13.data_ptr(), w2.data_ptr(),
            x.data_ptr())
    too_many_rows = lib.epx_moe_forward_noalloc(*args, 100000, 2, 2, 256, 128, None, ctypes.byref(cuda_error))
    too_wide = lib.epx_moe_forward_noalloc(*args, 64, 2, 2, 2048, 128, None, ctypes.byref(cuda_error))
    bad_shape = lib.epx_moe_forward_noalloc(*args, 64, 2, 2, 250, 128, None, ctypes.byref(cuda_error))
    assert (too_many_rows, too_wide, bad_shape) == (2, 2, 1)


def test_noalloc_entry_rejects_misaligned_pointers_on_the_host():
    """Rows move as 16-byte vectors: a pointer that is off by two bytes must come back as a bad
    argument from the host-side check (nothing is launched), not as a fault on the GPU."""
    lib = library()
    x, ids, weights, count, w13, w2 = problem(64, 2, 2, 256, 128, 64, 6)
    out = torch.empty((65, 256), dtype=torch.bfloat16, device="cuda")
    spare = torch.empty((65, 256), dtype=torch.bfloat16, device="cuda")
    cuda_error = ctypes.c_int(0)
    good = [x.data_ptr(), ids.data_ptr(), weights.data_ptr(), count.data_ptr(), w13.data_ptr(), w2.data_ptr(),
            out.data_ptr()]
    for index, skew in ((0, spare.data_ptr() + 2), (6, out.data_ptr() + 2), (1, ids.data_ptr() + 4),
                        (2, weights.data_ptr() + 2)):
        args = list(good)
        args[index] = skew
        code = lib.epx_moe_forward_noalloc(*args, 64, 2, 2, 256, 128, None, ctypes.byref(cuda_error))
        assert code == 1, (index, code)
    torch.cuda.synchronize()
