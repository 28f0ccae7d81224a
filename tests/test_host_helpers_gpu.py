"""Native helpers of the host-staged transport on a GPU: exact combine arithmetic (the
intermediate rounding is observable), index bounds reported through a status word, and the
registered-range check of the device-to-host copy (technique of the reference's
tests/test_native_cuda.py:57-110)."""

import ctypes

import pytest
import torch

from conftest import gpu_count

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(gpu_count() < 1, reason="needs a CUDA device")]


def test_add_partial_and_finish_combine_are_exact(native):
    stream = torch.cuda.current_stream().cuda_stream
    tokens, hidden = 5, 64
    remote = torch.zeros((tokens, hidden), dtype=torch.float32, device="cuda")
    local = torch.zeros((tokens, hidden), dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    first = torch.full((2, hidden), 2.0 ** -8, dtype=torch.bfloat16, device="cuda")
    second = torch.full((2, hidden), 2.0 ** -16, dtype=torch.bfloat16, device="cuda")
    mine = torch.ones((1, hidden), dtype=torch.bfloat16, device="cuda")
    native.add_partial(remote, first, torch.tensor([3, 1], device="cuda"), status, stream)
    native.add_partial(remote, second, torch.tensor([1, 4], device="cuda"), status, stream)
    native.add_partial(local, mine, torch.tensor([1], device="cuda"), status, stream)
    out = torch.empty((tokens, hidden), dtype=torch.bfloat16, device="cuda")
    native.finish_combine(remote, local, out, False, stream)
    single = torch.empty_like(out)
    native.finish_combine(remote + local, local, single, True, stream)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    two_step = ((torch.tensor(2.0 ** -8) + torch.tensor(2.0 ** -16)).to(torch.bfloat16).float() + 1.0).to(torch.bfloat16)
    one_step = torch.tensor(1.0 + 2.0 ** -8 + 2.0 ** -16).to(torch.bfloat16)
    assert two_step.item() != one_step.item()                  # the rounding point matters for these values
    assert (out[1].cpu() == two_step).all() and (single[1].cpu() == one_step).all()
    assert (out[3].float().cpu() == 2.0 ** -8).all() and (out[0] == 0).all() and (out[2] == 0).all()
    native.add_partial(remote, first, torch.tensor([0, 9], device="cuda"), status, stream)   # 9 is outside
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert torch.ones(2, device="cuda").sum().item() == 2      # reported, not trapped


def test_device_to_host_copy_needs_a_registered_destination(native):
    stream = torch.cuda.current_stream().cuda_stream
    source = torch.arange(256, dtype=torch.int32, device="cuda")
    buffer = (ctypes.c_char * 8192)()
    base = (ctypes.addressof(buffer) + 4095) // 4096 * 4096     # a page-aligned kilobyte inside it
    before = native.registered_host_ranges()
    native.register_host(base, 2048)
    try:
        with pytest.raises(ValueError):
            native.register_host(base + 1024, 2048)             # overlaps
        native.copy_d2h_async(source, base + 512, stream)
        torch.cuda.synchronize()
        landed = (ctypes.c_int32 * 256).from_address(base + 512)
        assert list(landed) == list(range(256))
        with pytest.raises(IndexError):
            native.copy_d2h_async(source, base + 1536, stream)  # the last 512 bytes would lie outside
        with pytest.raises(IndexError):
            native.copy_d2h_async(source, ctypes.addressof(buffer) + 6000, stream)
    finally:
        native.unregister_host(base)
    assert native.registered_host_ranges() == before
