"""tcgen05 grouped SwiGLU runner against a plain PyTorch FP32 statement of the same op."""

import pytest
import torch

from conftest import gpu_count

from ep_xpress_b200.ops import GroupedSwiGLU, swiglu_reference

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(gpu_count() < 1, reason="needs a CUDA device")]


def make_case(rows, topk, experts, hidden, inter, valid, seed, local_fraction=0.6):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = (torch.randn((rows, hidden), generator=g) * 0.5).to(torch.bfloat16)
    ids = torch.full((rows, topk), -1, dtype=torch.int64)
    for r in range(rows):
        chosen = torch.randperm(experts, generator=g)[:min(topk, experts)]
        keep = torch.rand(len(chosen), generator=g) < local_fraction
        ids[r, :len(chosen)] = torch.where(keep, chosen, torch.full_like(chosen, -1))
    weights = torch.rand((rows, topk), generator=g).to(torch.float32)
    w13 = (torch.randn((experts, 2 * inter, hidden), generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn((experts, hidden, inter), generator=g) * 0.05).to(torch.bfloat16)
    count = torch.tensor([valid], dtype=torch.int32)
    return [t.cuda() for t in (x, ids, weights, count, w13, w2)]


def assert_elementwise_close(got, want):
    """Every element within 2 % of the reference, plus an absolute allowance of one BF16 step of a
    value four times the tensor's typical magnitude: a row is a sum of per-slot results that are
    rounded to BF16 one by one, a slot result is often several times larger than the sum it
    cancels into, and a different FP32 accumulation order may flip one of those roundings."""
    got, want = got.float(), want.float()
    if not want.numel():
        return
    step = float(want.pow(2).mean().sqrt()) * 2.0 ** -5
    torch.testing.assert_close(got, want, rtol=2e-2, atol=max(step, 1e-6))


@pytest.mark.parametrize("gather_loads", [True, False])
@pytest.mark.parametrize("rows,topk,experts,hidden,inter,valid", [
    (64, 2, 2, 256, 128, 64),
    (300, 4, 3, 512, 256, 257),
    (1000, 8, 8, 1024, 384, 1000),
    (130, 8, 32, 256, 128, 0),
    (5, 2, 2, 256, 128, 3),
])
def test_matches_fp32_reference(rows, topk, experts, hidden, inter, valid, gather_loads):
    x, ids, weights, count, w13, w2 = make_case(rows, topk, experts, hidden, inter, valid, seed=rows)
    runner = GroupedSwiGLU(w13, w2, max_rows=rows, topk=topk, gather_loads=gather_loads)
    out = torch.full((rows, hidden), 7.0, dtype=torch.bfloat16, device="cuda")
    runner(x, ids, weights, count, out=out)
    runner.check()
    want = swiglu_reference(x, ids, weights, valid, w13, w2)
    assert_elementwise_close(out[:valid], want[:valid])
    assert (out[valid:] == 7.0).all()          # rows at or above valid_count are not touched
    again = torch.empty_like(out)
    runner(x, ids, weights, count, out=again)  # order of pairs inside an expert never changes a result
    assert torch.equal(again[:valid], out[:valid])


@pytest.mark.parametrize("pair_ctas", [False, True])
def test_benchmarked_shape_matches_fp32_reference(pair_ctas):
    """Hidden 7168, intermediate 2048 (112 k-steps, 16 and 28 column tiles): the shape of the layer
    benchmark, on a few experts and a few hundred rows, both kernels, gathered and pre-gathered
    activations bit-identical to each other."""
    rows, topk, experts, hidden, inter, valid = 520, 8, 4, 7168, 2048, 500
    x, ids, weights, count, w13, w2 = make_case(rows, topk, experts, hidden, inter, valid, seed=11, local_fraction=0.4)
    outs = []
    for gather_loads in (True, False):
        runner = GroupedSwiGLU(w13, w2, max_rows=rows, topk=topk, pair_ctas=pair_ctas, gather_loads=gather_loads)
        out = torch.full((rows, hidden), 7.0, dtype=torch.bfloat16, device="cuda")
        runner(x, ids, weights, count, out=out)
        runner.check()
        outs.append(out)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    want = swiglu_reference(x, ids, weights, valid, w13, w2)
    assert_elementwise_close(outs[0][:valid], want[:valid])
    assert (outs[0][valid:] == 7.0).all()


@pytest.mark.parametrize("rows,topk,experts,hidden,inter,valid", [
    (64, 2, 2, 256, 128, 64),
    (700, 4, 3, 512, 256, 650),
    (1000, 8, 8, 1024, 384, 1000),
])
def test_cta_pairs_match_fp32_reference_and_single_cta_path(rows, topk, experts, hidden, inter, valid):
    """tcgen05 cta_group::2 on clusters of two CTAs (256-row tiles) against the same oracle."""
    x, ids, weights, count, w13, w2 = make_case(rows, topk, experts, hidden, inter, valid, seed=rows + 1)
    pair = GroupedSwiGLU(w13, w2, max_rows=rows, topk=topk, pair_ctas=True)
    out = torch.full((rows, hidden), 7.0, dtype=torch.bfloat16, device="cuda")
    pair(x, ids, weights, count, out=out)
    pair.check()
    want = swiglu_reference(x, ids, weights, valid, w13, w2)
    assert_elementwise_close(out[:valid], want[:valid])
    assert (out[valid:] == 7.0).all()
    single = GroupedSwiGLU(w13, w2, max_rows=rows, topk=topk)
    other = torch.empty_like(out)
    single(x, ids, weights, count, out=other)
    assert torch.equal(other[:valid], out[:valid])     # same accumulation order per output row


def test_pair_bound_overflow_is_reported():
    x, ids, weights, count, w13, w2 = make_case(512, 4, 2, 256, 128, 512, seed=3, local_fraction=1.0)
    runner = GroupedSwiGLU(w13, w2, max_rows=512, topk=4, max_local_pairs=128)
    runner(x, ids, weights, count)
    with pytest.raises(RuntimeError, match="max_local_pairs"):
        runner.check()
