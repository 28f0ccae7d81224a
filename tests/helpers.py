"""Shared oracle checks for the device transport tests."""

import torch

from ep_xpress_b200.utils import routing


def check_dispatch(batches, plan, xs, capacities, *, zero_padding=True):
    expected_hidden = routing.dispatch_oracle(xs, plan)
    for rank, (batch, routes) in enumerate(zip(batches, plan.received)):
        valid = int(batch.valid_count.cpu().item())
        assert valid == routes.rows, f"rank {rank}: valid_count {valid} != {routes.rows}"
        assert batch.hidden.shape[0] == capacities[rank]
        assert torch.equal(batch.hidden[:valid].cpu().view(torch.int16), expected_hidden[rank].view(torch.int16)), \
            f"rank {rank}: hidden rows differ"
        assert torch.equal(batch.local_ids[:valid].cpu(), routes.local_ids), f"rank {rank}: local ids differ"
        assert torch.equal(batch.weights[:valid].cpu(), routes.weights), f"rank {rank}: weights differ"
        assert torch.equal(batch.inverse[:valid].cpu(), routes.inverse), f"rank {rank}: inverse differs"
        assert (batch.local_ids[valid:].cpu() == -1).all(), f"rank {rank}: padding ids"
        assert (batch.weights[valid:].cpu() == 0).all(), f"rank {rank}: padding weights"
        assert (batch.inverse[valid:].cpu() == -1).all(), f"rank {rank}: padding inverse"
        if zero_padding:
            assert (batch.hidden[valid:].cpu().view(torch.int16) == 0).all(), f"rank {rank}: padding rows"


def expected_partials(plan, xs, factors_by_rank=None):
    hidden = routing.dispatch_oracle(xs, plan)
    return [routing.scale_expert_oracle(hidden[r], plan.received[r].local_ids, plan.received[r].weights,
                                        None if factors_by_rank is None else factors_by_rank[r])
            for r in range(plan.world_size)]


def bits(tensor):
    return tensor.detach().cpu().contiguous().view(torch.int16)
