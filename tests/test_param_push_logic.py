"""Host-side bookkeeping of the all-gather on write (no GPU, no process group): when may
FSDP2's all-gather be replaced by a flag wait, and what sends it back to NCCL."""

from types import SimpleNamespace

import torch

from flashoptim_b200.parallel.fsdp import PushedAllGather
from flashoptim_b200.parallel.symm import ParamPush, PeerGradients


def _gather(n_params=3):
    params = [SimpleNamespace(sharded_param=torch.zeros(8, dtype=torch.bfloat16)) for _ in range(n_params)]
    rs = SimpleNamespace(dtype=torch.bfloat16, input_numel=2 * 8 * n_params, supported=False, fsdp_params=params)
    return PushedAllGather(SimpleNamespace(), rs), params


def test_not_current_until_a_push_and_after_invalidate():
    g, _ = _gather()
    assert not g.is_current()
    g.mark_pushed()
    assert g.is_current()
    g.invalidate()
    assert not g.is_current()


def test_in_place_change_of_a_shard_is_noticed():
    g, params = _gather()
    g.mark_pushed()
    params[1].sharded_param.add_(1)  # e.g. a checkpoint load or an fp32 import
    assert not g.is_current()
    g.mark_pushed()
    assert g.is_current()
    params[2].sharded_param.copy_(torch.ones(8))
    assert not g.is_current()


def test_reads_do_not_invalidate():
    g, params = _gather()
    g.mark_pushed()
    _ = params[0].sharded_param.float().sum() + params[0].sharded_param.view(-1)[0]
    assert g.is_current()


def test_unsupported_group_allocates_ordinary_memory():
    g, _ = _gather()
    assert g.target is None
    out = g.allocate((48,), dtype=torch.bfloat16, device=torch.device("cpu"))
    assert out.shape == (48,) and out.dtype == torch.bfloat16


def test_push_epoch_counts_launches_and_fills_the_kernel_arguments():
    from flashoptim_b200.ops import native

    class FakeGroup:
        world, rank = 2, 1

        def comm_args(self, buf, epoch, ready, done, grad_out=None, grad_out_sub=0):
            a = native.FoCommArgs()
            a.world, a.rank, a.epoch = self.world, self.rank, epoch
            return a

    buf = SimpleNamespace(ptrs=[4096, 8192], multicast_ptr=0)
    push = ParamPush(buf, channel=7, delta=64)
    pg = PeerGradients(FakeGroup(), buf, 0, 1)
    a = pg.next_args()
    assert a.push == 0  # nothing asked for
    pg.push = push
    a = pg.next_args()
    b = pg.next_args()
    assert (a.push, a.push_epoch, b.push_epoch, push.epoch) == (1, 1, 2, 2)
    assert (a.epoch, b.epoch) == (2, 3)
    assert [a.param_out[0], a.param_out[1]] == [4096, 8192] and not a.param_out_mc
    assert a.param_out_delta == 64 and a.pushed_channel == 7


def test_groups_with_an_empty_shard_on_some_rank_are_left_to_nccl():
    from flashoptim_b200.parallel.fsdp import _every_rank_has_rows

    assert _every_rank_has_rows(torch.zeros(16, 4), 8)
    assert _every_rank_has_rows(torch.zeros(9, 4), 8) is False   # chunks of 2: ranks 5..7 hold nothing
    assert _every_rank_has_rows(torch.zeros(15, 4), 8)           # last rank holds one row
    assert _every_rank_has_rows(torch.zeros(3), 4) is False      # chunks of 1: rank 3 is empty
    assert _every_rank_has_rows(torch.zeros(4), 4)
    assert _every_rank_has_rows(torch.zeros(1), 1)


def test_push_budget_takes_groups_in_order_while_they_fit():
    from flashoptim_b200.parallel.fsdp import select_push_groups

    assert select_push_groups([10, 0, 20, 30], None) == [True, False, True, True]
    assert select_push_groups([10, 20, 30, 5], 35) == [True, True, False, True]
    assert select_push_groups([10, 20], 0) == [False, False]


def test_poll_status_reports_a_timeout_one_call_late_without_waiting():
    import pytest

    from flashoptim_b200.parallel.symm import CommTimeoutError, PeerGroup

    peers = PeerGroup(device=torch.device("cpu"))   # one rank, host tensors: no symmetric memory needed
    peers.poll_status()
    peers.poll_status()                              # nothing recorded: stays quiet
    peers.status[0], peers.status[1] = 1 << 3, 2     # what a kernel writes when rank 1 never shows up
    peers.poll_status()                              # still the older copy
    with pytest.raises(CommTimeoutError, match="missing rank 1"):
        peers.poll_status()
    assert int(peers.status[0]) == 0                 # cleared for the next use
    peers.poll_status()
    peers.poll_status()


def test_oversized_groups_are_the_ones_far_above_the_median():
    from flashoptim_b200.parallel.fsdp import oversized_mask

    layer = 218_103_808 * 2
    assert oversized_mask([5 * layer] + [layer] * 32) == [True] + [False] * 32   # Llama-3-8B: embedding + head
    assert oversized_mask([layer] * 4) == [False] * 4
    assert oversized_mask([256, 2080, 32896, 33280]) == [False] * 4              # nothing beyond twice the median
    assert oversized_mask([7]) == [False]


def test_tuned_options_by_world_size_and_memory_grant():
    from flashoptim_b200.parallel import tuned_options

    two = tuned_options(2, 16 << 30)
    assert two["staged"] and not two["use_multicast"] and two["max_ctas"] == 0
    assert two["own_all_gather"] and two["all_gather_copy_engine"] and "push_params" not in two
    four, eight = tuned_options(4), tuned_options(8)
    assert four["use_multicast"] and four["max_ctas"] == 64 and eight["max_ctas"] == 48 and not eight["staged"]
    granted = tuned_options(8, 16 << 30, push_budget_bytes=32 << 30)
    assert granted["push_params"] and "own_all_gather" not in granted
    assert "push_params" not in tuned_options(8, 140 << 30, push_budget_bytes=32 << 30)  # does not fit the grant
