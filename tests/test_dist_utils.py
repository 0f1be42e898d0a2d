"""The spawn helper itself: failures surface with every rank's message, and the optional
second attempt reports the first failure as a warning instead of hiding it."""

import os

import pytest

from dist_utils import run_distributed


def _fails_until_marker_exists(rank, world, marker):
    if rank == 0 and not os.path.exists(marker):
        open(marker, "w").close()
        return ["first attempt fails on rank 0"]
    return []


def _always_fails(rank, world):
    return [f"rank {rank} is unhappy"]


def _raises(rank, world):
    if rank == 1:
        raise RuntimeError("boom on rank 1")
    return []


def test_failure_carries_every_ranks_message():
    with pytest.raises(AssertionError) as e:
        run_distributed(_always_fails, world_size=2, backend="gloo")
    assert "rank 0 is unhappy" in str(e.value) and "rank 1 is unhappy" in str(e.value)
    with pytest.raises(AssertionError, match="boom on rank 1"):
        run_distributed(_raises, world_size=2, backend="gloo")


def test_second_attempt_warns_about_the_first_failure(tmp_path):
    marker = str(tmp_path / "marker")
    with pytest.warns(UserWarning, match="first attempt fails on rank 0"):
        run_distributed(_fails_until_marker_exists, world_size=2, backend="gloo", args=(marker,), retries=1)
    os.remove(marker)
    with pytest.raises(AssertionError):  # CPU runs are not repeated by default
        run_distributed(_fails_until_marker_exists, world_size=2, backend="gloo", args=(marker,))
