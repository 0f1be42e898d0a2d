"""The spawn helper itself: failures surface with every rank's message, are never retried,
and can be written to a file."""

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


def test_a_failure_is_not_repeated_and_is_written_to_a_file(tmp_path, monkeypatch):
    marker = str(tmp_path / "marker")
    out = tmp_path / "failures"
    monkeypatch.setenv("FLASHOPTIM_B200_TEST_FAILURE_DIR", str(out))
    # a second attempt would find the marker and pass: the first failure must stand
    with pytest.raises(AssertionError, match="first attempt fails on rank 0"):
        run_distributed(_fails_until_marker_exists, world_size=2, backend="gloo", args=(marker,))
    files = list(out.iterdir())
    assert len(files) == 1 and "first attempt fails on rank 0" in files[0].read_text()
