"""Host-side segment table: chunk prefix and its cache (no GPU needed)."""

import numpy as np
import torch

from flashoptim_b200.ops.step import SegmentTable


def _rows(numels):
    rows = np.zeros((len(numels), 8), dtype=np.int64)
    rows[:, 7] = numels
    return rows


def test_chunk_prefix_counts_ceil_per_segment():
    cb = SegmentTable.chunk_prefix(np.array([1, 2048, 2049, 0, 8192]), 2048)
    assert cb.tolist() == [0, 1, 2, 4, 4, 8]


def test_prefix_is_rebuilt_when_the_chunk_size_changes():
    table = SegmentTable(torch.device("cpu"))
    rows = _rows([10000, 5])
    *_, total_small, on_dev = table.prepare(rows, chunk=2048)
    assert (total_small, on_dev) == (6, 0)
    # same lengths, other kernel family (larger chunk): the cached prefix must not be reused
    *_, total_large, _ = table.prepare(rows, chunk=8192)
    assert total_large == 3
    *_, total_again, _ = table.prepare(rows, chunk=2048)
    assert total_again == 6
