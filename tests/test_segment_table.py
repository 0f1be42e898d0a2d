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


def test_pack_rows_refuses_tensors_of_the_wrong_extent():
    import pytest

    from flashoptim_b200.optim._common import pack_rows
    from flashoptim_b200.optim.state import MaybeQuantizedTensor

    def state(n_codes, n_scales):
        s = MaybeQuantizedTensor(torch.zeros(1), try_quantize=False)
        s._data, s._quantized, s._scales = None, torch.zeros(n_codes, dtype=torch.int8), torch.zeros(
            n_scales, dtype=torch.float16)
        return s

    p = torch.zeros(100, dtype=torch.bfloat16)
    g = torch.zeros(100, dtype=torch.bfloat16)
    good = {"exp_avg": state(100, 4), "error_bits": torch.zeros(100, dtype=torch.int8)}
    rows = pack_rows([(p, g, good)], ("exp_avg",))
    assert rows[0, 7] == 100 and rows[0, 0] == p.data_ptr() and rows[0, 4] == good["exp_avg"].scales.data_ptr()
    assert pack_rows([(p, 4096, good)], ("exp_avg",))[0, 1] == 4096  # byte offset instead of a tensor
    for bad in (
        {"exp_avg": state(100, 3), "error_bits": good["error_bits"]},      # one scale short
        {"exp_avg": state(96, 4), "error_bits": good["error_bits"]},       # codes of another tensor
        {"exp_avg": good["exp_avg"], "error_bits": torch.zeros(50, dtype=torch.int8)},
    ):
        with pytest.raises(ValueError):
            pack_rows([(p, g, bad)], ("exp_avg",))
    with pytest.raises(ValueError):
        pack_rows([(p, torch.zeros(99, dtype=torch.bfloat16), good)], ("exp_avg",))
    with pytest.raises(ValueError):
        pack_rows([(p, torch.zeros(100), good)], ("exp_avg",))  # fp32 gradient for a bf16 parameter
    full = MaybeQuantizedTensor(torch.zeros(100), try_quantize=False, storage_dtype=torch.bfloat16)
    assert pack_rows([(p, g, {"exp_avg": full})], ("exp_avg",))[0, 3] == full.data.data_ptr()
    short = MaybeQuantizedTensor(torch.zeros(10), try_quantize=False, storage_dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        pack_rows([(p, g, {"exp_avg": short})], ("exp_avg",))


def test_every_optimizer_packs_a_consistent_table(monkeypatch):
    """The packing that feeds the CUDA kernels, run here on CPU tensors with the launch
    replaced by a recorder: one row per parameter, every address and length filled in, for
    every optimizer x dtype x master-weight width x state mode."""
    import warnings

    import torch.nn as nn

    import flashoptim_b200.optim.adam as adam_mod
    import flashoptim_b200.optim.lion as lion_mod
    import flashoptim_b200.optim.sgd as sgd_mod
    from flashoptim_b200 import FlashAdamW, FlashLion, FlashSGD, FlashSGDW

    seen = []

    def record(table, rows, dtype, err, mode_or_quantized, hyper):
        seen.append((rows.copy(), dtype, err, mode_or_quantized))

    monkeypatch.setattr(adam_mod, "launch_adam", record)
    monkeypatch.setattr(lion_mod, "launch_momentum", record)
    monkeypatch.setattr(sgd_mod, "launch_momentum", record)
    cases = [(FlashAdamW, {}, 2), (FlashLion, {}, 1), (FlashSGDW, {"momentum": 0.9}, 1), (FlashSGD, {}, 0)]
    for cls, kw, n_states in cases:
        for dtype, mwb in ((torch.bfloat16, 24), (torch.float16, 32), (torch.bfloat16, None), (torch.float32, None)):
            for quantize in (True, False):
                params = [nn.Parameter(torch.randn(n).to(dtype)) for n in (1, 33, 4096)]
                with warnings.catch_warnings():
                    warnings.simplefilter("ignore")
                    opt = cls(params, lr=1e-3, master_weight_bits=mwb, quantize=quantize, **kw)
                group = opt.param_groups[0]
                items = []
                for p in params:
                    opt._ensure_state_initialized(p, group)
                    items.append((p.data, torch.zeros_like(p.data), opt.state[p]))
                seen.clear()
                opt._pre_step_many([it[2] for it in items])
                opt._fused_step(items, group, 0)
                rows = np.concatenate([s[0] for s in seen])
                assert rows.shape == (3, 8) and sorted(rows[:, 7]) == [1, 33, 4096]
                err = {24: 1, 32: 2, None: 0}[mwb]
                assert all(s[2] == err for s in seen)
                assert (rows[:, 0] != 0).all() and (rows[:, 1] != 0).all()
                assert ((rows[:, 2] != 0) == (err != 0)).all()
                for k in range(2):
                    has_state = k < n_states
                    assert ((rows[:, 3 + 2 * k] != 0) == has_state).all()
                    assert ((rows[:, 4 + 2 * k] != 0) == (has_state and quantize)).all()
