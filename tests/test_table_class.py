"""Host-side classification of threshold tables (what the writer is told about them): sorted
tables may be searched, tables with at most one positive 16-bit-exact threshold per interval of
2^-9 may be looked up by interval on large writes (the flag BKV_FLAG_BINNED_TABLES)."""

import torch

from beyond_kv_cache_b200 import synth
from beyond_kv_cache_b200.quant.beyond_cute import _table_class, _tables_binned, _tables_sorted, prepare_qpoints_and_thresholds


def test_synthetic_and_default_tables_are_sorted_and_binned():
    for per_group in (False, True):
        _, thr = synth.make_tables(8, seed=3, per_group=per_group)
        assert _table_class(thr) == (True, True)
        assert _table_class(thr.float()) == (True, True)  # float32 copies of 16-bit values
    _, default = prepare_qpoints_and_thresholds(num_bits=4, device=torch.device("cpu"), q_points=None)  # the fp16 default tables
    assert _table_class(default) == (True, True)


def test_tables_the_indexed_look_up_must_not_take():
    _, thr = synth.make_tables(2, seed=1)
    close = thr.clone()
    e = torch.floor(close[:, 6].float() * 512)
    close[:, 6] = ((e + 0.25) / 512).to(close.dtype)  # ascending, but two thresholds inside one interval
    close[:, 7] = ((e + 0.75) / 512).to(close.dtype)
    assert _tables_sorted(close) and not _tables_binned(close)
    negative = thr.clone()
    negative[:, 0] = -0.125
    assert _tables_sorted(negative) and not _tables_binned(negative)
    zero = thr.clone()
    zero[:, 0] = 0.0  # a NaN quotient must count no threshold
    assert not _tables_binned(zero)
    unsorted = thr.clone()
    unsorted[:, [3, 9]] = unsorted[:, [9, 3]]
    assert _table_class(unsorted) == (False, False)
    fine = thr.float()
    fine[:, 5] = torch.nextafter(fine[:, 5], torch.tensor(2.0))  # one float32 step above a 16-bit value: the packed entry would drop it
    assert _tables_sorted(fine) and not _tables_binned(fine)
    above_one = thr.clone()
    above_one[:, 14] = 1.5  # never counted by either form: harmless
    assert _table_class(above_one) == (True, True)


def test_the_answer_follows_the_tensor_version():
    _, thr = synth.make_tables(1, seed=2)
    assert _tables_binned(thr)
    e = float(torch.floor(thr[0, 3].float() * 512))
    thr[0, 3] = (e + 0.25) / 512  # modified in place: the kept answer is stale and must not be used
    thr[0, 4] = (e + 0.75) / 512
    assert not _tables_binned(thr)
