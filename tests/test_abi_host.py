"""Host-side checks of the C ABI that need no GPU: the library loads, exports every entry
point the public header declares, and the ctypes binding lists the same names; the work
partition of the persistent decode kernel agrees with the part list its merging workers
derive (a host-only entry point, pure integer arithmetic)."""

import ctypes
import os
import re

import numpy as np
import pytest

from beyond_kv_cache_b200 import _lib

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "bkv_sm100.h")


def _declared():
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    return sorted(set(re.findall(r"\b(bkv_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_entry_point():
    lib = _lib.load()
    names = _declared()
    assert len(names) >= 18
    for name in names:
        assert getattr(lib, name) is not None
    assert sorted(_lib.SIGNATURES) == names  # the binding covers the header, and nothing else
    assert lib.bkv_abi_version() == 2
    assert lib.bkv_status_string(0) == b"ok"
    assert b"maximum" in lib.bkv_status_string(_lib.ERR_LIMIT)


def _partition(tiles, hv, sms, cap):
    arr = np.asarray(tiles, dtype=np.int32)
    return _lib.load().bkv_selftest_partition(arr.ctypes.data_as(ctypes.c_void_p), len(arr), hv, sms, cap)


@pytest.mark.parametrize("hv", [1, 2, 3, 8, 16, 37, 148])
def test_partition_and_part_lists_agree(hv):
    rng = np.random.default_rng(hv)
    shapes = [
        [512] * 64,                      # the benchmark shape: every request cut several times
        [8192],                          # one long request: one partial per CTA
        [1, 2, 0, 3, 1],                 # fewer tiles than workers
        [0, 0, 0],                       # nothing to attend
        [64] * 300,                      # many short requests, most of them whole
        list(rng.integers(0, 60, 1500)), # more requests than the in-kernel table holds
        list(rng.integers(0, 900, 37)) + [4100, 1, 2500],
        [7000, 3, 9000, 0, 1, 2000],
    ]
    for tiles in shapes:
        cap = max(max(tiles), 1)
        for sms in (148, 132, max(hv, 7)):
            if sms < hv:
                continue
            assert _partition(tiles, hv, sms, cap) == 0, (hv, sms, tiles[:8])
            assert _partition(tiles, hv, sms, 4 * cap) == 0  # a launch bucket larger than the longest request


def test_partition_selftest_rejects_bad_arguments():
    assert _partition([1, 2], 0, 148, 4) == -1
    assert _partition([1, 2], 200, 148, 4) == -1  # more heads than SMs
    assert _partition([9], 1, 148, 4) == -1       # a request longer than the bucket
