"""The allocation-free decode entry point (collected last on purpose).

Some users of the library cannot call cudaMalloc where they call us - a plugin living
inside somebody else's capture region, or an embedder with a fixed memory arena - so
`bkv_decode_noalloc_sm100` keeps its split workspace in a fixed array inside the library.
This test drives it through the C ABI twice in a row (the array is shared and keeps the
previous call's contents) and requires the same output as the regular entry point, which
gets a caller-allocated workspace, and - so that the test stands on its own - the CPU oracle
within the decode tolerance.  The result must not depend on whether other tests ran before it
in the same process."""

import numpy as np
import pytest
import torch

import oracle
from beyond_kv_cache_b200 import _lib, synth
from tests.helpers import oracle_cache, tables

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _call(fn, extra_ws, q, cache, bt, lens, lk, lv, out, out32, splits, max_seq_len):
    args = [q.data_ptr(), q.stride(0), _lib.BKV_BF16, cache.data_ptr(), cache.shape[0], cache.stride(0), 16, 2,
            _lib.BKV_BF16, bt.data_ptr(), bt.stride(0), lens.data_ptr(), lk.data_ptr(), lv.data_ptr(), _lib.BKV_F16,
            out.data_ptr(), _lib.BKV_BF16, out32.data_ptr()]
    args += extra_ws
    args += [splits, q.shape[0], q.shape[1], max_seq_len, synth.softmax_scale(), 0]
    args.append(_lib.current_stream(q.device))
    _lib.call(fn, *args)


def test_noalloc_entry_matches_workspace_entry_twice():
    lk, tk, lv, tv = tables(2, 17)
    lkd, lvd = lk.to(DEV), lv.to(DEV)
    for round_idx, lens in enumerate(([700, 130, 0, 64, 2049], [33, 1000, 512, 1, 90])):
        cache_np, bt_np = oracle_cache(lens, 2, 16, "bf16", 100 + round_idx, tk.float().numpy(), tv.float().numpy())
        cache, bt = torch.from_numpy(cache_np).to(DEV), torch.from_numpy(bt_np).to(DEV)
        lens_d = torch.tensor(lens, dtype=torch.int32, device=DEV)
        rng = np.random.default_rng(round_idx)
        q = torch.from_numpy(rng.standard_normal((len(lens), 8, 128)).astype(np.float32)).to(torch.bfloat16).to(DEV)
        max_seq_len = bt.shape[1] * 16
        for splits in (1, 5):
            rows = len(lens) * 8
            ws = [torch.empty((splits, rows, 128), device=DEV), torch.empty((splits, rows), device=DEV),
                  torch.empty((splits, rows), device=DEV)]
            want, want32 = torch.empty_like(q), torch.empty(q.shape, dtype=torch.float32, device=DEV)
            got, got32 = torch.full_like(q, 7.0), torch.full(q.shape, 7.0, dtype=torch.float32, device=DEV)
            _call("bkv_decode_sm100", [w.data_ptr() for w in ws], q, cache, bt, lens_d, lkd, lvd, want, want32, splits, max_seq_len)
            _call("bkv_decode_noalloc_sm100", [], q, cache, bt, lens_d, lkd, lvd, got, got32, splits, max_seq_len)
            torch.cuda.synchronize()
            # same kernels, same arithmetic: identical results (the tests' tolerance is 2e-3)
            assert torch.equal(got32, want32)
            assert torch.equal(got, want)
            assert float(want32.abs().max()) > 0
            truth = oracle.decode_attention(q.float().cpu().numpy(), cache_np, oracle.PageGeometry(16, 2), bt_np, lens,
                                            levels_k=lk.float().numpy(), levels_v=lv.float().numpy(),
                                            softmax_scale=synth.softmax_scale(), stat="bf16")
            assert float(np.abs(got32.cpu().numpy() - truth).max()) <= 2e-3


def test_noalloc_entry_rejects_oversized_launch():
    q = torch.zeros((1, 8, 128), dtype=torch.bfloat16, device=DEV)
    dummy = torch.zeros((8,), dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError, match="exceeds a documented maximum"):
        _lib.call("bkv_decode_noalloc_sm100", q.data_ptr(), q.stride(0), _lib.BKV_BF16, dummy.data_ptr(), 1, 1280, 16, 2,
                  _lib.BKV_BF16, dummy.data_ptr(), 1, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), _lib.BKV_F16,
                  q.data_ptr(), _lib.BKV_BF16, None, 32, 4096, 8, 16, 0.1, 0, _lib.current_stream(q.device))
