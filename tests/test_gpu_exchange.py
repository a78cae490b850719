"""The pushed KV-range exchange on ONE GPU.  Two "ranks" live in this process, each with its own
receive buffer; their exchange kernels run one after the other in one stream, so no kernel ever
waits for a kernel that runs beside it: the rank that goes first finds the other's record missing
and its BOUNDED wait runs out (it records that in its status word, leaves its output alone and
returns - nothing hangs), the rank that goes second finds both records, and when the first rank
repeats the step it finds them too.  The records are real range partials of a long request, and
the merged output is held to the oracle."""

import ctypes

import numpy as np
import pytest
import torch

import oracle
from beyond_kv_cache_b200 import _lib, parallel, synth
from beyond_kv_cache_b200.quant.beyond_cute import PagedLayout
from tests.helpers import oracle_cache, tables

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 2e-3


def _alloc(nbytes):
    buf, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
    _lib.call("bkv_kv_exchange_alloc", nbytes, ctypes.byref(buf), handle)
    return buf


def _merge(record, rows, peers, rank, step, timeout_ns, out, status):
    _lib.call("bkv_kv_exchange_merge_sm100", record.data_ptr(), rows, peers, 2, rank, step, timeout_ns, out.data_ptr(),
              _lib.BKV_F32, None, status.data_ptr(), _lib.current_stream(out.device))
    torch.cuda.synchronize()


def test_two_ranks_in_turn_and_a_wait_that_runs_out():
    lens = [9000, 130, 0, 64]
    heads_kv, bs = 2, 16
    lk, tk, lv, tv = tables(heads_kv, 8)
    cache, bt = oracle_cache(lens, heads_kv, bs, "bf16", 10, tk.float().numpy(), tv.float().numpy())
    q = torch.from_numpy(np.random.default_rng(4).standard_normal((4, 8, 128)).astype(np.float32)).to(torch.bfloat16)
    want = oracle.decode_attention(q.float().numpy(), cache, oracle.PageGeometry(bs, heads_kv), bt, lens,
                                   levels_k=lk.float().numpy(), levels_v=lv.float().numpy(),
                                   softmax_scale=synth.softmax_scale(), stat="bf16")
    layout = PagedLayout.build_hnd(bs, heads_kv, 128, 4, 32, 32)
    qd, cd, btd = q.to(DEV), torch.from_numpy(cache).to(DEV), torch.from_numpy(bt).to(DEV)
    lens_d = torch.tensor(lens, dtype=torch.int32, device=DEV)
    rows = 4 * 8
    records = []
    for rank in range(2):  # what each rank's range decode leaves: o | m | l in one block
        lo, hi = parallel.kv_range_for_rank(max(lens), bs, 2, rank)
        o, m, l = parallel.decode_range_partial(qd, cd, layout, btd, lens_d, lk.to(DEV), lv.to(DEV), token_lo=lo,
                                                token_hi=hi, softmax_scale=synth.softmax_scale(), stat_dtype=torch.bfloat16)
        records.append(torch.cat([o.reshape(-1), m.reshape(-1), l.reshape(-1)]).contiguous())
    nbytes = int(_lib.load().bkv_kv_exchange_bytes(2, rows))
    assert nbytes == (2 * 2 * rows * 130 + 4 + 4) * 4  # records, flag words, control words
    bufs = [_alloc(nbytes), _alloc(nbytes)]
    peers = (ctypes.c_uint64 * 2)(bufs[0].value, bufs[1].value)
    try:
        status = [torch.zeros(1, dtype=torch.int32, device=DEV) for _ in range(2)]
        outs = [torch.full((4, 8, 128), 7.0, dtype=torch.float32, device=DEV) for _ in range(2)]
        for step in (1, 2, 3):  # both buffer parities, and a slot that is reused
            status[1].zero_()
            outs[1].fill_(7.0)
            # rank 1 goes first: rank 0 has not published this step, the wait (200 us) runs out
            _merge(records[1], rows, peers, 1, step, 200_000, outs[1], status[1])
            assert int(status[1].item()) == 1
            assert bool((outs[1] == 7.0).all())  # untouched
            # rank 0 goes second: both records are in its buffer
            _merge(records[0], rows, peers, 0, step, 2_000_000_000, outs[0], status[0])
            assert int(status[0].item()) == 0
            assert np.abs(outs[0].cpu().numpy() - want).max() <= TOL
            # rank 1 repeats the step: now it finds both
            status[1].zero_()
            _merge(records[1], rows, peers, 1, step, 2_000_000_000, outs[1], status[1])
            assert int(status[1].item()) == 0
            assert torch.equal(outs[1], outs[0])
        assert not outs[0][2].any()  # the empty request
    finally:
        for b in bufs:
            _lib.call("bkv_kv_exchange_free", b)


def test_exchange_object_with_one_rank():
    """KvRangeExchange outside a process group: a world of one (push to itself, merge one record)."""
    lens = [700, 33]
    lk, tk, lv, tv = tables(2, 8)
    cache, bt = oracle_cache(lens, 2, 16, "f16", 3, tk.float().numpy(), tv.float().numpy())
    q = torch.from_numpy(np.random.default_rng(4).standard_normal((2, 8, 128)).astype(np.float32)).to(torch.float16)
    want = oracle.decode_attention(q.float().numpy(), cache, oracle.PageGeometry(16, 2), bt, lens,
                                   levels_k=lk.float().numpy(), levels_v=lv.float().numpy(),
                                   softmax_scale=synth.softmax_scale(), stat="f16")
    layout = PagedLayout.build_hnd(16, 2, 128, 4, 32, 32)
    ex = parallel.KvRangeExchange(rows=16, device=torch.device(DEV))
    try:
        out = torch.empty((2, 8, 128), dtype=torch.float16, device=DEV)
        out32 = torch.empty((2, 8, 128), dtype=torch.float32, device=DEV)
        for _ in range(3):
            parallel.decode_kv_range_split(q.to(DEV), torch.from_numpy(cache).to(DEV), layout, torch.from_numpy(bt).to(DEV),
                                           torch.tensor(lens, dtype=torch.int32, device=DEV), lk.to(DEV), lv.to(DEV), out,
                                           token_lo=0, token_hi=704, softmax_scale=synth.softmax_scale(),
                                           stat_dtype=torch.float16, exchange=ex, out_f32=out32)
        ex.check()
        assert np.abs(out32.cpu().numpy() - want).max() <= TOL
        # the step is counted on the device, so the launches are the same every time: a captured
        # graph replays range decode + exchange (both buffer parities), here with new queries
        qd, cd, btd = q.to(DEV), torch.from_numpy(cache).to(DEV), torch.from_numpy(bt).to(DEV)
        lens_d, lkd, lvd = torch.tensor(lens, dtype=torch.int32, device=DEV), lk.to(DEV), lv.to(DEV)
        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.graph(graph, stream=side):
            parallel.decode_kv_range_split(qd, cd, layout, btd, lens_d, lkd, lvd, out, token_lo=0, token_hi=704,
                                           softmax_scale=synth.softmax_scale(), stat_dtype=torch.float16, exchange=ex, out_f32=out32)
        torch.cuda.current_stream().wait_stream(side)
        for seed in (11, 12, 13):
            q2 = torch.from_numpy(np.random.default_rng(seed).standard_normal((2, 8, 128)).astype(np.float32)).to(torch.float16)
            qd.copy_(q2)
            graph.replay()
            torch.cuda.synchronize()
            want2 = oracle.decode_attention(q2.float().numpy(), cache, oracle.PageGeometry(16, 2), bt, lens,
                                            levels_k=lk.float().numpy(), levels_v=lv.float().numpy(),
                                            softmax_scale=synth.softmax_scale(), stat="f16")
            assert np.abs(out32.cpu().numpy() - want2).max() <= TOL
        ex.check()
        with pytest.raises(ValueError, match="another bucket"):
            parallel.decode_kv_range_split(q.to(DEV)[:1], torch.from_numpy(cache).to(DEV), layout, torch.from_numpy(bt).to(DEV),
                                           torch.tensor(lens, dtype=torch.int32, device=DEV), lk.to(DEV), lv.to(DEV), out[:1],
                                           token_lo=0, token_hi=704, softmax_scale=synth.softmax_scale(), exchange=ex)
    finally:
        ex.close()
