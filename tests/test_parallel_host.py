"""Host-side logic of the multi-GPU paths on CPU: partitioning, and the partial exchange
run as a world-size-2 gloo job whose merged result must equal single-process attention
(the per-rank arithmetic is the oracle's; the GPU form of the same exchange is covered by
tests/test_gpu_decode.py::test_kv_range_partials_merge_to_full)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from beyond_kv_cache_b200 import parallel, synth


def test_shard_requests_partitions_exactly():
    for batch in (0, 1, 7, 64, 4500):
        for world in (1, 2, 3, 8):
            parts = [parallel.shard_requests(batch, world, r) for r in range(world)]
            flat = [i for p in parts for i in p]
            assert flat == list(range(batch))
            sizes = [len(p) for p in parts]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        parallel.shard_requests(4, 2, 2)


def test_kv_ranges_are_page_aligned_and_cover():
    for seq_len in (0, 1, 15, 16, 17, 131072, 100003):
        for bs in (16, 128):
            for world in (1, 2, 8):
                rs = [parallel.kv_range_for_rank(seq_len, bs, world, r) for r in range(world)]
                covered = sorted(t for lo, hi in rs for t in (range(lo, hi) if seq_len < 1000 else ()))
                if seq_len < 1000:
                    assert covered == list(range(seq_len))
                assert rs[0][0] == 0 and sum(hi - lo for lo, hi in rs) == seq_len
                for (lo, hi), (lo2, _) in zip(rs, rs[1:]):
                    assert hi <= lo2 and lo % bs == 0 and lo <= hi
    assert parallel.kv_range_for_rank(131072, 16, 8, 3) == (49152, 65536)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, result_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(11)  # same data on every rank
        heads_kv, T, bs = 2, 150, 16
        geo = oracle.PageGeometry(bs, heads_kv)
        lk, tk = (t.float().numpy() for t in synth.make_tables(heads_kv, seed=2))
        k = rng.standard_normal((T, heads_kv, 128)).astype(np.float32)
        v = rng.standard_normal((T, heads_kv, 128)).astype(np.float32)
        q = rng.standard_normal((1, 8, 128)).astype(np.float32)
        pages = (T + bs - 1) // bs
        bt = rng.permutation(pages).astype(np.int32)[None, :]
        cache = np.zeros((pages, geo.block_i32), dtype=np.int32)
        slots = bt[0].astype(np.int64)[np.arange(T) // bs] * bs + np.arange(T) % bs
        oracle.write_pages(cache, geo, slots, k, v, thresholds_k=tk, thresholds_v=tk)
        lo, hi = parallel.kv_range_for_rank(T, bs, world, rank)
        o, m, l = oracle.decode_attention(q, cache, geo, bt, [T], levels_k=lk, levels_v=lk, softmax_scale=0.09,
                                          kv_range=(lo, hi), return_partials=True)
        o_all, m_all, l_all = parallel.gather_partials(
            torch.from_numpy(o.reshape(8, 128).astype(np.float32)), torch.from_numpy(m.reshape(8).astype(np.float32)),
            torch.from_numpy(l.reshape(8).astype(np.float32)))
        merged = oracle.merge_partials(o_all.numpy(), m_all.numpy(), l_all.numpy())
        full = oracle.decode_attention(q, cache, geo, bt, [T], levels_k=lk, levels_v=lk, softmax_scale=0.09)
        err = float(np.abs(merged - full.reshape(8, 128)).max())
        if rank == 0:
            with open(result_path, "w") as f:
                f.write(f"{err}\n{tuple(o_all.shape)}")
    finally:
        dist.destroy_process_group()


def test_kv_range_exchange_world2_gloo(tmp_path):
    result = tmp_path / "result.txt"
    mp.spawn(_rank_main, args=(2, _free_port(), str(result)), nprocs=2, join=True)
    err, shape = result.read_text().split("\n")
    assert float(err) < 1e-5
    assert shape == "(2, 8, 128)"
