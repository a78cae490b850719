"""KV-range split of one long sequence across two GPUs: every rank attends its own page
range from its own copy of the pages and every rank merges all partials; the result must match
the oracle over the whole sequence, both when the partials travel by NCCL all-gather and when
they are pushed into the peers' buffers (plain peer stores through CUDA IPC mappings, bounded
wait).  Needs two GPUs (skipped otherwise); ranks are child processes, NVLS off."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from beyond_kv_cache_b200 import parallel, synth
from beyond_kv_cache_b200.quant.beyond_cute import PagedLayout
from tests.helpers import oracle_cache, tables

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, result_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        lens = [20000 + 7, 333]  # same data on every rank
        heads_kv, bs = 2, 16
        lk, tk, lv, tv = tables(heads_kv, 3)
        cache, bt = oracle_cache(lens, heads_kv, bs, "bf16", 5, tk.float().numpy(), tv.float().numpy())
        q = torch.from_numpy(np.random.default_rng(2).standard_normal((2, 8, 128)).astype(np.float32)).to(torch.bfloat16)
        layout = PagedLayout.build_hnd(bs, heads_kv, 128, 4, 32, 32)
        lo, hi = parallel.kv_range_for_rank(max(lens), bs, world, rank)
        want = oracle.decode_attention(q.float().numpy(), cache, oracle.PageGeometry(bs, heads_kv), bt, lens,
                                       levels_k=lk.float().numpy(), levels_v=lv.float().numpy(),
                                       softmax_scale=synth.softmax_scale(), stat="bf16")
        args = (q.to(dev), torch.from_numpy(cache).to(dev), layout, torch.from_numpy(bt).to(dev),
                torch.tensor(lens, dtype=torch.int32, device=dev), lk.to(dev), lv.to(dev))
        err = 0.0
        exchange = parallel.KvRangeExchange(rows=2 * 8, device=dev)
        try:
            for ex in (None, exchange, exchange, exchange):  # NCCL form, then three pushed steps (both parities)
                out = torch.empty((2, 8, 128), dtype=torch.float32, device=dev)
                parallel.decode_kv_range_split(*args, out, token_lo=lo, token_hi=hi, softmax_scale=synth.softmax_scale(),
                                               stat_dtype=torch.bfloat16, exchange=ex)
                torch.cuda.synchronize()
                err = max(err, float(np.abs(out.cpu().numpy() - want).max()))
            exchange.check()
        finally:
            exchange.close()
        with open(f"{result_path}.{rank}", "w") as f:
            f.write(f"{err}")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_kv_range_split_over_nccl_and_pushed(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    path = str(tmp_path / "err")
    mp.spawn(_rank_main, args=(2, _free_port(), path), nprocs=2, join=True)
    for rank in range(2):
        with open(f"{path}.{rank}") as f:
            assert float(f.read()) <= TOL
