"""Timed CPU run of the oracle's decode path on a bounded sample (TEST/BENCH
INFRASTRUCTURE: used only by the ``cpu_baseline`` and ``--impl reference`` legs of
``bench.py``).

The reference's CPU implementation of this path is eager PyTorch
(``read_request_from_paged_cache`` + ``scaled_dot_product_attention`` per request,
``src/beyond/runtime/vllm/packed_backend.py:2342-2421``); it cannot travel to the
GPU box, so the numpy restatement in this package is what is timed (kind "port").
Requests are independent, so the sample is spread over worker processes, one per
host core, each holding its own packed pages.
"""

from __future__ import annotations

import multiprocessing as mp
import os
import time

import numpy as np

from . import PageGeometry, decode_attention, write_pages

_STATE = {}


def _build(args):
    """Encode one request's random context into a private packed cache (untimed)."""
    seed, ctx, heads_kv, heads_q, block_size, thr_k, thr_v, lv_k, lv_v, stat = args
    rng = np.random.default_rng(seed)
    geo = PageGeometry(block_size, heads_kv, 128)
    pages = (ctx + block_size - 1) // block_size
    cache = np.zeros((pages, geo.block_i32), dtype=np.int32)
    bt = rng.permutation(pages).astype(np.int32)[None, :]
    chunk = 2048
    for start in range(0, ctx, chunk):
        n = min(chunk, ctx - start)
        k = rng.standard_normal((n, heads_kv, 128)).astype(np.float32)
        v = rng.standard_normal((n, heads_kv, 128)).astype(np.float32)
        k[:, :, :4] *= 8.0
        pos = np.arange(start, start + n)
        slots = bt[0].astype(np.int64)[pos // block_size] * block_size + pos % block_size
        write_pages(cache, geo, slots, k, v, thresholds_k=thr_k, thresholds_v=thr_v, stat=stat)
    q = rng.standard_normal((1, heads_q, 128)).astype(np.float32)
    _STATE[seed] = (q, cache, geo, bt, ctx, lv_k, lv_v, stat)
    return seed


def _run(seed):
    q, cache, geo, bt, ctx, lv_k, lv_v, stat = _STATE[seed]
    t0 = time.perf_counter()
    out = decode_attention(q, cache, geo, bt, [ctx], levels_k=lv_k, levels_v=lv_v, softmax_scale=128**-0.5, stat=stat)
    return time.perf_counter() - t0, float(out.sum())


def _worker(conn, build_args):
    try:
        for a in build_args:
            _build(a)
        conn.send("ready")
        while True:
            msg = conn.recv()
            if msg == "stop":
                break
            conn.send([_run(a[0]) for a in build_args])
    finally:
        conn.close()


def time_decode_sample(*, requests: int, ctx: int, heads_kv: int, heads_q: int, block_size: int, tables, stat: str,
                       steps: int = 1, warmup: int = 0, workers: int | None = None):
    """Run ``requests`` independent single-token decodes of ``ctx`` tokens each on the
    host cores.  Returns ``(seconds_per_step, workers_used, packed_bytes_per_step)``,
    where a step attends every request once; wall time is the slowest worker's."""
    lv_k, thr_k, lv_v, thr_v = tables
    workers = max(1, min(workers or (os.cpu_count() or 1), requests))
    per = [[] for _ in range(workers)]
    for r in range(requests):
        per[r % workers].append((1000 + r, ctx, heads_kv, heads_q, block_size, thr_k, thr_v, lv_k, lv_v, stat))
    ctxm = mp.get_context("fork")
    procs = []
    for w in range(workers):
        parent, child = ctxm.Pipe()
        p = ctxm.Process(target=_worker, args=(child, per[w]), daemon=True)
        p.start()
        procs.append((p, parent))
    for _, conn in procs:
        assert conn.recv() == "ready"
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        for _, conn in procs:
            conn.send("go")
        for _, conn in procs:
            conn.recv()
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    for p, conn in procs:
        conn.send("stop")
        p.join(timeout=10)
    packed_bytes = requests * ctx * heads_kv * 160
    return float(np.mean(times)), workers, packed_bytes
