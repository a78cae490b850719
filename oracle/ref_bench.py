"""Timed CPU run of the REFERENCE's own implementation of the decode path on a bounded sample
(BENCH INFRASTRUCTURE: used only by the ``cpu_baseline`` and ``--impl reference`` legs of
``bench.py``).

What is timed is what the reference executes on a CPU for this path - its exact-mode attention
(``_page_table_decode_attention``, ``src/beyond/runtime/vllm/packed_backend.py:2342-2421``): per
request, ``read_request_from_paged_cache`` dequantises the context from the packed pages to
float32 (the staged ``quant/beyond_cute.py``, :2210-2395), the KV heads are repeated over their
query group, and ``torch.nn.functional.scaled_dot_product_attention`` attends one query token.
The packed pages are written by the reference's own ``write_tokens_to_paged_cache`` (untimed).
torch runs with every host core.  The quantiser and the reader are also timed on their own
(``quantize_k/v`` with and without ``pack_codes``, ``dequantize_k/v``), since the reference's
CPU numbers are dominated by Python-level packing.
"""

from __future__ import annotations

import os
import time

import numpy as np
import torch


def _tables(heads_kv: int):
    from beyond_kv_cache_b200 import synth  # seeded table generator only (no device code)

    lk, tk = synth.make_tables(heads_kv, seed=0, which="k")
    lv, tv = synth.make_tables(heads_kv, seed=0, which="v")
    return lk, tk, lv, tv


def build_sample(ref, *, requests: int, ctx: int, heads_kv: int, heads_q: int, block_size: int, stat_dtype):
    """`requests` private packed caches of `ctx` tokens each, written by the reference's writer."""
    lk, tk, lv, tv = _tables(heads_kv)
    layout = ref.PagedLayout.build_hnd(block_size, heads_kv, 128, 4, 32, 32)
    pages = (ctx + block_size - 1) // block_size
    sample = []
    for r in range(requests):
        gen = torch.Generator().manual_seed(1000 + r)
        table = torch.randperm(pages, generator=gen).to(torch.int32)
        cache = torch.zeros((pages, layout.block_i32), dtype=torch.int32)
        chunk = 2048
        for start in range(0, ctx, chunk):
            n = min(chunk, ctx - start)
            k = torch.randn((n, heads_kv, 128), generator=gen)
            v = torch.randn((n, heads_kv, 128), generator=gen)
            k[:, :, :4] *= 8.0
            pos = torch.arange(start, start + n)
            slots = (table[pos // block_size].to(torch.int64) * block_size + pos % block_size).to(torch.int32)
            ref.write_tokens_to_paged_cache(cache, layout, table.view(1, -1), slots, k.to(stat_dtype), v.to(stat_dtype),
                                            q_points_k=lk, q_points_v=lv, thresholds_k=tk, thresholds_v=tv)
        q = torch.randn((heads_q, 128), generator=gen)
        sample.append((cache, table, q))
    return {"layout": layout, "items": sample, "ctx": ctx, "heads_kv": heads_kv, "heads_q": heads_q,
            "tables": (lk, tk, lv, tv), "stat_dtype": stat_dtype}


def decode_step(ref, sample) -> float:
    """One pass of the reference exact-mode decode attention over every request of the sample."""
    lk, _, lv, _ = sample["tables"]
    rep = sample["heads_q"] // sample["heads_kv"]
    scale = 128.0**-0.5
    check = 0.0
    for cache, table, q in sample["items"]:
        k_ctx, v_ctx = ref.read_request_from_paged_cache(cache, sample["layout"], table, sample["ctx"], q_points_k=lk,
                                                         q_points_v=lv, out_dtype=torch.float32,
                                                         stat_dtype=sample["stat_dtype"])
        kr = k_ctx[0].repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)
        vr = v_ctx[0].repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)
        out = torch.nn.functional.scaled_dot_product_attention(q.view(1, -1, 1, 128), kr, vr, scale=scale)
        check += float(out.sum())
    return check


def time_decode_sample(ref, *, requests: int, ctx: int, heads_kv: int, heads_q: int, block_size: int, stat: str,
                       steps: int, warmup: int):
    """Returns (seconds per step, threads, packed bytes attended per step)."""
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    stat_dtype = torch.float16 if stat in ("fp16", "f16") else torch.bfloat16
    sample = build_sample(ref, requests=requests, ctx=ctx, heads_kv=heads_kv, heads_q=heads_q, block_size=block_size,
                          stat_dtype=stat_dtype)
    for _ in range(warmup):
        decode_step(ref, sample)
    t0 = time.perf_counter()
    for _ in range(max(1, steps)):
        decode_step(ref, sample)
    secs = (time.perf_counter() - t0) / max(1, steps)
    return secs, threads, requests * ctx * heads_kv * 160


def quantiser_numbers(ref, *, tokens: int = 4096, heads_kv: int = 8) -> dict:
    """Seconds for the reference's dense quantiser on `tokens` x `heads_kv` x 128 float16 rows (the
    config-0 amount): quantize_k + quantize_v, the same without the Python-level nibble packing
    (pack_codes replaced by a no-op while timing), and dequantize_k + dequantize_v."""
    torch.set_num_threads(os.cpu_count() or 1)
    lk, tk, lv, tv = _tables(heads_kv)
    gen = torch.Generator().manual_seed(5)
    k = torch.randn((1, tokens, heads_kv, 128), generator=gen).half()
    v = torch.randn((1, tokens, heads_kv, 128), generator=gen).half()

    def best(fn, reps=3):
        times = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            times.append(time.perf_counter() - t0)
        return min(times)

    packed = {}

    def quantise():
        packed["k"] = ref.quantize_k(k, 4, 32, q_points=lk, thresholds=tk)
        packed["v"] = ref.quantize_v(v, 4, 32, q_points=lv, thresholds=tv)

    t_quant = best(quantise)
    real_pack = ref.pack_codes
    try:
        ref.pack_codes = lambda codes, bits, pack_axis_first=False: torch.zeros((*codes.shape[:-1], 4), dtype=torch.int32)
        t_nopack = best(quantise)
    finally:
        ref.pack_codes = real_pack
    quantise()
    t_dequant = best(lambda: (ref.dequantize_k(packed["k"], q_points=lk), ref.dequantize_v(packed["v"], q_points=lv)))
    return {"rows": tokens * heads_kv, "quantize_kv_s": t_quant, "quantize_kv_without_pack_s": t_nopack,
            "dequantize_kv_s": t_dequant}
