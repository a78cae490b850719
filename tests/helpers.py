"""Shared helpers of the GPU parity tests (numpy <-> torch, oracle-built caches)."""

import numpy as np
import torch

import oracle
from beyond_kv_cache_b200 import synth
from beyond_kv_cache_b200.quant.beyond_cute import PagedLayout
from beyond_kv_cache_b200.quant.fa4_cute import beyond_mixed_decode_runtime as rt

KIND_TO_DTYPE = {"f16": torch.float16, "bf16": torch.bfloat16}


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def tables(heads, seed, per_group=True):
    """(levels_k, thr_k, levels_v, thr_v) fp16 CPU tensors."""
    lk, tk = synth.make_tables(heads, seed=seed, per_group=per_group, which="k")
    lv, tv = synth.make_tables(heads, seed=seed, per_group=per_group, which="v")
    return lk, tk, lv, tv


def oracle_cache(seq_lens, heads, block_size, kind, seed, thr_k, thr_v, spare=3):
    """Encode random K/V of the given lengths with the ORACLE into a paged cache with
    a random block table.  Returns (cache int32 ndarray, block_table int32 ndarray)."""
    rng = np.random.default_rng(seed)
    pages = [(n + block_size - 1) // block_size for n in seq_lens]
    width = max(max(pages), 1)
    total = sum(pages) + spare
    perm = rng.permutation(total)
    bt = np.full((len(seq_lens), width), -1, dtype=np.int32)
    geo = oracle.PageGeometry(block_size, heads, 128)
    # pages start out as random words, as in the reference's own tests (quant/tests/test_paged.py:528-536):
    # whatever a page holds beyond the positions written below - NaN and infinite statistics included -
    # must not reach the attention output
    cache = rng.integers(-(2**31), 2**31, (total, geo.block_i32)).astype(np.int32)
    cursor = 0
    for b, n in enumerate(seq_lens):
        bt[b, : pages[b]] = perm[cursor : cursor + pages[b]]
        cursor += pages[b]
        if n == 0:
            continue
        k = rng.standard_normal((n, heads, 128)).astype(np.float32)
        v = rng.standard_normal((n, heads, 128)).astype(np.float32)
        k[:, :, rng.choice(128, 4, replace=False)] *= 8.0
        k = oracle.stat_to_f32(oracle.round_to_stat(k, kind), kind)
        v = oracle.stat_to_f32(oracle.round_to_stat(v, kind), kind)
        pos = np.arange(n)
        slots = bt[b].astype(np.int64)[pos // block_size] * block_size + pos % block_size
        for c0 in range(0, n, 8192):  # the oracle's temporaries grow with the rows of a call
            c1 = min(n, c0 + 8192)
            oracle.write_pages(cache, geo, slots[c0:c1], k[c0:c1], v[c0:c1], thresholds_k=thr_k, thresholds_v=thr_v, stat=kind)
    return cache, bt


def gpu_decode(q, cache, bt, seq_lens, heads_kv, block_size, lk, lv, *, kind, splits=0, loader=0, max_seq_len=None, scale=None):
    """Run the product launcher (``splits=0``: persistent schedule, else the split grid with
    that count); returns (out in q.dtype, out_f32, spec), the tensors on the CPU."""
    dev = torch.device("cuda")
    layout = PagedLayout.build_hnd(block_size, heads_kv, 128, 4, 32, 32)
    qd = q.to(dev)
    cache_d = torch.from_numpy(cache).to(dev)
    bt_d = torch.from_numpy(bt).to(dev)
    lens_d = torch.tensor(list(seq_lens), dtype=torch.int32, device=dev)
    if max_seq_len is None:
        max_seq_len = max(block_size, ((max(seq_lens) + block_size - 1) // block_size) * block_size)
    rk, rv = rt.prepare_runtime_qpoints(lk.to(dev), lv.to(dev), heads_kv=heads_kv)
    spec = rt.make_runtime_spec(q=qd, cache=cache_d, layout=layout, block_table=bt_d, heads_q=q.shape[1],
                                max_seq_len=max_seq_len, num_splits=splits)
    ws = rt.allocate_runtime_workspace(spec, device=dev)
    out = torch.empty(q.shape, dtype=q.dtype, device=dev)
    out32 = torch.empty(q.shape, dtype=torch.float32, device=dev)
    rt.run_nonuniform_decode(spec=spec, q=qd, cache=cache_d, layout=layout, block_table=bt_d, seq_lens=lens_d,
                             k_qpoints_lane_major=rk, v_qpoints_code_major=rv, out=out, workspace=ws,
                             softmax_scale=scale if scale is not None else synth.softmax_scale(),
                             stat_dtype=KIND_TO_DTYPE[kind], out_f32=out32, loader=loader)
    torch.cuda.synchronize()
    return out.cpu(), out32.cpu(), spec
