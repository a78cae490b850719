"""Seeded synthetic tables and workloads with the shapes of the reference's benchmarks.

The reference measured on Llama-3.1-8B-shaped tensors with learned tables that are
not distributed with it; these generators stand in for both.  Tables follow the
validity rules the reference enforces on exported tables (strictly increasing after
fp16 rounding, minimum gap 2^-9, thresholds inside (0, 1);
``src/beyond/quantization/table_precision.py:19-70``,
``src/beyond/quantization/training.py:93-154``).
"""

from __future__ import annotations

import math

import numpy as np
import torch

MIN_GAP = 2.0**-9


def _project_increasing(values: np.ndarray, lo: float, hi: float, gap: float = MIN_GAP) -> np.ndarray:
    """Nearest-from-below/above monotone projection: sorted, inside [lo, hi], and
    consecutive entries at least ``gap`` apart."""
    v = np.clip(np.sort(np.asarray(values, dtype=np.float64)), lo, hi)
    for i in range(1, len(v)):
        v[i] = max(v[i], v[i - 1] + gap)
    v = np.minimum(v, hi)
    for i in range(len(v) - 2, -1, -1):
        v[i] = min(v[i], v[i + 1] - gap)
    return np.clip(v, lo, hi)


def make_tables(heads_kv: int, seed: int = 0, *, per_group: bool = False, which: str = "k"):
    """Levels ``(heads_kv*4, 16)`` and thresholds ``(heads_kv*4, 15)`` as fp16 CPU tensors.

    One table per KV head: 16 sorted uniform draws with the end points pinned at 0
    and 1, thresholds at the level mid-points plus U(-0.01, 0.01) jitter, projected to
    the validity rules above, then replicated over the head's four groups (with
    ``per_group`` every (head, group) gets its own draw).  K and V use different
    streams of the same seed."""
    rng = np.random.default_rng([int(seed), 0 if which == "k" else 1])
    n_tables = heads_kv * 4 if per_group else heads_kv
    levels = np.empty((n_tables, 16), dtype=np.float32)
    thresholds = np.empty((n_tables, 15), dtype=np.float32)
    for t in range(n_tables):
        lv = np.sort(rng.uniform(0.0, 1.0, 16))
        lv[0], lv[-1] = 0.0, 1.0
        lv = _project_increasing(lv, 0.0, 1.0)
        thr = (lv[:-1] + lv[1:]) / 2.0 + rng.uniform(-0.01, 0.01, 15)
        thr = _project_increasing(thr, MIN_GAP, 1.0 - MIN_GAP)
        levels[t], thresholds[t] = lv, thr
    lv16 = torch.from_numpy(levels).to(torch.float16)
    th16 = torch.from_numpy(thresholds).to(torch.float16)
    if not per_group:
        lv16 = lv16.repeat_interleave(4, dim=0)
        th16 = th16.repeat_interleave(4, dim=0)
    for name, t in (("levels", lv16), ("thresholds", th16)):
        if not bool((t[:, 1:] > t[:, :-1]).all()):
            raise RuntimeError(f"synthetic {name} collapse after fp16 rounding")
    return lv16.contiguous(), th16.contiguous()


def outlier_channels(heads_kv: int, seed: int = 0, count: int = 4) -> torch.Tensor:
    """Indices ``(heads_kv, count)`` of the K channels that are scaled by 8."""
    rng = np.random.default_rng([int(seed), 2])
    return torch.from_numpy(np.stack([rng.choice(128, size=count, replace=False) for _ in range(heads_kv)]))


def config0_inputs(seed: int = 0):
    """The CPU-sized parity configuration: batch 4, 32 query / 8 KV heads, head_dim
    128, context 1024; float32 Q, K, V ~ N(0,1) with the K outlier channels scaled
    by 8.  Returns numpy arrays ``q (4,32,128)``, ``k``/``v`` ``(4096,8,128)``
    (request-major rows) from a platform-stable generator."""
    rng = np.random.default_rng([int(seed), 7])
    batch, heads_q, heads_kv, dim, ctx = 4, 32, 8, 128, 1024
    q = rng.standard_normal((batch, heads_q, dim)).astype(np.float32)
    k = rng.standard_normal((batch * ctx, heads_kv, dim)).astype(np.float32)
    v = rng.standard_normal((batch * ctx, heads_kv, dim)).astype(np.float32)
    outl = outlier_channels(heads_kv, seed).numpy()
    for h in range(heads_kv):
        k[:, h, outl[h]] *= 8.0
    return q, k, v


def make_kv(tokens: int, heads_kv: int, *, seed: int, device, dtype=torch.bfloat16, chunk: int = 1 << 16):
    """K, V of shape ``(tokens, heads_kv, 128)``: N(0,1), K with 4 outlier channels
    per head scaled by 8.  Generated on ``device`` in chunks."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    k = torch.empty((tokens, heads_kv, 128), dtype=dtype, device=device)
    v = torch.empty_like(k)
    boost = torch.ones((heads_kv, 128), dtype=torch.float32, device=device)
    idx = outlier_channels(heads_kv, seed).to(device)
    boost.scatter_(1, idx, 8.0)
    for start in range(0, tokens, chunk):
        n = min(chunk, tokens - start)
        k[start : start + n] = (torch.randn((n, heads_kv, 128), generator=gen, device=device) * boost).to(dtype)
        v[start : start + n] = torch.randn((n, heads_kv, 128), generator=gen, device=device).to(dtype)
    return k, v


def random_block_table(batch: int, pages_per_seq: int, *, seed: int, device, spare_pages: int = 0):
    """A random permutation of physical pages dealt to ``batch`` requests:
    returns ``(block_table int32 (batch, pages_per_seq), num_pages)``."""
    total = batch * pages_per_seq
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    perm = torch.randperm(total + spare_pages, generator=gen)[:total].to(torch.int32)
    return perm.reshape(batch, pages_per_seq).to(device).contiguous(), total + spare_pages


def slots_for(block_table: torch.Tensor, block_size: int, start: int, count: int) -> torch.Tensor:
    """Flat slot ids of positions ``start .. start+count-1`` of every request,
    request-major: ``(batch*count,)`` int64."""
    pos = torch.arange(start, start + count, device=block_table.device)
    page = block_table[:, pos // block_size].to(torch.int64)
    return (page * block_size + (pos % block_size)).reshape(-1)


def softmax_scale(head_dim: int = 128) -> float:
    return 1.0 / math.sqrt(head_dim)
