"""Numpy restatement of the reference exact-mode decode attention (TEST ORACLE).

Follows ``_page_table_decode_attention`` of the reference
(``src/beyond/runtime/vllm/packed_backend.py:2342-2421``): for every request the
context is dequantised from the packed pages with the statistics *as stored*
(``read_request_from_paged_cache``), KV heads are repeated over their query
group, and plain scaled-dot-product attention of the single query token over
all ``seq_len`` positions is evaluated; ``seq_len == 0`` yields zeros
(:2368-2370).  The split-KV merge follows the reducer of
``quant/fa4_cute/beyond_mixed_decode_sm100.py:2983-3034``.

Scores and sums are evaluated in float64 so that this file is the "truth" the
CUDA kernel (float32 accumulation) is held to within the stated tolerance.
"""

from __future__ import annotations

import numpy as np

from .paged import PageGeometry, read_request


def _attend(q: np.ndarray, k_hat: np.ndarray, v_hat: np.ndarray, scale: float, group: int):
    """q (Hq, D); k_hat/v_hat (S, Hkv, D) -> unnormalised o (Hq, D), m (Hq,), l (Hq,)."""
    heads_q, dim = q.shape
    o = np.zeros((heads_q, dim), dtype=np.float64)
    m = np.zeros((heads_q,), dtype=np.float64)
    l = np.zeros((heads_q,), dtype=np.float64)
    for h in range(k_hat.shape[1]):  # the query heads of one group share their KV head
        rows = slice(h * group, (h + 1) * group)
        k64 = k_hat[:, h].astype(np.float64)
        v64 = v_hat[:, h].astype(np.float64)
        s = (q[rows].astype(np.float64) @ k64.T) * float(scale)
        m[rows] = s.max(axis=1)
        p = np.exp(s - m[rows, None])
        l[rows] = p.sum(axis=1)
        o[rows] = p @ v64
    return o, m, l


def decode_attention(
    q: np.ndarray,
    cache: np.ndarray,
    geom: PageGeometry,
    block_table: np.ndarray,
    seq_lens,
    *,
    levels_k=None,
    levels_v=None,
    softmax_scale: float,
    stat: str = "f16",
    kv_range: tuple[int, int] | None = None,
    return_partials: bool = False,
):
    """Single-token attention for a batch.  ``q`` is ``(B, Hq, D)``.

    ``kv_range=(lo, hi)`` restricts every request to positions ``lo <= t <
    min(hi, seq_len)`` (used by the KV-range-split tests); with
    ``return_partials`` the unnormalised ``(o, m, l)`` triple is returned
    instead of the normalised output."""
    q = np.asarray(q)
    B, Hq, D = q.shape
    group = Hq // geom.heads
    out = np.zeros((B, Hq, D), dtype=np.float64)
    ms = np.full((B, Hq), -np.inf, dtype=np.float64)
    ls = np.zeros((B, Hq), dtype=np.float64)
    for b in range(B):
        n = int(seq_lens[b])
        lo, hi = (0, n) if kv_range is None else (max(0, kv_range[0]), min(n, kv_range[1]))
        if n <= 0 or hi <= lo:
            continue
        pages = (n + geom.block_size - 1) // geom.block_size
        k_hat, v_hat = read_request(
            cache, geom, block_table[b, :pages], n, levels_k=levels_k, levels_v=levels_v, stat=stat
        )
        o, m, l = _attend(q[b].astype(np.float32), k_hat[lo:hi], v_hat[lo:hi], softmax_scale, group)
        if return_partials:
            out[b], ms[b], ls[b] = o, m, l
        else:
            out[b] = o / l[:, None]
    if return_partials:
        return out, ms, ls
    return out.astype(np.float32)


def merge_partials(o_parts: np.ndarray, m_parts: np.ndarray, l_parts: np.ndarray) -> np.ndarray:
    """Log-sum-exp merge of split partials along axis 0:
    ``o = sum_s e^{m_s-M} O_s / sum_s e^{m_s-M} l_s`` with ``M = max_s m_s``;
    rows whose every split is empty (``l == 0``) give zeros."""
    o_parts = np.asarray(o_parts, dtype=np.float64)
    m_parts = np.asarray(m_parts, dtype=np.float64)
    l_parts = np.asarray(l_parts, dtype=np.float64)
    M = m_parts.max(axis=0)
    safe_M = np.where(np.isfinite(M), M, 0.0)
    w = np.where(l_parts > 0, np.exp(np.where(np.isfinite(m_parts), m_parts, -np.inf) - safe_M), 0.0)
    den = (w * l_parts).sum(axis=0)
    num = (w[..., None] * o_parts).sum(axis=0)
    out = np.where(den[..., None] > 0, num / np.where(den[..., None] > 0, den[..., None], 1.0), 0.0)
    return out.astype(np.float32)
