"""Numpy restatement of the reference paged packed-cache ABI (TEST ORACLE).

Follows ``quant/beyond_cute.py`` of the reference:

* region sizes / offsets ... ``PagedLayout.build`` (:675-765)
* scatter of K ............. ``_write_flat_k_pk_to_cache`` (:1945-2040)
* scatter of V ............. ``write_v_pv_to_cache`` (:1859-1942)
* writer semantics ......... ``_write_tokens_to_paged_cache_reference`` (:2043-2144)
* read-back ................ ``read_request_from_paged_cache`` (:2210-2395)

A page is ``block_i32`` int32 words holding four regions: K codes, K statistics,
V codes, V statistics.  A statistics word carries the stored 16-bit scale in its
low half and the stored 16-bit minimum in its high half (:1992-1997, :1156-1164).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .quantizer import (
    GROUP,
    decode_groups,
    encode_groups,
    round_to_stat,
    stat_to_f32,
    unpack_nibbles,
)

ABI_TOKEN_MAJOR = "hnd_token_word"  # ABI v2, production
ABI_WORD_MAJOR = "head_word_token"  # ABI v1, legacy


@dataclass(frozen=True)
class PageGeometry:
    """Word offsets of one packed page (all in int32 units)."""

    block_size: int
    heads: int
    head_dim: int = 128
    abi: str = ABI_TOKEN_MAJOR

    def __post_init__(self):
        if self.head_dim % GROUP:
            raise ValueError(f"head_dim {self.head_dim} not divisible by group_size {GROUP}")
        if self.abi not in (ABI_TOKEN_MAJOR, ABI_WORD_MAJOR):
            raise ValueError(f"unsupported code_layout {self.abi!r}")

    @property
    def groups(self) -> int:
        return self.head_dim // GROUP

    @property
    def code_words(self) -> int:  # per region
        return self.heads * self.block_size * self.groups * 4

    @property
    def stat_words(self) -> int:  # per region
        return self.heads * self.block_size * self.groups

    @property
    def k_code_off(self) -> int:
        return 0

    @property
    def k_stat_off(self) -> int:
        return self.code_words

    @property
    def v_code_off(self) -> int:
        return self.code_words + self.stat_words

    @property
    def v_stat_off(self) -> int:
        return 2 * self.code_words + self.stat_words

    @property
    def block_i32(self) -> int:
        return 2 * self.code_words + 2 * self.stat_words

    # ---- word index inside a page, broadcastable over (tok, h, g, w) ----
    def code_index(self, tok, h, g, w):
        G, BS = self.groups, self.block_size
        if self.abi == ABI_TOKEN_MAJOR:
            return h * (BS * G * 4) + tok * (G * 4) + g * 4 + w  # (:2010-2016)
        return h * (G * 4 * BS) + (g * 4 + w) * BS + tok  # (:2025-2031)

    def k_stat_index(self, tok, h, g):
        G, BS = self.groups, self.block_size
        if self.abi == ABI_TOKEN_MAJOR:
            return h * (BS * G) + tok * G + g  # (:2017-2023)
        return h * (G * BS) + g * BS + tok  # (:2032-2038)

    def v_stat_index(self, tok, h, g):
        G, BS = self.groups, self.block_size
        return h * (G * BS) + g * BS + tok  # group-major in both ABIs (:1935-1941)


def _stat_words(scale_bits: np.ndarray, mn_bits: np.ndarray) -> np.ndarray:
    return (scale_bits.astype(np.uint32) | (mn_bits.astype(np.uint32) << np.uint32(16))).astype(
        np.uint32
    )


def write_pages(
    cache: np.ndarray,
    geom: PageGeometry,
    slots: np.ndarray,
    k: np.ndarray,
    v: np.ndarray,
    *,
    thresholds_k=None,
    thresholds_v=None,
    stat: str = "f16",
):
    """Encode ``k``/``v`` of shape ``(T, H, D)`` and scatter them into ``cache``
    (``(pages, block_i32)`` int32, modified in place).  Rows with ``slot < 0``
    leave the cache untouched (:2067-2130).  Returns the two encode dicts."""
    if cache.dtype != np.int32 or cache.ndim != 2 or cache.shape[1] != geom.block_i32:
        raise ValueError("cache must be (pages, block_i32) int32")
    T, H, D = k.shape
    if v.shape != k.shape or H != geom.heads or D != geom.head_dim:
        raise ValueError("K/V shape mismatch")
    ek = encode_groups(k, thresholds_k, stat=stat)
    ev = encode_groups(v, thresholds_v, stat=stat)
    slots = np.asarray(slots).astype(np.int64).reshape(-1)
    if slots.shape[0] != T:
        raise ValueError(f"slot_mapping has {slots.shape[0]} tokens, K has {T}")
    valid = slots >= 0
    if not valid.any():
        return ek, ev
    flat = cache.reshape(-1).view(np.uint32)
    page = (slots[valid] // geom.block_size)[:, None, None, None]
    tok = (slots[valid] % geom.block_size)[:, None, None, None]
    G = geom.groups
    h = np.arange(H, dtype=np.int64)[None, :, None, None]
    g = np.arange(G, dtype=np.int64)[None, None, :, None]
    w = np.arange(4, dtype=np.int64)[None, None, None, :]
    base = page * geom.block_i32
    code_idx = base + geom.code_index(tok, h, g, w)
    flat[(code_idx + geom.k_code_off).reshape(-1)] = ek["words"][valid].reshape(-1)
    flat[(code_idx + geom.v_code_off).reshape(-1)] = ev["words"][valid].reshape(-1)
    b3, t3, h3, g3 = base[..., 0], tok[..., 0], h[..., 0], g[..., 0]
    ks = b3 + geom.k_stat_off + geom.k_stat_index(t3, h3, g3)
    vs = b3 + geom.v_stat_off + geom.v_stat_index(t3, h3, g3)
    flat[ks.reshape(-1)] = _stat_words(ek["scale_bits"][valid], ek["mn_bits"][valid]).reshape(-1)
    flat[vs.reshape(-1)] = _stat_words(ev["scale_bits"][valid], ev["mn_bits"][valid]).reshape(-1)
    return ek, ev


def gather_request(cache: np.ndarray, geom: PageGeometry, block_ids, seq_len: int):
    """Collect the packed representation of one request: code words
    ``(S, H, G, 4)`` and statistic bit patterns ``(S, H, G)`` for K and V."""
    block_ids = np.asarray(block_ids).astype(np.int64).reshape(-1)
    BS, H, G = geom.block_size, geom.heads, geom.groups
    if block_ids.shape[0] * BS < seq_len:
        raise ValueError("not enough blocks for seq_len")
    pos = np.arange(seq_len, dtype=np.int64)
    page = block_ids[pos // BS][:, None, None, None]
    tok = (pos % BS)[:, None, None, None]
    h = np.arange(H, dtype=np.int64)[None, :, None, None]
    g = np.arange(G, dtype=np.int64)[None, None, :, None]
    w = np.arange(4, dtype=np.int64)[None, None, None, :]
    flat = cache.reshape(-1).view(np.uint32)
    base = page * geom.block_i32
    ci = base + geom.code_index(tok, h, g, w)
    k_words = flat[ci + geom.k_code_off]
    v_words = flat[ci + geom.v_code_off]
    b3, t3, h3, g3 = base[..., 0], tok[..., 0], h[..., 0], g[..., 0]
    k_stat = flat[b3 + geom.k_stat_off + geom.k_stat_index(t3, h3, g3)]
    v_stat = flat[b3 + geom.v_stat_off + geom.v_stat_index(t3, h3, g3)]
    lo = lambda a: (a & np.uint32(0xFFFF)).astype(np.uint16)  # noqa: E731  scale
    hi = lambda a: (a >> np.uint32(16)).astype(np.uint16)  # noqa: E731  minimum
    return {
        "k_words": k_words,
        "v_words": v_words,
        "k_scale_bits": lo(k_stat),
        "k_mn_bits": hi(k_stat),
        "v_scale_bits": lo(v_stat),
        "v_mn_bits": hi(v_stat),
    }


def read_request(
    cache: np.ndarray,
    geom: PageGeometry,
    block_ids,
    seq_len: int,
    *,
    levels_k=None,
    levels_v=None,
    stat: str = "f16",
    out: str = "f32",
):
    """Dequantise one request's context to ``(S, H, D)`` float32 arrays.
    ``out`` in {"f32", "f16", "bf16"} applies the final ``.to(out_dtype)``
    rounding of the reference (:2322-2326, :2390-2393); values are returned
    widened back to float32."""
    parts = gather_request(cache, geom, block_ids, seq_len)
    k_hat = decode_groups(
        unpack_nibbles(parts["k_words"]), levels_k, parts["k_scale_bits"], parts["k_mn_bits"], stat=stat
    )
    v_hat = decode_groups(
        unpack_nibbles(parts["v_words"]), levels_v, parts["v_scale_bits"], parts["v_mn_bits"], stat=stat
    )
    if out != "f32":
        k_hat = stat_to_f32(round_to_stat(k_hat, out), out)
        v_hat = stat_to_f32(round_to_stat(v_hat, out), out)
    return k_hat, v_hat
