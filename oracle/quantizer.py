"""Numpy restatement of the reference 4-bit / group-32 quantiser (TEST ORACLE).

Follows ``quant/beyond_cute.py`` of the reference:

* default tables ........ ``make_uniform_q_points`` / ``make_uniform_thresholds``
  (:75-93) and the storage rule of ``prepare_qpoints_and_thresholds`` (:116-195)
* bucket search ......... ``_bucketize`` (:250-264)
* nibble packing ........ ``pack_codes`` / ``unpack_codes`` (:358-431)
* encode ................ ``quantize_k`` (:439-486) == ``quantize_v`` (:525-584)
* reconstruction ........ ``dequantize_k`` (:489-517) == ``dequantize_v`` (:587-616)
* unrounded fake-QDQ .... ``_fake_quant_token_4d``
  (``src/beyond/runtime/vllm/packed_backend.py:1081-1154``)

All arithmetic is IEEE binary32 with round-to-nearest-even, one rounding per
operation, exactly as the eager torch CPU code of the reference performs it.
16-bit statistics are carried as raw ``uint16`` bit patterns plus a kind string
(``"f16"`` or ``"bf16"``) so the oracle does not depend on a bfloat16 dtype.
"""

from __future__ import annotations

import numpy as np

GROUP = 32  # scalars per quantisation group (SUPPORTED_GROUP_SIZES, :55)
LEVELS = 16  # 4-bit codes (SUPPORTED_BITS, :54)
_F32 = np.float32


# --------------------------------------------------------------------------- 16-bit
def round_to_stat(x: np.ndarray, kind: str) -> np.ndarray:
    """float32 -> 16-bit storage bits, round-to-nearest-even (``.to(stat_dtype)``)."""
    x = np.ascontiguousarray(x, dtype=_F32)
    if kind == "f16":
        return x.astype(np.float16).view(np.uint16)
    if kind == "bf16":
        bits = x.view(np.uint32).astype(np.uint64)
        is_nan = np.isnan(x)
        bias = np.uint64(0x7FFF) + ((bits >> np.uint64(16)) & np.uint64(1))
        out = ((bits + bias) >> np.uint64(16)).astype(np.uint16)
        out = np.where(is_nan, np.uint16(0x7FC0), out)
        return out.astype(np.uint16)
    raise TypeError(f"stat kind must be 'f16' or 'bf16', got {kind!r}")


def stat_to_f32(bits: np.ndarray, kind: str) -> np.ndarray:
    """16-bit storage bits -> float32 (exact widening)."""
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    if kind == "f16":
        return bits.view(np.float16).astype(_F32)
    if kind == "bf16":
        return (bits.astype(np.uint32) << np.uint32(16)).view(_F32)
    raise TypeError(f"stat kind must be 'f16' or 'bf16', got {kind!r}")


# --------------------------------------------------------------------------- tables
def uniform_levels() -> np.ndarray:
    """``i / 15`` evaluated in Python floats, then cast to float32 (:75-88)."""
    return np.array([i / 15 for i in range(LEVELS)], dtype=_F32)


def uniform_thresholds(levels: np.ndarray) -> np.ndarray:
    """Mid-points by division, not by ``* 0.5`` (:91-93)."""
    levels = np.asarray(levels, dtype=_F32)
    return ((levels[..., :-1] + levels[..., 1:]) / _F32(2.0)).astype(_F32)


def default_tables() -> tuple[np.ndarray, np.ndarray]:
    """Tables used when the caller passes none: fp16 storage of the uniform
    levels, thresholds rounded to fp16 from the float32 master mid-points
    (:136-148, :186-193).  Returned widened to float32."""
    master = uniform_levels()
    levels = master.astype(np.float16).astype(_F32)
    thresholds = uniform_thresholds(master).astype(np.float16).astype(_F32)
    return levels, thresholds


def _tables_for(values: np.ndarray, heads: int, groups: int, width: int, what: str) -> np.ndarray:
    """Broadcast a shared ``(width,)`` or per-(head, group) ``(heads*groups, width)``
    table to ``(heads, groups, width)`` float32 (:252-263, :268-286)."""
    t = np.asarray(values).astype(_F32)
    if t.ndim == 1:
        if t.shape[0] != width:
            raise ValueError(f"{what} must have {width} entries, got {t.shape}")
        return np.broadcast_to(t, (heads, groups, width))
    if t.ndim != 2 or t.shape != (heads * groups, width):
        raise ValueError(
            f"{what} table count {t.shape} != expected {(heads * groups, width)}"
        )
    return t.reshape(heads, groups, width)


# --------------------------------------------------------------------------- packing
def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """``(..., 32)`` uint8 codes -> ``(..., 4)`` uint32 words; code ``i`` occupies
    bits ``4*(i%8) .. 4*(i%8)+3`` of word ``i//8`` (:380-395)."""
    codes = np.asarray(codes)
    if codes.dtype != np.uint8:
        raise TypeError("codes must be uint8")
    if codes.shape[-1] != GROUP:
        raise ValueError(f"group_size {codes.shape[-1]} not in ({GROUP},)")
    c = codes.reshape(*codes.shape[:-1], 4, 8).astype(np.uint32)
    shifts = (np.arange(8, dtype=np.uint32) * np.uint32(4))
    return np.bitwise_or.reduce(c << shifts, axis=-1).astype(np.uint32)


def unpack_nibbles(words: np.ndarray) -> np.ndarray:
    """Inverse of :func:`pack_nibbles` (:398-431)."""
    words = np.asarray(words).astype(np.uint32)
    if words.shape[-1] != 4:
        raise ValueError(f"packed shape tail {words.shape[-1]} != words_per_group 4")
    shifts = (np.arange(8, dtype=np.uint32) * np.uint32(4))
    c = (words[..., None] >> shifts) & np.uint32(0xF)
    return c.reshape(*words.shape[:-1], GROUP).astype(np.uint8)


# --------------------------------------------------------------------------- encode
def encode_groups(x: np.ndarray, thresholds: np.ndarray | None = None, *, stat: str = "f16"):
    """Quantise ``x`` of shape ``(..., H, D)`` group-wise along ``D``.

    Returns a dict with ``codes`` uint8 ``(..., H, D//32, 32)``, ``words`` uint32
    ``(..., H, D//32, 4)``, ``scale_bits`` / ``mn_bits`` uint16 ``(..., H, D//32)``
    (stored 16-bit statistics) and the unrounded float32 ``scale`` / ``mn``.
    Order of operations is the reference's (:469-475): min, max, one float32
    subtract, clamp with ``float32(1e-6)``, one subtract, one IEEE divide, clamp
    to [0, 1], then ``#{j : thr[j] <= x_norm}``.
    """
    x = np.asarray(x)
    if x.ndim < 2:
        raise ValueError("expected x.shape=(..., H, D)")
    H, D = x.shape[-2], x.shape[-1]
    if D % GROUP:
        raise ValueError(f"head_dim {D} not divisible by group_size {GROUP}")
    G = D // GROUP
    if thresholds is None:
        thresholds = default_tables()[1]
    thr = _tables_for(thresholds, H, G, LEVELS - 1, "thresholds")
    xf = x.astype(_F32).reshape(*x.shape[:-1], G, GROUP)
    mn = xf.min(axis=-1)
    mx = xf.max(axis=-1)
    scale = np.maximum((mx - mn).astype(_F32), _F32(1e-6)).astype(_F32)
    delta = (xf - mn[..., None]).astype(_F32)
    x_norm = np.clip((delta / scale[..., None]).astype(_F32), _F32(0.0), _F32(1.0))
    # count of thresholds <= x_norm (== bucketize(right=True) for sorted tables)
    codes = (x_norm[..., None] >= thr[..., None, :]).sum(axis=-1).astype(np.uint8)
    return {
        "codes": codes,
        "words": pack_nibbles(codes),
        "scale_bits": round_to_stat(scale, stat),
        "mn_bits": round_to_stat(mn, stat),
        "scale": scale,
        "mn": mn,
        "stat": stat,
    }


# --------------------------------------------------------------------------- decode
def decode_groups(
    codes: np.ndarray,
    levels: np.ndarray | None,
    scale_bits: np.ndarray,
    mn_bits: np.ndarray,
    *,
    stat: str = "f16",
) -> np.ndarray:
    """``x_hat = f32(level[code]) * f32(stored scale) + f32(stored min)`` as two
    separately rounded float32 operations (:511-517).  ``codes`` is
    ``(..., H, G, 32)``; result is float32 ``(..., H, G*32)``."""
    codes = np.asarray(codes)
    H, G = codes.shape[-3], codes.shape[-2]
    if levels is None:
        levels = default_tables()[0]
    lv = _tables_for(levels, H, G, LEVELS, "q_points")
    lv_b = np.broadcast_to(lv[..., None, :], (*codes.shape, LEVELS))
    vals = np.take_along_axis(lv_b, codes[..., None].astype(np.int64), axis=-1)[..., 0]
    scale = stat_to_f32(scale_bits, stat)[..., None]
    mn = stat_to_f32(mn_bits, stat)[..., None]
    prod = (vals.astype(_F32) * scale).astype(_F32)
    out = (prod + mn).astype(_F32)
    return out.reshape(*codes.shape[:-2], G * GROUP)


def fake_qdq_unrounded(x: np.ndarray, levels: np.ndarray, thresholds: np.ndarray) -> np.ndarray:
    """Training-equivalent fake quantise/dequantise with *unrounded* float32
    statistics (``packed_backend.py:1125-1154``).  Codes are identical to
    :func:`encode_groups`; only the reconstruction differs."""
    enc = encode_groups(x, thresholds)
    codes = enc["codes"]
    H, G = codes.shape[-3], codes.shape[-2]
    lv = _tables_for(levels, H, G, LEVELS, "q_points")
    lv_b = np.broadcast_to(lv[..., None, :], (*codes.shape, LEVELS))
    vals = np.take_along_axis(lv_b, codes[..., None].astype(np.int64), axis=-1)[..., 0]
    out = ((vals * enc["scale"][..., None]).astype(_F32) + enc["mn"][..., None]).astype(_F32)
    return out.reshape(*codes.shape[:-2], G * GROUP)
