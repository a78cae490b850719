"""Environment readers and the packed-layout contract of the vLLM backend (reference
``src/beyond/runtime/vllm/config.py``); imports nothing heavy."""

from __future__ import annotations

import os

FAKE_QUANT_SUPPORTED_BITS = (1, 2, 3, 4, 5, 6)
REAL_PACKED_GROUP_SIZES = (32,)
_TRUE_WORDS = frozenset({"1", "true", "yes", "on", "enable", "enabled"})
_FALSE_WORDS = frozenset({"0", "false", "no", "off", "disable", "disabled", "none"})


def env_int(name: str, default: int) -> int:
    """Integer environment variable; unset or unparsable gives ``default`` (reference `:11-19`)."""
    try:
        return int(os.environ[name])
    except (KeyError, ValueError):
        return default


def env_bool(name: str, default: bool) -> bool:
    """Boolean environment variable in the project's permissive spelling (reference `:22-32`)."""
    word = os.environ.get(name, "").strip().lower()
    if word in _TRUE_WORDS:
        return True
    if word in _FALSE_WORDS and name in os.environ:
        return False
    return bool(default)


def env_bits(name: str) -> int:
    """Bit width of the fake-QDQ mode, refused outside 1..6 (reference `:35-42`)."""
    bits = env_int(name, 4)
    if bits not in FAKE_QUANT_SUPPORTED_BITS:
        raise ValueError(f"Beyond fakequant supports bits in {FAKE_QUANT_SUPPORTED_BITS}, got {bits}")
    return bits


def validate_real_packed_layout(bits: int, k_group_size: int, v_group_size: int) -> None:
    """The compressed backend exists for 4-bit codes in groups of 32 only (reference `:45-60`)."""
    if int(bits) != 4:
        raise NotImplementedError("BeyondPacked real backend supports only 4-bit")
    for name, size in (("k_group_size", k_group_size), ("v_group_size", v_group_size)):
        if int(size) not in REAL_PACKED_GROUP_SIZES:
            raise NotImplementedError(f"BeyondPacked real backend {name} must be 32, got {size}")
