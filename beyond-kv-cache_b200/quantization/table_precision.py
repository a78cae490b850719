"""Precision contract of the learned level / threshold tables (reference
``src/beyond/quantization/table_precision.py``).

Tables are optimised as float32 masters but deployed as IEEE binary16: the encode kernel
compares against, and the decode kernel multiplies by, exactly the float16 values.  A table
is valid for deployment only if rounding it to float16 keeps levels and thresholds strictly
increasing; the names and checks here are the reference's (`:12-70`), so a file written by
one side loads on the other.
"""

from __future__ import annotations

import torch

TABLE_PRECISION_ABI = "beyond.ieee-fp16-tables.v1"
LEGACY_TABLE_PRECISION_ABI = "beyond.legacy-fp32-tables.v0"
TABLE_STORAGE_DTYPE_NAME = "float16"
TABLE_COMPUTE_DTYPE_NAME = "float32"
TABLE_STORAGE_DTYPE = torch.float16
TABLE_MASTER_DTYPE = torch.float32

# Two binary16 units in the last place at 1.0 (2 * 2^-10): neighbouring table entries
# at least this far apart cannot collapse onto one float16 value (reference `:19-24`).
FP16_STRICT_MIN_GAP = 2.0**-9

_STORAGE_NAMES = {torch.float16: "float16", torch.float32: "float32"}


def fp16_ste_roundtrip(master: torch.Tensor) -> torch.Tensor:
    """Values as the deployed float16 table holds them, with the gradient of the float32
    master passed straight through (reference `:27-34`)."""
    if master.dtype != TABLE_MASTER_DTYPE:
        raise TypeError(f"quant-table master must be float32, got {master.dtype}")
    deployed = master.to(TABLE_STORAGE_DTYPE).to(TABLE_MASTER_DTYPE)
    if torch.is_grad_enabled() and master.requires_grad:
        return master + (deployed - master).detach()
    return deployed


def cast_table_for_storage(table: torch.Tensor) -> torch.Tensor:
    """Detached, contiguous CPU copy in the deployment dtype (reference `:37-39`)."""
    return table.detach().to(device="cpu", dtype=TABLE_STORAGE_DTYPE).contiguous()


def _rises(table: torch.Tensor) -> bool:
    return table.shape[-1] < 2 or bool((table[..., 1:] > table[..., :-1]).all())


def validate_fp16_storage_tables(quant_points: torch.Tensor, thresholds: torch.Tensor, *, label: str = "quant table") -> None:
    """Raise unless the pair satisfies the FP16 table ABI: float16 dtype, thresholds one
    shorter than the levels, finite, strictly increasing after rounding (reference `:46-70`)."""
    for name, t in (("quant_points", quant_points), ("thresholds", thresholds)):
        if t.dtype != TABLE_STORAGE_DTYPE:
            raise TypeError(f"{label}: {name} must be float16, got {t.dtype}")
    want = tuple(quant_points.shape[:-1]) + (int(quant_points.shape[-1]) - 1,)
    if tuple(thresholds.shape) != want:
        raise ValueError(f"{label}: thresholds shape {tuple(thresholds.shape)} does not match {want}")
    for name, t in (("quant_points", quant_points), ("thresholds", thresholds)):
        if not bool(torch.isfinite(t).all()):
            raise ValueError(f"{label}: {name} contain NaN or Inf")
    for name, t in (("quant_points", quant_points), ("thresholds", thresholds)):
        if not _rises(t):
            raise ValueError(f"{label}: {name} collapse after float16 rounding")


def storage_dtype_name(tensor: torch.Tensor) -> str:
    """Serialized name of a table tensor's dtype; only float16 and float32 exist (reference `:73-79`)."""
    try:
        return _STORAGE_NAMES[tensor.dtype]
    except KeyError:
        raise TypeError(f"unsupported quant-table storage dtype: {tensor.dtype}") from None


def torch_dtype_for_storage(name: str) -> torch.dtype:
    """Inverse of :func:`storage_dtype_name`; aliases such as "half" are refused (reference `:82-89`)."""
    key = str(name).strip().lower()
    for dtype, known in _STORAGE_NAMES.items():
        if key == known:
            return dtype
    raise ValueError(f"unsupported quant-table storage dtype: {name!r}")
