"""Per-layer quant configuration: load the trained ``quant_config_*.pt`` (or ``.json``)
file, validate every K/V projection entry, and hand the kernels the tables of one
attention layer (reference ``src/beyond/quantization/runtime_config.py``; the table
resolution and tensor-parallel slicing follow
``src/beyond/runtime/vllm/packed_backend.py:968-1014, 2040-2172``).

File format (written by the reference's training): a dict keyed by projection name, e.g.
``"model.layers.0.self_attn.k_proj"``, whose values hold ``quant_points`` ``(tables, 2^bits)``
or ``(2^bits,)``, ``thresholds`` one shorter, and optional ``num_bits``, ``grouping_dim``,
``table_axis``, ``group_size``, ``table_storage_dtype``, ``table_precision_abi``,
``table_compute_dtype``; fused-QKV exports nest ``{"k": {...}, "v": {...}}`` under
``*.qkv_proj`` / ``*.query_key_value``; ``__metadata__`` may name the base model.
"""

from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass
from typing import Iterator, Optional

import torch

from .table_precision import (
    LEGACY_TABLE_PRECISION_ABI,
    TABLE_COMPUTE_DTYPE_NAME,
    TABLE_PRECISION_ABI,
    storage_dtype_name,
    torch_dtype_for_storage,
)

_FALSE_WORDS = frozenset({"0", "false", "no", "off", "disable", "disabled", "none"})


@dataclass(frozen=True)
class LayerQuantConfig:
    """Tables of one projection (CPU tensors in their serialized dtype; reference `:80-92`)."""

    num_bits: int
    grouping_dim: str  # always "token"
    q_points: torch.Tensor  # (2^bits,) or (tables, 2^bits)
    thresholds: torch.Tensor  # (2^bits - 1,) or (tables, 2^bits - 1)
    table_storage_dtype: str
    table_precision_abi: str
    table_compute_dtype: str = TABLE_COMPUTE_DTYPE_NAME
    table_axis: str = "group"
    group_size: Optional[int] = None


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def _read_raw(path: str):
    if path.endswith(".pt"):
        try:
            return torch.load(path, map_location="cpu", weights_only=False)
        except TypeError:  # older torch without the keyword
            return torch.load(path, map_location="cpu")
    with open(path, "r") as f:
        return json.load(f)


def _base_model_of(raw: dict, path: str) -> Optional[str]:
    """Model the tables were trained for: metadata in the file, else ``metrics.json`` two
    directories up (reference `:47-65`)."""
    for key in ("__metadata__", "metadata"):
        meta = raw.get(key)
        if isinstance(meta, dict):
            name = meta.get("base_model") or meta.get("model_id")
            if name:
                return str(name)
    if isinstance(raw.get("base_model"), str) and raw["base_model"]:
        return raw["base_model"]
    metrics = os.path.join(os.path.dirname(os.path.dirname(path)), "metrics.json")
    try:
        with open(metrics, "r", encoding="utf-8") as f:
            found = json.load(f)
    except (OSError, json.JSONDecodeError, TypeError):
        return None
    name = found.get("base_model") if isinstance(found, dict) else None
    return str(name) if name else None


def _same_model(expected: str, actual: str) -> bool:
    def norm(v: str) -> str:
        return str(v).strip().replace("\\", "/").rstrip("/").lower()

    a, b = norm(expected), norm(actual)
    return a == b or a.rsplit("/", 1)[-1] == b.rsplit("/", 1)[-1]


def _projection_entries(raw: dict) -> Iterator[tuple[str, dict]]:
    """Flat ``*.k_proj`` / ``*.v_proj`` entries, unfolding fused-QKV exports (reference `:343-374`)."""
    for key, entry in raw.items():
        if not isinstance(entry, dict):
            continue
        if "quant_points" in entry and "thresholds" in entry:
            yield key, entry
            continue
        base = key
        for suffix in (".query_key_value", ".qkv_proj"):
            if key.endswith(suffix):
                base = key[: -len(suffix)]
        for short, proj in (("k", "k_proj"), ("v", "v_proj")):
            inner = entry.get(short)
            if isinstance(inner, dict) and "quant_points" in inner and "thresholds" in inner:
                flat = dict(inner)
                flat.setdefault("proj_type", proj)
                flat.setdefault("type", f"{entry.get('type', 'QuantizedQKVLinear')}.{short}")
                yield f"{base}.{proj}", flat


def _key_aliases(key: str) -> Iterator[str]:
    """The same projection under the module prefixes training and serving use
    (``model.`` / ``language_model.model.`` / ``model.language_model.``; reference `:377-415`)."""
    out = [key]
    for old, new in (("language_model.model.", "model.language_model."), ("model.language_model.", "language_model.model.")):
        if key.startswith(old):
            out.append(new + key[len(old):])
    if key.startswith("language_model.model."):
        out.append("model." + key[len("language_model.model."):])
    elif key.startswith("model."):
        out.append("language_model.model." + key[len("model."):])
    seen = set()
    for k in out:
        if k not in seen:
            seen.add(k)
            yield k


def _levels_in(entry: dict) -> int:
    q = entry["quant_points"]
    if torch.is_tensor(q):
        return int(q.shape[-1])
    row = q[0] if isinstance(q, list) and q and isinstance(q[0], list) else q
    return len(row)


def _parse_entry(key: str, entry: dict, expected_bits: Optional[int]) -> LayerQuantConfig:
    """Validate one projection entry (every check and message of reference `:148-270`)."""
    qp_raw, th_raw = torch.as_tensor(entry["quant_points"]), torch.as_tensor(entry["thresholds"])
    declared_storage = entry.get("table_storage_dtype")
    if declared_storage is None:
        q_name, t_name = storage_dtype_name(qp_raw), storage_dtype_name(th_raw)
        if q_name != t_name:
            raise ValueError(f"{key}: legacy q_points/thresholds storage dtypes differ: {q_name} vs {t_name}")
        storage = q_name
    else:
        storage = str(declared_storage).strip().lower()
    dtype = torch_dtype_for_storage(storage)
    qp, th = qp_raw.to(dtype=dtype).contiguous(), th_raw.to(dtype=dtype).contiguous()

    declared_abi = entry.get("table_precision_abi")
    if declared_abi is None:
        if storage == "float16":
            raise ValueError(f"{key}: float16 tables require an explicit table_precision_abi")
        abi = LEGACY_TABLE_PRECISION_ABI
    else:
        abi = str(declared_abi).strip()
    declared_compute = entry.get("table_compute_dtype")
    compute = str(declared_compute or TABLE_COMPUTE_DTYPE_NAME).strip().lower()
    if compute != TABLE_COMPUTE_DTYPE_NAME:
        raise ValueError(f"{key}: table_compute_dtype must be {TABLE_COMPUTE_DTYPE_NAME!r}, got {compute!r}")
    if storage == "float16" and abi != TABLE_PRECISION_ABI:
        raise ValueError(f"{key}: float16 tables require table_precision_abi={TABLE_PRECISION_ABI!r}")
    if abi == TABLE_PRECISION_ABI:
        if storage != "float16":
            raise ValueError(f"{key}: {TABLE_PRECISION_ABI!r} requires float16 table storage")
        if declared_storage is None:
            raise ValueError(f"{key}: {TABLE_PRECISION_ABI!r} requires explicit table_storage_dtype metadata")
        if declared_compute is None:
            raise ValueError(f"{key}: {TABLE_PRECISION_ABI!r} requires explicit table_compute_dtype metadata")
    elif abi != LEGACY_TABLE_PRECISION_ABI:
        raise ValueError(f"{key}: unsupported table_precision_abi={abi!r}")

    bits = int(entry.get("num_bits") or int.bit_length(_levels_in(entry) - 1))
    grouping = str(entry.get("grouping_dim") or "token").lower()
    if expected_bits is not None and bits != expected_bits:
        raise ValueError(f"{key}: num_bits={bits} doesn't match expected {expected_bits}")
    if grouping != "token":
        raise ValueError(f"{key}: grouping_dim={grouping!r} is unsupported; K/V quantization configs must be token-grouped")
    levels = 1 << bits
    if qp.dim() not in (1, 2):
        raise ValueError(f"{key}: q_points must be rank 1 or rank 2, got shape {tuple(qp.shape)}")
    if int(qp.shape[-1]) != levels:
        raise ValueError(f"{key}: q_points levels {qp.shape[-1]} != 2^{bits} = {levels}")
    want = tuple(qp.shape[:-1]) + (levels - 1,)
    if tuple(th.shape) != want:
        raise ValueError(f"{key}: thresholds shape {tuple(th.shape)} does not match expected {want}")

    axis = str(entry.get("table_axis") or "").lower() or ("group" if qp.dim() == 2 else "shared")
    if axis in ("per_group", "groups"):
        axis = "group"
    if axis not in ("shared", "group"):
        raise ValueError(f"{key}: unsupported table_axis={axis!r}")
    if axis == "shared" and qp.dim() != 1:
        raise ValueError(f"{key}: table_axis='shared' requires rank-1 q_points, got shape {tuple(qp.shape)}")
    if axis == "group" and qp.dim() != 2:
        raise ValueError(f"{key}: table_axis='group' requires rank-2 q_points, got shape {tuple(qp.shape)}")
    gs_raw = entry.get("group_size")
    group_size = None if gs_raw in (None, "") else int(gs_raw)
    if group_size is not None and group_size <= 0:
        raise ValueError(f"{key}: group_size must be positive, got {group_size}")

    if not torch.isfinite(qp).all():
        raise ValueError(f"{key}: q_points contain NaN or Inf")
    if not torch.isfinite(th).all():
        raise ValueError(f"{key}: thresholds contain NaN or Inf")
    if bool(((th < 0.0) | (th > 1.0)).any()):
        raise ValueError(f"{key}: thresholds must lie in normalized range [0, 1]")
    if qp.shape[-1] > 1 and not bool((qp[..., 1:] > qp[..., :-1]).all()):
        raise ValueError(f"{key}: q_points must be strictly increasing")
    if th.shape[-1] > 1 and not bool((th[..., 1:] > th[..., :-1]).all()):
        raise ValueError(f"{key}: thresholds must be strictly increasing")
    return LayerQuantConfig(num_bits=bits, grouping_dim=grouping, q_points=qp, thresholds=th, table_storage_dtype=storage,
                            table_precision_abi=abi, table_compute_dtype=compute, table_axis=axis, group_size=group_size)


class QuantConfig:
    """Whole-model table set keyed by ``"{attention module}.{k_proj|v_proj}"`` (reference `:95-330`)."""

    def __init__(self, per_layer: dict[str, LayerQuantConfig], expected_bits: Optional[int], *, source_path: str,
                 source_identity: str, source_model: Optional[str]):
        self._d = per_layer
        self.expected_bits = expected_bits
        self.source_path = source_path
        self.identity = source_identity
        self.source_model = source_model

    @classmethod
    def load(cls, path: str, *, expected_bits: Optional[int] = None, expected_model: Optional[str] = None,
             require_model_metadata: bool = False) -> "QuantConfig":
        path = os.path.abspath(path)
        identity = f"{path}:{_sha256(path)}"
        raw = _read_raw(path)
        meta = raw.get("__metadata__") if isinstance(raw, dict) else None
        if isinstance(meta, dict) and (
            str(meta.get("artifact_type") or "") == "beyond_uncompressed_kv_adapter_config"
            or meta.get("compressed_kv_cache") is False
            or meta.get("hard_forward") is False
        ):
            raise ValueError(f"{path}: uncompressed continuous KV adapter artifacts cannot be loaded as hard-QDQ "
                             "compressed quant configs")
        per_layer = {key: _parse_entry(key, entry, expected_bits) for key, entry in _projection_entries(raw)}
        if not per_layer:
            raise ValueError(f"{path}: quant config contains no K/V projection entries")
        cfg = cls(per_layer, expected_bits, source_path=path, source_identity=identity, source_model=_base_model_of(raw, path))
        cfg.validate_model(expected_model, require_metadata=bool(require_model_metadata))
        return cfg

    def for_attention_layer(self, layer_name: str, proj_type: str) -> Optional[LayerQuantConfig]:
        """``'model.layers.0.self_attn.attn'`` + ``'k_proj'`` -> that projection's tables, under
        any of the equivalent module prefixes."""
        base = layer_name[: -len(".attn")] if layer_name.endswith(".attn") else layer_name
        for alias in _key_aliases(f"{base}.{proj_type}"):
            if alias in self._d:
                return self._d[alias]
        return None

    def __len__(self) -> int:
        return len(self._d)

    def items(self):
        return self._d.items()

    def validate_model(self, expected_model: Optional[str], *, require_metadata: bool = False) -> None:
        if not expected_model:
            return
        if not self.source_model:
            if require_metadata:
                raise ValueError(f"{self.source_path}: cannot verify model identity for {expected_model!r}; add "
                                 "base_model metadata or keep the config beside its run metrics.json")
            return
        if not _same_model(expected_model, self.source_model):
            raise ValueError(f"{self.source_path}: quant config model {self.source_model!r} does not match requested "
                             f"model {expected_model!r}")


# ---- tables of one layer, as the kernels take them ------------------------------------------
def slice_group_tables_for_tensor_parallel(q_points: torch.Tensor, thresholds: torch.Tensor, local_tables: Optional[int], *,
                                           label: str, tp_rank: int = 0, tp_world: int = 1):
    """Rows of full-model per-(head, group) tables that belong to this tensor-parallel rank's
    KV heads (reference ``packed_backend.py:968-1014``): already-local and shared tables pass
    through, full tables are cut into ``tp_world`` equal runs, anything else is refused."""
    if q_points.dim() != 2 or thresholds.dim() != 2 or local_tables is None:
        return q_points, thresholds
    local, full = int(local_tables), int(q_points.shape[0])
    if full == local:
        return q_points, thresholds
    world = max(1, int(tp_world))
    if full == local * world:
        start = int(tp_rank) * local
        if start < 0 or start + local > full:
            raise ValueError(f"{label} per-group qtables cannot be sliced for tp_rank={tp_rank}, tp_world={world}: "
                             f"tables={full}, local_tables={local}")
        return q_points[start : start + local], thresholds[start : start + local]
    raise ValueError(f"{label} per-group qtable count {full} does not match local H * head_dim/group_size = {local}; "
                     f"tp_rank={tp_rank}, tp_world={world}. For tensor-parallel fake-quant inference, grouped qtables "
                     "must be either already local or full-model tables divisible across tensor-parallel ranks.")


def resolve_layer_tables(config: QuantConfig, layer_name: str, *, heads_kv: int, head_dim: int = 128, group_size: int = 32,
                         tp_rank: int = 0, tp_world: int = 1):
    """``(levels_k, thresholds_k, levels_v, thresholds_v)`` of one attention layer for this rank's
    ``heads_kv`` local KV heads: 4-bit tables, per (head, group) ``(heads_kv*head_dim/group_size, 16|15)``
    or shared ``(16|15,)``, float16 — what ``write_tokens_to_paged_cache`` and
    ``prepare_runtime_qpoints`` take."""
    out = []
    local = heads_kv * (head_dim // group_size)
    for proj in ("k_proj", "v_proj"):
        entry = config.for_attention_layer(layer_name, proj)
        if entry is None:
            raise KeyError(f"{layer_name}: no {proj} tables in {config.source_path}")
        if entry.num_bits != 4:
            raise ValueError(f"{layer_name}.{proj}: the packed cache holds 4-bit codes, the config has {entry.num_bits}")
        if entry.group_size not in (None, group_size):
            raise ValueError(f"{layer_name}.{proj}: group_size {entry.group_size} != {group_size}")
        qp, th = slice_group_tables_for_tensor_parallel(entry.q_points, entry.thresholds, local, label=f"{layer_name}.{proj}",
                                                        tp_rank=tp_rank, tp_world=tp_world)
        out += [qp.to(torch.float16).contiguous(), th.to(torch.float16).contiguous()]
    return tuple(out)


# ---- process-wide instance named by the environment (reference `:429-507`) -------------------
_cached: Optional[QuantConfig] = None
_cached_key: Optional[tuple] = None


def _env_enabled(name: str, default: bool) -> bool:
    value = os.environ.get(name)
    return bool(default) if value is None else value.strip().lower() not in _FALSE_WORDS


def get_config_from_env(*, force_reload: bool = False) -> Optional[QuantConfig]:
    """The config named by ``BEYOND_QUANT_CONFIG`` (``BEYOND_BITS``, ``BEYOND_MODEL_ID`` and
    ``BEYOND_QUANT_CONFIG_STRICT`` as in the reference), loaded once per distinct setting."""
    global _cached, _cached_key
    path = os.environ.get("BEYOND_QUANT_CONFIG")
    if not path:
        _cached, _cached_key = None, None
        return None
    bits_env = os.environ.get("BEYOND_BITS")
    key = (os.path.abspath(path), int(bits_env) if bits_env else None, os.environ.get("BEYOND_MODEL_ID"),
           _env_enabled("BEYOND_QUANT_CONFIG_STRICT", True))
    if not force_reload and _cached is not None and _cached_key == key:
        return _cached
    apath, bits, model, strict = key
    _cached = QuantConfig.load(apath, expected_bits=bits, expected_model=model if strict else None,
                               require_model_metadata=bool(strict and model))
    _cached_key = key
    return _cached
