"""Graph-safe launcher of the B200 packed decode attention kernel.

Mirror of the reference launcher ``quant/fa4_cute/beyond_mixed_decode_runtime.py``:
``DecodeRuntimeSpec``, ``prepare_runtime_qpoints``, ``make_runtime_spec``,
``allocate_runtime_workspace``, ``run_nonuniform_decode`` and
``clear_compiled_runtime_cache`` keep their names, arguments and error types.
Instead of JIT-compiling a CuTe DSL kernel per launch bucket, every call goes to the
pre-built sm_100a library through the C ABI (``bkv_decode_stream_sm100``, or
``bkv_decode_sm100`` for an explicit split count): nothing is compiled or allocated at
launch, so a launch is capturable without pre-warming.

Differences from the reference contract, all additive:

* pages of 16 and 32 tokens are accepted next to 64 and 128 (the reference
  launcher takes 64/128 only, ``beyond_mixed_decode_runtime.py:156-158``);
* the device must be a B200-class part (compute capability 10.x) instead of
  exactly (10, 3) (``:152-153``);
* split partials are kept in float32 (the reference keeps ``o_partial`` in the
  model dtype, ``:311-324``), which is what makes the 2e-3 output bound hold;
* ``run_nonuniform_decode`` takes two optional keywords: ``stat_dtype`` (dtype of
  the stored scale/min, default the model dtype as in the reference) and
  ``out_f32`` (an optional float32 copy of the result before rounding).
"""

from __future__ import annotations

import os
import threading
from dataclasses import dataclass
from typing import Optional

import torch

from ... import _lib
from ..beyond_cute import CODE_LAYOUT_HND_TOKEN_WORD, PagedLayout
from .beyond_decode_policy import (
    CVT_STAGE_CAP,
    KV_STAGE_CAP,
    normalize_reduction_kind,
    scheduled_pages_per_split,
    select_decode_launch_plan,
)

_DEFAULT_PAGE_SIZE = 128
_HEAD_DIM = 128
_GROUP_SIZE = 32
SUPPORTED_PAGE_SIZES = (16, 32, 64, 128)
_LOCK = threading.RLock()
_SM_COUNT: dict[int, int] = {}


@dataclass(frozen=True)
class DecodeRuntimeSpec:
    """Frozen description of one launch bucket (fields of the reference spec,
    ``beyond_mixed_decode_runtime.py:43-73``); hashable, used as a workspace key.
    ``persistent`` (additive) says that the bucket runs under the persistent schedule, which
    has no split count (``num_splits`` is then 1 and no split workspace is needed)."""

    device_index: int
    model_dtype: str
    qpoint_dtype: str
    batch_size: int
    heads_q: int
    heads_kv: int
    max_seq_len: int
    page_size: int
    num_splits: int
    physical_pages: int
    page_table_stride: int
    packed_page_stride_i32: int
    q_batch_stride: int
    kv_stage_cap: int
    cvt_stage_cap: int
    reduction_kind: str
    cluster_reduction: bool
    task_major_grid: bool
    direct_smem_store: bool
    wait_for_pdl_writer: bool
    persistent: bool = False

    @property
    def pages_per_split(self) -> int:
        return scheduled_pages_per_split(tiles=self.max_seq_len // self.page_size, splits=self.num_splits)


_DTYPE_NAMES = {torch.float16: "fp16", torch.bfloat16: "bf16"}
_DTYPES = {name: dtype for dtype, name in _DTYPE_NAMES.items()}


def _dtype_name(dtype: torch.dtype) -> str:
    try:
        return _DTYPE_NAMES[dtype]
    except KeyError:
        raise TypeError(f"expected fp16 or bf16, got {dtype}") from None


def _torch_dtype(name: str) -> torch.dtype:
    try:
        return _DTYPES[name]
    except KeyError:
        raise ValueError(f"unsupported dtype name {name!r}") from None


def _first_failure(checks):
    """``checks`` yields (ok, message) pairs in contract order; raise ValueError for the first
    pair that is not ok.  The messages are part of the interface (callers match fragments)."""
    for ok, message in checks:
        if not ok:
            raise ValueError(message)


class _ByteTables:
    """The expanded look-up tables of one layer's decode tables (128 KiB per kv head), built
    once by :func:`prepare_runtime_qpoints` and handed to every launch of that layer."""

    __slots__ = ("tables", "k_version", "v_version", "v_ref")

    def __init__(self, tables, k, v):
        self.tables, self.k_version, self.v_version, self.v_ref = tables, k._version, v._version, v


def _build_byte_tables(k_lane_major: torch.Tensor, v_code_major: torch.Tensor) -> torch.Tensor:
    heads_kv = int(k_lane_major.shape[0])
    with torch.cuda.device(k_lane_major.device):
        nbytes = int(_lib.load().bkv_decode_tables_bytes(heads_kv))
        tables = torch.empty((nbytes,), dtype=torch.uint8, device=k_lane_major.device)
        _lib.call(
            "bkv_decode_tables_sm100", k_lane_major.data_ptr(), v_code_major.data_ptr(),
            _lib.dtype_code(k_lane_major.dtype), heads_kv, _lib.FLAG_KLEVELS_LANE_MAJOR,
            tables.data_ptr(), nbytes, _lib.current_stream(k_lane_major.device),
        )
    return tables


def _byte_tables_of(k_lane_major: torch.Tensor, v_code_major: torch.Tensor) -> Optional[torch.Tensor]:
    """Tables attached by :func:`prepare_runtime_qpoints`, if they still describe these two
    tensors (same objects, not modified since); None makes the kernel build its own."""
    held = getattr(k_lane_major, "_bkv_byte_tables", None)
    if (
        held is None
        or held.v_ref is not v_code_major
        or held.k_version != k_lane_major._version
        or held.v_version != v_code_major._version
    ):
        return None
    return held.tables


def prepare_runtime_qpoints(
    q_points_k: torch.Tensor,
    q_points_v: torch.Tensor,
    *,
    heads_kv: int,
    storage_dtype: torch.dtype = torch.float16,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Decode-side level tables, once per layer: K as ``(Hkv, 16, 4)`` (level-major, group
    minor), V as ``(Hkv, 4, 16)``, both 16-bit — the shapes of the reference launcher
    (``beyond_mixed_decode_runtime.py:92-134``).  On a CUDA device the byte-indexed look-up
    tables of the decode kernel are expanded here too and travel with the K tensor."""
    if storage_dtype not in _DTYPE_NAMES:
        raise TypeError("runtime qpoints must use 16-bit fp16 or bf16 storage")
    groups = _HEAD_DIM // _GROUP_SIZE
    expected = int(heads_kv) * groups

    def grouped(table: torch.Tensor, label: str) -> torch.Tensor:
        _first_failure((
            (table.numel() == expected * 16,
             f"{label} qpoints require {expected} independent 16-point tables, got {table.numel()} values"),
            (table.ndim != 2 or tuple(table.shape) == (expected, 16),
             f"{label} qpoints must have shape ({expected}, 16), got {tuple(table.shape)}"),
            (table.ndim in (2, 3), f"{label} qpoints must be rank 2 or 3"),
        ))
        return table.reshape(int(heads_kv), groups, 16)

    k_lane_major = grouped(q_points_k, "K").permute(0, 2, 1).to(dtype=storage_dtype).contiguous()
    v_code_major = grouped(q_points_v, "V").to(dtype=storage_dtype).contiguous()
    if k_lane_major.is_cuda and v_code_major.is_cuda and not torch.cuda.is_current_stream_capturing():
        k_lane_major._bkv_byte_tables = _ByteTables(_build_byte_tables(k_lane_major, v_code_major), k_lane_major, v_code_major)
    return k_lane_major, v_code_major


def _sm_count(device: torch.device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    with _LOCK:
        if index not in _SM_COUNT:
            _SM_COUNT[index] = torch.cuda.get_device_properties(index).multi_processor_count
        return _SM_COUNT[index]


def persistent_schedule_supported(*, batch_size: int, physical_pages: int, heads_q: int, heads_kv: int) -> bool:
    """Limits of ``bkv_decode_stream_sm100``: at most 16384 requests per launch, page ids of
    26 bits and 2^20 (kv head x query-head quad, request) pairs; larger buckets use the split grid."""
    quads = (heads_q // heads_kv + 3) // 4
    return batch_size <= 16384 and physical_pages <= (1 << 26) and heads_kv * quads * batch_size <= (1 << 20)


def make_runtime_spec(
    *,
    q: torch.Tensor,
    cache: torch.Tensor,
    layout: PagedLayout,
    block_table: torch.Tensor,
    heads_q: int,
    max_seq_len: int,
    num_splits: int = 0,
    qpoint_dtype: torch.dtype = torch.float16,
    wait_for_pdl_writer: bool = False,
) -> DecodeRuntimeSpec:
    """Validate a launch bucket and freeze its launch plan (reference :137-302).

    ``num_splits <= 0`` leaves the schedule to the library: the persistent kernel (no split
    count) when the bucket fits its limits, else the split grid with the count the launch
    policy picks.  ``num_splits >= 1`` asks for the split grid with exactly that count."""
    if not q.is_cuda or not cache.is_cuda or not block_table.is_cuda:
        raise ValueError("q, packed cache, and block_table must be CUDA tensors")
    if torch.cuda.get_device_capability(q.device)[0] != 10:
        raise RuntimeError("the sm_100a packed-decode launcher requires a B200-class GPU (compute capability 10.x)")
    model_dtype = _dtype_name(q.dtype)
    qpoint_dtype_name = _dtype_name(qpoint_dtype)
    page_size = int(layout.block_size)
    heads_kv = int(layout.num_kv_heads)
    _first_failure((
        (page_size in SUPPORTED_PAGE_SIZES, "packed cache block_size must be 16, 32, 64 or 128"),
        (layout.code_layout == CODE_LAYOUT_HND_TOKEN_WORD and layout.abi_version == 2,
         "packed cache must use HND token-major ABI v2"),
        (layout.v_stats_group_major, "packed cache V statistics must retain PV group-major order"),
        (layout.bits == 4 and layout.k_group_size == _GROUP_SIZE and layout.v_group_size == _GROUP_SIZE
         and layout.head_dim == _HEAD_DIM, "launcher requires independent K/V Int4-G32-D128 cache"),
        (cache.dtype == torch.int32 and cache.ndim == 2 and cache.is_contiguous(),
         "cache must be contiguous (physical_pages, block_i32) int32"),
        (cache.ndim == 2 and int(cache.shape[1]) == int(layout.block_i32),
         "cache row stride does not match PagedLayout.block_i32"),
        (block_table.dtype == torch.int32 and block_table.ndim == 2, "block_table must be a rank-2 int32 CUDA tensor"),
        (block_table.ndim == 2 and block_table.stride(1) == 1, "block_table must be contiguous within each request row"),
        (max_seq_len > 0 and max_seq_len % page_size == 0,
         f"max_seq_len must be a positive multiple of page_size={page_size}"),
        (block_table.ndim == 2 and max_seq_len // page_size <= int(block_table.shape[1]),
         "launch bucket exceeds the block-table capacity"),
        (q.ndim == 3 and tuple(q.shape[1:]) == (int(heads_q), _HEAD_DIM), "q must have shape (B, Hq, D128)"),
        (q.ndim == 3 and int(q.shape[0]) > 0, "q decode batch must be non-empty"),
        (q.ndim == 3 and int(q.stride(2)) == 1 and int(q.stride(1)) == _HEAD_DIM,
         "q must be contiguous within each attention head"),
        (q.ndim == 3 and int(q.stride(0)) >= int(heads_q) * _HEAD_DIM, "q batch stride overlaps adjacent decode rows"),
        (int(heads_q) % heads_kv == 0, "heads_q must be divisible by heads_kv"),
        (int(heads_q) // heads_kv in (1, 2, 4, 8), "heads_q / heads_kv must be 1, 2, 4 or 8"),
    ))
    logical_pages = max_seq_len // page_size
    batch_size = int(q.shape[0])
    persistent = num_splits <= 0 and persistent_schedule_supported(
        batch_size=batch_size, physical_pages=int(cache.shape[0]), heads_q=int(heads_q), heads_kv=heads_kv)
    plan = None
    if persistent:
        num_splits = 1
    elif num_splits <= 0:
        plan = select_decode_launch_plan(
            tiles=logical_pages, batch=batch_size, heads_kv=heads_kv, sm_count=_sm_count(q.device),
            model_dtype=model_dtype, page_size=page_size,
        )
        num_splits = plan.splits
    if not 1 <= int(num_splits) <= 32:
        raise ValueError("num_splits must be in [1, 32]")
    reduction_kind = normalize_reduction_kind(
        os.environ.get("BEYOND_SM100_REDUCTION_KIND", os.environ.get("BEYOND_SM103_REDUCTION_KIND", "auto"))
    )
    return DecodeRuntimeSpec(
        device_index=q.device.index if q.device.index is not None else torch.cuda.current_device(),
        model_dtype=model_dtype,
        qpoint_dtype=qpoint_dtype_name,
        batch_size=batch_size,
        heads_q=int(heads_q),
        heads_kv=heads_kv,
        max_seq_len=int(max_seq_len),
        page_size=page_size,
        num_splits=int(num_splits),
        physical_pages=int(cache.shape[0]),
        page_table_stride=int(block_table.stride(0)),
        packed_page_stride_i32=int(layout.block_i32),
        q_batch_stride=int(q.stride(0)),
        kv_stage_cap=KV_STAGE_CAP,
        cvt_stage_cap=CVT_STAGE_CAP,
        reduction_kind=reduction_kind,
        cluster_reduction=False,
        task_major_grid=False,
        direct_smem_store=False,
        wait_for_pdl_writer=bool(wait_for_pdl_writer),
        persistent=persistent,
    )


def allocate_runtime_workspace(spec: DecodeRuntimeSpec, *, device: torch.device) -> dict[str, torch.Tensor]:
    """Allocate the workspace of a bucket once, before any CUDA-graph capture (reference
    :305-324).  A split-grid bucket gets the three float32 partial tensors; a persistent
    bucket gets the schedule's scratch under ``"stream"`` (its size depends on the device
    only) and empty partial tensors, since nothing would read them."""
    splits = 0 if spec.persistent else spec.num_splits
    partial_shape = (splits, spec.batch_size, spec.heads_q, 1, _HEAD_DIM)
    ws = {
        "o_partial": torch.empty(partial_shape, dtype=torch.float32, device=device),
        "m_partial": torch.empty(partial_shape[:-1], dtype=torch.float32, device=device),
        "l_partial": torch.empty(partial_shape[:-1], dtype=torch.float32, device=device),
    }
    if spec.persistent:
        ws["stream"] = _lib.stream_workspace(torch.device(device))
    return ws


def _validate_launch_tensors(*, spec, q, out, block_table, seq_lens, k_qpoints_lane_major, v_qpoints_code_major, workspace) -> None:
    expected_shape = (spec.batch_size, spec.heads_q, _HEAD_DIM)
    expected_q = spec.batch_size * spec.heads_q * _HEAD_DIM
    groups = _HEAD_DIM // _GROUP_SIZE
    expected_k, expected_v = (spec.heads_kv, 16, groups), (spec.heads_kv, groups, 16)
    _first_failure((
        (tuple(q.shape) == expected_shape and int(q.stride(2)) == 1 and int(q.stride(1)) == _HEAD_DIM
         and int(q.stride(0)) == spec.q_batch_stride, "q shape or fused-QKV batch stride changed after compilation"),
        (out.dtype == q.dtype and out.is_contiguous() and out.numel() == expected_q,
         "out must match the contiguous dense q bucket"),
        (block_table.dtype == torch.int32 and block_table.stride(1) == 1,
         "block_table must retain the compiled int32 row layout"),
        (int(block_table.stride(0)) == spec.page_table_stride, "block_table row stride changed after compilation"),
        (seq_lens.dtype == torch.int32 and seq_lens.is_contiguous(), "seq_lens must be contiguous int32"),
        (seq_lens.numel() >= spec.batch_size, "seq_lens is shorter than the decode batch"),
        (tuple(k_qpoints_lane_major.shape) == expected_k, f"K runtime qpoints must have shape {expected_k}"),
        (tuple(v_qpoints_code_major.shape) == expected_v, f"V runtime qpoints must have shape {expected_v}"),
        (k_qpoints_lane_major.is_contiguous() and v_qpoints_code_major.is_contiguous()
         and k_qpoints_lane_major.dtype == v_qpoints_code_major.dtype
         and _DTYPE_NAMES.get(k_qpoints_lane_major.dtype) == spec.qpoint_dtype,
         "K/V qpoints must be contiguous and share the compiled 16-bit dtype"),
    ))
    if spec.persistent:
        scratch = workspace.get("stream")
        if scratch is None or scratch.dtype != torch.uint8 or not scratch.is_contiguous():
            raise ValueError("stream workspace is missing: allocate it with allocate_runtime_workspace")
    elif spec.num_splits > 1:
        stats_numel = spec.num_splits * spec.batch_size * spec.heads_q
        partial = workspace.get("o_partial")
        _first_failure((
            (partial is not None and partial.dtype == torch.float32 and partial.is_contiguous()
             and partial.numel() >= spec.num_splits * expected_q, "o_partial workspace is missing or undersized"),
        ))
        for name in ("m_partial", "l_partial"):
            value = workspace.get(name)
            if value is None or value.dtype != torch.float32 or not value.is_contiguous() or value.numel() < stats_numel:
                raise ValueError(f"{name} workspace is missing or undersized")


def run_nonuniform_decode(
    *,
    spec: DecodeRuntimeSpec,
    q: torch.Tensor,
    cache: torch.Tensor,
    layout: PagedLayout,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    k_qpoints_lane_major: torch.Tensor,
    v_qpoints_code_major: torch.Tensor,
    out: torch.Tensor,
    workspace: dict[str, torch.Tensor],
    softmax_scale: float,
    stat_dtype: Optional[torch.dtype] = None,
    out_f32: Optional[torch.Tensor] = None,
    loader: int = 0,
) -> torch.Tensor:
    """Launch one dense single-token decode bucket on the current stream
    (reference :520-612).  No allocation, no host synchronisation.  ``loader`` (persistent
    buckets only) selects how tiles are brought into shared memory: 0 = 16-byte asynchronous
    copies, 1 = tensor copies."""
    _validate_launch_tensors(
        spec=spec, q=q, out=out, block_table=block_table, seq_lens=seq_lens,
        k_qpoints_lane_major=k_qpoints_lane_major, v_qpoints_code_major=v_qpoints_code_major,
        workspace=workspace,
    )
    if int(cache.shape[0]) != spec.physical_pages or int(cache.shape[1]) != spec.packed_page_stride_i32:
        raise ValueError("packed cache allocation changed after compilation")
    if out_f32 is not None and (out_f32.dtype != torch.float32 or not out_f32.is_contiguous() or out_f32.numel() != out.numel()):
        raise ValueError("out_f32 must be a contiguous float32 tensor of the output size")
    stat = stat_dtype if stat_dtype is not None else q.dtype
    flags = _lib.FLAG_KLEVELS_LANE_MAJOR | (_lib.FLAG_PDL_WAIT if spec.wait_for_pdl_writer else 0)
    if spec.persistent:
        scratch = workspace["stream"]
        _lib.call(
            "bkv_decode_stream_sm100",
            q.data_ptr(), spec.q_batch_stride, _lib.dtype_code(q.dtype),
            cache.data_ptr(), spec.physical_pages, spec.packed_page_stride_i32, spec.page_size,
            spec.heads_kv, _lib.dtype_code(stat),
            block_table.data_ptr(), spec.page_table_stride, seq_lens.data_ptr(),
            k_qpoints_lane_major.data_ptr(), v_qpoints_code_major.data_ptr(),
            _lib.dtype_code(k_qpoints_lane_major.dtype),
            out.data_ptr(), _lib.dtype_code(out.dtype), _lib.ptr(out_f32),
            scratch.data_ptr(), int(scratch.numel()),
            _lib.ptr(_byte_tables_of(k_qpoints_lane_major, v_qpoints_code_major)),
            spec.batch_size, spec.heads_q, spec.max_seq_len,
            float(softmax_scale), flags, int(loader), _lib.current_stream(q.device),
        )
        if os.environ.get("BEYOND_SM100_CHECK_STATUS") == "1" and not torch.cuda.is_current_stream_capturing():
            check_device_status()
        return out
    if loader:
        raise ValueError("the tile loader is a choice of the persistent schedule; this bucket uses the split grid")
    multi = spec.num_splits > 1
    _lib.call(
        "bkv_decode_sm100",
        q.data_ptr(), spec.q_batch_stride, _lib.dtype_code(q.dtype),
        cache.data_ptr(), spec.physical_pages, spec.packed_page_stride_i32, spec.page_size,
        spec.heads_kv, _lib.dtype_code(stat),
        block_table.data_ptr(), spec.page_table_stride, seq_lens.data_ptr(),
        k_qpoints_lane_major.data_ptr(), v_qpoints_code_major.data_ptr(),
        _lib.dtype_code(k_qpoints_lane_major.dtype),
        out.data_ptr(), _lib.dtype_code(out.dtype), _lib.ptr(out_f32),
        workspace["o_partial"].data_ptr() if multi else None,
        workspace["m_partial"].data_ptr() if multi else None,
        workspace["l_partial"].data_ptr() if multi else None,
        spec.num_splits, spec.batch_size, spec.heads_q, spec.max_seq_len,
        float(softmax_scale), flags, _lib.current_stream(q.device),
    )
    return out


_STATUS_TEXT = {
    2: "a bounded wait inside the decode kernel gave up (a copy into shared memory never completed); "
       "the outputs of that launch are incomplete and its workspace must be prepared again",
    3: "the decode kernel found its shared memory at an unexpected address and did nothing",
}


def check_device_status() -> None:
    """Read (and clear) the device-side status word of the decode kernels and raise ``BkvError``
    when a launch since the last check reported a failure.  The kernels never hang or trap: a wait
    that cannot complete runs into its time limit, sets this word and lets the launch finish, so the
    host has to look.  Synchronises the device - call it between steps, not inside a capture.
    ``run_nonuniform_decode`` calls it after every launch when ``BEYOND_SM100_CHECK_STATUS=1``
    (a debugging aid; it serialises host and device)."""
    import ctypes

    status = ctypes.c_int(0)
    _lib.call("bkv_decode_device_status", ctypes.byref(status))
    if status.value != 0:
        raise _lib.BkvError("bkv_decode_device_status", status.value,
                            _STATUS_TEXT.get(status.value, "unknown device status"))


def clear_compiled_runtime_cache() -> None:
    """Kept for interface parity (reference :615-620): nothing is JIT-compiled here,
    so there is nothing to drop; the capture-time refusal is preserved."""
    if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
        raise RuntimeError("cannot clear the decode compile cache during CUDA Graph capture")
