"""Graph-safe launcher of the B200 packed decode attention kernel.

Mirror of the reference launcher ``quant/fa4_cute/beyond_mixed_decode_runtime.py``:
``DecodeRuntimeSpec``, ``prepare_runtime_qpoints``, ``make_runtime_spec``,
``allocate_runtime_workspace``, ``run_nonuniform_decode`` and
``clear_compiled_runtime_cache`` keep their names, arguments and error types.
Instead of JIT-compiling a CuTe DSL kernel per launch bucket, every call goes to the
pre-built sm_100a library through the C ABI (``bkv_decode_sm100``): nothing is
compiled or allocated at launch, so a launch is capturable without pre-warming.

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
    conversion_stage_cap,
    normalize_reduction_kind,
    packed_kv_stage_cap,
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
    ``beyond_mixed_decode_runtime.py:43-73``); hashable, used as a workspace key."""

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

    @property
    def pages_per_split(self) -> int:
        return scheduled_pages_per_split(tiles=self.max_seq_len // self.page_size, splits=self.num_splits)


def _dtype_name(dtype: torch.dtype) -> str:
    if dtype == torch.float16:
        return "fp16"
    if dtype == torch.bfloat16:
        return "bf16"
    raise TypeError(f"expected fp16 or bf16, got {dtype}")


def _torch_dtype(name: str) -> torch.dtype:
    if name == "fp16":
        return torch.float16
    if name == "bf16":
        return torch.bfloat16
    raise ValueError(f"unsupported dtype name {name!r}")


def prepare_runtime_qpoints(
    q_points_k: torch.Tensor,
    q_points_v: torch.Tensor,
    *,
    heads_kv: int,
    storage_dtype: torch.dtype = torch.float16,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Decode-side level tables: K as ``(Hkv, 16, 4)`` (level-major, group minor),
    V as ``(Hkv, 4, 16)``, both 16-bit — the shapes of the reference launcher
    (``beyond_mixed_decode_runtime.py:92-134``)."""
    if storage_dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("runtime qpoints must use 16-bit fp16 or bf16 storage")
    groups = _HEAD_DIM // _GROUP_SIZE
    expected = int(heads_kv) * groups

    def grouped(table: torch.Tensor, label: str) -> torch.Tensor:
        if table.numel() != expected * 16:
            raise ValueError(
                f"{label} qpoints require {expected} independent 16-point tables, got {table.numel()} values"
            )
        if table.ndim == 2 and tuple(table.shape) != (expected, 16):
            raise ValueError(f"{label} qpoints must have shape ({expected}, 16), got {tuple(table.shape)}")
        if table.ndim not in (2, 3):
            raise ValueError(f"{label} qpoints must be rank 2 or 3")
        return table.reshape(int(heads_kv), groups, 16)

    k_lane_major = grouped(q_points_k, "K").permute(0, 2, 1).to(dtype=storage_dtype).contiguous()
    v_code_major = grouped(q_points_v, "V").to(dtype=storage_dtype).contiguous()
    return k_lane_major, v_code_major


def _sm_count(device: torch.device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    with _LOCK:
        if index not in _SM_COUNT:
            _SM_COUNT[index] = torch.cuda.get_device_properties(index).multi_processor_count
        return _SM_COUNT[index]


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
    """Validate a launch bucket and freeze its launch plan (reference :137-302)."""
    if not q.is_cuda or not cache.is_cuda or not block_table.is_cuda:
        raise ValueError("q, packed cache, and block_table must be CUDA tensors")
    if torch.cuda.get_device_capability(q.device)[0] != 10:
        raise RuntimeError("the sm_100a packed-decode launcher requires a B200-class GPU (compute capability 10.x)")
    model_dtype = _dtype_name(q.dtype)
    qpoint_dtype_name = _dtype_name(qpoint_dtype)
    page_size = int(layout.block_size)
    if page_size not in SUPPORTED_PAGE_SIZES:
        raise ValueError("packed cache block_size must be 16, 32, 64 or 128")
    if layout.code_layout != CODE_LAYOUT_HND_TOKEN_WORD or layout.abi_version != 2:
        raise ValueError("packed cache must use HND token-major ABI v2")
    if not layout.v_stats_group_major:
        raise ValueError("packed cache V statistics must retain PV group-major order")
    if (
        layout.bits != 4
        or layout.k_group_size != _GROUP_SIZE
        or layout.v_group_size != _GROUP_SIZE
        or layout.head_dim != _HEAD_DIM
    ):
        raise ValueError("launcher requires independent K/V Int4-G32-D128 cache")
    if cache.dtype != torch.int32 or cache.ndim != 2 or not cache.is_contiguous():
        raise ValueError("cache must be contiguous (physical_pages, block_i32) int32")
    if int(cache.shape[1]) != int(layout.block_i32):
        raise ValueError("cache row stride does not match PagedLayout.block_i32")
    if block_table.dtype != torch.int32 or block_table.ndim != 2:
        raise ValueError("block_table must be a rank-2 int32 CUDA tensor")
    if block_table.stride(1) != 1:
        raise ValueError("block_table must be contiguous within each request row")
    if max_seq_len <= 0 or max_seq_len % page_size:
        raise ValueError(f"max_seq_len must be a positive multiple of page_size={page_size}")
    logical_pages = max_seq_len // page_size
    if logical_pages > int(block_table.shape[1]):
        raise ValueError("launch bucket exceeds the block-table capacity")
    if q.ndim != 3 or tuple(q.shape[1:]) != (int(heads_q), _HEAD_DIM):
        raise ValueError("q must have shape (B, Hq, D128)")
    batch_size = int(q.shape[0])
    if batch_size <= 0:
        raise ValueError("q decode batch must be non-empty")
    if int(q.stride(2)) != 1 or int(q.stride(1)) != _HEAD_DIM:
        raise ValueError("q must be contiguous within each attention head")
    q_batch_stride = int(q.stride(0))
    if q_batch_stride < int(heads_q) * _HEAD_DIM:
        raise ValueError("q batch stride overlaps adjacent decode rows")
    if int(heads_q) % int(layout.num_kv_heads):
        raise ValueError("heads_q must be divisible by heads_kv")
    if int(heads_q) // int(layout.num_kv_heads) not in (1, 2, 4, 8):
        raise ValueError("heads_q / heads_kv must be 1, 2, 4 or 8")

    plan = None
    if num_splits <= 0:
        plan = select_decode_launch_plan(
            tiles=logical_pages,
            batch=batch_size,
            heads_kv=int(layout.num_kv_heads),
            sm_count=_sm_count(q.device),
            model_dtype=model_dtype,
            page_size=page_size,
        )
        num_splits = plan.splits
    if not 1 <= int(num_splits) <= 32:
        raise ValueError("num_splits must be in [1, 32]")
    pages_per_split = scheduled_pages_per_split(tiles=logical_pages, splits=int(num_splits))
    reduction_kind = normalize_reduction_kind(
        os.environ.get("BEYOND_SM100_REDUCTION_KIND", os.environ.get("BEYOND_SM103_REDUCTION_KIND", "auto"))
    )
    return DecodeRuntimeSpec(
        device_index=q.device.index if q.device.index is not None else torch.cuda.current_device(),
        model_dtype=model_dtype,
        qpoint_dtype=qpoint_dtype_name,
        batch_size=batch_size,
        heads_q=int(heads_q),
        heads_kv=int(layout.num_kv_heads),
        max_seq_len=int(max_seq_len),
        page_size=page_size,
        num_splits=int(num_splits),
        physical_pages=int(cache.shape[0]),
        page_table_stride=int(block_table.stride(0)),
        packed_page_stride_i32=int(layout.block_i32),
        q_batch_stride=q_batch_stride,
        kv_stage_cap=plan.kv_stage_cap if plan is not None else packed_kv_stage_cap(pages_per_split=pages_per_split),
        cvt_stage_cap=plan.cvt_stage_cap
        if plan is not None
        else conversion_stage_cap(splits=int(num_splits), pages_per_split=pages_per_split, model_dtype=model_dtype),
        reduction_kind=reduction_kind,
        cluster_reduction=False,
        task_major_grid=False,
        direct_smem_store=False,
        wait_for_pdl_writer=bool(wait_for_pdl_writer),
    )


def allocate_runtime_workspace(spec: DecodeRuntimeSpec, *, device: torch.device) -> dict[str, torch.Tensor]:
    """Allocate the split workspace once, before any CUDA-graph capture
    (reference :305-324).  All three tensors are float32."""
    partial_shape = (spec.num_splits, spec.batch_size, spec.heads_q, 1, _HEAD_DIM)
    ws = {
        "o_partial": torch.empty(partial_shape, dtype=torch.float32, device=device),
        "m_partial": torch.empty(partial_shape[:-1], dtype=torch.float32, device=device),
        "l_partial": torch.empty(partial_shape[:-1], dtype=torch.float32, device=device),
    }
    if stream_schedule_supported(spec):
        # scratch of the persistent schedule (partials of requests cut between workers);
        # its size depends on the device only
        with torch.cuda.device(device):
            nbytes = int(_lib.load().bkv_decode_stream_workspace_bytes())
        ws["stream"] = torch.empty((nbytes,), dtype=torch.uint8, device=device)
    return ws


def stream_schedule_supported(spec: DecodeRuntimeSpec) -> bool:
    """The persistent schedule (``bkv_decode_stream_sm100``) plans at most 16384 requests
    per launch and packs page ids into 26 bits; larger buckets use the split grid."""
    return spec.batch_size <= 16384 and spec.physical_pages <= (1 << 26)


def _validate_launch_tensors(*, spec, q, out, block_table, seq_lens, k_qpoints_lane_major, v_qpoints_code_major, workspace) -> None:
    expected_shape = (spec.batch_size, spec.heads_q, _HEAD_DIM)
    expected_q = spec.batch_size * spec.heads_q * _HEAD_DIM
    if (
        tuple(q.shape) != expected_shape
        or int(q.stride(2)) != 1
        or int(q.stride(1)) != _HEAD_DIM
        or int(q.stride(0)) != spec.q_batch_stride
    ):
        raise ValueError("q shape or fused-QKV batch stride changed after compilation")
    if out.dtype != q.dtype or not out.is_contiguous() or out.numel() != expected_q:
        raise ValueError("out must match the contiguous dense q bucket")
    if block_table.dtype != torch.int32 or block_table.stride(1) != 1:
        raise ValueError("block_table must retain the compiled int32 row layout")
    if int(block_table.stride(0)) != spec.page_table_stride:
        raise ValueError("block_table row stride changed after compilation")
    if seq_lens.dtype != torch.int32 or not seq_lens.is_contiguous():
        raise ValueError("seq_lens must be contiguous int32")
    if seq_lens.numel() < spec.batch_size:
        raise ValueError("seq_lens is shorter than the decode batch")
    groups = _HEAD_DIM // _GROUP_SIZE
    expected_k = (spec.heads_kv, 16, groups)
    expected_v = (spec.heads_kv, groups, 16)
    if tuple(k_qpoints_lane_major.shape) != expected_k:
        raise ValueError(f"K runtime qpoints must have shape {expected_k}")
    if tuple(v_qpoints_code_major.shape) != expected_v:
        raise ValueError(f"V runtime qpoints must have shape {expected_v}")
    if (
        not k_qpoints_lane_major.is_contiguous()
        or not v_qpoints_code_major.is_contiguous()
        or k_qpoints_lane_major.dtype != v_qpoints_code_major.dtype
        or _dtype_name(k_qpoints_lane_major.dtype) != spec.qpoint_dtype
    ):
        raise ValueError("K/V qpoints must be contiguous and share the compiled 16-bit dtype")
    if spec.num_splits > 1:
        stats_numel = spec.num_splits * spec.batch_size * spec.heads_q
        partial = workspace.get("o_partial")
        if partial is None or partial.dtype != torch.float32 or not partial.is_contiguous() or partial.numel() < spec.num_splits * expected_q:
            raise ValueError("o_partial workspace is missing or undersized")
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
    variant: int = 0,
) -> torch.Tensor:
    """Launch one dense single-token decode bucket on the current stream
    (reference :520-612).  No allocation, no host synchronisation."""
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
    use_stream = (variant == 0 or variant >= 40) and "stream" in workspace and stream_schedule_supported(spec)
    if use_stream:
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
            spec.batch_size, spec.heads_q, spec.max_seq_len,
            float(softmax_scale), flags, int(variant), _lib.current_stream(q.device),
        )
        return out
    if variant >= 40:
        raise ValueError("the persistent schedule was requested but this bucket does not support it")
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
        float(softmax_scale), flags, int(variant), _lib.current_stream(q.device),
    )
    return out


def clear_compiled_runtime_cache() -> None:
    """Kept for interface parity (reference :615-620): nothing is JIT-compiled here,
    so there is nothing to drop; the capture-time refusal is preserved."""
    if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
        raise RuntimeError("cannot clear the decode compile cache during CUDA Graph capture")
