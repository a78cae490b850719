"""Packed 4-bit / group-32 KV cache ops on B200 — host side.

Mirror of the reference module ``quant/beyond_cute.py`` for the serving hot path:
same public names, argument meaning and error behaviour, with every device
computation done by the hand-written sm_100a kernels of ``libbkv_sm100.so``.
There is no Triton path and no torch fallback: a call that the CUDA kernels cannot
serve raises.

Kept from the reference interface (file:line in the reference project):

* constants ``PACK_CHUNK`` … ``SUPPORTED_CODE_LAYOUTS`` (``quant/beyond_cute.py:53-58``)
* ``make_uniform_q_points`` / ``make_uniform_thresholds`` (:75-93)
* ``prepare_qpoints_and_thresholds`` (:116-195)
* ``pack_codes`` / ``unpack_codes`` (:358-431) — format helpers, any device
* ``PackedK`` / ``PackedV`` (:290-335), ``quantize_k`` / ``quantize_v`` (:439-486, :525-584),
  ``dequantize_k`` / ``dequantize_v`` (:489-517, :587-616) — here evaluated by the encode and
  read-back kernels (CUDA tensors only)
* ``PagedLayout.build`` / ``build_hnd`` (:629-786)
* ``write_tokens_to_paged_cache`` (:2147-2207)
* ``dequantize_paged_kv_to_dense`` (:1703-1856)
* ``read_request_from_paged_cache`` (:2210-2395) — here served by the read-back kernel

A CPU restatement of the same arithmetic exists as test infrastructure outside this package;
nothing here falls back to it.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _lib

PACK_CHUNK = 32
SUPPORTED_BITS = (4,)
SUPPORTED_GROUP_SIZES = (32,)
CODE_LAYOUT_HEAD_WORD_TOKEN = "head_word_token"
CODE_LAYOUT_HND_TOKEN_WORD = "hnd_token_word"
SUPPORTED_CODE_LAYOUTS = (CODE_LAYOUT_HEAD_WORD_TOKEN, CODE_LAYOUT_HND_TOKEN_WORD)

_HEAD_DIM = 128
_UNIFORM_TABLES: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}


# --------------------------------------------------------------------------- tables
def make_uniform_q_points(num_bits: int) -> torch.Tensor:
    """Uniform levels ``i / 15`` evaluated in Python floats, then float32; not
    ``linspace``, which differs by one ULP at some entries (reference :75-88)."""
    if int(num_bits) != 4:
        raise ValueError("Beyond inference keeps only 4-bit quantization")
    return torch.tensor([i / 15 for i in range(16)], dtype=torch.float32)


def make_uniform_thresholds(q_points: torch.Tensor) -> torch.Tensor:
    """Mid-points computed with a division by 2.0 (reference :91-93)."""
    return (q_points[:-1] + q_points[1:]) / 2.0


def _dev_key(device: torch.device) -> str:
    if device.type == "cuda":
        return f"cuda:{torch.cuda.current_device() if device.index is None else device.index}"
    return str(device)


def _storage_dtype(t: torch.Tensor) -> torch.dtype:
    return t.dtype if t.dtype in (torch.float16, torch.bfloat16) else torch.float32


def prepare_qpoints_and_thresholds(
    *,
    num_bits: int,
    device: torch.device,
    q_points: Optional[torch.Tensor],
    thresholds: Optional[torch.Tensor] = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Contiguous deployment tables on ``device``: 16-bit tables stay 16-bit,
    anything else becomes float32; the default is the fp16 uniform table whose
    thresholds are rounded from the float32 master mid-points (reference :116-195)."""
    if int(num_bits) != 4:
        raise ValueError("Beyond inference keeps only 4-bit quantization")
    device = torch.device(device)
    key = _dev_key(device)
    if q_points is None:
        if key not in _UNIFORM_TABLES:
            master = make_uniform_q_points(4)
            _UNIFORM_TABLES[key] = (
                master.to(device=device, dtype=torch.float16).contiguous(),
                make_uniform_thresholds(master).to(device=device, dtype=torch.float16).contiguous(),
            )
        qp, uniform_thr = _UNIFORM_TABLES[key]
    else:
        qp = q_points.to(device=device, dtype=_storage_dtype(q_points)).contiguous()
        uniform_thr = None
    if thresholds is not None:
        thr = thresholds.to(device=device, dtype=qp.dtype).contiguous()
        expected = tuple(qp.shape[:-1]) + (int(qp.shape[-1]) - 1,)
        if tuple(thr.shape) != expected:
            raise ValueError(f"thresholds shape {tuple(thr.shape)} != expected {expected}")
        return qp, thr
    if qp.dim() != 1:
        raise ValueError("thresholds are required for grouped q_points")
    if uniform_thr is not None:
        return qp, uniform_thr
    # mid-point thresholds of a caller's shared table: kept ON that tensor (with the version
    # they were derived from), never in a table keyed by its address, which a later tensor
    # could inherit
    held = getattr(qp, "_bkv_midpoints", None)
    if held is None or held[0] != qp._version:
        held = (qp._version, make_uniform_thresholds(qp.to(torch.float32)).to(dtype=qp.dtype).contiguous())
        qp._bkv_midpoints = held
    return qp, held[1]


def _validate_real_quant_params(num_bits: int, group_size: int) -> None:
    if int(num_bits) != 4:
        raise ValueError("real packed Beyond supports only 4-bit codes")
    if int(group_size) not in SUPPORTED_GROUP_SIZES:
        raise ValueError(f"group_size {group_size} not in {SUPPORTED_GROUP_SIZES}")


# --------------------------------------------------------------------------- nibble format
def pack_codes(codes: torch.Tensor, bits: int, pack_axis_first: bool = False) -> torch.Tensor:
    """``(..., 32)`` uint8 codes -> ``(..., 4)`` uint32 words, code ``i`` in bits
    ``4*(i%8)`` of word ``i//8`` (reference :358-395)."""
    if pack_axis_first:
        raise TypeError("pack_axis_first was removed from real 4-bit packing")
    if codes.dtype != torch.uint8:
        raise TypeError("codes must be uint8")
    _validate_real_quant_params(bits, int(codes.shape[-1]))
    c = codes.reshape(*codes.shape[:-1], 4, 8).to(torch.int64)
    shifts = torch.arange(0, 32, 4, device=codes.device, dtype=torch.int64)
    words = (c << shifts).sum(dim=-1)  # nibbles do not overlap, so sum == or
    return (words & 0xFFFFFFFF).to(torch.uint32)


def unpack_codes(packed: torch.Tensor, bits: int, num_codes: int, pack_axis_first: bool = False) -> torch.Tensor:
    """Inverse of :func:`pack_codes` (reference :398-431)."""
    if pack_axis_first:
        raise TypeError("pack_axis_first was removed from real 4-bit packing")
    _validate_real_quant_params(bits, num_codes)
    if packed.shape[-1] != 4:
        raise ValueError(f"packed shape tail {packed.shape[-1]} != words_per_group 4")
    w = packed.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(0, 32, 4, device=packed.device, dtype=torch.int64)
    c = (w.unsqueeze(-1) >> shifts) & 0xF
    return c.reshape(*packed.shape[:-1], 32).to(torch.uint8)


# --------------------------------------------------------------------------- page layout
@dataclass(frozen=True)
class PagedLayout:
    """Offsets, in 16-bit halves, of the four regions of one packed page; field
    names and values are those of the reference dataclass (reference :629-765)."""

    block_size: int
    num_kv_heads: int
    head_dim: int
    bits: int
    k_group_size: int
    v_group_size: int
    k_code_halves: int
    k_scale_halves: int
    k_min_halves: int
    v_code_halves: int
    v_scale_halves: int
    v_min_halves: int
    k_code_off: int
    k_scale_off: int
    k_min_off: int
    v_code_off: int
    v_scale_off: int
    v_min_off: int
    block_halves: int
    block_i32: int
    k_groups_per_block: int
    num_chunks_k: int
    num_chunks_v: int
    v_groups_per_token: int
    code_layout: str = CODE_LAYOUT_HEAD_WORD_TOKEN
    abi_version: int = 1
    stats_interleaved: bool = True
    v_stats_group_major: bool = True

    @classmethod
    def build(
        cls,
        block_size: int,
        num_kv_heads: int,
        head_dim: int,
        bits: int,
        k_group_size: int,
        v_group_size: int,
        code_layout: str = CODE_LAYOUT_HEAD_WORD_TOKEN,
    ) -> "PagedLayout":
        _validate_real_quant_params(bits, k_group_size)
        _validate_real_quant_params(bits, v_group_size)
        if code_layout not in SUPPORTED_CODE_LAYOUTS:
            raise ValueError(
                f"unsupported code_layout {code_layout!r}; expected one of {SUPPORTED_CODE_LAYOUTS}"
            )
        if head_dim % k_group_size != 0:
            raise ValueError(f"head_dim {head_dim} not divisible by k_group_size {k_group_size}")
        if head_dim % v_group_size != 0:
            raise ValueError(f"head_dim {head_dim} not divisible by v_group_size {v_group_size}")
        token_heads = int(num_kv_heads) * int(block_size)
        regions = []  # (name, halves) in page order
        for name, group in (("k", k_group_size), ("v", v_group_size)):
            groups = head_dim // group
            words_per_group = bits * group // 32
            regions.append((f"{name}_code", token_heads * groups * words_per_group * 2))
            regions.append((f"{name}_scale", token_heads * groups))
            regions.append((f"{name}_min", token_heads * groups))
        sizes, offsets, cursor = {}, {}, 0
        for name, halves in regions:
            sizes[name], offsets[name] = halves, cursor
            cursor += halves
        if cursor % 2:
            raise RuntimeError("page size is not a whole number of int32 words")
        return cls(
            block_size=block_size,
            num_kv_heads=num_kv_heads,
            head_dim=head_dim,
            bits=bits,
            k_group_size=k_group_size,
            v_group_size=v_group_size,
            k_code_halves=sizes["k_code"],
            k_scale_halves=sizes["k_scale"],
            k_min_halves=sizes["k_min"],
            v_code_halves=sizes["v_code"],
            v_scale_halves=sizes["v_scale"],
            v_min_halves=sizes["v_min"],
            k_code_off=offsets["k_code"],
            k_scale_off=offsets["k_scale"],
            k_min_off=offsets["k_min"],
            v_code_off=offsets["v_code"],
            v_scale_off=offsets["v_scale"],
            v_min_off=offsets["v_min"],
            block_halves=cursor,
            block_i32=cursor // 2,
            k_groups_per_block=head_dim // k_group_size,
            num_chunks_k=bits * k_group_size // 32,
            num_chunks_v=bits * v_group_size // 32,
            v_groups_per_token=head_dim // v_group_size,
            code_layout=code_layout,
            abi_version=2 if code_layout == CODE_LAYOUT_HND_TOKEN_WORD else 1,
            stats_interleaved=True,
            v_stats_group_major=True,
        )

    @classmethod
    def build_hnd(cls, block_size, num_kv_heads, head_dim, bits, k_group_size, v_group_size) -> "PagedLayout":
        """ABI v2: contiguous packed-D words inside each (head, token)."""
        return cls.build(
            block_size=block_size,
            num_kv_heads=num_kv_heads,
            head_dim=head_dim,
            bits=bits,
            k_group_size=k_group_size,
            v_group_size=v_group_size,
            code_layout=CODE_LAYOUT_HND_TOKEN_WORD,
        )


def _stat_dtype_from_model_dtype(dtype: torch.dtype) -> torch.dtype:
    if dtype in (torch.bfloat16, torch.float16):
        return dtype
    raise TypeError(f"Beyond stats require fp16/bf16 model dtype, got {dtype}")


# --------------------------------------------------------------------------- helpers
def _table_class(thr: torch.Tensor) -> tuple:
    """(sorted, binned) for a threshold tensor.

    sorted: every table is non-decreasing (the binary search is then identical to the reference's
    count).  binned: in addition every threshold is positive with the low four bits of its float32
    pattern clear (any 16-bit value) and every interval [e/512, (e+1)/512), e = 0..511, holds at
    most one threshold of a table, which lets large writes replace the search by one indexed
    look-up (tables that obey the 2^-9 minimum-gap rule of the reference's
    ``quantization/table_precision.py:19-24`` are of this kind).  The answer is kept on the tensor
    object itself, tagged with the tensor version it was computed for, so it can never be
    inherited by another table that the allocator later places at the same address.  Finding it
    out costs one device read; during stream capture an unclassified table is treated as
    unsorted and not binned (the counting search is always right, only slower)."""
    held = getattr(thr, "_bkv_sorted", None)
    if held is not None and held[0] == thr._version:
        return held[1]
    if thr.is_cuda and torch.cuda.is_current_stream_capturing():
        return (False, False)
    t = thr.float().reshape(-1, thr.shape[-1])
    is_sorted = t[:, 1:] >= t[:, :-1]
    # interval index of every threshold that can matter (those in [0, 1)); NaNs never count
    inside = (t >= 0) & (t < 1)
    bins = torch.where(inside, torch.floor(t * 512.0), torch.arange(t.shape[-1], device=t.device, dtype=t.dtype) - 1000.0)
    ordered = torch.sort(bins, dim=-1).values
    distinct = ordered[:, 1:] != ordered[:, :-1]
    plain = (t > 0).all() & ((t.contiguous().view(torch.int32) & 15) == 0).all()
    answers = torch.stack([is_sorted.all(), distinct.all() & plain]).tolist()
    known = (bool(answers[0]), bool(answers[0]) and bool(answers[1]))
    thr._bkv_sorted = (thr._version, known)
    return known


def _tables_sorted(thr: torch.Tensor) -> bool:
    return _table_class(thr)[0]


def _tables_binned(thr: torch.Tensor) -> bool:
    return _table_class(thr)[1]


def classify_tables(*thresholds: torch.Tensor) -> None:
    """Classify threshold tables now (one device read each), so that later writes through
    :func:`write_tokens_to_paged_cache` with these very tensors cost no host synchronisation."""
    for thr in thresholds:
        if thr is not None:
            _tables_sorted(thr)


def _layout_code(layout: PagedLayout) -> int:
    return (
        _lib.LAYOUT_HND_TOKEN_WORD
        if layout.code_layout == CODE_LAYOUT_HND_TOKEN_WORD
        else _lib.LAYOUT_HEAD_WORD_TOKEN
    )


def _writer_unsupported_reason(cache, layout, slot_mapping, k, v, k_dq_out, v_dq_out) -> Optional[str]:
    """The shape/device predicate of the reference writer (reference :1573-1616),
    returning why a call cannot be served instead of a bare False."""
    if not (cache.is_cuda and k.is_cuda and v.is_cuda and slot_mapping.is_cuda):
        return "cache, k, v and slot_mapping must be CUDA tensors"
    if cache.dtype != torch.int32 or cache.dim() != 2 or not cache.is_contiguous():
        return "cache must be a contiguous (pages, block_i32) int32 tensor"
    if k.dtype not in (torch.float16, torch.bfloat16, torch.float32) or v.dtype != k.dtype:
        return "k and v must share an fp16/bf16 (or fp32) dtype"
    if k.dim() != 3 or tuple(k.shape) != tuple(v.shape):
        return "k and v must both be (tokens, heads, head_dim)"
    if slot_mapping.dim() != 1 or slot_mapping.dtype not in (torch.int32, torch.int64):
        return "slot_mapping must be a 1-D int32/int64 tensor"
    if int(slot_mapping.numel()) != int(k.shape[0]):
        return "slot_mapping needs one entry per token"
    if (
        layout.bits != 4
        or layout.k_group_size != 32
        or layout.v_group_size != 32
        or layout.head_dim != _HEAD_DIM
        or layout.code_layout not in SUPPORTED_CODE_LAYOUTS
        or not layout.stats_interleaved
    ):
        return "only the 4-bit / group-32 / head_dim-128 page ABI is supported"
    if int(cache.shape[1]) != int(layout.block_i32):
        return "cache row length differs from layout.block_i32"
    if int(k.shape[1]) != int(layout.num_kv_heads) or int(k.shape[2]) != _HEAD_DIM:
        return "k/v head count or head_dim differs from the layout"
    if k.stride(2) != 1 or v.stride(2) != 1:
        return "k and v must be contiguous along head_dim"
    if (k_dq_out is None) != (v_dq_out is None):
        return "k_dq_out and v_dq_out must be given together"
    if k_dq_out is not None:
        for src, dst in ((k, k_dq_out), (v, v_dq_out)):
            if dst.device != src.device or dst.dtype != src.dtype or tuple(dst.shape) != tuple(src.shape):
                return "reconstruction outputs must match k/v in device, dtype and shape"
            if dst.stride(2) != 1:
                return "reconstruction outputs must be contiguous along head_dim"
    return None


def write_tokens_to_paged_cache(
    cache: torch.Tensor,
    layout: PagedLayout,
    block_table: torch.Tensor,
    slot_mapping: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    q_points_k: Optional[torch.Tensor] = None,
    q_points_v: Optional[torch.Tensor] = None,
    thresholds_k: Optional[torch.Tensor] = None,
    thresholds_v: Optional[torch.Tensor] = None,
    k_dq_out: Optional[torch.Tensor] = None,
    v_dq_out: Optional[torch.Tensor] = None,
    signal_pdl_dependents: bool = False,
    wait_for_pdl_predecessor: bool = False,
    require_fast: bool = False,
    stat_dtype: Optional[torch.dtype] = None,
) -> None:
    """Quantise, pack and scatter K/V rows into the packed page cache on the GPU.

    Same contract as the reference entry point (reference :2147-2207): ``cache`` (and
    ``k_dq_out`` / ``v_dq_out``, which may alias ``k`` / ``v``) are modified in place;
    ``block_table`` is unused; rows with ``slot < 0`` write nothing to the cache but
    are still reconstructed.  Codes and statistics are bit-identical to the reference
    quantiser ``quantize_k`` / ``quantize_v``.  The reference falls back to a torch
    oracle when its fused kernel cannot serve a call unless ``require_fast`` is set;
    this implementation has no fallback and raises ``RuntimeError`` in both cases.
    ``stat_dtype`` (extension) selects fp16/bf16 statistics independently of the input
    dtype; by default statistics use the model dtype as in the reference.
    ``wait_for_pdl_predecessor`` (extension) launches the writer as a programmatic dependent of
    the kernel in front of it on the stream: its set-up (tables) runs while that kernel drains and
    it waits for it before touching rows, slots or the cache - useful behind the kernel that
    produces K and V, or between the chunks of one long write.
    """
    del block_table, require_fast
    reason = _writer_unsupported_reason(cache, layout, slot_mapping, k, v, k_dq_out, v_dq_out)
    if reason is not None:
        raise RuntimeError(
            "Beyond production cache writes require the fused sm_100a writer; "
            f"the current device, dtype, layout, or shape is unsupported: {reason}."
        )
    if int(k.shape[0]) == 0:
        return
    if stat_dtype is None:
        stat_dtype = _stat_dtype_from_model_dtype(k.dtype)
    else:
        stat_dtype = _stat_dtype_from_model_dtype(stat_dtype)
    qp_k, thr_k = prepare_qpoints_and_thresholds(num_bits=4, device=k.device, q_points=q_points_k, thresholds=thresholds_k)
    qp_v, thr_v = prepare_qpoints_and_thresholds(num_bits=4, device=v.device, q_points=q_points_v, thresholds=thresholds_v)
    tables = int(layout.num_kv_heads) * 4
    for name, t, width in (("q_points_k", qp_k, 16), ("q_points_v", qp_v, 16), ("thresholds_k", thr_k, 15), ("thresholds_v", thr_v, 15)):
        if tuple(t.shape) not in {(width,), (tables, width)}:
            raise RuntimeError(
                "Beyond production cache writes require the fused sm_100a writer; "
                f"{name} has unsupported shape {tuple(t.shape)}."
            )
    if qp_k.dtype != qp_v.dtype:
        common = torch.float32
        qp_k, thr_k, qp_v, thr_v = (t.to(common) for t in (qp_k, thr_k, qp_v, thr_v))
    flags = _lib.FLAG_PDL_TRIGGER if signal_pdl_dependents else 0
    if wait_for_pdl_predecessor:
        # the launch may begin while the kernel in front of it on the stream drains; the writer reads
        # only its tables before it waits for that kernel
        flags |= _lib.FLAG_PDL_WAIT
    if not (_tables_sorted(thr_k) and _tables_sorted(thr_v)):
        flags |= _lib.FLAG_LINEAR_SEARCH
    elif _tables_binned(thr_k) and _tables_binned(thr_v):
        flags |= _lib.FLAG_BINNED_TABLES
    dq = k_dq_out is not None
    _lib.call(
        "bkv_encode_sm100",
        k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
        _lib.dtype_code(k.dtype),
        slot_mapping.data_ptr(), int(slot_mapping.dtype == torch.int64), slot_mapping.stride(0),
        int(k.shape[0]), int(layout.num_kv_heads),
        cache.data_ptr(), int(cache.shape[0]), int(cache.stride(0)), int(layout.block_size),
        _layout_code(layout), _lib.dtype_code(stat_dtype),
        thr_k.data_ptr(), thr_v.data_ptr(), qp_k.data_ptr(), qp_v.data_ptr(),
        _lib.dtype_code(qp_k.dtype), int(qp_k.dim() == 2), int(qp_v.dim() == 2),
        _lib.ptr(k_dq_out), _lib.ptr(v_dq_out),
        k_dq_out.stride(0) if dq else 0, k_dq_out.stride(1) if dq else 0,
        v_dq_out.stride(0) if dq else 0, v_dq_out.stride(1) if dq else 0,
        flags, _lib.current_stream(k.device),
    )


def _readback_tables(layout: PagedLayout, device, q_points_k, q_points_v):
    qp_k, _ = prepare_qpoints_and_thresholds(num_bits=4, device=device, q_points=q_points_k) if (
        q_points_k is None or q_points_k.dim() == 1
    ) else (q_points_k.to(device=device, dtype=_storage_dtype(q_points_k)).contiguous(), None)
    qp_v, _ = prepare_qpoints_and_thresholds(num_bits=4, device=device, q_points=q_points_v) if (
        q_points_v is None or q_points_v.dim() == 1
    ) else (q_points_v.to(device=device, dtype=_storage_dtype(q_points_v)).contiguous(), None)
    tables = int(layout.num_kv_heads) * 4
    if tuple(qp_k.shape) not in {(16,), (tables, 16)}:
        raise ValueError("K q_points do not match the packed HND tables")
    if tuple(qp_v.shape) not in {(16,), (tables, 16)}:
        raise ValueError("V q_points do not match the packed HND tables")
    if qp_k.dtype != qp_v.dtype:
        qp_k, qp_v = qp_k.float(), qp_v.float()
    return qp_k, qp_v


def dequantize_paged_kv_to_dense(
    cache: torch.Tensor,
    layout: PagedLayout,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    seq_start_loc: torch.Tensor,
    out_k: torch.Tensor,
    out_v: torch.Tensor,
    *,
    max_seq_len: int,
    q_points_k: Optional[torch.Tensor] = None,
    q_points_v: Optional[torch.Tensor] = None,
    stat_dtype: Optional[torch.dtype] = None,
) -> None:
    """Materialise a packed ABI-v2 batch into dense varlen K/V (reference :1703-1856).
    Unlike the reference (pages of 64/128 only) any page size is accepted; results
    are bit-identical to ``read_request_from_paged_cache``."""
    if not cache.is_cuda:
        raise RuntimeError("packed chunked-prefill dequantization requires CUDA")
    int32_on_cache = lambda t, rank: t.device == cache.device and t.dtype == torch.int32 and t.dim() == rank  # noqa: E731
    cache_abi_ok = (
        cache.dtype == torch.int32 and cache.dim() == 2 and cache.is_contiguous(),
        int32_on_cache(block_table, 2) and block_table.stride(-1) == 1,
        int32_on_cache(seq_lens, 1),
        int32_on_cache(seq_start_loc, 1) and int(seq_start_loc.numel()) == int(seq_lens.numel()) + 1,
        (layout.bits, layout.head_dim, layout.k_group_size, layout.v_group_size) == (4, _HEAD_DIM, 32, 32),
        layout.code_layout == CODE_LAYOUT_HND_TOKEN_WORD,
        cache.dim() == 2 and int(cache.shape[1]) == int(layout.block_i32),
    )
    if not all(cache_abi_ok):
        raise ValueError("unsupported packed chunked-prefill cache ABI")
    outputs_ok = (
        out_k.device == cache.device and out_v.device == cache.device,
        out_k.dtype in (torch.float16, torch.bfloat16, torch.float32) and out_v.dtype == out_k.dtype,
        out_k.dim() == 3 and tuple(out_v.shape) == tuple(out_k.shape),
        tuple(out_k.shape[1:]) == (layout.num_kv_heads, _HEAD_DIM),
        out_k.is_contiguous() and out_v.is_contiguous(),
    )
    if not all(outputs_ok):
        raise ValueError("dense chunked-prefill outputs must be contiguous FP16/BF16 HND tensors")
    max_seq_len = int(max_seq_len)
    if max_seq_len <= 0:
        return
    if int(block_table.shape[0]) != int(seq_lens.numel()):
        raise ValueError("block table and sequence-length batch dimensions differ")
    if int(block_table.shape[1]) * int(layout.block_size) < max_seq_len:
        raise ValueError("block table cannot cover max_seq_len")
    qp_k, qp_v = _readback_tables(layout, cache.device, q_points_k, q_points_v)
    stat = _stat_dtype_from_model_dtype(stat_dtype if stat_dtype is not None else out_k.dtype)
    _lib.call(
        "bkv_readback_sm100",
        cache.data_ptr(), int(cache.shape[0]), int(cache.stride(0)), int(layout.block_size),
        int(layout.num_kv_heads), _lib.dtype_code(stat),
        block_table.data_ptr(), block_table.stride(0), int(block_table.shape[1]),
        seq_lens.data_ptr(), seq_start_loc.data_ptr(), int(seq_lens.numel()), max_seq_len,
        qp_k.data_ptr(), qp_v.data_ptr(), _lib.dtype_code(qp_k.dtype),
        int(qp_k.dim() == 2), int(qp_v.dim() == 2),
        out_k.data_ptr(), out_v.data_ptr(), _lib.dtype_code(out_k.dtype),
        _lib.current_stream(cache.device),
    )


def read_request_from_paged_cache(
    cache: torch.Tensor,
    layout: PagedLayout,
    block_ids: torch.Tensor,
    seq_len: int,
    *,
    q_points_k: Optional[torch.Tensor] = None,
    q_points_v: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = torch.float16,
    stat_dtype: Optional[torch.dtype] = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Dequantise one request's context to ``(1, seq_len, H, D)`` K and V
    (reference :2210-2395), evaluated by the read-back kernel."""
    seq_len = int(seq_len)
    if int(block_ids.numel()) * int(layout.block_size) < seq_len:
        raise AssertionError("not enough blocks for seq_len")
    device = cache.device
    shape = (seq_len, int(layout.num_kv_heads), int(layout.head_dim))
    out_k = torch.empty(shape, dtype=out_dtype, device=device)
    out_v = torch.empty(shape, dtype=out_dtype, device=device)
    if seq_len > 0:
        table = block_ids.to(device=device, dtype=torch.int32).reshape(1, -1).contiguous()
        lens = torch.tensor([seq_len], dtype=torch.int32, device=device)
        starts = torch.tensor([0, seq_len], dtype=torch.int32, device=device)
        dequantize_paged_kv_to_dense(
            cache, layout, table, lens, starts, out_k, out_v,
            max_seq_len=seq_len, q_points_k=q_points_k, q_points_v=q_points_v,
            stat_dtype=stat_dtype if stat_dtype is not None else out_dtype,
        )
    return out_k.unsqueeze(0), out_v.unsqueeze(0)


# --------------------------------------------------------------------------- dense quantiser API
@dataclass
class PackedK:
    """Packed K state (reference :290-312): ``codes`` uint8 ``(B, S, H, D//G, G)``, ``packed``
    uint32 ``(B, S, H, D//G, 4)``, ``mn`` / ``scale`` 16-bit ``(B, S, H, D//G)``."""

    codes: torch.Tensor
    packed: torch.Tensor
    mn: torch.Tensor
    scale: torch.Tensor
    bits: int
    group_size: int
    pack_token_last: bool = False


@dataclass
class PackedV:
    """Packed V state (reference :315-335); with ``pack_token_last`` the token axis is the
    innermost one: ``packed`` ``(B, H, D//G, 4, S)``, ``mn`` / ``scale`` ``(B, H, D//G, S)``."""

    codes: torch.Tensor
    packed: torch.Tensor
    mn: torch.Tensor
    scale: torch.Tensor
    bits: int
    group_size: int
    pack_token_last: bool = False


_SCRATCH_BLOCK = 16  # page size of the private page pool the dense entry points run through


def _quantize_rows(x, num_bits, group_size, q_points, thresholds, stat_dtype):
    """Shared body of quantize_k / quantize_v (their arithmetic is the same, reference
    :463-475 and :552-564): the rows go through the encode-on-write kernel into a private page
    pool with consecutive slots, and the K regions of those pages are read back as the dense
    ``packed`` / ``scale`` / ``mn`` tensors."""
    _validate_real_quant_params(num_bits, group_size)
    if x.dim() != 4:
        raise ValueError("expected x.shape=(B, S, H, D)")
    B, S, H, D = (int(n) for n in x.shape)
    if D % group_size != 0:
        raise ValueError(f"head_dim {D} not divisible by group_size {group_size}")
    stat_dtype = _stat_dtype_from_model_dtype(stat_dtype or x.dtype)
    if not x.is_cuda:
        raise RuntimeError("quantize_k / quantize_v run on the sm_100a encode kernel: x must be a CUDA tensor")
    if D != _HEAD_DIM:
        raise RuntimeError(f"the sm_100a encode kernel handles head_dim {_HEAD_DIM}, got {D}")
    qp, thr = prepare_qpoints_and_thresholds(num_bits=num_bits, device=x.device, q_points=q_points, thresholds=thresholds)
    groups, tokens, bs = D // group_size, B * S, _SCRATCH_BLOCK
    pages = max(1, (tokens + bs - 1) // bs)
    layout = PagedLayout.build_hnd(bs, H, D, 4, group_size, group_size)
    cache = torch.zeros((pages, layout.block_i32), dtype=torch.int32, device=x.device)
    rows = x.reshape(tokens, H, D)
    if rows.stride(2) != 1:
        rows = rows.contiguous()
    if tokens:
        slots = torch.arange(tokens, dtype=torch.int64, device=x.device)
        write_tokens_to_paged_cache(cache, layout, None, slots, rows, rows, q_points_k=qp, q_points_v=qp,
                                    thresholds_k=thr, thresholds_v=thr, require_fast=True, stat_dtype=stat_dtype)
    code_words, stat_words = H * bs * 16, H * bs * groups
    packed = cache[:, :code_words].reshape(pages, H, bs, groups, 4).permute(0, 2, 1, 3, 4).reshape(pages * bs, H, groups, 4)
    packed = packed[:tokens].reshape(B, S, H, groups, 4).contiguous().view(torch.uint32)
    stats = cache[:, code_words : code_words + stat_words].reshape(pages, H, bs, groups).permute(0, 2, 1, 3)
    stats = stats.reshape(pages * bs, H, groups)[:tokens].reshape(B, S, H, groups).contiguous()
    halves = stats.view(stat_dtype).reshape(B, S, H, groups, 2)  # low half: scale, high half: minimum
    return packed, halves[..., 1].contiguous(), halves[..., 0].contiguous()


def quantize_k(
    x: torch.Tensor,
    num_bits: int,
    group_size: int,
    q_points: Optional[torch.Tensor] = None,
    thresholds: Optional[torch.Tensor] = None,
    pack_axis_first: bool = False,
    stat_dtype: Optional[torch.dtype] = None,
) -> PackedK:
    """Quantise K in ``(B, S, H, D)`` layout, grouping along D per token (reference :439-486),
    on the GPU; codes and statistics are bit-identical to the reference function."""
    if pack_axis_first:
        raise TypeError("pack_axis_first was removed; K is per-token")
    packed, mn, scale = _quantize_rows(x, num_bits, group_size, q_points, thresholds, stat_dtype)
    return PackedK(codes=unpack_codes(packed, num_bits, group_size), packed=packed, mn=mn, scale=scale,
                   bits=num_bits, group_size=group_size, pack_token_last=False)


def quantize_v(
    x: torch.Tensor,
    num_bits: int,
    group_size: int,
    q_points: Optional[torch.Tensor] = None,
    thresholds: Optional[torch.Tensor] = None,
    pack_token_last: bool = False,
    stat_dtype: Optional[torch.dtype] = None,
) -> PackedV:
    """Quantise V in ``(B, S, H, D)`` layout, grouping along D (reference :525-584)."""
    packed, mn, scale = _quantize_rows(x, num_bits, group_size, q_points, thresholds, stat_dtype)
    codes = unpack_codes(packed, num_bits, group_size)
    if pack_token_last:
        packed = packed.permute(0, 2, 3, 4, 1).contiguous()
        mn = mn.permute(0, 2, 3, 1).contiguous()
        scale = scale.permute(0, 2, 3, 1).contiguous()
    return PackedV(codes=codes, packed=packed, mn=mn, scale=scale, bits=num_bits, group_size=group_size,
                   pack_token_last=pack_token_last)


def _dequantize_rows(packed, q_points) -> torch.Tensor:
    """Shared body of dequantize_k / dequantize_v (reference :499-517, :596-616): the packed
    words and statistics are laid into a private page pool and reconstructed by the read-back
    kernel - ``level * scale + min`` in float32 as two rounded operations, then one rounding to
    the dtype of the statistics."""
    _validate_real_quant_params(packed.bits, packed.group_size)
    words, mn, scale = packed.packed, packed.mn, packed.scale
    if packed.pack_token_last:
        words = words.permute(0, 4, 1, 2, 3)
        mn = mn.permute(0, 3, 1, 2)
        scale = scale.permute(0, 3, 1, 2)
    if not mn.is_cuda:
        raise RuntimeError("dequantize_k / dequantize_v run on the sm_100a read-back kernel: CUDA tensors only")
    B, S, H, groups, _ = (int(n) for n in words.shape)
    if groups * packed.group_size != _HEAD_DIM:
        raise RuntimeError(f"the sm_100a read-back kernel handles head_dim {_HEAD_DIM}")
    tokens, bs = B * S, _SCRATCH_BLOCK
    out = torch.empty((tokens, H, _HEAD_DIM), dtype=mn.dtype, device=mn.device)
    if tokens == 0:
        return out.reshape(B, S, H, _HEAD_DIM)
    pages = (tokens + bs - 1) // bs
    layout = PagedLayout.build_hnd(bs, H, _HEAD_DIM, 4, packed.group_size, packed.group_size)
    cache = torch.zeros((pages, layout.block_i32), dtype=torch.int32, device=mn.device)
    code_words, stat_words = H * bs * 16, H * bs * groups
    padded = torch.zeros((pages * bs, H, groups, 4), dtype=torch.int32, device=mn.device)
    padded[:tokens] = words.reshape(tokens, H, groups, 4).view(torch.int32)
    cache[:, :code_words] = padded.reshape(pages, bs, H, groups, 4).permute(0, 2, 1, 3, 4).reshape(pages, code_words)
    halves = torch.zeros((pages * bs, H, groups, 2), dtype=mn.dtype, device=mn.device)
    halves[:tokens, ..., 0] = scale.reshape(tokens, H, groups)
    halves[:tokens, ..., 1] = mn.reshape(tokens, H, groups)
    stat_i32 = halves.view(torch.int32).reshape(pages, bs, H, groups)
    cache[:, code_words : code_words + stat_words] = stat_i32.permute(0, 2, 1, 3).reshape(pages, stat_words)
    table = torch.arange(pages, dtype=torch.int32, device=mn.device).reshape(1, pages)
    lens = torch.tensor([tokens], dtype=torch.int32, device=mn.device)
    starts = torch.tensor([0, tokens], dtype=torch.int32, device=mn.device)
    unused_v = torch.empty_like(out)
    dequantize_paged_kv_to_dense(cache, layout, table, lens, starts, out, unused_v, max_seq_len=tokens,
                                 q_points_k=q_points, q_points_v=q_points, stat_dtype=mn.dtype)
    return out.reshape(B, S, H, _HEAD_DIM)


def dequantize_k(packed: PackedK, q_points: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Reconstructed K ``(B, S, H, D)`` in the dtype of the packed statistics (reference :489-517)."""
    return _dequantize_rows(packed, q_points)


def dequantize_v(packed: PackedV, q_points: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Reconstructed V ``(B, S, H, D)`` in the dtype of the packed statistics (reference :587-616)."""
    return _dequantize_rows(packed, q_points)
