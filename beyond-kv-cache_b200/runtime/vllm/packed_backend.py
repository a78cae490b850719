"""vLLM attention-backend interface of the packed-KV path, on the B200 kernels.

Mirror of the *attention interface part* of the reference backend
(``src/beyond/runtime/vllm/packed_backend.py``): ``BeyondPackedSpec`` (:429-486),
``BeyondPackedImpl.forward`` (:3415-3820), its decode path
``_run_sm103_nonuniform_dense_decode`` (:2890-2994), the production prefill path
(:2424-2520) and ``BeyondPackedBackend`` (:4836-4888).  The scheduler / CUDA-graph /
prewarm machinery of that file is vLLM glue and is not rebuilt; this module does not
import vLLM, so it can be exercised the way the reference's own test does
(``tests/runtime/vllm/test_page_table_backend_exact.py:24-31``): construct the impl,
hand it a metadata object with the fields it reads, call ``forward``.

Request plans served (anything else fails closed with ``NotImplementedError`` like the
reference, :3644-3649, :3812-3820):

* all-decode batch (one query token per request): encode-on-write of the new token, then
  the fused packed decode kernel;
* all-prefill batch (every query covers its whole sequence): encode-on-write with
  in-place reconstruction of K/V, then causal attention over the *rounded* K/V.  The
  reference hands those to FlashAttention (a library call outside this path); here the
  dense attention is ``torch.nn.functional.scaled_dot_product_attention`` per request;
* homogeneous chunked prefill (every request: more than one query token behind context that
  is already cached; reference :2523-2625): encode-on-write of the chunk, read-back of every
  request's whole context into a bounded dense view, causal attention over that view.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ...quant.beyond_cute import (
    CODE_LAYOUT_HND_TOKEN_WORD,
    PagedLayout,
    classify_tables,
    dequantize_paged_kv_to_dense,
    prepare_qpoints_and_thresholds,
    write_tokens_to_paged_cache,
)
from ...quant.fa4_cute import beyond_mixed_decode_runtime as _rt
from .config import env_bool

BEYOND_BITS = 4
BEYOND_K_GROUP_SIZE = 32
BEYOND_V_GROUP_SIZE = 32
BEYOND_PACKED_BLOCK_SIZES = (16, 32, 64, 128)
_HEAD_SIZE = 128


def _paged_layout(block_size: int, num_kv_heads: int, head_size: int) -> PagedLayout:
    return PagedLayout.build_hnd(block_size, num_kv_heads, head_size, BEYOND_BITS, BEYOND_K_GROUP_SIZE, BEYOND_V_GROUP_SIZE)


def _infer_block_size(kv_cache: torch.Tensor, num_kv_heads: int, head_size: int) -> int:
    """Page size from the cache row length (reference ``_infer_block_size``): one token of one
    head takes 40 int32 words at head_size 128."""
    per_token = _paged_layout(1, num_kv_heads, head_size).block_i32
    block_size, rem = divmod(int(kv_cache.shape[1]), per_token)
    if rem or block_size <= 0:
        raise RuntimeError(f"kv_cache row length {kv_cache.shape[1]} is not a whole number of packed tokens")
    return block_size


@dataclass(frozen=True)
class BeyondPackedSpec:
    """KV-cache spec of the packed layout (reference :429-486): dtype int32, page size in
    bytes = ``block_i32 * 4`` (160 bytes per token per KV head at head_size 128)."""

    block_size: int
    num_kv_heads: int
    head_size: int
    dtype: torch.dtype = torch.int32

    @property
    def real_page_size_bytes(self) -> int:
        return _paged_layout(self.block_size, self.num_kv_heads, self.head_size).block_i32 * 4

    @property
    def page_size_bytes(self) -> int:
        return self.real_page_size_bytes


_VLLM_SPEC_CLASS = None


def vllm_spec_class():
    """``BeyondPackedSpec`` as a subclass of the installed vLLM's ``FullAttentionSpec`` (what the
    reference declares, :473-486), so that vLLM's cache managers and allocator accept it; built on
    first use because importing vLLM is slow and this module must work without it.  Raises
    ImportError when vLLM (or that class) is not importable."""
    global _VLLM_SPEC_CLASS
    if _VLLM_SPEC_CLASS is None:
        from vllm.v1.kv_cache_interface import FullAttentionSpec

        @dataclass(frozen=True, kw_only=True)
        class BeyondPackedVllmSpec(FullAttentionSpec):
            """KV-cache spec of the packed layout: the cache is a flat ``(num_blocks, block_i32)`` int32
            buffer, so a page is ``block_i32 * 4`` bytes whatever dtype and head size suggest."""

            @property
            def real_page_size_bytes(self) -> int:
                return _paged_layout(self.block_size, self.num_kv_heads, self.head_size).block_i32 * 4

        _VLLM_SPEC_CLASS = BeyondPackedVllmSpec
    return _VLLM_SPEC_CLASS


class BeyondPackedBackend:
    """Static description of the backend (reference :4836-4888)."""

    accept_output_buffer = True
    forward_includes_kv_cache_update = True

    @staticmethod
    def get_name() -> str:
        return "CUSTOM"

    @staticmethod
    def get_impl_cls():
        return BeyondPackedImpl

    @staticmethod
    def get_builder_cls():
        return BeyondPackedMetadataBuilder

    @staticmethod
    def get_supported_kernel_block_sizes() -> list[int]:
        return list(BEYOND_PACKED_BLOCK_SIZES)

    @classmethod
    def supports_block_size(cls, block_size: Optional[int]) -> bool:
        return block_size is None or int(block_size) in BEYOND_PACKED_BLOCK_SIZES

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int, cache_dtype_str: str = "auto") -> tuple[int, int]:
        if int(block_size) not in BEYOND_PACKED_BLOCK_SIZES:
            raise ValueError(f"packed cache block_size must be one of {BEYOND_PACKED_BLOCK_SIZES}")
        return (int(num_blocks), _paged_layout(block_size, num_kv_heads, head_size).block_i32)


@dataclass
class BeyondPackedMetadata:
    """What ``BeyondPackedImpl.forward`` reads (reference `:3437, :3477-3516`): the device
    tensors of vLLM's common attention metadata plus host mirrors of the per-request query
    offsets and sequence lengths, so that classifying the batch costs no device read."""

    num_actual_tokens: int
    query_start_loc: torch.Tensor
    seq_lens: torch.Tensor
    block_table: torch.Tensor
    slot_mapping: torch.Tensor
    max_query_len: int
    max_seq_len: int
    _beyond_query_start_loc_list: Optional[list] = None
    _beyond_seq_lens_list: Optional[list] = None


class BeyondPackedMetadataBuilder:
    """Builds :class:`BeyondPackedMetadata` from vLLM's ``CommonAttentionMetadata`` (reference
    ``BeyondPackedMetadataBuilder.build`` / ``.build_for_cudagraph_capture``, `:4719-4828`).
    The object is read by attribute name only, so any metadata carrying ``num_actual_tokens``,
    ``query_start_loc[_cpu]``, ``seq_lens[_cpu]``, ``block_table_tensor``, ``slot_mapping``,
    ``max_query_len`` and ``max_seq_len`` serves."""

    def __init__(self, kv_cache_spec=None, layer_names=None, vllm_config=None, device=None):
        self.kv_cache_spec = kv_cache_spec
        self.layer_names = layer_names
        self.vllm_config = vllm_config
        self.device = device

    @staticmethod
    def _host_list(common, name: str, count: int):
        mirror = getattr(common, f"{name}_cpu", None)
        if mirror is None:
            return None  # forward() falls back to one device read
        return [int(v) for v in mirror[:count].tolist()]

    def build(self, common_prefix_len: int, common_attn_metadata, fast_build: bool = False) -> BeyondPackedMetadata:
        c = common_attn_metadata
        num_reqs = int(getattr(c, "num_reqs", c.seq_lens.shape[0]))
        block_table = getattr(c, "block_table_tensor", None)
        if block_table is None:
            block_table = c.block_table
        return BeyondPackedMetadata(
            num_actual_tokens=int(c.num_actual_tokens), query_start_loc=c.query_start_loc, seq_lens=c.seq_lens,
            block_table=block_table, slot_mapping=c.slot_mapping, max_query_len=int(c.max_query_len),
            max_seq_len=int(c.max_seq_len),
            _beyond_query_start_loc_list=self._host_list(c, "query_start_loc", num_reqs + 1),
            _beyond_seq_lens_list=self._host_list(c, "seq_lens", num_reqs))

    def build_for_cudagraph_capture(self, common_attn_metadata) -> BeyondPackedMetadata:
        """Capture-time metadata: every request is a one-token decode at the bucket's longest
        context, whatever placeholder lengths the runner filled in (reference `:4790-4828`)."""
        m = self.build(0, common_attn_metadata)
        num_reqs = int(m.seq_lens.shape[0])
        m._beyond_query_start_loc_list = list(range(num_reqs + 1))
        m._beyond_seq_lens_list = [max(1, int(m.max_seq_len))] * num_reqs
        return m


_CHUNKED_PREFILL_WORKSPACE_MB = 1024  # bound of the dense read-back view (reference :2194-2220)


class BeyondPackedImpl:
    """Per-layer attention implementation (reference ``BeyondPackedImpl``)."""

    can_return_lse_for_decode = False

    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: Optional[int] = None, **_unused):
        self.num_heads = int(num_heads)
        self.head_size = int(head_size)
        self.scale = float(scale)
        self.num_kv_heads = int(num_kv_heads if num_kv_heads is not None else num_heads)
        self._tables = (None, None, None, None)
        self._device_tables: dict = {}
        self._workspaces: dict = {}
        self._dense_workspace = None

    # -- quantiser tables --------------------------------------------------------------
    def set_quant_tables(self, q_points_k, thresholds_k, q_points_v, thresholds_v) -> None:
        """Per-layer tables, shared ``(16,)/(15,)`` or per-(head, group) ``(Hkv*4, 16)/(Hkv*4, 15)``
        (what the reference resolves from its quant-config file, :2076-2172).  They are uploaded,
        classified and expanded for the decode kernel once per device, on first use, and those
        device tensors are kept alive here: a forward pass uploads and inspects nothing."""
        self._tables = (q_points_k, thresholds_k, q_points_v, thresholds_v)
        self._device_tables.clear()

    def _tables_on(self, device):
        """(q_points_k, thresholds_k, q_points_v, thresholds_v, runtime K levels, runtime V levels)."""
        key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
        held = self._device_tables.get(key)
        if held is None:
            qk, tk = prepare_qpoints_and_thresholds(num_bits=4, device=device, q_points=self._tables[0], thresholds=self._tables[1])
            qv, tv = prepare_qpoints_and_thresholds(num_bits=4, device=device, q_points=self._tables[2], thresholds=self._tables[3])
            if qk.dtype != qv.dtype:  # the kernels take one table dtype per call
                qk, tk, qv, tv = (t.to(torch.float32) for t in (qk, tk, qv, tv))
            classify_tables(tk, tv)  # sorted or not: decided here, once, not on the write path
            n = self.num_kv_heads * 4
            gk = qk if qk.dim() == 2 else qk.unsqueeze(0).expand(n, 16)
            gv = qv if qv.dim() == 2 else qv.unsqueeze(0).expand(n, 16)
            rk, rv = _rt.prepare_runtime_qpoints(gk.contiguous(), gv.contiguous(), heads_kv=self.num_kv_heads)
            held = self._device_tables[key] = (qk, tk, qv, tv, rk, rv)
        return held

    # -- forward -----------------------------------------------------------------------
    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, output_scale=None, output_block_scale=None):
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("BeyondPacked backend does not support fused output quantization.")
        if attn_metadata is None:
            return torch.zeros_like(query) if output is None else output.fill_(0)
        num_actual = int(attn_metadata.num_actual_tokens)
        q, k, v = query[:num_actual], key[:num_actual], value[:num_actual]
        if q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype:
            raise RuntimeError(
                "BeyondPacked CUSTOM backend supports fp16/bf16 Q/K/V tensors with a shared dtype; "
                f"got q={q.dtype}, k={k.dtype}, v={v.dtype}."
            )
        H_q, H_kv, D = self.num_heads, self.num_kv_heads, self.head_size
        if H_q % H_kv:
            raise ValueError(f"H_q={H_q} not multiple of H_kv={H_kv}")
        if H_q // H_kv > 8:
            raise NotImplementedError("packed path requires H_q / H_kv <= 8")
        if D != _HEAD_SIZE:
            raise NotImplementedError("the sm_100a packed path requires head_size 128")
        block_size = _infer_block_size(kv_cache, H_kv, D)
        layout = _paged_layout(block_size, H_kv, D)
        if output is None:
            output = torch.empty((num_actual, H_q, D), dtype=q.dtype, device=q.device)
        q_starts = getattr(attn_metadata, "_beyond_query_start_loc_list", None)
        if q_starts is None:
            q_starts = attn_metadata.query_start_loc.cpu().tolist()
        num_reqs = len(q_starts) - 1
        seq_lens_cpu = getattr(attn_metadata, "_beyond_seq_lens_list", None)
        if seq_lens_cpu is None:
            seq_lens_cpu = attn_metadata.seq_lens[:num_reqs].cpu().tolist()
        q_lens = [int(q_starts[i + 1]) - int(q_starts[i]) for i in range(num_reqs)]
        if num_reqs == 0 or num_actual == 0:
            return output
        tables = self._tables_on(q.device)
        slots = attn_metadata.slot_mapping[:num_actual]
        block_table = attn_metadata.block_table

        if all(n == 1 for n in q_lens) and num_actual == num_reqs:
            return self._decode(q, k, v, output, kv_cache, layout, block_table, attn_metadata.seq_lens, slots,
                                seq_lens_cpu, tables)
        if all(n == int(s) for n, s in zip(q_lens, seq_lens_cpu)):
            return self._prefill(q, k, v, output, kv_cache, layout, block_table, slots, q_starts, tables)
        if all(1 < n < int(s) for n, s in zip(q_lens, seq_lens_cpu)):
            return self._chunked_prefill(q, k, v, output, kv_cache, layout, block_table, attn_metadata.seq_lens, slots,
                                         q_starts, seq_lens_cpu, tables)
        raise NotImplementedError(
            "Beyond production attention could not represent this mixed or chunked-prefill scheduler plan."
        )

    def _decode(self, q, k, v, output, cache, layout, block_table, seq_lens, slots, seq_lens_cpu, tables):
        qk, tk, qv, tv, rk, rv = tables
        batch = int(q.shape[0])
        # Everything the attention grid reads before its programmatic wait - sequence lengths,
        # block table, queries, its workspace - is in place BEFORE the writer is launched, so that
        # the writer is the launch that immediately precedes the attention grid (the only launch
        # whose output that grid may not see until it has waited).
        if slots.dtype != torch.int32 or not slots.is_contiguous():
            slots = slots.to(torch.int32).contiguous()
        if seq_lens.dtype != torch.int32 or not seq_lens.is_contiguous():
            seq_lens = seq_lens.to(torch.int32).contiguous()
        bs = int(layout.block_size)
        need = max(int(x) for x in seq_lens_cpu)
        capacity = int(block_table.shape[1]) * bs
        bucket = bs
        while bucket < need:  # power-of-two launch bucket, capped by the block-table capacity (:372-393)
            bucket *= 2
        max_seq_len = min(bucket, capacity)
        # the writer lets the attention grid start its set-up early and that grid waits before its
        # first cache read (BEYOND_SM103_WRITER_PDL, on by default as in the reference :2955)
        writer_pdl = env_bool("BEYOND_SM103_WRITER_PDL", True)
        spec = _rt.make_runtime_spec(q=q, cache=cache, layout=layout, block_table=block_table, heads_q=self.num_heads,
                                     max_seq_len=max_seq_len, num_splits=0, qpoint_dtype=rk.dtype,
                                     wait_for_pdl_writer=writer_pdl)
        ws = self._workspaces.get(spec)
        if ws is None:
            ws = _rt.allocate_runtime_workspace(spec, device=q.device)
            self._workspaces[spec] = ws
        # the current token is written first and then attended like any other (:2953-2969)
        write_tokens_to_paged_cache(cache, layout, block_table, slots[:batch], k[:batch], v[:batch], q_points_k=qk,
                                    q_points_v=qv, thresholds_k=tk, thresholds_v=tv, signal_pdl_dependents=writer_pdl,
                                    require_fast=True)
        _rt.run_nonuniform_decode(spec=spec, q=q, cache=cache, layout=layout, block_table=block_table, seq_lens=seq_lens,
                                  k_qpoints_lane_major=rk, v_qpoints_code_major=rv, out=output[:batch], workspace=ws,
                                  softmax_scale=self.scale)
        return output

    def _dense_attention(self, q, k, v, output, q_starts, k_starts):
        """Causal attention of every request's queries over its dense keys, the last query row
        aligned with the last key (what the reference hands to FlashAttention's varlen call, a
        library outside this path; here one scaled_dot_product_attention per request)."""
        rep = self.num_heads // self.num_kv_heads
        for i in range(len(q_starts) - 1):
            s, e = int(q_starts[i]), int(q_starts[i + 1])
            ks, ke = int(k_starts[i]), int(k_starts[i + 1])
            if e <= s:
                continue
            qi = q[s:e].transpose(0, 1).unsqueeze(0)
            ki = k[ks:ke].repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)
            vi = v[ks:ke].repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)
            nq, nk = e - s, ke - ks
            if nq == nk:
                o = torch.nn.functional.scaled_dot_product_attention(qi, ki, vi, is_causal=True, scale=self.scale)
            else:  # query row r sees keys 0 .. nk - nq + r
                mask = torch.ones((nq, nk), dtype=torch.bool, device=q.device).tril(diagonal=nk - nq)
                o = torch.nn.functional.scaled_dot_product_attention(qi, ki, vi, attn_mask=mask, scale=self.scale)
            output[s:e].copy_(o.squeeze(0).transpose(0, 1))

    def _prefill(self, q, k, v, output, cache, layout, block_table, slots, q_starts, tables):
        qk, tk, qv, tv = tables[:4]
        # K/V are reconstructed in place so that attention sees exactly what the cache holds (:2481-2498)
        write_tokens_to_paged_cache(cache, layout, block_table, slots, k, v, q_points_k=qk, q_points_v=qv,
                                    thresholds_k=tk, thresholds_v=tv, k_dq_out=k, v_dq_out=v, require_fast=True)
        self._dense_attention(q, k, v, output, q_starts, q_starts)
        return output

    def _chunked_prefill(self, q, k, v, output, cache, layout, block_table, seq_lens, slots, q_starts, seq_lens_cpu, tables):
        """A chunk of every request's prompt behind context that is already cached (reference
        ``_run_production_chunked_prefill_forward``, :2523-2625): the chunk is committed to the
        packed cache, the whole context of every request is read back into one bounded dense
        view, and the chunk's queries attend that view causally."""
        qk, tk, qv, tv = tables[:4]
        num_reqs = len(q_starts) - 1
        total_k = sum(int(n) for n in seq_lens_cpu[:num_reqs])
        itemsize = torch.empty((), dtype=q.dtype).element_size()
        if 2 * total_k * self.num_kv_heads * self.head_size * itemsize > _CHUNKED_PREFILL_WORKSPACE_MB << 20:
            raise NotImplementedError(
                "Beyond production attention could not represent this mixed or chunked-prefill scheduler plan "
                f"(its dense read-back view would exceed {_CHUNKED_PREFILL_WORKSPACE_MB} MB)."
            )
        held = self._dense_workspace
        if held is None or held[0].shape[0] < total_k or held[0].dtype != q.dtype or held[0].device != q.device:
            shape = (total_k, self.num_kv_heads, self.head_size)
            held = self._dense_workspace = (torch.empty(shape, dtype=q.dtype, device=q.device),
                                            torch.empty(shape, dtype=q.dtype, device=q.device))
        dense_k, dense_v = held[0][:total_k], held[1][:total_k]
        k_starts = [0]
        for n in seq_lens_cpu[:num_reqs]:
            k_starts.append(k_starts[-1] + int(n))
        lens_gpu = seq_lens[:num_reqs]
        if lens_gpu.dtype != torch.int32 or not lens_gpu.is_contiguous():
            lens_gpu = lens_gpu.to(torch.int32).contiguous()
        starts_gpu = torch.tensor(k_starts, dtype=torch.int32, device=q.device)
        if slots.dtype != torch.int32 or not slots.is_contiguous():
            slots = slots.to(torch.int32).contiguous()
        if int(slots.numel()) != int(k.shape[0]):
            raise ValueError("slot_mapping must contain one entry per chunked-prefill K/V token")
        write_tokens_to_paged_cache(cache, layout, block_table, slots, k, v, q_points_k=qk, q_points_v=qv,
                                    thresholds_k=tk, thresholds_v=tv, require_fast=True)
        table = block_table[:num_reqs]
        if table.dtype != torch.int32 or table.stride(-1) != 1:
            table = table.to(torch.int32).contiguous()
        dequantize_paged_kv_to_dense(cache, layout, table, lens_gpu, starts_gpu, dense_k, dense_v,
                                     max_seq_len=max(int(n) for n in seq_lens_cpu[:num_reqs]),
                                     q_points_k=qk, q_points_v=qv, stat_dtype=q.dtype)
        self._dense_attention(q, dense_k, dense_v, output, q_starts, k_starts)
        return output
