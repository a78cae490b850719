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
  dense attention is ``torch.nn.functional.scaled_dot_product_attention`` per request.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ...quant.beyond_cute import (
    CODE_LAYOUT_HND_TOKEN_WORD,
    PagedLayout,
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


class BeyondPackedImpl:
    """Per-layer attention implementation (reference ``BeyondPackedImpl``)."""

    can_return_lse_for_decode = False

    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: Optional[int] = None, **_unused):
        self.num_heads = int(num_heads)
        self.head_size = int(head_size)
        self.scale = float(scale)
        self.num_kv_heads = int(num_kv_heads if num_kv_heads is not None else num_heads)
        self._tables = None
        self._workspaces: dict = {}

    # -- quantiser tables --------------------------------------------------------------
    def set_quant_tables(self, q_points_k, thresholds_k, q_points_v, thresholds_v) -> None:
        """Per-layer tables, shared ``(16,)/(15,)`` or per-(head, group) ``(Hkv*4, 16)/(Hkv*4, 15)``
        (what the reference resolves from its quant-config file, :2076-2172)."""
        self._tables = (q_points_k, thresholds_k, q_points_v, thresholds_v)
        self.__dict__.pop("_runtime_tables", None)

    def _resolve_tables(self, device):
        tables = getattr(self, "_tables", None) or (None, None, None, None)
        qk, tk = prepare_qpoints_and_thresholds(num_bits=4, device=device, q_points=tables[0], thresholds=tables[1])
        qv, tv = prepare_qpoints_and_thresholds(num_bits=4, device=device, q_points=tables[2], thresholds=tables[3])
        return qk, tk, qv, tv

    def _runtime_qpoints(self, qk, qv):
        cached = self.__dict__.get("_runtime_tables")
        if cached is None or cached[0] is not qk or cached[1] is not qv:
            n = self.num_kv_heads * 4
            gk = qk if qk.dim() == 2 else qk.unsqueeze(0).expand(n, 16)
            gv = qv if qv.dim() == 2 else qv.unsqueeze(0).expand(n, 16)
            rk, rv = _rt.prepare_runtime_qpoints(gk.contiguous(), gv.contiguous(), heads_kv=self.num_kv_heads)
            cached = (qk, qv, rk, rv)
            self._runtime_tables = cached
        return cached[2], cached[3]

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
        qk, tk, qv, tv = self._resolve_tables(q.device)
        slots = attn_metadata.slot_mapping[:num_actual]
        block_table = attn_metadata.block_table

        if all(n == 1 for n in q_lens) and num_actual == num_reqs:
            return self._decode(q, k, v, output, kv_cache, layout, block_table, attn_metadata.seq_lens, slots,
                                seq_lens_cpu, qk, tk, qv, tv)
        if all(n == int(s) for n, s in zip(q_lens, seq_lens_cpu)):
            return self._prefill(q, k, v, output, kv_cache, layout, block_table, slots, q_starts, qk, tk, qv, tv)
        raise NotImplementedError(
            "Beyond production attention could not represent this mixed or chunked-prefill scheduler plan."
        )

    def _decode(self, q, k, v, output, cache, layout, block_table, seq_lens, slots, seq_lens_cpu, qk, tk, qv, tv):
        batch = int(q.shape[0])
        if slots.dtype != torch.int32 or not slots.is_contiguous():
            slots = slots.to(torch.int32).contiguous()
        # the current token is written first and then attended like any other (:2953-2969); the
        # writer lets the attention grid start its set-up early and that grid waits before its
        # first cache read (BEYOND_SM103_WRITER_PDL, on by default as in the reference :2955)
        writer_pdl = env_bool("BEYOND_SM103_WRITER_PDL", True)
        write_tokens_to_paged_cache(cache, layout, block_table, slots[:batch], k[:batch], v[:batch], q_points_k=qk,
                                    q_points_v=qv, thresholds_k=tk, thresholds_v=tv, signal_pdl_dependents=writer_pdl,
                                    require_fast=True)
        bs = int(layout.block_size)
        need = max(int(x) for x in seq_lens_cpu)
        capacity = int(block_table.shape[1]) * bs
        bucket = bs
        while bucket < need:  # power-of-two launch bucket, capped by the block-table capacity (:372-393)
            bucket *= 2
        max_seq_len = min(bucket, capacity)
        rk, rv = self._runtime_qpoints(qk, qv)
        spec = _rt.make_runtime_spec(q=q, cache=cache, layout=layout, block_table=block_table, heads_q=self.num_heads,
                                     max_seq_len=max_seq_len, num_splits=0, qpoint_dtype=rk.dtype,
                                     wait_for_pdl_writer=writer_pdl)
        ws = self._workspaces.get(spec)
        if ws is None:
            ws = _rt.allocate_runtime_workspace(spec, device=q.device)
            self._workspaces[spec] = ws
        if seq_lens.dtype != torch.int32 or not seq_lens.is_contiguous():
            seq_lens = seq_lens.to(torch.int32).contiguous()
        _rt.run_nonuniform_decode(spec=spec, q=q, cache=cache, layout=layout, block_table=block_table, seq_lens=seq_lens,
                                  k_qpoints_lane_major=rk, v_qpoints_code_major=rv, out=output[:batch], workspace=ws,
                                  softmax_scale=self.scale)
        return output

    def _prefill(self, q, k, v, output, cache, layout, block_table, slots, q_starts, qk, tk, qv, tv):
        # K/V are reconstructed in place so that attention sees exactly what the cache holds (:2481-2498)
        write_tokens_to_paged_cache(cache, layout, block_table, slots, k, v, q_points_k=qk, q_points_v=qv,
                                    thresholds_k=tk, thresholds_v=tv, k_dq_out=k, v_dq_out=v, require_fast=True)
        rep = self.num_heads // self.num_kv_heads
        for i in range(len(q_starts) - 1):
            s, e = int(q_starts[i]), int(q_starts[i + 1])
            if e <= s:
                continue
            qi = q[s:e].transpose(0, 1).unsqueeze(0)
            ki = k[s:e].repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)
            vi = v[s:e].repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)
            o = torch.nn.functional.scaled_dot_product_attention(qi, ki, vi, is_causal=True, scale=self.scale)
            output[s:e].copy_(o.squeeze(0).transpose(0, 1))
        return output
