"""Multi-GPU forms of the packed decode path (one process per GPU, ``torch.distributed``).

The reference has no multi-GPU decode (its serving numbers are single-GPU; tensor
parallelism is delegated to vLLM).  Two shardings are provided here:

* **Request-batch sharding** — requests are independent, so every rank owns a slice of
  the batch with its own page pool; there is no collective on the data path
  (:func:`shard_requests`).
* **KV-range split of one long sequence** — rank ``r`` owns a contiguous, page-aligned
  range of positions, runs the decode kernel over it and produces an un-normalised
  partial ``(o, m, l)`` per (request, query head).  The partials (16.6 KB per rank for 32
  heads) are exchanged and merged by log-sum-exp, "splits = world size"
  (:func:`decode_kv_range_split`): with a :class:`KvRangeExchange` every rank stores its
  record straight into the other ranks' receive buffers over NVLink and one kernel pushes,
  waits (bounded) and merges; without one the records travel in one NCCL all-gather and the
  combine kernel merges them.  ``torch.distributed`` is used for set-up and for that
  all-gather only.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib
from .quant.beyond_cute import PagedLayout


def shard_requests(batch: int, world: int, rank: int) -> range:
    """Contiguous, balanced slice of ``range(batch)`` owned by ``rank`` (sizes differ by
    at most one; the first ``batch % world`` ranks get the extra request)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(int(batch), world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def kv_range_for_rank(seq_len: int, block_size: int, world: int, rank: int) -> tuple[int, int]:
    """Positions ``[lo, hi)`` of a ``seq_len``-token sequence owned by ``rank``: pages
    are dealt in contiguous, balanced runs so every boundary is page-aligned; the last
    non-empty range ends at ``seq_len``.  Ranks beyond the page count get ``(x, x)``."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    pages = (int(seq_len) + block_size - 1) // block_size
    pr = shard_requests(pages, world, rank)
    lo = pr.start * block_size
    hi = max(lo, min(pr.stop * block_size, int(seq_len)))
    return lo, hi


def gather_partials(o: torch.Tensor, m: torch.Tensor, l: torch.Tensor, group=None):
    """All-gather the per-rank partials: returns ``(world, rows, 128)``, ``(world, rows)``,
    ``(world, rows)`` tensors (any backend; NCCL on GPUs, gloo in the CPU tests)."""
    world = dist.get_world_size(group)
    packed = torch.cat([o.reshape(o.shape[0], -1), m.reshape(-1, 1), l.reshape(-1, 1)], dim=1).contiguous()
    flat = torch.empty((world * packed.shape[0], packed.shape[1]), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(flat, packed, group=group)  # rank-major concatenation along dim 0
    out = flat.view(world, packed.shape[0], packed.shape[1])
    d = o.shape[-1]
    return out[:, :, :d].contiguous(), out[:, :, d].contiguous(), out[:, :, d + 1].contiguous()


_WORKSPACES: dict = {}


def _stream_workspace(device: torch.device) -> torch.Tensor:
    """Scratch of the persistent schedule, one per device, allocated on first use (calls on
    one device are issued on one stream here, so they never overlap)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = _WORKSPACES[key] = _lib.stream_workspace(device)
    return ws


def decode_range_partial(
    q: torch.Tensor,
    cache: torch.Tensor,
    layout: PagedLayout,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    q_points_k: torch.Tensor,
    q_points_v: torch.Tensor,
    *,
    token_lo: int,
    token_hi: int,
    softmax_scale: float,
    stat_dtype: Optional[torch.dtype] = None,
):
    """Un-normalised attention of every request over positions ``[token_lo, token_hi)``
    (clipped to its ``seq_len``): ``o (rows,128)``, ``m (rows,)`` natural-log maximum,
    ``l (rows,)`` sum, all float32, rows = batch * query heads."""
    batch, heads_q = int(q.shape[0]), int(q.shape[1])
    rows = batch * heads_q
    o = torch.empty((rows, 128), dtype=torch.float32, device=q.device)
    m = torch.empty((rows,), dtype=torch.float32, device=q.device)
    l = torch.empty((rows,), dtype=torch.float32, device=q.device)
    if q_points_k.dtype != q_points_v.dtype:
        q_points_k, q_points_v = q_points_k.float(), q_points_v.float()
    stat = stat_dtype if stat_dtype is not None else q.dtype
    quads = (heads_q // int(layout.num_kv_heads) + 3) // 4
    if (batch <= 16384 and int(cache.shape[0]) <= (1 << 26) and layout.block_size in (16, 32, 64, 128)
            and int(layout.num_kv_heads) * quads * batch <= (1 << 20) and q_points_k.dtype != torch.float32):
        # persistent schedule: every SM works on the range even when it is one request's
        _lib.call(
            "bkv_decode_range_stream_sm100",
            q.data_ptr(), q.stride(0), _lib.dtype_code(q.dtype),
            cache.data_ptr(), int(cache.shape[0]), int(cache.stride(0)), int(layout.block_size),
            int(layout.num_kv_heads), _lib.dtype_code(stat),
            block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(),
            q_points_k.contiguous().data_ptr(), q_points_v.contiguous().data_ptr(), _lib.dtype_code(q_points_k.dtype),
            o.data_ptr(), m.data_ptr(), l.data_ptr(), _stream_workspace(q.device).data_ptr(),
            int(_stream_workspace(q.device).numel()), None, batch, heads_q, int(token_lo), int(token_hi),
            float(softmax_scale), 0, 0, _lib.current_stream(q.device),
        )
        return o, m, l
    _lib.call(
        "bkv_decode_range_sm100",
        q.data_ptr(), q.stride(0), _lib.dtype_code(q.dtype),
        cache.data_ptr(), int(cache.shape[0]), int(cache.stride(0)), int(layout.block_size),
        int(layout.num_kv_heads), _lib.dtype_code(stat),
        block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(),
        q_points_k.contiguous().data_ptr(), q_points_v.contiguous().data_ptr(), _lib.dtype_code(q_points_k.dtype),
        o.data_ptr(), m.data_ptr(), l.data_ptr(), batch, heads_q, int(token_lo), int(token_hi),
        float(softmax_scale), 0, _lib.current_stream(q.device),
    )
    return o, m, l


class KvRangeExchange:
    """Receive buffers of the pushed KV-range exchange, one per rank, mapped into every other
    rank of the node through CUDA IPC (``bkv_kv_exchange_*``).  Set-up is collective: every rank
    of ``group`` constructs the object at the same point (the IPC handles travel through
    ``all_gather_object``); after that a step needs no collective.  ``rows`` = batch x query
    heads of the decode bucket.  ``close()`` is collective too."""

    def __init__(self, rows: int, device: torch.device, group=None, timeout_s: float = 2.0):
        lib = _lib.load()
        self.group, self.rows, self.device = group, int(rows), torch.device(device)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.timeout_ns = int(timeout_s * 1e9)
        self._own = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.device):
            nbytes = int(lib.bkv_kv_exchange_bytes(self.world, self.rows))
            _lib.call("bkv_kv_exchange_alloc", nbytes, ctypes.byref(self._own), handle)
            handles = [bytes(handle)]
            if self.world > 1:
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(handle), group=group)
            self._peers = []
            for r in range(self.world):
                if r == self.rank:
                    self._peers.append(self._own.value)
                    continue
                peer = ctypes.c_void_p()
                _lib.call("bkv_kv_exchange_open", (ctypes.c_ubyte * 64).from_buffer_copy(handles[r]), ctypes.byref(peer))
                self._peers.append(peer.value)
        self._peer_array = (ctypes.c_uint64 * self.world)(*self._peers)
        self.status = torch.zeros((1,), dtype=torch.int32, device=self.device)
        self.record = torch.empty((self.rows * 130,), dtype=torch.float32, device=self.device)
        if self.world > 1:
            dist.barrier(group=group)  # every buffer is mapped everywhere before the first push

    def views(self):
        """(o, m, l) views of the record the range decode writes."""
        r = self.rows
        return self.record[: r * 128].view(r, 128), self.record[r * 128 : r * 129], self.record[r * 129 :]

    def merge(self, out: torch.Tensor, out_f32: Optional[torch.Tensor] = None) -> None:
        """Push this rank's record, wait for the others' and merge into ``out`` (one kernel)."""
        # step 0: the kernel numbers the steps with a counter in this rank's buffer, so the launch is
        # the same every time and can be replayed from a captured graph
        _lib.call("bkv_kv_exchange_merge_sm100", self.record.data_ptr(), self.rows, self._peer_array, self.world, self.rank,
                  0, self.timeout_ns, out.data_ptr(), _lib.dtype_code(out.dtype), _lib.ptr(out_f32),
                  self.status.data_ptr(), _lib.current_stream(self.device))

    def check(self) -> None:
        """Host-side check (synchronises): raises when a wait of an earlier step ran out."""
        if int(self.status.item()) != 0:
            raise _lib.BkvError("bkv_kv_exchange_merge_sm100", 1, "a peer's record did not arrive within the time limit")

    def close(self) -> None:
        if self._own.value is None:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)  # nobody pushes any more
        for r, peer in enumerate(self._peers):
            if r != self.rank:
                _lib.call("bkv_kv_exchange_close", ctypes.c_void_p(peer))
        if self.world > 1:
            dist.barrier(group=self.group)  # nobody maps this buffer any more
        _lib.call("bkv_kv_exchange_free", self._own)
        self._own = ctypes.c_void_p()


def decode_kv_range_split(
    q: torch.Tensor,
    cache: torch.Tensor,
    layout: PagedLayout,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    q_points_k: torch.Tensor,
    q_points_v: torch.Tensor,
    out: torch.Tensor,
    *,
    token_lo: int,
    token_hi: int,
    softmax_scale: float,
    stat_dtype: Optional[torch.dtype] = None,
    group=None,
    exchange: Optional[KvRangeExchange] = None,
    out_f32: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Decode attention of a batch whose KV positions are split across the ranks of
    ``group``: this rank attends ``[token_lo, token_hi)`` from its own pages and leaves one
    packed record ``o | m | l`` (rows x 130 float32).  With ``exchange`` the records are pushed
    into the peers' buffers and merged by one kernel; without it they are all-gathered in ONE
    NCCL collective and merged by the combine kernel, on every rank, into ``out``
    ``(batch, heads_q, 128)``.  ``q`` must be identical on all ranks.  Buffers are kept per
    (device, rows, world), so steady-state calls allocate nothing."""
    batch, heads_q = int(q.shape[0]), int(q.shape[1])
    rows = batch * heads_q
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if exchange is not None:
        if exchange.rows != rows or exchange.world != world:
            raise ValueError("the exchange was set up for another bucket (rows) or group")
        rec, every = exchange.record, None
    else:
        key = (q.device.type, q.device.index, rows, world)
        bufs = _RECORDS.get(key)
        if bufs is None:
            rec = torch.empty((rows * 130,), dtype=torch.float32, device=q.device)
            every = torch.empty((world * rows * 130,), dtype=torch.float32, device=q.device) if world > 1 else rec
            bufs = _RECORDS[key] = (rec, every)
        rec, every = bufs
    o, m, l = rec[: rows * 128].view(rows, 128), rec[rows * 128 : rows * 129], rec[rows * 129 :]
    if q_points_k.dtype != q_points_v.dtype:
        q_points_k, q_points_v = q_points_k.float(), q_points_v.float()
    stat = stat_dtype if stat_dtype is not None else q.dtype
    ws = _stream_workspace(q.device)
    byte_tables = _byte_tables_for(q_points_k, q_points_v, int(layout.num_kv_heads))
    _lib.call(
        "bkv_decode_range_stream_sm100",
        q.data_ptr(), q.stride(0), _lib.dtype_code(q.dtype),
        cache.data_ptr(), int(cache.shape[0]), int(cache.stride(0)), int(layout.block_size),
        int(layout.num_kv_heads), _lib.dtype_code(stat),
        block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(),
        q_points_k.contiguous().data_ptr(), q_points_v.contiguous().data_ptr(), _lib.dtype_code(q_points_k.dtype),
        o.data_ptr(), m.data_ptr(), l.data_ptr(), ws.data_ptr(), int(ws.numel()), _lib.ptr(byte_tables), batch, heads_q,
        int(token_lo), int(token_hi), float(softmax_scale), 0, 0, _lib.current_stream(q.device),
    )
    if exchange is not None:
        exchange.merge(out, out_f32)
        return out
    if world > 1:
        dist.all_gather_into_tensor(every, rec, group=group)  # rank-major records
    _lib.call("bkv_combine_packed_sm100", every.data_ptr(), world, rows, out.data_ptr(), _lib.dtype_code(out.dtype),
              _lib.ptr(out_f32), _lib.current_stream(q.device))
    return out


_RECORDS: dict = {}


def _byte_tables_for(q_points_k: torch.Tensor, q_points_v: torch.Tensor, heads_kv: int) -> Optional[torch.Tensor]:
    """The decode kernel's expanded look-up tables (128 KiB per kv head) for level tables in the
    canonical ``(heads_kv * 4, 16)`` order, built on first use and kept on the K tensor for as
    long as neither tensor is modified.  None (the kernel builds its own, per launch) for tables
    the builder does not take and while a stream is being captured before the first build."""
    if q_points_k.dtype not in (torch.float16, torch.bfloat16) or q_points_k.dtype != q_points_v.dtype:
        return None
    if tuple(q_points_k.shape) != (heads_kv * 4, 16) or tuple(q_points_v.shape) != (heads_kv * 4, 16):
        return None
    if not (q_points_k.is_contiguous() and q_points_v.is_contiguous()):
        return None
    held = getattr(q_points_k, "_bkv_range_tables", None)
    if held is not None and held[0] is q_points_v and held[1] == (q_points_k._version, q_points_v._version):
        return held[2]
    if torch.cuda.is_current_stream_capturing():
        return None
    with torch.cuda.device(q_points_k.device):
        nbytes = int(_lib.load().bkv_decode_tables_bytes(heads_kv))
        tables = torch.empty((nbytes,), dtype=torch.uint8, device=q_points_k.device)
        _lib.call("bkv_decode_tables_sm100", q_points_k.data_ptr(), q_points_v.data_ptr(), _lib.dtype_code(q_points_k.dtype),
                  heads_kv, 0, tables.data_ptr(), nbytes, _lib.current_stream(q_points_k.device))
    q_points_k._bkv_range_tables = (q_points_v, (q_points_k._version, q_points_v._version), tables)
    return tables
