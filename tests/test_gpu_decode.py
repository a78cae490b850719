"""Packed decode attention parity: the CUDA path (through the launcher mirror and the
C ABI) against the float64 oracle over the same packed pages.

Tolerances (stated by the task): |out_f32 - oracle| <= 2e-3 on the un-rounded float32
result; the bf16/fp16 output must be within one unit in the last place of the rounded
oracle."""

import numpy as np
import pytest
import torch

import oracle
from beyond_kv_cache_b200 import _lib, synth
from beyond_kv_cache_b200.quant.beyond_cute import PagedLayout
from tests.helpers import KIND_TO_DTYPE, gpu_decode, oracle_cache, tables

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 2e-3


def _ulp(x: torch.Tensor, dtype) -> torch.Tensor:
    """Spacing of `dtype` at |x| (normal range)."""
    mant = 7 if dtype == torch.bfloat16 else 10
    e = torch.floor(torch.log2(x.float().abs().clamp_min(2.0**-14)))
    return torch.pow(2.0, e - mant)


def _check_rounded(out: torch.Tensor, out32: torch.Tensor, want32: np.ndarray, err: float) -> None:
    """The 16-bit output is the round-to-nearest of the kernel's own float32 result and
    sits within one unit in the last place (plus the float32 error) of the rounded oracle."""
    assert torch.equal(out, out32.to(out.dtype))
    want = torch.from_numpy(want32).to(out.dtype)
    gap = (out.float() - want.float()).abs()
    assert bool((gap <= _ulp(want, out.dtype) + 2 * err).all())


def _check(q, cache, bt, lens, heads_kv, bs, lk, lv, kind, **kw):
    out, out32, spec = gpu_decode(q, cache, bt, lens, heads_kv, bs, lk, lv, kind=kind, **kw)
    want = oracle.decode_attention(
        q.float().numpy(), cache, oracle.PageGeometry(bs, heads_kv), bt, lens,
        levels_k=lk.float().numpy(), levels_v=lv.float().numpy(), softmax_scale=synth.softmax_scale(), stat=kind,
    )
    err = float(np.abs(out32.numpy() - want).max())
    assert err <= TOL, f"max-abs {err} > {TOL} (splits={spec.num_splits})"
    _check_rounded(out, out32, want, err)
    return err, spec


def _stream_abi_call(q, cache, bt, lens, lk, lv, out, *, heads_kv, bs, stat, max_seq_len, loader=0, q_dtype=None, out_dtype=None):
    """bkv_decode_stream_sm100 straight through the C ABI (no byte tables: the kernel builds them)."""
    ws = _lib.stream_workspace(q.device)
    _lib.call("bkv_decode_stream_sm100", q.data_ptr(), q.stride(0), q_dtype if q_dtype is not None else _lib.dtype_code(q.dtype),
              cache.data_ptr(), cache.shape[0], cache.stride(0), bs, heads_kv, stat, bt.data_ptr(), bt.stride(0),
              lens.data_ptr(), lk.data_ptr(), lv.data_ptr(), _lib.BKV_F16, out.data_ptr(),
              out_dtype if out_dtype is not None else _lib.dtype_code(out.dtype), None, ws.data_ptr(), ws.numel(), None,
              q.shape[0], q.shape[1], max_seq_len, synth.softmax_scale(), 0, loader, _lib.current_stream(q.device))
    torch.cuda.synchronize()


def test_config0_against_reference_output(golden):
    """Config 0 (float32 Q, fp16 statistics): the numbers the reference's own code
    produced (fp32 SDPA over its read-back cache), within 2e-3, straight through the
    C ABI - split grid with 1 and 4 splits, persistent schedule with both loaders; then the
    bf16-query form through the launcher mirror against the oracle."""
    g = golden["config0"]
    q, k, v = synth.config0_inputs(0)
    lk, tk, lv, tv = tables(8, 0, per_group=False)
    geo = oracle.PageGeometry(16, 8)
    bt = g["c0_block_table"]
    slots = (bt.astype(np.int64)[:, np.arange(1024) // 16] * 16 + np.arange(1024) % 16).reshape(-1)
    cache = np.zeros((256, geo.block_i32), dtype=np.int32)
    oracle.write_pages(cache, geo, slots, k, v, thresholds_k=tk.float().numpy(), thresholds_v=tv.float().numpy(), stat="f16")
    qd, cd, btd = torch.from_numpy(q).to(DEV), torch.from_numpy(cache).to(DEV), torch.from_numpy(bt).to(DEV)
    lens = torch.full((4,), 1024, dtype=torch.int32, device=DEV)
    lkd, lvd = lk.to(DEV), lv.to(DEV)
    out = torch.empty((4, 32, 128), dtype=torch.float32, device=DEV)
    for splits in (1, 4):
        ws = [torch.empty((splits, 4, 32, 128), device=DEV), torch.empty((splits, 4, 32), device=DEV), torch.empty((splits, 4, 32), device=DEV)]
        out.zero_()
        _lib.call("bkv_decode_sm100", qd.data_ptr(), qd.stride(0), _lib.BKV_F32, cd.data_ptr(), cd.shape[0], cd.stride(0),
                  16, 8, _lib.BKV_F16, btd.data_ptr(), btd.stride(0), lens.data_ptr(), lkd.data_ptr(), lvd.data_ptr(),
                  _lib.BKV_F16, out.data_ptr(), _lib.BKV_F32, None, ws[0].data_ptr(), ws[1].data_ptr(), ws[2].data_ptr(),
                  splits, 4, 32, 1024, synth.softmax_scale(), 0, _lib.current_stream(qd.device))
        torch.cuda.synchronize()
        assert np.abs(out.cpu().numpy() - g["c0_out"]).max() <= TOL
    for loader in (0, 1):
        out.zero_()
        _stream_abi_call(qd, cd, btd, lens, lkd, lvd, out, heads_kv=8, bs=16, stat=_lib.BKV_F16, max_seq_len=1024, loader=loader)
        assert np.abs(out.cpu().numpy() - g["c0_out"]).max() <= TOL
    qb = torch.from_numpy(q).to(torch.bfloat16)
    for kw in ({"splits": 2}, {"splits": 0}, {"splits": 0, "loader": 1}):
        _check(qb, cache, bt, [1024] * 4, 8, 16, lk, lv, "f16", **kw)


# every schedule the launcher offers: the split grid with fixed counts, the persistent one with both loaders
SCHEDULES = [{"splits": 1}, {"splits": 3}, {"splits": 0}, {"splits": 0, "loader": 1}]


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("bs,gqa,heads_kv", [(16, 4, 8), (64, 4, 2), (128, 8, 2), (32, 2, 4), (16, 1, 4)])
def test_ragged_batch(bs, gqa, heads_kv, kind):
    lens = [0, 1, bs - 1, bs, bs + 1, 5 * bs + 7, 333, 2]
    lk, tk, lv, tv = tables(heads_kv, 21)
    cache, bt = oracle_cache(lens, heads_kv, bs, kind, 77, tk.float().numpy(), tv.float().numpy())
    rng = np.random.default_rng(9)
    q = torch.from_numpy(rng.standard_normal((len(lens), heads_kv * gqa, 128)).astype(np.float32)).to(KIND_TO_DTYPE[kind])
    for kw in SCHEDULES:
        _check(q, cache, bt, lens, heads_kv, bs, lk, lv, kind, **kw)
        out, out32, _ = gpu_decode(q, cache, bt, lens, heads_kv, bs, lk, lv, kind=kind, **kw)
        assert not out[0].any() and not out32[0].any()  # seq_len 0 -> zeros


def test_long_context_many_splits():
    lens = [16 * 1024 + 5, 9000]
    lk, tk, lv, tv = tables(2, 3)
    cache, bt = oracle_cache(lens, 2, 16, "bf16", 5, tk.float().numpy(), tv.float().numpy())
    q = torch.from_numpy(np.random.default_rng(2).standard_normal((2, 8, 128)).astype(np.float32)).to(torch.bfloat16)
    for kw in ({"splits": 1}, {"splits": 7}, {"splits": 32}, {"splits": 0}, {"splits": 0, "loader": 1}):
        _check(q, cache, bt, lens, 2, 16, lk, lv, "bf16", **kw)


def test_one_request_of_128k_tokens():
    """A single 131 072-token request at the benchmark geometry (8 KV heads, 4 query heads each,
    16-token pages, 8192 pages): every CTA's share lies inside the one request, so each leaves one
    partial and the last CTA of every head merges a chain of about 18 of them.  The pages are
    filled by the encode kernel (held bit-exact to the oracle by its own tests) over random words;
    the attention is checked against the oracle's float64 evaluation of those very pages."""
    from beyond_kv_cache_b200.quant.beyond_cute import write_tokens_to_paged_cache

    n, heads_kv, bs = 131072, 8, 16
    lk, tk, lv, tv = tables(heads_kv, 3, per_group=False)
    layout = PagedLayout.build_hnd(bs, heads_kv, 128, 4, 32, 32)
    bt_d, num_pages = synth.random_block_table(1, n // bs, seed=41, device=DEV, spare_pages=2)
    cache_d = torch.randint(-(2**31), 2**31 - 1, (num_pages, layout.block_i32), dtype=torch.int64, device=DEV).to(torch.int32)
    k, v = synth.make_kv(n, heads_kv, seed=4, device=DEV, dtype=torch.float16)
    write_tokens_to_paged_cache(cache_d, layout, bt_d, synth.slots_for(bt_d, bs, 0, n), k, v, q_points_k=lk.to(DEV),
                                q_points_v=lv.to(DEV), thresholds_k=tk.to(DEV), thresholds_v=tv.to(DEV), require_fast=True)
    cache, bt = cache_d.cpu().numpy(), bt_d.cpu().numpy()
    del cache_d, k, v
    q = torch.from_numpy(np.random.default_rng(6).standard_normal((1, 32, 128)).astype(np.float32)).to(torch.bfloat16)
    want = oracle.decode_attention(q.float().numpy(), cache, oracle.PageGeometry(bs, heads_kv), bt, [n],
                                   levels_k=lk.float().numpy(), levels_v=lv.float().numpy(),
                                   softmax_scale=synth.softmax_scale(), stat="f16")
    for loader in (0, 1):
        out, out32, _ = gpu_decode(q, cache, bt, [n], heads_kv, bs, lk, lv, kind="f16", loader=loader)
        err = float(np.abs(out32.numpy() - want).max())
        assert err <= TOL, (loader, err)
        _check_rounded(out, out32, want, err)


@pytest.mark.parametrize("loader", [0, 1])
@pytest.mark.parametrize("bs,heads_kv,gqa,kind", [(16, 2, 4, "bf16"), (64, 4, 8, "f16"), (32, 3, 2, "bf16")])
def test_persistent_schedule_cut_requests(bs, heads_kv, gqa, kind, loader):
    """Many ragged requests under the persistent schedule: workers cut requests at arbitrary
    tiles, so whole-request outputs, two-part and many-part chains of partials and empty
    requests all occur in one launch; run twice on one workspace, which the first launch must
    leave ready for the second."""
    rng = np.random.default_rng(100 + bs)
    lens = [int(v) for v in rng.integers(0, 900, size=37)]
    lens[3], lens[11], lens[20], lens[36] = 0, 4100, 1, 2500
    lk, tk, lv, tv = tables(heads_kv, 31)
    cache, bt = oracle_cache(lens, heads_kv, bs, kind, 55, tk.float().numpy(), tv.float().numpy())
    q = torch.from_numpy(rng.standard_normal((len(lens), heads_kv * gqa, 128)).astype(np.float32)).to(KIND_TO_DTYPE[kind])
    _check(q, cache, bt, lens, heads_kv, bs, lk, lv, kind, loader=loader)
    out, out32, _ = gpu_decode(q, cache, bt, lens, heads_kv, bs, lk, lv, kind=kind, loader=loader)
    assert not out[3].any() and not out32[3].any()  # seq_len 0 -> zeros
    # same workspace, different batches back to back
    dev_q, dev_c, dev_bt = q.to(DEV), torch.from_numpy(cache).to(DEV), torch.from_numpy(bt).to(DEV)
    stat = _lib.dtype_code(KIND_TO_DTYPE[kind])
    ws = _lib.stream_workspace(dev_q.device)
    want = oracle.decode_attention(q.float().numpy(), cache, oracle.PageGeometry(bs, heads_kv), bt, lens,
                                   levels_k=lk.float().numpy(), levels_v=lv.float().numpy(),
                                   softmax_scale=synth.softmax_scale(), stat=kind)
    lkd, lvd = lk.to(DEV), lv.to(DEV)
    for trial, scale_lens in enumerate((1.0, 0.5, 1.0)):
        cur = [int(n * scale_lens) for n in lens]
        lens_d = torch.tensor(cur, dtype=torch.int32, device=DEV)
        got = torch.empty(q.shape, dtype=torch.float32, device=DEV)
        _lib.call("bkv_decode_stream_sm100", dev_q.data_ptr(), dev_q.stride(0), _lib.dtype_code(dev_q.dtype), dev_c.data_ptr(),
                  dev_c.shape[0], dev_c.stride(0), bs, heads_kv, stat, dev_bt.data_ptr(), dev_bt.stride(0), lens_d.data_ptr(),
                  lkd.data_ptr(), lvd.data_ptr(), _lib.BKV_F16, got.data_ptr(), _lib.BKV_F32, None, ws.data_ptr(), ws.numel(),
                  None, len(cur), q.shape[1], bt.shape[1] * bs, synth.softmax_scale(), 0, loader, _lib.current_stream(dev_q.device))
        torch.cuda.synchronize()
        if scale_lens == 1.0:
            assert np.abs(got.cpu().numpy() - want).max() <= TOL, trial
    assert not bool(ws[65792 : 65792 + (1 << 22)].any())  # the request counters are back at zero


@pytest.mark.parametrize("loader", [0, 1])
def test_persistent_schedule_many_heads_tiny_requests(loader):
    """Sixteen KV heads and requests of one to three tiles: one CTA per head, shares shorter than
    the straddle allowance, most warps without work."""
    lens = [1, 17, 0, 40, 16]
    lk, tk, lv, tv = tables(16, 13)
    cache, bt = oracle_cache(lens, 16, 16, "f16", 21, tk.float().numpy(), tv.float().numpy())
    q = torch.from_numpy(np.random.default_rng(8).standard_normal((len(lens), 32, 128)).astype(np.float32)).to(torch.float16)
    _check(q, cache, bt, lens, 16, 16, lk, lv, "f16", loader=loader)


def test_persistent_schedule_large_batch():
    """More requests than the in-kernel request table holds (1024): the prefix sums come
    from the planning kernel.  1500 requests of 0-39 tokens, some empty: with one to three
    tokens nothing averages a rounding error, so this is the case that holds the kernel's
    operand precision (exact fp16 queries, exact high + low parts of p * scale_v) to the bound."""
    rng = np.random.default_rng(12)
    lens = [int(v) for v in rng.integers(0, 40, size=1500)]
    lens[0], lens[1499] = 0, 333
    lk, tk, lv, tv = tables(2, 5)
    cache, bt = oracle_cache(lens, 2, 16, "bf16", 9, tk.float().numpy(), tv.float().numpy())
    q = torch.from_numpy(rng.standard_normal((len(lens), 8, 128)).astype(np.float32)).to(torch.bfloat16)
    out, out32, _ = gpu_decode(q, cache, bt, lens, 2, 16, lk, lv, kind="bf16")
    want = oracle.decode_attention(q.float().numpy(), cache, oracle.PageGeometry(16, 2), bt, lens,
                                   levels_k=lk.float().numpy(), levels_v=lv.float().numpy(),
                                   softmax_scale=synth.softmax_scale(), stat="bf16")
    gap = np.abs(out32.numpy() - want)
    assert float(gap.max()) <= TOL, float(gap.max())
    assert torch.equal(out, out32.to(out.dtype))
    assert not out[0].any()


def test_prepared_byte_tables_give_the_same_bits():
    """The look-up tables expanded once per layer (bkv_decode_tables_sm100, attached by
    prepare_runtime_qpoints) and the ones the kernel builds itself are the same tables."""
    lens = [700, 130, 0, 64, 2049]
    lk, tk, lv, tv = tables(2, 17)
    cache, bt = oracle_cache(lens, 2, 16, "bf16", 100, tk.float().numpy(), tv.float().numpy())
    q = torch.from_numpy(np.random.default_rng(1).standard_normal((len(lens), 8, 128)).astype(np.float32)).to(torch.bfloat16)
    _, with_tables, _ = gpu_decode(q, cache, bt, lens, 2, 16, lk, lv, kind="bf16")  # launcher: prepared tables
    qd, cd, btd = q.to(DEV), torch.from_numpy(cache).to(DEV), torch.from_numpy(bt).to(DEV)
    lens_d = torch.tensor(lens, dtype=torch.int32, device=DEV)
    own = torch.empty(q.shape, dtype=torch.float32, device=DEV)
    _stream_abi_call(qd, cd, btd, lens_d, lk.to(DEV), lv.to(DEV), own, heads_kv=2, bs=16, stat=_lib.BKV_BF16,
                     max_seq_len=bt.shape[1] * 16)
    assert torch.equal(own.cpu(), with_tables)


def test_fused_qkv_query_view_and_bucket_truncation():
    lens = [100, 40]
    lk, tk, lv, tv = tables(2, 4)
    cache, bt = oracle_cache(lens, 2, 16, "f16", 6, tk.float().numpy(), tv.float().numpy())
    rng = np.random.default_rng(3)
    fused = torch.from_numpy(rng.standard_normal((2, 8 + 4, 128)).astype(np.float32)).to(torch.float16)
    q = fused[:, :8]  # batch stride 12*128
    _check(q, cache, bt, lens, 2, 16, lk, lv, "f16", splits=2)
    # a launch bucket shorter than a request attends only the bucket (reference semantics)
    out, out32, _ = gpu_decode(q.contiguous(), cache, bt, lens, 2, 16, lk, lv, kind="f16", max_seq_len=64)
    want = oracle.decode_attention(q.float().numpy(), cache, oracle.PageGeometry(16, 2), bt, [64, 40],
                                   levels_k=lk.float().numpy(), levels_v=lv.float().numpy(),
                                   softmax_scale=synth.softmax_scale(), stat="f16")
    assert np.abs(out32.numpy() - want).max() <= TOL


def test_kv_range_partials_merge_to_full():
    """bkv_decode_range_sm100 over disjoint token ranges + bkv_combine_sm100 == full decode."""
    lens = [700, 130, 0, 64]
    lk, tk, lv, tv = tables(2, 8)
    cache, bt = oracle_cache(lens, 2, 16, "bf16", 10, tk.float().numpy(), tv.float().numpy())
    q = torch.from_numpy(np.random.default_rng(4).standard_normal((4, 8, 128)).astype(np.float32)).to(torch.bfloat16)
    want = oracle.decode_attention(q.float().numpy(), cache, oracle.PageGeometry(16, 2), bt, lens,
                                   levels_k=lk.float().numpy(), levels_v=lv.float().numpy(),
                                   softmax_scale=synth.softmax_scale(), stat="bf16")
    qd, cd, btd = q.to(DEV), torch.from_numpy(cache).to(DEV), torch.from_numpy(bt).to(DEV)
    lens_d = torch.tensor(lens, dtype=torch.int32, device=DEV)
    lkd, lvd = lk.to(DEV), lv.to(DEV)
    ranges = [(0, 256), (256, 512), (512, 768)]
    o = torch.empty((len(ranges), 4, 8, 128), dtype=torch.float32, device=DEV)
    m = torch.empty((len(ranges), 4, 8), dtype=torch.float32, device=DEV)
    l = torch.empty_like(m)
    stream = _lib.current_stream(qd.device)
    for i, (lo, hi) in enumerate(ranges):
        _lib.call("bkv_decode_range_sm100", qd.data_ptr(), qd.stride(0), _lib.BKV_BF16, cd.data_ptr(), cd.shape[0],
                  cd.stride(0), 16, 2, _lib.BKV_BF16, btd.data_ptr(), btd.stride(0), lens_d.data_ptr(),
                  lkd.data_ptr(), lvd.data_ptr(), _lib.BKV_F16, o[i].data_ptr(), m[i].data_ptr(), l[i].data_ptr(),
                  4, 8, lo, hi, synth.softmax_scale(), 0, stream)
    out = torch.empty((4, 8, 128), dtype=torch.float32, device=DEV)
    _lib.call("bkv_combine_sm100", o.data_ptr(), m.data_ptr(), l.data_ptr(), len(ranges), 32, out.data_ptr(),
              _lib.BKV_F32, None, stream)
    torch.cuda.synchronize()
    assert np.abs(out.cpu().numpy() - want).max() <= TOL
    # the partials themselves agree with the oracle's partials after normalisation
    po, pm, pl = oracle.decode_attention(q.float().numpy(), cache, oracle.PageGeometry(16, 2), bt, lens,
                                         levels_k=lk.float().numpy(), levels_v=lv.float().numpy(),
                                         softmax_scale=synth.softmax_scale(), stat="bf16",
                                         kv_range=ranges[1], return_partials=True)
    got = (o[1] / l[1].clamp_min(1e-30).unsqueeze(-1)).cpu().numpy()
    ref = po / np.maximum(pl, 1e-30)[..., None]
    live = pl > 0
    assert np.abs(got[live] - ref[live]).max() <= TOL
    assert not (l[1].cpu().numpy()[~live] != 0).any()


def test_kv_range_partials_under_the_persistent_schedule():
    """parallel.decode_range_partial (bkv_decode_range_stream_sm100) over disjoint token ranges,
    one of them a single very long request cut into many parts, + bkv_combine_sm100 == full
    decode; empty ranges give (0, -inf, 0)."""
    from beyond_kv_cache_b200 import parallel

    lens = [9000, 130, 0, 64]
    lk, tk, lv, tv = tables(2, 8)
    cache, bt = oracle_cache(lens, 2, 16, "bf16", 10, tk.float().numpy(), tv.float().numpy())
    q = torch.from_numpy(np.random.default_rng(4).standard_normal((4, 8, 128)).astype(np.float32)).to(torch.bfloat16)
    want = oracle.decode_attention(q.float().numpy(), cache, oracle.PageGeometry(16, 2), bt, lens,
                                   levels_k=lk.float().numpy(), levels_v=lv.float().numpy(),
                                   softmax_scale=synth.softmax_scale(), stat="bf16")
    layout = PagedLayout.build_hnd(16, 2, 128, 4, 32, 32)
    qd, cd, btd = q.to(DEV), torch.from_numpy(cache).to(DEV), torch.from_numpy(bt).to(DEV)
    lens_d = torch.tensor(lens, dtype=torch.int32, device=DEV)
    ranges = [(0, 48), (48, 4096), (4096, 16384)]
    parts = [parallel.decode_range_partial(qd, cd, layout, btd, lens_d, lk.to(DEV), lv.to(DEV), token_lo=lo, token_hi=hi,
                                           softmax_scale=synth.softmax_scale(), stat_dtype=torch.bfloat16)
             for lo, hi in ranges]
    o = torch.stack([p[0] for p in parts]).contiguous()
    m = torch.stack([p[1] for p in parts]).contiguous()
    l = torch.stack([p[2] for p in parts]).contiguous()
    out = torch.empty((4, 8, 128), dtype=torch.float32, device=DEV)
    _lib.call("bkv_combine_sm100", o.data_ptr(), m.data_ptr(), l.data_ptr(), len(ranges), 32, out.data_ptr(),
              _lib.BKV_F32, None, _lib.current_stream(qd.device))
    torch.cuda.synchronize()
    assert np.abs(out.cpu().numpy() - want).max() <= TOL
    assert not l[2][8:].any() and not o[2][8:].any()  # only request 0 reaches beyond 4096
    assert bool(torch.isinf(m[2][8:]).all())


def test_launcher_rejects_bad_contracts():
    from beyond_kv_cache_b200.quant.fa4_cute import beyond_mixed_decode_runtime as rt

    layout = PagedLayout.build_hnd(16, 2, 128, 4, 32, 32)
    cache = torch.zeros((4, layout.block_i32), dtype=torch.int32, device=DEV)
    bt = torch.zeros((1, 4), dtype=torch.int32, device=DEV)
    q = torch.zeros((1, 8, 128), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError, match="multiple of page_size"):
        rt.make_runtime_spec(q=q, cache=cache, layout=layout, block_table=bt, heads_q=8, max_seq_len=20)
    with pytest.raises(ValueError, match="block-table capacity"):
        rt.make_runtime_spec(q=q, cache=cache, layout=layout, block_table=bt, heads_q=8, max_seq_len=128)
    with pytest.raises(ValueError, match="ABI v2"):
        rt.make_runtime_spec(q=q, cache=cache, layout=PagedLayout.build(16, 2, 128, 4, 32, 32), block_table=bt, heads_q=8, max_seq_len=64)
    with pytest.raises(ValueError, match="CUDA tensors"):
        rt.make_runtime_spec(q=q.cpu(), cache=cache, layout=layout, block_table=bt, heads_q=8, max_seq_len=64)
    rk, rv = rt.prepare_runtime_qpoints(torch.rand(8, 16, device=DEV), torch.rand(8, 16, device=DEV), heads_kv=2)
    for splits in (2, 0):  # split grid: partial tensors; persistent schedule: its scratch
        spec = rt.make_runtime_spec(q=q, cache=cache, layout=layout, block_table=bt, heads_q=8, max_seq_len=64, num_splits=splits)
        assert spec.persistent == (splits == 0)
        with pytest.raises(ValueError, match="workspace"):
            rt.run_nonuniform_decode(spec=spec, q=q, cache=cache, layout=layout, block_table=bt,
                                     seq_lens=torch.ones(1, dtype=torch.int32, device=DEV), k_qpoints_lane_major=rk,
                                     v_qpoints_code_major=rv, out=torch.empty_like(q), workspace={}, softmax_scale=0.1)
    ws = rt.allocate_runtime_workspace(spec, device=q.device)
    assert ws["o_partial"].numel() == 0 and "stream" in ws  # nothing would read split partials here
    with pytest.raises(ValueError, match="invalid argument"):  # the maximum is taken before scaling
        rt.run_nonuniform_decode(spec=spec, q=q, cache=cache, layout=layout, block_table=bt,
                                 seq_lens=torch.ones(1, dtype=torch.int32, device=DEV), k_qpoints_lane_major=rk,
                                 v_qpoints_code_major=rv, out=torch.empty_like(q), workspace=ws, softmax_scale=-0.1)


