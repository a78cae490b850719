"""vLLM attention-backend boundary, driven the way the reference's own test drives it
(tests/runtime/vllm/test_page_table_backend_exact.py): construct the impl, hand it a
metadata namespace, call forward()."""

import math
import types

import numpy as np
import pytest
import torch

import oracle
from beyond_kv_cache_b200.runtime.vllm import packed_backend as mod
from tests.helpers import bits16, tables

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _impl(num_heads=8, num_kv_heads=2):
    return mod.BeyondPackedImpl(num_heads, 128, 1.0 / math.sqrt(128), num_kv_heads=num_kv_heads)


def test_backend_static_contract():
    b = mod.BeyondPackedBackend
    assert b.get_name() == "CUSTOM" and b.forward_includes_kv_cache_update
    assert b.get_kv_cache_shape(10, 128, 8, 128) == (10, 8 * 5120)
    assert b.get_kv_cache_shape(3, 16, 8, 128) == (3, 5120)
    assert b.supports_block_size(16) and not b.supports_block_size(48)
    assert mod.BeyondPackedSpec(128, 8, 128).real_page_size_bytes == 8 * 5120 * 4
    with pytest.raises(ValueError):
        b.get_kv_cache_shape(1, 48, 8, 128)


def test_prefill_then_decode_steps_match_oracle():
    rng = np.random.default_rng(7)
    heads_kv, heads_q, bs = 2, 8, 16
    lens = [37, 16, 70]
    lk, tk, lv, tv = tables(heads_kv, 9)
    impl = _impl(heads_q, heads_kv)
    impl.set_quant_tables(lk.to(DEV), tk.to(DEV), lv.to(DEV), tv.to(DEV))
    layout_words = mod.BeyondPackedBackend.get_kv_cache_shape(16, bs, heads_kv, 128)[1]
    cache = torch.zeros((16, layout_words), dtype=torch.int32, device=DEV)
    geo = oracle.PageGeometry(bs, heads_kv)
    ref_cache = np.zeros((16, geo.block_i32), dtype=np.int32)
    bt = torch.tensor([[3, 1, 4, 9, 15, -1], [7, 2, -1, -1, -1, -1], [0, 5, 6, 8, 10, 11]], dtype=torch.int32, device=DEV)
    bt_np = bt.cpu().numpy()

    # ---- prefill: every request's query covers its whole sequence ----
    total = sum(lens)
    q = torch.from_numpy(rng.standard_normal((total, heads_q, 128)).astype(np.float32)).to(torch.bfloat16).to(DEV)
    k = torch.from_numpy(rng.standard_normal((total, heads_kv, 128)).astype(np.float32)).to(torch.bfloat16).to(DEV)
    v = torch.from_numpy(rng.standard_normal((total, heads_kv, 128)).astype(np.float32)).to(torch.bfloat16).to(DEV)
    k_raw, v_raw = k.float().cpu().numpy(), v.float().cpu().numpy()
    starts = np.concatenate([[0], np.cumsum(lens)])
    slots = np.concatenate([bt_np[r].astype(np.int64)[np.arange(n) // bs] * bs + np.arange(n) % bs for r, n in enumerate(lens)])
    meta = types.SimpleNamespace(num_actual_tokens=total, query_start_loc=torch.tensor(starts, dtype=torch.int32, device=DEV),
                                 seq_lens=torch.tensor(lens, dtype=torch.int32, device=DEV), block_table=bt,
                                 slot_mapping=torch.tensor(slots, dtype=torch.int64, device=DEV), max_query_len=max(lens),
                                 max_seq_len=max(lens))
    out = impl.forward(None, q, k, v, cache, meta)
    ek, ev = oracle.write_pages(ref_cache, geo, slots, k_raw, v_raw, thresholds_k=tk.float().numpy(),
                                thresholds_v=tv.float().numpy(), stat="bf16")
    assert np.array_equal(cache.cpu().numpy(), ref_cache)
    k_hat = oracle.decode_groups(ek["codes"], lk.float().numpy(), ek["scale_bits"], ek["mn_bits"], stat="bf16")
    assert np.array_equal(bits16(k), oracle.round_to_stat(k_hat, "bf16"))  # K handed to attention == cache contents
    # causal attention over the rounded K/V
    for r, n in enumerate(lens):
        s, e = starts[r], starts[r + 1]
        kk, vv = k.float().cpu().numpy()[s:e], v.float().cpu().numpy()[s:e]
        qq = q.float().cpu().numpy()[s:e]
        for t in (0, n - 1):
            sc = np.einsum("hd,shd->hs", qq[t].astype(np.float64), np.repeat(kk[: t + 1], 4, axis=1)) / math.sqrt(128)
            p = np.exp(sc - sc.max(1, keepdims=True))
            want = np.einsum("hs,shd->hd", p / p.sum(1, keepdims=True), np.repeat(vv[: t + 1], 4, axis=1))
            assert np.abs(out[s + t].float().cpu().numpy() - want).max() < 2e-2  # bf16 SDPA

    # ---- two decode steps: append one token per request, attend the whole packed context ----
    for step in range(2):
        lens = [n + 1 for n in lens]
        qd = torch.from_numpy(rng.standard_normal((3, heads_q, 128)).astype(np.float32)).to(torch.bfloat16).to(DEV)
        kd = torch.from_numpy(rng.standard_normal((3, heads_kv, 128)).astype(np.float32)).to(torch.bfloat16).to(DEV)
        vd = torch.from_numpy(rng.standard_normal((3, heads_kv, 128)).astype(np.float32)).to(torch.bfloat16).to(DEV)
        pos = np.array([n - 1 for n in lens])
        slots = np.array([bt_np[r, pos[r] // bs] * bs + pos[r] % bs for r in range(3)], dtype=np.int64)
        meta = types.SimpleNamespace(num_actual_tokens=3, query_start_loc=torch.arange(4, dtype=torch.int32, device=DEV),
                                     seq_lens=torch.tensor(lens, dtype=torch.int32, device=DEV), block_table=bt,
                                     slot_mapping=torch.tensor(slots, dtype=torch.int64, device=DEV), max_query_len=1,
                                     max_seq_len=max(lens))
        out = torch.empty_like(qd)
        res = impl.forward(None, qd, kd, vd, cache, meta, output=out)
        assert res is out
        oracle.write_pages(ref_cache, geo, slots, kd.float().cpu().numpy(), vd.float().cpu().numpy(),
                           thresholds_k=tk.float().numpy(), thresholds_v=tv.float().numpy(), stat="bf16")
        assert np.array_equal(cache.cpu().numpy(), ref_cache)
        want = oracle.decode_attention(qd.float().cpu().numpy(), ref_cache, geo, bt_np, lens, levels_k=lk.float().numpy(),
                                       levels_v=lv.float().numpy(), softmax_scale=impl.scale, stat="bf16")
        got = out.float().cpu().numpy()
        assert np.abs(got - want).max() <= 2e-3 + np.abs(want).max() * 2.0**-8  # bf16 output rounding


def test_chunked_prefill_reads_back_the_whole_context():
    """Every request brings a chunk of several query tokens behind context that is already in
    the packed cache (the plan the reference serves at packed_backend.py:2523-2625, tested there
    by tests/runtime/vllm/test_page_table_backend_exact.py:125-245): the chunk is committed to
    the cache bit-exactly, and its queries attend, causally, the dequantised context plus chunk."""
    rng = np.random.default_rng(11)
    heads_kv, heads_q, bs = 2, 8, 16
    ctx, chunk = [21, 40, 5], [7, 16, 30]
    lk, tk, lv, tv = tables(heads_kv, 3)
    impl = _impl(heads_q, heads_kv)
    impl.set_quant_tables(lk.to(DEV), tk.to(DEV), lv.to(DEV), tv.to(DEV))
    geo = oracle.PageGeometry(bs, heads_kv)
    ref_cache = rng.integers(-(2**31), 2**31, (16, geo.block_i32)).astype(np.int32)
    bt_np = np.array([[3, 1, 4, -1], [7, 2, 12, 13], [0, 5, 6, -1]], dtype=np.int32)

    def slots_of(r, lo, hi):
        pos = np.arange(lo, hi)
        return bt_np[r].astype(np.int64)[pos // bs] * bs + pos % bs

    # the context already in the cache (written by the oracle)
    for r, n in enumerate(ctx):
        kc = oracle.stat_to_f32(oracle.round_to_stat(rng.standard_normal((n, heads_kv, 128)).astype(np.float32), "bf16"), "bf16")
        vc = oracle.stat_to_f32(oracle.round_to_stat(rng.standard_normal((n, heads_kv, 128)).astype(np.float32), "bf16"), "bf16")
        oracle.write_pages(ref_cache, geo, slots_of(r, 0, n), kc, vc, thresholds_k=tk.float().numpy(),
                           thresholds_v=tv.float().numpy(), stat="bf16")
    cache = torch.from_numpy(ref_cache.copy()).to(DEV)
    total = sum(chunk)
    q = torch.from_numpy(rng.standard_normal((total, heads_q, 128)).astype(np.float32)).to(torch.bfloat16).to(DEV)
    k = torch.from_numpy(rng.standard_normal((total, heads_kv, 128)).astype(np.float32)).to(torch.bfloat16).to(DEV)
    v = torch.from_numpy(rng.standard_normal((total, heads_kv, 128)).astype(np.float32)).to(torch.bfloat16).to(DEV)
    starts = np.concatenate([[0], np.cumsum(chunk)])
    seq = [c + n for c, n in zip(ctx, chunk)]
    slots = np.concatenate([slots_of(r, ctx[r], seq[r]) for r in range(3)])
    meta = types.SimpleNamespace(num_actual_tokens=total, query_start_loc=torch.tensor(starts, dtype=torch.int32, device=DEV),
                                 seq_lens=torch.tensor(seq, dtype=torch.int32, device=DEV),
                                 block_table=torch.from_numpy(bt_np).to(DEV),
                                 slot_mapping=torch.tensor(slots, dtype=torch.int64, device=DEV), max_query_len=max(chunk),
                                 max_seq_len=max(seq))
    k_before = k.clone()
    out = impl.forward(None, q, k, v, cache, meta)
    assert torch.equal(k, k_before)  # this plan does not reconstruct in place
    oracle.write_pages(ref_cache, geo, slots, k.float().cpu().numpy(), v.float().cpu().numpy(),
                       thresholds_k=tk.float().numpy(), thresholds_v=tv.float().numpy(), stat="bf16")
    assert np.array_equal(cache.cpu().numpy(), ref_cache)
    for r in range(3):
        pages = (seq[r] + bs - 1) // bs
        k_hat, v_hat = oracle.read_request(ref_cache, geo, bt_np[r, :pages], seq[r], levels_k=lk.float().numpy(),
                                           levels_v=lv.float().numpy(), stat="bf16")
        k_hat = oracle.stat_to_f32(oracle.round_to_stat(k_hat, "bf16"), "bf16")  # the dense view is bf16
        v_hat = oracle.stat_to_f32(oracle.round_to_stat(v_hat, "bf16"), "bf16")
        qq = q.float().cpu().numpy()[starts[r] : starts[r + 1]]
        for t in (0, chunk[r] // 2, chunk[r] - 1):
            upto = ctx[r] + t + 1
            sc = np.einsum("hd,shd->hs", qq[t].astype(np.float64), np.repeat(k_hat[:upto], 4, axis=1)) / math.sqrt(128)
            pr = np.exp(sc - sc.max(1, keepdims=True))
            want = np.einsum("hs,shd->hd", pr / pr.sum(1, keepdims=True), np.repeat(v_hat[:upto], 4, axis=1))
            assert np.abs(out[starts[r] + t].float().cpu().numpy() - want).max() < 2e-2  # bf16 SDPA


def test_unsupported_plans_fail_closed():
    impl = _impl()
    cache = torch.zeros((4, 2 * 16 * 40), dtype=torch.int32, device=DEV)
    q = torch.zeros((4, 8, 128), dtype=torch.bfloat16, device=DEV)
    kv = torch.zeros((4, 2, 128), dtype=torch.bfloat16, device=DEV)
    assert not impl.forward(None, q, kv, kv, cache, None).any()
    # a decode request next to a chunk of another request: no homogeneous plan covers it
    meta = types.SimpleNamespace(num_actual_tokens=4, query_start_loc=torch.tensor([0, 1, 4], dtype=torch.int32, device=DEV),
                                 seq_lens=torch.tensor([10, 10], dtype=torch.int32, device=DEV),
                                 block_table=torch.zeros((2, 4), dtype=torch.int32, device=DEV),
                                 slot_mapping=torch.arange(4, device=DEV), max_query_len=3, max_seq_len=10)
    with pytest.raises(NotImplementedError, match="mixed or chunked-prefill"):
        impl.forward(None, q, kv, kv, cache, meta)
    with pytest.raises(NotImplementedError, match="output quantization"):
        impl.forward(None, q, kv, kv, cache, meta, output_scale=torch.ones(1))
    with pytest.raises(RuntimeError, match="shared dtype"):
        impl.forward(None, q.float(), kv, kv, cache, meta)


def test_table_classification_is_not_inherited_through_a_reused_address():
    """A sorted threshold table is freed and an unsorted one of the same shape takes its place
    (the caching allocator hands out the same address): the writer must count thresholds for the
    new table instead of searching it."""
    from beyond_kv_cache_b200.quant import beyond_cute as bc

    rng = np.random.default_rng(5)
    lk, tk, lv, tv = tables(2, 1)
    layout = bc.PagedLayout.build_hnd(16, 2, 128, 4, 32, 32)
    geo = oracle.PageGeometry(16, 2)
    k = torch.from_numpy(rng.standard_normal((16, 2, 128)).astype(np.float32)).to(torch.bfloat16).to(DEV)
    slots = torch.arange(16, dtype=torch.int64, device=DEV)
    shuffled = tk.clone()
    shuffled[:, [2, 9]] = shuffled[:, [9, 2]]  # still 15 thresholds per table, no longer ascending
    results = []
    addresses = []
    for thr in (tk, shuffled):
        thr_d = thr.to(DEV)  # a fresh device tensor per round; the first is freed before the second exists
        addresses.append(thr_d.data_ptr())
        cache = torch.zeros((1, layout.block_i32), dtype=torch.int32, device=DEV)
        bc.write_tokens_to_paged_cache(cache, layout, None, slots, k, k, q_points_k=lk.to(DEV), q_points_v=lv.to(DEV),
                                       thresholds_k=thr_d, thresholds_v=thr_d, require_fast=True)
        want = np.zeros((1, geo.block_i32), dtype=np.int32)
        oracle.write_pages(want, geo, slots.cpu().numpy(), k.float().cpu().numpy(), k.float().cpu().numpy(),
                           thresholds_k=thr.float().numpy(), thresholds_v=thr.float().numpy(), stat="bf16")
        results.append(np.array_equal(cache.cpu().numpy(), want))
        del thr_d
    assert all(results), (results, addresses)
