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
    impl = mod.BeyondPackedImpl.__new__(mod.BeyondPackedImpl)
    impl.num_heads, impl.num_kv_heads, impl.head_size = num_heads, num_kv_heads, 128
    impl.scale = 1.0 / math.sqrt(128)
    impl._tables, impl._workspaces = None, {}
    return impl


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


def test_unsupported_plans_fail_closed():
    impl = _impl()
    cache = torch.zeros((4, 2 * 16 * 40), dtype=torch.int32, device=DEV)
    q = torch.zeros((3, 8, 128), dtype=torch.bfloat16, device=DEV)
    kv = torch.zeros((3, 2, 128), dtype=torch.bfloat16, device=DEV)
    assert not impl.forward(None, q, kv, kv, cache, None).any()
    meta = types.SimpleNamespace(num_actual_tokens=3, query_start_loc=torch.tensor([0, 3], dtype=torch.int32, device=DEV),
                                 seq_lens=torch.tensor([10], dtype=torch.int32, device=DEV),
                                 block_table=torch.zeros((1, 4), dtype=torch.int32, device=DEV),
                                 slot_mapping=torch.arange(3, device=DEV), max_query_len=3, max_seq_len=10)
    with pytest.raises(NotImplementedError, match="chunked-prefill"):
        impl.forward(None, q, kv, kv, cache, meta)
    with pytest.raises(NotImplementedError, match="output quantization"):
        impl.forward(None, q, kv, kv, cache, meta, output_scale=torch.ones(1))
    with pytest.raises(RuntimeError, match="shared dtype"):
        impl.forward(None, q.float(), kv, kv, cache, meta)
