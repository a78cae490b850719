"""Paged read-back and slot derivation: exact against the reference-produced vectors
and the oracle."""

import numpy as np
import pytest
import torch

import oracle
from beyond_kv_cache_b200 import _lib
from beyond_kv_cache_b200.quant.beyond_cute import (
    PagedLayout,
    dequantize_paged_kv_to_dense,
    read_request_from_paged_cache,
)
from tests.helpers import KIND_TO_DTYPE, bits16, oracle_cache, tables

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_read_request_matches_reference_bits(golden, kind):
    g = golden["writer"]
    layout = PagedLayout.build_hnd(16, 2, 128, 4, 32, 32)
    cache = torch.from_numpy(g[f"w_cache_bs16_v2_{kind}"]).to(DEV)
    lk = torch.from_numpy(g["w_lv_k"]).to(torch.float16).to(DEV)
    lv = torch.from_numpy(g["w_lv_v"]).to(torch.float16).to(DEV)
    dt = KIND_TO_DTYPE[kind]
    k, v = read_request_from_paged_cache(cache, layout, torch.tensor([2, 0], dtype=torch.int32, device=DEV), 20,
                                         q_points_k=lk, q_points_v=lv, out_dtype=dt, stat_dtype=dt)
    for got, key in ((k, "k"), (v, "v")):
        want_bits = g[f"w_read_{key}_bits_bs16_v2_{kind}"].reshape(1, 20, 2, 128)
        ok = np.isfinite(oracle.stat_to_f32(want_bits, kind))
        assert np.array_equal(bits16(got)[ok], want_bits[ok])


@pytest.mark.parametrize("bs,heads,lens", [
    (16, 2, [137, 255, 0, 1]), (64, 2, [137, 255, 0, 1]), (128, 2, [137, 255, 0, 1]),
    (16, 1, [33, 5]), (32, 3, [70, 0, 129]), (16, 6, [97, 64]), (16, 40, [19, 40]),
    # more positions than warps in the grid: every warp walks several tokens, page ids read ahead
    (16, 8, [2000, 1777, 0, 1999, 1500, 2000]),
])
@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_batched_readback_matches_oracle(bs, heads, lens, kind):
    lk, tk, lv, tv = tables(heads, 13)
    cache, bt = oracle_cache(lens, heads, bs, kind, 31, tk.float().numpy(), tv.float().numpy())
    dt = KIND_TO_DTYPE[kind]
    total = sum(lens)
    out_k = torch.full((total, heads, 128), 7.0, dtype=dt, device=DEV)
    out_v = torch.full_like(out_k, 7.0)
    starts = torch.tensor(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32), device=DEV)
    dequantize_paged_kv_to_dense(
        torch.from_numpy(cache).to(DEV), PagedLayout.build_hnd(bs, heads, 128, 4, 32, 32), torch.from_numpy(bt).to(DEV),
        torch.tensor(lens, dtype=torch.int32, device=DEV), starts, out_k, out_v, max_seq_len=max(lens),
        q_points_k=lk.to(DEV), q_points_v=lv.to(DEV),
    )
    geo = oracle.PageGeometry(bs, heads)
    s = 0
    for b, n in enumerate(lens):
        if n:
            pages = (n + bs - 1) // bs
            k, v = oracle.read_request(cache, geo, bt[b, :pages], n, levels_k=lk.float().numpy(),
                                       levels_v=lv.float().numpy(), stat=kind, out=kind)
            assert np.array_equal(bits16(out_k[s : s + n]), oracle.round_to_stat(k, kind))
            assert np.array_equal(bits16(out_v[s : s + n]), oracle.round_to_stat(v, kind))
        s += n


def test_derive_last_token_slots():
    bt = torch.tensor([[5, 2, -1], [7, 1, 3], [4, 0, 0], [-1, 0, 0]], dtype=torch.int32, device=DEV)
    lens = torch.tensor([17, 48, 0, 3], dtype=torch.int32, device=DEV)
    out = torch.full((4,), 99, dtype=torch.int32, device=DEV)
    _lib.call("bkv_derive_slots_sm100", lens.data_ptr(), bt.data_ptr(), bt.stride(0), bt.shape[1], 16, 4,
              out.data_ptr(), _lib.current_stream(bt.device))
    assert out.cpu().tolist() == [2 * 16 + 0, 3 * 16 + 15, -1, -1]
