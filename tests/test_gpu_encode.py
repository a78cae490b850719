"""Encode-on-write parity: the CUDA writer against the oracle and the golden page
bytes produced by the reference (bit-exact)."""

import hashlib

import numpy as np
import pytest
import torch

import oracle
from beyond_kv_cache_b200 import _lib, synth
from beyond_kv_cache_b200.quant.beyond_cute import (
    CODE_LAYOUT_HEAD_WORD_TOKEN,
    CODE_LAYOUT_HND_TOKEN_WORD,
    PagedLayout,
    write_tokens_to_paged_cache,
)
from oracle.paged import ABI_TOKEN_MAJOR, ABI_WORD_MAJOR
from tests.helpers import KIND_TO_DTYPE, bits16, tables

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("abi", ["v2", "v1"])
@pytest.mark.parametrize("bs", [16, 64])
def test_writer_matches_reference_bytes(golden, bs, abi, kind):
    g = golden["writer"]
    code_layout = CODE_LAYOUT_HND_TOKEN_WORD if abi == "v2" else CODE_LAYOUT_HEAD_WORD_TOKEN
    layout = PagedLayout.build(bs, 2, 128, 4, 32, 32, code_layout=code_layout)
    pages = 6 if bs == 16 else 2
    seed_pages = np.random.default_rng(99).integers(-(2**31), 2**31, (pages, layout.block_i32)).astype(np.int32)
    cache = torch.from_numpy(seed_pages).to(DEV)
    dt = KIND_TO_DTYPE[kind]
    k = torch.from_numpy(g["w_k32"]).to(dt).to(DEV)
    v = torch.from_numpy(g["w_v32"]).to(dt).to(DEV)
    k_in, v_in = k.clone(), v.clone()
    tab = {n: torch.from_numpy(g[n]).to(torch.float16).to(DEV) for n in ("w_lv_k", "w_th_k", "w_lv_v", "w_th_v")}
    slots = torch.from_numpy(g[f"w_slots_bs{bs}"]).to(DEV)
    write_tokens_to_paged_cache(
        cache, layout, torch.zeros((1, 1), dtype=torch.int32, device=DEV), slots, k, v,
        q_points_k=tab["w_lv_k"], q_points_v=tab["w_lv_v"], thresholds_k=tab["w_th_k"], thresholds_v=tab["w_th_v"],
        k_dq_out=k, v_dq_out=v, require_fast=True,
    )
    tag = f"bs{bs}_{abi}_{kind}"
    assert np.array_equal(cache.cpu().numpy(), g[f"w_cache_{tag}"])
    assert np.array_equal(bits16(k), g[f"w_kdq_bits_{tag}"])  # in place, slot -1 rows too
    assert np.array_equal(bits16(v), g[f"w_vdq_bits_{tag}"])
    assert not torch.equal(k, k_in) and not torch.equal(v, v_in)


@pytest.mark.parametrize("case", ["ties_f16", "ties_bf16", "divrn"])
def test_known_answer_vectors(golden, case):
    g = golden["kat"]
    kind = "bf16" if case.endswith("bf16") else "f16"
    prefix = "divrn" if case == "divrn" else "ties"
    x = torch.from_numpy(g[f"{case}_x"]).to(KIND_TO_DTYPE[kind]).reshape(1, 1, 128).to(DEV)
    thr = torch.from_numpy(g[f"{prefix}_thresholds"]).to(torch.float16).to(DEV)
    lv = torch.from_numpy(g[f"{prefix}_levels"]).to(torch.float16).to(DEV)
    layout = PagedLayout.build_hnd(16, 1, 128, 4, 32, 32)
    cache = torch.zeros((1, layout.block_i32), dtype=torch.int32, device=DEV)
    write_tokens_to_paged_cache(
        cache, layout, None, torch.tensor([3], dtype=torch.int32, device=DEV), x, x.clone(),
        q_points_k=lv, q_points_v=lv, thresholds_k=thr, thresholds_v=thr, require_fast=True,
    )
    parts = oracle.paged.gather_request(cache.cpu().numpy(), oracle.PageGeometry(16, 1), [0], 4)
    for which in ("k", "v"):
        codes = oracle.unpack_nibbles(parts[f"{which}_words"])[3, 0]
        assert np.array_equal(codes, g[f"{case}_codes"])
        assert np.array_equal(parts[f"{which}_scale_bits"][3, 0], g[f"{case}_scale_bits"])
        assert np.array_equal(parts[f"{which}_mn_bits"][3, 0], g[f"{case}_mn_bits"])
    if case == "divrn":
        assert int(oracle.unpack_nibbles(parts["k_words"])[3, 0, 0, 2]) == 11


def test_config0_cache_checksum(golden):
    """fp32 rows, fp16 statistics, 16-token pages, random block table: the whole cache
    must hash to the value the reference's quantiser produced."""
    g = golden["config0"]
    q, k, v = synth.config0_inputs(0)
    lk, tk, lv, tv = tables(8, 0, per_group=False)
    layout = PagedLayout.build_hnd(16, 8, 128, 4, 32, 32)
    bt = torch.from_numpy(g["c0_block_table"]).to(DEV)
    slots = synth.slots_for(bt, 16, 0, 1024)
    cache = torch.zeros((256, layout.block_i32), dtype=torch.int32, device=DEV)
    write_tokens_to_paged_cache(
        cache, layout, bt, slots, torch.from_numpy(k).to(DEV), torch.from_numpy(v).to(DEV),
        q_points_k=lk.to(DEV), q_points_v=lv.to(DEV), thresholds_k=tk.to(DEV), thresholds_v=tv.to(DEV),
        require_fast=True, stat_dtype=torch.float16,
    )
    got = cache.cpu().numpy()
    assert np.array_equal(got[int(g["c0_page0_id"][0])], g["c0_page0"])
    assert np.array_equal(np.frombuffer(hashlib.sha256(got.tobytes()).digest(), dtype=np.uint8), g["c0_cache_sha256"])


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("tokens,heads,shared", [(8, 2, True), (513, 8, False), (1, 4, False), (40, 40, False),
                                                 (20000, 8, False), (19500, 6, False), (19000, 3, False),
                                                 # mid-size writes: a token's heads split over 4 / 2 warps
                                                 (8192, 8, False), (10000, 4, False)])
def test_writer_matches_oracle_random(tokens, heads, shared, kind):
    rng = np.random.default_rng(2708 + tokens)
    dt = KIND_TO_DTYPE[kind]
    bs = 64
    pages = max(12, tokens // bs + 2)
    geo = oracle.PageGeometry(bs, heads, 128)
    seed_pages = rng.integers(-(2**31), 2**31, (pages, geo.block_i32)).astype(np.int32)
    k = torch.from_numpy(rng.standard_normal((tokens, heads, 128)).astype(np.float32)).to(dt)
    v = torch.from_numpy((rng.standard_normal((tokens, heads, 128)) * 3).astype(np.float32)).to(dt)
    if tokens >= 8192:
        # values far below the group's range: their quotients lie under 2^-60, where the encoder's
        # shared-divisor quotient is not redone with the IEEE division when the tables are fp16
        k[::7, :, 5] = 2.0**-100
        k[::11, :, 40] = -(2.0**-63)
        k[::13, :, 41] = 2.0**-61
        v[::5, :, 77] = 2.0**-70
        v[::9, 0, 64:96] = torch.tensor([2.0**-90, -(2.0**-90)] * 16).to(dt)  # a whole group of tiny values
    slots = rng.permutation(pages * bs)[:tokens].astype(np.int64)
    slots[::17] = -1
    if shared:
        lk = tk = lv = tv = None
        thr_k = thr_v = None
    else:
        lk, tk, lv, tv = (t.to(DEV) for t in tables(heads, 5))
        thr_k, thr_v = tk.float().cpu().numpy(), tv.float().cpu().numpy()
    expect = seed_pages.copy()
    oracle.write_pages(expect, geo, slots, k.float().numpy(), v.float().numpy(), thresholds_k=thr_k, thresholds_v=thr_v, stat=kind)
    cache = torch.from_numpy(seed_pages).to(DEV)
    layout = PagedLayout.build_hnd(bs, heads, 128, 4, 32, 32)
    # K and V arrive as views into a fused QKV projection (non-contiguous token stride)
    fused = torch.zeros((tokens, heads * 3, 128), dtype=dt, device=DEV)
    fused[:, heads : 2 * heads] = k.to(DEV)
    fused[:, 2 * heads :] = v.to(DEV)
    write_tokens_to_paged_cache(
        cache, layout, None, torch.from_numpy(slots).to(DEV), fused[:, heads : 2 * heads], fused[:, 2 * heads :],
        q_points_k=lk, q_points_v=lv, thresholds_k=tk, thresholds_v=tv, require_fast=True,
    )
    assert np.array_equal(cache.cpu().numpy(), expect)


def _threshold_hitting_rows(rng, tokens, heads, thr16):
    """float32 rows whose normalised values land exactly on thresholds and interval borders: every
    group holds 0 and 1 (so scale = 1, min = 0 and x_norm = x), the rest are thresholds of the
    group's own table, their fp16 neighbours, and multiples of 2^-9 with their float32 neighbours."""
    x = np.empty((tokens, heads, 128), dtype=np.float32)
    thr = thr16.float().numpy().reshape(heads, 4, 15)
    for h in range(heads):
        for g in range(4):
            t = thr[h, g]
            neighbours = np.concatenate([t, np.nextafter(t.astype(np.float16), np.float16(0)).astype(np.float32),
                                         np.nextafter(t.astype(np.float16), np.float16(1)).astype(np.float32)])
            borders = rng.integers(0, 513, 64).astype(np.float32) / 512.0
            borders = np.concatenate([borders, np.nextafter(borders, np.float32(0)), np.nextafter(borders, np.float32(1))])
            pool = np.clip(np.concatenate([neighbours, borders]), 0.0, 1.0).astype(np.float32)
            x[:, h, 32 * g : 32 * g + 32] = rng.choice(pool, (tokens, 32))
            x[:, h, 32 * g] = 0.0
            x[:, h, 32 * g + 1] = 1.0
    return x


@pytest.mark.parametrize("kind,table_dtype,heads,shared", [("f16", torch.float16, 8, False), ("bf16", torch.float16, 3, False),
                                                        ("f16", torch.float32, 8, False), ("bf16", torch.float16, 8, True)])
def test_large_writes_with_classified_tables(kind, table_dtype, heads, shared):
    """Writes large enough for the indexed look-up (tables with at most one threshold per interval
    of 2^-9): page bytes and the in-place reconstruction against the oracle, on random rows and on
    rows whose normalised values sit exactly on thresholds and interval borders."""
    from beyond_kv_cache_b200.quant.beyond_cute import _tables_binned

    rng = np.random.default_rng(41 + heads)
    # (the indexed form takes writes of 96 tokens per SM and more)
    tokens, bs = 96 * torch.cuda.get_device_properties(0).multi_processor_count + 300, 16
    dt = KIND_TO_DTYPE[kind]
    lk, tk, lv, tv = tables(heads, 9, per_group=not shared)
    if shared:
        lk, tk, lv, tv = lk[:1].reshape(16), tk[:1].reshape(15), lv[:1].reshape(16), tv[:1].reshape(15)
        tk_all, tv_all = tk.repeat(heads * 4, 1), tv.repeat(heads * 4, 1)
    else:
        tk_all, tv_all = tk, tv
    k32 = rng.standard_normal((tokens, heads, 128)).astype(np.float32)
    v32 = _threshold_hitting_rows(rng, tokens, heads, tv_all)
    k32[::3] = _threshold_hitting_rows(rng, len(k32[::3]), heads, tk_all)
    k = torch.from_numpy(k32).to(dt)
    v = torch.from_numpy(v32).to(dt)
    pages = tokens // bs + 5
    geo = oracle.PageGeometry(bs, heads, 128)
    seed_pages = rng.integers(-(2**31), 2**31, (pages, geo.block_i32)).astype(np.int32)
    slots = rng.permutation(pages * bs)[:tokens].astype(np.int64)
    slots[::29] = -1
    expect = seed_pages.copy()
    oracle.write_pages(expect, geo, slots, k.float().numpy(), v.float().numpy(), thresholds_k=tk.float().numpy(),
                       thresholds_v=tv.float().numpy(), stat=kind)
    tabs = [t.to(table_dtype).to(DEV) for t in (lk, tk, lv, tv)]
    assert _tables_binned(tabs[1]) and _tables_binned(tabs[3])
    cache = torch.from_numpy(seed_pages).to(DEV)
    kd, vd = k.to(DEV), v.to(DEV)
    write_tokens_to_paged_cache(cache, PagedLayout.build_hnd(bs, heads, 128, 4, 32, 32), None, torch.from_numpy(slots).to(DEV), kd, vd,
                                q_points_k=tabs[0], q_points_v=tabs[2], thresholds_k=tabs[1], thresholds_v=tabs[3],
                                k_dq_out=kd, v_dq_out=vd, require_fast=True)
    assert np.array_equal(cache.cpu().numpy(), expect)
    for got, src, lvl, thr in ((kd, k, lk, tk), (vd, v, lv, tv)):
        enc = oracle.encode_groups(src.float().numpy(), thr.float().numpy(), stat=kind)
        want = oracle.decode_groups(enc["codes"], lvl.float().numpy(), enc["scale_bits"], enc["mn_bits"], stat=kind)
        assert np.array_equal(bits16(got), bits16(torch.from_numpy(want).to(dt)))  # slot -1 rows too


@pytest.mark.parametrize("chunk", [15000, 8192, 1000])
def test_chunks_chained_as_programmatic_dependents(chunk):
    """One long write issued as chunks on one stream, every chunk signalling its dependents early and
    launched as a programmatic dependent of the chunk in front (both the indexed and the searching
    form, by chunk size): the same page bytes as the oracle's single write."""
    heads, bs, tokens = 8, 16, 3 * chunk + 77
    rng = np.random.default_rng(chunk)
    lk, tk, lv, tv = (t.to(DEV) for t in tables(heads, 11))
    k = torch.from_numpy(rng.standard_normal((tokens, heads, 128)).astype(np.float32)).to(torch.bfloat16)
    v = torch.from_numpy((rng.standard_normal((tokens, heads, 128)) * 2).astype(np.float32)).to(torch.bfloat16)
    geo = oracle.PageGeometry(bs, heads, 128)
    pages = tokens // bs + 3
    seed_pages = rng.integers(-(2**31), 2**31, (pages, geo.block_i32)).astype(np.int32)
    slots = rng.permutation(pages * bs)[:tokens].astype(np.int64)
    expect = seed_pages.copy()
    oracle.write_pages(expect, geo, slots, k.float().numpy(), v.float().numpy(), thresholds_k=tk.float().cpu().numpy(),
                       thresholds_v=tv.float().cpu().numpy(), stat="bf16")
    cache = torch.from_numpy(seed_pages).to(DEV)
    kd, vd, sd = k.to(DEV), v.to(DEV), torch.from_numpy(slots).to(DEV)
    layout = PagedLayout.build_hnd(bs, heads, 128, 4, 32, 32)
    for c0 in range(0, tokens, chunk):
        write_tokens_to_paged_cache(cache, layout, None, sd[c0:c0 + chunk], kd[c0:c0 + chunk], vd[c0:c0 + chunk],
                                    q_points_k=lk, q_points_v=lv, thresholds_k=tk, thresholds_v=tv, require_fast=True,
                                    signal_pdl_dependents=True, wait_for_pdl_predecessor=c0 > 0)
    torch.cuda.synchronize()
    assert np.array_equal(cache.cpu().numpy(), expect)


def test_tables_with_two_thresholds_in_one_interval_keep_the_search():
    from beyond_kv_cache_b200.quant.beyond_cute import _tables_binned, _tables_sorted

    heads, tokens, bs = 2, 96 * torch.cuda.get_device_properties(0).multi_processor_count + 100, 16
    lk, tk, lv, tv = tables(heads, 3)
    tk = tk.clone()
    e = torch.floor(tk[:, 6].float() * 512)
    tk[:, 6] = ((e + 0.25) / 512).to(tk.dtype)  # sorted, but two thresholds inside one interval of 2^-9
    tk[:, 7] = ((e + 0.75) / 512).to(tk.dtype)
    assert _tables_sorted(tk.to(DEV)) and not _tables_binned(tk.to(DEV))
    negative = tv.clone()
    negative[:, 0] = -0.25
    assert not _tables_binned(negative.to(DEV))
    rng = np.random.default_rng(5)
    k = torch.from_numpy(rng.standard_normal((tokens, heads, 128)).astype(np.float32)).to(torch.float16)
    geo = oracle.PageGeometry(bs, heads, 128)
    pages = tokens // bs + 1
    expect = np.zeros((pages, geo.block_i32), dtype=np.int32)
    slots = np.arange(tokens, dtype=np.int64)
    oracle.write_pages(expect, geo, slots, k.float().numpy(), k.float().numpy(), thresholds_k=tk.float().numpy(),
                       thresholds_v=tv.float().numpy())
    cache = torch.zeros((pages, geo.block_i32), dtype=torch.int32, device=DEV)
    write_tokens_to_paged_cache(cache, PagedLayout.build_hnd(bs, heads, 128, 4, 32, 32), None, torch.from_numpy(slots).to(DEV),
                                k.to(DEV), k.to(DEV), q_points_k=lk.to(DEV), q_points_v=lv.to(DEV), thresholds_k=tk.to(DEV),
                                thresholds_v=tv.to(DEV), require_fast=True)
    assert np.array_equal(cache.cpu().numpy(), expect)


def test_unsorted_thresholds_use_the_counting_rule():
    heads = 1
    thr = torch.tensor([0.5, 0.1, 0.9, 0.3, 0.7, 0.2, 0.8, 0.4, 0.6, 0.15, 0.25, 0.35, 0.45, 0.55, 0.65], dtype=torch.float16)
    lv = torch.linspace(0, 1, 16, dtype=torch.float16)
    rng = np.random.default_rng(1)
    x = torch.from_numpy(rng.standard_normal((5, heads, 128)).astype(np.float32)).to(torch.float16)
    geo = oracle.PageGeometry(16, heads)
    expect = np.zeros((1, geo.block_i32), dtype=np.int32)
    slots = np.arange(5, dtype=np.int64)
    oracle.write_pages(expect, geo, slots, x.float().numpy(), x.float().numpy(),
                       thresholds_k=thr.float().numpy(), thresholds_v=thr.float().numpy())
    cache = torch.zeros((1, geo.block_i32), dtype=torch.int32, device=DEV)
    write_tokens_to_paged_cache(cache, PagedLayout.build_hnd(16, heads, 128, 4, 32, 32), None,
                                torch.from_numpy(slots).to(DEV), x.to(DEV), x.to(DEV),
                                q_points_k=lv.to(DEV), q_points_v=lv.to(DEV), thresholds_k=thr.to(DEV), thresholds_v=thr.to(DEV))
    assert np.array_equal(cache.cpu().numpy(), expect)


def test_empty_and_rejected_inputs():
    layout = PagedLayout.build_hnd(16, 2, 128, 4, 32, 32)
    cache = torch.zeros((2, layout.block_i32), dtype=torch.int32, device=DEV)
    empty = torch.zeros((0, 2, 128), dtype=torch.float16, device=DEV)
    write_tokens_to_paged_cache(cache, layout, None, torch.zeros((0,), dtype=torch.int32, device=DEV), empty, empty, require_fast=True)
    assert not cache.any()
    k = torch.zeros((1, 2, 128), dtype=torch.float16)
    with pytest.raises(RuntimeError, match="fused sm_100a writer"):
        write_tokens_to_paged_cache(cache.cpu(), layout, None, torch.zeros((1,), dtype=torch.int32), k, k, require_fast=True)
    with pytest.raises(RuntimeError, match="fused sm_100a writer"):  # no silent fallback without require_fast either
        write_tokens_to_paged_cache(cache.cpu(), layout, None, torch.zeros((1,), dtype=torch.int32), k, k)
    bad = PagedLayout.build_hnd(16, 2, 96, 4, 32, 32)
    with pytest.raises(RuntimeError):
        write_tokens_to_paged_cache(torch.zeros((2, bad.block_i32), dtype=torch.int32, device=DEV), bad, None,
                                    torch.zeros((1,), dtype=torch.int32, device=DEV),
                                    torch.zeros((1, 2, 96), dtype=torch.float16, device=DEV),
                                    torch.zeros((1, 2, 96), dtype=torch.float16, device=DEV), require_fast=True)


@pytest.mark.parametrize("mode", [0, 1])
def test_shared_divisor_division_is_the_ieee_division(mode):
    """The encoder's division by a shared divisor (reciprocal + exact-remainder correction)
    against __fdiv_rn on 2^28 pseudo-random operand pairs: zero bitwise mismatches, both in
    the quantiser's operand domain and over all finite positive pairs."""
    bad = torch.zeros((1,), dtype=torch.int64, device="cuda")
    for seed in (1, 2):
        _lib.call("bkv_selftest_division_sm100", seed, 1 << 27, mode, bad.data_ptr(), _lib.current_stream(bad.device))
    torch.cuda.synchronize()
    assert int(bad.item()) == 0
