"""The nibble format and the dense quantiser API of the ops module, in the form of the
reference's own tests (quant/tests/test_pack_roundtrip.py:19-142).  pack_codes / unpack_codes are
pure format helpers and run anywhere; quantize_* / dequantize_* run on the encode and read-back
kernels, so their cases need a GPU (and head_dim 128, the one size those kernels take; the
reference's cases use 96)."""

import numpy as np
import pytest
import torch

import oracle
from beyond_kv_cache_b200.quant.beyond_cute import (
    PackedK,
    PackedV,
    dequantize_k,
    dequantize_v,
    pack_codes,
    quantize_k,
    quantize_v,
    unpack_codes,
)
from tests.helpers import bits16


@pytest.mark.parametrize("shape_prefix", [(), (3,), (2, 4)])
def test_pack_unpack_roundtrip_4bit(shape_prefix):
    torch.manual_seed(0)
    codes = torch.randint(0, 16, (*shape_prefix, 32), dtype=torch.uint8)
    packed = pack_codes(codes, 4)
    assert packed.shape == (*shape_prefix, 4) and packed.dtype == torch.uint32
    recovered = unpack_codes(packed, 4, 32)
    assert recovered.shape == codes.shape and torch.equal(recovered, codes)
    # the same words as the oracle's restatement of the reference layout: code i in bits 4*(i%8) of word i//8
    assert np.array_equal(packed.view(torch.int32).numpy().view(np.uint32), oracle.pack_nibbles(codes.numpy()))


def test_pack_axis_first_removed():
    codes = torch.zeros(32, dtype=torch.uint8)
    with pytest.raises(TypeError, match="pack_axis_first"):
        pack_codes(codes, 4, pack_axis_first=True)
    with pytest.raises(TypeError, match="pack_axis_first"):
        unpack_codes(torch.zeros(4, dtype=torch.uint32), 4, 32, pack_axis_first=True)


def test_pack_layout_boundary_values():
    assert torch.all(pack_codes(torch.zeros(32, dtype=torch.uint8), 4).view(torch.int32) == 0)
    packed_max = pack_codes(torch.full((32,), 15, dtype=torch.uint8), 4)
    assert packed_max.numel() == 4
    assert sum(bin(int(w) & 0xFFFFFFFF).count("1") for w in packed_max.view(torch.int32).tolist()) == 128
    one = torch.zeros(32, dtype=torch.uint8)
    one[9] = 0xA  # word 1, bits 4..7
    assert pack_codes(one, 4).view(torch.int32).tolist() == [0, 0xA0, 0, 0]


def test_pack_rejects_removed_sizes():
    with pytest.raises(ValueError, match="group_size"):
        pack_codes(torch.zeros(24, dtype=torch.uint8), 4)
    with pytest.raises(ValueError, match="4-bit"):
        pack_codes(torch.zeros(32, dtype=torch.uint8), 2)
    with pytest.raises(TypeError, match="uint8"):
        pack_codes(torch.zeros(32, dtype=torch.int32), 4)
    with pytest.raises(ValueError, match="words_per_group"):
        unpack_codes(torch.zeros(3, dtype=torch.uint32), 4, 32)


def test_dense_quantiser_has_no_cpu_path():
    x = torch.zeros((1, 2, 2, 128), dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        quantize_k(x, 4, 32)
    with pytest.raises(TypeError, match="pack_axis_first"):
        quantize_k(x, 4, 32, pack_axis_first=True)
    with pytest.raises(ValueError, match="group_size"):
        quantize_v(x, 4, 16)
    with pytest.raises(TypeError, match="fp16/bf16"):
        quantize_k(x.float(), 4, 32)  # float32 rows need an explicit stat_dtype, as in the reference


# ---------------------------------------------------------------------------------- GPU
gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("kind,dtype", [("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_known_answers_through_quantize_k(golden, kind, dtype):
    """The reference's two known-answer groups (quant/tests/test_paged.py:688-694, :746-771)."""
    g = golden["kat"]
    thr, lv = torch.from_numpy(g["ties_thresholds"]).half().cuda(), torch.from_numpy(g["ties_levels"]).half().cuda()
    x = torch.from_numpy(g[f"ties_{kind}_x"]).to(dtype).view(1, 1, 1, 128).cuda()
    pk = quantize_k(x, 4, 32, q_points=lv, thresholds=thr)
    assert isinstance(pk, PackedK) and pk.codes.shape == (1, 1, 1, 4, 32) and pk.packed.shape == (1, 1, 1, 4, 4)
    assert np.array_equal(pk.codes.cpu().numpy().reshape(4, 32), g[f"ties_{kind}_codes"])
    assert np.array_equal(bits16(pk.scale).reshape(4), g[f"ties_{kind}_scale_bits"])
    assert np.array_equal(bits16(pk.mn).reshape(4), g[f"ties_{kind}_mn_bits"])
    if kind == "f16":
        x = torch.from_numpy(g["divrn_x"]).half().view(1, 1, 1, 128).cuda()
        pk = quantize_k(x, 4, 32, q_points=torch.from_numpy(g["divrn_levels"]).half().cuda(),
                        thresholds=torch.from_numpy(g["divrn_thresholds"]).half().cuda())
        assert np.array_equal(pk.codes.cpu().numpy().reshape(4, 32), g["divrn_codes"])
        assert int(pk.codes[0, 0, 0, 0, 2]) == 11  # the IEEE-division boundary: 11, not 12
        assert np.array_equal(pk.packed.cpu().view(torch.int32).numpy().view(np.uint32).reshape(4, 4), g["divrn_words"])
        assert np.array_equal(bits16(pk.scale).reshape(4), g["divrn_scale_bits"])
        assert np.array_equal(bits16(pk.mn).reshape(4), g["divrn_mn_bits"])


@gpu
def test_config0_rows_through_quantize_k(golden):
    """Float32 rows with fp16 statistics (config 0): codes and statistics of the first 64 tokens
    as the reference's quantize_k produced them."""
    from beyond_kv_cache_b200 import synth
    from tests.helpers import tables

    g = golden["config0"]
    _, k, _ = synth.config0_inputs(0)
    lk, tk, _, _ = tables(8, 0, per_group=False)
    x = torch.from_numpy(k[:64]).view(1, 64, 8, 128).cuda()
    pk = quantize_k(x, 4, 32, q_points=lk.cuda(), thresholds=tk.cuda(), stat_dtype=torch.float16)
    assert np.array_equal(pk.codes.cpu().numpy()[0], g["c0_k_codes_head"])
    assert np.array_equal(bits16(pk.scale)[0], g["c0_k_scale_bits_head"])
    assert np.array_equal(bits16(pk.mn)[0], g["c0_k_mn_bits_head"])


@gpu
@pytest.mark.parametrize("kind,dtype", [("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_roundtrip_equals_the_writer_reconstruction(golden, kind, dtype):
    """dequantize(quantize(x)) with per-(head, group) tables: the bits the reference's writer
    leaves in k_dq_out / v_dq_out for the same rows."""
    g = golden["writer"]
    k = torch.from_numpy(g["w_k32"]).to(dtype).view(1, 37, 2, 128).cuda()
    v = torch.from_numpy(g["w_v32"]).to(dtype).view(1, 37, 2, 128).cuda()
    lk, tk = torch.from_numpy(g["w_lv_k"]).half().cuda(), torch.from_numpy(g["w_th_k"]).half().cuda()
    lv, tv = torch.from_numpy(g["w_lv_v"]).half().cuda(), torch.from_numpy(g["w_th_v"]).half().cuda()
    k_hat = dequantize_k(quantize_k(k, 4, 32, q_points=lk, thresholds=tk), q_points=lk)
    v_hat = dequantize_v(quantize_v(v, 4, 32, q_points=lv, thresholds=tv), q_points=lv)
    assert k_hat.dtype == dtype and k_hat.shape == k.shape
    assert np.array_equal(bits16(k_hat)[0], g[f"w_kdq_bits_bs16_v2_{kind}"])
    assert np.array_equal(bits16(v_hat)[0], g[f"w_vdq_bits_bs16_v2_{kind}"])


@gpu
def test_quantize_v_token_last_matches_token_major():
    torch.manual_seed(16)
    B, S, H, D = 2, 11, 2, 128
    x = torch.randn(B, S, H, D, dtype=torch.float16, device="cuda")
    pv = quantize_v(x, 4, 32)
    pv_tl = quantize_v(x, 4, 32, pack_token_last=True)
    assert isinstance(pv_tl, PackedV) and pv_tl.pack_token_last is True
    assert pv_tl.packed.shape == (B, H, D // 32, 4, S) and pv_tl.scale.shape == (B, H, D // 32, S)
    assert torch.equal(pv_tl.packed.permute(0, 4, 1, 2, 3).contiguous().view(torch.int32), pv.packed.view(torch.int32))
    assert torch.equal(dequantize_v(pv), dequantize_v(pv_tl))


@gpu
def test_uniform_default_tables_and_budget():
    """Default (uniform fp16) tables: the same codes as the float fake-QDQ path with those tables,
    values within the tolerance the reference uses for this comparison (1e-2,
    quant/tests/test_pack_roundtrip.py:75-80), no per-sequence residue, 4 bits per scalar."""
    torch.manual_seed(7)
    B, S, H, D = 1, 19, 2, 128
    x = torch.randn(B, S, H, D, dtype=torch.float16, device="cuda")
    pk = quantize_k(x, 4, 32)
    assert not hasattr(pk, "residual")
    y = dequantize_k(pk)
    assert y.shape == x.shape and y.dtype == x.dtype
    assert pk.packed.element_size() * pk.packed.numel() == B * S * H * D * 4 // 8
    from beyond_kv_cache_b200.quant.beyond_cute import prepare_qpoints_and_thresholds

    levels, thresholds = prepare_qpoints_and_thresholds(num_bits=4, device=torch.device("cpu"), q_points=None)  # fp16 defaults
    want = oracle.fake_qdq_unrounded(x.float().cpu().numpy(), levels.float().numpy(), thresholds.float().numpy())
    assert np.abs(y.float().cpu().numpy() - want).max() <= 1e-2  # what fp16 storage of (scale, minimum) and of y costs
