"""Generate the golden fixtures of this directory by running the REFERENCE's own
Python code (``quant/beyond_cute.py`` of wsxhjnb1/Beyond-KV-Cache) on CPU.

Usage (needs the reference checkout; the fixtures themselves are committed, so the
tests never need it):

    BEYOND_REFERENCE=/path/to/Beyond-KV-Cache python tests/golden/make_golden.py [kat writer config0 fakeqdq]

(no names: all four files).

Inputs come from ``numpy.random.default_rng`` (bit-stable across platforms) and are
stored or check-summed next to the reference outputs.  Nothing here imports the
oracle or the product package except the seeded table/shape helpers in ``synth``.
"""

from __future__ import annotations

import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
# the reference checkout: $BEYOND_REFERENCE, else a directory "reference" beside this repository
REF = os.environ.get("BEYOND_REFERENCE", os.path.join(os.path.dirname(REPO), "reference"))
sys.dont_write_bytecode = True
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(REF, "src"))
sys.path.insert(0, REPO)

import quant.beyond_cute as ref  # noqa: E402  (the reference module)

from beyond_kv_cache_b200 import synth  # noqa: E402


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def kat_cases() -> dict:
    out = {}
    # (1) values exactly on thresholds: quant/tests/test_paged.py:688-694
    thresholds = (torch.arange(1, 16, dtype=torch.float32) / 16).to(torch.float16)
    q_points = (torch.arange(16, dtype=torch.float32) / 15).to(torch.float16)
    for name, dt in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        group = torch.zeros(32, dtype=dt)
        group[1] = 1
        group[2:17] = thresholds.to(dt)
        x = group.repeat(4).view(1, 1, 1, 128)
        pk = ref.quantize_k(x, 4, 32, q_points=q_points, thresholds=thresholds)
        out[f"ties_{name}_x"] = x.float().numpy().reshape(128)
        out[f"ties_{name}_codes"] = pk.codes.numpy().reshape(4, 32)
        out[f"ties_{name}_scale_bits"] = bits16(pk.scale).reshape(4)
        out[f"ties_{name}_mn_bits"] = bits16(pk.mn).reshape(4)
    out["ties_thresholds"] = thresholds.float().numpy()
    out["ties_levels"] = q_points.float().numpy()
    # (2) IEEE-division rounding boundary: quant/tests/test_paged.py:746-771
    group = torch.zeros(32, dtype=torch.float16)
    group[0], group[1], group[2] = -18080.0, 1677.0, -1.5751953125
    thr = torch.tensor(
        [0.05, 0.10, 0.15, 0.20, 0.25, 0.30, 0.35, 0.40, 0.45, 0.50, 0.70, 0.9150390625, 0.94, 0.96, 0.98],
        dtype=torch.float16,
    )
    lv = torch.linspace(0.0, 1.0, 16, dtype=torch.float16)
    x = group.repeat(4).view(1, 1, 1, 128)
    pk = ref.quantize_k(x, 4, 32, q_points=lv, thresholds=thr)
    out["divrn_x"] = x.float().numpy().reshape(128)
    out["divrn_thresholds"] = thr.float().numpy()
    out["divrn_levels"] = lv.float().numpy()
    out["divrn_codes"] = pk.codes.numpy().reshape(4, 32)
    out["divrn_scale_bits"] = bits16(pk.scale).reshape(4)
    out["divrn_mn_bits"] = bits16(pk.mn).reshape(4)
    out["divrn_words"] = pk.packed.view(torch.int32).numpy().view(np.uint32).reshape(4, 4)
    # (3) default tables
    qp, th = ref.prepare_qpoints_and_thresholds(num_bits=4, device=torch.device("cpu"), q_points=None)
    out["uniform_levels_f32"] = ref.make_uniform_q_points(4).numpy()
    out["uniform_thresholds_f32"] = ref.make_uniform_thresholds(ref.make_uniform_q_points(4)).numpy()
    out["default_levels_bits"] = bits16(qp)
    out["default_thresholds_bits"] = bits16(th)
    return out


def layout_cases() -> dict:
    out = {}
    fields = ["k_code_off", "k_scale_off", "k_min_off", "v_code_off", "v_scale_off", "v_min_off", "block_halves", "block_i32"]
    rows = []
    for bs, h, d in [(16, 8, 128), (64, 8, 128), (128, 8, 128), (128, 4, 128), (16, 2, 96), (32, 2, 64)]:
        lay = ref.PagedLayout.build_hnd(bs, h, d, 4, 32, 32)
        rows.append([bs, h, d] + [getattr(lay, f) for f in fields])
    out["layout_rows"] = np.array(rows, dtype=np.int64)
    return out


def writer_cases() -> dict:
    """Reference page bytes for a small ragged write, both ABIs, both stat dtypes."""
    out = {}
    rng = np.random.default_rng(2708)
    T, H = 37, 2
    k32 = rng.standard_normal((T, H, 128)).astype(np.float32)
    v32 = rng.standard_normal((T, H, 128)).astype(np.float32)
    k32[:, :, 5] *= 8.0
    lv_k, th_k = synth.make_tables(H, seed=11, per_group=True, which="k")
    lv_v, th_v = synth.make_tables(H, seed=11, per_group=True, which="v")
    out["w_k32"], out["w_v32"] = k32, v32
    out["w_lv_k"], out["w_th_k"] = lv_k.float().numpy(), th_k.float().numpy()
    out["w_lv_v"], out["w_th_v"] = lv_v.float().numpy(), th_v.float().numpy()
    for bs in (16, 64):
        pages = 6 if bs == 16 else 2
        slots = rng.permutation(pages * bs)[:T].astype(np.int32)
        slots[::9] = -1
        out[f"w_slots_bs{bs}"] = slots
        for abi in (ref.CODE_LAYOUT_HND_TOKEN_WORD, ref.CODE_LAYOUT_HEAD_WORD_TOKEN):
            lay = ref.PagedLayout.build(bs, H, 128, 4, 32, 32, code_layout=abi)
            for name, dt in (("f16", torch.float16), ("bf16", torch.bfloat16)):
                k = torch.from_numpy(k32).to(dt)
                v = torch.from_numpy(v32).to(dt)
                seed_pages = np.random.default_rng(99).integers(-(2**31), 2**31, (pages, lay.block_i32)).astype(np.int32)
                cache = torch.from_numpy(seed_pages.copy())
                k_dq, v_dq = torch.empty_like(k), torch.empty_like(v)
                ref.write_tokens_to_paged_cache(
                    cache, lay, torch.zeros((1, 1), dtype=torch.int32), torch.from_numpy(slots), k, v,
                    q_points_k=lv_k, q_points_v=lv_v, thresholds_k=th_k, thresholds_v=th_v,
                    k_dq_out=k_dq, v_dq_out=v_dq,
                )
                tag = f"bs{bs}_{'v2' if abi == ref.CODE_LAYOUT_HND_TOKEN_WORD else 'v1'}_{name}"
                out[f"w_cache_{tag}"] = cache.numpy()
                out[f"w_kdq_bits_{tag}"] = bits16(k_dq)
                out[f"w_vdq_bits_{tag}"] = bits16(v_dq)
                if abi == ref.CODE_LAYOUT_HND_TOKEN_WORD and bs == 16:
                    # read-back of the first ceil(20/16) pages' worth of one request
                    ids = torch.tensor([2, 0], dtype=torch.int32)
                    kk, vv = ref.read_request_from_paged_cache(
                        cache, lay, ids, 20, q_points_k=lv_k, q_points_v=lv_v, out_dtype=dt, stat_dtype=dt
                    )
                    out[f"w_read_k_bits_{tag}"] = bits16(kk)
                    out[f"w_read_v_bits_{tag}"] = bits16(vv)
    out["w_seed_note"] = np.array([99], dtype=np.int64)
    return out


def config0_case() -> dict:
    out = {}
    B, Hq, Hkv, D, ctx, bs = 4, 32, 8, 128, 1024, 16
    q, k, v = synth.config0_inputs(0)
    lv_k, th_k = synth.make_tables(Hkv, seed=0, which="k")
    lv_v, th_v = synth.make_tables(Hkv, seed=0, which="v")
    lay = ref.PagedLayout.build_hnd(bs, Hkv, D, 4, 32, 32)
    pages_per_seq = ctx // bs
    bt, num_pages = synth.random_block_table(B, pages_per_seq, seed=0, device="cpu")
    slots = synth.slots_for(bt, bs, 0, ctx).to(torch.int32)
    cache = torch.zeros((num_pages, lay.block_i32), dtype=torch.int32)
    kt, vt = torch.from_numpy(k).unsqueeze(0), torch.from_numpy(v).unsqueeze(0)
    pk = ref.quantize_k(kt, 4, 32, q_points=lv_k, thresholds=th_k, stat_dtype=torch.float16)
    pv = ref.quantize_v(vt, 4, 32, q_points=lv_v, thresholds=th_v, stat_dtype=torch.float16)
    ref._write_flat_k_pk_to_cache(cache, lay, slots, pk)
    ref.write_v_pv_to_cache(cache, lay, slots, pv)
    scale = 1.0 / np.sqrt(D)
    outs = []
    for b in range(B):
        kk, vv = ref.read_request_from_paged_cache(
            cache, lay, bt[b], ctx, q_points_k=lv_k, q_points_v=lv_v, out_dtype=torch.float32, stat_dtype=torch.float16
        )
        rep = Hq // Hkv
        kr = kk[0].repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)
        vr = vv[0].repeat_interleave(rep, dim=1).transpose(0, 1).unsqueeze(0)
        qr = torch.from_numpy(q[b]).unsqueeze(1).unsqueeze(0)  # (1, Hq, 1, D)
        o = torch.nn.functional.scaled_dot_product_attention(qr, kr, vr, scale=float(scale))
        outs.append(o[0, :, 0, :].numpy())
    out["c0_out"] = np.stack(outs).astype(np.float32)
    out["c0_cache_sha256"] = np.frombuffer(bytes.fromhex(sha(cache.numpy())), dtype=np.uint8)
    out["c0_inputs_sha256"] = np.frombuffer(bytes.fromhex(sha(np.concatenate([q.ravel(), k.ravel(), v.ravel()]))), dtype=np.uint8)
    out["c0_page0"] = cache.numpy()[int(bt[0, 0])].copy()
    out["c0_page0_id"] = np.array([int(bt[0, 0])], dtype=np.int64)
    out["c0_block_table"] = bt.numpy()
    out["c0_k_codes_head"] = pk.codes[0, :64].numpy()  # first 64 tokens
    out["c0_k_scale_bits_head"] = bits16(pk.scale[0, :64])
    out["c0_k_mn_bits_head"] = bits16(pk.mn[0, :64])
    return out


def fakeqdq_case() -> dict:
    """The training-equivalent fake quantise/dequantise path (float statistics, never rounded to
    16 bits) as the reference's own layer evaluates it: ``UnifiedQuantLayer`` with per-group tables
    (``src/beyond/quantization/layers.py:1398-1475``), the layer that ``_fake_quant_token_4d``
    (``src/beyond/runtime/vllm/packed_backend.py:1081-1154``) is defined to agree with and that
    ``quant/tests/test_pack_roundtrip.py:56-103`` compares the packed path against."""
    from beyond.quantization.layers import UnifiedQuantLayer

    out = {}
    B, S, H, D = 2, 13, 2, 128
    rng = np.random.default_rng(505)
    x32 = rng.standard_normal((B, S, H, D)).astype(np.float32)
    x32[..., 7] *= 8.0
    layer = UnifiedQuantLayer(num_bits=4, group_size=32, grouping_dim="token", quant_width=H * D)
    levels, thresholds = layer.materialize_quant_tables()
    out["fq_x32"] = x32
    out["fq_levels"] = levels.detach().float().numpy()
    out["fq_thresholds"] = thresholds.detach().float().numpy()
    with torch.no_grad():
        out["fq_y32"] = layer(torch.from_numpy(x32).reshape(B, S, H * D)).reshape(B, S, H, D).numpy()
        for name, dt in (("f16", torch.float16), ("bf16", torch.bfloat16)):
            y = layer(torch.from_numpy(x32).to(dt).reshape(B, S, H * D)).reshape(B, S, H, D)
            out[f"fq_y_bits_{name}"] = bits16(y)
    return out


def main() -> None:
    torch.manual_seed(0)
    makers = {
        "kat": lambda: {**kat_cases(), **layout_cases()},
        "writer": writer_cases,
        "config0": config0_case,
        "fakeqdq": fakeqdq_case,
    }
    for name in sys.argv[1:] or list(makers):
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **makers[name]())
        print(f"{name}.npz", os.path.getsize(os.path.join(HERE, f"{name}.npz")), "bytes")


if __name__ == "__main__":
    main()
