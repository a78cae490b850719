"""Quant-config loader and FP16 table ABI (CPU): the behaviours the reference's own loader
tests pin (tests/runtime/vllm/test_quant_config.py, tests/test_table_precision.py), on files
generated here, plus the table resolution the kernels use and, when the reference tree is
present, a field-by-field comparison with the reference loader on the same files."""

import json
import os
import sys

import pytest
import torch

from beyond_kv_cache_b200.quantization import runtime_config as rc
from beyond_kv_cache_b200.quantization import table_precision as tp


def _tables(num_tables, bits, *, dtype=torch.float32, seed=0):
    g = torch.Generator().manual_seed(seed)
    levels = 1 << bits
    qp = torch.sort(torch.rand((num_tables, levels), generator=g), dim=-1).values
    qp = qp + torch.arange(levels) * 2.0**-8  # keep neighbours apart after float16 rounding
    qp = (qp - qp[:, :1]) / (qp[:, -1:] - qp[:, :1])
    th = (qp[:, 1:] + qp[:, :-1]) / 2
    return qp.to(dtype), th.to(dtype)


def _entry(num_tables=32, bits=4, **extra):
    qp, th = _tables(num_tables, bits)
    e = {"type": "UnifiedQuantLayer", "num_bits": bits, "grouping_dim": "token", "table_axis": "group",
         "quant_points": qp, "thresholds": th}
    e.update(extra)
    return e


def _fp16_entry(num_tables=32, **extra):
    qp, th = _tables(num_tables, 4)
    e = {"num_bits": 4, "grouping_dim": "token", "quant_points": tp.cast_table_for_storage(qp),
         "thresholds": tp.cast_table_for_storage(th), "table_storage_dtype": "float16",
         "table_precision_abi": tp.TABLE_PRECISION_ABI, "table_compute_dtype": "float32"}
    e.update(extra)
    return e


def _save(tmp_path, raw, name="quant_config_4bit.pt"):
    path = str(tmp_path / name)
    if name.endswith(".pt"):
        torch.save(raw, path)
    else:
        def plain(v):
            if torch.is_tensor(v):
                return v.tolist()
            if isinstance(v, dict):
                return {k: plain(x) for k, x in v.items()}
            return v
        with open(path, "w") as f:
            json.dump(plain(raw), f)
    return path


def test_loads_grouped_tables_and_finds_the_layer(tmp_path):
    raw = {f"model.layers.{i}.self_attn.{p}": _entry() for i in range(2) for p in ("k_proj", "v_proj")}
    for name in ("cfg.pt", "cfg.json"):
        cfg = rc.QuantConfig.load(_save(tmp_path, raw, name), expected_bits=4)
        assert len(cfg) == 4
        k = cfg.for_attention_layer("model.layers.1.self_attn.attn", "k_proj")
        assert k is not None and k.num_bits == 4 and k.table_axis == "group"
        assert tuple(k.q_points.shape) == (32, 16) and tuple(k.thresholds.shape) == (32, 15)
        assert k.table_storage_dtype == "float32" and k.table_precision_abi == tp.LEGACY_TABLE_PRECISION_ABI
        assert cfg.for_attention_layer("model.layers.7.self_attn.attn", "k_proj") is None
        assert cfg.identity.startswith(os.path.abspath(str(tmp_path)))


def test_module_prefix_aliases(tmp_path):
    raw = {"model.language_model.layers.0.self_attn.k_proj": _entry(), "model.layers.3.self_attn.v_proj": _entry()}
    cfg = rc.QuantConfig.load(_save(tmp_path, raw))
    assert cfg.for_attention_layer("language_model.model.layers.0.self_attn.attn", "k_proj") is not None
    assert cfg.for_attention_layer("language_model.model.layers.3.self_attn.attn", "v_proj") is not None


def test_fused_qkv_exports_are_unfolded(tmp_path):
    for suffix in ("query_key_value", "qkv_proj"):
        raw = {f"model.layers.0.self_attn.{suffix}": {"type": "QuantizedQKVLinear", "k": _entry(), "v": _entry()}}
        cfg = rc.QuantConfig.load(_save(tmp_path, raw, f"{suffix}.pt"))
        assert cfg.for_attention_layer("model.layers.0.self_attn.attn", "k_proj") is not None
        assert cfg.for_attention_layer("model.layers.0.self_attn.attn", "v_proj") is not None


@pytest.mark.parametrize("mutate,fragment", [
    (lambda e: e.update(num_bits=5, quant_points=_tables(4, 5)[0], thresholds=_tables(4, 5)[1]), "num_bits"),
    (lambda e: e.update(grouping_dim="sequence"), "token-grouped"),
    (lambda e: e.update(thresholds=e["thresholds"][:, :-1]), "thresholds shape"),
    (lambda e: e.update(quant_points=e["quant_points"].flip(-1)), "strictly increasing"),
    (lambda e: e.update(thresholds=e["thresholds"] + 2.0), "normalized range"),
    (lambda e: e.update(table_axis="shared"), "rank-1"),
    (lambda e: e.update(group_size=0), "group_size must be positive"),
])
def test_invalid_entries_are_refused(tmp_path, mutate, fragment):
    e = _entry()
    mutate(e)
    with pytest.raises(ValueError, match=fragment):
        rc.QuantConfig.load(_save(tmp_path, {"model.layers.0.self_attn.k_proj": e}), expected_bits=4)


def test_fp16_table_abi_rules(tmp_path):
    key = "model.layers.0.self_attn.k_proj"
    cfg = rc.QuantConfig.load(_save(tmp_path, {key: _fp16_entry()}))
    got = cfg.for_attention_layer("model.layers.0.self_attn.attn", "k_proj")
    assert got.q_points.dtype == torch.float16 and got.table_precision_abi == tp.TABLE_PRECISION_ABI
    tp.validate_fp16_storage_tables(got.q_points, got.thresholds, label=key)
    with pytest.raises(ValueError, match="float16 tables require"):
        rc.QuantConfig.load(_save(tmp_path, {key: _fp16_entry(table_precision_abi=tp.LEGACY_TABLE_PRECISION_ABI)}))
    e = _fp16_entry()
    del e["table_precision_abi"]
    with pytest.raises(ValueError, match="explicit table_precision_abi"):
        rc.QuantConfig.load(_save(tmp_path, {key: e}))
    e = _fp16_entry()
    del e["table_compute_dtype"]
    with pytest.raises(ValueError, match="explicit table_compute_dtype"):
        rc.QuantConfig.load(_save(tmp_path, {key: e}))
    with pytest.raises(ValueError, match="requires float16 table storage"):
        rc.QuantConfig.load(_save(tmp_path, {key: _entry(table_storage_dtype="float32", table_precision_abi=tp.TABLE_PRECISION_ABI,
                                                          table_compute_dtype="float32")}))


def test_model_identity(tmp_path):
    run = tmp_path / "run" / "configs"
    run.mkdir(parents=True)
    (tmp_path / "run" / "metrics.json").write_text(json.dumps({"base_model": "org/Llama-3.1-8B"}))
    path = _save(run, {"model.layers.0.self_attn.k_proj": _entry()})
    assert rc.QuantConfig.load(path, expected_model="other-org/llama-3.1-8b").source_model == "org/Llama-3.1-8B"
    with pytest.raises(ValueError, match="does not match requested model"):
        rc.QuantConfig.load(path, expected_model="org/Mistral-7B")
    embedded = _save(tmp_path, {"__metadata__": {"base_model": "org/Qwen3-8B"}, "model.layers.0.self_attn.k_proj": _entry()})
    assert rc.QuantConfig.load(embedded).source_model == "org/Qwen3-8B"
    bare = _save(tmp_path, {"model.layers.0.self_attn.k_proj": _entry()}, "bare.pt")
    rc.QuantConfig.load(bare, expected_model="org/x")  # unknown origin is accepted unless metadata is required
    with pytest.raises(ValueError, match="cannot verify model identity"):
        rc.QuantConfig.load(bare, expected_model="org/x", require_model_metadata=True)


def test_other_artifacts_and_empty_files_are_refused(tmp_path):
    adapter = {"__metadata__": {"artifact_type": "beyond_uncompressed_kv_adapter_config"}, "model.layers.0.self_attn.k_proj": _entry()}
    with pytest.raises(ValueError, match="uncompressed continuous KV adapter"):
        rc.QuantConfig.load(_save(tmp_path, adapter))
    with pytest.raises(ValueError, match="no K/V projection entries"):
        rc.QuantConfig.load(_save(tmp_path, {"note": "nothing here"}, "empty.pt"))


def test_env_loader_caches_and_reloads(monkeypatch, tmp_path):
    path = _save(tmp_path, {"model.layers.0.self_attn.k_proj": _entry()})
    monkeypatch.setenv("BEYOND_QUANT_CONFIG", path)
    monkeypatch.setenv("BEYOND_BITS", "4")
    monkeypatch.delenv("BEYOND_MODEL_ID", raising=False)
    first = rc.get_config_from_env()
    assert first is rc.get_config_from_env()
    torch.save({"model.layers.0.self_attn.k_proj": _entry(seed=5) if False else _entry(num_tables=8)}, path)
    again = rc.get_config_from_env(force_reload=True)
    assert again is not first and again.identity != first.identity
    monkeypatch.delenv("BEYOND_QUANT_CONFIG")
    assert rc.get_config_from_env() is None


def test_tables_of_a_layer_for_the_kernels_and_tensor_parallel_slicing(tmp_path):
    raw = {f"model.layers.0.self_attn.{p}": _fp16_entry(num_tables=32) for p in ("k_proj", "v_proj")}  # 8 KV heads x 4 groups
    cfg = rc.QuantConfig.load(_save(tmp_path, raw))
    lk, tk, lv, tv = rc.resolve_layer_tables(cfg, "model.layers.0.self_attn.attn", heads_kv=8)
    assert tuple(lk.shape) == (32, 16) and tuple(tv.shape) == (32, 15) and lk.dtype == torch.float16
    full_k = cfg.for_attention_layer("model.layers.0.self_attn.attn", "k_proj").q_points
    for rank in range(4):  # 2 local KV heads per rank
        lk_r, tk_r, _, _ = rc.resolve_layer_tables(cfg, "model.layers.0.self_attn.attn", heads_kv=2, tp_rank=rank, tp_world=4)
        assert torch.equal(lk_r, full_k[rank * 8 : rank * 8 + 8]) and tuple(tk_r.shape) == (8, 15)
    with pytest.raises(ValueError, match="does not match local"):
        rc.resolve_layer_tables(cfg, "model.layers.0.self_attn.attn", heads_kv=3, tp_rank=0, tp_world=2)
    with pytest.raises(KeyError):
        rc.resolve_layer_tables(cfg, "model.layers.9.self_attn.attn", heads_kv=8)
    # the resolved tables are what the packed writer's table preparation accepts
    from beyond_kv_cache_b200.quant.beyond_cute import prepare_qpoints_and_thresholds
    qp, th = prepare_qpoints_and_thresholds(num_bits=4, device=torch.device("cpu"), q_points=lk, thresholds=tk)
    assert qp.dtype == torch.float16 and torch.equal(qp, lk) and torch.equal(th, tk)


def test_table_precision_contract():
    master = torch.tensor([0.1, 0.2, 0.30001], requires_grad=True)
    seen = tp.fp16_ste_roundtrip(master)
    assert torch.equal(seen.detach(), master.detach().half().float())
    seen.sum().backward()
    assert torch.equal(master.grad, torch.ones(3))
    with pytest.raises(TypeError):
        tp.fp16_ste_roundtrip(master.detach().half())
    with pytest.raises(ValueError, match="collapse"):
        tp.validate_fp16_storage_tables(torch.tensor([[0.0, 0.5, 0.5]], dtype=torch.float16),
                                        torch.tensor([[0.25, 0.75]], dtype=torch.float16), label="t")
    with pytest.raises(TypeError):
        tp.validate_fp16_storage_tables(torch.zeros((1, 3)), torch.zeros((1, 2), dtype=torch.float16))
    assert tp.storage_dtype_name(torch.zeros(1, dtype=torch.float16)) == "float16"
    assert tp.torch_dtype_for_storage(" Float32 ") == torch.float32
    with pytest.raises(ValueError):
        tp.torch_dtype_for_storage("half")
    assert tp.FP16_STRICT_MIN_GAP == 2.0**-9


def test_matches_the_reference_loader_when_present(tmp_path):
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref_src = os.path.join(os.environ.get("BEYOND_REFERENCE", os.path.join(os.path.dirname(repo), "reference")), "src")
    if not os.path.isdir(ref_src):
        pytest.skip("reference tree not present")
    sys.path.insert(0, ref_src)
    try:
        try:
            from beyond.quantization import runtime_config as ref
        except Exception as exc:  # the reference package may need modules this container lacks
            pytest.skip(f"reference loader does not import here: {exc!r}")
        raw = {"__metadata__": {"base_model": "org/m"},
               "model.layers.0.self_attn.k_proj": _fp16_entry(),
               "model.layers.0.self_attn.v_proj": _entry(num_tables=32, group_size=32),
               "model.layers.1.self_attn.qkv_proj": {"k": _entry(), "v": _entry()}}
        path = _save(tmp_path, raw)
        ours, theirs = rc.QuantConfig.load(path, expected_bits=4), ref.QuantConfig.load(path, expected_bits=4)
        assert ours.identity == theirs.identity and ours.source_model == theirs.source_model
        assert sorted(k for k, _ in ours.items()) == sorted(k for k, _ in theirs.items())
        for key, a in ours.items():
            b = dict(theirs.items())[key]
            assert torch.equal(a.q_points, b.q_points) and torch.equal(a.thresholds, b.thresholds)
            for field in ("num_bits", "grouping_dim", "table_storage_dtype", "table_precision_abi", "table_compute_dtype",
                          "table_axis", "group_size"):
                assert getattr(a, field) == getattr(b, field), field
    finally:
        sys.path.remove(ref_src)
