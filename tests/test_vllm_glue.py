"""vLLM-facing glue on CPU: environment readers, the layout contract, the metadata builder
and the registry wiring (against a stand-in for the vLLM modules it touches)."""

import sys
import types
from types import SimpleNamespace

import pytest
import torch

from beyond_kv_cache_b200.runtime.vllm import config, packed_backend, registration


def test_env_readers(monkeypatch):
    monkeypatch.setenv("X_INT", "12")
    monkeypatch.setenv("X_BAD", "twelve")
    assert config.env_int("X_INT", 3) == 12 and config.env_int("X_BAD", 3) == 3 and config.env_int("X_UNSET", 3) == 3
    for word, want in (("Yes", True), ("off", False), ("enabled", True), ("none", False), ("maybe", True)):
        monkeypatch.setenv("X_BOOL", word)
        assert config.env_bool("X_BOOL", True) is want
    assert config.env_bool("X_UNSET", False) is False
    monkeypatch.setenv("X_BITS", "7")
    with pytest.raises(ValueError, match="supports bits"):
        config.env_bits("X_BITS")
    monkeypatch.setenv("X_BITS", "4")
    assert config.env_bits("X_BITS") == 4


def test_real_packed_layout_contract():
    config.validate_real_packed_layout(4, 32, 32)
    with pytest.raises(NotImplementedError, match="only 4-bit"):
        config.validate_real_packed_layout(5, 32, 32)
    with pytest.raises(NotImplementedError, match="k_group_size"):
        config.validate_real_packed_layout(4, 64, 32)
    with pytest.raises(NotImplementedError, match="v_group_size"):
        config.validate_real_packed_layout(4, 32, 16)


def test_metadata_builder_mirrors_the_request_plan_on_the_host():
    common = SimpleNamespace(
        num_reqs=3, num_actual_tokens=3, max_query_len=1, max_seq_len=40,
        query_start_loc=torch.tensor([0, 1, 2, 3], dtype=torch.int32), query_start_loc_cpu=torch.tensor([0, 1, 2, 3]),
        seq_lens=torch.tensor([40, 7, 19], dtype=torch.int32), seq_lens_cpu=torch.tensor([40, 7, 19]),
        block_table_tensor=torch.zeros((3, 3), dtype=torch.int32), slot_mapping=torch.tensor([39, 70, 118]))
    builder = packed_backend.BeyondPackedBackend.get_builder_cls()()
    m = builder.build(0, common)
    assert m.num_actual_tokens == 3 and m._beyond_seq_lens_list == [40, 7, 19] and m._beyond_query_start_loc_list == [0, 1, 2, 3]
    assert m.block_table is common.block_table_tensor and m.max_seq_len == 40
    cap = builder.build_for_cudagraph_capture(common)
    assert cap._beyond_seq_lens_list == [40, 40, 40] and cap._beyond_query_start_loc_list == [0, 1, 2, 3]
    del common.seq_lens_cpu
    assert builder.build(0, common)._beyond_seq_lens_list is None  # forward() then reads the device tensor


def test_register_backend_without_a_registry_is_a_no_op(monkeypatch):
    monkeypatch.setitem(sys.modules, "vllm.v1.attention.backends.registry", None)  # import fails
    assert registration.register_backend() is False


def test_register_backend_wires_registry_manager_and_spec(monkeypatch):
    calls = {}

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        monkeypatch.setitem(sys.modules, name, m)
        return m

    class FullAttentionManager:
        pass

    class Attention:
        def __init__(self, name):
            self.attn_backend = SimpleNamespace(get_name=lambda: name)
            self.attn_type, self.num_kv_heads, self.head_size = "decoder", 8, 128

        def get_kv_cache_spec(self, vllm_config):
            return "stock"

    from dataclasses import dataclass

    @dataclass(frozen=True, kw_only=True)
    class FullAttentionSpec:  # the fields the packed spec relies on
        block_size: int
        num_kv_heads: int
        head_size: int
        dtype: object = None

    monkeypatch.setattr(packed_backend, "_VLLM_SPEC_CLASS", None)
    manager_map = {}
    for pkg in ("vllm", "vllm.v1", "vllm.v1.attention", "vllm.v1.attention.backends", "vllm.v1.core",
                "vllm.model_executor", "vllm.model_executor.layers", "vllm.model_executor.layers.attention"):
        mod(pkg)
    mod("vllm.v1.attention.backends.registry", AttentionBackendEnum=SimpleNamespace(CUSTOM="CUSTOM"),
        register_backend=lambda slot, qualname: calls.update(slot=slot, qualname=qualname))
    mod("vllm.v1.kv_cache_interface", FullAttentionSpec=FullAttentionSpec)
    mod("vllm.v1.core.single_type_kv_cache_manager", FullAttentionManager=FullAttentionManager, spec_manager_map=manager_map)
    mod("vllm.model_executor.layers.attention.attention", Attention=Attention)
    mod("vllm.v1.attention.backend", AttentionType=SimpleNamespace(DECODER="decoder"))

    assert registration.register_backend() is True
    assert calls["slot"] == "CUSTOM" and calls["qualname"].endswith("packed_backend.BeyondPackedBackend")
    spec_cls = packed_backend.vllm_spec_class()
    assert issubclass(spec_cls, FullAttentionSpec) and manager_map[spec_cls] is FullAttentionManager
    cfg = SimpleNamespace(cache_config=SimpleNamespace(block_size=16))
    spec = Attention("CUSTOM").get_kv_cache_spec(cfg)
    assert isinstance(spec, spec_cls) and spec.real_page_size_bytes == 16 * 8 * 160
    assert Attention("FLASH_ATTN").get_kv_cache_spec(cfg) == "stock"
    patched = Attention.get_kv_cache_spec
    assert registration.register_backend() is True and Attention.get_kv_cache_spec is patched  # idempotent


def test_packed_spec_against_the_installed_vllm(monkeypatch):
    """Against the vLLM that is actually installed (skipped when it does not import here): the
    packed spec is a KVCacheSpec that vLLM's page-size arithmetic accepts, its page is the packed
    page, and the registry has the CUSTOM slot the backend registers into."""
    pytest.importorskip("vllm")
    try:
        from vllm.v1.attention.backends.registry import AttentionBackendEnum
        from vllm.v1.kv_cache_interface import FullAttentionSpec, KVCacheSpec
    except Exception as exc:  # an installed vLLM whose pieces need a GPU driver to import
        pytest.skip(f"vLLM interfaces not importable here: {exc!r}")
    import torch

    monkeypatch.setattr(packed_backend, "_VLLM_SPEC_CLASS", None)
    spec_cls = packed_backend.vllm_spec_class()
    assert issubclass(spec_cls, FullAttentionSpec) and issubclass(spec_cls, KVCacheSpec)
    spec = spec_cls(block_size=16, num_kv_heads=8, head_size=128, dtype=torch.int32)
    assert spec.real_page_size_bytes == 5120 * 4 == packed_backend.BeyondPackedSpec(16, 8, 128).real_page_size_bytes
    assert spec.page_size_bytes == 5120 * 4  # what the allocator sizes the pool with
    big = spec_cls(block_size=128, num_kv_heads=8, head_size=128, dtype=torch.int32)
    assert big.page_size_bytes == 8 * 5120 * 4
    assert hasattr(AttentionBackendEnum, "CUSTOM")
    shape = packed_backend.BeyondPackedBackend.get_kv_cache_shape(7, 16, 8, 128)
    assert shape[0] * shape[1] * 4 == 7 * spec.page_size_bytes
