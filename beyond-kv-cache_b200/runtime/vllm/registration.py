"""Registers the packed backend with vLLM (reference ``src/beyond/runtime/vllm/registration.py``).

Done here: the ``CUSTOM`` slot of vLLM's attention-backend registry points at
``BeyondPackedBackend``; caches described by the packed spec (a subclass of vLLM's
``FullAttentionSpec``, ``packed_backend.vllm_spec_class``) are managed by the stock full-attention
manager; ``Attention.get_kv_cache_spec`` returns that spec for layers served by the backend.  Not done here: the reference's scheduler, static-buffer, replay-warm-up and
graph-bucket patches of vLLM internals (reference `:23-25, :59`), which are serving glue
outside the packed-KV path.
"""

from __future__ import annotations


def register_backend() -> bool:
    """Wire the backend into vLLM; returns False (and does nothing) when this vLLM has no
    backend registry (the reference returns silently in that case, `:8-12`)."""
    try:
        from vllm.v1.attention.backends.registry import AttentionBackendEnum
        from vllm.v1.attention.backends.registry import register_backend as register
    except ImportError:
        return False

    import torch

    from . import packed_backend as backend

    cls = backend.BeyondPackedBackend
    register(AttentionBackendEnum.CUSTOM, f"{cls.__module__}.{cls.__qualname__}")

    from vllm.v1.core.single_type_kv_cache_manager import FullAttentionManager, spec_manager_map

    # one full-attention cache per layer, whatever its byte layout
    spec_cls = backend.vllm_spec_class()
    spec_manager_map.setdefault(spec_cls, FullAttentionManager)

    from vllm.model_executor.layers.attention.attention import Attention
    from vllm.v1.attention.backend import AttentionType

    if not getattr(Attention.get_kv_cache_spec, "_beyond_patched", False):
        stock = Attention.get_kv_cache_spec

        def get_kv_cache_spec(self, vllm_config):
            if self.attn_backend.get_name() != "CUSTOM":
                return stock(self, vllm_config)
            if self.attn_type != AttentionType.DECODER:
                raise AssertionError("BeyondPacked only supports DECODER attention")
            return spec_cls(block_size=vllm_config.cache_config.block_size, num_kv_heads=self.num_kv_heads,
                            head_size=self.head_size, dtype=torch.int32)

        get_kv_cache_spec._beyond_patched = True
        Attention.get_kv_cache_spec = get_kv_cache_spec
    return True
