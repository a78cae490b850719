"""B200-native packed-KV serving hot path: encode-on-write and fused paged decode
attention over the 4-bit / group-32 cache, as hand-written sm_100a CUDA behind a C ABI.

Sub-packages mirror the module paths of the reference project so that a caller swaps
imports and nothing else:

* ``quant.beyond_cute``                          <- ``quant/beyond_cute.py``
* ``quant.fa4_cute.beyond_decode_policy``        <- ``quant/fa4_cute/beyond_decode_policy.py``
* ``quant.fa4_cute.beyond_mixed_decode_runtime`` <- ``quant/fa4_cute/beyond_mixed_decode_runtime.py``
* ``runtime.vllm.packed_backend``                <- attention-backend interface of
  ``src/beyond/runtime/vllm/packed_backend.py``

The directory is named ``beyond-kv-cache_b200``; Python imports it as
``beyond_kv_cache_b200`` (see the alias package of that name at the repository root).
"""

__version__ = "0.1.0"
