"""CPU oracle for the packed-KV hot path (TEST INFRASTRUCTURE, not product code).

This package restates, in plain numpy, the arithmetic of the reference's
4-bit/G32 quantiser, its paged cache ABI and its exact-mode decode attention.
Each function cites the reference file:line it follows.  The oracle is pinned
against vectors produced by the reference's own Python code (see
``tests/golden/make_golden.py`` and ``tests/test_oracle_golden.py``).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference
legs of ``bench.py`` may import this package.  The product package never does:
it calls the sm_100a CUDA library and raises when that library is missing.
"""

from .quantizer import (  # noqa: F401
    GROUP,
    LEVELS,
    decode_groups,
    encode_groups,
    fake_qdq_unrounded,
    pack_nibbles,
    round_to_stat,
    stat_to_f32,
    uniform_levels,
    uniform_thresholds,
    unpack_nibbles,
)
from .paged import PageGeometry, read_request, write_pages  # noqa: F401
from .attention import decode_attention, merge_partials  # noqa: F401
