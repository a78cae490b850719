"""Launch policy of the split-grid form of the B200 packed decode (pure Python, no device access).

Mirror of the reference policy module ``quant/fa4_cute/beyond_decode_policy.py``: the same
``DecodeLaunchPlan`` fields and the entry points the launcher calls, so the launcher and its
callers do not change.  The numbers are not the reference's B300 look-up tables.  On B200 the
production kernel is persistent and has no split count at all; a plan is only drawn up for the
general split grid (``bkv_decode_sm100``: one small CTA per (split, kv head, request)), whose one
shape-dependent choice is the split-KV count.  It comes from a resident-wave cost model of that
kernel (the reference's counterpart is ``modeled_splits``, :165-201).  The reference's other
choices - reducer variant, staging depths, cluster reduction, grid order, direct shared-memory
stores (:204-334) - have no counterpart in this kernel and are recorded in the plan as the
constants below.
"""

from __future__ import annotations

from dataclasses import dataclass

TILE_TOKENS = 16  # tokens per step of the cost model
MAX_SPLITS = 32  # same cap as the reference launcher (runtime.py:217-218)
REDUCTION_KIND = "lse_combine"  # the one log-sum-exp combine kernel
KV_STAGE_CAP = 1  # the split grid reads pages with plain loads: nothing is staged
CVT_STAGE_CAP = 1  # dequantisation happens in registers

_RESIDENT_CTAS_PER_SM = 12  # 128-thread CTAs of the split grid that share an SM
_CTA_FIXED_STEPS = 6.0  # prologue + warp merge + epilogue of one CTA, in 16-token steps
_COMBINE_BASE_STEPS = 24.0  # extra launch + partial round trip when splits > 1
_COMBINE_PER_SPLIT = 0.02  # per (request, split) reducer work
_REFERENCE_REDUCERS = ("parallel", "cta4", "warp_parallel", "warp_parallel2")


@dataclass(frozen=True)
class DecodeLaunchPlan:
    """Concrete launch configuration for one decode bucket (field names of the
    reference plan, ``beyond_decode_policy.py:8-19``)."""

    splits: int
    pages_per_split: int
    reduction_kind: str
    kv_stage_cap: int
    cvt_stage_cap: int
    cluster_reduction: bool
    task_major_grid: bool
    direct_smem_store: bool


def _require_positive(**values: int) -> None:
    bad = [name for name, value in values.items() if int(value) <= 0]
    if bad:
        raise ValueError(f"launch-policy inputs must be positive: {', '.join(bad)}")


def scheduled_pages_per_split(
    *, tiles: int, splits: int, adaptive_split_base: int = 0, adaptive_extra_tasks: int = 0
) -> int:
    """Largest number of pages any decode CTA visits: pages are dealt round-robin,
    so it is ``ceil(tiles / splits)``.  The adaptive-schedule arguments of the
    reference signature (:115-162) are accepted for compatibility and must be 0."""
    if int(tiles) <= 0 or int(splits) <= 0:
        raise ValueError("scheduled-page inputs must be positive: tiles, splits")
    if adaptive_split_base or adaptive_extra_tasks:
        raise ValueError("the B200 kernel has no adaptive split schedule")
    return (int(tiles) + int(splits) - 1) // int(splits)


def modeled_splits(
    *, tiles: int, batch: int, heads_kv: int, sm_count: int, max_splits: int = MAX_SPLITS, page_size: int = TILE_TOKENS
) -> int:
    """Split-KV count that minimises ``waves * (pages_per_split + fixed) + reducer``.

    ``waves = ceil(batch * heads_kv * splits / (sm_count * resident CTAs))``.  More splits
    shorten each CTA and smooth the last wave, but every CTA pays a fixed cost and
    ``splits > 1`` adds the combine launch.  ``tiles`` counts pages of ``page_size`` tokens
    (``page_size / 16`` steps each).  Never more than ``tiles`` or ``max_splits``."""
    _require_positive(
        tiles=tiles, batch=batch, heads_kv=heads_kv, sm_count=sm_count, max_splits=max_splits, page_size=page_size
    )
    tasks = int(batch) * int(heads_kv)
    slots = int(sm_count) * _RESIDENT_CTAS_PER_SM
    steps_per_page = max(1.0, int(page_size) / TILE_TOKENS)

    def cost(splits: int) -> tuple[float, int]:
        waves = (tasks * splits + slots - 1) // slots
        per_cta = ((int(tiles) + splits - 1) // splits) * steps_per_page + _CTA_FIXED_STEPS
        total = waves * per_cta
        if splits > 1:
            total += _COMBINE_BASE_STEPS + _COMBINE_PER_SPLIT * int(batch) * splits
        return total, splits  # ties go to the smaller count

    return min(range(1, min(int(max_splits), int(tiles)) + 1), key=cost)


def normalize_reduction_kind(kind: str) -> str:
    """Accept ``auto`` and the reference's reducer names (``BEYOND_SM103_REDUCTION_KIND``,
    :227-251) as aliases of the single combine kernel; anything else is an error."""
    kind = str(kind).strip().lower()
    if kind != "auto" and kind != REDUCTION_KIND and kind not in _REFERENCE_REDUCERS:
        raise ValueError(
            "BEYOND_SM103_REDUCTION_KIND must be auto, parallel, cta4, warp_parallel, or warp_parallel2"
        )
    return REDUCTION_KIND


def select_decode_launch_plan(
    *, tiles: int, batch: int, heads_kv: int, sm_count: int, model_dtype: str, page_size: int = TILE_TOKENS
) -> DecodeLaunchPlan:
    """Plan for one bucket of the split grid; ``tiles`` is the number of *pages* of the bucket
    (``max_seq_len // page_size``), as in the reference (:337-433)."""
    _require_positive(tiles=tiles, batch=batch, heads_kv=heads_kv, sm_count=sm_count)
    if model_dtype not in {"fp16", "bf16"}:
        raise ValueError(f"unsupported model_dtype: {model_dtype}")
    splits = modeled_splits(tiles=tiles, batch=batch, heads_kv=heads_kv, sm_count=sm_count, page_size=page_size)
    return DecodeLaunchPlan(
        splits=splits,
        pages_per_split=scheduled_pages_per_split(tiles=tiles, splits=splits),
        reduction_kind=REDUCTION_KIND,
        kv_stage_cap=KV_STAGE_CAP,
        cvt_stage_cap=CVT_STAGE_CAP,
        cluster_reduction=False,
        task_major_grid=False,
        direct_smem_store=False,
    )
