"""Launch policy of the B200 packed decode kernel (pure Python, no device access).

Mirror of the reference policy module ``quant/fa4_cute/beyond_decode_policy.py``:
the same function names and the same ``DecodeLaunchPlan`` fields, so the launcher
and its callers do not change.  The numbers are not the reference's B300 look-up
tables: the B200 kernel keeps one persistent-size CTA per SM that owns a *run* of
16-token tiles, so its only shape-dependent choice is the split-KV count, which is
taken from a resident-wave cost model of that kernel (reference model:
``modeled_splits``, ``quant/fa4_cute/beyond_decode_policy.py:165-201``).
"""

from __future__ import annotations

from dataclasses import dataclass

TILE_TOKENS = 16  # tokens one warp consumes per step of the sm_100a kernel
MAX_SPLITS = 32  # same cap as the reference launcher (runtime.py:217-218)

# Cost-model constants, in units of "one 16-token tile processed by one CTA".
_CTA_FIXED_TILES = 40.0  # table build + prologue + epilogue of one CTA
_COMBINE_BASE_TILES = 16.0  # extra launch + partial round trip when splits > 1
_COMBINE_PER_SPLIT = 0.02  # per (request, split) reducer work
_REDUCTION_KINDS = ("lse_combine", "parallel", "cta4", "warp_parallel", "warp_parallel2")


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

    One CTA is resident per SM, so ``waves = ceil(batch * heads_kv * splits /
    sm_count)``.  More splits shorten each CTA and smooth the last wave, but every
    CTA pays a fixed cost and ``splits > 1`` adds the combine launch.  ``tiles``
    counts pages of ``page_size`` tokens (``page_size / 16`` kernel steps each)."""
    _require_positive(
        tiles=tiles, batch=batch, heads_kv=heads_kv, sm_count=sm_count, max_splits=max_splits, page_size=page_size
    )
    tasks = int(batch) * int(heads_kv)
    steps_per_page = max(1.0, int(page_size) / TILE_TOKENS)

    def cost(splits: int) -> tuple[float, int]:
        waves = (tasks * splits + sm_count - 1) // sm_count
        per_cta = ((tiles + splits - 1) // splits) * steps_per_page + _CTA_FIXED_TILES
        total = waves * per_cta
        if splits > 1:
            total += _COMBINE_BASE_TILES + _COMBINE_PER_SPLIT * batch * splits
        return total, splits

    return min(range(1, min(int(max_splits), int(tiles)) + 1), key=cost)


def select_reduction_kind(*, batch: int, splits: int, pages_per_split: int | None = None) -> str:
    """The B200 build has a single log-sum-exp combine kernel; the reference's
    three reducer variants (:227-251) collapse into it."""
    _require_positive(batch=batch, splits=splits)
    if pages_per_split is not None:
        _require_positive(pages_per_split=pages_per_split)
    return "lse_combine"


def normalize_reduction_kind(kind: str) -> str:
    """Accept the reference's reducer names as aliases of the single combine kernel."""
    kind = str(kind).strip().lower()
    if kind == "auto":
        return "lse_combine"
    if kind not in _REDUCTION_KINDS:
        raise ValueError(
            "BEYOND_SM103_REDUCTION_KIND must be auto, parallel, cta4, warp_parallel, or warp_parallel2"
        )
    return "lse_combine"


def packed_kv_stage_cap(*, pages_per_split: int) -> int:
    """Depth of the per-warp page ring (tiles in flight per warp)."""
    if int(pages_per_split) <= 0:
        raise ValueError("packed-KV stage input must be positive: pages_per_split")
    return 4


def conversion_stage_cap(*, splits: int, pages_per_split: int, model_dtype: str | None = None) -> int:
    """Dequantisation happens in registers, so there is no conversion staging."""
    _require_positive(splits=splits, pages_per_split=pages_per_split)
    if model_dtype not in (None, "fp16", "bf16"):
        raise ValueError(f"unsupported model_dtype: {model_dtype}")
    return 1


def select_cluster_splits(*, tiles: int, batch: int, heads_kv: int) -> int:
    """No thread-block-cluster reduction in this build: always 0."""
    _require_positive(tiles=tiles, batch=batch, heads_kv=heads_kv)
    return 0


def select_direct_smem_store(*, batch: int, heads_kv: int, splits: int, pages_per_split: int) -> bool:
    _require_positive(batch=batch, heads_kv=heads_kv, splits=splits, pages_per_split=pages_per_split)
    return False


def select_task_major_grid(*, batch: int, splits: int, pages_per_split: int) -> bool:
    _require_positive(batch=batch, splits=splits, pages_per_split=pages_per_split)
    return False


def select_decode_launch_plan(
    *, tiles: int, batch: int, heads_kv: int, sm_count: int, model_dtype: str, page_size: int = TILE_TOKENS
) -> DecodeLaunchPlan:
    """Plan for one bucket; ``tiles`` is the number of *pages* of the bucket
    (``max_seq_len // page_size``), as in the reference (:337-433)."""
    _require_positive(tiles=tiles, batch=batch, heads_kv=heads_kv, sm_count=sm_count)
    if model_dtype not in {"fp16", "bf16"}:
        raise ValueError(f"unsupported model_dtype: {model_dtype}")
    splits = modeled_splits(tiles=tiles, batch=batch, heads_kv=heads_kv, sm_count=sm_count, page_size=page_size)
    pages = scheduled_pages_per_split(tiles=tiles, splits=splits)
    return DecodeLaunchPlan(
        splits=splits,
        pages_per_split=pages,
        reduction_kind=select_reduction_kind(batch=batch, splits=splits, pages_per_split=pages),
        kv_stage_cap=packed_kv_stage_cap(pages_per_split=pages),
        cvt_stage_cap=conversion_stage_cap(splits=splits, pages_per_split=pages, model_dtype=model_dtype),
        cluster_reduction=False,
        task_major_grid=False,
        direct_smem_store=False,
    )
