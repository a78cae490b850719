"""Launch policy of the split grid (pure Python).  The invariants are those the reference
holds its own policy to (tests/test_sm100_nonuniform_decode_policy.py:28-120) where they carry
over: the largest CTA chunk is ceil(tiles / splits), non-positive inputs are refused, the
modelled split count never exceeds the tiles or the cap of 32, and the plan is consistent.
The reference's frozen B300 frontier values do not apply to this kernel."""

import pytest

from beyond_kv_cache_b200.quant.fa4_cute.beyond_decode_policy import (
    MAX_SPLITS,
    DecodeLaunchPlan,
    modeled_splits,
    normalize_reduction_kind,
    scheduled_pages_per_split,
    select_decode_launch_plan,
)


@pytest.mark.parametrize("tiles,splits,expected", [(24, 3, 8), (25, 4, 7), (8, 8, 1), (1, 1, 1), (513, 32, 17)])
def test_largest_cta_chunk(tiles, splits, expected):
    assert scheduled_pages_per_split(tiles=tiles, splits=splits) == expected


@pytest.mark.parametrize("kwargs", [
    {"tiles": 0, "splits": 1},
    {"tiles": 8, "splits": 0},
    {"tiles": 8, "splits": 3, "adaptive_split_base": 0, "adaptive_extra_tasks": 1},
    {"tiles": 8, "splits": 4, "adaptive_split_base": 2, "adaptive_extra_tasks": 1},
])
def test_inconsistent_schedules_are_refused(kwargs):
    with pytest.raises(ValueError):
        scheduled_pages_per_split(**kwargs)


def test_split_count_bounds():
    assert modeled_splits(tiles=3, batch=1, heads_kv=4, sm_count=148) <= 3
    assert modeled_splits(tiles=8192, batch=1, heads_kv=4, sm_count=148) <= MAX_SPLITS
    assert modeled_splits(tiles=8192, batch=1, heads_kv=8, sm_count=148, max_splits=5) <= 5
    assert modeled_splits(tiles=1, batch=64, heads_kv=8, sm_count=148) == 1
    # a grid that already fills the machine several times over gains nothing from splitting
    assert modeled_splits(tiles=64, batch=4096, heads_kv=8, sm_count=148) == 1
    # one long request cannot occupy the machine without splitting
    assert modeled_splits(tiles=8192, batch=1, heads_kv=8, sm_count=148) > 8


def test_split_count_never_falls_when_the_context_grows():
    for batch in (1, 5, 16, 64):
        counts = [modeled_splits(tiles=t, batch=batch, heads_kv=8, sm_count=148) for t in (1, 4, 24, 128, 1024, 8192)]
        assert counts == sorted(counts), (batch, counts)


@pytest.mark.parametrize("bad", [
    {"tiles": 0}, {"batch": 0}, {"heads_kv": -1}, {"sm_count": 0}, {"max_splits": 0}, {"page_size": 0},
])
def test_non_positive_inputs_are_refused(bad):
    args = {"tiles": 16, "batch": 4, "heads_kv": 8, "sm_count": 148, **bad}
    with pytest.raises(ValueError, match="must be positive"):
        modeled_splits(**args)


def test_plan_is_consistent():
    plan = select_decode_launch_plan(tiles=512, batch=4, heads_kv=8, sm_count=148, model_dtype="bf16", page_size=16)
    assert isinstance(plan, DecodeLaunchPlan)
    assert plan.splits == modeled_splits(tiles=512, batch=4, heads_kv=8, sm_count=148, page_size=16)
    assert plan.pages_per_split == scheduled_pages_per_split(tiles=512, splits=plan.splits)
    assert plan.reduction_kind == "lse_combine"
    assert not (plan.cluster_reduction or plan.task_major_grid or plan.direct_smem_store)
    with pytest.raises(ValueError, match="unsupported model_dtype"):
        select_decode_launch_plan(tiles=512, batch=4, heads_kv=8, sm_count=148, model_dtype="fp32")
    with pytest.raises(ValueError, match="must be positive"):
        select_decode_launch_plan(tiles=0, batch=4, heads_kv=8, sm_count=148, model_dtype="bf16")


def test_reducer_names_of_the_reference_are_aliases():
    for name in ("auto", "parallel", "cta4", "warp_parallel", "warp_parallel2", " AUTO "):
        assert normalize_reduction_kind(name) == "lse_combine"
    with pytest.raises(ValueError, match="BEYOND_SM103_REDUCTION_KIND"):
        normalize_reduction_kind("tree")


def test_device_status_is_turned_into_an_exception(monkeypatch):
    """The error-reporting path on the host (no device involved): whatever the status entry point
    reports is raised with its meaning; zero is silent."""
    from beyond_kv_cache_b200 import _lib
    from beyond_kv_cache_b200.quant.fa4_cute import beyond_mixed_decode_runtime as rt

    reported = {"value": 0}

    def fake_call(name, ref):
        assert name == "bkv_decode_device_status"
        ref._obj.value = reported["value"]

    monkeypatch.setattr(_lib, "call", fake_call)
    rt.check_device_status()
    reported["value"] = 2
    with pytest.raises(_lib.BkvError, match="bounded wait"):
        rt.check_device_status()
    reported["value"] = 3
    with pytest.raises(_lib.BkvError, match="unexpected address"):
        rt.check_device_status()
