#!/usr/bin/env python
"""Headline benchmark: packed-KV decode attention, one layer, Llama-3.1-8B shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--batch B] [--ctx C] [--page P] [--splits S] [--stat fp16|bf16] [--no-extras]

A *step* is one pass of the hot path over one decode batch: fused paged decode attention of
one query token per request over its packed 4-bit cache.  Default workload (N=1): batch 64,
32 query / 8 KV heads, head_dim 128, context 8192, 16-token pages, random block table, bf16
queries; the cache holds real codes produced by the encode-on-write kernel from N(0,1) K/V
with four K outlier channels per head scaled by 8.

``value``  : packed-cache bytes attended per second (5 effective bits per scalar:
             seq_len * Hkv * 160 B per request), all ranks, inputs resident in HBM.  The timed
             region is exactly ``--steps`` steps; it is repeated until at least 200 steps have
             run and the median region is reported (``timed_regions`` says how many).
``e2e``    : the same metric for the full serving step through the public API with
             HOST inputs: pinned q / new-token K,V / slots / seq_lens -> device,
             encode-on-write of the new token, decode attention, output -> host.
``parity`` : max-abs error of the timed output of four of the batch's requests against the
             float64 CPU oracle over the same packed pages (checked outside the timed region).
On one GPU the line also carries the other measurements the path is judged by (``--no-extras``
skips them): ``sweep`` (contexts 1K / 32K / 128K at 4M KV tokens, with the bf16-KV kernels of the
same shape), ``vs_bf16_kv`` at the default workload, ``encode`` and ``readback`` on 262 144 rows
and the serving step of 256 sequences.  N > 1 (torchrun): every rank owns its own batch and page
pool (request-batch sharding, no collective on the data path), time is the max over ranks, and
``kv_split`` reports one 128K-token sequence whose KV range is split over the ranks.

``--impl reference`` times the reference's own CPU implementation of the same path (its
exact-mode attention: page read-back + float32 scaled-dot-product attention per request, staged
under ``oracle/_ref`` by ``oracle/make_ref.py``) on all host cores, on a bounded sample of the
same workload; without the staged module it times the numpy restatement (kind "port").
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

HEADS_Q, HEADS_KV, HEAD_DIM = 32, 8, 128
BYTES_PER_TOKEN_HEAD = 160  # 64 B K codes + 16 B K stats + 64 B V codes + 16 B V stats
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--splits", type=int, default=0, help="0 = launch policy")
    ap.add_argument("--stat", default="fp16", choices=["fp16", "bf16"])
    ap.add_argument("--loader", type=int, default=0, choices=[0, 1],
                    help="persistent schedule: 0 = 16-byte asynchronous copies (default), 1 = tensor copies")
    ap.add_argument("--cpu-sample-requests", type=int, default=0, help="0 = eight requests (one per core for the port)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline, e2e, parity and CPU baseline: no sweep / bf16 / encode / read-back / KV-split records")
    ap.add_argument("--dense-baseline", action="store_true",
                    help="also time bf16-KV decode attention on the same shapes: this library's plain kernel and, "
                         "when importable, flash_attn's flash_attn_with_kvcache (library code, reported as such)")
    ap.add_argument("--e2e-eager", action="store_true",
                    help="issue the end-to-end step's calls directly instead of replaying a captured CUDA graph")
    ap.add_argument("--serve", action="store_true",
                    help="encode-on-write plus decode at serving batch: 256 sequences prefill 1024 K/V tokens into "
                         "the packed cache, then 128 decode steps append one token each and run attention")
    ap.add_argument("--kv-split", action="store_true",
                    help="one 128K-token sequence whose KV range is split over the ranks (torchrun): per-rank "
                         "range decode, NCCL all-gather of the partials, log-sum-exp merge on every rank")
    ap.add_argument("--box", action="store_true",
                    help="whole-model decode: random-init Llama-3.1-8B (library GEMMs) with the packed attention "
                         "backend in every layer, 4500 requests x 1024-token contexts + 128 generated tokens")
    ap.add_argument("--box-batch", type=int, default=4500, help="requests over all GPUs (--box)")
    ap.add_argument("--box-wave", type=int, default=2250, help="most requests resident on one GPU at a time (--box)")
    ap.add_argument("--box-layers", type=int, default=32)
    ap.add_argument("--reference-kernel", action="store_true",
                    help="one attempt at the reference's own CuTe-DSL decode kernel (installed, unmodified, under "
                         "baseline/_ref) on this GPU at 128-token pages, next to this library's kernel on the same pages; "
                         "only its device-capability check is answered for it, since its launcher admits SM 10.3 alone")
    ap.add_argument("--sweep", action="store_true",
                    help="context sweep 1K..128K at 4M KV tokens on one GPU, with the bf16-KV baselines")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def ncu_traffic_bytes(workload: str):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, if any."""
    path = os.path.join(REPO, "profiles", "ncu_traffic.json")
    try:
        with open(path) as f:
            return json.load(f).get(workload)
    except Exception:
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only queries) on a
    background thread while the timed region runs."""

    REASONS = {
        "hw_slowdown": 0x8,
        "hw_thermal_slowdown": 0x40,
        "sw_thermal_slowdown": 0x20,
        "sw_power_cap": 0x4,
    }

    def __init__(self, index: int, period_s: float = 0.005):
        import threading

        self.samples, self.reason_bits, self.max_mhz, self.error = [], 0, None, None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
            handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))

            def loop():
                while not self._stop.is_set():
                    try:
                        self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                        self.reason_bits |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                    except Exception as exc:  # keep the benchmark alive if a query is unsupported
                        self.error = repr(exc)
                        return
                    time.sleep(period_s)

            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
        except Exception as exc:
            self.error = repr(exc)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        reasons = sorted(name for name, bit in self.REASONS.items() if self.reason_bits & bit)
        out = {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
               "reasons": reasons, "samples": len(self.samples)}
        if self.error:
            out["note"] = self.error
        return out


def cpu_decode_baseline(args, sample_requests: int, steps: int = 1, warmup: int = 0):
    """The path on the host cores: the reference's own code when it is staged under oracle/_ref
    (kind "reference"), else the numpy restatement (kind "port")."""
    from oracle import make_ref

    stat = "f16" if args.stat == "fp16" else "bf16"
    ref = None
    try:
        ref = make_ref.load_ref()
    except Exception as exc:  # a staged module that does not import here: say so, use the port
        print(f"bench: staged reference module failed to import ({exc!r}); timing the port", file=sys.stderr)
    if ref is not None:
        from oracle import ref_bench

        requests = sample_requests or 8
        secs, threads, nbytes = ref_bench.time_decode_sample(
            ref, requests=requests, ctx=args.ctx, heads_kv=HEADS_KV, heads_q=HEADS_Q, block_size=args.page, stat=stat,
            steps=steps, warmup=warmup)
        out = {
            "value": nbytes / secs / 1e9, "unit": "GB/s", "cores": threads, "kind": "reference",
            "sample": f"{requests} of the batch's requests x ctx {args.ctx}, one decode step each through the reference's "
                      f"own CPU path (read_request_from_paged_cache + float32 scaled_dot_product_attention per request), "
                      f"torch with {threads} threads",
            "seconds_per_step": secs, "same_config": False,
        }
        try:
            out["quantiser"] = ref_bench.quantiser_numbers(ref)
        except Exception as exc:
            out["quantiser"] = {"unavailable": repr(exc)}
        return out
    from beyond_kv_cache_b200 import synth
    from oracle.cpu_bench import time_decode_sample

    lk, tk = synth.make_tables(HEADS_KV, seed=0, which="k")
    lv, tv = synth.make_tables(HEADS_KV, seed=0, which="v")
    tabs = tuple(t.float().numpy() for t in (lk, tk, lv, tv))
    cores = os.cpu_count() or 1
    requests = sample_requests or cores
    secs, workers, nbytes = time_decode_sample(
        requests=requests, ctx=args.ctx, heads_kv=HEADS_KV, heads_q=HEADS_Q, block_size=args.page, tables=tabs,
        stat=stat, steps=steps, warmup=warmup, workers=cores)
    return {
        "value": nbytes / secs / 1e9,
        "unit": "GB/s",
        "cores": workers,
        "kind": "port",
        "sample": f"{requests} of the batch's requests x ctx {args.ctx}, one decode step each, numpy float64 "
                  f"attention over the packed pages, {workers} worker processes (oracle/_ref is not staged)",
        "seconds_per_step": secs, "same_config": False,
    }


def run_reference(args):
    """The reference arm: rank 0 alone runs and prints; a CPU number does not grow with the GPUs,
    so the line says n_gpus 1 whatever --gpus was."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 5))
    warm = 1 if args.warmup > 0 else 0
    base = cpu_decode_baseline(args, args.cpu_sample_requests, steps=steps, warmup=warm)
    line = {
        "impl": "reference",
        "metric": "packed_kv_decode_attention_throughput",
        "value": base["value"],
        "unit": "GB/s",
        "n_gpus": 1,
        "gpus_requested": args.gpus,
        "steps": steps,
        "warmup": warm,
        "ms_per_step": base["seconds_per_step"] * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32" if base["kind"] == "reference" else "f64",
        "data": "synthetic",
        "config": workload_config(args, note="bounded CPU sample: " + base["sample"]),
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample", "same_config")},
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if "quantiser" in base:
        line["cpu_baseline"]["quantiser"] = base["quantiser"]
    print(json.dumps(line), flush=True)


def workload_config(args, note: str | None = None):
    cfg = {
        "workload": f"llama-3.1-8b-shaped single-layer decode: batch {args.batch}/GPU x ctx {args.ctx}, "
                    f"{HEADS_Q} q / {HEADS_KV} kv heads, head_dim {HEAD_DIM}, {args.page}-token pages, random block table",
        "batch_per_gpu": args.batch,
        "context": args.ctx,
        "page_tokens": args.page,
        "stat_dtype": args.stat,
        "query_dtype": "bf16",
        "l2_policy": "inputs larger than L2 (packed cache >> 126 MB), no flush",
        "sharding": "request batch per GPU, no data-path collective",
    }
    if note:
        cfg["note"] = note
    return cfg


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    from beyond_kv_cache_b200 import _lib, synth
    from beyond_kv_cache_b200.quant.beyond_cute import PagedLayout, write_tokens_to_paged_cache
    from beyond_kv_cache_b200.quant.fa4_cute import beyond_mixed_decode_runtime as rt

    _lib.load()  # fail loudly when the CUDA library is missing
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path for the product")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    if args.reference_kernel:
        print(json.dumps(measure_reference_kernel(args, dev)), flush=True)
        return
    if args.kv_split:
        line = measure_kv_split(args, world, rank, local_rank, dev)
        if rank == 0:
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    if args.box:
        line = measure_box(args, world, rank, local_rank, dev)
        if rank == 0:
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    if args.serve:
        line = measure_serve(args, world, rank, local_rank, dev)
        if rank == 0:
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    if args.sweep:
        # context sweep at a constant 4M KV tokens (batch = 4M / context), one JSON line per point
        for batch, ctx in [(4096, 1024), (1024, 4096), (256, 16384), (128, 32768), (64, 65536), (32, 131072)]:
            line = measure(sweep_point(args, batch, ctx), world, rank, local_rank, dev, light=True)
            if rank == 0:
                print(json.dumps(line), flush=True)
            torch.cuda.empty_cache()
    else:
        line = measure(args, world, rank, local_rank, dev)
        torch.cuda.empty_cache()
        if not args.no_extras:
            if world > 1:
                record = guarded(lambda: kv_split_record(measure_kv_split(args, world, rank, local_rank, dev)))
                if rank == 0:
                    line["kv_split"] = record
            else:
                add_single_gpu_records(line, args, rank, local_rank, dev)
        if rank == 0:
            print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def guarded(fn):
    """A side record must never cost the headline: a failure becomes its own entry."""
    try:
        return fn()
    except Exception as exc:  # noqa: BLE001
        return {"failed": repr(exc)}


def sweep_point(args, batch, ctx):
    point = argparse.Namespace(**vars(args))
    point.batch, point.ctx = batch, ctx
    point.steps, point.no_cpu_baseline, point.dense_baseline = min(args.steps, 100), True, True
    return point


def kv_split_record(line):
    if line is None:
        return None
    keys = ("us_per_layer", "nccl_all_gather_form_us_per_layer", "value", "unit", "n_gpus", "scaling", "parity", "exchange", "config")
    return {k: line[k] for k in keys if k in line}


def add_single_gpu_records(line, args, rank, local_rank, dev):
    """The measurements next to the headline (one GPU): context sweep with the bf16-KV kernels,
    bf16-KV at the headline workload, encode / read-back / serving step."""
    import torch

    peak, _ = measured_peak()

    def bf16_ratio(rec):
        dense = rec.get("dense_kv_baseline") or {}
        lib = dense.get("library_flash_attn") or {}
        out = {"packed_us": rec["us_per_layer"], "own_bf16_kernel_us": dense.get("us_per_layer"),
               "flash_attn_bf16_us": lib.get("us_per_layer"), "flash_attn_page_tokens": lib.get("page_tokens")}
        if lib.get("us_per_layer"):
            out["speedup_vs_flash_attn_bf16"] = lib["us_per_layer"] / rec["us_per_layer"]
        elif "unavailable" in lib:
            out["flash_attn_unavailable"] = lib["unavailable"]
        if dense.get("us_per_layer"):
            out["speedup_vs_own_bf16_kernel"] = dense["us_per_layer"] / rec["us_per_layer"]
        return out

    def sweep():
        points = []
        for batch, ctx in [(4096, 1024), (128, 32768), (32, 131072)]:
            rec = measure(sweep_point(args, batch, ctx), 1, rank, local_rank, dev, light=True)
            torch.cuda.empty_cache()
            points.append({"context": ctx, "batch": batch, "us": rec["us_per_layer"], "frac": rec["roofline"]["frac"],
                           "GBps": rec["roofline"]["achieved"], "vs_bf16_kv": bf16_ratio(rec)})
        return points

    def headline_bf16():
        point = argparse.Namespace(**vars(args))
        point.steps, point.no_cpu_baseline, point.dense_baseline = min(args.steps, 100), True, True
        rec = measure(point, 1, rank, local_rank, dev, light=True)
        torch.cuda.empty_cache()
        return bf16_ratio(rec)

    def serve():
        rec = measure_serve(args, 1, rank, local_rank, dev)
        torch.cuda.empty_cache()
        return rec

    line["vs_bf16_kv"] = guarded(headline_bf16)
    line["sweep"] = guarded(sweep)
    served = guarded(serve)
    if "failed" in served:
        line["encode"] = line["readback"] = line["serving_step"] = served
    else:
        enc, rb = served["prefill_encode"], served["readback"]
        line["encode"] = {"ms": enc["ms"], "frac": enc["frac_of_peak"], "GBps": enc["GBps"], "rows": enc["tokens"],
                          "bytes_per_token_head": 672, "ms_in_chunks_of_8192_tokens": enc["ms_in_chunks_of_8192_tokens"],
                          "frac_in_chunks": enc["frac_of_peak"] * enc["ms"] / enc["ms_in_chunks_of_8192_tokens"],
                          "with_reconstruction": served["prefill_encode_reconstruct"]}
        line["readback"] = {"ms": rb["ms"], "frac": rb["frac_of_peak"], "GBps": rb["GBps"], "rows": enc["tokens"],
                            "bytes_per_token_head": 672}
        line["serving_step"] = dict(served["decode_steps"], workload=served["config"]["workload"],
                                    tokens_per_s_one_layer=served["value"])


def measure_kv_split(args, world, rank, local_rank, dev, ctx: int = 131072):
    """One sequence of `ctx` tokens; rank r holds and attends only its page-aligned share of the
    KV range (strong scaling); the un-normalised partials (32 heads x 130 floats per rank) are
    pushed into every peer's receive buffer and merged on every rank (the NCCL all-gather form
    is timed next to it)."""
    import torch
    import torch.distributed as dist

    from beyond_kv_cache_b200 import parallel, synth
    from beyond_kv_cache_b200.quant.beyond_cute import PagedLayout, write_tokens_to_paged_cache

    BS = args.page
    stat_dtype = torch.float16 if args.stat == "fp16" else torch.bfloat16
    layout = PagedLayout.build_hnd(BS, HEADS_KV, HEAD_DIM, 4, 32, 32)
    lo, hi = parallel.kv_range_for_rank(ctx, BS, world, rank)
    pages_total = (ctx + BS - 1) // BS
    # the block table names every page of the sequence; only this rank's range is filled
    block_table, num_pages = synth.random_block_table(1, pages_total, seed=3, device=dev)
    cache = torch.zeros((num_pages, layout.block_i32), dtype=torch.int32, device=dev)
    lk, tk = (t.to(dev) for t in synth.make_tables(HEADS_KV, seed=0, which="k"))
    lv, tv = (t.to(dev) for t in synth.make_tables(HEADS_KV, seed=0, which="v"))
    if hi > lo:
        k, v = synth.make_kv(hi - lo, HEADS_KV, seed=11 + rank, device=dev)
        write_tokens_to_paged_cache(cache, layout, block_table, synth.slots_for(block_table, BS, lo, hi - lo), k, v,
                                    q_points_k=lk, q_points_v=lv, thresholds_k=tk, thresholds_v=tv,
                                    require_fast=True, stat_dtype=stat_dtype)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)  # the same query on every rank
    q = torch.randn((1, HEADS_Q, HEAD_DIM), generator=gen, device=dev).to(torch.bfloat16)
    seq_lens = torch.full((1,), ctx, dtype=torch.int32, device=dev)
    out = torch.empty((1, HEADS_Q, HEAD_DIM), dtype=torch.bfloat16, device=dev)
    scale = synth.softmax_scale()

    out32 = torch.empty((1, HEADS_Q, HEAD_DIM), dtype=torch.float32, device=dev)
    exchange = parallel.KvRangeExchange(rows=HEADS_Q, device=dev)

    def timed(ex):
        def step():
            parallel.decode_kv_range_split(q, cache, layout, block_table, seq_lens, lk, lv, out, token_lo=lo, token_hi=hi,
                                           softmax_scale=scale, stat_dtype=stat_dtype, exchange=ex, out_f32=out32)

        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        steps = min(max(args.steps, 200), 500)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def timed_graph(ex, reps=20):
        """The same step replayed from a captured graph (what a serving engine does): device time
        without the host's launch work between the steps."""
        def step():
            parallel.decode_kv_range_split(q, cache, layout, block_table, seq_lens, lk, lv, out, token_lo=lo, token_hi=hi,
                                           softmax_scale=scale, stat_dtype=stat_dtype, exchange=ex, out_f32=out32)

        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.graph(graph, stream=side):
            for _ in range(reps):
                step()
        torch.cuda.current_stream(dev).wait_stream(side)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        g_ms = e0.elapsed_time(e1) / (10 * reps)
        if world > 1:
            t = torch.tensor([g_ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            g_ms = float(t.item())
        return g_ms

    try:
        eager_ms = timed(exchange)
        exchange.check()
        ms = timed_graph(exchange)
        exchange.check()
        pushed_out = out32.clone()
        nccl_ms = timed(None) if world > 1 else None
    finally:
        exchange.close()

    # ---- parity: every rank evaluates the oracle's partial over its own range; rank 0 merges them ----
    import numpy as np

    import oracle

    kind = "f16" if args.stat == "fp16" else "bf16"
    geo = oracle.PageGeometry(BS, HEADS_KV)
    part = torch.zeros((HEADS_Q, HEAD_DIM + 2), dtype=torch.float64, device=dev)
    part[:, HEAD_DIM] = float("-inf")
    if hi > lo:
        ids = block_table[0, lo // BS : (hi + BS - 1) // BS].long()
        local = cache[ids].cpu().numpy()  # this rank's pages, renumbered from 0
        o, m, l = oracle.decode_attention(q.float().cpu().numpy(), local, geo, np.arange(len(ids), dtype=np.int32)[None, :],
                                          [hi - lo], levels_k=lk.float().cpu().numpy(), levels_v=lv.float().cpu().numpy(),
                                          softmax_scale=scale, stat=kind, return_partials=True)
        part[:, :HEAD_DIM] = torch.from_numpy(o[0]).to(dev)
        part[:, HEAD_DIM] = torch.from_numpy(m[0]).to(dev)
        part[:, HEAD_DIM + 1] = torch.from_numpy(l[0]).to(dev)
    parts = [torch.empty_like(part) for _ in range(world)] if world > 1 else [part]
    if world > 1:
        dist.all_gather(parts, part)
    if rank != 0:
        return None
    stacked = torch.stack(parts).cpu().numpy()
    want = oracle.merge_partials(stacked[:, None, :, :HEAD_DIM], stacked[:, None, :, HEAD_DIM], stacked[:, None, :, HEAD_DIM + 1])
    max_abs = float(np.abs(pushed_out.cpu().numpy() - want).max())
    nbytes = ctx * HEADS_KV * BYTES_PER_TOKEN_HEAD
    line = {
        "metric": "kv_range_split_decode_attention",
        "value": nbytes / (ms * 1e-3) / 1e9,
        "unit": "GB/s",
        "n_gpus": world,
        "us_per_layer": ms * 1e3,
        "timing": "20 steps per captured graph, 10 replays; eager launches: %.1f us per step" % (eager_ms * 1e3),
        "scaling": "strong",
        "exchange": "pushed: peer stores into IPC-mapped receive buffers + flags, one kernel pushes / waits (bounded) / merges",
        "parity": {"max_abs": max_abs, "requests": 1, "oracle": "float64 partials per rank over its range, merged by log-sum-exp"},
        "config": {"workload": f"one sequence x ctx {ctx}, {HEADS_Q} q / {HEADS_KV} kv heads, {BS}-token pages, "
                               f"KV range split over {world} GPU(s)"},
        "data": "synthetic",
    }
    if nccl_ms is not None:
        line["nccl_all_gather_form_us_per_layer"] = nccl_ms * 1e3
    return line


def measure_reference_kernel(args, dev, page: int = 128):
    """The reference's CuTe-DSL kernel (``quant/fa4_cute`` of the reference, installed unmodified under
    ``baseline/_ref``) and this library's kernel over the SAME packed pages of `page` tokens: both
    outputs against each other, both timed.  The reference launcher refuses every device but SM 10.3
    (``beyond_mixed_decode_runtime.py:152-153``); its question about the device capability is answered
    with (10, 3) for the duration of its calls, nothing else of it is touched.  Whatever the DSL, its
    compiler or the launch report is returned as text; nothing is retried."""
    import contextlib

    import torch

    from beyond_kv_cache_b200 import synth
    from beyond_kv_cache_b200.quant.beyond_cute import PagedLayout, write_tokens_to_paged_cache
    from beyond_kv_cache_b200.quant.fa4_cute import beyond_mixed_decode_runtime as rt

    B, ctx = args.batch, args.ctx
    record = {"metric": "reference_cute_kernel_same_box", "config": {"workload": f"batch {B} x ctx {ctx}, {HEADS_Q} q / "
              f"{HEADS_KV} kv heads, {page}-token pages, bf16 queries and statistics"}, "device": torch.cuda.get_device_name(dev),
              "capability": list(torch.cuda.get_device_capability(dev))}
    layout = PagedLayout.build_hnd(page, HEADS_KV, HEAD_DIM, 4, 32, 32)
    pages_per_seq = (ctx + page - 1) // page
    block_table, num_pages = synth.random_block_table(B, pages_per_seq, seed=0, device=dev)
    cache = torch.zeros((num_pages, layout.block_i32), dtype=torch.int32, device=dev)
    lk, tk = (t.to(dev) for t in synth.make_tables(HEADS_KV, seed=0, which="k"))
    lv, tv = (t.to(dev) for t in synth.make_tables(HEADS_KV, seed=0, which="v"))
    chunk = 2048
    for start in range(0, ctx, chunk):
        n = min(chunk, ctx - start)
        k, v = synth.make_kv(B * n, HEADS_KV, seed=start, device=dev)
        write_tokens_to_paged_cache(cache, layout, block_table, synth.slots_for(block_table, page, start, n), k, v,
                                    q_points_k=lk, q_points_v=lv, thresholds_k=tk, thresholds_v=tv, require_fast=True)
    q = torch.randn((B, HEADS_Q, HEAD_DIM), device=dev).to(torch.bfloat16)
    seq_lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    scale = synth.softmax_scale()
    max_seq_len = pages_per_seq * page

    def timed(step, reps):
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            step()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3

    # ---- this library on the same pages ----
    rk, rv = rt.prepare_runtime_qpoints(lk, lv, heads_kv=HEADS_KV)
    spec = rt.make_runtime_spec(q=q, cache=cache, layout=layout, block_table=block_table, heads_q=HEADS_Q, max_seq_len=max_seq_len)
    ws = rt.allocate_runtime_workspace(spec, device=dev)
    ours = torch.empty_like(q)

    def our_step():
        rt.run_nonuniform_decode(spec=spec, q=q, cache=cache, layout=layout, block_table=block_table, seq_lens=seq_lens,
                                 k_qpoints_lane_major=rk, v_qpoints_code_major=rv, out=ours, workspace=ws, softmax_scale=scale)

    record["this_library_us"] = timed(our_step, min(args.steps, 200))

    # ---- the reference kernel ----
    ref_root = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "quant", "fa4_cute")):
        record["reference"] = {"unavailable": "baseline/_ref holds no installed reference (pip install --target baseline/_ref <checkout>/quant)"}
        return record
    sys.path.insert(0, ref_root)

    @contextlib.contextmanager
    def answering_sm103():
        real = torch.cuda.get_device_capability
        torch.cuda.get_device_capability = lambda device=None: (10, 3)
        try:
            yield
        finally:
            torch.cuda.get_device_capability = real

    try:
        import quant.beyond_cute as ref_ops
        import quant.fa4_cute.beyond_mixed_decode_runtime as ref_rt

        ref_layout = ref_ops.PagedLayout.build_hnd(page, HEADS_KV, HEAD_DIM, 4, 32, 32)
        theirs = torch.empty_like(q)
        with answering_sm103():
            ref_k, ref_v = ref_rt.prepare_runtime_qpoints(lk, lv, heads_kv=HEADS_KV, storage_dtype=torch.float16)
            ref_spec = ref_rt.make_runtime_spec(q=q, cache=cache, layout=ref_layout, block_table=block_table, heads_q=HEADS_Q,
                                                max_seq_len=max_seq_len, num_splits=0, qpoint_dtype=torch.float16)
            ref_ws = ref_rt.allocate_runtime_workspace(ref_spec, device=dev)

            def ref_step():
                ref_rt.run_nonuniform_decode(spec=ref_spec, q=q, cache=cache, layout=ref_layout, block_table=block_table,
                                             seq_lens=seq_lens, k_qpoints_lane_major=ref_k, v_qpoints_code_major=ref_v,
                                             out=theirs, workspace=ref_ws, softmax_scale=scale)

            t0 = time.perf_counter()
            ref_step()  # compiles on first use
            torch.cuda.synchronize()
            record["reference"] = {"first_call_s": time.perf_counter() - t0, "num_splits": ref_spec.num_splits}
            our_step()
            torch.cuda.synchronize()
            record["reference"]["max_abs_vs_this_library"] = float((theirs.float() - ours.float()).abs().max().item())
            # both against the float64 oracle over the same pages, rounded to the output type (request 0)
            import numpy as np

            import oracle

            ids = block_table[0, :pages_per_seq].long()
            want = oracle.decode_attention(q[0:1].float().cpu().numpy(), cache[ids].cpu().numpy(), oracle.PageGeometry(page, HEADS_KV),
                                           np.arange(pages_per_seq, dtype=np.int32)[None, :], [ctx], levels_k=lk.float().cpu().numpy(),
                                           levels_v=lv.float().cpu().numpy(), softmax_scale=scale, stat="bf16")
            want16 = torch.from_numpy(want).to(q.dtype).float().numpy()
            record["reference"]["bf16_output_max_abs_vs_rounded_oracle"] = float(np.abs(theirs[0:1].float().cpu().numpy() - want16).max())
            record["this_library_bf16_output_max_abs_vs_rounded_oracle"] = float(np.abs(ours[0:1].float().cpu().numpy() - want16).max())
            record["oracle_max_abs_value"] = float(np.abs(want16).max())
            record["reference"]["us"] = timed(ref_step, min(args.steps, 200))
    except BaseException as exc:  # noqa: BLE001  (DSL / compiler / launch refusals are the record)
        import traceback

        record["reference"] = {"failed": f"{type(exc).__name__}: {exc}"[:2000], "traceback_tail": traceback.format_exc()[-1500:]}
    return record


def measure_box(args, world, rank, local_rank, dev, prompt: int = 1024, gen_steps: int = 128):
    """Whole-model decode throughput.  A random-init Llama-3.1-8B-shaped decoder (hidden 4096,
    32 / 8 heads, FFN 14336, vocabulary 128256, bf16 weights N(0, 0.02)) whose GEMMs, norms and
    activation are plain torch library calls and whose attention is `BeyondPackedImpl.forward`
    (encode-on-write + packed decode) with per-layer, per-head tables.  The `--box-batch`
    requests are dealt to the ranks (weights replicated, no collective); a rank that cannot hold
    its share at once runs it in waves.  The packed caches of the 1024-token contexts are filled
    by the encode kernel from synthetic K/V rows (a prefill of a random-init model yields
    equally arbitrary rows); the timed region is the `gen_steps` decode steps, each one CUDA
    graph replay of the full model step including sampling (arg-max) and slot derivation."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    from beyond_kv_cache_b200 import _lib, synth
    from beyond_kv_cache_b200.quant.beyond_cute import PagedLayout, write_tokens_to_paged_cache
    from beyond_kv_cache_b200.runtime.vllm.packed_backend import BeyondPackedImpl, BeyondPackedMetadata

    LAYERS, HID, FFN, VOCAB, BS = args.box_layers, 4096, 14336, 128256, args.page
    mine = len(range(rank, args.box_batch, world))
    waves = max(1, -(-mine // args.box_wave))
    batch = -(-mine // waves)  # requests resident per wave (the last wave is padded to the same shape)
    layout = PagedLayout.build_hnd(BS, HEADS_KV, HEAD_DIM, 4, 32, 32)
    pages_per_seq = -(-(prompt + gen_steps) // BS)
    block_table, num_pages = synth.random_block_table(batch, pages_per_seq, seed=rank, device=dev)

    def weight(*shape):
        return torch.empty(shape, dtype=torch.bfloat16, device=dev).normal_(0.0, 0.02)

    torch.manual_seed(1234)  # the same replica on every rank
    embed, lm_head, final_norm = weight(VOCAB, HID), weight(HID, VOCAB), torch.ones(HID, dtype=torch.bfloat16, device=dev)
    layers = []
    for li in range(LAYERS):
        impl = BeyondPackedImpl(HEADS_Q, HEAD_DIM, synth.softmax_scale(), HEADS_KV)
        lk, tk = (t.to(dev) for t in synth.make_tables(HEADS_KV, seed=li, which="k"))
        lv, tv = (t.to(dev) for t in synth.make_tables(HEADS_KV, seed=li, which="v"))
        impl.set_quant_tables(lk, tk, lv, tv)
        layers.append({
            "impl": impl, "tables": (lk, tk, lv, tv),
            "wqkv": weight(HID, (HEADS_Q + 2 * HEADS_KV) * HEAD_DIM), "wo": weight(HEADS_Q * HEAD_DIM, HID),
            "wgu": weight(HID, 2 * FFN), "wdown": weight(FFN, HID),
            "n1": torch.ones(HID, dtype=torch.bfloat16, device=dev), "n2": torch.ones(HID, dtype=torch.bfloat16, device=dev),
            "cache": torch.zeros((num_pages, layout.block_i32), dtype=torch.int32, device=dev),
        })
    inv_freq = 1.0 / (500000.0 ** (torch.arange(0, HEAD_DIM, 2, device=dev, dtype=torch.float32) / HEAD_DIM))
    angles = torch.arange(pages_per_seq * BS, device=dev, dtype=torch.float32)[:, None] * inv_freq[None, :]
    rope_cos, rope_sin = angles.cos(), angles.sin()

    def fill_caches(seed):
        # contexts of `prompt` tokens: one synthetic block of rows, written request block by request block
        rows = 64
        k, v = synth.make_kv(rows * prompt, HEADS_KV, seed=seed, device=dev)
        for layer in layers:
            lk, tk, lv, tv = layer["tables"]
            for r0 in range(0, batch, rows):
                n = min(rows, batch - r0)
                slots = synth.slots_for(block_table[r0:r0 + n], BS, 0, prompt)
                write_tokens_to_paged_cache(layer["cache"], layout, block_table, slots, k[: n * prompt], v[: n * prompt],
                                            q_points_k=lk, q_points_v=lv, thresholds_k=tk, thresholds_v=tv,
                                            require_fast=True)

    seq_lens = torch.full((batch,), prompt, dtype=torch.int32, device=dev)
    slots = torch.zeros((batch,), dtype=torch.int32, device=dev)
    tokens = torch.zeros((batch,), dtype=torch.int64, device=dev)
    attn_out = torch.empty((batch, HEADS_Q, HEAD_DIM), dtype=torch.bfloat16, device=dev)
    meta = BeyondPackedMetadata(
        num_actual_tokens=batch, query_start_loc=torch.arange(batch + 1, dtype=torch.int32, device=dev), seq_lens=seq_lens,
        block_table=block_table, slot_mapping=slots, max_query_len=1, max_seq_len=pages_per_seq * BS,
        _beyond_query_start_loc_list=list(range(batch + 1)), _beyond_seq_lens_list=[pages_per_seq * BS] * batch)
    stream = lambda: torch.cuda.current_stream(dev).cuda_stream  # noqa: E731
    QW, KW = HEADS_Q * HEAD_DIM, HEADS_KV * HEAD_DIM

    def rope(x, cos, sin):
        x1, x2 = x[..., : HEAD_DIM // 2].float(), x[..., HEAD_DIM // 2:].float()
        return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(torch.bfloat16)

    def attention(layer, q, k, v):
        return layer["impl"].forward(None, q, k, v, layer["cache"], meta, output=attn_out)

    def model_step():
        seq_lens.add_(1)  # the token being generated joins its context
        _lib.call("bkv_derive_slots_sm100", seq_lens.data_ptr(), block_table.data_ptr(), block_table.stride(0),
                  block_table.shape[1], BS, batch, slots.data_ptr(), stream())
        pos = (seq_lens - 1).long()
        cos, sin = rope_cos[pos][:, None, :], rope_sin[pos][:, None, :]
        x = embed[tokens]
        for layer in layers:
            qkv = F.rms_norm(x, (HID,), layer["n1"], 1e-5) @ layer["wqkv"]
            q = rope(qkv[:, :QW].view(batch, HEADS_Q, HEAD_DIM), cos, sin)
            k = rope(qkv[:, QW:QW + KW].view(batch, HEADS_KV, HEAD_DIM), cos, sin)
            v = qkv[:, QW + KW:].view(batch, HEADS_KV, HEAD_DIM)
            x = x + attention(layer, q, k, v).view(batch, QW) @ layer["wo"]
            gu = F.rms_norm(x, (HID,), layer["n2"], 1e-5) @ layer["wgu"]
            x = x + (F.silu(gu[:, :FFN]) * gu[:, FFN:]) @ layer["wdown"]
        logits = F.rms_norm(x, (HID,), final_norm, 1e-5) @ lm_head
        tokens.copy_(logits.argmax(dim=-1))

    q_fixed = torch.randn((batch, HEADS_Q, HEAD_DIM), device=dev).to(torch.bfloat16)
    k_fixed, v_fixed = synth.make_kv(batch, HEADS_KV, seed=5, device=dev)

    def attention_only_step():  # the 32 attention calls of one step on their own (share of the step)
        for layer in layers:
            attention(layer, q_fixed, k_fixed, v_fixed)

    def reset(seed):
        seq_lens.fill_(prompt)
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)
        tokens.copy_(torch.randint(0, VOCAB, (batch,), generator=gen, device=dev))

    fill_caches(100 + rank)
    reset(rank)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):  # eager passes: workspaces and library handles exist before capture
        model_step()
        attention_only_step()
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize(dev)
    graph, attn_graph = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        model_step()
    with torch.cuda.graph(attn_graph):
        attention_only_step()

    def timed(g, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            g.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1)

    total_ms, attn_ms = 0.0, 0.0
    sampler = None
    for wave in range(waves):
        if wave:
            fill_caches(100 + rank + 1000 * wave)
        reset(rank + 1000 * wave)
        for _ in range(max(3, min(args.warmup, 5))):
            graph.replay()
        reset(rank + 1000 * wave)
        seq_lens.fill_(prompt + gen_steps // 2)  # attention alone at the mid-generation context length
        attn_ms += timed(attn_graph, 5) / 5
        reset(rank + 1000 * wave)
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        if rank == 0 and sampler is None:
            sampler = ClockSampler(local_rank, period_s=0.02)
        total_ms += timed(graph, gen_steps)
    clocks = sampler.stop() if sampler is not None else None
    finite = bool(torch.isfinite(attn_out.float()).all().item()) and int(seq_lens.max().item()) == prompt + gen_steps
    if world > 1:
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    if rank != 0:
        return None
    if not finite:
        raise SystemExit("box decode: non-finite attention output or wrong final context length")
    generated = args.box_batch * gen_steps
    step_ms = total_ms / (waves * gen_steps)
    return {
        "metric": "decode_tokens_per_s_box",
        "value": generated / (total_ms * 1e-3),
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": gen_steps,
        "ms_per_step": step_ms,
        "attention_ms_per_step": attn_ms / waves,
        "attention_share": (attn_ms / waves) / step_ms,
        "higher_is_better": True,
        "scaling": "strong",
        "dtype": "bf16 weights and activations; 4-bit codes + 16-bit group statistics in the KV cache",
        "data": "synthetic (random-init weights, uniform token ids, encode-filled contexts)",
        "config": {"workload": f"random-init Llama-3.1-8B shape, {LAYERS} layers, {args.box_batch} requests x {prompt}-token "
                               f"contexts + {gen_steps} generated tokens over {world} GPU(s): {batch} resident per GPU x "
                               f"{waves} wave(s); {BS}-token pages; GEMMs / norms / activation are torch library calls, "
                               f"attention is the packed backend"},
        "clocks": clocks,
    }


def measure_serve(args, world, rank, local_rank, dev, seqs: int = 256, prompt: int = 1024, gen_steps: int = 128):
    """Encode-on-write + decode at serving batch (one layer): prefill `seqs` x `prompt` bf16
    K/V tokens through the encode kernel, then `gen_steps` decode steps, each appending one
    token per sequence (encode) and attending the whole packed context (decode)."""
    import torch
    import torch.distributed as dist

    from beyond_kv_cache_b200 import synth
    from beyond_kv_cache_b200.quant.beyond_cute import PagedLayout, write_tokens_to_paged_cache
    from beyond_kv_cache_b200.quant.fa4_cute import beyond_mixed_decode_runtime as rt

    BS = args.page
    stat_dtype = torch.float16 if args.stat == "fp16" else torch.bfloat16
    layout = PagedLayout.build_hnd(BS, HEADS_KV, HEAD_DIM, 4, 32, 32)
    pages_per_seq = (prompt + gen_steps + BS - 1) // BS
    block_table, num_pages = synth.random_block_table(seqs, pages_per_seq, seed=rank, device=dev)
    cache = torch.zeros((num_pages, layout.block_i32), dtype=torch.int32, device=dev)
    lk, tk = (t.to(dev) for t in synth.make_tables(HEADS_KV, seed=0, which="k"))
    lv, tv = (t.to(dev) for t in synth.make_tables(HEADS_KV, seed=0, which="v"))
    rk, rv = rt.prepare_runtime_qpoints(lk, lv, heads_kv=HEADS_KV)
    k, v = synth.make_kv(seqs * prompt, HEADS_KV, seed=7 + rank, device=dev)
    slots = synth.slots_for(block_table, BS, 0, prompt)

    def encode(kk, vv, ss, signal=False, dependent=False):
        write_tokens_to_paged_cache(cache, layout, block_table, ss, kk, vv, q_points_k=lk, q_points_v=lv,
                                    thresholds_k=tk, thresholds_v=tv, require_fast=True, stat_dtype=stat_dtype,
                                    signal_pdl_dependents=signal, wait_for_pdl_predecessor=dependent)

    def timed(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    prefill_ms = timed(lambda: encode(k, v, slots), 20)
    prefill_bytes = seqs * prompt * HEADS_KV * (512 + 160)  # bf16 K and V rows in, packed row out

    # the same rows in scheduler-sized chunks of 8192 tokens (32 launches)
    chunk = 8192
    # (every chunk lets the next one begin its set-up while it drains and is itself launched as a
    # programmatic dependent: what a writer does behind the kernel that produces its rows; the plain
    # launches are timed next to it)
    def chunked(chained):
        def encode_chunks():
            for c0 in range(0, seqs * prompt, chunk):
                encode(k[c0:c0 + chunk], v[c0:c0 + chunk], slots[c0:c0 + chunk], signal=chained, dependent=chained and c0 > 0)
        graph = torch.cuda.CUDAGraph()
        cside = torch.cuda.Stream(device=dev)
        cside.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.graph(graph, stream=cside):
            encode_chunks()
        torch.cuda.current_stream(dev).wait_stream(cside)
        return timed(graph.replay, 20)
    chunked_ms = chunked(True)
    chunked_plain_ms = chunked(False)

    # the prefill writer: encode + reconstruction of K/V in place (attention then sees what the cache holds)
    k_rec, v_rec = k.clone(), v.clone()
    recon_ms = timed(lambda: write_tokens_to_paged_cache(
        cache, layout, block_table, slots, k_rec, v_rec, q_points_k=lk, q_points_v=lv, thresholds_k=tk, thresholds_v=tv,
        k_dq_out=k_rec, v_dq_out=v_rec, require_fast=True, stat_dtype=stat_dtype), 20)
    del k_rec, v_rec
    encode(k, v, slots)  # the cache holds the original rows again
    recon_bytes = seqs * prompt * HEADS_KV * (512 + 160 + 512)

    # read-back of the same contexts to dense bf16 K/V (what chunked prefill attends over)
    from beyond_kv_cache_b200.quant.beyond_cute import dequantize_paged_kv_to_dense
    dense_k, dense_v = torch.empty_like(k), torch.empty_like(v)
    prompt_lens = torch.full((seqs,), prompt, dtype=torch.int32, device=dev)
    starts = torch.arange(0, (seqs + 1) * prompt, prompt, dtype=torch.int32, device=dev)
    readback_ms = timed(lambda: dequantize_paged_kv_to_dense(cache, layout, block_table, prompt_lens, starts, dense_k,
                                                             dense_v, max_seq_len=prompt, q_points_k=lk, q_points_v=lv,
                                                             stat_dtype=stat_dtype), 20)
    del dense_k, dense_v

    q = torch.randn((seqs, HEADS_Q, HEAD_DIM), device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    k1, v1 = synth.make_kv(seqs, HEADS_KV, seed=99 + rank, device=dev)
    spec = rt.make_runtime_spec(q=q, cache=cache, layout=layout, block_table=block_table, heads_q=HEADS_Q,
                                max_seq_len=pages_per_seq * BS, num_splits=args.splits, wait_for_pdl_writer=True)
    ws = rt.allocate_runtime_workspace(spec, device=dev)
    lens = [torch.full((seqs,), prompt + i + 1, dtype=torch.int32, device=dev) for i in range(gen_steps)]
    step_slots = [synth.slots_for(block_table, BS, prompt + i, 1) for i in range(gen_steps)]
    scale = synth.softmax_scale()

    def generate():
        for i in range(gen_steps):
            encode(k1, v1, step_slots[i], signal=True)  # the decode grid starts its set-up behind it
            rt.run_nonuniform_decode(spec=spec, q=q, cache=cache, layout=layout, block_table=block_table,
                                     seq_lens=lens[i], k_qpoints_lane_major=rk, v_qpoints_code_major=rv, out=out,
                                     workspace=ws, softmax_scale=scale, stat_dtype=stat_dtype, loader=args.loader if spec.persistent else 0)

    gen_ms = timed(generate, 5)
    # the writer alone, one token per sequence: 50 launches per CUDA-graph replay so that the host's
    # launch rate does not bound the figure
    append_graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.graph(append_graph, stream=side):
        for _ in range(50):
            encode(k1, v1, step_slots[0])
    torch.cuda.current_stream(dev).wait_stream(side)
    append_ms = timed(append_graph.replay, 10) / 50
    if rank != 0:
        return None
    peak, peak_kind = measured_peak()
    attended = sum((prompt + i + 1) for i in range(gen_steps)) * seqs * HEADS_KV * BYTES_PER_TOKEN_HEAD
    return {
        "metric": "serve_encode_decode_one_layer",
        "value": world * seqs * gen_steps / (gen_ms * 1e-3),
        "unit": "decode tokens/s (one layer)",
        "n_gpus": world,
        "config": {"workload": f"{seqs} sequences/GPU x {prompt}-token prefill + {gen_steps} decode steps, "
                               f"{HEADS_Q} q / {HEADS_KV} kv heads, {BS}-token pages"},
        "prefill_encode": {"ms": prefill_ms, "tokens": seqs * prompt,
                           "GBps": prefill_bytes / (prefill_ms * 1e-3) / 1e9,
                           "frac_of_peak": prefill_bytes / (prefill_ms * 1e-3) / 1e9 / peak,
                           "bytes_per_token_head": 672, "peak_source": peak_kind,
                           "ms_in_chunks_of_8192_tokens": chunked_ms,
                           "ms_in_chunks_of_8192_tokens_plain_launches": chunked_plain_ms,
                           "chunks": "32 launches in one captured graph; each chunk is launched as a programmatic "
                                     "dependent of the one in front (set-up overlaps its drain) unless 'plain'"},
        "prefill_encode_reconstruct": {"ms": recon_ms, "GBps": recon_bytes / (recon_ms * 1e-3) / 1e9,
                                       "frac_of_peak": recon_bytes / (recon_ms * 1e-3) / 1e9 / peak,
                                       "bytes_per_token_head": 1184},
        "readback": {"ms": readback_ms, "GBps": prefill_bytes / (readback_ms * 1e-3) / 1e9,
                     "frac_of_peak": prefill_bytes / (readback_ms * 1e-3) / 1e9 / peak,
                     "bytes_per_token_head": 672},
        "decode_steps": {"ms_per_step": gen_ms / gen_steps, "steps": gen_steps, "append_encode_ms": append_ms,
                         "attended_GBps": attended / (gen_ms * 1e-3) / 1e9},
        "data": "synthetic",
    }


def measure(args, world, rank, local_rank, dev, light: bool = False):
    """Build the packed cache for one (batch, context) point, time the decode step and (unless
    `light`) the end-to-end serving step, check a sample of the output against the oracle and time
    the CPU baseline; returns the JSON line (rank 0) or None."""
    import torch
    import torch.distributed as dist

    from beyond_kv_cache_b200 import _lib, synth
    from beyond_kv_cache_b200.quant.beyond_cute import PagedLayout, write_tokens_to_paged_cache
    from beyond_kv_cache_b200.quant.fa4_cute import beyond_mixed_decode_runtime as rt

    B, ctx, BS = args.batch, args.ctx, args.page
    stat_dtype = torch.float16 if args.stat == "fp16" else torch.bfloat16
    layout = PagedLayout.build_hnd(BS, HEADS_KV, HEAD_DIM, 4, 32, 32)
    pages_per_seq = (ctx + BS - 1) // BS + 1  # room for the appended tokens of the e2e steps
    block_table, num_pages = synth.random_block_table(B, pages_per_seq, seed=rank, device=dev)
    cache = torch.zeros((num_pages, layout.block_i32), dtype=torch.int32, device=dev)
    lk, tk = (t.to(dev) for t in synth.make_tables(HEADS_KV, seed=0, which="k"))
    lv, tv = (t.to(dev) for t in synth.make_tables(HEADS_KV, seed=0, which="v"))

    # ---- fill the cache with real codes through the encode-on-write kernel (untimed) ----
    chunk = 2048
    for start in range(0, ctx, chunk):
        n = min(chunk, ctx - start)
        k, v = synth.make_kv(B * n, HEADS_KV, seed=1000 * rank + start, device=dev)
        slots = synth.slots_for(block_table, BS, start, n)
        write_tokens_to_paged_cache(cache, layout, block_table, slots, k, v, q_points_k=lk, q_points_v=lv,
                                    thresholds_k=tk, thresholds_v=tv, require_fast=True, stat_dtype=stat_dtype)
    del k, v
    gen = torch.Generator(device=dev)
    gen.manual_seed(77 + rank)
    q = torch.randn((B, HEADS_Q, HEAD_DIM), generator=gen, device=dev).to(torch.bfloat16)
    seq_lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    out = torch.empty_like(q)
    max_seq_len = pages_per_seq * BS
    rk, rv = rt.prepare_runtime_qpoints(lk, lv, heads_kv=HEADS_KV)
    spec = rt.make_runtime_spec(q=q, cache=cache, layout=layout, block_table=block_table, heads_q=HEADS_Q,
                                max_seq_len=max_seq_len, num_splits=args.splits)
    # the serving step runs the decode grid as a programmatic dependent of the cache writer
    spec_pdl = rt.make_runtime_spec(q=q, cache=cache, layout=layout, block_table=block_table, heads_q=HEADS_Q,
                                    max_seq_len=max_seq_len, num_splits=args.splits, wait_for_pdl_writer=True)
    ws = rt.allocate_runtime_workspace(spec, device=dev)
    scale = synth.softmax_scale()
    streamed = spec.persistent

    def decode_step(out_f32=None):
        rt.run_nonuniform_decode(spec=spec, q=q, cache=cache, layout=layout, block_table=block_table,
                                 seq_lens=seq_lens, k_qpoints_lane_major=rk, v_qpoints_code_major=rv, out=out,
                                 workspace=ws, softmax_scale=scale, stat_dtype=stat_dtype, out_f32=out_f32,
                                 loader=args.loader if spec.persistent else 0)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(args.warmup, 3)):
        decode_step()
    sync_all()
    # Exactly args.steps steps per timed region; the region is repeated until at least 200 steps have
    # run (a region of a few milliseconds is too short for the clock sampler) and the median counts.
    regions = 1 if light else max(1, -(-200 // max(1, args.steps)))
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    region_ms = []
    for _ in range(regions):
        ev0.record()
        for _ in range(args.steps):
            decode_step()
        ev1.record()
        sync_all()
        region_ms.append(max_over_ranks(ev0.elapsed_time(ev1)))
    clocks = sampler.stop() if sampler else None
    ms_per_step = statistics.median(region_ms) / args.steps
    packed_bytes = B * ctx * HEADS_KV * BYTES_PER_TOKEN_HEAD  # per rank per step
    value = world * packed_bytes / (ms_per_step * 1e-3) / 1e9

    dense = None
    if args.dense_baseline and rank == 0:
        dense = time_dense_baseline(torch, _lib, dev, B, ctx, BS, block_table, q, scale, args)
    if light:
        if rank != 0:
            return None
        peak, peak_kind = measured_peak()
        achieved = packed_bytes / (ms_per_step * 1e-3) / 1e9
        line = {"metric": "packed_kv_decode_attention_throughput", "value": value, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "us_per_layer": ms_per_step * 1e3,
                "config": dict(workload_config(args), schedule="persistent" if streamed else "split"),
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "peak_source": f"{peak_kind} copy bandwidth", "algorithmic_bytes_per_launch": packed_bytes},
                "clocks": clocks}
        if dense is not None:
            line["dense_kv_baseline"] = dense
        return line

    # ---- the timed output against the oracle, on a sample of the batch (outside any timed region) ----
    parity = guarded(lambda: oracle_sample_check(torch, decode_step, q, out, cache, block_table, ctx, BS, lk, lv, scale,
                                                 args.stat)) if rank == 0 else None

    # ---- end-to-end serving step with host inputs --------------------------------------
    # The caller's step: fill one pinned staging buffer (q | new K row | new V row | seq_lens |
    # slots), one host->device copy, encode-on-write, decode, one device->host copy of the
    # output, wait.  The device part is captured once into a CUDA graph through the public API
    # (the launcher neither allocates nor synchronises) and replayed per step, the way a serving
    # engine drives it; --e2e-eager issues the same calls directly.
    e2e_steps = min(max(args.steps, 200), 500)
    nq, nkv = B * HEADS_Q * HEAD_DIM, B * HEADS_KV * HEAD_DIM
    stage_bytes = (nq + 2 * nkv) * 2 + 2 * B * 4
    h_in = torch.empty((stage_bytes,), dtype=torch.uint8).pin_memory()
    d_in = torch.empty((stage_bytes,), dtype=torch.uint8, device=dev)

    def views(buf):
        o1, o2, o3, o4 = nq * 2, (nq + nkv) * 2, (nq + 2 * nkv) * 2, (nq + 2 * nkv) * 2 + B * 4
        return (buf[:o1].view(torch.bfloat16).view(B, HEADS_Q, HEAD_DIM),
                buf[o1:o2].view(torch.bfloat16).view(B, HEADS_KV, HEAD_DIM),
                buf[o2:o3].view(torch.bfloat16).view(B, HEADS_KV, HEAD_DIM),
                buf[o3:o4].view(torch.int32), buf[o4:].view(torch.int32))

    h_q, h_k, h_v, h_lens, h_slots = views(h_in)
    d_q, d_k, d_v, d_lens, d_slots = views(d_in)
    h_q.copy_(torch.randn((B, HEADS_Q, HEAD_DIM)).to(torch.bfloat16))
    h_k.copy_(torch.randn((B, HEADS_KV, HEAD_DIM)).to(torch.bfloat16))
    h_v.copy_(torch.randn((B, HEADS_KV, HEAD_DIM)).to(torch.bfloat16))
    h_out = torch.empty((B, HEADS_Q, HEAD_DIM), dtype=torch.bfloat16).pin_memory()
    bt_cpu = block_table.cpu()
    spare = BS  # tokens of head-room in the last page

    def device_part():
        d_in.copy_(h_in, non_blocking=True)
        write_tokens_to_paged_cache(cache, layout, block_table, d_slots, d_k, d_v, q_points_k=lk, q_points_v=lv,
                                    thresholds_k=tk, thresholds_v=tv, require_fast=True, stat_dtype=stat_dtype,
                                    signal_pdl_dependents=True)
        rt.run_nonuniform_decode(spec=spec_pdl, q=d_q, cache=cache, layout=layout, block_table=block_table,
                                 seq_lens=d_lens, k_qpoints_lane_major=rk, v_qpoints_code_major=rv, out=out,
                                 workspace=ws, softmax_scale=scale, stat_dtype=stat_dtype, loader=args.loader if spec.persistent else 0)
        h_out.copy_(out, non_blocking=True)

    # slot of the appended token for every position the steps cycle through (the scheduler's
    # bookkeeping, done once; a step only copies its row into the staging buffer)
    step_pos = [ctx + i for i in range(spare)]
    step_slots = torch.stack([bt_cpu[:, pos // BS] * BS + pos % BS for pos in step_pos]).to(torch.int32)

    def host_inputs(i: int):
        h_lens.fill_(step_pos[i % spare] + 1)
        h_slots.copy_(step_slots[i % spare])

    graph, e2e_mode = None, "eager"
    if not args.e2e_eager:
        try:
            host_inputs(0)
            device_part()  # every lazily created resource exists before the capture
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                device_part()
            torch.cuda.current_stream().wait_stream(side)
            graph, e2e_mode = g, "cuda_graph"
        except Exception as exc:  # capture not possible here: time the eager calls and say so
            graph, e2e_mode = None, f"eager (graph capture failed: {exc!r})"
            torch.cuda.synchronize()

    def e2e_step(i: int):
        host_inputs(i)
        if graph is not None:
            graph.replay()
        else:
            device_part()
        torch.cuda.current_stream().synchronize()  # the caller needs the result of this step

    for i in range(3):
        e2e_step(i)
    sync_all()
    t0 = time.perf_counter()
    ev0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    ev1.record()
    sync_all()
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(max(ev0.elapsed_time(ev1), 0.0)) / e2e_steps
    h2d = stage_bytes
    d2h = h_out.numel() * 2
    e2e_value = world * packed_bytes / (e2e_ms * 1e-3) / 1e9

    if rank == 0:
        peak, peak_kind = measured_peak()
        achieved = packed_bytes / (ms_per_step * 1e-3) / 1e9  # one GPU, one launch of the dominant kernel
        workload_key = f"decode_b{B}_ctx{ctx}_p{BS}"
        line = {
            "metric": "packed_kv_decode_attention_throughput",
            "value": value,
            "unit": "GB/s",
            "n_gpus": world,
            "steps": args.steps,
            "timed_regions": regions,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step,
            "us_per_layer": ms_per_step * 1e3,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f16 tensor-core operands, f32 accumulate" if streamed else "f32",
            "data": "synthetic",
            "config": dict(workload_config(args), num_splits=0 if streamed else spec.num_splits,
                           schedule="persistent" if streamed else "split", loader=args.loader),
            "roofline": {
                "bound": "hbm",
                "achieved": achieved,
                "peak": peak,
                "unit": "GB/s",
                "frac": achieved / peak,
                "peak_source": f"{peak_kind} copy bandwidth",
                "algorithmic_bytes_per_launch": packed_bytes,
                "traffic": ncu_traffic_bytes(workload_key),
                "note": "duration is the whole step (one decode kernel; + the combine kernel under --splits)",
            },
            "e2e": {"value": e2e_value, "unit": "GB/s", "mode": e2e_mode, "ms_per_step": e2e_ms, "wall_ms_per_step": e2e_wall_ms / e2e_steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": args.steps * (2 if (not streamed and spec.num_splits > 1) else 1),
            "clocks": clocks,
            "parity": parity,
        }
        if dense is not None:
            line["dense_kv_baseline"] = dense
        if world == 1 and not args.no_cpu_baseline:
            base = cpu_decode_baseline(args, args.cpu_sample_requests)
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample", "same_config")}
            if "quantiser" in base:
                line["cpu_baseline"]["quantiser"] = base["quantiser"]
        return line
    return None


def oracle_sample_check(torch, decode_step, q, out, cache, block_table, ctx, BS, lk, lv, scale, stat, requests: int = 4):
    """Run the timed step once more, this time also asking for the un-rounded float32 result, and
    compare the rows of `requests` of its requests with the float64 oracle evaluated over the same
    packed pages (copied to the host): float32 result within 2e-3, 16-bit output within one unit in
    the last place of the rounded oracle."""
    import numpy as np

    import oracle

    out32 = torch.empty(out.shape, dtype=torch.float32, device=out.device)
    decode_step(out32)
    torch.cuda.synchronize()
    B = int(q.shape[0])
    picks = sorted({0, B // 3, (2 * B) // 3, B - 1})[:requests]
    pages = (ctx + BS - 1) // BS
    geo = oracle.PageGeometry(BS, HEADS_KV)
    kind = "f16" if stat == "fp16" else "bf16"
    worst, worst_16, ulps = 0.0, 0.0, 0.0
    for b in picks:
        ids = block_table[b, :pages].long()
        local = cache[ids].cpu().numpy()  # this request's pages, renumbered 0 .. pages-1
        want = oracle.decode_attention(q[b : b + 1].float().cpu().numpy(), local, geo,
                                       np.arange(pages, dtype=np.int32)[None, :], [ctx], levels_k=lk.float().cpu().numpy(),
                                       levels_v=lv.float().cpu().numpy(), softmax_scale=scale, stat=kind)
        worst = max(worst, float(np.abs(out32[b : b + 1].cpu().numpy() - want).max()))
        want16 = torch.from_numpy(want).to(out.dtype).float().numpy()
        gap16 = np.abs(out[b : b + 1].float().cpu().numpy() - want16)
        worst_16 = max(worst_16, float(gap16.max()))
        big = np.abs(want16) >= 2.0**-6  # units in the last place mean something for values of ordinary size
        ulp = np.exp2(np.floor(np.log2(np.abs(want16[big]))) - 7)  # bf16 spacing
        ulps = max(ulps, float((gap16[big] / ulp).max()) if big.any() else 0.0)
    return {"max_abs": worst, "requests": len(picks), "request_ids": picks, "tolerance": 2e-3,
            "compared": "float32 result of the timed kernel vs float64 oracle over the same packed pages (oracle/)",
            "bf16_output_max_abs_vs_rounded_oracle": worst_16, "bf16_output_max_ulps_vs_rounded_oracle": ulps}


def time_dense_baseline(torch, _lib, dev, B, ctx, BS, block_table, q, scale, args):
    """bf16-KV decode attention on the same shapes and block table (512 B per token-head)."""
    from beyond_kv_cache_b200.quant.fa4_cute.beyond_decode_policy import modeled_splits

    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    splits = modeled_splits(tiles=int(block_table.shape[1]), batch=B, heads_kv=HEADS_KV, sm_count=sms, page_size=BS)
    num_pages = int(block_table.max().item()) + 1
    k_pages = torch.randn((num_pages, BS, HEADS_KV, HEAD_DIM), device=dev).to(torch.bfloat16)
    v_pages = torch.randn((num_pages, BS, HEADS_KV, HEAD_DIM), device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    seq_lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    o = torch.empty((splits, B, HEADS_Q, HEAD_DIM), dtype=torch.float32, device=dev)
    m = torch.empty((splits, B, HEADS_Q), dtype=torch.float32, device=dev)
    l = torch.empty_like(m)

    def step():
        _lib.call("bkv_decode_dense_sm100", q.data_ptr(), q.stride(0), _lib.BKV_BF16, k_pages.data_ptr(),
                  v_pages.data_ptr(), _lib.BKV_BF16, num_pages, BS, HEADS_KV, block_table.data_ptr(),
                  block_table.stride(0), seq_lens.data_ptr(), out.data_ptr(), _lib.BKV_BF16, o.data_ptr(),
                  m.data_ptr(), l.data_ptr(), splits, B, HEADS_Q, block_table.shape[1] * BS, scale,
                  _lib.current_stream(dev))

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    reps = max(3, min(args.steps, 20))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    nbytes = B * ctx * HEADS_KV * 512
    result = {"us_per_layer": ms * 1e3, "GBps_bf16_bytes": nbytes / (ms * 1e-3) / 1e9, "bytes_per_token_head": 512,
              "kernel": "bkv_decode_dense_sm100 (this library, CUDA cores)"}
    del k_pages, v_pages
    result["library_flash_attn"] = time_flash_attn_library(torch, dev, B, ctx, q, scale, max(3, min(args.steps, 50)))
    return result


def time_flash_attn_library(torch, dev, B, ctx, q, scale, steps):
    """flash_attn_with_kvcache on a paged bf16 cache of the same shape (library code, not part
    of this product: the strongest bf16-KV decode kernel available in the image).  Its paged
    mode needs 256-token pages."""
    try:
        from flash_attn import flash_attn_with_kvcache
    except Exception as exc:
        return {"unavailable": repr(exc)}
    try:
        page = 256
        pages_per_seq = (ctx + page - 1) // page
        num_pages = B * pages_per_seq
        gen = torch.Generator(device=dev)
        gen.manual_seed(5)
        bt = torch.randperm(num_pages, generator=gen, device=dev).to(torch.int32).view(B, pages_per_seq)
        kc = torch.randn((num_pages, page, HEADS_KV, HEAD_DIM), device=dev).to(torch.bfloat16)
        vc = torch.randn((num_pages, page, HEADS_KV, HEAD_DIM), device=dev).to(torch.bfloat16)
        lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        q4 = q.view(B, 1, HEADS_Q, HEAD_DIM)

        def step():
            return flash_attn_with_kvcache(q4, kc, vc, cache_seqlens=lens, block_table=bt, softmax_scale=scale)

        for _ in range(3):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        nbytes = B * ctx * HEADS_KV * 512
        return {"us_per_layer": ms * 1e3, "GBps_bf16_bytes": nbytes / (ms * 1e-3) / 1e9, "page_tokens": page,
                "kernel": "flash_attn.flash_attn_with_kvcache"}
    except Exception as exc:
        return {"unavailable": repr(exc)}


if __name__ == "__main__":
    main()
