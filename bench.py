"""Benchmark of the packed-KV decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode|pack|alloc]
    python bench.py --impl reference ...         # CPU restatement of the reference path

One "step" of the default workload is one decode step of the full-depth
Llama-3.1-8B attention shape (32 layers x batch 16 x 8 KV heads / 32 query heads,
head_dim 128, context 32768, 2048 kept tokens per head at the 1/8 fp16 - 1/4 8-bit -
3/8 4-bit - 1/4 2-bit mix, 64 of 128 K channels kept as 16@8b + 24@4b + 24@2b):
a fresh bf16 query per (sequence, layer, head) against the static packed cache.
With N GPUs the KV heads are sharded (8/N per rank, no collective on the data path).
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

CFG3 = dict(name="config 3", layers=32, batch=16, kv_heads=8, q_heads=32, context=32768, budget=2048, config_id=3,
            workload="config 3: full-depth decode, Llama-3.1-8B attention shape — 32 layers x batch 16 x 8 KV heads "
                     "(32 q heads, head_dim 128), context 32768, 2048 kept tokens/head (1/8 fp16, 1/4 8b, 3/8 4b, 1/4 2b), "
                     "64 K channels kept (16@8b,24@4b,24@2b), bf16 q per step")
CFG4 = dict(name="config 4", layers=80, batch=4, kv_heads=8, q_heads=64, context=131072, budget=8192, config_id=4,
            workload="config 4: long-context decode, Qwen2.5-72B attention shape — 80 layers x batch 4 x 8 KV heads "
                     "(64 q heads, head_dim 128), context 131072, 8192 kept tokens/head (config-0 bit mix), "
                     "64 K channels kept, bf16 q per step")
L2_BYTES = 126 * 1024 * 1024
PERSISTENT = None                        # --persistent 0/1 forces the kernel form (default: the library's choice)
METRIC = "packed-KV decode-attn tokens/s"

# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of one fused-kernel launch in
# the committed ncu capture (profiles/; an 8-layer launch); traffic grows with the units processed,
# so the ratio carries over to the full launch.
NCU_TRAFFIC_BYTES_PER_ALGO_BYTE = 1.025
# dram__bytes_read.sum + dram__bytes_write.sum of the packing launches of one config-1 step in the
# committed ncu launch list (profiles/; a one-pass capture of the full workload)
PACK_NCU_TRAFFIC_BYTES = 664.9e6


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def config_dict(cfg, small):
    """The workload description both arms (CUDA and CPU reference) print, key for key."""
    return {"workload": cfg["workload"], "batch": cfg["batch"], "layers": cfg["layers"], "kv_heads": cfg["kv_heads"],
            "q_heads": cfg["q_heads"], "token_budget": cfg["budget"], "context": cfg["context"], "small": bool(small)}


# ── clocks: sampled through NVML (read-only) while the timed regions run ─────
class ClockSampler:
    REASONS = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
               0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
               0x100: "display_clock_setting"}

    def __init__(self, cuda_index: int, period_s: float = 0.004):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self.period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = cuda_index
            if vis:
                ids = [v.strip() for v in vis.split(",") if v.strip()]
                if cuda_index < len(ids) and ids[cuda_index].isdigit():
                    phys = int(ids[cuda_index])
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ── workload construction ────────────────────────────────────────────────────
def unit_bytes(pl, nv, seq_part=None) -> int:
    """Algorithmic bytes of one packed (sequence, layer): packed K and V rows of every head's live
    rows (those of `seq_part` = (i, n), part i of n of each of the head's phases; default all), their
    V scale / zero point, fp16 rows, and the K scale / zero point of the head."""
    from rdkv_b200.sharding import part_rows
    sb = pl.seg_bounds_per_head.cpu().tolist()
    n16 = pl.n_v16_per_head.cpu().tolist()
    k_row = sum(t.shape[-1] for t in (pl.K_2bit, pl.K_4bit, pl.K_8bit) if t is not None)
    part, parts = (0, 1) if seq_part is None else seq_part
    per_row = [32 + 4, 64 + 4, 128 + 4, 256]
    total = 0
    for (n2, n4, n8), n in zip(sb, n16):
        for p, (lo, hi) in enumerate(part_rows((n2, n4, n8, n), part, parts)):
            total += (hi - lo) * (k_row + per_row[p])
        total += 2 * 2 * pl.K_ch_scale.shape[-1]
    return total


def build_decode_cache(cfg, h0, h1, replica, device):
    """Packed cache of this rank's KV heads [h0,h1) for every (layer, sequence): synthetic K/V of
    the full context generated on the device from the unit's seed, bits prescribed by ranked
    lognormal importances, packed by the library's own (parity-checked) packer."""
    from rdkv_b200 import synth
    from rdkv_b200.packing import pack_kv
    g = cfg["q_heads"] // cfg["kv_heads"]
    layers, nvs = [], []
    for layer in range(cfg["layers"]):
        for seq in range(cfg["batch"]):
            seed = synth.unit_seed(cfg["config_id"], layer, seq) + 100003 * replica
            K, V = synth.make_kv(cfg["kv_heads"], cfg["context"], seed=seed, device=device)
            vb = synth.make_v_bits(cfg["kv_heads"], cfg["context"], cfg["budget"], seed=seed, device=device)
            kb = synth.make_k_bits(cfg["kv_heads"], seed=seed, device=device)
            pl, nv = pack_kv(K[:, h0:h1], V[:, h0:h1], vb[h0:h1], kb[h0:h1], g, build_mask=False)
            layers.append(pl)
            nvs.append(nv)
            del K, V
    return layers, nvs


def timed_steps(fn, steps, barrier):
    """Time `steps` calls of fn(i) with CUDA events on the current stream; returns ms."""
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()          # a profiler run with --profile-from-start off sees the timed regions only
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    barrier()
    return e0.elapsed_time(e1)


def max_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def repeated_regions(fn, steps, barrier, world, device, *, min_reps=10, target_ms=60.0, max_reps=60):
    """The `steps`-step region timed several times (each bracketed by barrier + synchronize, max over
    ranks): at least `min_reps` times and until the timed GPU work adds up to `target_ms`.
    Returns (median ms of a region, dict with reps / min / max / total)."""
    first = max_over_ranks(timed_steps(fn, steps, barrier), world, device)
    reps = int(min(max_reps, max(min_reps, -(-target_ms // max(first, 1e-3)))))
    times = [first] + [max_over_ranks(timed_steps(fn, steps, barrier), world, device) for _ in range(reps - 1)]
    return statistics.median(times), {"reps": len(times), "ms_min": min(times), "ms_max": max(times),
                                      "timed_region_s": sum(times) / 1e3}


def measure_decode(cfg, rank, world, device, *, steps, warmup, seq_parts=1, chunks=None, want_e2e=False,
                   e2e_slices=None, small=False, e2e_graph=None):
    """One decode workload on this rank's share: KV heads sharded over world/seq_parts head groups,
    the live rows of every head split over seq_parts ranks (row windows of the same packed layer,
    records merged after one all-gather per step).  Returns a dict of timings and byte counts
    (identical on every rank after the max over ranks), plus the tables for the CPU baseline."""
    from rdkv_b200 import sharding
    from rdkv_b200.decode import DecodeTable, packed_decode_attention, packed_decode_attention_host
    H_kv = cfg["kv_heads"]
    head_rank, head_world, part = sharding.grid(rank, world, seq_parts)
    assert H_kv % head_world == 0, "KV heads are sharded across head groups: their number must divide 8"
    h0, h1 = sharding.head_shard(head_rank, head_world, H_kv)
    g = cfg["q_heads"] // H_kv
    Hq_loc = (h1 - h0) * g
    n_views = cfg["layers"] * cfg["batch"]
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)
    group = None
    if seq_parts > 1:                                        # one process group per set of ranks that share heads
        for hr in range(head_world):
            gr = dist.new_group(list(range(hr * seq_parts, (hr + 1) * seq_parts)))
            if hr == head_rank:
                group = gr

    # enough distinct cache replicas that consecutive steps cannot be served from L2
    tables, step_bytes, seq_part = [], None, None
    while True:
        layers, nvs = build_decode_cache(cfg, h0, h1, len(tables), device)
        tb = DecodeTable(layers, nvs, Hq_loc, n_chunks=chunks, persistent=PERSISTENT)
        seq_part = (part, seq_parts) if seq_parts > 1 else None
        step_bytes = sum(unit_bytes(pl, nv, seq_part) for pl, nv in zip(layers, nvs))
        tables.append(tb)
        if len(tables) * step_bytes >= 2.2 * L2_BYTES or small:
            break
    R = len(tables)
    gen = torch.Generator(device=device)
    gen.manual_seed(4242 + head_rank)                        # ranks that share heads draw the same queries
    n_q = min(steps + warmup, 16 if cfg["q_heads"] > 32 else 64)
    q_pool = [(torch.randn(n_views, Hq_loc, 128, generator=gen, device=device) / 128 ** 0.5).to(torch.bfloat16)
              for _ in range(n_q)]
    out = torch.empty((n_views, Hq_loc, 128), dtype=torch.float32, device=device)
    n_rows = n_views * Hq_loc
    if seq_parts > 1:
        rec = torch.empty((n_rows, 132), dtype=torch.float32, device=device)
        gathered = torch.empty((seq_parts * n_rows, 132), dtype=torch.float32, device=device)

    def step(i):
        if seq_parts == 1:
            packed_decode_attention(q_pool[i % n_q], tables[i % R], out=out)
        else:
            sharding.sequence_split_attention(q_pool[i % n_q], tables[i % R], group, part=part, n_parts=seq_parts,
                                              record=rec, gathered=gathered)

    for i in range(warmup):
        step(i)
    sampler = ClockSampler(device.index if device.index is not None else 0)
    with sampler:
        ms, timing = repeated_regions(step, steps, barrier, world, device)

    # the fused kernel alone (dominant) inside the same loop, and what follows it in a sequence split
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    torch.cuda.synchronize()
    barrier()
    torch.cuda.profiler.start()
    with sampler:
        for i in range(steps):
            tb = tables[i % R]
            ev[i][0].record()
            if seq_parts == 1:
                packed_decode_attention(q_pool[i % n_q], tb, out=out)
                ev[i][1].record()
            else:
                packed_decode_attention(q_pool[i % n_q], tb, out_partial=rec, seq_part=seq_part)
                ev[i][1].record()
                sharding.combine_across_ranks(rec, group, gathered=gathered)
            ev[i][2].record()
        torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    fused_ms = max_over_ranks(statistics.mean(e[0].elapsed_time(e[1]) for e in ev), world, device)
    if seq_parts == 1:
        # a step is exactly one launch of the fused kernel and the launches run back to back: the timed
        # region per step is the kernel's average duration too (the per-launch event pairs of the pass
        # above add their own gaps; the smaller of the two is reported)
        fused_ms = min(fused_ms, ms / steps)
    after_ms = max_over_ranks(statistics.mean(e[1].elapsed_time(e[2]) for e in ev), world, device)

    res = {"ms_region": ms, "timing": timing, "fused_ms": fused_ms, "after_ms": after_ms, "step_bytes": step_bytes,
           "replicas": R, "tables": tables, "out": out, "q0": q_pool[0], "sampler": sampler, "h": (h0, h1),
           "n_views": n_views, "Hq_loc": Hq_loc}
    if want_e2e:
        # end to end through the public call with host buffers: pinned q in, pinned out back, every step
        # (two query buffers in turn; the call records each (buffer, table) pair's copies and launches
        # as a graph on its second use and replays it afterwards, so every pair is warmed up twice)
        q_host = [q.cpu().pin_memory() for q in q_pool[:min(n_q, 2)]]
        out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()

        def e2e_step(i):
            packed_decode_attention_host(q_host[i % len(q_host)], tables[i % R], out_host, slices=e2e_slices,
                                         graph=e2e_graph)

        for i in range(max(min(warmup, 3), 2 * len(q_host) * R + 1)):
            e2e_step(i)
        with sampler:
            e2e_ms, e2e_timing = repeated_regions(e2e_step, steps, barrier, world, device, min_reps=5, target_ms=30.0)
        res["e2e_ms_region"], res["e2e_timing"] = e2e_ms, e2e_timing
        res["e2e_ranges"] = len(tables[0]._host_io.ranges)
    for tb in tables:
        tb.check_status()
    return res


def grid_name(world, seq_parts):
    return f"{world // seq_parts}x{seq_parts}"


def run_decode(args, rank, world, device):
    cfg = dict(CFG3)
    if args.small:
        cfg.update(layers=2, batch=2, context=4096, budget=1024)
    if args.layers:
        cfg.update(layers=args.layers)
    m = measure_decode(cfg, rank, world, device, steps=args.steps, warmup=args.warmup, chunks=args.chunks,
                       want_e2e=True, e2e_slices=args.e2e_slices, small=args.small,
                       e2e_graph=None if args.e2e_graph is None else bool(args.e2e_graph))
    t0 = m["tables"][0]
    k_rest, rows_rest, n_whole = t0.plan(t0.n_views)
    h0, h1 = m["h"]
    line = None
    if rank == 0:
        peak, peak_kind = load_peaks()
        ms = m["ms_region"]
        tokens = cfg["batch"] * args.steps
        sec = ms / 1e3
        step_bytes = m["step_bytes"]
        total_step_bytes = step_bytes * world            # every rank holds the same number of heads
        achieved = step_bytes / (m["fused_ms"] / 1e3) / 1e9   # per-GPU GB/s of the dominant kernel
        e2e_ms = m["e2e_ms_region"]
        line = {
            "metric": METRIC, "value": tokens / sec, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "u8 codes / fp16 scales, fp32 accumulate",
            "data": "synthetic",
            "config": config_dict(cfg, args.small or args.layers),
            "detail": {
                "parallelism": f"kv-head sharding x{world} (no data-path collective)",
                "launches_per_step": 1,
                "kernel_form": ("persistent (resident CTAs draw the items from a counter)"
                                if (t0.persistent if t0.persistent is not None else
                                    (k_rest == 1 and t0.n_views * (h1 - h0) >= t0.PERSISTENT_MIN_ROUNDS * t0._sms * t0.CTAS_PER_SM))
                                and t0._can_persist() else "one CTA per item"),
                "l2": f"{m['replicas']} cache replica(s) rotated per step, {m['replicas'] * step_bytes / 2**20:.0f} MiB per GPU "
                      f"> 2 x 126 MiB L2; no flush needed",
                "launch_shape": ("one CTA per (view, KV head)" if k_rest == 1
                                 else f"{n_whole} (view, KV head) units whole, the other "
                                      f"{t0.n_views * (h1 - h0) - n_whole} in {k_rest} chunks of {rows_rest} "
                                      "rows merged in the kernel"),
                "timing": dict(m["timing"], note="value = median over the repeated regions of `steps` steps each"),
            },
            "hbm_gbs": total_step_bytes * args.steps / sec / 1e9,
            "hbm_frac_of_8tbs": total_step_bytes * args.steps / sec / 1e9 / (8000.0 * world),
            "algorithmic_bytes_per_step": total_step_bytes,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES_PER_ALGO_BYTE * step_bytes,
                         "peak_kind": peak_kind, "kernel": "decode_fused_kernel", "kernel_ms": m["fused_ms"],
                         "algorithmic_bytes_per_launch": step_bytes},
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": m["q0"].numel() * m["q0"].element_size() * world,
                    "d2h_bytes_per_step": m["out"].numel() * m["out"].element_size() * world,
                    "ms_per_step": e2e_ms / args.steps, "reps": m["e2e_timing"]["reps"]},
            # (value pass + per-kernel event pass: one launch per step; host-buffer pass: one per view range)
            "gpu_launches": args.steps * (m["timing"]["reps"] + 1) + args.steps * m["e2e_timing"]["reps"] * m["e2e_ranges"],
            "clocks": m["sampler"].summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_decode_baseline(cfg, m["tables"][0], layers_per_sample=1, steps=2)
    tables0 = m["tables"]
    del m
    if args.no_also or args.small or args.layers:
        return line
    # the other configurations, measured briefly in the same run and carried under "also"
    del tables0
    torch.cuda.empty_cache()
    also = {}
    grids = [1] + ([2] if world % 2 == 0 and world >= 2 else [])
    c4 = []
    for sp in grids:
        r4 = measure_decode(dict(CFG4), rank, world, device, steps=min(args.steps, 16), warmup=3, seq_parts=sp)
        if rank == 0:
            peak, _ = load_peaks()
            per_step = r4["ms_region"] / min(args.steps, 16)
            c4.append({"grid": grid_name(world, sp) + " (head groups x sequence parts)",
                       "value": CFG4["batch"] / (per_step / 1e3), "unit": "tokens/s", "ms_per_step": per_step,
                       "kernel_ms": r4["fused_ms"], "allgather_plus_combine_us": r4["after_ms"] * 1e3 if sp > 1 else 0.0,
                       "algorithmic_bytes_per_gpu": r4["step_bytes"],
                       "roofline_frac_per_gpu": r4["step_bytes"] / (r4["fused_ms"] / 1e3) / 1e9 / peak,
                       "timing": r4["timing"]})
        del r4
        torch.cuda.empty_cache()
    if rank == 0:
        also["config4"] = {"config": config_dict(CFG4, False), "grids": c4,
                           "note": "sequence parts = row windows of the same packed layer per rank; one NCCL all-gather "
                                   "of [rows,132] fp32 records per step, then the log-sum-exp combine kernel"}
    if world == 1:
        short = argparse.Namespace(**vars(args))
        short.steps, short.warmup, short.no_cpu_baseline, short.layers = min(args.steps, 10), 3, True, None
        pk = run_pack(short, rank, world, device)
        torch.cuda.empty_cache()
        al = run_alloc(short, rank, world, device)
        if rank == 0:
            also["pack"] = {k: pk[k] for k in ("metric", "value", "unit", "ms_per_step", "config", "roofline")}
            also["alloc"] = {k: al[k] for k in ("metric", "value", "unit", "ms_per_step", "config", "roofline")}
    if rank == 0:
        line["also"] = also
    return line


def run_decode_long(args, rank, world, device):
    """Config 4 as a workload of its own: KV heads over world/seq_parts head groups, the live rows
    of every head over seq_parts ranks (NCCL all-gather of the records + combine per step)."""
    cfg = dict(CFG4)
    if args.small:
        cfg.update(layers=2, batch=2, context=8192, budget=2048)
    if args.layers:
        cfg.update(layers=args.layers)
    sp = args.seq_parts
    m = measure_decode(cfg, rank, world, device, steps=args.steps, warmup=args.warmup, seq_parts=sp,
                       chunks=args.chunks, small=args.small)
    if rank != 0:
        return None
    peak, peak_kind = load_peaks()
    ms = m["ms_region"]
    sec = ms / 1e3
    tokens = cfg["batch"] * args.steps
    step_bytes = m["step_bytes"]
    achieved = step_bytes / (m["fused_ms"] / 1e3) / 1e9
    line = {
        "metric": METRIC, "value": tokens / sec, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "u8 codes / fp16 scales, fp32 accumulate", "data": "synthetic",
        "config": config_dict(cfg, args.small or args.layers),
        "detail": {"parallelism": f"{grid_name(world, sp)} (KV-head groups x sequence parts)",
                   "collective": ("none on the data path" if sp == 1 else
                                  "one NCCL all-gather of [rows,132] fp32 records per step + log-sum-exp combine kernel"),
                   "allgather_plus_combine_us": m["after_ms"] * 1e3 if sp > 1 else 0.0,
                   "l2": f"{m['replicas']} cache replica(s), {m['replicas'] * step_bytes / 2**20:.0f} MiB read per GPU and rotation",
                   "timing": m["timing"]},
        "hbm_gbs": step_bytes * world * args.steps / sec / 1e9,
        "algorithmic_bytes_per_step": step_bytes * world,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES_PER_ALGO_BYTE * step_bytes, "peak_kind": peak_kind,
                     "kernel": "decode_fused_kernel", "kernel_ms": m["fused_ms"],
                     "algorithmic_bytes_per_launch": step_bytes},
        "gpu_launches": args.steps * (m["timing"]["reps"] + 1) * (1 if sp == 1 else 2),
        "clocks": m["sampler"].summary(),
    }
    return line


# ── CPU arm: the oracle's dequantise-then-attend on the host cores ───────────
def _layer_to_np(pl):
    d = {}
    for k, v in vars(pl).items():
        if k.startswith("_"):
            continue
        d[k] = v.detach().cpu().numpy() if torch.is_tensor(v) else v
    if d.get("softmax_mask") is None:
        import numpy as np
        H = d["V_scale"].shape[1]
        g = d["K_ch_perm_padded_idx_for_Q"].shape[0] // H
        col = np.arange(d["T_eff_k"])[None]
        live = (col < d["T_eff_per_head"][:, None]) | ((col >= d["T_eff"]) &
                                                        (col < d["T_eff"] + d["n_v16_per_head"][:, None]))
        d["softmax_mask"] = np.repeat(np.where(live, 0.0, -np.inf).astype(np.float32), g, axis=0)
    return d


def cpu_attend_time(units, q_np, cores, steps, decode_steps_amortised=256):
    """units: list of (layer dict, new_v_only).  Returns seconds per step over all units:
    dequantise once (amortised over the decode run) + fp32 attention per step."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor
    from oracle import ref_packing as RP

    def dequant(u):
        layer, nv = u
        return RP.unpack_k(layer, 128)[0].astype(np.float32), RP.unpack_v(layer, nv, 128)[0].astype(np.float32), \
            layer["softmax_mask"]

    def attend(args):
        (Kh, Vh, mask), q = args
        g = q.shape[0] // Kh.shape[0]
        s = np.einsum("hgd,htd->hgt", q.reshape(Kh.shape[0], g, 128), Kh) / np.float32(128 ** 0.5)
        s = s + mask.reshape(Kh.shape[0], g, -1)
        p = np.exp(s - s.max(-1, keepdims=True))
        return np.einsum("hgt,htd->hgd", p / p.sum(-1, keepdims=True), Vh)

    with ThreadPoolExecutor(cores) as ex:
        t0 = time.perf_counter()
        deq = list(ex.map(dequant, units))
        t_deq = time.perf_counter() - t0
        times = []
        for s in range(steps):
            t0 = time.perf_counter()
            list(ex.map(attend, [(d, q_np[s % len(q_np)][i]) for i, d in enumerate(deq)]))
            times.append(time.perf_counter() - t0)
    return t_deq / decode_steps_amortised + statistics.median(times), t_deq, statistics.median(times)


def cpu_decode_baseline(cfg, table, layers_per_sample, steps):
    """Bounded sample: `layers_per_sample` layer(s) x full batch, timed on all host cores and
    scaled linearly to the full depth (decode cost is linear in layers)."""
    import numpy as np
    cores = os.cpu_count() or 1
    n_units = layers_per_sample * cfg["batch"]
    units = [(_layer_to_np(pl), None if nv is None else nv.detach().cpu().numpy())
             for pl, nv in table.source[:n_units]]
    rng = np.random.default_rng(0)
    q = [(rng.standard_normal((n_units, cfg["q_heads"], 128)) / 128 ** 0.5).astype(np.float32) for _ in range(2)]
    per_step, t_deq, t_att = cpu_attend_time(units, q, cores, steps)
    full_step = per_step * cfg["layers"] / layers_per_sample
    return {"value": cfg["batch"] / full_step, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{layers_per_sample} of {cfg['layers']} layers x batch {cfg['batch']} x {cfg['kv_heads']} heads, "
                      f"{steps} steps, numpy dequantise-then-attend on {cores} threads; dequantise "
                      f"({t_deq:.2f}s) amortised over 256 steps + attend {t_att:.3f}s/step; scaled linearly to 32 layers"}


def run_reference_arm(args, rank, world):
    """The reference's CPU path — dequantise the packed cache, then plain attention
    (obkv_accel/trizone_decompress.py:185-333 + softmax attention) — as restated in numpy under
    oracle/, on all host cores, rank 0 only.  The reference is Python on torch; its sources are not
    on the benchmark machine, so the restatement is what is timed everywhere (kind "port")."""
    if rank != 0:
        return None
    import numpy as np
    from oracle import ref_packing as RP
    from rdkv_b200 import synth
    cfg = dict(CFG4 if args.workload == "decode-long" else CFG3)
    if args.small:
        cfg.update(layers=2, batch=2, context=4096, budget=1024)
    if args.layers:
        cfg.update(layers=args.layers)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = cfg["q_heads"] // cfg["kv_heads"]
    units = []
    for seq in range(cfg["batch"]):
        seed = synth.unit_seed(cfg["config_id"], 0, seq)
        K, V = synth.make_kv(cfg["kv_heads"], cfg["context"], seed=seed)
        vb = synth.make_v_bits(cfg["kv_heads"], cfg["context"], cfg["budget"], seed=seed)
        kb = synth.make_k_bits(cfg["kv_heads"], seed=seed)
        units.append(RP.pack_kv(K.numpy(), V.numpy(), vb.numpy(), kb.numpy(), g))
    rng = np.random.default_rng(0)
    q = [(rng.standard_normal((len(units), cfg["q_heads"], 128)) / 128 ** 0.5).astype(np.float32) for _ in range(4)]
    cpu_attend_time(units, q, cores, max(1, args.warmup))
    per_step, t_deq, t_att = cpu_attend_time(units, q, cores, args.steps)
    full_step = per_step * cfg["layers"]
    value = cfg["batch"] / full_step
    sample = (f"each step = 1 of {cfg['layers']} layers x batch {cfg['batch']} x {cfg['kv_heads']} heads "
              f"(dequantise {t_deq:.2f}s amortised over 256 steps + attend {t_att:.3f}s), scaled linearly to "
              f"{cfg['layers']} layers; numpy on {cores} threads")
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": full_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp32 (numpy)", "data": "synthetic",
        "config": config_dict(cfg, args.small or args.layers),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# ── prefill workloads (configs 1 and 2); single GPU ─────────────────────────
def run_pack(args, rank, world, device):
    """Config 1: quantise-and-bitpack of 32 layers x 8 KV heads x 32768 tokens x 128 fp16 K and V
    (budget 4096 kept tokens/head at the config-0 mix, 64 kept K channels).  One step = all layers
    through pack_kv_layers (every layer in one pass: one host read of the segment counts)."""
    if rank != 0:
        return None
    from rdkv_b200 import synth
    from rdkv_b200.packing import pack_kv_layers
    L, H, T, N = (args.layers or 32), 8, 32768, 4096
    Ks, Vs, vbs, kbs = [], [], [], []
    for layer in range(L):
        seed = synth.unit_seed(1, layer)
        K, V = synth.make_kv(H, T, seed=seed, device=device)
        Ks.append(K); Vs.append(V)
        vbs.append(synth.make_v_bits(H, T, N, seed=seed, device=device))
        kbs.append(synth.make_k_bits(H, seed=seed, device=device))
    v_bits, k_bits = torch.stack(vbs).to(torch.int16), torch.stack(kbs).to(torch.int16)
    del vbs, kbs
    state = {}

    def step(i):
        state["batch"] = pack_kv_layers(Ks, Vs, v_bits, k_bits, 4, build_mask=False, k_passes=args.k_passes)

    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(device.index or 0)
    with sampler:
        ms = timed_steps(step, args.steps, lambda: None)
    sec = ms / 1e3 / args.steps
    # the launches alone (device time of the two partition and the two packing kernels), for the roofline
    spans = []
    torch.cuda.profiler.start()
    for i in range(args.steps):
        state["batch"] = pack_kv_layers(Ks, Vs, v_bits, k_bits, 4, build_mask=False, k_passes=args.k_passes, launch_events=spans)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    # per call two spans: the two partition launches, the packing launches (V pass, one-pass K)
    kern_ms = sum(a.elapsed_time(b) for a, b in spans) / args.steps
    out_bytes = 0
    for pl, nv in state["batch"]:
        out_bytes += sum(t.numel() * t.element_size() for t in
                         (pl.K_2bit, pl.K_4bit, pl.K_8bit, pl.V_2bit, pl.V_4bit, pl.V_8bit, pl.V_scale,
                          pl.V_zp, pl.K_ch_scale, pl.K_ch_zp, nv) if t is not None)
    nominal = L * H * T * 128 * 2 * 2                       # all fp16 K and V bytes of the context
    # what has to move: kept rows of K and of V read once, the bit maps read once, packed bytes written
    # (the second reading of the kept K rows by the quantise pass is the kernels' own choice, not counted)
    moved = L * H * N * 256 * 2 + v_bits.numel() * v_bits.element_size() + k_bits.numel() * k_bits.element_size() + out_bytes
    peak, kind = load_peaks()
    line = {"metric": "prefill quantise-and-bitpack GB/s of fp16 input consumed", "value": nominal / sec / 1e9,
            "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 in, u8 codes out (fp32 math)",
            "data": "synthetic",
            "config": {"workload": f"config 1: pack {L} layers x 8 KV heads x 32768 tokens x 128, budget 4096/head, "
                                   "all layers in one pass (pack_kv_layers)",
                       "l2": "4.3 GB of inputs per step > L2"},
            "roofline": {"bound": "hbm", "achieved": moved / (kern_ms / 1e3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": moved / (kern_ms / 1e3) / 1e9 / peak,
                         "traffic": PACK_NCU_TRAFFIC_BYTES, "peak_kind": kind,
                         "kernel": "2 x partition_kernel + pack_v128_batched_kernel + pack_k_onepass_batched_kernel",
                         "kernel_ms": kern_ms, "algorithmic_bytes_per_step": moved},
            "gpu_launches": 4 * 2 * args.steps, "clocks": sampler.summary()}
    if not args.no_cpu_baseline:
        from oracle import ref_packing as RP
        K, V, vb, kb = Ks[0].cpu().numpy(), Vs[0].cpu().numpy(), v_bits[0].cpu().numpy(), k_bits[0].cpu().numpy()
        t0 = time.perf_counter()
        RP.pack_kv(K, V, vb, kb, 4)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": (nominal / L) / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                                "sample": f"1 of {L} layers, numpy oracle pack_kv, {dt:.2f}s"}
    return line


def run_score(args, rank, world, device):
    """Importance scoring of one layer in config-1 shape (8 KV heads x 4 query heads x 32-position
    observation window over 32768 tokens, fp16) followed by the default pooling (avg, 5, reflect)."""
    if rank != 0:
        return None
    from rdkv_b200.scoring import _score_one_layer, apply_score_pooling, obs_window_scores
    B, H, g, W, T, D = 1, 8, 4, 32, 32768, 128
    gen = torch.Generator(device=device)
    gen.manual_seed(77)
    n_rep = 4                                               # rotate inputs: 4 x 201 MB > L2
    aws = [torch.softmax(torch.randn(B, H, g, W, T, generator=gen, device=device) * 2, dim=-1).half() for _ in range(n_rep)]
    qs = [torch.randn(B, H, g, W, D, generator=gen, device=device).half() for _ in range(n_rep)]
    ks = [torch.randn(B, H, T, D, generator=gen, device=device).half() for _ in range(n_rep)]

    def step(i):
        j = i % n_rep
        tok, ch = _score_one_layer(aws[j], qs[j], None, ks[j], D, k=ks[j])
        apply_score_pooling(tok[0], "avg", 5, "reflect")

    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(device.index or 0)
    with sampler:
        ms = timed_steps(step, args.steps, lambda: None)
    sec = ms / 1e3 / args.steps
    moved = aws[0].numel() * 2 + ks[0].numel() * 2 + qs[0].numel() * 2 + H * T * 4 * 3
    peak, kind = load_peaks()
    # the same scores straight from the window's queries and the keys (no attention weights in memory),
    # and what producing the weights first costs (matmul, mask, softmax by torch; then the scoring kernel)
    q_obs = [q.view(B, H * g, W, D) for q in qs]
    mask = torch.arange(T, device=device)[None, :] > torch.arange(T - W, T, device=device)[:, None]

    def fused(i):
        tok, ch = obs_window_scores(q_obs[i % n_rep], ks[i % n_rep])
        apply_score_pooling(tok[0], "avg", 5, "reflect")

    def two_step(i):
        j = i % n_rep
        aw = torch.matmul(q_obs[j], ks[j].repeat_interleave(g, dim=1).transpose(-1, -2)) * (1.0 / D ** 0.5)
        aw = aw.masked_fill_(mask[None, None], float("-inf")).softmax(dim=-1)
        tok, ch = _score_one_layer(aw.view(B, H, g, W, T), qs[j], None, ks[j], D, k=ks[j])
        apply_score_pooling(tok[0], "avg", 5, "reflect")

    extra = {}
    for name, fn in (("from_queries_and_keys", fused), ("weights_by_torch_then_scoring", two_step)):
        for i in range(args.warmup):
            fn(i)
        with sampler:
            t_ms = timed_steps(fn, args.steps, lambda: None) / args.steps
        nbytes = ks[0].numel() * 2 + q_obs[0].numel() * 2 + H * T * 4 * 3
        extra[name] = {"ms_per_step": t_ms, "algorithmic_bytes": nbytes, "frac_of_hbm_peak": nbytes / (t_ms / 1e3) / 1e9 / peak}
    return {"metric": "importance scoring + pooling, layers/s", "value": 1.0 / sec, "unit": "layers/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp16 in, fp32 accumulate", "data": "synthetic",
            "config": {"workload": "score one layer: aw [1,8,4,32,32768] fp16, K [1,8,32768,128] fp16, avg-5 reflect pooling",
                       "l2": "4 input sets of 201 MB rotated > L2"},
            "roofline": {"bound": "hbm", "achieved": moved / sec / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": moved / sec / 1e9 / peak, "traffic": None, "peak_kind": kind,
                         "kernel": "score_layer_kernel + pool_kernel (whole step, 2 launches)",
                         "algorithmic_bytes_per_step": moved},
            "obs_window": extra,
            "gpu_launches": (2 + 4 + 2) * args.steps, "clocks": sampler.summary()}


def run_alloc(args, rank, world, device):
    """Config 2: 256 V rows of 32768 token scores + 256 K rows of 128 channel scores, lognormal(0,1.5),
    budget 2.0 bits/token for V, per-head K budget derived from the V result; 60 bisection steps."""
    if rank != 0:
        return None
    from rdkv_b200 import synth
    from rdkv_b200.knapsack_solver import knapsack_bit_allocation_batched
    rows = 256
    eps = synth.ALLOC_EPSILON
    sv = synth.make_scores(rows, 32768, seed=synth.unit_seed(2), device=device)
    sk = synth.make_scores(rows, 128, seed=synth.unit_seed(2, 1), device=device)

    def step(i):
        vb = knapsack_bit_allocation_batched(sv, 2.0, epsilon=eps, max_iters=60)
        t_eff = (vb > 0).sum(dim=1).clamp(min=1).float()
        k_avg = (0.5 * 2 * 4096 * 128 * 16) / (128 * t_eff)
        knapsack_bit_allocation_batched(sk, k_avg, epsilon=eps, max_iters=60)

    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(device.index or 0)
    with sampler:
        ms = timed_steps(step, args.steps, lambda: None)
    sec = ms / 1e3 / args.steps
    bytes_ = rows * 32768 * (4 + 8) + rows * 128 * (4 + 8)
    peak, kind = load_peaks()
    line = {"metric": "batched bit allocator rows/s (V rows of 32768 + K rows of 128)", "value": 2 * rows / sec,
            "unit": "rows/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 compare/select, int64 out",
            "data": "synthetic", "config": {"workload": "config 2: 256 V rows x 32768 + 256 K rows x 128, 60-step bisection",
                                            "l2": "latency/ALU-bound; inputs 34 MB"},
            "roofline": {"bound": "hbm", "achieved": bytes_ / sec / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": bytes_ / sec / 1e9 / peak, "traffic": None, "peak_kind": kind,
                         "kernel": "knapsack_seed_kernel + knapsack_solve_kernel",
                         "note": "scores read once (4 B) + int64 decisions written (8 B); the kernel is ALU/latency-bound"},
            "gpu_launches": 4 * args.steps, "clocks": sampler.summary()}
    if not args.no_cpu_baseline:
        from oracle.ref_knapsack import knapsack_batched
        t0 = time.perf_counter()
        knapsack_batched(sv[:8].cpu().numpy(), 2.0, eps, max_iters=60)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 8 / dt, "unit": "rows/s", "cores": 1, "kind": "port",
                                "sample": f"8 of 256 V rows, numpy oracle, {dt:.2f}s"}
    return line


def run_aux(args, rank, world, device):
    """The small kernels around the hot path, each timed alone on config-3-sized inputs: the
    decompressor (one launch per layer), the uncompressed-tail kernel, the log-sum-exp combine, block
    scoring of the blockwise decoder and the token / channel partition.  One step = each of them once."""
    if rank != 0:
        return None
    from rdkv_b200 import synth
    from rdkv_b200.blockwise import _score_block
    from rdkv_b200.decode import DecodeTable, lse_combine, packed_decode_attention, tail_attention_partial
    from rdkv_b200.decompress import unpack_trizone_to_past_kv
    from rdkv_b200.packing import TriZoneCache, pack_kv, partition_by_bits
    L, H, g, T, N = (args.layers or 8), 8, 4, 32768, 2048
    layers, nvs = [], []
    for layer in range(L):
        seed = synth.unit_seed(3, layer, 0)
        K, V = synth.make_kv(H, T, seed=seed, device=device)
        pl, nv = pack_kv(K, V, synth.make_v_bits(H, T, N, seed=seed, device=device),
                         synth.make_k_bits(H, seed=seed, device=device), g)
        layers.append(pl); nvs.append(nv)
        del K, V
    cache = TriZoneCache(packed=tuple(layers), new_v_only=nvs, new_both_k=[None] * L, new_both_v=[None] * L,
                         original_seq_len=T)
    gen = torch.Generator(device=device); gen.manual_seed(5)
    n_views, cap = 128, 1024
    q = (torch.randn(n_views, H * g, 128, generator=gen, device=device) / 128 ** 0.5).half()
    new_k = torch.randn(n_views, H, cap, 128, generator=gen, device=device).half()
    new_v = torch.randn(n_views, H, cap, 128, generator=gen, device=device).half()
    recs = torch.randn(512 * H * g, 2, 132, generator=gen, device=device)
    recs[:, :, 1] = recs[:, :, 1].abs() + 0.5
    bq = torch.randn(L, H * g, 64, 128, generator=gen, device=device).half()
    bk = torch.randn(L, 1, H, 64, 128, generator=gen, device=device).half()
    vbits = synth.make_v_bits(H * 32, T, 4096, seed=11, device=device).to(torch.int16)
    kbits = synth.make_k_bits(H * 32, seed=11, device=device).to(torch.int16)
    # the whole attention block of a decode step over 128 views (8 layers x batch 16 of config 3) with a
    # 1024-row fp16 tail (the reference's latency protocol generates 1024 tokens): packed zones alone,
    # the one-launch form (rotation, new token, tail, packed zones) and the three-launch form
    cfg8 = dict(CFG3); cfg8.update(layers=8)
    dl, dnv = build_decode_cache(cfg8, 0, H, 0, device)
    dtab = DecodeTable(dl, dnv, H * g)
    dbytes = sum(unit_bytes(pl, nv, None) for pl, nv in zip(dl, dnv))
    k_cur = torch.randn(n_views, H, 128, generator=gen, device=device).half()
    v_cur = torch.randn(n_views, H, 128, generator=gen, device=device).half()
    pos = torch.rand(n_views, 64, generator=gen, device=device) * 500.0
    rope = (torch.cos(pos), torch.sin(pos))
    dout = torch.empty(n_views, H * g, 128, device=device)
    tail_bytes = n_views * H * (cap - 1) * 128 * 2 * 2
    # the two-stage operators on one config-3 layer: score / weighted-sum mode of the fused kernel, and
    # the scalar kernels that serve shapes outside it (called through the C ABI on the same layer)
    import ctypes as C
    from rdkv_b200._lib import check, lib, ptr, q_dtype_tag, stream_ptr
    from rdkv_b200.k_kernel import k_mixed_qk_dot_into
    from rdkv_b200.packing import layer_view
    from rdkv_b200.v_kernel import v_dequant_weighted_sum_dispatch_into
    pl0, nv0 = layers[0], nvs[0]
    T_k = int(pl0.T_eff_k)
    q1 = q[0].contiguous()
    sc = torch.empty(H * g, T_k, device=device)
    w1 = torch.softmax(torch.randn(H * g, T_k, generator=gen, device=device), -1)
    o1 = torch.empty(H * g, 128, device=device)
    view0, _keep0 = layer_view(pl0, nv0)
    k_bytes, v_bytes = H * N * 34 + H * 256, H * N * (67.5 + 32) + w1.numel() * 4

    def scalar_k():
        check(lib().rdkv_k_scores(C.byref(view0), ptr(q1), q_dtype_tag(q1), q1.stride(0), H * g, H, T_k, ptr(sc),
                                  sc.stride(0), stream_ptr(device)), "rdkv_k_scores")

    def scalar_v():
        check(lib().rdkv_v_weighted_sum(C.byref(view0), ptr(w1), w1.stride(0), H * g, H, ptr(o1), o1.stride(0),
                                        stream_ptr(device)), "rdkv_v_weighted_sum")

    parts = {
        "k_mixed_qk_dot_into, one layer (decode_fused_kernel, score mode)": (
            lambda: k_mixed_qk_dot_into(q1, pl0, T_k, sc), k_bytes + sc.numel() * 4),
        "v_dequant_weighted_sum_dispatch_into, one layer (decode_fused_kernel, weighted-sum mode)": (
            lambda: v_dequant_weighted_sum_dispatch_into(w1, pl0, o1, V16=nv0[0], n_v16_per_head=pl0.n_v16_per_head,
                                                         max_T_v=pl0.T_eff), v_bytes),
        "k_scores_kernel (scalar), one layer": (scalar_k, k_bytes + sc.numel() * 4),
        "v_weighted_sum_kernel (scalar), one layer": (scalar_v, v_bytes),
        "decode block, packed zones only (decode_fused_kernel)": (lambda: packed_decode_attention(q, dtab, out=dout), dbytes),
        "decode block, one launch: rotation + new token + 1023-row tail + packed zones (decode_fused_kernel, tail mode)": (
            lambda: packed_decode_attention(q, dtab, out=dout, new_k=new_k, new_v=new_v, n_new=cap - 1, k_cur=k_cur,
                                            v_cur=v_cur, rope=rope, append=False), dbytes + tail_bytes),
        "decode block, three launches: packed zones + tail_attn_partial_kernel + lse_combine_kernel": (
            lambda: packed_decode_attention(q, dtab, out=dout, new_k=new_k, new_v=new_v, n_new=cap - 1, one_launch=False),
            dbytes + tail_bytes),
        "unpack_layer_kernel": (lambda: unpack_trizone_to_past_kv(cache, head_dim=128),
                                L * H * (N * (34 + 67.5) + 2 * N * 128 * 2)),
        "tail_attn_partial_kernel": (lambda: tail_attention_partial(q, new_k, new_v, cap, H),
                                     n_views * H * cap * 128 * 2 * 2),
        "lse_combine_kernel": (lambda: lse_combine(recs), recs.numel() * 4 + recs.shape[0] * 128 * 4),
        "block_score_kernel": (lambda: [_score_block(bq[l], bk[l], num_kv_groups=g, causal=False) for l in range(L)],
                               L * (H * g * 64 + H * 64) * 128 * 2),
        "partition_kernel": (lambda: (partition_by_bits(vbits, 0), partition_by_bits(kbits, 1)),
                             vbits.numel() * 2 * 3 + kbits.numel() * 2 * 3),
    }
    peak, kind = load_peaks()
    out = {}
    sampler = ClockSampler(device.index or 0)
    for name, (fn, nbytes) in parts.items():
        for _ in range(args.warmup):
            fn()
        with sampler:
            ms = timed_steps(lambda i: fn(), args.steps, lambda: None) / args.steps
        out[name] = {"ms": ms, "algorithmic_bytes": int(nbytes), "gbs": nbytes / (ms / 1e3) / 1e9,
                     "frac_of_hbm_peak": nbytes / (ms / 1e3) / 1e9 / peak}
    return {"metric": "auxiliary kernels, ms per call", "value": sum(v["ms"] for v in out.values()), "unit": "ms",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp16 / u8", "data": "synthetic",
            "config": {"workload": f"aux: decompress {L} config-3 layers; tail attention 128 views x 8 heads x 1024 rows; "
                                   "combine 16384 x 2 records; block scores of 64-token blocks; partition 256 x 32768 maps"},
            "kernels": out, "peak_kind": kind, "gpu_launches": args.steps * (4 + 1 + 1 + 3 + L + 1 + 1 + L + 2),
            "clocks": sampler.summary()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="rdkv_b200", choices=["rdkv_b200", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "decode-long", "pack", "alloc", "score", "aux"])
    ap.add_argument("--seq-parts", type=int, default=1,
                    help="decode-long: ranks that split the live rows of the same heads (1 = KV-head sharding only)")
    ap.add_argument("--persistent", type=int, default=None, choices=[0, 1],
                    help="force the per-item (0) or the persistent (1) form of the fused kernel")
    ap.add_argument("--no-also", action="store_true", help="default workload: skip the brief runs of the other configurations")
    ap.add_argument("--small", action="store_true", help="2 layers x batch 2 (smoke-sized case)")
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (profiling-sized runs)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--chunks", type=int, default=None, help="force this many chunks per (view, KV head) (default: planned)")
    ap.add_argument("--k-passes", type=int, default=0, choices=[0, 1, 3],
                    help="pack workload: K packed in one pass over the kept rows (1), in three (3), or as the library chooses (0)")
    ap.add_argument("--e2e-slices", type=int, default=None,
                    help="view ranges (streams) the host-buffer call overlaps its copies and kernels over")
    ap.add_argument("--e2e-graph", type=int, choices=(0, 1), default=None,
                    help="host-buffer call: 1 = replay a recorded graph, 0 = stream form (default: the call's own choice)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    global PERSISTENT
    PERSISTENT = None if args.persistent is None else bool(args.persistent)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        line = run_reference_arm(args, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    try:
        if args.workload == "decode":
            line = run_decode(args, rank, world, device)
        elif args.workload == "decode-long":
            line = run_decode_long(args, rank, world, device)
        elif args.workload == "pack":
            line = run_pack(args, rank, world, device)
        elif args.workload == "score":
            line = run_score(args, rank, world, device)
        elif args.workload == "aux":
            line = run_aux(args, rank, world, device)
        else:
            line = run_alloc(args, rank, world, device)
        if rank == 0 and line is not None:
            print(json.dumps(line), flush=True)
    finally:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
