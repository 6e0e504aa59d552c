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

CFG3 = dict(layers=32, batch=16, kv_heads=8, q_heads=32, context=32768, budget=2048, config_id=3)
L2_BYTES = 126 * 1024 * 1024
METRIC = "packed-KV decode-attn tokens/s"

# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of one fused-kernel launch in
# the committed ncu capture (profiles/; an 8-layer launch: 286.4 MB moved for 280.2 MB algorithmic);
# traffic grows with the units processed, so the ratio carries over to the full launch.
NCU_TRAFFIC_BYTES_PER_ALGO_BYTE = 1.022
# the same ratio for the four packing launches of config 1 (profiles/: 934.7 MB moved for 945.4 MB
# algorithmic; the launch list is a one-pass capture of the full workload)
PACK_NCU_TRAFFIC_BYTES_PER_ALGO_BYTE = 0.989


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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
def unit_bytes(pl, nv) -> int:
    """Algorithmic bytes of one packed (sequence, layer): live packed K and V rows, scale/zp, fp16 rows."""
    sb = pl.seg_bounds_per_head.cpu().tolist()
    n16 = pl.n_v16_per_head.cpu().tolist()
    k_row = sum(t.shape[-1] for t in (pl.K_2bit, pl.K_4bit, pl.K_8bit) if t is not None)
    total = 0
    for (n2, n4, n8), n in zip(sb, n16):
        rows = n2 + n4 + n8 + n
        total += rows * k_row + 2 * 2 * pl.K_ch_scale.shape[-1]
        total += n2 * 32 + n4 * 64 + n8 * 128 + (n2 + n4 + n8) * 4 + n * 256
    return total


def build_decode_cache(cfg, h0, h1, replica, device):
    """Packed cache of this rank's KV heads [h0,h1) for every (layer, sequence): synthetic K/V of
    the full context generated on the device from the unit's seed, bits prescribed by ranked
    lognormal importances, packed by the library's own (parity-checked) packer."""
    from rdkv_b200 import synth
    from rdkv_b200.packing import pack_kv
    g = cfg["q_heads"] // cfg["kv_heads"]
    layers, nvs, nbytes = [], [], 0
    for layer in range(cfg["layers"]):
        for seq in range(cfg["batch"]):
            seed = synth.unit_seed(cfg["config_id"], layer, seq) + 100003 * replica
            K, V = synth.make_kv(cfg["kv_heads"], cfg["context"], seed=seed, device=device)
            vb = synth.make_v_bits(cfg["kv_heads"], cfg["context"], cfg["budget"], seed=seed, device=device)
            kb = synth.make_k_bits(cfg["kv_heads"], seed=seed, device=device)
            pl, nv = pack_kv(K[:, h0:h1], V[:, h0:h1], vb[h0:h1], kb[h0:h1], g, build_mask=False)
            layers.append(pl)
            nvs.append(nv)
            nbytes += unit_bytes(pl, nv)
            del K, V
    return layers, nvs, nbytes


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


def run_decode(args, rank, world, device):
    from rdkv_b200._lib import lib
    from rdkv_b200.decode import DecodeTable, packed_decode_attention, packed_decode_attention_host
    cfg = dict(CFG3)
    if args.small:
        cfg.update(layers=2, batch=2, context=4096, budget=1024)
    if args.layers:
        cfg.update(layers=args.layers)
    H_kv = cfg["kv_heads"]
    assert H_kv % world == 0, "KV heads are sharded across ranks: world size must divide 8"
    h0, h1 = rank * H_kv // world, (rank + 1) * H_kv // world
    g = cfg["q_heads"] // H_kv
    Hq_loc = (h1 - h0) * g
    n_views = cfg["layers"] * cfg["batch"]
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)

    # enough distinct cache replicas that consecutive steps cannot be served from L2
    tables, step_bytes = [], None
    while True:
        layers, nvs, nbytes = build_decode_cache(cfg, h0, h1, len(tables), device)
        tables.append(DecodeTable(layers, nvs, Hq_loc, n_chunks=args.chunks))
        step_bytes = nbytes
        if len(tables) * nbytes >= 2.2 * L2_BYTES or args.small:
            break
    R = len(tables)
    gen = torch.Generator(device=device)
    gen.manual_seed(4242 + rank)
    n_q = min(args.steps + args.warmup, 64)
    q_pool = [(torch.randn(n_views, Hq_loc, 128, generator=gen, device=device) / 128 ** 0.5).to(torch.bfloat16)
              for _ in range(n_q)]
    out = torch.empty((n_views, Hq_loc, 128), dtype=torch.float32, device=device)

    def step(i):
        packed_decode_attention(q_pool[i % n_q], tables[i % R], out=out)

    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(device.index if device.index is not None else 0)
    with sampler:
        ms = timed_steps(step, args.steps, barrier)
    ms = max_over_ranks(ms, world, device)

    # per-kernel duration of the fused kernel (dominant) inside the same loop, for the roofline
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    with sampler:
        for i in range(args.steps):
            tb = tables[i % R]
            ev[i][0].record()
            packed_decode_attention(q_pool[i % n_q], tb, out=out)
            ev[i][1].record()
        torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    fused_ms = statistics.mean(a.elapsed_time(b) for a, b in ev)
    fused_ms = max_over_ranks(fused_ms, world, device)

    # end to end through the public call with host buffers: pinned q in, pinned out back, every step
    q_host = [q.cpu().pin_memory() for q in q_pool[:min(n_q, 8)]]
    q_dev = q_pool[0]
    out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()

    def e2e_step(i):
        # uploads the queries, runs the kernel and downloads the results in view ranges on
        # separate streams; returns when out_host holds the step's results
        packed_decode_attention_host(q_host[i % len(q_host)], tables[i % R], out_host, slices=args.e2e_slices)

    for i in range(min(args.warmup, 3)):
        e2e_step(i)
    with sampler:
        e2e_ms = timed_steps(e2e_step, args.steps, barrier)
    e2e_ms = max_over_ranks(e2e_ms, world, device)

    for tb in tables:
        tb.check_status()
    t0 = tables[0]
    v_main, k_rest, rows_rest = t0.unit_plan(t0.n_views)
    launches = 1
    if rank != 0:
        return None
    peak, peak_kind = load_peaks()
    tokens = cfg["batch"] * args.steps
    sec = ms / 1e3
    total_step_bytes = step_bytes * world            # every rank holds the same number of heads
    achieved = step_bytes / (fused_ms / 1e3) / 1e9   # per-GPU GB/s of the dominant kernel
    traffic = None if NCU_TRAFFIC_BYTES_PER_ALGO_BYTE is None else NCU_TRAFFIC_BYTES_PER_ALGO_BYTE * step_bytes
    line = {
        "metric": METRIC, "value": tokens / sec, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "u8 codes / fp16 scales, fp32 accumulate",
        "data": "synthetic",
        "config": {
            "workload": "config 3: full-depth decode, Llama-3.1-8B attention shape — 32 layers x batch 16 x "
                        "8 KV heads (32 q heads, head_dim 128), context 32768, 2048 kept tokens/head "
                        "(1/8 fp16, 1/4 8b, 3/8 4b, 1/4 2b), 64 K channels kept (16@8b,24@4b,24@2b), bf16 q per step",
            "batch": cfg["batch"], "layers": cfg["layers"], "kv_heads": H_kv, "q_heads": cfg["q_heads"],
            "token_budget": cfg["budget"], "context": cfg["context"],
            "parallelism": f"kv-head sharding x{world} (no data-path collective)",
            "launches_per_step": launches,
            "l2": f"{R} cache replica(s) rotated per step, {R * step_bytes / 2**20:.0f} MiB per GPU "
                  f"> 2 x 126 MiB L2; no flush needed",
            "small": bool(args.small or args.layers),
            "launch_shape": ("one CTA per (view, KV head)" if k_rest == 1
                             else f"{t0.plan(t0.n_views)[2]} (view, KV head) units whole, the other "
                                  f"{t0.n_views * (h1 - h0) - t0.plan(t0.n_views)[2]} in {k_rest} chunks of {rows_rest} "
                                  "rows merged in the kernel"),
        },
        "hbm_gbs": total_step_bytes * args.steps / sec / 1e9,
        "hbm_frac_of_8tbs": total_step_bytes * args.steps / sec / 1e9 / (8000.0 * world),
        "algorithmic_bytes_per_step": total_step_bytes,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": traffic, "peak_kind": peak_kind,
                     "kernel": "decode_fused_kernel", "kernel_ms": fused_ms,
                     "algorithmic_bytes_per_launch": step_bytes},
        "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s",
                "h2d_bytes_per_step": q_dev.numel() * q_dev.element_size() * world,
                "d2h_bytes_per_step": out.numel() * out.element_size() * world,
                "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": launches * args.steps,
        "clocks": sampler.summary(),
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_decode_baseline(cfg, tables[0], layers_per_sample=1, steps=2)
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
    """The reference's CPU path (numpy restatement under oracle/) on the host cores, rank 0 only."""
    if rank != 0:
        return None
    import numpy as np
    from oracle import ref_packing as RP
    from rdkv_b200 import synth
    cfg = dict(CFG3)
    if args.small:
        cfg.update(layers=2, batch=2, context=4096, budget=1024)
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
        "config": {"workload": "config 3 decode (same as the CUDA arm)", "batch": cfg["batch"],
                   "layers": cfg["layers"], "kv_heads": cfg["kv_heads"], "q_heads": cfg["q_heads"],
                   "token_budget": cfg["budget"], "context": cfg["context"], "small": bool(args.small)},
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
        state["batch"] = pack_kv_layers(Ks, Vs, v_bits, k_bits, 4, build_mask=False)

    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(device.index or 0)
    with sampler:
        ms = timed_steps(step, args.steps, lambda: None)
    sec = ms / 1e3 / args.steps
    # the three packing launches alone (device time of the dominant kernels), for the roofline
    spans = []
    torch.cuda.profiler.start()
    for i in range(args.steps):
        state["batch"] = pack_kv_layers(Ks, Vs, v_bits, k_bits, 4, build_mask=False, launch_events=spans)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    kern_ms = statistics.mean(a.elapsed_time(b) for a, b in spans)
    out_bytes = 0
    for pl, nv in state["batch"]:
        out_bytes += sum(t.numel() * t.element_size() for t in
                         (pl.K_2bit, pl.K_4bit, pl.K_8bit, pl.V_2bit, pl.V_4bit, pl.V_8bit, pl.V_scale,
                          pl.V_zp, pl.K_ch_scale, pl.K_ch_zp, nv) if t is not None)
    nominal = L * H * T * 128 * 2 * 2                       # all fp16 K and V bytes of the context
    # kept rows of V read once, kept rows of K read twice (extrema pass, quantise pass), packed bytes written
    moved = L * H * N * 256 * 3 + out_bytes
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
                         "traffic": moved * PACK_NCU_TRAFFIC_BYTES_PER_ALGO_BYTE, "peak_kind": kind,
                         "kernel": "pack_v128_batched_kernel + pack_k_minmax128_batched_kernel + pack_k_params_batched_kernel + pack_k_quant_batched_kernel",
                         "kernel_ms": kern_ms, "algorithmic_bytes_per_step": moved},
            "gpu_launches": 6 * args.steps, "clocks": sampler.summary()}
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
    from rdkv_b200.scoring import _score_one_layer, apply_score_pooling
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
    return {"metric": "importance scoring + pooling, layers/s", "value": 1.0 / sec, "unit": "layers/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp16 in, fp32 accumulate", "data": "synthetic",
            "config": {"workload": "score one layer: aw [1,8,4,32,32768] fp16, K [1,8,32768,128] fp16, avg-5 reflect pooling",
                       "l2": "4 input sets of 201 MB rotated > L2"},
            "roofline": {"bound": "hbm", "achieved": moved / sec / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": moved / sec / 1e9 / peak, "traffic": None, "peak_kind": kind,
                         "kernel": "token_score_kernel + channel_ksq_kernel + pool_kernel (whole step, 5 launches)",
                         "algorithmic_bytes_per_step": moved},
            "gpu_launches": 4 * args.steps, "clocks": sampler.summary()}


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="rdkv_b200", choices=["rdkv_b200", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "pack", "alloc", "score"])
    ap.add_argument("--small", action="store_true", help="2 layers x batch 2 (smoke-sized case)")
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (profiling-sized runs)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--chunks", type=int, default=None, help="force this many chunks per (view, KV head) (default: planned)")
    ap.add_argument("--e2e-slices", type=int, default=None,
                    help="view ranges (streams) the host-buffer call overlaps its copies and kernels over")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
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
        elif args.workload == "pack":
            line = run_pack(args, rank, world, device)
        elif args.workload == "score":
            line = run_score(args, rank, world, device)
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
