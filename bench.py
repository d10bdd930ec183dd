#!/usr/bin/env python
"""Benchmark of the KV-cache data path: multi-layer paged-KV swap over PCIe (headline) and the
paged gather in HBM (secondary, single-GPU runs).

    python bench.py --gpus N --steps K --warmup W          # this implementation
    python bench.py --impl reference ...                    # the CPU restatement on the host cores

A *step* is one pass of the hot path over one batch: one swap-out call (HBM -> pinned host pool)
and one swap-in call (host pool -> HBM, other device blocks) of the workload's block count, all
layers, K and V.  Each rank owns its own cache, pool and PCIe link; there is no collective on the
data path, so scaling is weak (per-GPU work fixed).  torch.distributed is used only for the start
barrier and the max-over-ranks reduction of the device-side time.

Prints ONE JSON line (rank 0).  `value` is the whole-job GB/s of the Llama-3-8B step with the id
lists resident on the device; `e2e` drives the same step through the public API
(PagedKVCache.swap_out / swap_in) with host-resident id lists and reads the status word back every
step.  Every timed leg is followed by a byte-for-byte check of what its last step moved
(`verified`).  The same line carries short runs of the other configurations as flat objects:
`config4` (Llama-3-70B TP8 shard, every N), `overlap` (layer-wise prefetch next to a GEMM, N = 1)
and `gather` (paged gather, N = 1); the scalars a reader needs first are repeated inside `roofline`.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

from heterofusedkernels_b200 import workloads as wl  # noqa: E402

GB = 1e9


# --------------------------------------------------------------------------- workloads
def geometry(name: str):
    """Shapes of the benchmark configurations (seeded synthetic data stands in for serving traffic)."""
    from types import SimpleNamespace as NS

    fp8 = getattr(torch, "float8_e4m3fn", torch.uint8)
    table = {
        "llama3_8b_swap": NS(layers=32, num_blocks=20000, block_size=16, kv_heads=8, head_dim=128,
                             dtype=torch.bfloat16, host_slots=40000, n_swap=512),
        "llama3_70b_tp8_swap": NS(layers=80, num_blocks=6000, block_size=128, kv_heads=1, head_dim=128,
                                  dtype=torch.bfloat16, host_slots=24000, n_swap=2048),
        "qwen2_7b_fp8_swap": NS(layers=28, num_blocks=8192, block_size=16, kv_heads=4, head_dim=128,
                                dtype=fp8, host_slots=16384, n_swap=256),
        "qwen2_7b_fp8_prefetch": NS(layers=28, num_blocks=8192, block_size=16, kv_heads=4, head_dim=128,
                                    dtype=fp8, host_slots=16384, n_swap=256),
        "block_transfer": NS(layers=1, num_blocks=1, block_size=1, kv_heads=1, head_dim=128, dtype=torch.int8,
                             host_slots=1, n_swap=1),
        "embedding_gather": NS(layers=1, num_blocks=1, block_size=1, kv_heads=1, head_dim=512, dtype=torch.float16,
                               host_slots=1, n_swap=1),
        "migrate": NS(layers=32, num_blocks=4096, block_size=16, kv_heads=8, head_dim=128,
                      dtype=torch.bfloat16, host_slots=0, n_swap=512),
        "tiny": NS(layers=2, num_blocks=64, block_size=16, kv_heads=8, head_dim=128, dtype=torch.float16,
                   host_slots=128, n_swap=8),
    }
    g = table[name]
    g.name = name
    g.elt = torch.empty((), dtype=g.dtype).element_size()
    g.block_bytes = g.block_size * g.kv_heads * g.head_dim * g.elt
    g.swap_bytes = g.n_swap * g.layers * 2 * g.block_bytes
    return g


def mem_available_bytes() -> int:
    for line in Path("/proc/meminfo").read_text().splitlines():
        if line.startswith("MemAvailable:"):
            return int(line.split()[1]) * 1024
    return 0


def fill_random_bytes(t: torch.Tensor, seed: int) -> None:
    """Cheap seeded fill on the device: random bytes (for fp8 without the NaN codes 0x7F/0xFF)."""
    gen = torch.Generator(device=t.device).manual_seed(seed)
    flat = t.view(torch.uint8).view(-1)
    step = 1 << 30
    for i in range(0, flat.numel(), step):
        part = flat[i:i + step]
        part.copy_(torch.randint(0, 254, part.shape, dtype=torch.uint8, device=t.device, generator=gen))
        if t.element_size() == 1:
            part += (part >= 0x7F).to(torch.uint8)


def traffic_ratio(kernel: str, default: float) -> tuple:
    """DRAM bytes per algorithmic byte of a kernel, from the tracked summary of its ncu capture."""
    try:
        entry = json.loads((ROOT / "profiles" / "traffic.json").read_text())[kernel]
        return float(entry["dram_bytes_per_algorithmic_byte"]), entry["source"]
    except (OSError, KeyError, ValueError):
        return default, "profiles/traffic.json missing: ratio assumed"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 100 ms in the background."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU baseline
def cpu_baseline_swap(g, steps: int, warmup: int, budget_s: float = 25.0) -> dict:
    """The torch CPU restatement (index_select / index_copy_ per layer) on the host cores.

    Sample: the full step's bytes (n_swap blocks, every layer, K and V, out then in) on a cache and a
    pool shrunk to 2*n_swap blocks, so only the pools are smaller, not the bytes moved."""
    from oracle import kv_oracle as o

    # launchers such as torchrun export OMP_NUM_THREADS=1; the CPU arm uses every host core
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    nb = 2 * g.n_swap
    shape = (nb, g.block_size, g.kv_heads, g.head_dim)
    store = torch.empty((2, g.layers) + shape[:1] + (g.block_bytes,), dtype=torch.uint8)
    store.random_(0, 254, generator=torch.Generator().manual_seed(0))
    dev_k = list(store[0].unbind(0))
    dev_v = list(store[1].unbind(0))
    pool = torch.zeros((nb, g.layers, 2, g.block_bytes), dtype=torch.uint8)
    times = []
    t_start = time.perf_counter()
    for s in range(warmup + steps):
        ids = wl.distinct_ids(g.n_swap, nb, 10 + s)
        slots = wl.distinct_ids(g.n_swap, nb, 20 + s)
        back = wl.distinct_ids(g.n_swap, nb, 30 + s)
        t0 = time.perf_counter()
        o.swap_out(dev_k, dev_v, pool, ids, slots)
        o.swap_in(dev_k, dev_v, pool, back, slots)
        dt = time.perf_counter() - t0
        if s >= warmup:
            times.append(dt)
        if time.perf_counter() - t_start > budget_s and len(times) >= 1:
            break
    mean = sum(times) / len(times)
    return {"value": 2 * g.swap_bytes / mean / GB, "unit": "GB/s", "cores": torch.get_num_threads(),
            "host_cpus": os.cpu_count(), "kind": "port",
            "sample": (f"{len(times)} full steps ({g.n_swap} blocks x {g.layers} layers x K,V, out then in = "
                       f"{2 * g.swap_bytes} bytes each) on a cache and pool shrunk to {nb} blocks; torch CPU "
                       "index_select/index_copy_ per layer"),
            "ms_per_step": mean * 1e3, "steps": len(times)}


# --------------------------------------------------------------------------- PCIe peak
def measure_pcie_peak(pool_u8: torch.Tensor, device) -> dict:
    """Best-of-5 cudaMemcpyAsync of up to 1 GiB between the pinned pool and device memory."""
    n = min(pool_u8.numel(), 1 << 30)
    host = pool_u8[:n]
    dev = torch.empty(n, dtype=torch.uint8, device=device)
    res = {}
    for name, dst, src in (("h2d", dev, host), ("d2h", host, dev)):
        best = 0.0
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            dst.copy_(src, non_blocking=True)
            b.record()
            b.synchronize()
            best = max(best, n / (a.elapsed_time(b) * 1e-3) / GB)
        res[name] = best
    res["bytes"] = n
    res["pinned"] = bool(host.is_pinned())
    del dev
    return res


def measure_pcie_concurrent(ctx, pool_u8: torch.Tensor, device) -> dict:
    """cudaMemcpyAsync rates with EVERY rank copying at the same time, after a barrier: 8 back-to-back
    copies of 1 GiB in one direction (h2d, d2h), and 4 + 4 copies in both directions at once on two
    streams (bidir: both directions' bytes over the time until both are done).  These are the
    denominators for N > 1: what the host (root complexes, memory) gives N links at once, as opposed
    to one link alone."""
    n = min(pool_u8.numel() // 2, 1 << 30)
    host, host2 = pool_u8[:n], pool_u8[n:2 * n]
    dev = torch.empty(n, dtype=torch.uint8, device=device)
    dev2 = torch.empty(n, dtype=torch.uint8, device=device)
    res = {}
    for name, dst, src in (("h2d", dev, host), ("d2h", host, dev)):
        dst.copy_(src, non_blocking=True)
        ctx.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(8):
            dst.copy_(src, non_blocking=True)
        b.record()
        b.synchronize()
        res[name] = 8 * n / (a.elapsed_time(b) * 1e-3) / GB
        ctx.barrier()
    s1, s2 = torch.cuda.Stream(device), torch.cuda.Stream(device)
    main = torch.cuda.current_stream(device)
    ctx.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    s1.wait_event(a)
    s2.wait_event(a)
    with torch.cuda.stream(s1):
        for _ in range(4):
            host.copy_(dev, non_blocking=True)       # d2h
    with torch.cuda.stream(s2):
        for _ in range(4):
            dev2.copy_(host2, non_blocking=True)     # h2d
    main.wait_stream(s1)
    main.wait_stream(s2)
    b.record()
    b.synchronize()
    res["bidir_total"] = 8 * n / (a.elapsed_time(b) * 1e-3) / GB
    ctx.barrier()
    del dev, dev2
    return res


# --------------------------------------------------------------------------- verification
def _pool_bytes(cache) -> torch.Tensor:
    """[slots, layers, 2, block_bytes] byte view of the host pool."""
    return cache.host_pool.view(torch.uint8).view(cache.host_slots, cache.layers, 2, cache.block_bytes)


def _cache_bytes(cache, kv: int, layer: int) -> torch.Tensor:
    t = (cache.v_caches if kv else cache.k_caches)[layer]
    return t.view(torch.uint8).view(cache.num_blocks, cache.block_bytes)


def verify_swap(cache, pairs, layers=None) -> dict:
    """Byte-for-byte check of swapped data: for every (device ids, host slots) pair list, every layer
    and K and V, cache[block] must equal pool[slot].  The device blocks are compared with the host
    slots on the device, 64 MiB at a time; a small sample also goes through the CPU oracle."""
    from oracle import kv_oracle as o

    pool = _pool_bytes(cache)
    layers = range(cache.layers) if layers is None else layers
    bad, checked = [], 0
    for name, dev_ids, slots in pairs:
        dev_ids_d = dev_ids.to(cache.device)
        slots_c = slots.cpu()
        for l in layers:
            for kv in (0, 1):
                want = pool[:, l, kv].index_select(0, slots_c).to(cache.device, non_blocking=True)
                got = _cache_bytes(cache, kv, l).index_select(0, dev_ids_d)
                checked += want.numel()
                if not torch.equal(got, want):
                    bad.append((name, l, kv))
        # the oracle on a sample: three blocks, first and last layer
        n = min(3, dev_ids.numel())
        ls = sorted({layers[0], layers[-1]}) if len(layers) else []
        if n and ls:
            small_k = [_cache_bytes(cache, 0, l).index_select(0, dev_ids_d[:n]).cpu() for l in ls]
            small_v = [_cache_bytes(cache, 1, l).index_select(0, dev_ids_d[:n]).cpu() for l in ls]
            ref = torch.zeros((n, len(ls), 2, cache.block_bytes), dtype=torch.uint8)
            o.swap_out(small_k, small_v, ref, torch.arange(n), torch.arange(n))
            have = pool.index_select(0, slots_c[:n])[:, ls]
            if not torch.equal(ref, have):
                bad.append((name, "oracle sample"))
    torch.cuda.synchronize(cache.device)
    return {"verified": not bad, "bytes_checked": checked, "mismatches": bad[:8]}


# --------------------------------------------------------------------------- the swap step
class SwapBench:
    """One rank's swap workload: the cache, the pool, the per-step id sets and the ways to run a step.

    Set 0 primes the pool (one untimed swap-out); step s >= 1 uses set s: swap-out of o_ids[s] into
    slots[s] and swap-in into i_ids[s] (other blocks) from slots[s] ("own": the blocks just swapped
    out come back) or from slots[s-1] ("prev": the blocks swapped out one step earlier come back,
    which lets the two directions of a step run independently).

    Variants (`--variant`):
      sequential  swap-out then swap-in of the same slots, one stream (N = 1 default)
      stagger     even ranks as sequential; odd ranks swap-in (prev) first, then swap-out
      bidir       swap-out and swap-in (prev) concurrently on two streams
      bidir_paced the same with the swap-out's stores paced (PagedKVCache.BIDIR_OUT_PACE_GBS), which
                  keeps the swap-in's read requests from being crowded out of the upstream lanes
      interleave:k  the step's lists cut into k parts, out/in parts alternating on one stream
                    (odd ranks: in (prev) first)
    """

    def __init__(self, g, cache, ctx, pkg, n_sets: int, mover, aiv, staging_mb: int, slot_runs: int = 0):
        self.g, self.cache, self.ctx, self.pkg = g, cache, ctx, pkg
        self.mover, self.aiv, self.staging_bytes = mover, aiv, staging_mb << 20
        from heterofusedkernels_b200 import ranks

        self.sets = ranks.rank_id_sets(ctx.rank, n_sets + 1, g.n_swap, g.num_blocks, cache.host_slots)
        if slot_runs:
            # the slots of a step form runs of `slot_runs` consecutive slots at seeded random places, as a
            # free list hands them out (HostSlotPool); consecutive steps use different cells of the grid
            run = min(int(slot_runs), g.n_swap)
            cells = cache.host_slots // run
            need = (g.n_swap + run - 1) // run
            assert cells >= 2 * need, "host pool too small for disjoint runs"
            gen = torch.Generator().manual_seed(99 + ctx.rank)
            new_sets = []
            for s, (o_ids, _, i_ids) in enumerate(self.sets):
                pick = torch.randperm(cells // 2, generator=gen)[:need] * 2 + (s % 2)
                slots = (pick.unsqueeze(1) * run + torch.arange(run).unsqueeze(0)).reshape(-1)[:g.n_swap]
                new_sets.append((o_ids, slots, i_ids))
            self.sets = new_sets
        self.dev_sets = [tuple(t.to(cache.device) for t in s) for s in self.sets]
        self.pin_sets = [tuple(t.pin_memory() for t in s) for s in self.sets]
        self.side = [torch.cuda.Stream(cache.device), torch.cuda.Stream(cache.device)]
        self.pace = None           # GB/s of the swap-outs of the running variant (bidir_paced)
        self.launches = 0          # swap calls issued so far
        self.launches_timed = 0    # ... of which inside the last run's timed region

    # one call each way; ids: device tensors (value leg) or pinned host tensors (e2e leg)
    def _out(self, ids, slots, slots_cpu):
        self.launches += 1
        if self.pace:
            self.cache.swap_out(ids, slots, aiv=self.aiv, mover=None if isinstance(self.mover, str) else self.mover,
                                pace_gbs=self.pace)
        elif isinstance(self.mover, str) and self.mover.startswith("hybrid"):
            self.cache.swap_out(ids, slots_cpu, aiv=self.aiv, mover=self.mover)
        elif self.mover == "staged":
            self.cache.swap_out_staged(ids, slots_cpu, staging_bytes=self.staging_bytes, aiv=self.aiv)
        else:
            self.cache.swap_out(ids, slots, aiv=self.aiv, mover=self.mover)

    def _in(self, ids, slots, slots_cpu):
        self.launches += 1
        if isinstance(self.mover, str) and self.mover.startswith("hybrid"):
            self.cache.swap_in(ids, slots_cpu, aiv=self.aiv, mover=self.mover)
        elif self.mover == "staged":
            self.cache.swap_in_staged(ids, slots_cpu, staging_bytes=self.staging_bytes, aiv=self.aiv)
        else:
            self.cache.swap_in(ids, slots, aiv=self.aiv, mover=self.mover)

    def prime(self):
        o_ids, slots, _ = self.dev_sets[0]
        self._out(o_ids, slots, self.sets[0][1])
        torch.cuda.synchronize(self.cache.device)

    def plan(self, variant: str):
        """(in_source, order, parts, two_streams) of this rank for a variant."""
        odd = self.ctx.world > 1 and self.ctx.rank % 2 == 1
        if variant == "sequential":
            return "own", "out_first", 1, False
        if variant == "stagger":
            return ("prev", "in_first", 1, False) if odd else ("own", "out_first", 1, False)
        if variant in ("bidir", "bidir_paced"):
            return "prev", "out_first", 1, True
        if variant.startswith("interleave:"):
            k = max(1, int(variant.split(":")[1]))
            return ("prev", "in_first", k, False) if odd else ("own", "out_first", k, False)
        raise ValueError(f"unknown variant {variant}")

    def run(self, variant: str, steps: int, warmup: int, e2e: bool) -> dict:
        """Runs warmup + steps steps (sets 1..warmup+steps); returns this rank's timings and the
        verification of the last step."""
        cache, ctx = self.cache, self.ctx
        src_mode, order, parts, two = self.plan(variant)
        self.pace = type(cache).BIDIR_OUT_PACE_GBS if variant == "bidir_paced" else None
        use = self.pin_sets if e2e else self.dev_sets
        main = torch.cuda.current_stream(cache.device)
        t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        out_ev, in_ev = [], []
        self.prime()
        status_acc = 0
        for s in range(1, warmup + steps + 1):
            o_ids, slots, i_ids = use[s]
            src_slots = slots if src_mode == "own" else use[s - 1][1]
            src_slots_cpu = self.sets[s][1] if src_mode == "own" else self.sets[s - 1][1]
            if s == warmup + 1:
                ctx.barrier()
                t_start.record()
                launches_before = self.launches
            timed = s > warmup
            if two:
                fork = torch.cuda.Event()
                fork.record()
                evs = []
                for stream, fn, args in ((self.side[0], self._out, (o_ids, slots, self.sets[s][1])),
                                         (self.side[1], self._in, (i_ids, src_slots, src_slots_cpu))):
                    stream.wait_event(fork)
                    with torch.cuda.stream(stream):
                        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        a.record()
                        fn(*args)
                        b.record()
                    evs.append((a, b))
                main.wait_stream(self.side[0])
                main.wait_stream(self.side[1])
                if timed:
                    out_ev.append([evs[0]])
                    in_ev.append([evs[1]])
            else:
                n = o_ids.numel()
                cuts = [(n * j) // parts for j in range(parts + 1)]
                step_out, step_in = [], []
                for j in range(parts):
                    lo, hi = cuts[j], cuts[j + 1]
                    calls = [("out", self._out, (o_ids[lo:hi], slots[lo:hi], self.sets[s][1][lo:hi])),
                             ("in", self._in, (i_ids[lo:hi], src_slots[lo:hi], src_slots_cpu[lo:hi]))]
                    if order == "in_first":
                        calls.reverse()
                    for kind, fn, args in calls:
                        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        a.record()
                        fn(*args)
                        b.record()
                        (step_out if kind == "out" else step_in).append((a, b))
                if timed:
                    out_ev.append(step_out)
                    in_ev.append(step_in)
            if e2e:
                status_acc |= cache.status()    # device -> host read of the step's result
        t_end.record()
        self.launches_timed = self.launches - launches_before
        ctx.barrier()
        status = status_acc | cache.status()
        last = warmup + steps
        o_ids, slots, i_ids = self.sets[last]
        src = slots if src_mode == "own" else self.sets[last - 1][1]
        ver = verify_swap(cache, [("swap_out", o_ids, slots), ("swap_in", i_ids, src)])
        out_ms = [sum(a.elapsed_time(b) for a, b in st) for st in out_ev]
        in_ms = [sum(a.elapsed_time(b) for a, b in st) for st in in_ev]
        return {"local_ms_per_step": t_start.elapsed_time(t_end) / steps, "out_ms": out_ms, "in_ms": in_ms,
                "status": status, "verified": ver["verified"] and status == 0, "verify": ver,
                "plan": {"swap_in_source": src_mode, "order": order, "parts": parts, "two_streams": two}}


# --------------------------------------------------------------------------- gather leg
def bench_gather(device, steps: int, warmup: int, mover, aiv, num_seqs: int = 64) -> dict:
    """Paged gather, Llama-3-8B layout: 64 sequences of 512..8192 tokens (seeded), block tables that are
    disjoint slices of a seeded permutation of a 40000-block cache, all 32 layers, K and V, one launch.
    After the timed launches every sequence of every layer, K and V, is compared with a device-side
    index_select of the same pages."""
    from heterofusedkernels_b200.connector import PagedKVCache

    layers, nblocks, bs, heads, hd = 32, 40000, 16, 8, 128
    lens = wl.gather_seq_lens(seed=0)[:num_seqs]
    total = sum(lens)
    if num_seqs < 64:  # reduced batch (profiling): a cache just large enough for it
        nblocks = sum((n + bs - 1) // bs for n in lens) + 256
    token_bytes = heads * hd * 2
    need = 2 * layers * nblocks * bs * token_bytes + 2 * layers * total * token_bytes
    free, _ = torch.cuda.mem_get_info(device)
    note = ""
    if need > free - (4 << 30):
        nblocks = max(sum((n + bs - 1) // bs for n in lens) + 1,
                      int((free - (6 << 30) - 2 * layers * total * token_bytes) // (2 * layers * bs * token_bytes)))
        note = f"cache shrunk to {nblocks} blocks to fit free HBM"
    cache = PagedKVCache(layers, nblocks, bs, heads, hd, torch.bfloat16, device)
    fill_random_bytes(cache._k_store, 1)
    fill_random_bytes(cache._v_store, 2)
    tables_cpu = wl.block_tables_for(lens, bs, nblocks, seed=1)
    tables = tables_cpu.to(device)
    lens_t = torch.tensor(lens, device=device)
    k_out = torch.empty((layers, total, heads, hd), dtype=torch.bfloat16, device=device)
    v_out = torch.empty_like(k_out)
    algo = 2 * total * token_bytes * 2 * layers  # read + write of K and V outputs
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s in range(warmup + steps):
        if s >= warmup:
            ev[s - warmup][0].record()
        cache.paged_gather(tables, lens_t, k_out, v_out, aiv=aiv, mover=mover)
        if s >= warmup:
            ev[s - warmup][1].record()
    torch.cuda.synchronize()
    ms = [a.elapsed_time(b) for a, b in ev]
    status = cache.status()
    # full check: token t of the batch lives in cache row block*block_size + offset
    rows = []
    for s, n in enumerate(lens):
        nb = (n + bs - 1) // bs
        r = (tables_cpu[s, :nb].unsqueeze(1) * bs + torch.arange(bs).unsqueeze(0)).reshape(-1)[:n]
        rows.append(r)
    rows = torch.cat(rows).to(device)
    bad = []
    for l in range(layers):
        for name, caches, out in (("K", cache.k_caches, k_out), ("V", cache.v_caches, v_out)):
            ref = caches[l].view(torch.int16).view(nblocks * bs, heads * hd).index_select(0, rows)
            if not torch.equal(ref, out[l].view(torch.int16).view(total, heads * hd)):
                bad.append((l, name))
    mean_ms = sum(ms) / len(ms)
    res = {"workload": "llama3_8b_gather", "total_tokens": total, "num_seqs": len(lens), "layers": layers,
           "cache_blocks": nblocks, "algorithmic_bytes": algo, "ms_per_launch": mean_ms, "best_ms": min(ms),
           "value": algo / (mean_ms * 1e-3) / GB, "unit": "GB/s", "status_word": status,
           "verified": not bad and status == 0,
           "verify": {"what": f"all {len(lens)} sequences x {layers} layers x K,V against a device-side index_select",
                      "bytes_checked": 2 * layers * total * token_bytes, "mismatches": bad[:8]},
           "note": note}
    del cache, k_out, v_out
    torch.cuda.empty_cache()
    return res


# --------------------------------------------------------------------------- embedding-lookup leg
def bench_embedding_gather(device, args, pkg) -> dict:
    """The regime the reference publishes gather numbers for (pcieThrough/tests/test_gather.py,
    test_gather_combine.py, tests/README.md): fp16 rows of 512 elements (1 KiB) looked up in a 4 M-row
    (4 GiB) pinned host table, batches of 16..1024 ids, end-to-end host time over many calls.
    Three ways of issuing: one op call per batch, one call for a 10x batch ("combine"), and a CUDA graph
    of 10 calls replayed."""
    rows_n, dim = 4_000_000, 512
    table = pkg.memory.alloc_numa_pinned_tensor(rows_n * dim * 2).view(torch.float16).view(rows_n, dim)
    table.view(torch.int64).view(-1).copy_(torch.arange(rows_n * dim // 4, dtype=torch.int64))  # every row distinct
    op = torch.ops.pcie_through.gather
    run_count = 300
    out_rows = []
    gen = torch.Generator().manual_seed(0)
    for bs in (16, 32, 64, 128, 256, 512, 1024):
        ids = torch.randint(0, rows_n, (run_count, bs), generator=gen, dtype=torch.int64).to(device)
        dst = torch.empty((bs, dim), dtype=torch.float16, device=device)
        row = {"batch": bs}
        for label, aiv in (("default", None), ("aiv4", 4)):
            for r in range(20):
                op(table, dst, ids[r], aiv)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for r in range(run_count):
                op(table, dst, ids[r], aiv)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            row[f"per_call_ms_per_10_{label}"] = dt / run_count * 10 * 1e3
            row[f"per_call_GBps_{label}"] = bs * run_count * dim * 2 / dt / GB
        ok = torch.equal(dst.cpu().view(torch.int16), table[ids[run_count - 1].cpu()].view(torch.int16))
        # combine: 10x the ids in one call
        big_ids = ids.view(run_count // 10, 10 * bs)
        big_dst = torch.empty((10 * bs, dim), dtype=torch.float16, device=device)
        for label, aiv in (("", None), ("_aiv8", 8), ("_aiv16", 16), ("_aiv64", 64)):
            for r in range(5):
                op(table, big_dst, big_ids[r], aiv)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for r in range(run_count // 10):
                op(table, big_dst, big_ids[r], aiv)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            row["combine_ms_per_call" + label] = dt / (run_count // 10) * 1e3
            row["combine_GBps" + label] = bs * run_count * dim * 2 / dt / GB
        ok = ok and torch.equal(big_dst.cpu().view(torch.int16),
                                table[big_ids[run_count // 10 - 1].cpu()].view(torch.int16))
        # CUDA graph of 10 calls (ten different id rows), replayed
        side = torch.cuda.Stream(device)
        dsts = [torch.empty_like(dst) for _ in range(10)]
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for r in range(10):
                op(table, dsts[r], ids[r], None)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for r in range(10):
                    op(table, dsts[r], ids[r], None)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(run_count // 10):
            graph.replay()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        row["graph_ms_per_10"] = dt / (run_count // 10) * 1e3
        row["graph_GBps"] = bs * run_count * dim * 2 / dt / GB
        ok = ok and torch.equal(dsts[9].cpu().view(torch.int16), table[ids[9].cpu()].view(torch.int16))
        row["verified"] = bool(ok)
        out_rows.append(row)
    status = int(torch.ops.pcie_through.device_status())
    best = max(r["combine_GBps"] for r in out_rows)
    return {"metric": "embedding_gather_GBps", "value": best, "unit": "GB/s", "n_gpus": 1, "steps": run_count,
            "warmup": 20, "ms_per_step": None, "higher_is_better": True, "dtype": "u8", "data": "synthetic",
            "config": {"workload": "embedding_gather", "table_rows": rows_n, "row_bytes": dim * 2,
                       "table": "4 GiB pinned, device-mapped host memory", "calls_per_batch_size": run_count},
            "rows": out_rows, "status_word": status, "gpu_launches": run_count,
            "reference_published_ascend_910c": {
                "source": "pcieThrough/tests/README.md:36-42 (ms per 10 calls / GB/s; combine: ms per call / GB/s)",
                "gather_aiv4": {"16": [0.114, 1.43], "32": [0.108, 3.04], "64": [0.108, 6.09], "128": [0.107, 12.20],
                                "256": [0.121, 21.59], "512": [0.211, 24.11], "1024": [0.404, 25.98]},
                "combine": {"16": [0.011, 15.82], "32": [0.014, 22.99], "64": [0.026, 25.22], "128": [0.049, 26.96],
                            "256": [0.049, 26.96], "512": [0.181, 28.93], "1024": [0.357, 29.29]}}}


# --------------------------------------------------------------------------- single-block transfer leg
def bench_block_transfer(device, args, pkg) -> dict:
    """The reference's KV transfer measurement (pcieThrough/tests/test_transfer_kernel.py:50-88,
    tests/README.md:64-75): int8 blocks [1024, L, H, 128] moved host->device one op per block with the
    [B,L,H,D] -> L x [H,B,D] re-layout, two alternating streams, per-op bandwidth from events; plus the
    multi-block form (swap_in_relayout / swap_out_relayout), 16 blocks per call."""
    op = torch.ops.pcie_through
    rows = []
    for (B, L, H, D) in ((1024, 32, 1, 128), (1024, 32, 8, 128), (1024, 64, 1, 128), (1024, 64, 8, 128)):
        nbytes = B * L * H * D
        host_blocks, dev_blocks, n_ops = 24, 16, 16
        raw = pkg.memory.alloc_numa_pinned_tensor(host_blocks * nbytes)
        raw.view(torch.int64).copy_(torch.arange(raw.numel() // 8, dtype=torch.int64))
        pool = raw.view(host_blocks, B, L, H, D)
        dev = torch.zeros((L, dev_blocks, H, B, D), dtype=torch.int8, device=device)
        ptr_tabs = [torch.tensor([dev[l, i].data_ptr() for l in range(L)], dtype=torch.int64).to(device)
                    for i in range(dev_blocks)]
        layer_ptrs = torch.tensor([dev[l].data_ptr() for l in range(L)], dtype=torch.int64).to(device)
        streams = [torch.cuda.Stream(device) for _ in range(2)]
        staging = [torch.empty((B, L, H, D), dtype=torch.int8, device=device) for _ in range(2)]
        row = {"block": [B, L, H, D], "bytes_per_op": nbytes}
        for fused in (False, True):
            for aiv_label, aiv, n_streams in (("default", None, 2), ("aiv4", 4, 2), ("one_stream", None, 1)):
                best = 0.0
                for rep in range(3):
                    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                           for _ in range(n_ops)]
                    torch.cuda.synchronize()
                    for i in range(n_ops):
                        with torch.cuda.stream(streams[i % n_streams]):
                            evs[i][0].record()
                            if fused:
                                op.fused_memcpy_multi_layer_block_transfer(ptr_tabs[i], pool[i], staging[i % 2], aiv)
                            else:
                                op.multi_layer_block_transfer(ptr_tabs[i], pool[i], aiv)
                            evs[i][1].record()
                    torch.cuda.synchronize()
                    ms = sum(a.elapsed_time(b) for a, b in evs) / n_ops   # the reference's formula (:86-88)
                    best = max(best, nbytes / (ms * 1e6))
                row[("fused_memcpy" if fused else "zero_copy") + "_GBps_" + aiv_label] = best
        ok = torch.equal(pool[3], dev[:, 3].cpu().permute(2, 0, 1, 3))
        # multi-block form: all 16 blocks in one call, both directions
        ids = torch.arange(dev_blocks, device=device)
        slots = torch.arange(dev_blocks, device=device) + 4
        for name, fn in (("swap_in_relayout", op.swap_in_relayout), ("swap_out_relayout", op.swap_out_relayout)):
            best = 0.0
            for rep in range(4):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn(layer_ptrs, pool, ids, slots, dev_blocks)
                b.record()
                b.synchronize()
                best = max(best, dev_blocks * nbytes / (a.elapsed_time(b) * 1e6))
            row[name + "_16_blocks_GBps"] = best
        ok = ok and torch.equal(pool[4 + 5], dev[:, 5].cpu().permute(2, 0, 1, 3))
        row["verified"] = bool(ok)
        rows.append(row)
        del raw, pool, dev, staging
        torch.cuda.empty_cache()
    return {"metric": "block_transfer_GBps", "value": max(r["zero_copy_GBps_default"] for r in rows), "unit": "GB/s",
            "n_gpus": 1, "steps": 16, "warmup": 0, "ms_per_step": None, "higher_is_better": True, "dtype": "u8",
            "data": "synthetic", "config": {"workload": "block_transfer", "dtype": "int8", "streams": 2},
            "rows": rows, "gpu_launches": 16,
            "reference_published_ascend_910c": {
                "source": "pcieThrough/tests/README.md:72-75 (GB/s per op, 4 AIV)",
                "[1024,32,1,128]": {"zero_copy": 9.65, "fused_memcpy": 15.50},
                "[1024,32,8,128]": {"zero_copy": 26.52, "fused_memcpy": 19.49},
                "[1024,64,1,128]": {"zero_copy": 22.03, "fused_memcpy": 20.92},
                "[1024,64,8,128]": {"zero_copy": 34.11, "fused_memcpy": 22.55}}}


# --------------------------------------------------------------------------- overlap leg
class OverlapBench:
    """Layer-wise prefetch pipeline (Qwen2-7B-style fp8 cache, 28 layers): while a bf16
    [8192x3584]x[3584x18944] GEMM runs for layer l on the main stream, 256 blocks of the next layer(s)
    are swapped in on a side stream and 256 other blocks of layer l are swapped out on a second one,
    through LayerwisePrefetcher.  `group` layers share one launch per direction (their GEMMs still run
    one per layer).  Reports swap GB/s per direction under overlap, the GEMM slowdown, and a
    byte-for-byte check of every block and slot the pipeline touched."""

    MAX_GROUP = 8

    def __init__(self, g, device, pkg, host_raw=None, pool_layout="slot_major", slot_runs=False):
        from heterofusedkernels_b200.connector import LayerwisePrefetcher, PagedKVCache

        self.g, self.device, self.pkg = g, device, pkg
        self.pool_layout, self.slot_runs = pool_layout, slot_runs
        self.cache = PagedKVCache(g.layers, g.num_blocks, g.block_size, g.kv_heads, g.head_dim, g.dtype, device,
                                  host_slots=g.host_slots if host_raw is None else
                                  min(g.host_slots, host_raw.numel() // (g.layers * 2 * g.block_bytes)),
                                  host_raw=host_raw, pool_layout=pool_layout)
        fill_random_bytes(self.cache._k_store, 1)
        fill_random_bytes(self.cache._v_store, 2)
        self.pf = LayerwisePrefetcher(self.cache)       # shipped default: two side streams, paced swap-out
        self.pf_one = LayerwisePrefetcher(self.cache, one_stream=True)
        self.pf_unpaced = LayerwisePrefetcher(self.cache, evict_pace_gbs=0)
        self.a = torch.randn(8192, 3584, device=device, dtype=torch.bfloat16)
        self.b = torch.randn(3584, 18944, device=device, dtype=torch.bfloat16)
        self.c = torch.empty(8192, 18944, device=device, dtype=torch.bfloat16)
        self.flops = 2 * 8192 * 3584 * 18944
        self.L = g.layers
        gen = torch.Generator().manual_seed(5)
        # per layer: blocks to bring in / their slots, other blocks to push out / their (other) slots
        self.ids_cpu = []
        pool = _pool_bytes(self.cache)
        for l in range(self.L):
            perm = torch.randperm(g.num_blocks, generator=gen)
            sl = torch.randperm(self.cache.host_slots, generator=gen)
            n = g.n_swap
            if slot_runs:   # two runs of consecutive slots, as a fresh free list hands them out
                base = int(torch.randint(0, self.cache.host_slots - 2 * n, (1,), generator=gen))
                sl = torch.arange(base, base + 2 * n)
            self.ids_cpu.append((perm[:n], sl[:n], perm[n:2 * n], sl[n:2 * n]))
        self.ids = [tuple(t.to(device) for t in x) for x in self.ids_cpu]
        # known random bytes wherever a swap-in will read: the in-slots of layer l, for layer l and the
        # layers a launch that starts at l may cover with it (MAX_GROUP layers per launch at most)
        rnd = torch.randint(0, 254, (g.n_swap, self.MAX_GROUP) + tuple(pool.shape[2:]), dtype=torch.uint8,
                            generator=torch.Generator().manual_seed(6))
        for l in range(self.L):
            w = min(self.MAX_GROUP, self.L - l)
            pool[self.ids_cpu[l][1], l:l + w] = rnd[:, :w]
        self.layer_bytes = g.n_swap * 2 * g.block_bytes
        self.main = torch.cuda.current_stream(device)

    def warm(self, seconds: float):
        t = time.perf_counter()
        while time.perf_counter() - t < seconds:
            self.gemm_pass()

    def gemm_pass(self) -> float:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(self.L):
            torch.matmul(self.a, self.b, out=self.c)
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1)

    def groups(self, group: int):
        assert 1 <= group <= self.MAX_GROUP
        return [range(a, min(a + group, self.L)) for a in range(0, self.L, group)]

    def run(self, kind, ctas, group: int = 1, with_gemm: bool = True, directions=("in", "out"), markers=False) -> dict:
        """One pass over all layers.  kind: None (the prefetcher's shipped defaults), "vector" or
        "vector@<threads>x<loads in flight>[+pad<KiB of unused shared memory>]", "bulk" or "bulk@<stage bytes>x<stages>[+lag<k>]", "staged"
        (packing kernel + copy-engine transfers) or "copy_engine" (one copy per chunk)."""
        pkg, cache, L = self.pkg, self.cache, self.L
        pace = None
        if kind and "+pace" in kind:       # "...+pace40": the evict's stores paced to 40 GB/s
            kind, p_txt = kind.rsplit("+pace", 1)
            pace, kind = float(p_txt), (kind or None)
        pf = self.pf
        for suffix, which in (("+1stream", self.pf_one), ("+unpaced", self.pf_unpaced)):
            if kind and kind.endswith(suffix):
                pf, kind = which, (kind[:-len(suffix)] or None)
        lib = pkg.capi.lib()
        base_kind = (kind or "").split("@")[0].split("+")[0]
        mv = {"": None, "vector": pkg.capi.MOVER_VECTOR, "bulk": pkg.capi.MOVER_BULK, "staged": "staged",
              "copy_engine": None}[base_kind]
        geo = tuple(int(x) for x in kind.split("@")[1].split("+")[0].split("x")) if kind and "@" in kind else (0, 0)
        lag = int(kind.split("+lag")[1]) if kind and "+lag" in kind else 0
        pad_kib = int(kind.split("+pad")[1]) if kind and "+pad" in kind else 0
        pkg.capi.check(lib.hfk_set_vector_smem_pad(pad_kib * 1024), "hfk_set_vector_smem_pad")
        if base_kind == "vector":
            pkg.capi.check(lib.hfk_set_vector_geometry(*geo), "hfk_set_vector_geometry")
        else:
            pkg.capi.check(lib.hfk_set_bulk_geometry(*geo), "hfk_set_bulk_geometry")
        pkg.capi.check(lib.hfk_set_bulk_lag(lag), "hfk_set_bulk_lag")
        groups = self.groups(group)
        ev_in, ev_out = [], []
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for gi, layers in enumerate(groups):
            nxt = groups[(gi + 1) % len(groups)]
            in_ids, in_slots, _, _ = self.ids[nxt.start]
            _, _, out_ids, out_slots = self.ids[layers.start]
            in_slots_cpu, out_slots_cpu = self.ids_cpu[nxt.start][1], self.ids_cpu[layers.start][3]
            if kind == "copy_engine":
                ci_n, ci_l = self.ids_cpu[nxt.start], self.ids_cpu[layers.start]
                with torch.cuda.stream(pf.in_stream):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    torch.ops.pcie_through.swap_in_copy_engine(cache.k_ptrs_cpu[nxt.start:nxt.stop], cache.v_ptrs_cpu[nxt.start:nxt.stop],
                                                               cache.host_pool[:, nxt.start:nxt.stop], ci_n[0], ci_n[1], cache.num_blocks)
                    b.record()
                ev_in.append((a, b, len(nxt)))
                with torch.cuda.stream(pf.out_stream):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    torch.ops.pcie_through.swap_out_copy_engine(cache.k_ptrs_cpu[layers.start:layers.stop], cache.v_ptrs_cpu[layers.start:layers.stop],
                                                                cache.host_pool[:, layers.start:layers.stop], ci_l[2], ci_l[3], cache.num_blocks)
                    b.record()
                ev_out.append((a, b, len(layers)))
            else:
                if "in" in directions:
                    pf.in_stream.wait_stream(self.main)
                    with torch.cuda.stream(pf.in_stream):
                        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        if markers:
                            lib.hfk_debug_stamp_marker(pf.in_stream.cuda_stream)
                        a.record()
                    pf.prefetch(nxt, in_ids, in_slots, aiv=ctas, mover=mv, after=False, host_slot_ids_cpu=in_slots_cpu)
                    with torch.cuda.stream(pf.in_stream):
                        b.record()
                    ev_in.append((a, b, len(nxt)))
                if "out" in directions:
                    pf.out_stream.wait_stream(self.main)
                    with torch.cuda.stream(pf.out_stream):
                        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        if markers:
                            lib.hfk_debug_stamp_marker(pf.out_stream.cuda_stream)
                        a.record()
                    pf.evict(layers, out_ids, out_slots, aiv=ctas, mover=mv, after=False, host_slot_ids_cpu=out_slots_cpu,
                             pace_gbs=pace)
                    with torch.cuda.stream(pf.out_stream):
                        b.record()
                    ev_out.append((a, b, len(layers)))
            if with_gemm:
                for _ in layers:
                    torch.matmul(self.a, self.b, out=self.c)
        e1.record()
        pf.quiesce()
        torch.cuda.synchronize()
        lib.hfk_set_bulk_geometry(0, 0)
        lib.hfk_set_vector_geometry(0, 0)
        lib.hfk_set_vector_smem_pad(0)
        lib.hfk_set_bulk_lag(0)

        def rate(evs):
            if not evs:
                return None, None
            per = [n * self.layer_bytes / (x.elapsed_time(y) * 1e-3) / GB for x, y, n in evs]
            return statistics.median(per), statistics.median(x.elapsed_time(y) for x, y, _ in evs)

        in_gbs, in_ms = rate(ev_in)
        out_gbs, out_ms = rate(ev_out)
        # both directions of a group together: bytes both ways over first start .. last end
        pair = None
        if len(ev_in) == len(ev_out) and ev_in:
            per = []
            for (a_i, b_i, n_i), (a_o, b_o, n_o) in zip(ev_in, ev_out):
                span = max(x.elapsed_time(y) for x in (a_i, a_o) for y in (b_i, b_o))
                per.append((n_i + n_o) * self.layer_bytes / (span * 1e-3) / GB)
            pair = statistics.median(per)
        return {"main_ms": e0.elapsed_time(e1), "in_gbs": in_gbs, "out_gbs": out_gbs, "in_ms_median": in_ms,
                "out_ms_median": out_ms, "pair_gbs": pair, "launches": len(ev_in) + len(ev_out)}

    def verify(self, group: int) -> dict:
        """Every block a swap-in wrote equals its slot and every slot a swap-out wrote equals its block,
        for the id lists a pass with `group` layers per launch uses."""
        bad, checked = [], 0
        groups = self.groups(group)
        for layers in groups:
            # both launches that touch this group of layers take their lists from its first layer
            in_ids, in_slots, out_ids, out_slots = self.ids_cpu[layers.start]
            r = verify_swap(self.cache, [("swap_in", in_ids, in_slots), ("swap_out", out_ids, out_slots)], layers=layers)
            checked += r["bytes_checked"]
            bad += r["mismatches"]
        return {"verified": not bad, "bytes_checked": checked, "mismatches": bad[:8]}

    def measure(self, kind, ctas, group: int, reps: int) -> dict:
        self.run(kind, ctas, group)  # warm-up
        alone, runs = [], []
        for _ in range(reps):
            alone.append(self.gemm_pass())
            runs.append(self.run(kind, ctas, group))
        solo = self.run(kind, ctas, group, with_gemm=False)
        t_a = statistics.median(alone)
        med_main = statistics.median(r["main_ms"] for r in runs)
        ver = self.verify(group)
        return {"mover": kind or "default", "ctas_per_direction": ctas or "default", "layers_per_launch": group,
                "side_streams": 1 if "+1stream" in (kind or "") else 2, "pool_layout": self.pool_layout, "slots": "runs" if self.slot_runs else "random",
                "gemm_ms_alone": t_a, "gemm_ms_overlapped": med_main,
                "gemm_slowdown_pct": 100.0 * (med_main / t_a - 1.0),
                "gemm_tflops_alone": self.L * self.flops / (t_a * 1e-3) / 1e12,
                "swap_in_gbs": statistics.median(r["in_gbs"] for r in runs),
                "swap_out_gbs": statistics.median(r["out_gbs"] for r in runs),
                "swap_in_gbs_no_gemm": solo["in_gbs"], "swap_out_gbs_no_gemm": solo["out_gbs"],
                "both_directions_gbs": statistics.median(r["pair_gbs"] for r in runs) if runs[0]["pair_gbs"] else None,
                "both_directions_gbs_no_gemm": solo["pair_gbs"],
                "launches_per_pass": runs[0]["launches"], "verified": ver["verified"],
                "bytes_checked": ver["bytes_checked"]}

    def stamps(self, kind, ctas, group: int, direction: str) -> dict:
        """Scheduling delay of the swap launches of one direction next to the GEMM: a one-thread marker
        kernel is enqueued in front of every swap launch and every CTA stamps its SM id and its start /
        end times (the same %globaltimer)."""
        lib = self.pkg.capi.lib()
        cap = 8192
        buf = torch.zeros(1 + 4 * cap, dtype=torch.int64, device=self.device)
        self.run(kind, ctas, group, directions=(direction,))
        self.pkg.capi.check(lib.hfk_debug_set_stamps(buf.data_ptr(), buf.numel() * 8), "hfk_debug_set_stamps")
        self.run(kind, ctas, group, directions=(direction,), markers=True)
        self.pkg.capi.check(lib.hfk_debug_set_stamps(None, 0), "hfk_debug_set_stamps")
        w = buf.cpu()
        n = min(int(w[0]), cap)
        rec = w[1:1 + 4 * n].view(n, 4)
        marks = sorted(int(r[2]) for r in rec if (int(r[0]) >> 32) == 0)
        ctas_rec = [(int(r[0]) & 0xffffffff, int(r[2]), int(r[3])) for r in rec if (int(r[0]) >> 32) != 0]
        delays, spans, sms, spreads = [], [], set(), []
        for i, m in enumerate(marks):
            nxt = marks[i + 1] if i + 1 < len(marks) else 1 << 62
            mine = [c for c in ctas_rec if m <= c[1] < nxt]
            if not mine:
                continue
            first, last_start, end = min(c[1] for c in mine), max(c[1] for c in mine), max(c[2] for c in mine)
            delays.append((first - m) * 1e-3)
            spreads.append((last_start - first) * 1e-3)
            spans.append((end - first) * 1e-3)
            sms |= {c[0] for c in mine}
        med = lambda x: statistics.median(x) if x else None  # noqa: E731
        return {"mover": kind or "default", "ctas": ctas, "direction": direction, "launches": len(delays),
                "first_cta_start_after_marker_us_median": med(delays),
                "first_cta_start_after_marker_us_max": max(delays) if delays else None,
                "last_cta_start_after_first_us_median": med(spreads),
                "kernel_span_us_median": med(spans), "distinct_sms": len(sms), "records": n}


def overlap_summary(ob: OverlapBench, reps: int, group: int) -> dict:
    """The `overlap` object of the default line: the prefetcher's shipped defaults."""
    sampler = ClockSampler(ob.device.index or 0)
    ob.warm(1.5)
    m = ob.measure(None, None, group, reps)
    one = ob.measure("+1stream", None, group, max(2, reps // 2))
    clocks = sampler.stop()
    status = ob.cache.status()
    return {"workload": "qwen2_7b_fp8_prefetch",
            "mover": "LayerwisePrefetcher defaults (bulk mover, 2 KiB x 4 ring, 64 CTAs; two side streams, "
                     "swap-out paced to 40 GB/s)",
            "layers_per_launch": group, "gemm_slowdown_pct": m["gemm_slowdown_pct"], "swap_in_gbs": m["swap_in_gbs"],
            "swap_out_gbs": m["swap_out_gbs"], "both_directions_gbs": m["both_directions_gbs"],
            "swap_in_gbs_no_gemm": m["swap_in_gbs_no_gemm"], "swap_out_gbs_no_gemm": m["swap_out_gbs_no_gemm"],
            "one_stream_swap_in_gbs": one["swap_in_gbs"], "one_stream_swap_out_gbs": one["swap_out_gbs"],
            "one_stream_both_directions_gbs": one["both_directions_gbs"],
            "one_stream_gemm_slowdown_pct": one["gemm_slowdown_pct"],
            "one_stream_swap_in_gbs_no_gemm": one["swap_in_gbs_no_gemm"],
            "one_stream_swap_out_gbs_no_gemm": one["swap_out_gbs_no_gemm"],
            "gemm_tflops": m["gemm_tflops_alone"],
            "gemm_ms_alone": m["gemm_ms_alone"], "gemm_ms_overlapped": m["gemm_ms_overlapped"],
            "bytes_per_layer_per_direction": ob.layer_bytes,
            "verified": bool(m["verified"] and one["verified"] and status == 0),
            "bytes_checked": m["bytes_checked"], "status_word": status, "sm_mhz": clocks.get("sm_mhz"),
            "clock_reasons": ",".join(clocks.get("reasons", [])), "reps": reps}


def bench_overlap(g, device, args, pkg) -> dict:
    """The full overlap study: movers x CTA counts x layers per launch, the large (Llama-3-8B-size)
    swap next to the GEMM loop, and the scheduling-delay stamps."""
    ob = OverlapBench(g, device, pkg)
    ob.warm(2.0)
    sampler = ClockSampler(device.index or 0)
    reps = args.overlap_reps
    variants = []
    table = [(None, None, 1), (None, None, 2), (None, None, 4), (None, None, 8),
             ("+pace44", None, 4), ("+pace42", None, 4), ("+pace41", None, 4), ("+pace38", None, 4), ("+unpaced", None, 4),
             ("+1stream", None, 1), ("+1stream", None, 4), ("+1stream", None, 8),
             ("bulk+1stream", 32, 4), ("bulk@4096x4+1stream", 32, 4), ("bulk@16384x8+1stream", 8, 8),
             ("vector+1stream", 16, 4), ("vector@256x8+1stream", 32, 4), ("vector+unpaced", 16, 4)]
    if args.overlap_quick:
        table = table[:2]
    for kind, ctas, group in table:
        variants.append(ob.measure(kind, ctas, group, reps))
    stamps = []
    for kind, ctas in (() if args.overlap_quick else
                       (("+1stream", None), ("bulk@4096x4+1stream", 32), ("bulk@16384x8+1stream", 4),
                        ("vector+1stream", 16), ("vector@256x8+1stream", 32))):
        for direction in ("in", "out"):
            stamps.append(ob.stamps(kind, ctas, 1, direction))
    status = ob.cache.status()
    del ob
    torch.cuda.empty_cache()
    # the same pipeline on a layer-major pool with slots handed out as runs: one copy-engine transfer per
    # layer and direction (staged), next to the kernel movers on the same layout
    ob = OverlapBench(g, device, pkg, pool_layout="layer_major", slot_runs=True)
    for kind, ctas, group in (("staged+1stream", None, 4), ("staged@2048x4+1stream", 64, 4), (None, None, 4)):
        variants.append(ob.measure(kind, ctas, group, reps))
    clocks = sampler.stop()
    status |= ob.cache.status()
    ok = [v for v in variants if v["mover"] != "copy_engine" and v["gemm_slowdown_pct"] < 10.0]
    pick = max(ok or variants, key=lambda v: v["swap_in_gbs"] + v["swap_out_gbs"])
    L = g.layers
    return {"metric": "kv_swap_GBps_under_gemm_overlap", "value": (pick["swap_in_gbs"] + pick["swap_out_gbs"]) / 2,
            "unit": "GB/s", "n_gpus": 1, "steps": reps, "warmup": 1, "ms_per_step": pick["gemm_ms_overlapped"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": g.name, "layers": L, "blocks_per_layer_per_direction": g.n_swap,
                       "bytes_per_layer_per_direction": ob.layer_bytes, "kv_dtype": "float8_e4m3fn",
                       "device_blocks": g.num_blocks, "host_slots": ob.cache.host_slots,
                       "gemm": "bf16 [8192x3584]x[3584x18944] per layer (torch.matmul)",
                       "pool sizes": "8192 device / 16384 host blocks (not fixed by the configuration; chosen here)"},
            "picked": pick, "variants": variants, "stamps": stamps, "clocks": clocks, "status_word": status,
            "verified": all(v["verified"] for v in variants),
            "gpu_launches": sum(v["launches_per_pass"] for v in variants) * reps}


def bench_large_swap_beside_gemm(sb: SwapBench, device, steps: int) -> dict:
    """One Llama-3-8B-size swap step (1.07 GB each way) while a GEMM loop occupies the main stream."""
    a = torch.randn(8192, 3584, device=device, dtype=torch.bfloat16)
    b = torch.randn(3584, 18944, device=device, dtype=torch.bfloat16)
    c = torch.empty(8192, 18944, device=device, dtype=torch.bfloat16)
    side = torch.cuda.Stream(device, priority=-1)
    main = torch.cuda.current_stream(device)

    def gemms(n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            torch.matmul(a, b, out=c)
        e1.record()
        return e0, e1

    t = time.perf_counter()
    while time.perf_counter() - t < 1.5:
        e0, e1 = gemms(28)
        e1.synchronize()
    n_gemm = 60   # about 50 ms of GEMMs, longer than one swap step
    alone = []
    for _ in range(3):
        e0, e1 = gemms(n_gemm)
        e1.synchronize()
        alone.append(e0.elapsed_time(e1))
    res = []
    sb.prime()
    for s in range(1, steps + 1):
        o_ids, slots, i_ids = sb.dev_sets[s]
        torch.cuda.synchronize()
        g0 = torch.cuda.Event()
        g0.record()
        side.wait_event(g0)
        with torch.cuda.stream(side):
            x0, x1, x2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            x0.record()
            sb._out(o_ids, slots, sb.sets[s][1])
            x1.record()
            sb._in(i_ids, slots, sb.sets[s][1])
            x2.record()
        e0, e1 = gemms(n_gemm)
        main.wait_stream(side)
        torch.cuda.synchronize()
        res.append((e0.elapsed_time(e1), x0.elapsed_time(x1), x1.elapsed_time(x2)))
    ver = verify_swap(sb.cache, [("swap_out", sb.sets[steps][0], sb.sets[steps][1]),
                                 ("swap_in", sb.sets[steps][2], sb.sets[steps][1])])
    t_a = statistics.median(alone)
    return {"gemm_ms_alone": t_a, "gemm_ms_with_swap": statistics.median(r[0] for r in res),
            "gemm_slowdown_pct": 100.0 * (statistics.median(r[0] for r in res) / t_a - 1.0),
            "swap_out_gbs": sb.g.swap_bytes / (statistics.median(r[1] for r in res) * 1e-3) / GB,
            "swap_in_gbs": sb.g.swap_bytes / (statistics.median(r[2] for r in res) * 1e-3) / GB,
            "note": "the swap step covers about 80 % of the GEMM loop, so the slowdown is diluted by that factor",
            "verified": ver["verified"]}


# --------------------------------------------------------------------------- GPU <-> GPU migration leg
def bench_migrate(g, args, pkg) -> dict:
    """KV block migration between the caches of two GPUs of one box (one process, two devices):
    512 blocks x 32 layers x K,V of the Llama-3-8B layout (1.07 GB) from GPU 0's cache into other
    blocks of GPU 1's cache.  Pull (the destination GPU runs the kernel: peer loads over NVLink),
    push (the source GPU runs it: peer stores), the copy-engine twin (one cudaMemcpyPeerAsync per
    chunk, fewer blocks) and a plain 1 GiB peer copy as the NVLink denominator; every result is
    compared byte for byte with the source blocks."""
    from heterofusedkernels_b200.connector import PagedKVCache

    assert torch.cuda.device_count() >= 2, "the migration leg needs two GPUs in one process"
    d0, d1 = torch.device("cuda", 0), torch.device("cuda", 1)
    lib = pkg.capi.lib()
    src = PagedKVCache(g.layers, g.num_blocks, g.block_size, g.kv_heads, g.head_dim, g.dtype, d0)
    dst = PagedKVCache(g.layers, g.num_blocks, g.block_size, g.kv_heads, g.head_dim, g.dtype, d1)
    for i, t in enumerate((src._k_store, src._v_store, dst._k_store, dst._v_store)):
        fill_random_bytes(t, 10 + i)
    gen = torch.Generator().manual_seed(3)
    nbytes = g.swap_bytes
    # NVLink denominator: one contiguous peer copy of 1 GiB
    a0 = torch.empty(1 << 30, dtype=torch.uint8, device=d0)
    a1 = torch.empty(1 << 30, dtype=torch.uint8, device=d1)
    peer = 0.0
    with torch.cuda.device(d1):
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            a1.copy_(a0, non_blocking=True)
            e1.record()
            e1.synchronize()
            peer = max(peer, a0.numel() / (e0.elapsed_time(e1) * 1e-3) / GB)
    del a0, a1

    def check(s_ids, d_ids) -> bool:
        ok = True
        for sk, dk in ((src._k_store, dst._k_store), (src._v_store, dst._v_store)):
            for l0 in range(0, g.layers, 8):
                want = sk[l0:l0 + 8].index_select(1, s_ids.to(d0)).to(d1)
                got = dk[l0:l0 + 8].index_select(1, d_ids.to(d1))
                ok = ok and torch.equal(want.view(torch.int16), got.view(torch.int16))
        return ok

    rows = {}
    for mode, run_dev in (("pull", d1), ("push", d0)):
        for ctas in (None, 148, 296, 592):
            best, ok = 0.0, True
            for rep in range(args.warmup + args.steps):
                s_ids = torch.randperm(g.num_blocks, generator=gen)[:g.n_swap]
                d_ids = torch.randperm(g.num_blocks, generator=gen)[:g.n_swap]
                with torch.cuda.device(run_dev):
                    torch.cuda.synchronize(d0)
                    torch.cuda.synchronize(d1)
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    s_dev, d_dev = s_ids.to(run_dev), d_ids.to(run_dev)
                    e0.record()
                    src.migrate_to(dst, s_dev, d_dev, aiv=ctas, run_on="dst" if mode == "pull" else "src")
                    e1.record()
                    e1.synchronize()
                    if rep >= args.warmup:
                        best = max(best, nbytes / (e0.elapsed_time(e1) * 1e-3) / GB)
                if rep == args.warmup + args.steps - 1:
                    ok = check(s_ids, d_ids)
            rows[f"{mode}_ctas_{ctas or 'default'}"] = {"GBps": best, "verified": ok}
    # copy-engine twin: one cudaMemcpyPeerAsync per 32 KiB chunk (64 blocks = 4096 copies)
    n_ce = 64
    s_ids = torch.randperm(g.num_blocks, generator=gen)[:n_ce]
    d_ids = torch.randperm(g.num_blocks, generator=gen)[:n_ce]
    md = pkg.capi.MigrateDesc()
    md.src_k_layer_ptrs, md.src_v_layer_ptrs = src.k_ptrs_cpu.data_ptr(), src.v_ptrs_cpu.data_ptr()
    md.dst_k_layer_ptrs, md.dst_v_layer_ptrs = dst.k_ptrs_cpu.data_ptr(), dst.v_ptrs_cpu.data_ptr()
    md.src_block_ids, md.dst_block_ids = s_ids.data_ptr(), d_ids.data_ptr()
    md.ids_are_int64, md.layers, md.n_blocks, md.block_bytes = 1, g.layers, n_ce, g.block_bytes
    md.src_block_stride = md.dst_block_stride = g.block_bytes
    md.num_src_blocks = md.num_dst_blocks = g.num_blocks
    with torch.cuda.device(d1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        pkg.capi.check(lib.hfk_migrate_blocks_copy_engine(C.byref(md), 0, 1, torch.cuda.current_stream(d1).cuda_stream),
                       "hfk_migrate_blocks_copy_engine")
        e1.record()
        e1.synchronize()
        rows["copy_engine_per_chunk"] = {"GBps": n_ce * g.layers * 2 * g.block_bytes / (e0.elapsed_time(e1) * 1e-3) / GB,
                                         "verified": check(s_ids, d_ids), "copies": n_ce * g.layers * 2}
    status = src.status() | dst.status()
    best_key = max((k for k in rows if k.startswith(("pull", "push"))), key=lambda k: rows[k]["GBps"])
    return {"metric": "kv_migrate_GBps", "value": rows[best_key]["GBps"], "unit": "GB/s", "n_gpus": 2, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": nbytes / rows[best_key]["GBps"] / 1e6, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": "migrate", "layers": g.layers, "blocks": g.n_swap, "bytes": nbytes,
                       "layout": "Llama-3-8B: bf16 [16, 8, 128] blocks, 4096-block caches on GPU 0 and GPU 1",
                       "l2": "1.07 GB of distinct blocks per launch (larger than L2)"},
            "best": best_key, "rows": rows, "verified": all(r["verified"] for r in rows.values()),
            "roofline": {"bound": "nvlink", "achieved": rows[best_key]["GBps"], "peak": peer, "unit": "GB/s",
                         "frac": rows[best_key]["GBps"] / peer, "traffic": None,
                         "peak_source": "live cudaMemcpy of 1 GiB GPU 0 -> GPU 1, best of 5 (pool reference: 770 GB/s "
                                        "per direction)"},
            "status_word": status, "gpu_launches": args.steps}


# --------------------------------------------------------------------------- main
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="llama3_8b_swap")
    ap.add_argument("--mover", default="auto", choices=["auto", "vector", "bulk", "staged"])
    ap.add_argument("--variant", default="default",
                    help="how a step is issued: sequential | stagger | bidir | interleave:<k>; "
                         "default = sequential on one GPU, the multi-GPU default otherwise")
    ap.add_argument("--variants", default="", help="comma-separated extra variants to time after the main one")
    ap.add_argument("--staging-mb", type=int, default=1024, help="staging buffer of the staged mover (MiB)")
    ap.add_argument("--staged-lanes", type=int, default=0, help="copy streams of the staged mover (0 = library default)")
    ap.add_argument("--slot-runs", type=int, default=0,
                    help="each step's host slots come as runs of this many consecutive slots (0 = random slots)")
    ap.add_argument("--aiv", type=int, default=0, help="CTAs per swap kernel (0 = library default)")
    ap.add_argument("--gather-aiv", type=int, default=0)
    ap.add_argument("--host-slots", type=int, default=0, help="override the host pool size (slots)")
    ap.add_argument("--device-blocks", type=int, default=0, help="override the device cache size (blocks)")
    ap.add_argument("--no-spread", action="store_true", help="use GPU ordinal = LOCAL_RANK even when more GPUs are visible")
    ap.add_argument("--no-gather", action="store_true")
    ap.add_argument("--no-config4", action="store_true", help="skip the short Llama-3-70B TP8 run")
    ap.add_argument("--no-allocator-leg", action="store_true", help="skip the run with allocator-ordered host slots")
    ap.add_argument("--no-overlap", action="store_true", help="skip the short prefetch-next-to-a-GEMM run")
    ap.add_argument("--overlap-group", type=int, default=0, help="layers per prefetch launch (0 = shipped default)")
    ap.add_argument("--overlap-reps", type=int, default=5)
    ap.add_argument("--overlap-quick", action="store_true", help="overlap study: the shipped defaults only")
    ap.add_argument("--beside-gemm", action="store_true", help="also time the full swap step next to a GEMM loop")
    ap.add_argument("--gather-only", action="store_true", help="run only the paged-gather leg")
    ap.add_argument("--gather-seqs", type=int, default=64, help="sequences in the gather batch")
    ap.add_argument("--gather-hints", type=int, default=-1, help="L2 hints of the bulk gather (-1 = library default)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "b200":
        args.warmup = max(args.warmup, 3)

    from heterofusedkernels_b200 import ranks

    ctx = ranks.RankContext.from_env()
    rank, local_rank, world = ctx.rank, ctx.local_rank, ctx.world
    g = geometry(args.workload)
    if args.device_blocks:
        g.num_blocks = args.device_blocks
    config = {"workload": g.name, "layers": g.layers, "block_size": g.block_size, "kv_heads": g.kv_heads,
              "head_dim": g.head_dim, "kv_dtype": str(g.dtype).replace("torch.", ""),
              "blocks_per_swap": g.n_swap, "device_blocks": g.num_blocks,
              "bytes_per_direction_per_gpu": g.swap_bytes, "parallelism": f"{world} independent ranks, no collective",
              "l2": "inputs larger than L2 (each direction moves >= 1 GB of distinct blocks per step)"}

    if args.impl == "reference":
        # the reference semantics (torch CPU index_select / index_copy_ per layer) on the host cores
        if rank != 0:
            return
        cb = cpu_baseline_swap(g, args.steps, args.warmup, budget_s=150.0)
        line = {"impl": "reference", "metric": "kv_swap_GBps", "value": cb["value"], "unit": "GB/s",
                "n_gpus": args.gpus, "steps": cb["steps"], "warmup": args.warmup,
                "ms_per_step": cb["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "u8", "data": "synthetic", "config": config, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    import heterofusedkernels_b200 as pkg
    from heterofusedkernels_b200.connector import PagedKVCache

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    pkg.load_ops()
    lib = pkg.capi.lib()
    if args.gather_hints >= 0:
        pkg.capi.check(lib.hfk_set_gather_tuning(args.gather_hints, -1), "hfk_set_gather_tuning")
    if args.staged_lanes:
        pkg.capi.check(lib.hfk_set_staged_copy_lanes(args.staged_lanes), "hfk_set_staged_copy_lanes")
    # fewer ranks than visible GPUs: spread them over the PCI bus order (ranks.spread_device_index)
    dev_index = local_rank if args.no_spread else ranks.spread_device_index(local_rank, world, torch.cuda.device_count())
    torch.cuda.set_device(dev_index)
    device = torch.device("cuda", dev_index)
    ctx.init("nccl", device)
    barrier, max_over_ranks = ctx.barrier, ctx.max_over_ranks

    mover = {"auto": None, "vector": pkg.capi.MOVER_VECTOR, "bulk": pkg.capi.MOVER_BULK, "staged": "staged"}[args.mover]
    aiv = args.aiv if args.aiv > 0 else None

    if args.gather_only:
        res = bench_gather(device, args.steps, args.warmup, mover if mover != "staged" else None,
                           args.gather_aiv if args.gather_aiv > 0 else None, args.gather_seqs)
        print(json.dumps({"metric": "paged_gather_GBps", "value": res["value"], "unit": "GB/s", "n_gpus": 1,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_launch"],
                          "higher_is_better": True, "dtype": "u8", "data": "synthetic", "gpu_launches": args.steps,
                          "config": {"workload": "llama3_8b_gather", "num_seqs": args.gather_seqs}, "gather": res}),
              flush=True)
        return
    if g.name == "migrate":
        print(json.dumps(bench_migrate(g, args, pkg)), flush=True)
        return
    if g.name == "block_transfer":
        print(json.dumps(bench_block_transfer(device, args, pkg)), flush=True)
        return
    if g.name == "embedding_gather":
        print(json.dumps(bench_embedding_gather(device, args, pkg)), flush=True)
        return
    if g.name == "qwen2_7b_fp8_prefetch":
        print(json.dumps(bench_overlap(g, device, args, pkg)), flush=True)
        return

    # ---- workload state (outside every timed region) -----------------------------------
    slot_bytes = g.layers * 2 * g.block_bytes
    host_slots = args.host_slots or g.host_slots
    host_slots, pool_note = ranks.host_pool_slots(host_slots, slot_bytes, g.n_swap, world, mem_available_bytes())
    t0 = time.perf_counter()
    cache = PagedKVCache(g.layers, g.num_blocks, g.block_size, g.kv_heads, g.head_dim, g.dtype, device,
                         host_slots=host_slots)
    setup_pool_s = time.perf_counter() - t0
    host_raw = cache._host_raw
    fill_random_bytes(cache._k_store, 100 + rank)
    fill_random_bytes(cache._v_store, 200 + rank)
    variant = args.variant
    candidates = [variant]
    if variant == "default":
        # one GPU: swap-out then swap-in.  Several ranks on one host: the step is timed in each of the
        # MULTI_GPU_VARIANTS issue orders and the faster one is reported (all of them in `variants`)
        candidates = ["sequential"] if world == 1 else list(MULTI_GPU_VARIANTS)
        variant = candidates[0]
    config.update({"host_slots": host_slots, "host_pool_bytes": host_slots * slot_bytes, "pool_note": pool_note,
                   "host_pool_layout": "[slot][layer][K|V][block] (2 MiB-class contiguous per slot)",
                   "numa_node": pkg.memory.device_numa_node(), "pool_setup_s": round(setup_pool_s, 2),
                   "gpu_ordinal_of_rank": "spread over the visible GPUs in PCI bus order" if not args.no_spread
                   else "LOCAL_RANK", "visible_gpus": torch.cuda.device_count(), "variant": variant,
                   "variant_meaning": VARIANT_TEXT.get(variant.split(":")[0], "")})

    n_sets = args.warmup + args.steps
    sb = SwapBench(g, cache, ctx, pkg, n_sets, mover, aiv, args.staging_mb, slot_runs=args.slot_runs)
    config["host_slots_per_step"] = (f"runs of {args.slot_runs} consecutive slots" if args.slot_runs
                                     else "random distinct slots")

    pcie = measure_pcie_peak(host_raw.view(torch.uint8), device) if rank == 0 else None
    barrier()
    pcie_conc = None
    if world > 1:
        mine = measure_pcie_concurrent(ctx, host_raw.view(torch.uint8), device)
        pcie_conc = ctx.gather_floats([mine["h2d"], mine["d2h"], mine["bidir_total"]])

    def timed_leg(bench: SwapBench, var: str, steps: int, warmup: int, e2e: bool) -> dict:
        r = bench.run(var, steps, warmup, e2e)
        r["ms_per_step"] = max_over_ranks(r["local_ms_per_step"])
        r["all_verified"] = max_over_ranks(0.0 if r["verified"] else 1.0) == 0.0
        r["value"] = ranks.aggregate_gbs(2 * bench.g.swap_bytes, world, r["ms_per_step"])
        r["out_gbs"] = bench.g.swap_bytes / (statistics.mean(r["out_ms"]) * 1e-3) / GB
        r["in_gbs"] = bench.g.swap_bytes / (statistics.mean(r["in_ms"]) * 1e-3) / GB
        return r

    # ---- value leg: ids resident on the device, kernels only -----------------------------
    tried = {}
    val = None
    for cand in candidates:
        sampler = ClockSampler(dev_index) if rank == 0 else None
        r = timed_leg(sb, cand, args.steps, args.warmup, e2e=False)
        r["launches_timed"] = sb.launches_timed
        r["clocks"] = sampler.stop() if sampler else None
        tried[cand] = r
        if val is None or r["value"] > val["value"]:      # the value is a max over ranks: every rank picks the same
            val, variant = r, cand
    launches_value, clocks = val["launches_timed"], val["clocks"]
    config.update({"variant": variant, "variant_meaning": VARIANT_TEXT.get(variant.split(":")[0], ""),
                   "variants_tried": {k: round(v["value"], 3) for k, v in tried.items()}})
    bus = (C.c_char * 32)()
    lib.hfk_device_pci_bus_id(-1, bus, 32)
    per_rank = ctx.gather_floats([pkg.memory.device_numa_node(), val["out_gbs"], val["in_gbs"],
                                  val["local_ms_per_step"], int(bus.value.decode().split(":")[1], 16),
                                  1.0 if val["verified"] else 0.0])

    # ---- e2e leg: public API, host-resident id lists, status read back every step ------------
    e2 = timed_leg(sb, variant, args.steps, args.warmup, e2e=True)
    id_bytes = 4 * g.n_swap * 8
    e2e = {"value": e2["value"], "unit": "GB/s", "ms_per_step": e2["ms_per_step"],
           "h2d_bytes_per_step": g.swap_bytes + id_bytes, "d2h_bytes_per_step": g.swap_bytes + 4,
           "verified": e2["all_verified"],
           "api": "PagedKVCache.swap_out/swap_in -> torch.ops.pcie_through.*; payload moves between HBM and the "
                  "pinned host pool inside the timed region",
           "mover": ("picked by the connector from the host-resident id lists: " +
                     str(cache._pick_mover(sb.pin_sets[1][1]) or "kernels")) if mover is None else args.mover}

    # ---- optional extra variants on the same state ---------------------------------------------
    extra = {}
    for var_full in [v for v in args.variants.split(",") if v]:
        var = var_full
        if "+pace" in var:     # e.g. bidir+pace44: swap-outs of the bulk mover paced to 44 GB/s
            var, pace = var.split("+pace")
            pkg.capi.check(lib.hfk_set_swap_out_pace(int(float(pace) * 1000)), "hfk_set_swap_out_pace")
        if var.startswith("staged"):   # "staged" or "staged:<lanes>"
            lanes = int(var.split(":")[1]) if ":" in var else 0
            lib.hfk_set_staged_copy_lanes(lanes)
            sb.mover = "staged"
            r = timed_leg(sb, variant, args.steps, args.warmup, e2e=False)
            sb.mover = mover
            lib.hfk_set_staged_copy_lanes(args.staged_lanes)
        elif var.startswith("mover=hybrid"):
            sb.mover = var.split("=")[1]
            r = timed_leg(sb, variant, args.steps, args.warmup, e2e=False)
            sb.mover = mover
        elif var.startswith("mover="):
            sb.mover = {"vector": pkg.capi.MOVER_VECTOR, "bulk": pkg.capi.MOVER_BULK}[var.split("=")[1]]
            r = timed_leg(sb, variant, args.steps, args.warmup, e2e=False)
            sb.mover = mover
        else:
            r = timed_leg(sb, var, args.steps, args.warmup, e2e=False)
        lib.hfk_set_swap_out_pace(0)
        per = ctx.gather_floats([r["out_gbs"], r["in_gbs"]])
        extra[var_full] = {"value": r["value"], "ms_per_step": r["ms_per_step"], "verified": r["all_verified"],
                      "swap_out_GBps_per_rank": [round(p[0], 2) for p in per],
                      "swap_in_GBps_per_rank": [round(p[1], 2) for p in per], "plan_rank0": r["plan"]}
    # ---- the same step with the slots a fresh free list hands out (one run per step), public API ----
    # PagedKVCache then picks the staged mover by itself: the copy engine crosses the link.
    alloc_leg = None
    if world == 1 and not args.slot_runs and not args.no_allocator_leg:
        sb_runs = SwapBench(g, cache, ctx, pkg, n_sets, None, aiv, args.staging_mb, slot_runs=g.n_swap)
        r = timed_leg(sb_runs, variant, args.steps, args.warmup, e2e=True)
        alloc_leg = {"value": r["value"], "unit": "GB/s", "ms_per_step": r["ms_per_step"], "swap_out_GBps": r["out_gbs"],
                     "swap_in_GBps": r["in_gbs"], "verified": r["all_verified"],
                     "slots": f"one run of {g.n_swap} consecutive host slots per step (HostSlotPool order)",
                     "mover": "picked by PagedKVCache.swap_out/swap_in: staged (packing kernel + copy-engine "
                              "transfers of up to 64 MiB)"}
        del sb_runs
    beside = None
    if args.beside_gemm and world == 1:
        beside = bench_large_swap_beside_gemm(sb, device, min(args.steps, 5))

    # ---- Llama-3-70B TP8 shard, short run on the same pinned buffer (every N) -------------------
    config4 = None
    del sb, cache
    torch.cuda.empty_cache()
    if not args.no_config4 and g.name == "llama3_8b_swap":
        g4 = geometry("llama3_70b_tp8_swap")
        slot4 = g4.layers * 2 * g4.block_bytes
        slots4 = min(g4.host_slots, host_raw.numel() // slot4)
        if slots4 >= 2 * g4.n_swap:
            cache4 = PagedKVCache(g4.layers, g4.num_blocks, g4.block_size, g4.kv_heads, g4.head_dim, g4.dtype, device,
                                  host_slots=slots4, host_raw=host_raw)
            fill_random_bytes(cache4._k_store, 300 + rank)
            fill_random_bytes(cache4._v_store, 400 + rank)
            sb4 = SwapBench(g4, cache4, ctx, pkg, 4, mover, aiv, args.staging_mb)
            r4 = timed_leg(sb4, variant, 3, 1, e2e=False)
            per4 = ctx.gather_floats([r4["out_gbs"], r4["in_gbs"]])
            config4 = {"workload": g4.name, "steps": 3, "warmup": 1, "value": r4["value"], "unit": "GB/s",
                       "ms_per_step": r4["ms_per_step"], "bytes_per_direction_per_gpu": g4.swap_bytes,
                       "swap_out_GBps_per_gpu_mean": statistics.mean(p[0] for p in per4),
                       "swap_in_GBps_per_gpu_mean": statistics.mean(p[1] for p in per4),
                       "swap_out_GBps_per_rank": [round(p[0], 2) for p in per4],
                       "swap_in_GBps_per_rank": [round(p[1], 2) for p in per4],
                       "host_slots": slots4, "device_blocks": g4.num_blocks, "variant": variant,
                       "pool_note": "" if slots4 == g4.host_slots else
                       f"host pool of {slots4} slots on the pinned buffer shared with the Llama-3-8B run "
                       f"(configuration: {g4.host_slots}); transferred set unchanged",
                       "verified": r4["all_verified"]}
            del sb4, cache4
            torch.cuda.empty_cache()

    # ---- prefetch pipeline next to a GEMM, shipped defaults, short run (N = 1) --------------------
    overlap = None
    if world == 1 and not args.no_overlap and g.name == "llama3_8b_swap":
        g5 = geometry("qwen2_7b_fp8_prefetch")
        ob = OverlapBench(g5, device, pkg, host_raw=host_raw)
        overlap = overlap_summary(ob, reps=args.overlap_reps, group=args.overlap_group or DEFAULT_PREFETCH_GROUP)
        del ob
        torch.cuda.empty_cache()

    # ---- gather leg (single-GPU runs) ------------------------------------------------------
    gather = None
    if world == 1 and not args.no_gather and g.name != "tiny":
        gather = bench_gather(device, max(args.steps, 5), args.warmup, mover if mover != "staged" else None,
                              args.gather_aiv if args.gather_aiv > 0 else None)

    if rank != 0:
        ctx.close()
        return

    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except OSError:
        pass
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    hbm_src = "MEASURED_PEAKS.json hbm_gbs (of measured)" if peaks else "6650 GB/s (of fallback)"
    out_gbs, in_gbs = val["out_gbs"], val["in_gbs"]
    achieved = 2 * g.swap_bytes / ((statistics.mean(val["out_ms"]) + statistics.mean(val["in_ms"])) * 1e-3) / GB
    pcie_peak = (pcie["h2d"] + pcie["d2h"]) / 2
    ratio, ratio_src = traffic_ratio("kv_swap_kernel", 1.0097)
    roofline = {"bound": "pcie", "kernel": "kv_swap_*_kernel (swap-out and swap-in launches)",
                "achieved": achieved, "peak": pcie_peak, "unit": "GB/s", "frac": achieved / pcie_peak,
                "traffic": int(ratio * g.swap_bytes), "traffic_source": ratio_src,
                "peak_source": "live cudaMemcpyAsync of 1 GiB pinned<->device, best of 5, mean of the two "
                               "directions (MEASURED_PEAKS.json holds no PCIe figure)",
                "swap_out_achieved": out_gbs, "swap_out_peak": pcie["d2h"], "swap_out_frac": out_gbs / pcie["d2h"],
                "swap_in_achieved": in_gbs, "swap_in_peak": pcie["h2d"], "swap_in_frac": in_gbs / pcie["h2d"],
                "nominal_gen5_x16": 63.0, "algorithmic_bytes_per_launch": g.swap_bytes,
                "e2e_per_gpu": e2["value"] / world, "e2e_frac": e2["value"] / world / pcie_peak,
                "verified": bool(val["all_verified"] and e2["all_verified"])}
    for k, v in tried.items():
        if k != variant:
            roofline[f"value_{k.replace(':', '_')}"] = v["value"]
    if pcie_conc is not None:
        # N > 1: what the host gives N links at once is the meaningful denominator
        agg_out = sum(r[1] for r in per_rank)
        agg_in = sum(r[2] for r in per_rank)
        conc_h2d = sum(r[0] for r in pcie_conc)
        conc_d2h = sum(r[1] for r in pcie_conc)
        conc_bidir = sum(r[2] for r in pcie_conc)
        roofline.update({
            "swap_out_aggregate": agg_out, "swap_in_aggregate": agg_in,
            "concurrent_d2h_aggregate": conc_d2h, "concurrent_h2d_aggregate": conc_h2d,
            "concurrent_bidir_aggregate": conc_bidir,
            "frac_out_vs_concurrent": agg_out / conc_d2h, "frac_in_vs_concurrent": agg_in / conc_h2d,
            "frac_vs_concurrent_bidir": val["value"] / conc_bidir,
            "concurrent_note": "cudaMemcpyAsync with every rank copying at once: one direction (8 x 1 GiB) and both "
                               "directions on two streams (4 + 4 x 1 GiB, both directions' bytes over the time "
                               "until both are done); roofline.peak is one link alone"})
    if alloc_leg is not None:
        roofline.update({"e2e_allocator_slots_gbs": alloc_leg["value"],
                         "e2e_allocator_slots_frac": alloc_leg["value"] / pcie_peak,
                         "e2e_allocator_slots_verified": alloc_leg["verified"]})
    if config4 is not None:
        roofline.update({"config4_value": config4["value"], "config4_ms_per_step": config4["ms_per_step"],
                         "config4_swap_out_GBps_per_gpu": config4["swap_out_GBps_per_gpu_mean"],
                         "config4_swap_in_GBps_per_gpu": config4["swap_in_GBps_per_gpu_mean"],
                         "config4_verified": config4["verified"]})
    if overlap is not None:
        roofline.update({"overlap_gemm_slowdown_pct": overlap["gemm_slowdown_pct"],
                         "overlap_swap_in_gbs": overlap["swap_in_gbs"], "overlap_swap_out_gbs": overlap["swap_out_gbs"],
                         "overlap_both_directions_gbs": overlap["both_directions_gbs"],
                         "overlap_one_stream_swap_in_gbs": overlap["one_stream_swap_in_gbs"],
                         "overlap_one_stream_swap_out_gbs": overlap["one_stream_swap_out_gbs"],
                         "overlap_one_stream_gemm_slowdown_pct": overlap["one_stream_gemm_slowdown_pct"],
                         "overlap_one_stream_swap_in_gbs_no_gemm": overlap["one_stream_swap_in_gbs_no_gemm"],
                         "overlap_one_stream_swap_out_gbs_no_gemm": overlap["one_stream_swap_out_gbs_no_gemm"],
                         "overlap_swap_in_gbs_no_gemm": overlap["swap_in_gbs_no_gemm"],
                         "overlap_swap_out_gbs_no_gemm": overlap["swap_out_gbs_no_gemm"],
                         "overlap_gemm_tflops": overlap["gemm_tflops"], "overlap_verified": overlap["verified"]})
    line = {"metric": "kv_swap_GBps", "value": val["value"], "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": val["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic", "config": config,
            "per_gpu": val["value"] / world, "e2e": e2e, "gpu_launches": launches_value, "roofline": roofline,
            "verified": roofline["verified"], "clocks": clocks, "status_word": val["status"] | e2["status"],
            "mover": args.mover, "aiv": args.aiv or "default", "pcie_memcpy_peak": pcie,
            "verify": {"what": "after each timed leg, the last step's host slots against their source blocks and the "
                               "swapped-in blocks against their slots, every layer, K and V, on every rank; plus "
                               "the CPU oracle on a sample", "bytes_checked_rank0": val["verify"]["bytes_checked"],
                       "mismatches_rank0": val["verify"]["mismatches"]},
            "pcie_memcpy_concurrent_per_rank": None if pcie_conc is None else
            [{"rank": i, "h2d": r[0], "d2h": r[1], "bidir_total": r[2]} for i, r in enumerate(pcie_conc)],
            "per_rank": [{"rank": i, "numa_node": int(r[0]), "pci_bus": "%02x" % int(r[4]), "swap_out_GBps": r[1],
                          "swap_in_GBps": r[2], "ms_per_step": r[3], "verified": bool(r[5])}
                         for i, r in enumerate(per_rank)],
            "host": {"cpus": os.cpu_count(), "mem_available_GB": round(mem_available_bytes() / 1e9, 1)}}
    if extra:
        line["variants"] = extra
    if alloc_leg is not None:
        line["allocator_slots"] = alloc_leg
    if beside is not None:
        line["beside_gemm"] = beside
    if config4 is not None:
        line["config4"] = config4
    if overlap is not None:
        line["overlap"] = overlap
    if gather is not None:
        gr, gsrc = traffic_ratio("paged_gather_kernel", 0.9957)
        gather["roofline"] = {"bound": "hbm", "kernel": "paged_gather_*_kernel", "achieved": gather["value"],
                              "peak": hbm_peak, "unit": "GB/s", "frac": gather["value"] / hbm_peak,
                              "traffic": int(gr * gather["algorithmic_bytes"]), "traffic_source": gsrc,
                              "peak_source": hbm_src, "nominal": 8000.0}
        roofline.update({"gather_achieved": gather["value"], "gather_frac_of_hbm": gather["value"] / hbm_peak,
                         "gather_verified": gather["verified"]})
        line["gather"] = gather
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_swap(g, 10, 1)
    print(json.dumps(line), flush=True)
    ctx.close()


# Issue orders of a step that are timed when several ranks share the host (see SwapBench): which one
# is faster depends on the host — how far its device->host path sags with several links writing at
# once — so the default run measures them and reports the faster.
MULTI_GPU_VARIANTS = ("bidir_paced", "stagger")
# Layers per launch of the prefetch pipeline in the default line's `overlap` run.
DEFAULT_PREFETCH_GROUP = 4
VARIANT_TEXT = {
    "sequential": "swap-out then swap-in of the same slots, one stream",
    "stagger": "odd ranks swap-in (the previous step's slots) first, even ranks swap-out first",
    "bidir": "swap-out and swap-in (the previous step's slots) concurrently on two streams per rank",
    "bidir_paced": "swap-out (stores paced to 40 GB/s) and swap-in (the previous step's slots) concurrently on two "
                   "streams per rank",
    "interleave": "each step cut into k parts, swap-out and swap-in parts alternating; odd ranks start with swap-in",
}


if __name__ == "__main__":
    main()
