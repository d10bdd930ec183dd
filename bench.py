#!/usr/bin/env python
"""Benchmark of the KV-cache data path: multi-layer paged-KV swap over PCIe (headline) and the
paged gather in HBM (secondary, single-GPU runs).

    python bench.py --gpus N --steps K --warmup W          # this implementation
    python bench.py --impl reference ...                    # the CPU restatement on the host cores

A *step* is one pass of the hot path over one batch: one swap-out call (HBM -> pinned host pool)
followed by one swap-in call (host pool -> HBM, other device blocks) of the workload's block
count, all layers, K and V.  Each rank owns its own cache, pool and PCIe link; there is no
collective on the data path, so scaling is weak (per-GPU work fixed).  torch.distributed is used
only for the start barrier and the max-over-ranks reduction of the device-side time.

Prints ONE JSON line (rank 0).  `value` is the whole-job GB/s with the id lists resident on the
device; `e2e` drives the same step through the public API (PagedKVCache.swap_out / swap_in) with
host-resident id lists and reads the status word back every step.
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
        ids = o.distinct_ids(g.n_swap, nb, 10 + s)
        slots = o.distinct_ids(g.n_swap, nb, 20 + s)
        back = o.distinct_ids(g.n_swap, nb, 30 + s)
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
    """cudaMemcpyAsync rate with EVERY rank copying at the same time: 8 back-to-back copies of 1 GiB per
    direction after a barrier.  This is the denominator for N > 1: what the host (root complexes, memory)
    gives N links at once, as opposed to one link alone."""
    n = min(pool_u8.numel(), 1 << 30)
    host = pool_u8[:n]
    dev = torch.empty(n, dtype=torch.uint8, device=device)
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
    del dev
    return res


# --------------------------------------------------------------------------- gather leg
def bench_gather(device, steps: int, warmup: int, mover, aiv, num_seqs: int = 64) -> dict:
    """Paged gather, Llama-3-8B layout: 64 sequences of 512..8192 tokens (seeded), block tables that are
    disjoint slices of a seeded permutation of a 40000-block cache, all 32 layers, K and V, one launch."""
    from heterofusedkernels_b200.connector import PagedKVCache
    from oracle import kv_oracle as o

    layers, nblocks, bs, heads, hd = 32, 40000, 16, 8, 128
    lens = o.gather_seq_lens(seed=0)[:num_seqs]
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
    tables = o.block_tables_for(lens, bs, nblocks, seed=1).to(device)
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
    # spot check against torch indexing on the device (layer 3, K, sequence 5)
    s5 = min(5, len(lens) - 1)
    nb5 = (lens[s5] + bs - 1) // bs
    ref = cache.k_caches[3][tables[s5, :nb5]].flatten(0, 1)[:lens[s5]]
    start = sum(lens[:s5])
    ok = torch.equal(ref.view(torch.int16), k_out[3, start:start + lens[s5]].view(torch.int16))
    mean_ms = sum(ms) / len(ms)
    res = {"workload": "llama3_8b_gather", "total_tokens": total, "num_seqs": len(lens), "layers": layers,
           "algorithmic_bytes": algo, "ms_per_launch": mean_ms, "best_ms": min(ms),
           "value": algo / (mean_ms * 1e-3) / GB, "unit": "GB/s", "status_word": status, "spot_check_ok": bool(ok),
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
        for r in range(5):
            op(table, big_dst, big_ids[r], None)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for r in range(run_count // 10):
            op(table, big_dst, big_ids[r], None)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        row["combine_ms_per_call"] = dt / (run_count // 10) * 1e3
        row["combine_GBps"] = bs * run_count * dim * 2 / dt / GB
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
def bench_overlap(g, device, args, pkg) -> dict:
    """Layer-wise prefetch pipeline (Qwen2-7B-style fp8 cache, 28 layers): while a bf16
    [8192x3584]x[3584x18944] GEMM runs for layer l on the main stream, 256 blocks of layer l+1 are
    swapped in on a side stream and 256 other blocks of layer l are swapped out on a second one.
    Reports swap GB/s per direction under overlap and the GEMM slowdown, per data mover."""
    from heterofusedkernels_b200.connector import LayerwisePrefetcher, PagedKVCache

    cache = PagedKVCache(g.layers, g.num_blocks, g.block_size, g.kv_heads, g.head_dim, g.dtype, device,
                         host_slots=g.host_slots)
    fill_random_bytes(cache._k_store, 1)
    fill_random_bytes(cache._v_store, 2)
    pf = LayerwisePrefetcher(cache)
    a = torch.randn(8192, 3584, device=device, dtype=torch.bfloat16)
    b = torch.randn(3584, 18944, device=device, dtype=torch.bfloat16)
    c = torch.empty(8192, 18944, device=device, dtype=torch.bfloat16)
    flops = 2 * 8192 * 3584 * 18944
    L = g.layers
    gen = torch.Generator().manual_seed(5)
    ids = []
    for l in range(L):
        perm = torch.randperm(g.num_blocks, generator=gen)
        sl = torch.randperm(g.host_slots, generator=gen)
        ids.append((perm[:g.n_swap].to(device), sl[:g.n_swap].to(device),
                    perm[g.n_swap:2 * g.n_swap].to(device), sl[g.n_swap:2 * g.n_swap].to(device)))
    cpu_ids = [tuple(t.cpu() for t in x) for x in ids]
    layer_bytes = g.n_swap * 2 * g.block_bytes
    main = torch.cuda.current_stream()

    def gemm_pass():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(L):
            torch.matmul(a, b, out=c)
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1)

    def swap_only(kind, ctas):
        """both directions concurrently, no GEMM: the swap's own rate"""
        return overlapped(kind, ctas, with_gemm=False)

    def overlapped(kind, ctas, with_gemm=True):
        # kind: "vector", "copy_engine", "bulk" (library ring) or "bulk@<stage bytes>x<stages>": smaller
        # rings let the single-warp CTAs fit next to the GEMM's CTAs on an SM
        mv = pkg.capi.MOVER_VECTOR if kind == "vector" else (pkg.capi.MOVER_BULK if kind.startswith("bulk") else None)
        ring = tuple(int(x) for x in kind.split("@")[1].split("x")) if "@" in kind else (0, 0)
        pkg.capi.lib().hfk_set_bulk_geometry(*ring)
        ev_in = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(L)]
        ev_out = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(L)]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        pf.in_stream.wait_event(e0)
        pf.out_stream.wait_event(e0)
        for l in range(L):
            nxt = (l + 1) % L
            in_ids, in_slots, out_ids, out_slots = ids[l]
            if kind == "copy_engine":
                ci = cpu_ids[l]
                with torch.cuda.stream(pf.in_stream):
                    ev_in[l][0].record()
                    torch.ops.pcie_through.swap_in_copy_engine(cache.k_ptrs_cpu[nxt:nxt + 1], cache.v_ptrs_cpu[nxt:nxt + 1],
                                                               pf.pools[nxt], ci[0], ci[1], cache.num_blocks)
                    ev_in[l][1].record()
                with torch.cuda.stream(pf.out_stream):
                    ev_out[l][0].record()
                    torch.ops.pcie_through.swap_out_copy_engine(cache.k_ptrs_cpu[l:l + 1], cache.v_ptrs_cpu[l:l + 1],
                                                                pf.pools[l], ci[2], ci[3], cache.num_blocks)
                    ev_out[l][1].record()
            else:
                with torch.cuda.stream(pf.in_stream):
                    ev_in[l][0].record()
                pf.prefetch(nxt, in_ids, in_slots, aiv=ctas, mover=mv)
                with torch.cuda.stream(pf.in_stream):
                    ev_in[l][1].record()
                with torch.cuda.stream(pf.out_stream):
                    ev_out[l][0].record()
                pf.evict(l, out_ids, out_slots, aiv=ctas, mover=mv)
                with torch.cuda.stream(pf.out_stream):
                    ev_out[l][1].record()
            if with_gemm:
                torch.matmul(a, b, out=c)
        e1.record()
        main.wait_stream(pf.in_stream)
        main.wait_stream(pf.out_stream)
        torch.cuda.synchronize()
        t_in = [x.elapsed_time(y) for x, y in ev_in]
        t_out = [x.elapsed_time(y) for x, y in ev_out]
        return {"main_ms": e0.elapsed_time(e1), "in_gbs": layer_bytes / (statistics.median(t_in) * 1e-3) / GB,
                "out_gbs": layer_bytes / (statistics.median(t_out) * 1e-3) / GB,
                "in_ms_median": statistics.median(t_in), "out_ms_median": statistics.median(t_out)}

    # The GEMM runs under the 1 kW power cap, so its time drifts by several percent as the part
    # warms up.  Warm up for about two seconds, then alternate alone / overlapped passes and compare
    # medians taken over the same stretch of time.
    t_warm = time.perf_counter()
    while time.perf_counter() - t_warm < 2.0:
        gemm_pass()
    sampler = ClockSampler(device.index or 0)
    variants = []
    alone_all = []
    reps = 7
    for kind, ctas in (("bulk", 2), ("bulk", 4), ("bulk", 8), ("bulk", 16), ("bulk@4096x8", 8), ("bulk@4096x8", 16),
                       ("bulk@2048x4", 32), ("bulk@2048x8", 16), ("bulk@2048x8", 32), ("bulk@2048x8", 64),
                       ("bulk@4096x4", 16), ("bulk@4096x4", 32), ("vector", 4), ("vector", 8), ("vector", 16),
                       ("vector", 32), ("copy_engine", 0)):
        overlapped(kind, ctas)  # warm-up
        alone, runs = [], []
        for _ in range(reps if kind != "copy_engine" else 3):
            alone.append(gemm_pass())
            runs.append(overlapped(kind, ctas))
        alone_all += alone
        t_a = statistics.median(alone)
        med_main = statistics.median(r["main_ms"] for r in runs)
        solo = swap_only(kind, ctas)
        variants.append({"mover": kind, "ctas_per_direction": ctas, "gemm_ms_alone": t_a,
                         "gemm_ms_overlapped": med_main, "gemm_slowdown_pct": 100.0 * (med_main / t_a - 1.0),
                         "swap_in_gbs": statistics.median(r["in_gbs"] for r in runs),
                         "swap_out_gbs": statistics.median(r["out_gbs"] for r in runs),
                         "swap_in_gbs_no_gemm": solo["in_gbs"], "swap_out_gbs_no_gemm": solo["out_gbs"]})
    pkg.capi.lib().hfk_set_bulk_geometry(0, 0)
    t_alone = statistics.median(alone_all)
    t_alone2 = statistics.median([gemm_pass() for _ in range(3)])
    clocks = sampler.stop()
    status = cache.status()
    ok = [v for v in variants if v["mover"] in ("bulk", "vector") and v["gemm_slowdown_pct"] < 10.0]
    pick = max(ok or variants, key=lambda v: v["swap_in_gbs"] + v["swap_out_gbs"])
    return {"metric": "kv_swap_GBps_under_gemm_overlap", "value": (pick["swap_in_gbs"] + pick["swap_out_gbs"]) / 2,
            "unit": "GB/s", "n_gpus": 1, "steps": reps, "warmup": 1, "ms_per_step": pick["gemm_ms_overlapped"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": g.name, "layers": L, "blocks_per_layer_per_direction": g.n_swap,
                       "bytes_per_layer_per_direction": layer_bytes, "kv_dtype": "float8_e4m3fn",
                       "device_blocks": g.num_blocks, "host_slots": g.host_slots,
                       "gemm": "bf16 [8192x3584]x[3584x18944] per layer (torch.matmul)",
                       "pool sizes": "8192 device / 16384 host blocks (not fixed by the configuration; chosen here)"},
            "gemm_alone_ms": t_alone, "gemm_alone_ms_after": t_alone2, "gemm_alone_tflops": L * flops / (t_alone * 1e-3) / 1e12,
            "picked": pick, "variants": variants, "clocks": clocks, "status_word": status,
            "gpu_launches": 2 * L * reps}


# --------------------------------------------------------------------------- main
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="llama3_8b_swap")
    ap.add_argument("--mover", default="auto", choices=["auto", "vector", "bulk", "staged"])
    ap.add_argument("--staging-mb", type=int, default=1024, help="staging buffer of the staged mover (MiB)")
    ap.add_argument("--aiv", type=int, default=0, help="CTAs per swap kernel (0 = library default)")
    ap.add_argument("--gather-aiv", type=int, default=0)
    ap.add_argument("--host-slots", type=int, default=0, help="override the host pool size (slots)")
    ap.add_argument("--device-blocks", type=int, default=0, help="override the device cache size (blocks)")
    ap.add_argument("--no-spread", action="store_true", help="use GPU ordinal = LOCAL_RANK even when more GPUs are visible")
    ap.add_argument("--stagger", type=int, default=1, help="N > 1: odd ranks run swap-in before swap-out (1) or not (0)")
    ap.add_argument("--no-gather", action="store_true")
    ap.add_argument("--gather-only", action="store_true", help="run only the paged-gather leg")
    ap.add_argument("--gather-seqs", type=int, default=64, help="sequences in the gather batch")
    ap.add_argument("--gather-hints", type=int, default=-1, help="L2 hints of the bulk gather (-1 = library default)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

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
        cb = cpu_baseline_swap(g, args.steps, min(args.warmup, 1), budget_s=120.0)
        line = {"impl": "reference", "metric": "kv_swap_GBps", "value": cb["value"], "unit": "GB/s",
                "n_gpus": args.gpus, "steps": cb["steps"], "warmup": min(args.warmup, 1),
                "ms_per_step": cb["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "u8", "data": "synthetic", "config": config, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    import heterofusedkernels_b200 as pkg
    from heterofusedkernels_b200.connector import PagedKVCache

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    pkg.load_ops()
    if args.gather_hints >= 0:
        pkg.capi.check(pkg.capi.lib().hfk_set_gather_tuning(args.gather_hints, -1), "hfk_set_gather_tuning")
    # fewer ranks than visible GPUs: spread them over the PCI bus order (ranks.spread_device_index)
    dev_index = local_rank if args.no_spread else ranks.spread_device_index(local_rank, world, torch.cuda.device_count())
    torch.cuda.set_device(dev_index)
    device = torch.device("cuda", dev_index)
    ctx.init("nccl", device)
    barrier, max_over_ranks = ctx.barrier, ctx.max_over_ranks

    mover = {"auto": None, "vector": pkg.capi.MOVER_VECTOR, "bulk": pkg.capi.MOVER_BULK, "staged": None}[args.mover]
    staged = args.mover == "staged"
    aiv = args.aiv if args.aiv > 0 else None

    if args.gather_only:
        res = bench_gather(device, args.steps, args.warmup, mover, args.gather_aiv if args.gather_aiv > 0 else None,
                           args.gather_seqs)
        print(json.dumps({"metric": "paged_gather_GBps", "value": res["value"], "unit": "GB/s", "n_gpus": 1,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_launch"],
                          "higher_is_better": True, "dtype": "u8", "data": "synthetic", "gpu_launches": args.steps,
                          "config": {"workload": "llama3_8b_gather", "num_seqs": args.gather_seqs}, "gather": res}),
              flush=True)
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
    fill_random_bytes(cache._k_store, 100 + rank)
    fill_random_bytes(cache._v_store, 200 + rank)
    config.update({"host_slots": host_slots, "host_pool_bytes": host_slots * slot_bytes, "pool_note": pool_note,
                   "host_pool_layout": "[slot][layer][K|V][block] (2 MiB-class contiguous per slot)",
                   "numa_node": pkg.memory.device_numa_node(), "pool_setup_s": round(setup_pool_s, 2),
                   "gpu_ordinal_of_rank": "spread over the visible GPUs in PCI bus order" if not args.no_spread
                   else "LOCAL_RANK", "visible_gpus": torch.cuda.device_count(),
                   "direction_order": "odd ranks swap-in first, even ranks swap-out first" if (args.stagger and world > 1)
                   else "swap-out then swap-in on every rank"})

    n_sets = args.warmup + args.steps
    sets = ranks.rank_id_sets(rank, n_sets, g.n_swap, g.num_blocks, host_slots)
    dev_sets = [tuple(t.to(device) for t in s) for s in sets]
    pin_sets = [tuple(t.pin_memory() for t in s) for s in sets]

    pcie = measure_pcie_peak(cache._host_raw.view(torch.uint8), device) if rank == 0 else None
    barrier()
    pcie_conc = None
    if world > 1:
        mine = measure_pcie_concurrent(ctx, cache._host_raw.view(torch.uint8), device)
        pcie_conc = ctx.gather_floats([mine["h2d"], mine["d2h"]])

    def do_out(dev_ids, slots_dev, slots_cpu):
        if staged:
            cache.swap_out_staged(dev_ids, slots_cpu, staging_bytes=args.staging_mb << 20)
        else:
            cache.swap_out(dev_ids, slots_dev, aiv=aiv, mover=mover)

    def do_in(dev_ids, slots_dev, slots_cpu):
        if staged:
            cache.swap_in_staged(dev_ids, slots_cpu, staging_bytes=args.staging_mb << 20)
        else:
            cache.swap_in(dev_ids, slots_dev, aiv=aiv, mover=mover)

    # ---- value leg: ids resident on the device, kernels only -----------------------------
    # With several ranks the odd ones run each step's two calls in the other order (swap-in of a slot
    # set first, then the swap-out), so that at any time about half the links carry host->device and
    # half device->host traffic: the host's paths are full duplex, and all ranks writing at once or
    # all reading at once leaves one direction idle.
    in_first = bool(args.stagger and world > 1 and rank % 2 == 1)

    def run_value():
        evs = []
        for s in range(n_sets):
            o_ids, slots, i_ids = dev_sets[s]
            if s == args.warmup:
                barrier()
                t_start.record()
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            e[0].record()
            if in_first:
                do_in(i_ids, slots, sets[s][1])
            else:
                do_out(o_ids, slots, sets[s][1])
            e[1].record()
            if in_first:
                do_out(o_ids, slots, sets[s][1])
            else:
                do_in(i_ids, slots, sets[s][1])
            e[2].record()
            if s >= args.warmup:
                evs.append(e)
        t_end.record()
        barrier()
        return evs

    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(dev_index) if rank == 0 else None
    evs = run_value()
    clocks = sampler.stop() if sampler else None
    total_ms = max_over_ranks(t_start.elapsed_time(t_end))
    ms_per_step = total_ms / args.steps
    first_ms = [e[0].elapsed_time(e[1]) for e in evs]
    second_ms = [e[1].elapsed_time(e[2]) for e in evs]
    out_ms, in_ms = (second_ms, first_ms) if in_first else (first_ms, second_ms)
    status = cache.status()
    value = ranks.aggregate_gbs(2 * g.swap_bytes, world, ms_per_step)
    bus = (C.c_char * 32)()
    pkg.capi.lib().hfk_device_pci_bus_id(-1, bus, 32)
    per_rank = ctx.gather_floats([pkg.memory.device_numa_node(), g.swap_bytes / (statistics.mean(out_ms) * 1e-3) / GB,
                                  g.swap_bytes / (statistics.mean(in_ms) * 1e-3) / GB,
                                  t_start.elapsed_time(t_end) / args.steps, int(bus.value.decode().split(":")[1], 16)])

    # ---- e2e leg: public API, host-resident id lists, status read back every step ------------
    e2e_start, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    status_host = torch.zeros(1, dtype=torch.int64)
    for s in range(n_sets):
        o_ids, slots, i_ids = pin_sets[s]
        if s == args.warmup:
            barrier()
            e2e_start.record()
        if in_first:
            do_in(i_ids, slots, sets[s][1])  # ids: pinned host -> device inside the call
            do_out(o_ids, slots, sets[s][1])
        else:
            do_out(o_ids, slots, sets[s][1])
            do_in(i_ids, slots, sets[s][1])
        status_host[0] = cache.status()                         # device -> host read of the step's result
    e2e_end.record()
    barrier()
    e2e_ms = max_over_ranks(e2e_start.elapsed_time(e2e_end)) / args.steps
    id_bytes = 4 * g.n_swap * 8
    e2e = {"value": world * 2 * g.swap_bytes / (e2e_ms * 1e-3) / GB, "unit": "GB/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": g.swap_bytes + id_bytes, "d2h_bytes_per_step": g.swap_bytes + 4,
           "api": "PagedKVCache.swap_out/swap_in -> torch.ops.pcie_through.swap_out/swap_in; payload moves "
                  "between HBM and the pinned host pool inside the timed region"}

    # ---- gather leg (single-GPU runs) ------------------------------------------------------
    host_pool_keepalive = cache  # noqa: F841
    gather = None
    if world == 1 and not args.no_gather and g.name != "tiny":
        del cache, host_pool_keepalive, dev_sets
        torch.cuda.empty_cache()
        gather = bench_gather(device, max(args.steps, 5), args.warmup, mover,
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
    out_gbs = g.swap_bytes / (statistics.mean(out_ms) * 1e-3) / GB
    in_gbs = g.swap_bytes / (statistics.mean(in_ms) * 1e-3) / GB
    achieved = 2 * g.swap_bytes / ((statistics.mean(out_ms) + statistics.mean(in_ms)) * 1e-3) / GB
    pcie_peak = (pcie["h2d"] + pcie["d2h"]) / 2
    roofline = {"bound": "pcie", "kernel": "kv_swap_*_kernel (swap-out and swap-in launches)",
                "achieved": achieved, "peak": pcie_peak, "unit": "GB/s", "frac": achieved / pcie_peak,
                "traffic": int(1.0841e9 * g.swap_bytes / 1073741824),
                "traffic_source": "dram__bytes_read+write of one ncu capture of the swap-out launch at this step size "
                                  "(1.0769 GB read + 0.0072 GB written per 1.0737 GB moved), scaled by bytes moved",
                "peak_source": "live cudaMemcpyAsync of 1 GiB pinned<->device, best of 5, mean of the two "
                               "directions (MEASURED_PEAKS.json holds no PCIe figure)",
                "swap_out": {"achieved": out_gbs, "peak": pcie["d2h"], "frac": out_gbs / pcie["d2h"]},
                "swap_in": {"achieved": in_gbs, "peak": pcie["h2d"], "frac": in_gbs / pcie["h2d"]},
                "nominal_gen5_x16": 63.0, "algorithmic_bytes_per_launch": g.swap_bytes}
    if pcie_conc is not None:
        # N > 1: what the host gives N links at once is the meaningful denominator
        agg_out = sum(r[1] for r in per_rank)
        agg_in = sum(r[2] for r in per_rank)
        conc_d2h = sum(r[1] for r in pcie_conc)
        conc_h2d = sum(r[0] for r in pcie_conc)
        roofline["all_ranks_concurrent"] = {
            "swap_out_aggregate": agg_out, "memcpy_d2h_aggregate": conc_d2h, "frac_out": agg_out / conc_d2h,
            "swap_in_aggregate": agg_in, "memcpy_h2d_aggregate": conc_h2d, "frac_in": agg_in / conc_h2d,
            "note": "cudaMemcpyAsync with every rank copying at once (8 x 1 GiB per direction after a barrier); "
                    "roofline.peak above is one link alone"}
    line = {"metric": "kv_swap_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic", "config": config,
            "per_gpu": value / world, "e2e": e2e, "gpu_launches": 2 * args.steps, "roofline": roofline,
            "clocks": clocks, "status_word": status, "mover": args.mover, "aiv": args.aiv or "default",
            "pcie_memcpy_peak": pcie,
            "pcie_memcpy_concurrent_per_rank": None if pcie_conc is None else
            [{"rank": i, "h2d": r[0], "d2h": r[1]} for i, r in enumerate(pcie_conc)],
            "per_rank": [{"rank": i, "numa_node": int(r[0]), "pci_bus": "%02x" % int(r[4]), "swap_out_GBps": r[1],
                          "swap_in_GBps": r[2], "ms_per_step": r[3]} for i, r in enumerate(per_rank)],
            "host": {"cpus": os.cpu_count(), "mem_available_GB": round(mem_available_bytes() / 1e9, 1)}}
    if gather is not None:
        gather["roofline"] = {"bound": "hbm", "kernel": "paged_gather_*_kernel", "achieved": gather["value"],
                              "peak": hbm_peak, "unit": "GB/s", "frac": gather["value"] / hbm_peak,
                              "traffic": int(0.9957 * gather["algorithmic_bytes"]),
                              "traffic_source": "one ncu capture of an 8-sequence batch (10.241 GB DRAM read+write for "
                                                "10.285 GB algorithmic), scaled by the tokens gathered",
                              "peak_source": hbm_src, "nominal": 8000.0}
        line["gather"] = gather
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_swap(g, 10, 1)
    print(json.dumps(line), flush=True)
    ctx.close()


if __name__ == "__main__":
    main()
