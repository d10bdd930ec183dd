"""Multi-GPU plumbing of the data path: one process per GPU, no collective on the data.

Each rank swaps its own tensor-parallel KV-head shard between its own cache and its own
NUMA-local pool over its own PCIe link (the reference likewise assumes one device per
process, common/csrc/managed_memory/managed_mem.cpp:245-266).  torch.distributed is used
for two things only: a start barrier so that all links are loaded during the same window,
and the max-over-ranks of the device-side time.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Tuple

import torch


@dataclass
class RankContext:
    rank: int
    local_rank: int
    world: int
    dist: object = None      # torch.distributed when world > 1
    device: object = None

    @classmethod
    def from_env(cls) -> "RankContext":
        return cls(int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
                   int(os.environ.get("WORLD_SIZE", "1")))

    def init(self, backend: str, device=None) -> "RankContext":
        self.device = device
        if self.world > 1:
            import torch.distributed as dist

            if not dist.is_initialized():
                kw = {"device_id": device} if (backend == "nccl" and device is not None) else {}
                dist.init_process_group(backend, rank=self.rank, world_size=self.world, **kw)
            self.dist = dist
        return self

    def barrier(self) -> None:
        if self.dist is not None:
            self.dist.barrier()
        if self.device is not None and torch.device(self.device).type == "cuda":
            torch.cuda.synchronize(self.device)

    def max_over_ranks(self, x: float) -> float:
        if self.dist is None:
            return float(x)
        t = torch.tensor([x], dtype=torch.float64, device=self.device if self.device is not None else "cpu")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def gather_floats(self, values) -> List[List[float]]:
        """Every rank's vector of floats, in rank order, on every rank (per-GPU figures for the report)."""
        if self.dist is None:
            return [[float(v) for v in values]]
        dev = self.device if self.device is not None else "cpu"
        mine = torch.tensor([float(v) for v in values], dtype=torch.float64, device=dev)
        out = [torch.zeros_like(mine) for _ in range(self.world)]
        self.dist.all_gather(out, mine)
        return [t.tolist() for t in out]

    def close(self) -> None:
        if self.dist is not None and self.dist.is_initialized():
            self.dist.destroy_process_group()
        self.dist = None


def spread_device_index(local_rank: int, world: int, visible: int) -> int:
    """GPU ordinal for a local rank when fewer ranks than visible GPUs run: ranks are spread evenly
    over the ordinals (0 and 4 of 8 for two ranks, 0, 2, 4, 6 for four).  CUDA orders devices by PCI
    bus, so neighbouring ordinals tend to hang off the same host bridge; spreading the ranks gives each
    its own share of the host's PCIe and memory paths.  With world == visible it is the identity."""
    if visible <= 0 or world >= visible:
        return local_rank % max(visible, 1)
    return (local_rank * visible) // world


def rank_id_sets(rank: int, n_sets: int, n_swap: int, num_blocks: int, host_slots: int,
                 seed: int = 1234) -> List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
    """Per-rank seeded id lists for `n_sets` steps: (device ids to swap out, host slots, device ids to
    swap in).  Within a set each list holds distinct ids and the swap-in ids differ from the swap-out
    ids (the blocks come back to *other* device blocks); the slots of consecutive sets are disjoint, so a
    step may read the previous step's slots while it writes its own.  Different ranks get different
    lists.  Needs num_blocks >= 2*n_swap and host_slots >= 2*n_swap."""
    assert num_blocks >= 2 * n_swap and host_slots >= 2 * n_swap, "pools too small for disjoint id sets"
    gen = torch.Generator().manual_seed(seed + rank)
    sets = []
    prev_slots = torch.empty(0, dtype=torch.int64)
    for _ in range(n_sets):
        blocks = torch.randperm(num_blocks, generator=gen)
        out_ids, in_ids = blocks[:n_swap], blocks[n_swap:2 * n_swap]
        cand = torch.randperm(host_slots, generator=gen)[:2 * n_swap]
        if prev_slots.numel():
            cand = cand[~torch.isin(cand, prev_slots)]
        slots = cand[:n_swap]
        prev_slots = slots
        sets.append((out_ids.clone(), slots.clone(), in_ids.clone()))
    return sets


def aggregate_gbs(bytes_per_rank_per_step: int, world: int, ms_per_step_max: float) -> float:
    """Whole-job GB/s: the bytes all ranks moved in a step over the slowest rank's step time."""
    return world * bytes_per_rank_per_step / (ms_per_step_max * 1e-3) / 1e9


def host_pool_slots(wanted: int, slot_bytes: int, n_swap: int, world: int, mem_available: int,
                    fraction: float = 0.6) -> Tuple[int, str]:
    """Slots each rank may pin: the host's available memory is shared by `world` ranks.  The pool is
    shrunk when it does not fit; the transferred set (n_swap blocks) never is."""
    budget = int(mem_available * fraction / max(world, 1))
    if wanted * slot_bytes <= budget:
        return wanted, ""
    slots = max(2 * n_swap, budget // slot_bytes)
    return slots, f"host pool shrunk to {slots} slots (MemAvailable), transferred set unchanged"
