"""Seeded synthetic workloads with the shapes of the five benchmark configurations.

The reference measures on synthetic tensors (pcieThrough/tests/test_transfer_kernel.py:28-37,
test_gather.py:35-47); the configurations here name model *layouts* (Llama-3-8B / 70B TP8,
Qwen2-7B-style fp8) and stand in for serving traffic.  The generators are plain torch CPU code
used by the benchmark, the tests and the CPU oracle alike; nothing here computes a result.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence

import torch


@dataclass
class Geometry:
    name: str
    layers: int
    num_blocks: int      # device cache blocks per layer (K and V each)
    block_size: int
    kv_heads: int
    head_dim: int
    dtype: torch.dtype
    host_slots: int
    n_swap: int          # blocks per swap call
    seq_lens: List[int] = field(default_factory=list)

    @property
    def elt(self) -> int:
        return torch.empty((), dtype=self.dtype).element_size()

    @property
    def token_bytes(self) -> int:
        return self.kv_heads * self.head_dim * self.elt

    @property
    def block_bytes(self) -> int:
        return self.block_size * self.token_bytes

    def swap_bytes(self) -> int:
        """algorithmic bytes of one swap call, one direction"""
        return self.n_swap * self.layers * 2 * self.block_bytes


FP8 = getattr(torch, "float8_e4m3fn", torch.uint8)

CONFIGS = {
    # tiny Llama-style cache, fp16, the CPU-runnable case
    "tiny": Geometry("tiny", 2, 64, 16, 8, 128, torch.float16, 128, 8, [40, 100]),
    # Llama-3-8B KV layout, 512-block swap, 1.07 GB per direction
    "llama3_8b_swap": Geometry("llama3_8b_swap", 32, 20000, 16, 8, 128, torch.bfloat16, 40000, 512),
    # paged gather, Llama-3-8B layout, 64 sequences of 512..8192 tokens in a 40000-block cache
    "llama3_8b_gather": Geometry("llama3_8b_gather", 32, 40000, 16, 8, 128, torch.bfloat16, 0, 0),
    # Llama-3-70B TP8 shard: 1 kv head, 128-token blocks
    "llama3_70b_tp8_swap": Geometry("llama3_70b_tp8_swap", 80, 6000, 128, 1, 128, torch.bfloat16, 24000, 2048),
    # Qwen2-7B-style fp8 cache, layer-wise prefetch of 256 blocks
    "qwen2_7b_fp8_prefetch": Geometry("qwen2_7b_fp8_prefetch", 28, 8192, 16, 4, 128, FP8, 16384, 256),
}


def gather_seq_lens(seed: int = 0, num_seqs: int = 64, lo: int = 512, hi: int = 8192) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (num_seqs,), generator=g).tolist()


def random_kv_bytes(shape: Sequence[int], dtype: torch.dtype, seed: int) -> torch.Tensor:
    """Seeded cache contents: N(0,1) for float types; for fp8 e4m3 uniform random bytes
    without the two NaN codes 0x7F / 0xFF."""
    g = torch.Generator().manual_seed(seed)
    if dtype in (torch.float16, torch.bfloat16, torch.float32):
        return torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype)
    if dtype == torch.int8:
        return torch.randint(-128, 128, tuple(shape), generator=g, dtype=torch.int8)
    raw = torch.randint(0, 254, tuple(shape), generator=g, dtype=torch.int16)
    # map 0..253 onto the byte codes with 0x7F and 0xFF left out
    raw = raw + (raw >= 0x7F).to(torch.int16)
    raw = raw.to(torch.uint8)
    assert not bool(((raw == 0x7F) | (raw == 0xFF)).any())
    return raw.view(dtype) if dtype != torch.uint8 else raw


def distinct_ids(n: int, universe: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randperm(universe, generator=g)[:n].to(torch.int64)


def block_tables_for(seq_lens: Sequence[int], block_size: int, num_blocks: int, seed: int) -> torch.Tensor:
    """[num_seqs, max_blocks] int64; the rows are disjoint slices of one seeded permutation of
    the cache's blocks, unused entries are -1."""
    nbs = [(n + block_size - 1) // block_size for n in seq_lens]
    perm = torch.randperm(num_blocks, generator=torch.Generator().manual_seed(seed))
    assert sum(nbs) <= num_blocks
    table = torch.full((len(seq_lens), max(nbs) if nbs else 0), -1, dtype=torch.int64)
    pos = 0
    for s, nb in enumerate(nbs):
        table[s, :nb] = perm[pos:pos + nb]
        pos += nb
    return table
