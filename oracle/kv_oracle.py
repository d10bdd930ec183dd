"""CPU oracle of the KV-cache data path.  TEST INFRASTRUCTURE ONLY.

Nothing that ships imports this file: only ``tests/``, ``__graft_entry__.smoke()``
and the CPU-baseline / reference legs of ``bench.py`` may, and there only as the
checker or the timed CPU baseline — never as the product path.

Two kinds of functions live here.

1. *Literal restatements* of the reference's device code, loop for loop, in numpy
   (``*_literal``).  They follow the AscendC index arithmetic, including the host
   tiling, so that the vectorised forms below can be checked against the
   reference's own algorithm and not only against themselves:
     - ``block_transfer_literal``: KVTransfer::MultiLayerBlockTransfer::Process /
       blockTransposeCopy (pcieThrough/csrc/kernel/multi_layer_block_transfer_kernel.h:42-82)
       with the plan of GenerateMultiLayerBlockTransferTiling
       (pcieThrough/csrc/host/tiling/multi_layer_block_transfer.cpp:19-56);
     - ``row_gather_literal``: Gather::MteCopy::init / LoadStoreFunc
       (pcieThrough/csrc/kernel/gather.h:35-134).
2. *Vectorised forms* on torch CPU tensors — the semantics the GPU path must
   reproduce bit for bit:
     - ``block_transfer``: ``dev[l] = host.permute(1, 2, 0, 3)[l]``, the property the
       reference's test asserts (pcieThrough/tests/test_transfer_kernel.py:77-83);
     - ``row_gather``: ``table.index_select(0, ids)``
       (pcieThrough/tests/test_gather.py:14-29);
     - ``swap_out`` / ``swap_in`` / ``paged_gather``: per-layer
       ``index_select`` / ``index_copy_`` — multi-block operators the reference does
       not have; their definition is the torch CPU form itself.

Pinning — PARITY UNPINNED in the strict sense.  The reference ships no golden vectors or known-answer files for this path:
its tests generate constant data at run time (test_transfer_kernel.py:32 fills the
pool with 2; test_gather.py:40-41 never writes the zero-filled table) and cannot be
imported here (they need torch_npu and an NPU).  The oracle is therefore pinned to the
two assertions those tests make (permute equality, row-by-row equality), checked on
seeded random data in ``tests/test_oracle.py``, and to the committed fixtures under
``tests/golden`` that ``tests/golden/make_golden.py`` generated from it.  Those are pins to
properties and to the oracle's own output, not to vectors produced by the reference: for the
multi-block operators (swap_out, swap_in, paged_gather, relayout_swap_*) no upstream
counterpart exists, so their parity is unpinned by construction.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import numpy as np
import torch

# ----------------------------------------------------------------------------
# 1. literal restatements of the reference kernels
# ----------------------------------------------------------------------------

UB_BYTES = 192 * 1024  # unified buffer of one AIV core (gather.h:43, tiling via GetCoreMemSize)


@dataclass
class TransferTiling:
    """MultiLayerBlockTransferTilingData (multi_layer_block_transfer_tiling.h:16-29)."""
    tokens_per_core: int
    tokens_per_inner_loop: int
    per_token_bytes: int


def transfer_tiling(aiv: int, elt: int, B: int, L: int, H: int, D: int, ub: int = UB_BYTES) -> TransferTiling:
    """GenerateMultiLayerBlockTransferTiling (tiling/multi_layer_block_transfer.cpp:19-56)."""
    tokens_per_core = (B + aiv - 1) // aiv                       # :34
    base = 2 * L * H * D * elt                                   # :37  (BUFF_NUM = 2)
    if not ub > base:                                            # :39
        raise ValueError("Per Token Buffer Size is greater than UBSize")
    max_tokens = (ub - 256) // base                              # :40-41
    max_tokens = min(tokens_per_core, max_tokens)                # :42
    if max_tokens <= 0:                                          # :43
        raise ValueError("Max tokens per loop on chip is less than or equal to 0")
    if (D * elt) % 32 or (L * H * D * elt) % 32:                 # :49-54 copy lengths in 32-byte units
        raise ValueError("copy lengths must be multiples of 32 bytes")
    return TransferTiling(tokens_per_core, max_tokens, L * H * D * elt)


def block_transfer_literal(host_block: np.ndarray, aiv: int = 2) -> List[np.ndarray]:
    """[B,L,H,D] host block -> L arrays [H,B,D], following kernel.h:42-82 loop for loop."""
    B, L, H, D = host_block.shape
    til = transfer_tiling(aiv, host_block.itemsize, B, L, H, D)
    flat = host_block.reshape(-1)
    dev = [np.zeros(H * B * D, dtype=host_block.dtype) for _ in range(L)]
    for core in range(aiv):                                      # Process(), kernel.h:74-82
        start = core * til.tokens_per_core
        end = min(B, start + til.tokens_per_core)
        tok = start
        while tok < end:
            n = min(til.tokens_per_inner_loop, end - tok)
            # stage 1 (:52): n tokens x (L*H*D) contiguous elements into the on-chip buffer
            first = tok * L * H * D
            ub = flat[first:first + n * L * H * D].copy()
            # stage 2 (:59-69): per (layer, head), n strided runs of D elements
            for l in range(L):
                for h in range(H):
                    src = l * H * D + h * D
                    dst = h * B * D + tok * D
                    for i in range(n):   # blockCount = n, srcStride skips the other (l,h) of a token
                        dev[l][dst + i * D: dst + (i + 1) * D] = ub[src + i * L * H * D: src + i * L * H * D + D]
            tok += til.tokens_per_inner_loop
    return [d.reshape(H, B, D) for d in dev]


def row_gather_literal(table: np.ndarray, ids: np.ndarray, aiv: int = 2) -> np.ndarray:
    """dst[i,:] = table[ids[i],:] with the core/round partition of gather.h:35-134."""
    num_ids = int(ids.shape[0])
    row_bytes = table.shape[1] * table.itemsize
    block_num = min(aiv, num_ids) if num_ids else 1              # gather_torch.cpp:48
    dst = np.zeros((num_ids, table.shape[1]), dtype=table.dtype)
    base, rem = divmod(num_ids, block_num)                       # gather.h:45-46
    slot = ids.itemsize
    per_round = UB_BYTES // (2 * (row_bytes + slot))             # :58
    per_round = per_round // (32 // slot) * (32 // slot)         # :62
    for b in range(block_num):
        n_mine = base + (1 if b < rem else 0)                    # :51
        first = b * base + (b if b < rem else rem)               # :52
        rounds = (n_mine + per_round - 1) // per_round if per_round else 0   # :63-64
        for r in range(rounds):
            n = per_round if r != rounds - 1 else n_mine - r * per_round    # :86-91
            ub = np.empty((n, table.shape[1]), dtype=table.dtype)
            for i in range(n):                                   # :106-112
                ub[i] = table[int(ids[first + r * per_round + i])]
            dst[first + r * per_round: first + r * per_round + n] = ub      # :119-122
    return dst


# ----------------------------------------------------------------------------
# 2. vectorised torch-CPU forms (the semantics to reproduce)
# ----------------------------------------------------------------------------

def _u8(t: torch.Tensor) -> torch.Tensor:
    """Byte view sharing storage with `t` (the path moves bytes; dtypes only set sizes)."""
    return t if t.dtype == torch.uint8 else t.view(torch.uint8)


def block_transfer(host_block: torch.Tensor) -> List[torch.Tensor]:
    """L tensors [H,B,D]: the permute the reference test asserts (test_transfer_kernel.py:81-82)."""
    return [x.contiguous() for x in host_block.permute(1, 2, 0, 3).unbind(0)]


def row_gather(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    return table.index_select(0, ids.to(torch.int64))


def swap_out(dev_k: Sequence[torch.Tensor], dev_v: Sequence[torch.Tensor], host_pool: torch.Tensor,
             device_block_ids: torch.Tensor, host_slot_ids: torch.Tensor) -> None:
    """host_pool[slot, l, kv] = cache_kv[l][block] for every layer, in place.

    dev_k / dev_v: per-layer CPU images of the device caches, [num_blocks, ...chunk dims];
    host_pool: [slots, layers, 2, ...chunk dims]."""
    ids = device_block_ids.to(torch.int64)
    slots = host_slot_ids.to(torch.int64)
    host_pool, dev_k, dev_v = _u8(host_pool), [_u8(t) for t in dev_k], [_u8(t) for t in dev_v]
    for l in range(len(dev_k)):
        host_pool[:, l, 0].index_copy_(0, slots, dev_k[l].index_select(0, ids))
        host_pool[:, l, 1].index_copy_(0, slots, dev_v[l].index_select(0, ids))


def swap_in(dev_k: Sequence[torch.Tensor], dev_v: Sequence[torch.Tensor], host_pool: torch.Tensor,
            device_block_ids: torch.Tensor, host_slot_ids: torch.Tensor) -> None:
    """cache_kv[l][block] = host_pool[slot, l, kv] for every layer, in place."""
    ids = device_block_ids.to(torch.int64)
    slots = host_slot_ids.to(torch.int64)
    host_pool, dev_k, dev_v = _u8(host_pool), [_u8(t) for t in dev_k], [_u8(t) for t in dev_v]
    for l in range(len(dev_k)):
        dev_k[l].index_copy_(0, ids, host_pool[:, l, 0].index_select(0, slots))
        dev_v[l].index_copy_(0, ids, host_pool[:, l, 1].index_select(0, slots))


def relayout_swap_in(dev_layers: Sequence[torch.Tensor], host_pool: torch.Tensor,
                     device_block_ids: torch.Tensor, host_slot_ids: torch.Tensor) -> None:
    """Multi-block form of the reference's transfer: for every listed block,
    dev_layers[l][block] ([H,B,D]) = host_pool[slot] ([B,L,H,D]).permute(1,2,0,3)[l]
    (the permute asserted in pcieThrough/tests/test_transfer_kernel.py:81-83).  In place."""
    ids, slots = device_block_ids.to(torch.int64), host_slot_ids.to(torch.int64)
    pool = _u8(host_pool)
    for l, cache in enumerate(dev_layers):
        src = pool.index_select(0, slots)[:, :, l].permute(0, 2, 1, 3)   # [n, H, B, D bytes]
        _u8(cache).index_copy_(0, ids, src.contiguous())


def relayout_swap_out(dev_layers: Sequence[torch.Tensor], host_pool: torch.Tensor,
                      device_block_ids: torch.Tensor, host_slot_ids: torch.Tensor) -> None:
    """The inverse: host_pool[slot][:, l] = dev_layers[l][block].permute(1,0,2).  In place."""
    ids, slots = device_block_ids.to(torch.int64), host_slot_ids.to(torch.int64)
    pool = _u8(host_pool)
    for l, cache in enumerate(dev_layers):
        src = _u8(cache).index_select(0, ids).permute(0, 2, 1, 3)        # [n, B, H, D bytes]
        pool[:, :, l].index_copy_(0, slots, src.contiguous())


def paged_gather(dev_k: Sequence[torch.Tensor], dev_v: Sequence[torch.Tensor], block_tables: torch.Tensor,
                 seq_lens: torch.Tensor, block_size: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Contiguous per-sequence K and V: out[l] = cat_s( cache[l][table[s]].flatten(0,1)[:len_s] ).

    dev_k / dev_v: per-layer [num_blocks, block_size, ...token dims].  Returns
    ([layers, total_tokens, ...token dims]) x 2."""
    lens = [int(x) for x in seq_lens.tolist()]
    dtype = dev_k[0].dtype
    outs = ([], [])
    for l in range(len(dev_k)):
        for kv, cache in enumerate((_u8(dev_k[l]), _u8(dev_v[l]))):
            parts = []
            for s, n in enumerate(lens):
                nb = (n + block_size - 1) // block_size
                pages = cache.index_select(0, block_tables[s, :nb].to(torch.int64))
                parts.append(pages.flatten(0, 1)[:n])
            outs[kv].append(torch.cat(parts, 0) if parts else cache.new_zeros((0,) + tuple(cache.shape[2:])))
    return torch.stack(outs[0], 0).view(dtype), torch.stack(outs[1], 0).view(dtype)


def migrate_blocks(src_k: Sequence[torch.Tensor], src_v: Sequence[torch.Tensor], dst_k: Sequence[torch.Tensor],
                   dst_v: Sequence[torch.Tensor], src_ids: torch.Tensor, dst_ids: torch.Tensor) -> None:
    """dst_kv[l][dst_ids] = src_kv[l][src_ids] for every layer, in place: blocks moved between two
    caches (two GPUs' caches in the product; two sets of CPU tensors here)."""
    s, d = src_ids.to(torch.int64), dst_ids.to(torch.int64)
    for src, dst in zip(list(src_k) + list(src_v), list(dst_k) + list(dst_v)):
        _u8(dst).index_copy_(0, d, _u8(src).index_select(0, s))


# ----------------------------------------------------------------------------
# 3. seeded workload generators: shared with the benchmark, so they live in the package
# ----------------------------------------------------------------------------
from heterofusedkernels_b200.workloads import (CONFIGS, FP8, Geometry, block_tables_for, distinct_ids,  # noqa: E402,F401
                                               gather_seq_lens, random_kv_bytes)
