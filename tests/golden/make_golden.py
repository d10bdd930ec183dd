"""Generates the committed fixtures of tests/golden from the CPU oracle.

    python tests/golden/make_golden.py

The reference holds no golden vectors for this path (its tests build constant data at
run time), so the fixtures pin the oracle itself: small cases are stored whole
(inputs and the output of the *literal* loop-for-loop restatement of the reference
kernels), the tiny benchmark configuration is stored as id lists plus SHA-256 digests
of its seeded inputs and expected outputs.
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from oracle import kv_oracle as o  # noqa: E402


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def tiny_case():
    """The tiny configuration: fp16 caches [64,16,8,128] x 2 layers, 8-block swap, gather of 40+100 tokens."""
    g = o.CONFIGS["tiny"]
    shape = (g.num_blocks, g.block_size, g.kv_heads, g.head_dim)
    dev_k = [o.random_kv_bytes(shape, g.dtype, seed=0 + 2 * l) for l in range(g.layers)]
    dev_v = [o.random_kv_bytes(shape, g.dtype, seed=1 + 2 * l) for l in range(g.layers)]
    dev_ids = o.distinct_ids(g.n_swap, g.num_blocks, seed=100)
    slots = o.distinct_ids(g.n_swap, g.host_slots, seed=101)
    back_ids = o.distinct_ids(g.n_swap, g.num_blocks, seed=102)
    tables = o.block_tables_for(g.seq_lens, g.block_size, g.num_blocks, seed=103)
    return g, dev_k, dev_v, dev_ids, slots, back_ids, tables


def main() -> None:
    # 1. block transfer, stored whole; expected = literal restatement of the AscendC loops
    host = o.random_kv_bytes((16, 3, 2, 32), torch.int8, seed=7)
    lit = o.block_transfer_literal(host.numpy(), aiv=4)
    np.savez_compressed(HERE / "block_transfer_int8.npz", host_block=host.numpy(), expected=np.stack(lit, 0))

    # 2. row gather, stored whole (fp16 as raw uint16); expected = literal restatement
    table = o.random_kv_bytes((50, 64), torch.float16, seed=8)
    ids = torch.randint(0, 50, (37,), generator=torch.Generator().manual_seed(9))
    exp = o.row_gather_literal(table.view(torch.int16).numpy(), ids.numpy(), aiv=4)
    np.savez_compressed(HERE / "row_gather_fp16.npz", table=table.view(torch.int16).numpy(), ids=ids.numpy(),
                        expected=exp)

    # 3. tiny configuration: ids + digests
    g, dev_k, dev_v, dev_ids, slots, back_ids, tables = tiny_case()
    pool = torch.zeros((g.host_slots, g.layers, 2, g.block_size, g.kv_heads, g.head_dim), dtype=g.dtype)
    digests = {"inputs": {"dev_k": [sha(t) for t in dev_k], "dev_v": [sha(t) for t in dev_v]}}
    o.swap_out(dev_k, dev_v, pool, dev_ids, slots)
    digests["host_pool_after_swap_out"] = sha(pool)
    k2 = [torch.zeros_like(t) for t in dev_k]
    v2 = [torch.zeros_like(t) for t in dev_v]
    o.swap_in(k2, v2, pool, back_ids, slots)
    digests["dev_k_after_swap_in_to_zeroed_cache"] = [sha(t) for t in k2]
    digests["dev_v_after_swap_in_to_zeroed_cache"] = [sha(t) for t in v2]
    ko, vo = o.paged_gather(dev_k, dev_v, tables, torch.tensor(g.seq_lens), g.block_size)
    digests["gather_k_out"] = sha(ko)
    digests["gather_v_out"] = sha(vo)
    digests["ids"] = {"device_block_ids": dev_ids.tolist(), "host_slot_ids": slots.tolist(),
                      "swap_in_device_block_ids": back_ids.tolist(), "block_tables": tables.tolist(),
                      "seq_lens": g.seq_lens}
    (HERE / "tiny_digests.json").write_text(json.dumps(digests, indent=1) + "\n")
    print("wrote", sorted(p.name for p in HERE.iterdir()))


if __name__ == "__main__":
    main()
