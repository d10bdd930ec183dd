"""The CPU oracle against the reference tests' assertions and the committed fixtures (no GPU)."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import kv_oracle as o

GOLDEN = Path(__file__).resolve().parent / "golden"


def sha(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


@pytest.mark.parametrize("B,L,H,D,dtype,aiv", [
    (16, 3, 2, 32, torch.int8, 4), (64, 1, 1, 128, torch.int8, 2), (32, 4, 2, 64, torch.float16, 4),
    (24, 2, 8, 16, torch.bfloat16, 5), (7, 2, 1, 8, torch.float32, 3)])
def test_block_transfer_literal_matches_reference_test_assertion(B, L, H, D, dtype, aiv):
    host = o.random_kv_bytes((B, L, H, D), dtype, seed=B + L)
    view = host.view(torch.int16) if dtype in (torch.float16, torch.bfloat16) else host
    lit = o.block_transfer_literal(view.numpy(), aiv=aiv)
    vec = o.block_transfer(view)
    for l in range(L):
        assert np.array_equal(lit[l], vec[l].numpy())
    # the reference's own assertion: host_block == dev_block.permute(2, 0, 1, 3)
    # (pcieThrough/tests/test_transfer_kernel.py:77-83; device layout [L, H, B, D])
    dev = torch.from_numpy(np.stack(lit, 0))
    assert torch.equal(view, dev.permute(2, 0, 1, 3))


def test_transfer_tiling_follows_reference_limits():
    t = o.transfer_tiling(aiv=4, elt=1, B=1024, L=32, H=1, D=128)
    assert t.tokens_per_core == 256
    assert t.tokens_per_inner_loop == (192 * 1024 - 256) // (2 * 32 * 128)
    with pytest.raises(ValueError):
        o.transfer_tiling(aiv=4, elt=2, B=16, L=64, H=8, D=128)  # per-token image exceeds the buffer
    with pytest.raises(ValueError):
        o.transfer_tiling(aiv=4, elt=1, B=16, L=2, H=1, D=24)    # not a multiple of 32 bytes


@pytest.mark.parametrize("rows,cols,n,aiv,idt", [(50, 64, 37, 4, np.int64), (9, 512, 3, 8, np.int64),
                                                (100, 16, 1000, 4, np.int32), (5, 8, 0, 2, np.int64)])
def test_row_gather_literal_matches_index_select(rows, cols, n, aiv, idt):
    table = o.random_kv_bytes((rows, cols), torch.float16, seed=rows).view(torch.int16)
    ids = torch.randint(0, rows, (n,), generator=torch.Generator().manual_seed(n))
    lit = o.row_gather_literal(table.numpy(), ids.numpy().astype(idt), aiv)
    assert np.array_equal(lit, o.row_gather(table, ids).numpy())
    # the reference's check (pcieThrough/tests/test_gather.py:14-29): row i of dst == table[ids[i]]
    for i in range(n):
        assert np.array_equal(lit[i], table[int(ids[i])].numpy())


def test_golden_block_transfer():
    z = np.load(GOLDEN / "block_transfer_int8.npz")
    vec = o.block_transfer(torch.from_numpy(z["host_block"]))
    assert np.array_equal(np.stack([v.numpy() for v in vec], 0), z["expected"])


def test_golden_row_gather():
    z = np.load(GOLDEN / "row_gather_fp16.npz")
    out = o.row_gather(torch.from_numpy(z["table"]), torch.from_numpy(z["ids"]))
    assert np.array_equal(out.numpy(), z["expected"])


def test_golden_tiny_configuration_digests():
    from tests.golden.make_golden import tiny_case

    d = json.loads((GOLDEN / "tiny_digests.json").read_text())
    g, dev_k, dev_v, dev_ids, slots, back_ids, tables = tiny_case()
    assert [sha(t) for t in dev_k] == d["inputs"]["dev_k"], "seeded inputs drifted"
    assert dev_ids.tolist() == d["ids"]["device_block_ids"] and tables.tolist() == d["ids"]["block_tables"]
    pool = torch.zeros((g.host_slots, g.layers, 2, g.block_size, g.kv_heads, g.head_dim), dtype=g.dtype)
    o.swap_out(dev_k, dev_v, pool, dev_ids, slots)
    assert sha(pool) == d["host_pool_after_swap_out"]
    ko, vo = o.paged_gather(dev_k, dev_v, tables, torch.tensor(g.seq_lens), g.block_size)
    assert sha(ko) == d["gather_k_out"] and sha(vo) == d["gather_v_out"]


def test_swap_round_trip_and_untouched_slots():
    g = o.CONFIGS["tiny"]
    shape = (g.num_blocks, g.block_size, g.kv_heads, g.head_dim)
    k = [o.random_kv_bytes(shape, g.dtype, l) for l in range(2)]
    v = [o.random_kv_bytes(shape, g.dtype, 10 + l) for l in range(2)]
    pool = torch.full((32, 2, 2) + shape[1:], 3.0, dtype=g.dtype)
    ids, slots = o.distinct_ids(8, 64, 1), o.distinct_ids(8, 32, 2)
    o.swap_out(k, v, pool, ids, slots)
    untouched = [s for s in range(32) if s not in slots.tolist()]
    assert bool((pool[untouched] == 3.0).all())
    for i in range(8):
        assert torch.equal(pool[slots[i], 1, 0], k[1][ids[i]]) and torch.equal(pool[slots[i], 0, 1], v[0][ids[i]])
    k2, v2 = [t.clone() for t in k], [t.clone() for t in v]
    for t in k2 + v2:
        t[ids] = 0
    o.swap_in(k2, v2, pool, ids, slots)
    assert all(torch.equal(a, b) for a, b in zip(k + v, k2 + v2))


def test_paged_gather_partial_last_block_and_layout():
    B = 4
    cache = [torch.arange(10 * B * 2, dtype=torch.int16).view(10, B, 2)]
    tables = torch.tensor([[7, 2, -1], [5, 9, 1]])
    lens = torch.tensor([5, 12])
    ko, _ = o.paged_gather(cache, cache, tables, lens, B)
    assert ko.shape == (1, 17, 2)
    assert torch.equal(ko[0, :4], cache[0][7]) and torch.equal(ko[0, 4], cache[0][2][0])
    assert torch.equal(ko[0, 5:9], cache[0][5]) and torch.equal(ko[0, 13:17], cache[0][1])


def test_fp8_bytes_exclude_nan_codes():
    raw = o.random_kv_bytes((64, 1024), o.FP8, seed=5).view(torch.uint8)
    assert not bool(((raw == 0x7F) | (raw == 0xFF)).any())
    assert len(torch.unique(raw)) == 254


def test_algorithmic_bytes_of_the_benchmark_configurations():
    assert o.CONFIGS["tiny"].swap_bytes() == 1_048_576
    assert o.CONFIGS["llama3_8b_swap"].swap_bytes() == 1_073_741_824
    assert o.CONFIGS["llama3_70b_tp8_swap"].swap_bytes() == 10_737_418_240
    g = o.CONFIGS["qwen2_7b_fp8_prefetch"]
    assert g.n_swap * 2 * g.block_bytes == 4_194_304  # one layer, one direction


def test_relayout_swap_is_the_block_transfer_per_block_and_round_trips():
    B, L, H, D = 8, 3, 2, 32
    pool = o.random_kv_bytes((6, B, L, H, D), torch.int8, seed=1)
    dev = [torch.zeros((10, H, B, D), dtype=torch.int8) for _ in range(L)]
    ids, slots = torch.tensor([7, 2, 9]), torch.tensor([5, 0, 3])
    o.relayout_swap_in(dev, pool, ids, slots)
    for i in range(3):
        lit = o.block_transfer_literal(pool[slots[i]].numpy(), aiv=2)      # the reference kernel, block by block
        for l in range(L):
            assert np.array_equal(dev[l][ids[i]].numpy(), lit[l])
    assert all(int(d[[0, 1, 3, 4, 5, 6, 8]].abs().sum()) == 0 for d in dev)  # other blocks untouched
    pool2 = torch.zeros_like(pool)
    o.relayout_swap_out(dev, pool2, ids, slots)
    assert torch.equal(pool2[slots], pool[slots]) and int(pool2[[1, 2, 4]].abs().sum()) == 0
