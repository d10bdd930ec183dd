"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle — bit exact.

Every comparison is on raw bytes (the path moves bytes; random bit patterns may be NaNs).
"""
import ctypes as C
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import kv_oracle as o
from tests.helpers import (PinnedPool, dev_zeros, gather_desc, ptr_table, relayout_desc, stream_handle, swap_desc,
                           u8)

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
MOVERS = [pytest.param(1, id="vector"), pytest.param(2, id="bulk")]  # HFK_MOVER_VECTOR, HFK_MOVER_BULK


def sha(t):
    return hashlib.sha256(t.contiguous().cpu().view(torch.uint8).numpy().tobytes()).hexdigest()


def same_bytes(a, b):
    return torch.equal(u8(a.cpu()), u8(b.cpu()))


class SwapCase:
    """Random caches on CPU (oracle side) and GPU (device side) plus a pinned host pool."""

    def __init__(self, hfk, dev, layers, num_blocks, chunk_shape, dtype, host_slots, seed=0,
                 pool_layout="block_major", block_pad=0):
        self.hfk, self.dev, self.layers, self.num_blocks = hfk, dev, layers, num_blocks
        shape = (num_blocks,) + tuple(chunk_shape)
        self.cpu_k = [o.random_kv_bytes(shape, dtype, seed + 2 * l) for l in range(layers)]
        self.cpu_v = [o.random_kv_bytes(shape, dtype, seed + 2 * l + 1) for l in range(layers)]
        if block_pad:  # device blocks padded: stride > block bytes
            padded = (num_blocks, chunk_shape[0] + block_pad) + tuple(chunk_shape[1:])
            self.store_k = [dev_zeros(padded, dtype, dev) for _ in range(layers)]
            self.store_v = [dev_zeros(padded, dtype, dev) for _ in range(layers)]
            self.gpu_k = [s[:, :chunk_shape[0]] for s in self.store_k]
            self.gpu_v = [s[:, :chunk_shape[0]] for s in self.store_v]
            for g, c in zip(self.gpu_k + self.gpu_v, self.cpu_k + self.cpu_v):
                g.copy_(c)
            self.k_ptrs, self.v_ptrs = ptr_table(self.store_k, dev), ptr_table(self.store_v, dev)
            self.dev_stride = self.store_k[0].stride(0) * self.store_k[0].element_size()
        else:
            self.gpu_k = [t.to(dev) for t in self.cpu_k]
            self.gpu_v = [t.to(dev) for t in self.cpu_v]
            self.k_ptrs, self.v_ptrs = ptr_table(self.gpu_k, dev), ptr_table(self.gpu_v, dev)
            self.dev_stride = None
        if pool_layout == "block_major":
            self.pool = PinnedPool((host_slots, layers, 2) + tuple(chunk_shape), dtype)
            self.pool_view = self.pool.tensor
        else:  # layer-major storage [2, layers, slots, chunk] seen as [slots, layers, 2, chunk]
            self.pool = PinnedPool((2, layers, host_slots) + tuple(chunk_shape), dtype)
            self.pool_view = self.pool.tensor.permute(2, 1, 0, *range(3, 3 + len(chunk_shape)))
        self.pool.tensor.view(torch.uint8).fill_(0xA5)
        self.cpu_pool = self.pool_view.clone()

    def desc(self, dev_ids, slots):
        return swap_desc(self.k_ptrs, self.v_ptrs, self.pool_view, self.pool.alias, dev_ids, slots,
                         self.num_blocks, self.dev_stride)

    def close(self):
        self.pool.close()


def run_swap(hfk, fn, desc, mover, ctas=0):
    hfk.check(fn(C.byref(desc), mover, ctas, stream_handle()), "swap")
    torch.cuda.synchronize()


# ------------------------------------------------------------------ swaps ---
@pytest.mark.parametrize("mover", MOVERS)
def test_tiny_configuration_swap_out_then_in_matches_oracle_and_golden(hfk, cuda_device, mover):
    from tests.golden.make_golden import tiny_case

    g, cpu_k, cpu_v, dev_ids, slots, back_ids, _ = tiny_case()
    gold = json.loads((GOLDEN / "tiny_digests.json").read_text())
    case = SwapCase(hfk, cuda_device, g.layers, g.num_blocks, (g.block_size, g.kv_heads, g.head_dim), g.dtype,
                    g.host_slots)
    try:
        for gk, ck in zip(case.gpu_k + case.gpu_v, cpu_k + cpu_v):
            gk.copy_(ck)
        case.pool.tensor.zero_()
        ids_d, slots_d = dev_ids.to(cuda_device), slots.to(cuda_device)
        run_swap(hfk, hfk.lib().hfk_swap_out, case.desc(ids_d, slots_d), mover)
        assert sha(case.pool.tensor) == gold["host_pool_after_swap_out"]
        ref_pool = torch.zeros_like(case.pool.tensor)
        o.swap_out(cpu_k, cpu_v, ref_pool, dev_ids, slots)
        assert same_bytes(case.pool.tensor, ref_pool)
        # swap-in to other device ids of a zeroed cache
        for t in case.gpu_k + case.gpu_v:
            t.zero_()
        back_d = back_ids.to(cuda_device)
        run_swap(hfk, hfk.lib().hfk_swap_in, case.desc(back_d, slots_d), mover)
        assert [sha(t) for t in case.gpu_k] == gold["dev_k_after_swap_in_to_zeroed_cache"]
        assert [sha(t) for t in case.gpu_v] == gold["dev_v_after_swap_in_to_zeroed_cache"]
        assert hfk.device_status() == 0
    finally:
        case.close()


SWAP_SHAPES = [
    # layers, blocks, chunk_shape, dtype, slots, n, layout, pad, id dtype
    (1, 8, (1, 1, 8), torch.float16, 8, 8, "block_major", 0, torch.int64),           # 16-byte chunks
    (3, 40, (3, 1, 8), torch.float16, 50, 17, "layer_major", 0, torch.int32),        # 48-byte chunks
    (2, 64, (16, 4, 128), o.FP8, 96, 33, "block_major", 0, torch.int64),             # 8 KiB fp8 chunks
    (2, 48, (20, 8, 128), torch.bfloat16, 64, 48, "layer_major", 0, torch.int64),    # 40 KiB: > one ring stage
    (2, 32, (128, 1, 128), torch.bfloat16, 40, 1, "block_major", 0, torch.int64),    # one block, 32 KiB
    (1, 3000, (2, 1, 64), torch.int8, 3000, 2500, "block_major", 0, torch.int64),    # more ids than one smem tile
    (2, 30, (16, 2, 64), torch.float16, 30, 30, "block_major", 3, torch.int64),      # padded device blocks
    (80, 16, (8, 1, 128), torch.bfloat16, 16, 9, "block_major", 0, torch.int32),     # many layers
]


@pytest.mark.parametrize("mover", MOVERS)
@pytest.mark.parametrize("shape", SWAP_SHAPES, ids=[str(i) for i in range(len(SWAP_SHAPES))])
def test_swap_out_and_in_shapes_layouts_and_id_types(hfk, cuda_device, mover, shape):
    _swap_round_trip(hfk, cuda_device, mover, shape)


@pytest.mark.parametrize("ring", [(16384, 8), (32768, 3), (128, 2)], ids=["16Kx8", "32Kx3", "128x2"])
@pytest.mark.parametrize("shape", SWAP_SHAPES, ids=[str(i) for i in range(len(SWAP_SHAPES))])
def test_swap_with_the_ring_of_large_launches_forced(hfk, cuda_device, ring, shape):
    """Launches below 256 MiB take the small ring by default; the ring that 1 GB launches use (and two
    extreme ones) is forced here so that it sees the small shapes too."""
    hfk.check(hfk.lib().hfk_set_bulk_geometry(*ring), "hfk_set_bulk_geometry")
    try:
        _swap_round_trip(hfk, cuda_device, 2, shape)
    finally:
        hfk.lib().hfk_set_bulk_geometry(0, 0)


@pytest.mark.parametrize("pace_mbs", [500, 20000, 1000000])
def test_paced_swap_out_moves_the_same_bytes(hfk, cuda_device, pace_mbs):
    """hfk_swap_out_paced spaces the stores in time; the bytes are those of hfk_swap_out."""
    case = SwapCase(hfk, cuda_device, 3, 40, (16, 2, 64), torch.bfloat16, 48, seed=17)
    try:
        ids, slots = o.distinct_ids(25, 40, 1), o.distinct_ids(25, 48, 2)
        d = case.desc(ids.to(cuda_device), slots.to(cuda_device))
        lib = hfk.lib()
        for mover in (0, 2):
            case.pool.tensor.view(torch.uint8).fill_(0xA5)
            hfk.check(lib.hfk_swap_out_paced(C.byref(d), mover, 3, pace_mbs, stream_handle()), "paced swap-out")
            torch.cuda.synchronize()
            expect = case.cpu_pool.clone()
            o.swap_out(case.cpu_k, case.cpu_v, expect, ids, slots)
            assert same_bytes(case.pool_view, expect)
        assert lib.hfk_swap_out_paced(C.byref(d), 1, 0, pace_mbs, stream_handle()) == hfk.HFK_ERR_UNSUPPORTED
        assert lib.hfk_swap_out_paced(C.byref(d), 0, 0, -5, stream_handle()) == hfk.HFK_ERR_INVALID_ARG
        assert hfk.device_status() == 0
    finally:
        case.close()


def _swap_round_trip(hfk, cuda_device, mover, shape):
    layers, blocks, chunk, dtype, nslots, n, layout, pad, idt = shape
    case = SwapCase(hfk, cuda_device, layers, blocks, chunk, dtype, nslots, seed=11, pool_layout=layout,
                    block_pad=pad)
    try:
        ids, slots = o.distinct_ids(n, blocks, 1).to(idt), o.distinct_ids(n, nslots, 2).to(idt)
        run_swap(hfk, hfk.lib().hfk_swap_out, case.desc(ids.to(cuda_device), slots.to(cuda_device)), mover, ctas=5)
        o.swap_out(case.cpu_k, case.cpu_v, case.cpu_pool, ids, slots)
        assert same_bytes(case.pool_view, case.cpu_pool)      # copied slots right, every other byte untouched
        # swap back into different blocks
        ids2 = o.distinct_ids(n, blocks, 3).to(idt)
        run_swap(hfk, hfk.lib().hfk_swap_in, case.desc(ids2.to(cuda_device), slots.to(cuda_device)), mover, ctas=7)
        o.swap_in(case.cpu_k, case.cpu_v, case.cpu_pool, ids2, slots)
        for g, c in zip(case.gpu_k + case.gpu_v, case.cpu_k + case.cpu_v):
            assert same_bytes(g, c)
        assert hfk.device_status() == 0
    finally:
        case.close()


def test_swap_empty_id_list_is_a_no_op(hfk, cuda_device):
    case = SwapCase(hfk, cuda_device, 1, 4, (1, 1, 8), torch.float16, 4)
    try:
        empty = torch.zeros(0, dtype=torch.int64, device=cuda_device)
        d = case.desc(empty, empty)
        assert hfk.lib().hfk_swap_out(C.byref(d), 0, 0, stream_handle()) == 0
        torch.cuda.synchronize()
        assert bool((case.pool.tensor.view(torch.uint8) == 0xA5).all())
    finally:
        case.close()


@pytest.mark.parametrize("mover", MOVERS)
def test_out_of_range_ids_are_skipped_and_reported_not_dereferenced(hfk, cuda_device, mover):
    case = SwapCase(hfk, cuda_device, 2, 16, (4, 1, 64), torch.float16, 16, seed=5)
    try:
        ids = torch.tensor([3, 99, 5, -1, 7], dtype=torch.int64)
        slots = torch.tensor([0, 1, 400, 2, 3], dtype=torch.int64)
        run_swap(hfk, hfk.lib().hfk_swap_out, case.desc(ids.to(cuda_device), slots.to(cuda_device)), mover)
        bits = hfk.device_status()
        assert bits == (hfk.HFK_DEV_BAD_DEVICE_BLOCK_ID | hfk.HFK_DEV_BAD_HOST_SLOT_ID)
        good = torch.tensor([0, 4])
        o.swap_out(case.cpu_k, case.cpu_v, case.cpu_pool, ids[good], slots[good])
        assert same_bytes(case.pool_view, case.cpu_pool)
        assert hfk.device_status() == 0  # reading clears
    finally:
        case.close()


def test_copy_engine_variant_matches_oracle(hfk, cuda_device):
    case = SwapCase(hfk, cuda_device, 3, 20, (16, 2, 64), torch.bfloat16, 24, seed=9)
    try:
        ids, slots = o.distinct_ids(10, 20, 1), o.distinct_ids(10, 24, 2)
        kp = torch.tensor([t.data_ptr() for t in case.gpu_k], dtype=torch.int64)
        vp = torch.tensor([t.data_ptr() for t in case.gpu_v], dtype=torch.int64)
        d = swap_desc(kp, vp, case.pool_view, case.pool.ptr, ids, slots, 20)  # host arrays, host address
        hfk.check(hfk.lib().hfk_swap_copy_engine(C.byref(d), 1, stream_handle()), "copy engine out")
        torch.cuda.synchronize()
        o.swap_out(case.cpu_k, case.cpu_v, case.cpu_pool, ids, slots)
        assert same_bytes(case.pool_view, case.cpu_pool)
        ids2 = o.distinct_ids(10, 20, 3)
        d = swap_desc(kp, vp, case.pool_view, case.pool.ptr, ids2, slots, 20)
        hfk.check(hfk.lib().hfk_swap_copy_engine(C.byref(d), 0, stream_handle()), "copy engine in")
        torch.cuda.synchronize()
        o.swap_in(case.cpu_k, case.cpu_v, case.cpu_pool, ids2, slots)
        for g, c in zip(case.gpu_k + case.gpu_v, case.cpu_k + case.cpu_v):
            assert same_bytes(g, c)
    finally:
        case.close()


# ----------------------------------------------------------- paged gather ---
def run_gather(hfk, dev, cpu_k, cpu_v, tables, lens, block_size, mover, idt=torch.int64, ctas=0, total=None):
    layers = len(cpu_k)
    gk, gv = [t.to(dev) for t in cpu_k], [t.to(dev) for t in cpu_v]
    total = int(lens.sum()) if total is None else total
    tok_shape = tuple(cpu_k[0].shape[2:])
    k_out = dev_zeros((layers, total) + tok_shape, cpu_k[0].dtype, dev)
    v_out = torch.zeros_like(k_out)
    kp, vp = ptr_table(gk, dev), ptr_table(gv, dev)
    d = gather_desc(kp, vp, k_out, v_out, tables.to(idt).to(dev), lens.to(idt).to(dev), block_size,
                    cpu_k[0].shape[0])
    hfk.check(hfk.lib().hfk_paged_gather(C.byref(d), mover, ctas, stream_handle()), "paged_gather")
    torch.cuda.synchronize()
    return k_out, v_out


@pytest.mark.parametrize("mover", MOVERS)
def test_tiny_configuration_paged_gather_matches_oracle_and_golden(hfk, cuda_device, mover):
    from tests.golden.make_golden import tiny_case

    g, cpu_k, cpu_v, _, _, _, tables = tiny_case()
    gold = json.loads((GOLDEN / "tiny_digests.json").read_text())
    lens = torch.tensor(g.seq_lens)
    k_out, v_out = run_gather(hfk, cuda_device, cpu_k, cpu_v, tables, lens, g.block_size, mover)
    assert sha(k_out) == gold["gather_k_out"] and sha(v_out) == gold["gather_v_out"]
    ko, vo = o.paged_gather(cpu_k, cpu_v, tables, lens, g.block_size)
    assert same_bytes(k_out, ko) and same_bytes(v_out, vo)
    assert hfk.device_status() == 0


GATHER_CASES = [
    # layers, blocks, block_size, tok_shape, dtype, lens, id dtype
    (2, 64, 16, (8, 128), torch.bfloat16, [40, 100, 0, 16, 1, 33], torch.int64),
    (1, 32, 4, (1, 8), torch.float16, [4, 8, 3, 0, 0, 17], torch.int32),          # 16-byte tokens
    (3, 50, 128, (1, 128), torch.bfloat16, [128, 129, 700, 5], torch.int64),      # 32 KiB pages, 70B shard layout
    (2, 40, 16, (4, 128), o.FP8, [250, 1, 64], torch.int64),                       # fp8
    (1, 30, 20, (8, 128), torch.float16, [41, 400], torch.int64),                  # 40 KiB pages: > one ring stage
    (1, 600, 1, (2, 8), torch.int8, list(range(0, 33)), torch.int64),              # block_size 1, 33 sequences
    (2, 6000, 2, (1, 8), torch.float16, [(7 * i) % 5 for i in range(2500)], torch.int32),  # more sequences than one launch's walk table
]


@pytest.mark.parametrize("mover", MOVERS)
@pytest.mark.parametrize("case", GATHER_CASES, ids=[str(i) for i in range(len(GATHER_CASES))])
def test_paged_gather_ragged_batches(hfk, cuda_device, mover, case):
    layers, blocks, bs, tok, dtype, lens, idt = case
    shape = (blocks, bs) + tok
    cpu_k = [o.random_kv_bytes(shape, dtype, 40 + l) for l in range(layers)]
    cpu_v = [o.random_kv_bytes(shape, dtype, 60 + l) for l in range(layers)]
    tables = o.block_tables_for(lens, bs, blocks, seed=7)
    lens_t = torch.tensor(lens)
    k_out, v_out = run_gather(hfk, cuda_device, cpu_k, cpu_v, tables, lens_t, bs, mover, idt, ctas=6)
    ko, vo = o.paged_gather(cpu_k, cpu_v, tables, lens_t, bs)
    assert same_bytes(k_out, ko) and same_bytes(v_out, vo)
    assert hfk.device_status() == 0


@pytest.mark.parametrize("mover", MOVERS)
def test_paged_gather_reports_bad_table_entries_and_lengths(hfk, cuda_device, mover):
    bs, blocks = 4, 16
    cpu_k = [o.random_kv_bytes((blocks, bs, 2, 8), torch.float16, 1)]
    cpu_v = [o.random_kv_bytes((blocks, bs, 2, 8), torch.float16, 2)]
    tables = torch.tensor([[1, 99, 3], [4, 5, 6]])
    lens = torch.tensor([12, 8])
    k_out, _ = run_gather(hfk, cuda_device, cpu_k, cpu_v, tables, lens, bs, mover)
    assert hfk.device_status() == hfk.HFK_DEV_BAD_DEVICE_BLOCK_ID
    ko, _ = o.paged_gather(cpu_k, cpu_v, torch.tensor([[1, 0, 3], [4, 5, 6]]), lens, bs)
    ko[0, 4:8] = 0  # the page with the bad id stays untouched (zeros)
    assert same_bytes(k_out, ko)
    # a sequence longer than its table row is clamped and reported; an output that is too small is not overrun
    lens = torch.tensor([100, 8])
    run_gather(hfk, cuda_device, cpu_k, cpu_v, torch.tensor([[1, 2, 3], [4, 5, 6]]), lens, bs, mover, total=20)
    assert hfk.device_status() & hfk.HFK_DEV_BAD_SEQ_LEN
    k_small, _ = run_gather(hfk, cuda_device, cpu_k, cpu_v, torch.tensor([[1, 2, 3], [4, 5, 6]]),
                            torch.tensor([12, 8]), bs, mover, total=16)
    assert hfk.device_status() & hfk.HFK_DEV_BAD_SEQ_LEN
    full, _ = o.paged_gather(cpu_k, cpu_v, torch.tensor([[1, 2, 3], [4, 5, 6]]), torch.tensor([12, 8]), bs)
    assert same_bytes(k_small[:, :16], full[:, :16])


# ------------------------------------------------------- Group R: gather ---
@pytest.mark.parametrize("cols,dtype", [(8, torch.float16), (32, torch.float16), (512, torch.float16),
                                        (512, torch.bfloat16), (1024, torch.float16), (16384, torch.bfloat16),
                                        (50, torch.float16), (7, torch.int8), (6, torch.float16), (520, torch.int8)])
@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
def test_row_gather_device_table(hfk, cuda_device, cols, dtype, idt):
    rows, n = 300, 257
    table = o.random_kv_bytes((rows, cols), dtype, seed=cols)
    ids = torch.randint(0, rows, (n,), generator=torch.Generator().manual_seed(1)).to(idt)
    t_d, ids_d = table.to(cuda_device), ids.to(cuda_device)
    dst = dev_zeros((n, cols), dtype, cuda_device)
    rb = cols * table.element_size()
    hfk.check(hfk.lib().hfk_gather(t_d.data_ptr(), dst.data_ptr(), ids_d.data_ptr(), int(idt == torch.int64), n,
                                   rb, rows, 4, stream_handle()), "gather")
    torch.cuda.synchronize()
    assert same_bytes(dst, o.row_gather(u8(table).view(rows, rb), ids))
    assert hfk.device_status() == 0


def test_row_gather_host_registered_table_and_golden(hfk, cuda_device):
    z = np.load(GOLDEN / "row_gather_fp16.npz")
    table, ids = torch.from_numpy(z["table"]), torch.from_numpy(z["ids"])
    pool = PinnedPool(tuple(table.shape), torch.int16)
    try:
        pool.tensor.copy_(table)
        dst = torch.zeros((ids.numel(), table.shape[1]), dtype=torch.int16, device=cuda_device)
        ids_d = ids.to(cuda_device)
        hfk.check(hfk.lib().hfk_gather(pool.alias, dst.data_ptr(), ids_d.data_ptr(), 1, ids.numel(),
                                       table.shape[1] * 2, table.shape[0], 0, stream_handle()), "gather")
        torch.cuda.synchronize()
        assert np.array_equal(dst.cpu().numpy(), z["expected"])
    finally:
        pool.close()


def test_row_gather_bad_ids_are_reported(hfk, cuda_device):
    table = torch.arange(64, dtype=torch.int32, device=cuda_device).view(8, 8)
    ids = torch.tensor([1, 8, -2, 7], device=cuda_device)
    dst = torch.full((4, 8), -1, dtype=torch.int32, device=cuda_device)
    hfk.check(hfk.lib().hfk_gather(table.data_ptr(), dst.data_ptr(), ids.data_ptr(), 1, 4, 32, 8, 0, stream_handle()),
              "gather")
    assert hfk.device_status() == hfk.HFK_DEV_BAD_ROW_ID
    assert torch.equal(dst[0], table[1]) and torch.equal(dst[3], table[7]) and bool((dst[1:3] == -1).all())


# ------------------------------------- Group R: multi_layer_block_transfer ---
def transfer_case(dev, B, L, H, D, dtype, seed=0):
    host = o.random_kv_bytes((B, L, H, D), dtype, seed)
    dev_layers = [dev_zeros((H, B, D), dtype, dev) for _ in range(L)]
    return host, dev_layers, ptr_table(dev_layers, dev)


@pytest.mark.parametrize("B,L,H,D,dtype", [
    (1024, 1, 1, 128, torch.int8), (1024, 32, 1, 128, torch.int8), (1024, 64, 1, 128, torch.int8),  # the reference's own grid
    (256, 4, 8, 128, torch.bfloat16), (33, 3, 2, 16, torch.int8), (16, 2, 2, 8, torch.float16), (5, 7, 3, 4, torch.float32)])
@pytest.mark.parametrize("fused", [False, True])
def test_multi_layer_block_transfer_matches_reference_assertion(hfk, cuda_device, B, L, H, D, dtype, fused):
    host, dev_layers, ptrs = transfer_case(cuda_device, B, L, H, D, dtype, seed=B + L)
    pool = PinnedPool((B, L, H, D), dtype)
    try:
        pool.tensor.copy_(host)
        elt = host.element_size()
        if fused:
            staging = torch.empty(B * L * H * D * elt, dtype=torch.uint8, device=cuda_device)
            rc = hfk.lib().hfk_fused_memcpy_multi_layer_block_transfer(
                ptrs.data_ptr(), pool.ptr, staging.data_ptr(), B, L, H, D, elt, 4, stream_handle())
        else:
            rc = hfk.lib().hfk_multi_layer_block_transfer(ptrs.data_ptr(), pool.alias, B, L, H, D, elt, 4,
                                                          stream_handle())
        hfk.check(rc, "transfer")
        torch.cuda.synchronize()
        expect = o.block_transfer(host)
        for l in range(L):
            assert same_bytes(dev_layers[l], expect[l])
        # the reference's assertion (pcieThrough/tests/test_transfer_kernel.py:81-83)
        dev_block = torch.stack([u8(t.cpu()).view(H, B, D * elt) for t in dev_layers], 0)
        assert torch.equal(u8(host).view(B, L, H, D * elt), dev_block.permute(2, 0, 1, 3))
    finally:
        pool.close()


def test_multi_layer_block_transfer_golden(hfk, cuda_device):
    z = np.load(GOLDEN / "block_transfer_int8.npz")
    host = torch.from_numpy(z["host_block"])
    B, L, H, D = host.shape
    _, dev_layers, ptrs = transfer_case(cuda_device, B, L, H, D, torch.int8)
    src = host.to(cuda_device)  # a device-resident source is allowed as well
    hfk.check(hfk.lib().hfk_multi_layer_block_transfer(ptrs.data_ptr(), src.data_ptr(), B, L, H, D, 1, 0,
                                                       stream_handle()), "transfer")
    torch.cuda.synchronize()
    assert np.array_equal(torch.stack(dev_layers, 0).cpu().numpy(), z["expected"])


# ------------------------------------- multi-block swap in the reference's host format ---
@pytest.mark.parametrize("B,L,H,D,dtype,blocks,slots,n,idt", [
    (1024, 4, 1, 128, torch.int8, 6, 8, 5, torch.int64),       # the reference's block shape, several blocks
    (16, 32, 8, 128, torch.bfloat16, 40, 48, 33, torch.int64),  # Llama-3-8B geometry
    (16, 3, 2, 8, torch.float16, 20, 20, 20, torch.int32),      # 16-byte head rows
    (4, 2, 1, 4, torch.float32, 2000, 1500, 1200, torch.int64),  # more ids than one shared-memory tile
])
def test_relayout_swap_in_and_out_match_oracle(hfk, cuda_device, B, L, H, D, dtype, blocks, slots, n, idt):
    pool = PinnedPool((slots, B, L, H, D), dtype)
    try:
        pool.tensor.copy_(o.random_kv_bytes((slots, B, L, H, D), dtype, seed=3))
        cpu_pool = pool.tensor.clone()
        cpu_dev = [o.random_kv_bytes((blocks, H, B, D), dtype, seed=10 + l) for l in range(L)]
        gpu_dev = [t.to(cuda_device) for t in cpu_dev]
        ptrs = ptr_table(gpu_dev, cuda_device)
        ids, sl = o.distinct_ids(n, blocks, 1).to(idt), o.distinct_ids(n, slots, 2).to(idt)
        d = relayout_desc(ptrs, pool.tensor, pool.alias, ids.to(cuda_device), sl.to(cuda_device), blocks)
        hfk.check(hfk.lib().hfk_swap_relayout(C.byref(d), 0, 6, stream_handle()), "relayout in")
        torch.cuda.synchronize()
        o.relayout_swap_in(cpu_dev, cpu_pool, ids, sl)
        for g, c in zip(gpu_dev, cpu_dev):
            assert same_bytes(g, c)
        # and out again into other slots
        ids2, sl2 = o.distinct_ids(n, blocks, 4).to(idt), o.distinct_ids(n, slots, 5).to(idt)
        d = relayout_desc(ptrs, pool.tensor, pool.alias, ids2.to(cuda_device), sl2.to(cuda_device), blocks)
        hfk.check(hfk.lib().hfk_swap_relayout(C.byref(d), 1, 0, stream_handle()), "relayout out")
        torch.cuda.synchronize()
        o.relayout_swap_out(cpu_dev, cpu_pool, ids2, sl2)
        assert same_bytes(pool.tensor, cpu_pool)
        assert hfk.device_status() == 0
    finally:
        pool.close()


def test_relayout_swap_single_block_equals_multi_layer_block_transfer(hfk, cuda_device):
    """With one block the multi-block op is the reference's operator."""
    z = np.load(GOLDEN / "block_transfer_int8.npz")
    host = torch.from_numpy(z["host_block"])
    B, L, H, D = host.shape
    pool = PinnedPool((3, B, L, H, D), torch.int8)
    try:
        pool.tensor[1].copy_(host)
        gpu_dev = [dev_zeros((4, H, B, D), torch.int8, cuda_device) for _ in range(L)]
        ptrs = ptr_table(gpu_dev, cuda_device)
        ids, sl = torch.tensor([2], device=cuda_device), torch.tensor([1], device=cuda_device)
        d = relayout_desc(ptrs, pool.tensor, pool.alias, ids, sl, 4)
        hfk.check(hfk.lib().hfk_swap_relayout(C.byref(d), 0, 0, stream_handle()), "relayout in")
        bad = relayout_desc(ptrs, pool.tensor, pool.alias, torch.tensor([9], device=cuda_device), sl, 4)
        hfk.check(hfk.lib().hfk_swap_relayout(C.byref(bad), 0, 0, stream_handle()), "relayout bad id")
        torch.cuda.synchronize()
        assert np.array_equal(torch.stack([g[2] for g in gpu_dev], 0).cpu().numpy(), z["expected"])
        assert hfk.device_status() == hfk.HFK_DEV_BAD_DEVICE_BLOCK_ID
    finally:
        pool.close()


# ------------------------------------------------------ staged copy-engine mover ---
@pytest.mark.parametrize("staging_slots", [1, 3, 64])
def test_staged_swap_matches_oracle(hfk, cuda_device, staging_slots):
    layers, blocks, chunk, nslots, n = 3, 40, (16, 2, 64), 50, 17
    case = SwapCase(hfk, cuda_device, layers, blocks, chunk, torch.bfloat16, nslots, seed=21)
    try:
        slot_bytes = layers * 2 * 16 * 2 * 64 * 2
        staging = torch.empty(staging_slots * slot_bytes, dtype=torch.uint8, device=cuda_device)
        ids = o.distinct_ids(n, blocks, 1)
        rest = [x for x in o.distinct_ids(nslots, nslots, 2).tolist() if not 5 <= x <= 10][:n - 6]
        slots = torch.tensor(list(range(5, 11)) + rest)                   # distinct, starts with a consecutive run
        ids_d = ids.to(cuda_device)
        d = case.desc(ids_d, ids_d)
        lib = hfk.lib()
        hfk.check(lib.hfk_swap_staged(C.byref(d), slots.data_ptr(), case.pool.ptr, staging.data_ptr(), staging.numel(),
                                      1, 0, stream_handle()), "staged out")
        torch.cuda.synchronize()
        o.swap_out(case.cpu_k, case.cpu_v, case.cpu_pool, ids, slots)
        assert same_bytes(case.pool_view, case.cpu_pool)
        ids2 = o.distinct_ids(n, blocks, 3)
        ids2_d = ids2.to(cuda_device)
        d = case.desc(ids2_d, ids2_d)
        hfk.check(lib.hfk_swap_staged(C.byref(d), slots.data_ptr(), case.pool.ptr, staging.data_ptr(), staging.numel(),
                                      0, 8, stream_handle()), "staged in")
        torch.cuda.synchronize()
        o.swap_in(case.cpu_k, case.cpu_v, case.cpu_pool, ids2, slots)
        for g, c in zip(case.gpu_k + case.gpu_v, case.cpu_k + case.cpu_v):
            assert same_bytes(g, c)
        assert hfk.device_status() == 0
        # errors: a staging buffer below one slot, a slot id out of range (checked on the host), a layer-major pool
        assert lib.hfk_swap_staged(C.byref(d), slots.data_ptr(), case.pool.ptr, staging.data_ptr(), slot_bytes - 16,
                                   0, 0, stream_handle()) == hfk.HFK_ERR_TOO_LARGE
        bad = slots.clone()
        bad[3] = nslots
        assert lib.hfk_swap_staged(C.byref(d), bad.data_ptr(), case.pool.ptr, staging.data_ptr(), staging.numel(),
                                   0, 0, stream_handle()) == hfk.HFK_ERR_INVALID_ARG
        d.host_kv_stride = d.host_slot_stride * nslots    # K and V in two separate arrays: valid, but not slot-contiguous
        assert lib.hfk_swap_staged(C.byref(d), slots.data_ptr(), case.pool.ptr, staging.data_ptr(), staging.numel(),
                                   0, 0, stream_handle()) == hfk.HFK_ERR_UNSUPPORTED
    finally:
        case.close()


def test_bounded_wait_gives_up_and_reports_instead_of_hanging(hfk, cuda_device):
    """A wait on a barrier nobody completes runs out after its limit; the kernel returns, the status
    word says so and the context keeps working."""
    import time

    lib = hfk.lib()
    assert hfk.device_status() == 0
    t0 = time.perf_counter()
    hfk.check(lib.hfk_selftest_wait_timeout(20000, stream_handle()), "selftest")   # 20 ms
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert 0.015 < dt < 1.0
    assert hfk.device_status() == hfk.HFK_DEV_WAIT_TIMEOUT
    x = torch.arange(8, device=cuda_device)
    assert int(x.sum()) == 28 and hfk.device_status() == 0
    assert lib.hfk_selftest_wait_timeout(0, stream_handle()) == hfk.HFK_ERR_INVALID_ARG


# ------------------------------------------------------------- seeded random geometries ---
def _rand_cases(n, seed):
    g = torch.Generator().manual_seed(seed)

    def r(lo, hi):
        return int(torch.randint(lo, hi + 1, (1,), generator=g))

    cases = []
    for i in range(n):
        layers, blocks = r(1, 5), r(4, 48)
        tok_elems = 8 * r(1, 40)                      # fp16 elements per token row: 16-byte multiples
        bs = r(1, 24)
        cases.append(dict(i=i, layers=layers, blocks=blocks, bs=bs, tok=tok_elems, slots=r(blocks, 2 * blocks),
                          n=r(1, blocks), mover=r(1, 2), ctas=r(1, 40), layout=("block_major", "layer_major")[r(0, 1)],
                          idt=(torch.int64, torch.int32)[r(0, 1)], stage=(4096, 8192, 16384, 32768)[r(0, 3)],
                          stages=r(3, 6)))
    return cases


@pytest.mark.parametrize("c", _rand_cases(24, 2024), ids=lambda c: f"case{c['i']}")
def test_random_geometries_swap_gather_and_staged(hfk, cuda_device, c):
    lib = hfk.lib()
    assert lib.hfk_set_bulk_geometry(c["stage"], c["stages"]) == 0
    case = SwapCase(hfk, cuda_device, c["layers"], c["blocks"], (c["bs"], 1, c["tok"]), torch.float16, c["slots"],
                    seed=300 + c["i"], pool_layout=c["layout"])
    try:
        ids = o.distinct_ids(c["n"], c["blocks"], 1).to(c["idt"])
        slots = o.distinct_ids(c["n"], c["slots"], 2).to(c["idt"])
        run_swap(hfk, lib.hfk_swap_out, case.desc(ids.to(cuda_device), slots.to(cuda_device)), c["mover"], c["ctas"])
        o.swap_out(case.cpu_k, case.cpu_v, case.cpu_pool, ids, slots)
        assert same_bytes(case.pool_view, case.cpu_pool)
        ids2 = o.distinct_ids(c["n"], c["blocks"], 3).to(c["idt"])
        if c["layout"] == "block_major" and c["i"] % 2 == 0:   # staged mover needs a slot-contiguous pool
            staging = torch.empty(3 * c["layers"] * 2 * c["bs"] * c["tok"] * 2 + 64, dtype=torch.uint8,
                                  device=cuda_device)
            d = case.desc(ids2.to(cuda_device), ids2.to(cuda_device))
            hfk.check(lib.hfk_swap_staged(C.byref(d), slots.data_ptr(), case.pool.ptr, staging.data_ptr(),
                                          staging.numel(), 0, c["ctas"], stream_handle()), "staged in")
            torch.cuda.synchronize()
        else:
            run_swap(hfk, lib.hfk_swap_in, case.desc(ids2.to(cuda_device), slots.to(cuda_device)), c["mover"], c["ctas"])
        o.swap_in(case.cpu_k, case.cpu_v, case.cpu_pool, ids2, slots)
        for g, cc in zip(case.gpu_k + case.gpu_v, case.cpu_k + case.cpu_v):
            assert same_bytes(g, cc)
        # gather a ragged batch out of the same caches
        gen = torch.Generator().manual_seed(c["i"])
        lens, left = [], c["blocks"]
        while left > 0 and len(lens) < 7:
            nb = int(torch.randint(0, left + 1, (1,), generator=gen))
            lens.append(max(0, nb * c["bs"] - int(torch.randint(0, c["bs"], (1,), generator=gen))) if nb else 0)
            left -= nb
        if sum(lens) == 0:
            lens[0] = 1
        tables = o.block_tables_for(lens, c["bs"], c["blocks"], seed=c["i"])
        if tables.shape[1] == 0:
            tables = torch.zeros((len(lens), 1), dtype=torch.int64)
        lens_t = torch.tensor(lens)
        k_out, v_out = run_gather(hfk, cuda_device, case.cpu_k, case.cpu_v, tables, lens_t, c["bs"], c["mover"],
                                  c["idt"], ctas=c["ctas"])
        ko, vo = o.paged_gather(case.cpu_k, case.cpu_v, tables, lens_t, c["bs"])
        assert same_bytes(k_out, ko) and same_bytes(v_out, vo)
        assert hfk.device_status() == 0
    finally:
        case.close()
        lib.hfk_set_bulk_geometry(0, 0)
