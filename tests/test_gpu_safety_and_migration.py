"""GPU tests of the inputs that must never become a device fault (bad entries in device-resident
pointer tables, errors returned before anything is enqueued, the read-and-clear status word) and of
the block migration between two caches, on one GPU and — when the box has two — across NVLink.
Everything goes through the C ABI and is compared with the CPU oracle on raw bytes."""
import ctypes as C

import pytest
import torch

from oracle import kv_oracle as o
from tests.helpers import PinnedPool, dev_zeros, gather_desc, ptr_table, relayout_desc, stream_handle, swap_desc, u8
from tests.test_gpu_parity import MOVERS, SwapCase, run_swap, same_bytes

pytestmark = pytest.mark.gpu


def _corrupt(table: torch.Tensor, entry: int, how: str) -> torch.Tensor:
    t = table.clone()
    t[entry] = 0 if how == "null" else int(t[entry]) + 8   # 8 = not a multiple of 16
    return t


@pytest.mark.parametrize("mover", MOVERS)
@pytest.mark.parametrize("how", ["null", "misaligned"])
def test_bad_layer_pointers_are_skipped_and_reported_not_dereferenced(hfk, cuda_device, mover, how):
    """A null or misaligned layer base in the device pointer table: that layer's K (or V) is skipped,
    HFK_DEV_BAD_LAYER_PTR is raised, every other chunk is moved, and no bad address is ever formed."""
    layers = 3
    case = SwapCase(hfk, cuda_device, layers, 16, (4, 2, 64), torch.float16, 16, seed=31)
    try:
        ids, slots = o.distinct_ids(6, 16, 1), o.distinct_ids(6, 16, 2)
        ids_d, slots_d = ids.to(cuda_device), slots.to(cuda_device)
        good_k = case.k_ptrs
        case.k_ptrs = _corrupt(good_k, 1, how)      # K of layer 1 is unusable
        run_swap(hfk, hfk.lib().hfk_swap_out, case.desc(ids_d, slots_d), mover)
        assert hfk.device_status() == hfk.HFK_DEV_BAD_LAYER_PTR
        expect = case.cpu_pool.clone()
        o.swap_out(case.cpu_k, case.cpu_v, expect, ids, slots)
        expect[:, 1, 0] = case.cpu_pool[:, 1, 0]    # K chunks of layer 1 stay as they were
        assert same_bytes(case.pool_view, expect)
        # swap-in with the same bad table: layer 1's K cache keeps its contents
        before = case.gpu_k[1].clone()
        ids2 = o.distinct_ids(6, 16, 3)
        run_swap(hfk, hfk.lib().hfk_swap_in, case.desc(ids2.to(cuda_device), slots_d), mover)
        assert hfk.device_status() == hfk.HFK_DEV_BAD_LAYER_PTR
        assert same_bytes(case.gpu_k[1], before)
        keep = case.cpu_k[1].clone()
        o.swap_in(case.cpu_k, case.cpu_v, expect, ids2, slots)
        case.cpu_k[1] = keep
        for g, c in zip(case.gpu_k + case.gpu_v, case.cpu_k + case.cpu_v):
            assert same_bytes(g, c)
        case.k_ptrs = good_k
        run_swap(hfk, hfk.lib().hfk_swap_out, case.desc(ids_d, slots_d), mover)
        assert hfk.device_status() == 0
    finally:
        case.close()


@pytest.mark.parametrize("mover", MOVERS)
def test_paged_gather_skips_a_bad_layer_pointer(hfk, cuda_device, mover):
    layers, blocks, bs = 3, 24, 4
    shape = (blocks, bs, 2, 32)
    cpu_k = [o.random_kv_bytes(shape, torch.float16, 2 * l) for l in range(layers)]
    cpu_v = [o.random_kv_bytes(shape, torch.float16, 2 * l + 1) for l in range(layers)]
    lens = torch.tensor([9, 4, 13])
    tables = o.block_tables_for(lens.tolist(), bs, blocks, seed=3)
    gk, gv = [t.to(cuda_device) for t in cpu_k], [t.to(cuda_device) for t in cpu_v]
    total = int(lens.sum())
    k_out = dev_zeros((layers, total, 2, 32), torch.float16, cuda_device)
    v_out = torch.zeros_like(k_out)
    kp, vp = ptr_table(gk, cuda_device), _corrupt(ptr_table(gv, cuda_device), 2, "misaligned")
    d = gather_desc(kp, vp, k_out, v_out, tables.to(cuda_device), lens.to(cuda_device), bs, blocks)
    hfk.check(hfk.lib().hfk_paged_gather(C.byref(d), mover, 0, stream_handle()), "paged_gather")
    torch.cuda.synchronize()
    assert hfk.device_status() == hfk.HFK_DEV_BAD_LAYER_PTR
    ko, vo = o.paged_gather(cpu_k, cpu_v, tables, lens, bs)
    vo[2] = 0                                        # V of layer 2 was skipped: the output stays zero
    assert same_bytes(k_out, ko) and same_bytes(v_out, vo)


def test_block_transfer_and_relayout_skip_a_bad_layer_pointer(hfk, cuda_device):
    B, L, H, D = 16, 3, 2, 16
    host = o.random_kv_bytes((B, L, H, D), torch.int8, seed=4)
    pool = PinnedPool((2, B, L, H, D), torch.int8)
    try:
        pool.tensor[0].copy_(host)
        pool.tensor[1].copy_(host)
        layers = [dev_zeros((H, B, D), torch.int8, cuda_device) for _ in range(L)]
        ptrs = _corrupt(ptr_table(layers, cuda_device), 0, "null")
        hfk.check(hfk.lib().hfk_multi_layer_block_transfer(ptrs.data_ptr(), pool.alias, B, L, H, D, 1, 4,
                                                           stream_handle()), "transfer")
        torch.cuda.synchronize()
        assert hfk.device_status() == hfk.HFK_DEV_BAD_LAYER_PTR
        expect = o.block_transfer(host)
        assert int(layers[0].abs().sum()) == 0
        for l in (1, 2):
            assert same_bytes(layers[l], expect[l])
        # the multi-block form: caches [blocks, H, B, D], layer 2 misaligned
        caches = [dev_zeros((4, H, B, D), torch.int8, cuda_device) for _ in range(L)]
        lp = _corrupt(ptr_table(caches, cuda_device), 2, "misaligned")
        ids = torch.tensor([3, 1], device=cuda_device)
        slots = torch.tensor([0, 1], device=cuda_device)
        d = relayout_desc(lp, pool.tensor, pool.alias, ids, slots, 4)
        hfk.check(hfk.lib().hfk_swap_relayout(C.byref(d), 0, 0, stream_handle()), "relayout in")
        torch.cuda.synchronize()
        assert hfk.device_status() == hfk.HFK_DEV_BAD_LAYER_PTR
        assert int(caches[2].abs().sum()) == 0
        for l in (0, 1):
            assert same_bytes(caches[l][3], expect[l]) and same_bytes(caches[l][1], expect[l])
    finally:
        pool.close()


def test_staged_transfer_errors_leave_the_stream_and_the_staging_bytes_untouched(hfk, cuda_device):
    """head_dim*elt = 8 is rejected (HFK_ERR_ALIGNMENT) before the host->staging copy is enqueued:
    the staging buffer keeps its bytes, and a following valid call is bit exact."""
    lib = hfk.lib()
    B, L, H, D = 32, 2, 2, 8
    host8 = o.random_kv_bytes((B, L, H, D), torch.int8, seed=1)          # 8-byte heads: not transferable
    pool8 = PinnedPool((B, L, H, D), torch.int8)
    good = o.random_kv_bytes((B, L, H, 16), torch.int8, seed=2)
    pool = PinnedPool((B, L, H, 16), torch.int8)
    try:
        pool8.tensor.copy_(host8)
        pool.tensor.copy_(good)
        layers = [dev_zeros((H, B, 16), torch.int8, cuda_device) for _ in range(L)]
        ptrs = ptr_table(layers, cuda_device)
        staging = torch.full((B * L * H * 16,), 0x5A, dtype=torch.uint8, device=cuda_device)
        rc = lib.hfk_fused_memcpy_multi_layer_block_transfer(ptrs.data_ptr(), pool8.ptr, staging.data_ptr(), B, L, H, D, 1,
                                                             0, stream_handle())
        assert rc == hfk.HFK_ERR_ALIGNMENT
        rc = lib.hfk_fused_memcpy_multi_layer_block_transfer_static(ptrs.data_ptr(), pool8.ptr, B, L, H, D, 1, 0,
                                                                    stream_handle())
        assert rc == hfk.HFK_ERR_ALIGNMENT
        torch.cuda.synchronize()
        assert bool((staging == 0x5A).all())
        for call in ("caller", "static"):
            for t in layers:
                t.zero_()
            if call == "caller":
                rc = lib.hfk_fused_memcpy_multi_layer_block_transfer(ptrs.data_ptr(), pool.ptr, staging.data_ptr(), B, L, H,
                                                                     16, 1, 0, stream_handle())
            else:
                rc = lib.hfk_fused_memcpy_multi_layer_block_transfer_static(ptrs.data_ptr(), pool.ptr, B, L, H, 16, 1, 0,
                                                                            stream_handle())
            hfk.check(rc, call)
            torch.cuda.synchronize()
            for t, e in zip(layers, o.block_transfer(good)):
                assert same_bytes(t, e)
    finally:
        pool8.close()
        pool.close()


def test_status_word_is_read_and_cleared_in_one_step_and_is_per_device(hfk, cuda_device):
    lib = hfk.lib()
    side = torch.cuda.Stream(cuda_device)
    assert hfk.device_status() == 0
    table = torch.zeros((4, 16), dtype=torch.uint8, device=cuda_device)
    dst = torch.zeros((2, 16), dtype=torch.uint8, device=cuda_device)
    ids = torch.tensor([1, 9], device=cuda_device)                      # 9 is out of range
    with torch.cuda.stream(side):
        hfk.check(lib.hfk_gather(table.data_ptr(), dst.data_ptr(), ids.data_ptr(), 1, 2, 16, 4, 0,
                                 side.cuda_stream), "gather")
    side.synchronize()
    # a read on another stream sees the bit (the word belongs to the device, not to a stream) ...
    assert hfk.device_status(torch.cuda.current_stream().cuda_stream) == hfk.HFK_DEV_BAD_ROW_ID
    # ... and has cleared it for everybody
    assert hfk.device_status(side.cuda_stream) == 0


# ------------------------------------------------------------------ migration ---
def _migrate_desc(hfk, src_k, src_v, dst_k, dst_v, src_ids, dst_ids, block_bytes, n_src, n_dst, tables_on):
    d = hfk.MigrateDesc()
    tabs = [ptr_table(x, tables_on) for x in (src_k, src_v, dst_k, dst_v)]
    d.src_k_layer_ptrs, d.src_v_layer_ptrs = tabs[0].data_ptr(), tabs[1].data_ptr()
    d.dst_k_layer_ptrs, d.dst_v_layer_ptrs = tabs[2].data_ptr(), tabs[3].data_ptr()
    d.src_block_ids, d.dst_block_ids = src_ids.data_ptr(), dst_ids.data_ptr()
    d.ids_are_int64 = 1 if src_ids.dtype == torch.int64 else 0
    d.layers, d.n_blocks, d.block_bytes = len(src_k), src_ids.numel(), block_bytes
    d.src_block_stride = d.dst_block_stride = block_bytes
    d.num_src_blocks, d.num_dst_blocks = n_src, n_dst
    return d, tabs


@pytest.mark.parametrize("layers,src_blocks,dst_blocks,chunk,dtype,n,idt", [
    (2, 16, 24, (16, 8, 128), torch.float16, 8, torch.int64),      # 32 KiB chunks (Llama layout)
    (3, 40, 40, (3, 1, 8), torch.float16, 17, torch.int32),        # 48-byte chunks
    (28, 64, 48, (16, 4, 128), o.FP8, 33, torch.int64),            # fp8, many layers
    (1, 3000, 3000, (2, 1, 64), torch.int8, 2500, torch.int64),    # more ids than one smem tile
])
def test_migrate_blocks_between_two_caches_on_one_gpu(hfk, cuda_device, layers, src_blocks, dst_blocks, chunk, dtype,
                                                      n, idt):
    mk = lambda nb, seed: [o.random_kv_bytes((nb,) + chunk, dtype, seed + i) for i in range(layers)]  # noqa: E731
    src_k, src_v, dst_k, dst_v = mk(src_blocks, 0), mk(src_blocks, 100), mk(dst_blocks, 200), mk(dst_blocks, 300)
    g = [[t.to(cuda_device) for t in x] for x in (src_k, src_v, dst_k, dst_v)]
    src_ids, dst_ids = o.distinct_ids(n, src_blocks, 1).to(idt), o.distinct_ids(n, dst_blocks, 2).to(idt)
    bb = src_k[0][0].numel() * src_k[0].element_size()
    s_d, d_d = src_ids.to(cuda_device), dst_ids.to(cuda_device)
    d, _tabs = _migrate_desc(hfk, *g, s_d, d_d, bb, src_blocks, dst_blocks, cuda_device)
    hfk.check(hfk.lib().hfk_migrate_blocks(C.byref(d), 0, stream_handle()), "migrate")
    torch.cuda.synchronize()
    assert hfk.device_status() == 0
    o.migrate_blocks(src_k, src_v, dst_k, dst_v, src_ids, dst_ids)
    for gpu, cpu in zip(g[2] + g[3], dst_k + dst_v):
        assert same_bytes(gpu, cpu)
    for gpu, cpu in zip(g[0] + g[1], src_k + src_v):                  # the source is only read
        assert same_bytes(gpu, cpu)


def test_migrate_blocks_reports_bad_ids_and_the_copy_engine_twin_matches(hfk, cuda_device):
    layers, blocks, chunk = 2, 12, (4, 2, 64)
    mk = lambda seed: [o.random_kv_bytes((blocks,) + chunk, torch.float16, seed + i) for i in range(layers)]  # noqa: E731
    src_k, src_v, dst_k, dst_v = mk(0), mk(10), mk(20), mk(30)
    g = [[t.to(cuda_device) for t in x] for x in (src_k, src_v, dst_k, dst_v)]
    bb = 4 * 2 * 64 * 2
    src_ids = torch.tensor([0, 5, 99, 7], dtype=torch.int64)
    dst_ids = torch.tensor([1, -3, 2, 3], dtype=torch.int64)
    d, _tabs = _migrate_desc(hfk, *g, src_ids.to(cuda_device), dst_ids.to(cuda_device), bb, blocks, blocks, cuda_device)
    hfk.check(hfk.lib().hfk_migrate_blocks(C.byref(d), 3, stream_handle()), "migrate")
    torch.cuda.synchronize()
    assert hfk.device_status() == hfk.HFK_DEV_BAD_DEVICE_BLOCK_ID
    good = torch.tensor([0, 3])
    o.migrate_blocks(src_k, src_v, dst_k, dst_v, src_ids[good], dst_ids[good])
    for gpu, cpu in zip(g[2] + g[3], dst_k + dst_v):
        assert same_bytes(gpu, cpu)
    # copy-engine twin: host arrays, one copy per chunk
    s2, d2 = o.distinct_ids(5, blocks, 4), o.distinct_ids(5, blocks, 5)
    dd, _tabs2 = _migrate_desc(hfk, *g, s2, d2, bb, blocks, blocks, "cpu")
    hfk.check(hfk.lib().hfk_migrate_blocks_copy_engine(C.byref(dd), 0, 0, stream_handle()), "migrate copy engine")
    torch.cuda.synchronize()
    o.migrate_blocks(src_k, src_v, dst_k, dst_v, s2, d2)
    for gpu, cpu in zip(g[2] + g[3], dst_k + dst_v):
        assert same_bytes(gpu, cpu)


def test_migrate_blocks_between_two_gpus_pull_and_push(hfk, cuda_device):
    """Two caches on two GPUs: the destination GPU pulls over NVLink (peer loads), then the source GPU
    pushes other blocks (peer stores); both against the oracle.  Needs a box with two GPUs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    if not torch.cuda.can_device_access_peer(0, 1):
        pytest.skip("GPU 0 cannot address GPU 1 as a peer")
    dev0, dev1 = torch.device("cuda", 0), torch.device("cuda", 1)
    lib = hfk.lib()
    layers, blocks, chunk = 4, 64, (16, 8, 128)
    mk = lambda seed: [o.random_kv_bytes((blocks,) + chunk, torch.bfloat16, seed + i) for i in range(layers)]  # noqa: E731
    src_k, src_v, dst_k, dst_v = mk(0), mk(10), mk(20), mk(30)
    g_src = [[t.to(dev0) for t in x] for x in (src_k, src_v)]
    g_dst = [[t.to(dev1) for t in x] for x in (dst_k, dst_v)]
    bb = 16 * 8 * 128 * 2
    for run_on, other, seed in ((dev1, 0, 1), (dev0, 1, 3)):     # pull on GPU 1, then push from GPU 0
        src_ids, dst_ids = o.distinct_ids(20, blocks, seed), o.distinct_ids(20, blocks, seed + 1)
        with torch.cuda.device(run_on):
            hfk.check(lib.hfk_enable_peer_access(other), "peer access")
            d, _tabs = _migrate_desc(hfk, g_src[0], g_src[1], g_dst[0], g_dst[1], src_ids.to(run_on), dst_ids.to(run_on),
                                     bb, blocks, blocks, run_on)
            hfk.check(lib.hfk_migrate_blocks(C.byref(d), 0, torch.cuda.current_stream(run_on).cuda_stream), "migrate")
            torch.cuda.synchronize(run_on)
            assert hfk.device_status(torch.cuda.current_stream(run_on).cuda_stream) == 0
        o.migrate_blocks(src_k, src_v, dst_k, dst_v, src_ids, dst_ids)
        for gpu, cpu in zip(g_dst[0] + g_dst[1], dst_k + dst_v):
            assert same_bytes(gpu, cpu)
    # the copy-engine twin across the two GPUs
    s2, d2 = o.distinct_ids(6, blocks, 8), o.distinct_ids(6, blocks, 9)
    dd, _tabs2 = _migrate_desc(hfk, g_src[0], g_src[1], g_dst[0], g_dst[1], s2, d2, bb, blocks, blocks, "cpu")
    with torch.cuda.device(dev1):
        hfk.check(lib.hfk_migrate_blocks_copy_engine(C.byref(dd), 0, 1, torch.cuda.current_stream(dev1).cuda_stream),
                  "migrate copy engine")
        torch.cuda.synchronize(dev1)
    o.migrate_blocks(src_k, src_v, dst_k, dst_v, s2, d2)
    for gpu, cpu in zip(g_dst[0] + g_dst[1], dst_k + dst_v):
        assert same_bytes(gpu, cpu)
    torch.cuda.set_device(cuda_device)
