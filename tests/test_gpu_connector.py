"""The caller-side shim on the GPU: slot allocation from the free list, the staged mover with its
copy lanes, the prefetcher's ordering against the compute stream, layer ranges, and swaps that run
while a matmul loop occupies the main stream — all against the CPU oracle on raw bytes."""
import pytest
import torch

from oracle import kv_oracle as o
from tests.helpers import u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(cuda_device):
    import pcie_through  # noqa: F401
    from heterofusedkernels import memory

    return torch.ops.pcie_through, memory


def _filled_cache(device, layers, blocks, bs, heads, hd, dtype, slots, seed=0, pool_layout="slot_major"):
    from heterofusedkernels_b200.connector import PagedKVCache

    cache = PagedKVCache(layers, blocks, bs, heads, hd, dtype, device, host_slots=slots, pool_layout=pool_layout)
    shape = (blocks, bs, heads, hd)
    cpu_k = [o.random_kv_bytes(shape, dtype, seed + 2 * l) for l in range(layers)]
    cpu_v = [o.random_kv_bytes(shape, dtype, seed + 2 * l + 1) for l in range(layers)]
    for d, s in zip(cache.k_caches + cache.v_caches, cpu_k + cpu_v):
        d.copy_(s)
    torch.cuda.synchronize()
    return cache, cpu_k, cpu_v


@pytest.mark.parametrize("lanes", [1, 2, 4])
def test_swaps_driven_by_the_slot_allocator_and_the_staged_copy_lanes(ops, cuda_device, lanes):
    """swap_out without slot ids takes a run of consecutive slots from the free list; the staged mover
    then crosses the link with few large copies, dealt to `lanes` copy streams."""
    import heterofusedkernels_b200 as pkg

    lib = pkg.capi.lib()
    cache, cpu_k, cpu_v = _filled_cache(cuda_device, 3, 64, 16, 2, 64, torch.bfloat16, 96, seed=3)
    ref_pool = torch.zeros_like(cache.host_pool)
    pkg.capi.check(lib.hfk_set_staged_copy_lanes(lanes), "lanes")
    try:
        ids_a = o.distinct_ids(20, 64, 1)
        slots_a = cache.swap_out(ids_a, mover="staged")                        # one run of 20 slots
        assert slots_a.tolist() == list(range(20)) and cache.slot_pool.free_count == 76
        ids_b = o.distinct_ids(30, 64, 2)
        slots_b = cache.swap_out(ids_b)                                         # kernel mover, next run
        assert slots_b.tolist() == list(range(20, 50))
        o.swap_out(cpu_k, cpu_v, ref_pool, ids_a, slots_a)
        o.swap_out(cpu_k, cpu_v, ref_pool, ids_b, slots_b)
        torch.cuda.synchronize()
        assert torch.equal(u8(cache.host_pool), u8(ref_pool))
        # bring the first set back into other blocks and free its slots; the hole is reused by the next request
        back = o.distinct_ids(20, 64, 3)
        cache.swap_in(back, slots_a, mover="staged", release=True)
        o.swap_in(cpu_k, cpu_v, ref_pool, back, slots_a)
        torch.cuda.synchronize()
        for d, c in zip(cache.k_caches + cache.v_caches, cpu_k + cpu_v):
            assert torch.equal(u8(d.cpu()), u8(c))
        assert cache.slot_pool.runs() == [(0, 20), (50, 46)]
        ids_c = o.distinct_ids(12, 64, 4)
        slots_c = cache.swap_out(ids_c, mover="staged")                        # best fit: the 20-slot hole
        assert slots_c.tolist() == list(range(12))
        ids_d = o.distinct_ids(50, 64, 5)
        slots_d = cache.swap_out(ids_d, mover="staged")                        # no run holds 50: two runs, longest first
        assert sorted(slots_d.tolist()) == list(range(12, 16)) + list(range(50, 96))
        o.swap_out(cpu_k, cpu_v, ref_pool, ids_c, slots_c)
        o.swap_out(cpu_k, cpu_v, ref_pool, ids_d, slots_d)
        torch.cuda.synchronize()
        assert torch.equal(u8(cache.host_pool), u8(ref_pool))
        with pytest.raises(RuntimeError, match="exhausted"):
            cache.swap_out(o.distinct_ids(10, 64, 6))
        assert cache.status() == 0
    finally:
        lib.hfk_set_staged_copy_lanes(0)


@pytest.mark.parametrize("fraction", ["0.5", "0.0", "1.0", "0.37"])
def test_hybrid_mover_splits_a_swap_between_copy_engine_and_kernel(ops, cuda_device, fraction):
    cache, cpu_k, cpu_v = _filled_cache(cuda_device, 3, 64, 16, 2, 64, torch.bfloat16, 96, seed=13)
    ref_pool = torch.zeros_like(cache.host_pool)
    ids, slots, back = o.distinct_ids(41, 64, 1), o.distinct_ids(41, 96, 2), o.distinct_ids(41, 64, 3)
    cache.swap_out(ids, slots, mover="hybrid:" + fraction)
    cache.swap_in(back, slots, mover="hybrid:" + fraction)
    o.swap_out(cpu_k, cpu_v, ref_pool, ids, slots)
    o.swap_in(cpu_k, cpu_v, ref_pool, back, slots)
    torch.cuda.synchronize()
    assert torch.equal(u8(cache.host_pool), u8(ref_pool))
    for d, c in zip(cache.k_caches + cache.v_caches, cpu_k + cpu_v):
        assert torch.equal(u8(d.cpu()), u8(c))
    assert cache.status() == 0


def test_evict_right_after_a_kernel_wrote_the_blocks_reads_the_new_bytes(ops, cuda_device):
    """No global synchronisation: the main stream is kept busy, then writes the blocks, and evict is
    issued immediately.  The swap-out stream must wait for the writes."""
    from heterofusedkernels_b200.connector import LayerwisePrefetcher

    cache, cpu_k, cpu_v = _filled_cache(cuda_device, 2, 32, 16, 4, 128, torch.float16, 32, seed=7)
    pf = LayerwisePrefetcher(cache)
    a = torch.randn(4096, 4096, device=cuda_device, dtype=torch.bfloat16)
    ids = o.distinct_ids(12, 32, 1).to(cuda_device)
    slots = o.distinct_ids(12, 32, 2).to(cuda_device)
    new_k = o.random_kv_bytes((12, 16, 4, 128), torch.float16, 91).to(cuda_device)
    new_v = o.random_kv_bytes((12, 16, 4, 128), torch.float16, 92).to(cuda_device)
    torch.cuda.synchronize()
    for _ in range(30):                     # some milliseconds of work ahead of the writes
        a = a @ a
        a = a / a.abs().max().clamp_min(1)
    cache.k_caches[1].index_copy_(0, ids, new_k)
    cache.v_caches[1].index_copy_(0, ids, new_v)
    done = pf.evict(1, ids, slots)
    # and the other way round: a prefetch must not overwrite blocks before the kernel ahead of it has read them
    snapshot = cache.k_caches[0].index_select(0, ids)       # reads the blocks on the main stream
    cache.host_pool.view(torch.uint8).view(32, 2, 2, -1)[:, 0] = 0x3C
    pf.prefetch(0, ids, slots)
    done.synchronize()
    pf.in_stream.synchronize()
    torch.cuda.synchronize()
    pool = cache.host_pool
    assert torch.equal(u8(pool[slots.cpu(), 1, 0]), u8(new_k.cpu()))
    assert torch.equal(u8(pool[slots.cpu(), 1, 1]), u8(new_v.cpu()))
    assert torch.equal(u8(snapshot.cpu()), u8(cpu_k[0][ids.cpu()]))
    assert bool((cache.k_caches[0].index_select(0, ids).view(torch.uint8) == 0x3C).all())
    assert cache.status() == 0


@pytest.mark.parametrize("group", [1, 3])
@pytest.mark.parametrize("pool_layout,mover", [("slot_major", None), ("slot_major", 2), ("layer_major", None),
                                               ("layer_major", "staged"), ("slot_major", "staged")])
def test_prefetch_and_evict_next_to_a_matmul_loop_are_bit_exact(ops, cuda_device, group, pool_layout, mover):
    """Swap-in of the next layers and swap-out of the current ones on the side streams while matmuls run
    on the main stream; `group` layers per launch; kernel movers and the staged (copy-engine) mover, on
    both pool layouts.  Checked against the oracle afterwards."""
    from heterofusedkernels_b200.connector import LayerwisePrefetcher

    layers, blocks, slots = 6, 64, 96
    cache, cpu_k, cpu_v = _filled_cache(cuda_device, layers, blocks, 16, 4, 128, o.FP8, slots, seed=11,
                                        pool_layout=pool_layout)
    cache.host_pool.view(torch.uint8).copy_(o.random_kv_bytes(tuple(cache.host_pool.shape), o.FP8, 5).view(torch.uint8))
    ref_pool = cache.host_pool.clone()
    pf = LayerwisePrefetcher(cache)
    a = torch.randn(2048, 2048, device=cuda_device, dtype=torch.bfloat16)
    b = torch.randn(2048, 2048, device=cuda_device, dtype=torch.bfloat16)
    c = torch.empty_like(a)
    spans = [range(s, min(s + group, layers)) for s in range(0, layers, group)]
    plans = []
    for i, span in enumerate(spans):
        perm = torch.randperm(blocks, generator=torch.Generator().manual_seed(20 + i))
        sl = torch.randperm(slots, generator=torch.Generator().manual_seed(40 + i))
        if i % 2 == 1:   # every other launch gets its slots as two runs, the way the free list hands them out
            sl = torch.arange(20 + i, 20 + i + 19)
        plans.append((perm[:10], sl[:10], perm[10:19], sl[10:19]))
    torch.cuda.synchronize()
    for i, span in enumerate(spans):
        in_ids, in_slots, out_ids, out_slots = (t.to(cuda_device) for t in plans[i])
        pf.prefetch(span, in_ids, in_slots, mover=mover, host_slot_ids_cpu=plans[i][1])
        pf.evict(span, out_ids, out_slots, mover=mover, host_slot_ids_cpu=plans[i][3])
        for _ in range(4 * len(span)):
            torch.matmul(a, b, out=c)
        for l in span:
            pf.wait(l)
            pf.wait_evicted(l)
    pf.quiesce()
    torch.cuda.synchronize()
    for i, span in enumerate(spans):
        in_ids, in_slots, out_ids, out_slots = plans[i]
        ks, vs = [cpu_k[l] for l in span], [cpu_v[l] for l in span]
        view = ref_pool[:, span.start:span.stop]
        o.swap_out(ks, vs, view, out_ids, out_slots)
        o.swap_in(ks, vs, view, in_ids, in_slots)
    assert torch.equal(u8(cache.host_pool), u8(ref_pool))
    for d, cpu in zip(cache.k_caches + cache.v_caches, cpu_k + cpu_v):
        assert torch.equal(u8(d.cpu()), u8(cpu))
    assert cache.status() == 0


def test_connector_migrates_blocks_between_two_caches(ops, cuda_device):
    src, src_k, src_v = _filled_cache(cuda_device, 3, 32, 16, 2, 64, torch.float16, 0, seed=1)
    dst, dst_k, dst_v = _filled_cache(cuda_device, 3, 48, 16, 2, 64, torch.float16, 0, seed=50)
    s_ids, d_ids = o.distinct_ids(14, 32, 1), o.distinct_ids(14, 48, 2)
    src.migrate_to(dst, s_ids, d_ids)
    # and inside one cache (a block copy): disjoint source and destination blocks
    perm = o.distinct_ids(20, 48, 3)
    dst.migrate_to(dst, perm[:10], perm[10:])
    torch.cuda.synchronize()
    o.migrate_blocks(src_k, src_v, dst_k, dst_v, s_ids, d_ids)
    o.migrate_blocks(dst_k, dst_v, dst_k, dst_v, perm[:10], perm[10:])
    for d, c in zip(dst.k_caches + dst.v_caches, dst_k + dst_v):
        assert torch.equal(u8(d.cpu()), u8(c))
    assert dst.status() == 0
    if torch.cuda.device_count() >= 2 and torch.cuda.can_device_access_peer(1, 0):
        far, far_k, far_v = _filled_cache(torch.device("cuda", 1), 3, 40, 16, 2, 64, torch.float16, 0, seed=80)
        f_ids = o.distinct_ids(9, 40, 4)
        push_ids = torch.tensor([x for x in range(40) if x not in f_ids.tolist()][:5])
        src.migrate_to(far, s_ids[:9], f_ids, run_on="dst")      # GPU 1 pulls over NVLink
        src.migrate_to(far, s_ids[9:], push_ids, run_on="src")   # GPU 0 pushes
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        o.migrate_blocks(src_k, src_v, far_k, far_v, s_ids[:9], f_ids)
        o.migrate_blocks(src_k, src_v, far_k, far_v, s_ids[9:], push_ids)
        for d, c in zip(far.k_caches + far.v_caches, far_k + far_v):
            assert torch.equal(u8(d.cpu()), u8(c))
        torch.cuda.set_device(cuda_device)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_sequence_of_connector_operations_matches_a_cpu_model(ops, cuda_device, seed):
    """A seeded random run of what a KV-offload connector does — swap blocks out to slots the free list
    hands out, bring some back into other blocks and release their slots, copy blocks inside the cache,
    gather sequences — mirrored step by step on CPU tensors with the oracle; caches, pool and gathered
    sequences must agree byte for byte at the end, and the free list must account for every slot."""
    import random

    rng = random.Random(seed)
    layers, blocks, bs, heads, hd, slots = 3, 96, 8, 2, 32, 80
    cache, cpu_k, cpu_v = _filled_cache(cuda_device, layers, blocks, bs, heads, hd, torch.float16, slots, seed=100 + seed)
    cache.host_pool.view(torch.uint8).fill_(0x11)
    ref_pool = cache.host_pool.clone()
    held = []                                    # (slots tensor) of swapped-out block groups still on the host
    for step in range(40):
        op = rng.choice(["out", "out", "in", "copy", "gather"])
        if op == "out" and cache.slot_pool.free_count >= 12:
            n = rng.randint(1, 12)
            ids = torch.tensor(rng.sample(range(blocks), n))
            mover = rng.choice([None, 1, 2, "staged", "hybrid:0.5"])
            got = cache.swap_out(ids, mover=mover)                      # slots from the free list
            o.swap_out(cpu_k, cpu_v, ref_pool, ids, got)
            held.append(got)
        elif op == "in" and held:
            got = held.pop(rng.randrange(len(held)))
            ids = torch.tensor(rng.sample(range(blocks), got.numel()))
            cache.swap_in(ids, got, mover=rng.choice([None, 1, 2, "staged", "hybrid:0.3"]), release=True)
            o.swap_in(cpu_k, cpu_v, ref_pool, ids, got)
        elif op == "copy":
            pick = rng.sample(range(blocks), 2 * rng.randint(1, 10))
            src, dst = torch.tensor(pick[:len(pick) // 2]), torch.tensor(pick[len(pick) // 2:])
            cache.migrate_to(cache, src, dst)
            o.migrate_blocks(cpu_k, cpu_v, cpu_k, cpu_v, src, dst)
        elif op == "gather":
            lens = [rng.randint(0, 5 * bs) for _ in range(rng.randint(1, 5))]
            lens[0] = max(lens[0], 1)
            tables = o.block_tables_for(lens, bs, blocks, seed=step)
            k_out, v_out = cache.paged_gather(tables, torch.tensor(lens))
            ko, vo = o.paged_gather(cpu_k, cpu_v, tables, torch.tensor(lens), bs)
            assert torch.equal(u8(k_out.cpu()), u8(ko)) and torch.equal(u8(v_out.cpu()), u8(vo)), f"step {step}"
    torch.cuda.synchronize()
    assert torch.equal(u8(cache.host_pool), u8(ref_pool))
    for d, c in zip(cache.k_caches + cache.v_caches, cpu_k + cpu_v):
        assert torch.equal(u8(d.cpu()), u8(c))
    assert cache.slot_pool.free_count == slots - sum(h.numel() for h in held)
    assert cache.status() == 0
