"""The torch operator surface (torch.ops.pcie_through.* + heterofusedkernels.memory) on the GPU,
written the way the reference's own tests drive it (pcieThrough/tests/test_transfer_kernel.py,
test_gather.py) but with seeded random data and exact byte comparison."""
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


@pytest.mark.parametrize("layers", [1, 32])
@pytest.mark.parametrize("num_blocks", [1, 8])
@pytest.mark.parametrize("use_fused_copy", [False, True])
def test_multi_layer_block_kv_transfer_like_the_reference_test(ops, cuda_device, layers, num_blocks, use_fused_copy):
    """Mirror of test_multi_layer_block_kv_transfer (test_transfer_kernel.py:15-88): a pool of host
    blocks [B,L,H,D] from alloc_numa_pinned_tensor, device blocks [L,H,B,D], per-block pointer tables,
    two alternating streams, aiv=4."""
    op, memory = ops
    block_size, heads, head_dim, dtype = 1024, 1, 128, torch.int8
    total_host_blocks, total_dev_blocks, simultaneous = 12, 8, 2
    host_shape = (total_host_blocks, block_size, layers, heads, head_dim)
    raw = memory.alloc_numa_pinned_tensor(total_host_blocks * block_size * layers * heads * head_dim)
    raw.copy_(o.random_kv_bytes((raw.numel(),), torch.int8, seed=layers + num_blocks))
    host_blocks = list(raw.view(dtype).view(host_shape).unbind(0))
    device_blocks = list(torch.zeros((total_dev_blocks, layers, heads, block_size, head_dim), dtype=dtype,
                                     device=cuda_device).unbind(0))
    ptrs = []
    for t in device_blocks:
        p = torch.empty(layers, dtype=torch.int64)
        for i in range(layers):
            p[i] = t[i].data_ptr()
        ptrs.append(p.to(cuda_device))
    streams = [torch.cuda.Stream() for _ in range(simultaneous)]
    staging = [torch.empty([block_size, layers, heads, head_dim], dtype=dtype, device=cuda_device)
               for _ in range(simultaneous)]
    torch.cuda.synchronize()
    for i in range(num_blocks):
        with torch.cuda.stream(streams[i % simultaneous]):
            if use_fused_copy:
                op.fused_memcpy_multi_layer_block_transfer(ptrs[i], host_blocks[i], staging[i % simultaneous], 4)
            else:
                op.multi_layer_block_transfer(ptrs[i], host_blocks[i], 4)
    for s in streams:
        s.synchronize()
    for i in range(num_blocks):
        back = device_blocks[i].cpu()
        assert torch.equal(host_blocks[i], back.permute(2, 0, 1, 3))  # the reference's assertion (:81-83)


def test_gather_like_the_reference_benchmark(ops, cuda_device):
    """test_gather.py:31-61 with a written table: pinned fp16 table, ids on the device, aiv=4."""
    op, memory = ops
    rows, dim = 20000, 512
    table = memory.alloc_numa_pinned_tensor(rows * dim * 2).view(torch.float16).view(rows, dim)
    table.copy_(o.random_kv_bytes((rows, dim), torch.float16, seed=3))
    for bs in (8, 64, 1000, 2040):
        ids = torch.randint(0, rows, (bs,), generator=torch.Generator().manual_seed(bs)).to(cuda_device)
        dst = torch.zeros((bs, dim), dtype=torch.float16, device=cuda_device)
        op.gather(table, dst, ids, aiv=4)
        op.gather(table, dst, ids)  # default core count
        torch.cuda.synchronize()
        assert torch.equal(u8(dst.cpu()), u8(table[ids.cpu()]))
    # a table that already lives on the device is accepted (pcieThrough/README.md:18)
    dev_table = table.to(cuda_device)
    dst = torch.zeros((8, dim), dtype=torch.float16, device=cuda_device)
    ids = torch.arange(8, device=cuda_device, dtype=torch.int32) * 7
    op.gather(dev_table, dst, ids, 2)
    assert torch.equal(u8(dst.cpu()), u8(table[ids.cpu().long()]))


def test_memory_module_on_a_real_device(ops, cuda_device):
    _, memory = ops
    t = memory.alloc_numa_pinned_tensor(1 << 20)
    assert t.dtype == torch.int8 and t.device.type == "cpu" and t.numel() == 1 << 20 and int(t.abs().sum()) == 0
    assert t.is_pinned()
    alias = memory.get_device_ptr(t.data_ptr())
    assert alias != 0 and memory.get_device_ptr(t.data_ptr() + 4096) == alias + 4096
    before = memory.registry_count()
    plain = torch.empty(4096, dtype=torch.float16)          # pageable tensor: registered in place
    assert memory.host_register(plain) != 0 and memory.registry_count() == before + 1
    memory.host_unregister(plain)
    with pytest.raises(RuntimeError, match="Device must be CPU"):
        memory.host_register(torch.zeros(4, device=cuda_device))
    ptr = t.data_ptr()
    del t                                                  # the tensor owns the mapping
    assert memory.get_device_ptr(ptr) == 0


def test_error_behaviour_of_the_ops(ops, cuda_device):
    op, memory = ops
    dst = torch.zeros((4, 16), dtype=torch.float16, device=cuda_device)
    ids = torch.zeros(4, dtype=torch.int64, device=cuda_device)
    with pytest.raises(RuntimeError, match="not inside a range registered"):
        op.gather(torch.zeros((8, 16), dtype=torch.float16), dst, ids)      # unregistered host table
    table = torch.zeros((8, 16), dtype=torch.float16, device=cuda_device)
    with pytest.raises(RuntimeError, match="Number of AIV blocks should be positive"):
        op.gather(table, dst, ids, 0)
    with pytest.raises(RuntimeError, match="int64 or int32"):
        op.gather(table, dst, ids.to(torch.float32))
    host = memory.alloc_numa_pinned_tensor(16 * 2 * 1 * 24).view(16, 2, 1, 24)
    ptrs = torch.zeros(2, dtype=torch.int64, device=cuda_device)
    with pytest.raises(RuntimeError, match="multiple of 16"):
        op.multi_layer_block_transfer(ptrs, host)                           # 24-byte head rows
    with pytest.raises(RuntimeError, match="expected 2"):
        op.multi_layer_block_transfer(torch.zeros(3, dtype=torch.int64, device=cuda_device),
                                      memory.alloc_numa_pinned_tensor(16 * 2 * 32).view(16, 2, 1, 32))


@pytest.mark.parametrize("mover", [None, 1, 2])
def test_connector_swap_and_gather_round_trip(ops, cuda_device, mover):
    from heterofusedkernels_b200.connector import PagedKVCache

    g = o.CONFIGS["tiny"]
    cache = PagedKVCache(g.layers, g.num_blocks, g.block_size, g.kv_heads, g.head_dim, g.dtype, cuda_device,
                         host_slots=g.host_slots)
    shape = (g.num_blocks, g.block_size, g.kv_heads, g.head_dim)
    cpu_k = [o.random_kv_bytes(shape, g.dtype, 2 * l) for l in range(g.layers)]
    cpu_v = [o.random_kv_bytes(shape, g.dtype, 2 * l + 1) for l in range(g.layers)]
    for d, s in zip(cache.k_caches + cache.v_caches, cpu_k + cpu_v):
        d.copy_(s)
    ids, slots, back = o.distinct_ids(8, 64, 1), o.distinct_ids(8, 128, 2), o.distinct_ids(8, 64, 3)
    cache.swap_out(ids.tolist(), slots.tolist(), mover=mover)              # python lists are accepted
    cache.swap_in(back, slots, mover=mover)
    ref_pool = torch.zeros_like(cache.host_pool)
    o.swap_out(cpu_k, cpu_v, ref_pool, ids, slots)
    o.swap_in(cpu_k, cpu_v, ref_pool, back, slots)
    torch.cuda.synchronize()
    assert torch.equal(u8(cache.host_pool), u8(ref_pool))
    tables = o.block_tables_for(g.seq_lens, g.block_size, g.num_blocks, seed=4)
    k_out, v_out = cache.paged_gather(tables, torch.tensor(g.seq_lens), mover=mover)
    ko, vo = o.paged_gather(cpu_k, cpu_v, tables, torch.tensor(g.seq_lens), g.block_size)
    assert torch.equal(u8(k_out.cpu()), u8(ko)) and torch.equal(u8(v_out.cpu()), u8(vo))
    # staged mover (packing kernel + one copy-engine transfer per slot)
    cache.swap_out_staged(back, slots, staging_bytes=1 << 20)
    cache.swap_in_staged(ids, slots, staging_bytes=1 << 20)
    o.swap_out(cpu_k, cpu_v, ref_pool, back, slots)
    o.swap_in(cpu_k, cpu_v, ref_pool, ids, slots)
    torch.cuda.synchronize()
    assert torch.equal(u8(cache.host_pool), u8(ref_pool))
    for dt, ct in zip(cache.k_caches + cache.v_caches, cpu_k + cpu_v):
        assert torch.equal(u8(dt.cpu()), u8(ct))
    # copy-engine twins
    cache.swap_out_copy_engine(ids, slots)
    torch.cuda.synchronize()
    o.swap_out(cpu_k, cpu_v, ref_pool, ids, slots)
    assert torch.equal(u8(cache.host_pool), u8(ref_pool))
    assert cache.status() == 0


def test_layerwise_prefetcher_moves_single_layers(ops, cuda_device):
    from heterofusedkernels_b200.connector import LayerwisePrefetcher, PagedKVCache

    cache = PagedKVCache(4, 32, 16, 4, 128, o.FP8, cuda_device, host_slots=48)
    for i, t in enumerate(cache.k_caches + cache.v_caches):
        t.copy_(o.random_kv_bytes(tuple(t.shape), o.FP8, 50 + i))
    cache.host_pool.view(torch.uint8).copy_(o.random_kv_bytes(tuple(cache.host_pool.shape), o.FP8, 9).view(torch.uint8))
    cpu_k = [t.cpu() for t in cache.k_caches]
    cpu_v = [t.cpu() for t in cache.v_caches]
    ref_pool = cache.host_pool.clone()
    pf = LayerwisePrefetcher(cache)
    torch.cuda.synchronize()
    for l in range(4):
        in_ids, in_slots = o.distinct_ids(6, 32, 10 + l).to(cuda_device), o.distinct_ids(6, 24, 20 + l).to(cuda_device)
        out_ids = torch.tensor([i for i in range(32) if i not in in_ids.tolist()][:5], device=cuda_device)
        out_slots = (o.distinct_ids(5, 24, 30 + l) + 24).to(cuda_device)
        pf.prefetch(l, in_ids, in_slots)
        pf.evict(l, out_ids, out_slots)
        pf.wait(l)
        o.swap_out([cpu_k[l]], [cpu_v[l]], ref_pool[:, l:l + 1], out_ids.cpu(), out_slots.cpu())
        o.swap_in([cpu_k[l]], [cpu_v[l]], ref_pool[:, l:l + 1], in_ids.cpu(), in_slots.cpu())
    torch.cuda.synchronize()
    assert torch.equal(u8(cache.host_pool), u8(ref_pool))
    for d, c in zip(cache.k_caches + cache.v_caches, cpu_k + cpu_v):
        assert torch.equal(u8(d.cpu()), u8(c))


def test_relayout_swap_ops(ops, cuda_device):
    op, memory = ops
    B, L, H, D, slots, blocks, n = 64, 4, 2, 128, 10, 12, 7
    pool = memory.alloc_numa_pinned_tensor(slots * B * L * H * D * 2).view(torch.bfloat16).view(slots, B, L, H, D)
    pool.copy_(o.random_kv_bytes((slots, B, L, H, D), torch.bfloat16, seed=1))
    cpu_pool = pool.clone()
    cpu_dev = [o.random_kv_bytes((blocks, H, B, D), torch.bfloat16, seed=5 + l) for l in range(L)]
    gpu_dev = [t.to(cuda_device) for t in cpu_dev]
    ptrs = torch.tensor([t.data_ptr() for t in gpu_dev], dtype=torch.int64).to(cuda_device)
    ids, sl = o.distinct_ids(n, blocks, 1), o.distinct_ids(n, slots, 2)
    op.swap_in_relayout(ptrs, pool, ids.to(cuda_device), sl.to(cuda_device), blocks)
    o.relayout_swap_in(cpu_dev, cpu_pool, ids, sl)
    ids2, sl2 = o.distinct_ids(n, blocks, 3), o.distinct_ids(n, slots, 4)
    op.swap_out_relayout(ptrs, pool, ids2.to(cuda_device), sl2.to(cuda_device), blocks, None, 8)
    o.relayout_swap_out(cpu_dev, cpu_pool, ids2, sl2)
    torch.cuda.synchronize()
    assert torch.equal(u8(pool), u8(cpu_pool))
    for g, c in zip(gpu_dev, cpu_dev):
        assert torch.equal(u8(g.cpu()), u8(c))


def test_swap_and_gather_ops_replay_from_a_cuda_graph(ops, cuda_device):
    """The ops neither allocate nor synchronise, so a serving engine can capture them; the reference
    leaves graph capture open (multi_layer_block_transfer_torch.cpp:57)."""
    from heterofusedkernels_b200.connector import PagedKVCache

    g = o.CONFIGS["tiny"]
    cache = PagedKVCache(g.layers, g.num_blocks, g.block_size, g.kv_heads, g.head_dim, g.dtype, cuda_device,
                         host_slots=g.host_slots)
    shape = (g.num_blocks, g.block_size, g.kv_heads, g.head_dim)
    ids = o.distinct_ids(8, 64, 1).to(cuda_device)
    slots = o.distinct_ids(8, 128, 2).to(cuda_device)
    back = o.distinct_ids(8, 64, 3).to(cuda_device)
    tables = o.block_tables_for(g.seq_lens, g.block_size, g.num_blocks, seed=4).to(cuda_device)
    lens = torch.tensor(g.seq_lens, device=cuda_device)
    k_out = torch.zeros((g.layers, sum(g.seq_lens), g.kv_heads, g.head_dim), dtype=g.dtype, device=cuda_device)
    v_out = torch.zeros_like(k_out)

    def step():
        cache.swap_out(ids, slots)
        cache.swap_in(back, slots)
        cache.paged_gather(tables, lens, k_out, v_out)

    side = torch.cuda.Stream(cuda_device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        step()                                   # warm-up outside the capture
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            step()
    for rep in range(2):                         # new cache contents, same graph
        cpu_k = [o.random_kv_bytes(shape, g.dtype, 100 * rep + 2 * l) for l in range(g.layers)]
        cpu_v = [o.random_kv_bytes(shape, g.dtype, 100 * rep + 2 * l + 1) for l in range(g.layers)]
        for d, s in zip(cache.k_caches + cache.v_caches, cpu_k + cpu_v):
            d.copy_(s)
        cache.host_pool.zero_()
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        ref_pool = torch.zeros_like(cache.host_pool)
        o.swap_out(cpu_k, cpu_v, ref_pool, ids.cpu(), slots.cpu())
        o.swap_in(cpu_k, cpu_v, ref_pool, back.cpu(), slots.cpu())
        ko, vo = o.paged_gather(cpu_k, cpu_v, tables.cpu(), lens.cpu(), g.block_size)
        assert torch.equal(u8(cache.host_pool), u8(ref_pool))
        assert torch.equal(u8(k_out.cpu()), u8(ko)) and torch.equal(u8(v_out.cpu()), u8(vo))
    assert cache.status() == 0
