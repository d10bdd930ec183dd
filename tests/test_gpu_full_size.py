"""The benchmark configurations at their full transfer sizes, through size-independent properties:
swap-out -> swap-in round trip into other blocks reproduces the source blocks, nothing else in the
cache changes, and the gather equals a device-side index_select.  (The oracle itself runs on the touched
blocks only; the pools are not duplicated on the CPU.)"""
import pytest
import torch

from oracle import kv_oracle as o
from tests.helpers import u8

pytestmark = pytest.mark.gpu


def _fill(t, seed):
    from bench import fill_random_bytes

    fill_random_bytes(t, seed)


def _checksum(t):
    """Order-sensitive 64-bit checksum of a device tensor's bytes."""
    w = t.contiguous().view(torch.int64).view(-1)
    idx = torch.arange(w.numel(), device=w.device, dtype=torch.int64)
    return int((w * (2 * idx + 1)).sum().item())


@pytest.mark.parametrize("name,dev_blocks,slots", [
    ("llama3_8b_swap", 20000, 4096),        # 512 blocks x 32 layers x K,V x 32 KiB = 1.07 GB per direction
    ("llama3_70b_tp8_swap", 6000, 4200),    # 2048 blocks x 80 layers x K,V x 32 KiB = 10.7 GB per direction
    ("qwen2_7b_fp8_prefetch", 8192, 4096),  # 256 blocks x 28 layers, 8 KiB fp8 chunks
])
@pytest.mark.parametrize("mover", [pytest.param(1, id="vector"), pytest.param(2, id="bulk")])
def test_full_size_swap_round_trip(cuda_device, name, dev_blocks, slots, mover):
    from heterofusedkernels_b200.connector import PagedKVCache

    g = o.CONFIGS[name]
    free, _ = torch.cuda.mem_get_info()
    need = 2 * g.layers * dev_blocks * g.block_bytes
    if need > free - (8 << 30):
        pytest.skip("not enough free HBM for the full-size cache")
    cache = PagedKVCache(g.layers, dev_blocks, g.block_size, g.kv_heads, g.head_dim, g.dtype, cuda_device,
                         host_slots=slots)  # the host pool is shrunk, the transferred set is not
    _fill(cache._k_store, 1)
    _fill(cache._v_store, 2)
    assert cache.swap_bytes(g.n_swap) == g.swap_bytes()
    perm = torch.randperm(dev_blocks, generator=torch.Generator().manual_seed(7))
    src, dst = perm[:g.n_swap].to(cuda_device), perm[g.n_swap:2 * g.n_swap].to(cuda_device)
    rest = perm[2 * g.n_swap:].to(cuda_device)
    slot_ids = torch.randperm(slots, generator=torch.Generator().manual_seed(8))[:g.n_swap].to(cuda_device)
    rest_sum = [_checksum(cache._k_store[:, rest[:256]]), _checksum(cache._v_store[:, rest[:256]])]
    cache.swap_out(src, slot_ids, mover=mover)
    cache.swap_in(dst, slot_ids, mover=mover)
    torch.cuda.synchronize()
    assert cache.status() == 0
    # property: the destination blocks now hold the source blocks' bytes, every layer, K and V
    for store in (cache._k_store, cache._v_store):
        for l0 in range(0, g.layers, 8):
            a = store[l0:l0 + 8].index_select(1, src)
            b = store[l0:l0 + 8].index_select(1, dst)
            assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    assert rest_sum == [_checksum(cache._k_store[:, rest[:256]]), _checksum(cache._v_store[:, rest[:256]])]
    # oracle on a sample of the touched blocks: host slot == source block, bit for bit
    for i in (0, g.n_swap // 2, g.n_swap - 1):
        s, b = int(slot_ids[i]), int(src[i])
        for l in (0, g.layers - 1):
            assert torch.equal(u8(cache.host_pool[s, l, 0]), u8(cache.k_caches[l][b].cpu()))
            assert torch.equal(u8(cache.host_pool[s, l, 1]), u8(cache.v_caches[l][b].cpu()))


@pytest.mark.parametrize("mover", [pytest.param(1, id="vector"), pytest.param(2, id="bulk")])
def test_full_size_paged_gather_equals_device_index_select(cuda_device, mover):
    """64 sequences of 512..8192 tokens (seeded), 32 layers, bf16 [16, 8, 128] pages, in the
    configuration's 40000-block cache (83.9 GB + 36.1 GB of outputs); when less HBM is free the cache
    falls back to 20000 blocks — the gathered set (about 17 thousand pages per layer) stays the full one."""
    from heterofusedkernels_b200.connector import PagedKVCache

    g = o.CONFIGS["llama3_8b_gather"]
    lens = o.gather_seq_lens(seed=0)
    torch.cuda.empty_cache()
    free, _ = torch.cuda.mem_get_info()
    total = sum(lens)
    blocks = g.num_blocks
    need = lambda nb: 2 * g.layers * nb * g.block_bytes + 2 * g.layers * total * g.token_bytes  # noqa: E731
    if need(blocks) > free - (10 << 30):
        blocks = 20000
    if need(blocks) > free - (8 << 30):
        pytest.skip("not enough free HBM")
    cache = PagedKVCache(g.layers, blocks, g.block_size, g.kv_heads, g.head_dim, g.dtype, cuda_device)
    _fill(cache._k_store, 3)
    _fill(cache._v_store, 4)
    tables = o.block_tables_for(lens, g.block_size, blocks, seed=1)
    lens_t = torch.tensor(lens)
    k_out, v_out = cache.paged_gather(tables, lens_t, mover=mover)
    torch.cuda.synchronize()
    assert cache.status() == 0 and k_out.shape == (g.layers, total, g.kv_heads, g.head_dim)
    tables_d = tables.to(cuda_device)
    start = 0
    for s, n in enumerate(lens):
        nb = (n + g.block_size - 1) // g.block_size
        for store, out in ((cache._k_store, k_out), (cache._v_store, v_out)):
            ref = store[:, tables_d[s, :nb]].flatten(1, 2)[:, :n]
            assert torch.equal(ref.view(torch.int16), out[:, start:start + n].view(torch.int16)), f"sequence {s}"
        start += n
    # oracle on one layer of one sequence, through the CPU
    s, l = 7, 5
    nb = (lens[s] + g.block_size - 1) // g.block_size
    cpu_pages = cache.k_caches[l][tables_d[s, :nb]].cpu()
    small_table = torch.arange(nb).view(1, -1)
    ko, _ = o.paged_gather([cpu_pages], [cpu_pages], small_table, torch.tensor([lens[s]]), g.block_size)
    st = sum(lens[:s])
    assert torch.equal(u8(ko[0]), u8(k_out[l, st:st + lens[s]].cpu()))
