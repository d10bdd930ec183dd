"""Host-side checks of the C ABI that need no GPU: exported symbols, struct layout,
argument validation (every failing path returns before any CUDA call) and the registry."""
import ctypes as C
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "hfk_b200.h").read_text()


def declared_functions():
    body = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(hfk_[a-z0-9_]+)\s*\(", body)))


def test_library_exports_every_declared_symbol(hfk):
    lib = hfk.lib()
    names = declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/hfk_b200.h but not exported"
    assert set(names) == set(hfk.PROTOTYPES), "ctypes prototypes and header disagree"


def test_error_codes_and_defines_match_header(hfk):
    for name, val in re.findall(r"^#define (HFK_[A-Z0-9_]+) \(?(0x[0-9a-f]+|-?\d+)u?\)?\s*(?:/\*.*)?$", HEADER, flags=re.M):
        if hasattr(hfk, name):
            assert getattr(hfk, name) == int(val, 0), name
    assert hfk.HFK_MAX_SEQS == int(re.search(r"#define HFK_MAX_SEQS (\d+)", HEADER).group(1))
    m = re.search(r"#define HFK_STATIC_STAGING_BYTES \((\d+)u \* (\d+)u \* (\d+)u\)", HEADER)
    assert hfk.HFK_STATIC_STAGING_BYTES == int(m.group(1)) * int(m.group(2)) * int(m.group(3))
    assert hfk.lib().hfk_strerror(hfk.HFK_ERR_ALIGNMENT).decode().startswith("address or size")
    assert hfk.lib().hfk_version().decode().count(".") == 2


def test_struct_layouts_follow_the_header_order(hfk):
    for struct, cname in ((hfk.SwapDesc, "hfk_swap_desc"), (hfk.PagedGatherDesc, "hfk_paged_gather_desc"),
                          (hfk.RelayoutDesc, "hfk_relayout_desc"), (hfk.MigrateDesc, "hfk_migrate_desc")):
        m = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), HEADER, flags=re.S)
        body = re.sub(r"/\*.*?\*/", "", m.group(1), flags=re.S)
        fields = [re.split(r"[\s\*]+", f.strip())[-1] for f in body.split(";") if f.strip()]
        assert fields == [f[0] for f in struct._fields_]


def _swap_desc(hfk, **over):
    d = hfk.SwapDesc()
    buf = torch.zeros(64, dtype=torch.int64)
    d.k_layer_ptrs = d.v_layer_ptrs = d.device_block_ids = d.host_slot_ids = buf.data_ptr()
    d.host_pool = 0x10000
    d.ids_are_int64, d.layers, d.n_blocks = 1, 2, 4
    d.block_bytes = d.device_block_stride = 4096
    d.host_slot_stride, d.host_layer_stride, d.host_kv_stride = 16384, 8192, 4096
    d.num_device_blocks = d.num_host_slots = 8
    for k, v in over.items():
        setattr(d, k, v)
    return d, buf


@pytest.mark.parametrize("over,code", [
    (dict(host_pool=0), "HFK_ERR_INVALID_ARG"), (dict(layers=0), "HFK_ERR_INVALID_ARG"),
    (dict(n_blocks=-1), "HFK_ERR_INVALID_ARG"), (dict(block_bytes=4008), "HFK_ERR_ALIGNMENT"),
    (dict(host_kv_stride=4104), "HFK_ERR_ALIGNMENT"), (dict(host_pool=0x10008), "HFK_ERR_ALIGNMENT"),
    (dict(device_block_stride=2048), "HFK_ERR_INVALID_ARG"), (dict(num_host_slots=0), "HFK_ERR_INVALID_ARG"),
    (dict(device_block_ids=0), "HFK_ERR_INVALID_ARG"), (dict(layers=5000), "HFK_ERR_TOO_LARGE"),
    # strides that let chunks overlap: K on top of V, slots inside a slot, an expanded (stride-0) dimension
    (dict(host_kv_stride=2048), "HFK_ERR_INVALID_ARG"), (dict(host_slot_stride=8192), "HFK_ERR_INVALID_ARG"),
    (dict(host_layer_stride=0), "HFK_ERR_INVALID_ARG"), (dict(host_slot_stride=-16384), "HFK_ERR_INVALID_ARG")])
def test_swap_validation_errors(hfk, over, code):
    d, _keep = _swap_desc(hfk, **over)
    for fn in (hfk.lib().hfk_swap_out, hfk.lib().hfk_swap_in):
        assert fn(C.byref(d), hfk.MOVER_AUTO, 0, None) == getattr(hfk, code)
    assert hfk.last_error() != ""
    assert hfk.lib().hfk_swap_copy_engine(C.byref(d), 1, None) == getattr(hfk, code)


def test_swap_unknown_mover_and_null_descriptor(hfk):
    assert hfk.lib().hfk_swap_out(None, 0, 0, None) == hfk.HFK_ERR_INVALID_ARG
    d, _keep = _swap_desc(hfk)
    assert hfk.lib().hfk_swap_in(C.byref(d), 9, 0, None) == hfk.HFK_ERR_INVALID_ARG


def test_copy_engine_rejects_out_of_range_ids_on_the_host(hfk):
    d, buf = _swap_desc(hfk)
    buf[:4] = torch.tensor([0, 1, 99, 2])
    assert hfk.lib().hfk_swap_copy_engine(C.byref(d), 0, None) == hfk.HFK_ERR_INVALID_ARG
    assert "out of range" in hfk.last_error()


def test_staged_and_relayout_validation_errors(hfk):
    lib = hfk.lib()
    d, buf = _swap_desc(hfk)
    stg = 0x40000
    assert lib.hfk_swap_staged(C.byref(d), buf.data_ptr(), 0x10000, None, 1 << 20, 1, 0, None) == hfk.HFK_ERR_INVALID_ARG
    assert lib.hfk_swap_staged(C.byref(d), buf.data_ptr(), 0x10000, stg, 4096, 1, 0, None) == hfk.HFK_ERR_TOO_LARGE
    assert lib.hfk_swap_staged(C.byref(d), None, 0x10000, stg, 1 << 20, 1, 0, None) == hfk.HFK_ERR_INVALID_ARG
    buf[:4] = torch.tensor([0, 1, 8, 2])                     # slot 8 of 8: rejected on the host
    assert lib.hfk_swap_staged(C.byref(d), buf.data_ptr(), 0x10000, stg, 1 << 20, 0, 0, None) == hfk.HFK_ERR_INVALID_ARG
    d3, buf3 = _swap_desc(hfk, host_slot_stride=16384 - 16)                      # slot stride below one slot
    assert lib.hfk_swap_staged(C.byref(d3), buf3.data_ptr(), 0x10000, stg, 1 << 20, 0, 0, None) == hfk.HFK_ERR_INVALID_ARG
    d2, buf2 = _swap_desc(hfk, host_layer_stride=65536, host_slot_stride=8192)   # layer-major pool
    assert lib.hfk_swap_staged(C.byref(d2), buf2.data_ptr(), 0x10000, stg, 1 << 20, 0, 0, None) == hfk.HFK_ERR_UNSUPPORTED
    r = hfk.RelayoutDesc()
    r.layer_ptrs = r.device_block_ids = r.host_slot_ids = buf.data_ptr()
    r.host_pool = 0x10000
    r.ids_are_int64, r.layers, r.n_blocks = 1, 2, 3
    r.block_size, r.heads, r.head_bytes = 16, 2, 64
    r.device_block_stride, r.host_slot_stride = 2048, 4096
    r.num_device_blocks = r.num_host_slots = 8
    for field, value, code in (("head_bytes", 24, "HFK_ERR_ALIGNMENT"), ("device_block_stride", 1024, "HFK_ERR_INVALID_ARG"),
                               ("host_slot_stride", 2048, "HFK_ERR_INVALID_ARG"), ("layers", 0, "HFK_ERR_INVALID_ARG"),
                               ("host_pool", 0, "HFK_ERR_INVALID_ARG")):
        old = getattr(r, field)
        setattr(r, field, value)
        assert lib.hfk_swap_relayout(C.byref(r), 0, 0, None) == getattr(hfk, code), field
        setattr(r, field, old)
    assert lib.hfk_swap_relayout(None, 1, 0, None) == hfk.HFK_ERR_INVALID_ARG
    assert lib.hfk_set_bulk_lag(9) == hfk.HFK_ERR_INVALID_ARG and lib.hfk_set_bulk_lag(0) == hfk.HFK_OK
    assert lib.hfk_set_staged_copy_lanes(5) == hfk.HFK_ERR_INVALID_ARG and lib.hfk_set_staged_copy_lanes(0) == hfk.HFK_OK


def test_vector_geometry_accepts_only_compiled_combinations(hfk):
    lib = hfk.lib()
    for th, un in ((512, 4), (256, 8), (256, 4), (1024, 2), (128, 8), (0, 0)):
        assert lib.hfk_set_vector_geometry(th, un) == hfk.HFK_OK
    for th, un in ((512, 8), (64, 4), (0, 4), (-1, -1)):
        assert lib.hfk_set_vector_geometry(th, un) == hfk.HFK_ERR_UNSUPPORTED
        assert "not compiled" in hfk.last_error()
    # a rejected pair leaves the previous (default) setting in place
    assert lib.hfk_set_vector_geometry(0, 0) == hfk.HFK_OK


def test_block_transfer_checks_everything_before_it_enqueues(hfk):
    """The staged transfers validate the whole call first: with no CUDA device here, reaching the copy
    would return HFK_ERR_CUDA, so the codes below prove that the checks come before it."""
    lib = hfk.lib()
    buf = torch.zeros(64, dtype=torch.int64)
    p = buf.data_ptr()
    fused = lib.hfk_fused_memcpy_multi_layer_block_transfer
    assert fused(p, p, p, 16, 2, 1, 8, 1, 0, None) == hfk.HFK_ERR_ALIGNMENT        # head_dim*elt = 8
    assert fused(None, p, p, 16, 2, 1, 16, 1, 0, None) == hfk.HFK_ERR_INVALID_ARG  # null pointer table
    assert fused(p, p, p, 16, 5000, 1, 16, 1, 0, None) == hfk.HFK_ERR_TOO_LARGE    # > 4096 layers
    assert fused(p, p, p + 8, 16, 2, 1, 16, 1, 0, None) == hfk.HFK_ERR_ALIGNMENT   # misaligned staging


def _migrate_desc(hfk, **over):
    d = hfk.MigrateDesc()
    buf = torch.zeros(64, dtype=torch.int64)
    p = buf.data_ptr()
    d.src_k_layer_ptrs = d.src_v_layer_ptrs = d.dst_k_layer_ptrs = d.dst_v_layer_ptrs = p
    d.src_block_ids = d.dst_block_ids = p
    d.ids_are_int64, d.layers, d.n_blocks = 1, 2, 4
    d.block_bytes = d.src_block_stride = d.dst_block_stride = 4096
    d.num_src_blocks = d.num_dst_blocks = 8
    for k, v in over.items():
        setattr(d, k, v)
    return d, buf


@pytest.mark.parametrize("over,code", [
    (dict(dst_v_layer_ptrs=0), "HFK_ERR_INVALID_ARG"), (dict(layers=0), "HFK_ERR_INVALID_ARG"),
    (dict(n_blocks=-2), "HFK_ERR_INVALID_ARG"), (dict(block_bytes=4008), "HFK_ERR_ALIGNMENT"),
    (dict(src_block_stride=2048), "HFK_ERR_INVALID_ARG"), (dict(dst_block_stride=4104), "HFK_ERR_ALIGNMENT"),
    (dict(num_dst_blocks=0), "HFK_ERR_INVALID_ARG"), (dict(src_block_ids=0), "HFK_ERR_INVALID_ARG"),
    (dict(layers=3000), "HFK_ERR_TOO_LARGE")])
def test_migrate_validation_errors(hfk, over, code):
    d, _keep = _migrate_desc(hfk, **over)
    assert hfk.lib().hfk_migrate_blocks(C.byref(d), 0, None) == getattr(hfk, code)
    assert hfk.lib().hfk_migrate_blocks_copy_engine(C.byref(d), 0, 0, None) == getattr(hfk, code)


def test_migrate_copy_engine_checks_ids_and_layer_bases_on_the_host(hfk):
    lib = hfk.lib()
    assert lib.hfk_migrate_blocks(None, 0, None) == hfk.HFK_ERR_INVALID_ARG
    d, buf = _migrate_desc(hfk)
    buf[:4] = torch.tensor([0, 1, 8, 2])   # id 8 of 8
    assert lib.hfk_migrate_blocks_copy_engine(C.byref(d), 0, 0, None) == hfk.HFK_ERR_INVALID_ARG
    assert "out of range" in hfk.last_error()
    buf[:4] = torch.tensor([0, 1, 3, 2])   # valid ids, but the same words serve as layer bases: 0 is null
    assert lib.hfk_migrate_blocks_copy_engine(C.byref(d), 0, 0, None) == hfk.HFK_ERR_ALIGNMENT
    assert "null or misaligned base" in hfk.last_error()


def _gather_desc(hfk, **over):
    d = hfk.PagedGatherDesc()
    buf = torch.zeros(64, dtype=torch.int64)
    d.k_layer_ptrs = d.v_layer_ptrs = d.block_tables = d.seq_lens = buf.data_ptr()
    d.k_out, d.v_out = 0x20000, 0x30000
    d.ids_are_int64, d.layers, d.num_seqs = 1, 2, 2
    d.max_blocks_per_seq = d.block_table_stride = 4
    d.block_size, d.token_bytes = 16, 256
    d.device_block_stride = 4096
    d.out_layer_stride = 256 * 100
    d.num_device_blocks, d.total_tokens = 8, 100
    for k, v in over.items():
        setattr(d, k, v)
    return d, buf


@pytest.mark.parametrize("over,code", [
    (dict(k_out=0), "HFK_ERR_INVALID_ARG"), (dict(token_bytes=250), "HFK_ERR_ALIGNMENT"),
    (dict(num_seqs=2**30, max_blocks_per_seq=1, block_table_stride=1), "HFK_ERR_TOO_LARGE"), (dict(block_table_stride=2), "HFK_ERR_INVALID_ARG"),
    (dict(device_block_stride=2048), "HFK_ERR_INVALID_ARG"), (dict(v_out=0x30004), "HFK_ERR_ALIGNMENT"),
    (dict(out_layer_stride=256), "HFK_ERR_INVALID_ARG"), (dict(block_size=0), "HFK_ERR_INVALID_ARG")])
def test_paged_gather_validation_errors(hfk, over, code):
    d, _keep = _gather_desc(hfk, **over)
    assert hfk.lib().hfk_paged_gather(C.byref(d), hfk.MOVER_AUTO, 0, None) == getattr(hfk, code)


def test_group_r_validation_errors(hfk):
    lib = hfk.lib()
    assert lib.hfk_gather(None, 0x1000, 0x2000, 1, 4, 64, 0, 0, None) == hfk.HFK_ERR_INVALID_ARG
    assert lib.hfk_gather(0x1000, 0x2000, 0x3000, 1, 4, 0, 0, 0, None) == hfk.HFK_ERR_INVALID_ARG
    assert lib.hfk_gather(0x1000, 0x2000, None, 1, 0, 64, 0, 0, None) == hfk.HFK_OK  # nothing to do
    # head_dim*elt not a multiple of 16 bytes; the reference wants 32-byte multiples
    # (pcieThrough/csrc/host/tiling/multi_layer_block_transfer.cpp:49-54)
    assert lib.hfk_multi_layer_block_transfer(0x1000, 0x2000, 16, 2, 1, 24, 1, 0, None) == hfk.HFK_ERR_ALIGNMENT
    assert lib.hfk_multi_layer_block_transfer(None, 0x2000, 16, 2, 1, 32, 1, 0, None) == hfk.HFK_ERR_INVALID_ARG
    assert lib.hfk_multi_layer_block_transfer(0x1000, 0x2000, 0, 2, 1, 32, 1, 0, None) == hfk.HFK_ERR_INVALID_ARG
    assert lib.hfk_fused_memcpy_multi_layer_block_transfer(0x1000, 0x2000, None, 16, 2, 1, 32, 1, 0, None) \
        == hfk.HFK_ERR_INVALID_ARG
    assert lib.hfk_set_bulk_geometry(100, 4) == hfk.HFK_ERR_INVALID_ARG
    assert lib.hfk_set_bulk_geometry(65536, 8) == hfk.HFK_ERR_TOO_LARGE
    assert lib.hfk_set_bulk_geometry(0, 0) == hfk.HFK_OK


# ---- registry (managed_mem.cpp semantics) under the test driver ----------------
@pytest.fixture()
def registry(hfk):
    lib = hfk.lib()
    lib.hfk_unregister_all()
    lib.hfk_registry_set_test_driver(1)
    yield lib
    lib.hfk_unregister_all()
    lib.hfk_registry_set_test_driver(0)


def test_registry_range_lookup_duplicates_and_removal(registry):
    lib = registry
    a = torch.zeros(4096, dtype=torch.uint8)
    b = torch.zeros(8192, dtype=torch.uint8)
    pa, pb = a.data_ptr(), b.data_ptr()
    alias_a = lib.hfk_register_ptr(pa, a.numel())
    assert alias_a and lib.hfk_registry_count() == 1
    assert lib.hfk_register_ptr(pa, a.numel()) == alias_a and lib.hfk_registry_count() == 1  # same base twice
    lib.hfk_register_ptr(pb, b.numel())
    assert lib.hfk_registry_count() == 2
    # interior pointers translate by offset; one-past-the-end does not
    assert lib.hfk_get_device_ptr(pa + 100) == alias_a + 100
    assert lib.hfk_get_device_ptr(pb + 8191) != 0
    assert lib.hfk_get_device_ptr(pb + 8192) in (0, lib.hfk_get_device_ptr(pb + 8192))  # may fall in a's range
    assert lib.hfk_get_record_size(pb + 5) == 8192
    assert lib.hfk_get_device_ptr(0) == 0 and lib.hfk_get_record_size(None) == 0
    assert lib.hfk_unregister_ptr(pa) == 0 and lib.hfk_registry_count() == 1
    assert lib.hfk_get_device_ptr(pa + 100) == 0 or pb <= pa + 100 < pb + 8192
    assert lib.hfk_unregister_ptr(pa) == 0          # unknown pointer: not an error (managed_mem.cpp:110-113)
    assert lib.hfk_register_ptr(None, 16) is None   # null / zero size are rejected (managed_mem.cpp:46)
    assert lib.hfk_register_ptr(pa, 0) is None
    lib.hfk_unregister_all()
    assert lib.hfk_registry_count() == 0


def test_numa_pinned_allocation_is_zeroed_registered_and_freed(registry, hfk):
    lib = registry
    n = 3 << 20
    p = lib.hfk_alloc_pinned_numa_ptr(n, -1)
    assert p, hfk.last_error()
    buf = (C.c_uint8 * n).from_address(p)
    t = torch.frombuffer(buf, dtype=torch.uint8)
    assert int(t.sum()) == 0
    assert lib.hfk_get_record_size(p + n - 1) == n and lib.hfk_get_device_ptr(p + 7) == p + 7
    del t, buf
    assert lib.hfk_free_pinned_numa_ptr(p) == 0
    assert lib.hfk_get_device_ptr(p) == 0
    assert lib.hfk_free_pinned_numa_ptr(p) == hfk.HFK_ERR_INVALID_ARG  # not ours any more
    assert lib.hfk_alloc_pinned_numa_ptr(0, -1) is None


def test_numa_bind_to_node_zero_or_clean_failure(registry, hfk):
    p = registry.hfk_alloc_pinned_numa_ptr(1 << 20, 0)
    if p:
        assert registry.hfk_free_pinned_numa_ptr(p) == 0
    else:
        assert "mbind" in hfk.last_error()
    assert registry.hfk_alloc_pinned_numa_ptr(1 << 20, 900) is None  # no such node: mbind refuses


def test_memory_module_surface(registry):
    """heterofusedkernels.memory keeps the reference's three names (common/csrc/pybind.cpp:7-11)."""
    from heterofusedkernels_b200 import build

    build.build_all()
    from heterofusedkernels import memory

    t = torch.empty(1000, 16, dtype=torch.float16)
    alias = memory.host_register(t)
    assert alias == t.data_ptr()  # test driver: identity alias
    assert memory.get_device_ptr(t.data_ptr() + 32) == alias + 32
    assert memory.get_device_ptr(12345) == 0
    memory.host_unregister(t)
    assert memory.get_device_ptr(t.data_ptr()) == 0


def test_torch_ops_are_registered_with_reference_schemas():
    from heterofusedkernels_b200 import build

    build.build_all()
    import pcie_through  # noqa: F401  (loads the operator library, like the reference)

    schema = str(torch.ops.pcie_through.gather.default._schema)
    assert schema == "pcie_through::gather(Tensor gmEmbed, Tensor gmEmbedDst, Tensor gmIds, int? aiv=None) -> ()"
    schema = str(torch.ops.pcie_through.multi_layer_block_transfer.default._schema)
    assert schema == ("pcie_through::multi_layer_block_transfer(Tensor deviceBlockCachePtrs, "
                      "Tensor hostBlockCache, int? aiv=None) -> ()")
    schema = str(torch.ops.pcie_through.fused_memcpy_multi_layer_block_transfer.default._schema)
    assert schema == ("pcie_through::fused_memcpy_multi_layer_block_transfer(Tensor deviceBlockCachePtrs, "
                      "Tensor hostBlockCache, Tensor stagingBlockCache, int? aiv=None) -> ()")
    for name in ("swap_out", "swap_in", "paged_gather", "swap_out_copy_engine", "swap_in_copy_engine"):
        assert hasattr(torch.ops.pcie_through, name)
    # no CPU implementation of any kernel: an all-CPU call is refused by the dispatcher
    with pytest.raises(NotImplementedError):
        torch.ops.pcie_through.gather(torch.zeros(4, 4), torch.zeros(2, 4), torch.zeros(2, dtype=torch.long))


def test_registry_is_safe_under_concurrent_registration_and_lookup(registry):
    """Lookups take the shared lock, mutations the exclusive one (managed_mem.cpp:31,47,143)."""
    import threading

    lib = registry
    bufs = [torch.zeros(4096, dtype=torch.uint8) for _ in range(64)]
    errors = []

    def writer(lo, hi):
        for _ in range(20):
            for b in bufs[lo:hi]:
                if not lib.hfk_register_ptr(b.data_ptr(), b.numel()):
                    errors.append("register failed")
            for b in bufs[lo:hi]:
                lib.hfk_unregister_ptr(b.data_ptr())

    def reader():
        for _ in range(2000):
            for b in bufs[::7]:
                alias = lib.hfk_get_device_ptr(b.data_ptr() + 5)
                if alias not in (0, b.data_ptr() + 5):
                    errors.append("wrong alias")

    threads = [threading.Thread(target=writer, args=(i * 16, (i + 1) * 16)) for i in range(4)]
    threads += [threading.Thread(target=reader) for _ in range(3)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert errors == [] and lib.hfk_registry_count() == 0


def test_accepted_host_strides_never_let_two_chunks_share_a_byte(hfk):
    """Property: whenever the swap validation accepts a (slot, layer, K|V) stride triple, a brute-force
    walk over every chunk finds no two chunks that overlap.  (The check is a sufficient condition — nested
    strides — so some exotic non-overlapping layouts are refused; none that overlaps is accepted.)"""
    import itertools
    import random

    rng = random.Random(11)
    accepted = refused_but_fine = 0
    for _ in range(600):
        bb = rng.choice([16, 32, 48, 64])
        layers, slots = rng.randint(1, 3), rng.randint(1, 4)
        strides = [rng.choice([0, 16, 32, 48, 64, 96, 128, 192, 256, 384, 512, 768, 1024]) for _ in range(3)]
        # n_blocks = 0: the call validates everything and returns before it would launch anything
        d, _keep = _swap_desc(hfk, block_bytes=bb, device_block_stride=bb, layers=layers, num_host_slots=slots,
                              host_slot_stride=strides[0], host_layer_stride=strides[1], host_kv_stride=strides[2],
                              n_blocks=0)
        rc = hfk.lib().hfk_swap_out(C.byref(d), hfk.MOVER_AUTO, 0, None)
        starts = [s * strides[0] + l * strides[1] + kv * strides[2]
                  for s, l, kv in itertools.product(range(slots), range(layers), range(2))]
        overlap = any(abs(a - b) < bb for a, b in itertools.combinations(starts, 2))
        if rc == hfk.HFK_ERR_INVALID_ARG:
            refused_but_fine += not overlap
            continue
        assert rc == hfk.HFK_OK, rc
        assert not overlap, (bb, layers, slots, strides)
        accepted += 1
    assert accepted > 20        # the generator does produce valid layouts
