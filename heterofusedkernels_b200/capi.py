"""ctypes view of the C ABI declared in ``include/hfk_b200.h``.

This is the same boundary a non-Python host (cgo, JNI, a C++ serving engine) would
bind; the parity tests call the kernels through it.  Loading fails loudly when
``libhfk_b200.so`` has not been built: there is no fallback implementation.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_DIR = Path(__file__).resolve().parent / "lib"
LIB_PATH = LIB_DIR / "libhfk_b200.so"

# status codes / enums of hfk_b200.h
HFK_OK = 0
HFK_ERR_INVALID_ARG = -1
HFK_ERR_ALIGNMENT = -2
HFK_ERR_NOT_REGISTERED = -3
HFK_ERR_CUDA = -4
HFK_ERR_TOO_LARGE = -5
HFK_ERR_NO_MEMORY = -6
HFK_ERR_UNSUPPORTED = -7

HFK_DEV_BAD_DEVICE_BLOCK_ID = 0x1
HFK_DEV_BAD_HOST_SLOT_ID = 0x2
HFK_DEV_BAD_ROW_ID = 0x4
HFK_DEV_BAD_SEQ_LEN = 0x8
HFK_DEV_WAIT_TIMEOUT = 0x10
HFK_DEV_BAD_LAYER_PTR = 0x20

MOVER_AUTO, MOVER_VECTOR, MOVER_BULK = 0, 1, 2
HFK_MAX_SEQS = 1024
HFK_STATIC_STAGING_BYTES = 8 * 1024 * 1024


class SwapDesc(C.Structure):
    """struct hfk_swap_desc"""
    _fields_ = [
        ("k_layer_ptrs", C.c_void_p),
        ("v_layer_ptrs", C.c_void_p),
        ("host_pool", C.c_void_p),
        ("device_block_ids", C.c_void_p),
        ("host_slot_ids", C.c_void_p),
        ("ids_are_int64", C.c_int),
        ("layers", C.c_int),
        ("n_blocks", C.c_int64),
        ("block_bytes", C.c_int64),
        ("device_block_stride", C.c_int64),
        ("host_slot_stride", C.c_int64),
        ("host_layer_stride", C.c_int64),
        ("host_kv_stride", C.c_int64),
        ("num_device_blocks", C.c_int64),
        ("num_host_slots", C.c_int64),
    ]


class RelayoutDesc(C.Structure):
    """struct hfk_relayout_desc"""
    _fields_ = [
        ("layer_ptrs", C.c_void_p),
        ("host_pool", C.c_void_p),
        ("device_block_ids", C.c_void_p),
        ("host_slot_ids", C.c_void_p),
        ("ids_are_int64", C.c_int),
        ("layers", C.c_int),
        ("n_blocks", C.c_int64),
        ("block_size", C.c_int64),
        ("heads", C.c_int64),
        ("head_bytes", C.c_int64),
        ("device_block_stride", C.c_int64),
        ("host_slot_stride", C.c_int64),
        ("num_device_blocks", C.c_int64),
        ("num_host_slots", C.c_int64),
    ]


class MigrateDesc(C.Structure):
    """struct hfk_migrate_desc"""
    _fields_ = [
        ("src_k_layer_ptrs", C.c_void_p),
        ("src_v_layer_ptrs", C.c_void_p),
        ("dst_k_layer_ptrs", C.c_void_p),
        ("dst_v_layer_ptrs", C.c_void_p),
        ("src_block_ids", C.c_void_p),
        ("dst_block_ids", C.c_void_p),
        ("ids_are_int64", C.c_int),
        ("layers", C.c_int),
        ("n_blocks", C.c_int64),
        ("block_bytes", C.c_int64),
        ("src_block_stride", C.c_int64),
        ("dst_block_stride", C.c_int64),
        ("num_src_blocks", C.c_int64),
        ("num_dst_blocks", C.c_int64),
    ]


class PagedGatherDesc(C.Structure):
    """struct hfk_paged_gather_desc"""
    _fields_ = [
        ("k_layer_ptrs", C.c_void_p),
        ("v_layer_ptrs", C.c_void_p),
        ("k_out", C.c_void_p),
        ("v_out", C.c_void_p),
        ("out_layer_stride", C.c_int64),
        ("block_tables", C.c_void_p),
        ("seq_lens", C.c_void_p),
        ("ids_are_int64", C.c_int),
        ("layers", C.c_int),
        ("num_seqs", C.c_int64),
        ("max_blocks_per_seq", C.c_int64),
        ("block_table_stride", C.c_int64),
        ("block_size", C.c_int64),
        ("token_bytes", C.c_int64),
        ("device_block_stride", C.c_int64),
        ("num_device_blocks", C.c_int64),
        ("total_tokens", C.c_int64),
    ]


# name -> (restype, argtypes); every symbol include/hfk_b200.h declares
PROTOTYPES = {
    "hfk_strerror": (C.c_char_p, [C.c_int]),
    "hfk_last_error_message": (C.c_char_p, []),
    "hfk_version": (C.c_char_p, []),
    "hfk_device_status": (C.c_int, [C.POINTER(C.c_uint), C.c_void_p]),
    "hfk_selftest_wait_timeout": (C.c_int, [C.c_uint, C.c_void_p]),
    "hfk_set_bulk_geometry": (C.c_int, [C.c_int, C.c_int]),
    "hfk_set_bulk_lag": (C.c_int, [C.c_int]),
    "hfk_set_vector_geometry": (C.c_int, [C.c_int, C.c_int]),
    "hfk_set_vector_smem_pad": (C.c_int, [C.c_int]),
    "hfk_set_swap_out_pace": (C.c_int, [C.c_int]),
    "hfk_set_gather_tuning": (C.c_int, [C.c_int, C.c_int]),
    "hfk_set_staged_copy_lanes": (C.c_int, [C.c_int]),
    "hfk_debug_set_stamps": (C.c_int, [C.c_void_p, C.c_size_t]),
    "hfk_debug_stamp_marker": (C.c_int, [C.c_void_p]),
    "hfk_migrate_blocks": (C.c_int, [C.POINTER(MigrateDesc), C.c_int, C.c_void_p]),
    "hfk_migrate_blocks_copy_engine": (C.c_int, [C.POINTER(MigrateDesc), C.c_int, C.c_int, C.c_void_p]),
    "hfk_enable_peer_access": (C.c_int, [C.c_int]),
    "hfk_register_ptr": (C.c_void_p, [C.c_void_p, C.c_size_t]),
    "hfk_unregister_ptr": (C.c_int, [C.c_void_p]),
    "hfk_get_device_ptr": (C.c_size_t, [C.c_size_t]),
    "hfk_get_record_size": (C.c_size_t, [C.c_void_p]),
    "hfk_registry_count": (C.c_int, []),
    "hfk_unregister_all": (None, []),
    "hfk_registry_set_test_driver": (None, [C.c_int]),
    "hfk_device_numa_node": (C.c_int, [C.c_int]),
    "hfk_device_pci_bus_id": (C.c_int, [C.c_int, C.c_char_p, C.c_size_t]),
    "hfk_alloc_pinned_numa_ptr": (C.c_void_p, [C.c_size_t, C.c_int]),
    "hfk_free_pinned_numa_ptr": (C.c_int, [C.c_void_p]),
    "hfk_gather": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_size_t, C.c_size_t,
                             C.c_size_t, C.c_int, C.c_void_p]),
    "hfk_multi_layer_block_transfer": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                                 C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "hfk_fused_memcpy_multi_layer_block_transfer": (
        C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                  C.c_int64, C.c_int, C.c_void_p]),
    "hfk_fused_memcpy_multi_layer_block_transfer_static": (
        C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int,
                  C.c_void_p]),
    "hfk_swap_out": (C.c_int, [C.POINTER(SwapDesc), C.c_int, C.c_int, C.c_void_p]),
    "hfk_swap_out_paced": (C.c_int, [C.POINTER(SwapDesc), C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "hfk_swap_in": (C.c_int, [C.POINTER(SwapDesc), C.c_int, C.c_int, C.c_void_p]),
    "hfk_swap_copy_engine": (C.c_int, [C.POINTER(SwapDesc), C.c_int, C.c_void_p]),
    "hfk_swap_staged": (C.c_int, [C.POINTER(SwapDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int,
                                  C.c_int, C.c_void_p]),
    "hfk_swap_relayout": (C.c_int, [C.POINTER(RelayoutDesc), C.c_int, C.c_int, C.c_void_p]),
    "hfk_paged_gather": (C.c_int, [C.POINTER(PagedGatherDesc), C.c_int, C.c_int, C.c_void_p]),
}

_lib = None


class HfkError(RuntimeError):
    def __init__(self, code: int, op: str, detail: str):
        super().__init__(f"{op}: error {code} ({detail})")
        self.code = code


def lib() -> C.CDLL:
    """The loaded C-ABI library; raises when it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: run `python -m heterofusedkernels_b200.build` "
                "(the CUDA library is required; there is no fallback path)")
        handle = C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def last_error() -> str:
    return lib().hfk_last_error_message().decode()


def check(rc: int, op: str) -> None:
    if rc != HFK_OK:
        raise HfkError(rc, op, f"{lib().hfk_strerror(rc).decode()}: {last_error()}")


def device_status(stream: int = 0) -> int:
    bits = C.c_uint(0)
    check(lib().hfk_device_status(C.byref(bits), stream), "hfk_device_status")
    return bits.value
