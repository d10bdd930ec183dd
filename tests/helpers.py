"""Helpers shared by the GPU parity tests: descriptors for the C ABI built from torch tensors."""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence

import torch

from heterofusedkernels_b200 import capi


def u8(t: torch.Tensor) -> torch.Tensor:
    """Flat byte view of the logical contents."""
    return t.contiguous().view(torch.uint8).reshape(-1)


def dev_zeros(shape, dtype: torch.dtype, device) -> torch.Tensor:
    """Zero-filled device tensor of any dtype (built from bytes, so fp8 works too)."""
    n = torch.empty((), dtype=dtype).element_size()
    for d in shape:
        n *= d
    return torch.zeros(n, dtype=torch.uint8, device=device).view(dtype).view(*shape)


def ptr_table(tensors: Sequence[torch.Tensor], device) -> torch.Tensor:
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64).to(device)


def stream_handle() -> int:
    return torch.cuda.current_stream().cuda_stream


def swap_desc(k_ptrs: torch.Tensor, v_ptrs: torch.Tensor, host_pool: torch.Tensor, host_alias: int,
              dev_ids: torch.Tensor, slot_ids: torch.Tensor, num_device_blocks: int,
              device_block_stride: int | None = None) -> capi.SwapDesc:
    """host_pool: CPU tensor [slots, layers, 2, ...chunk]; host_alias: device alias of its data_ptr."""
    elt = host_pool.element_size()
    chunk = 1
    for d in host_pool.shape[3:]:
        chunk *= d
    d = capi.SwapDesc()
    d.k_layer_ptrs = k_ptrs.data_ptr()
    d.v_layer_ptrs = v_ptrs.data_ptr()
    d.host_pool = host_alias
    d.device_block_ids = dev_ids.data_ptr()
    d.host_slot_ids = slot_ids.data_ptr()
    d.ids_are_int64 = 1 if dev_ids.dtype == torch.int64 else 0
    d.layers = host_pool.shape[1]
    d.n_blocks = dev_ids.numel()
    d.block_bytes = chunk * elt
    d.device_block_stride = device_block_stride or d.block_bytes
    d.host_slot_stride = host_pool.stride(0) * elt
    d.host_layer_stride = host_pool.stride(1) * elt
    d.host_kv_stride = host_pool.stride(2) * elt
    d.num_device_blocks = num_device_blocks
    d.num_host_slots = host_pool.shape[0]
    return d


def gather_desc(k_ptrs, v_ptrs, k_out, v_out, tables, lens, block_size, num_device_blocks) -> capi.PagedGatherDesc:
    d = capi.PagedGatherDesc()
    d.k_layer_ptrs = k_ptrs.data_ptr()
    d.v_layer_ptrs = v_ptrs.data_ptr()
    d.k_out = k_out.data_ptr()
    d.v_out = v_out.data_ptr()
    d.out_layer_stride = k_out.stride(0) * k_out.element_size()
    d.block_tables = tables.data_ptr()
    d.seq_lens = lens.data_ptr()
    d.ids_are_int64 = 1 if tables.dtype == torch.int64 else 0
    d.layers = k_out.shape[0]
    d.num_seqs = tables.shape[0]
    d.max_blocks_per_seq = tables.shape[1]
    d.block_table_stride = tables.stride(0)
    d.block_size = block_size
    d.token_bytes = k_out.stride(1) * k_out.element_size()
    d.device_block_stride = block_size * d.token_bytes
    d.num_device_blocks = num_device_blocks
    d.total_tokens = k_out.shape[1]
    return d


class PinnedPool:
    """A registered host pool allocated through the C ABI (hfk_alloc_pinned_numa_ptr)."""

    def __init__(self, shape: Sequence[int], dtype: torch.dtype):
        lib = capi.lib()
        self.nbytes = int(torch.empty((), dtype=dtype).element_size())
        for s in shape:
            self.nbytes *= s
        node = lib.hfk_device_numa_node(-1)
        self.ptr = lib.hfk_alloc_pinned_numa_ptr(self.nbytes, node if node >= -1 else -1)
        if not self.ptr:
            raise RuntimeError("pinned allocation failed: " + capi.last_error())
        buf = (C.c_uint8 * self.nbytes).from_address(self.ptr)
        self.tensor = torch.frombuffer(buf, dtype=torch.uint8).view(dtype).view(*shape)
        self.alias = lib.hfk_get_device_ptr(self.ptr)

    def close(self):
        if self.ptr:
            self.tensor = None
            capi.check(capi.lib().hfk_free_pinned_numa_ptr(self.ptr), "free")
            self.ptr = 0


def relayout_desc(layer_ptrs, host_pool: torch.Tensor, host_alias: int, dev_ids, slot_ids, num_device_blocks,
                  device_block_stride=None) -> capi.RelayoutDesc:
    """host_pool: CPU tensor [slots, B, L, H, D]."""
    elt = host_pool.element_size()
    _, B, L, H, D = host_pool.shape
    d = capi.RelayoutDesc()
    d.layer_ptrs = layer_ptrs.data_ptr()
    d.host_pool = host_alias
    d.device_block_ids = dev_ids.data_ptr()
    d.host_slot_ids = slot_ids.data_ptr()
    d.ids_are_int64 = 1 if dev_ids.dtype == torch.int64 else 0
    d.layers = L
    d.n_blocks = dev_ids.numel()
    d.block_size, d.heads, d.head_bytes = B, H, D * elt
    d.device_block_stride = device_block_stride or H * B * D * elt
    d.host_slot_stride = host_pool.stride(0) * elt
    d.num_device_blocks = num_device_blocks
    d.num_host_slots = host_pool.shape[0]
    return d
