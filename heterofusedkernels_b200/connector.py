"""Caller-side shim: how a KV-offload connector of a serving engine drives the ops.

The reference has no serving engine; its test sketches the caller: build the
per-layer pointer table once on the CPU and move it to the device
(pcieThrough/tests/test_transfer_kernel.py:42-47), allocate the host pool with
``memory.alloc_numa_pinned_tensor`` (:28-34) and alternate streams per transfer
(:50-72).  ``PagedKVCache`` holds exactly that state for a vLLM-style cache —
per layer one K and one V tensor ``[num_blocks, block_size, kv_heads, head_dim]``
— plus a free list of host slots, and forwards to ``torch.ops.pcie_through.*``.
"""
from __future__ import annotations

import bisect
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

import heterofusedkernels_b200 as _pkg


class HostSlotPool:
    """Free list of host slots that hands out *runs* of consecutive slots when it can.

    A swapped-out block occupies one slot of the pinned pool until it is swapped in again
    (the reference test's pool is such an array of block slots, test_transfer_kernel.py:28-34).
    Consecutive slots are contiguous in host memory, so a request served by one run lets the
    staged mover cross the link with a few large copy-engine transfers instead of one per slot.

    ``alloc(n)`` takes the smallest free run that holds n slots; when no run is long enough it
    takes the longest runs first.  ``free(slots)`` returns slots and merges neighbouring runs.
    """

    def __init__(self, num_slots: int):
        self.num_slots = int(num_slots)
        self._starts: List[int] = [0] if num_slots > 0 else []   # sorted starts of the free runs
        self._len: Dict[int, int] = {0: self.num_slots} if num_slots > 0 else {}
        self.free_count = self.num_slots

    def largest_run(self) -> int:
        return max(self._len.values(), default=0)

    def runs(self) -> List[Tuple[int, int]]:
        """Free runs as (first slot, length), in slot order."""
        return [(s, self._len[s]) for s in self._starts]

    def _take(self, start: int, n: int) -> range:
        length = self._len.pop(start)
        i = bisect.bisect_left(self._starts, start)
        del self._starts[i]
        if length > n:
            self._starts.insert(i, start + n)
            self._len[start + n] = length - n
        self.free_count -= n
        return range(start, start + n)

    def alloc(self, n: int) -> torch.Tensor:
        """n distinct free slots as an int64 CPU tensor; raises when fewer than n are free."""
        if n < 0 or n > self.free_count:
            raise RuntimeError(f"host pool exhausted: {n} slots wanted, {self.free_count} free")
        if n == 0:
            return torch.empty(0, dtype=torch.int64)
        fits = [s for s in self._starts if self._len[s] >= n]
        if fits:
            best = min(fits, key=lambda s: (self._len[s], s))
            return torch.tensor(list(self._take(best, n)), dtype=torch.int64)
        out: List[int] = []
        for start in sorted(self._starts, key=lambda s: (-self._len[s], s)):
            take = min(self._len[start], n - len(out))
            out.extend(self._take(start, take))
            if len(out) == n:
                break
        return torch.tensor(out, dtype=torch.int64)

    def free(self, slots) -> None:
        ids = sorted(int(x) for x in (slots.tolist() if torch.is_tensor(slots) else slots))
        i = 0
        while i < len(ids):
            j = i
            while j + 1 < len(ids) and ids[j + 1] == ids[j] + 1:
                j += 1
            self._insert_run(ids[i], j - i + 1)
            i = j + 1

    def _insert_run(self, start: int, n: int) -> None:
        if start < 0 or start + n > self.num_slots:
            raise ValueError(f"slots {start}..{start + n - 1} are outside the pool")
        i = bisect.bisect_left(self._starts, start)
        prev = self._starts[i - 1] if i > 0 else None
        nxt = self._starts[i] if i < len(self._starts) else None
        if (prev is not None and prev + self._len[prev] > start) or (nxt is not None and start + n > nxt):
            raise ValueError(f"slots {start}..{start + n - 1} are already free")
        self.free_count += n
        if prev is not None and prev + self._len[prev] == start:      # merge with the run before
            start, n = prev, n + self._len.pop(prev)
            i -= 1
            del self._starts[i]
        if nxt is not None and start + n == nxt:                        # and with the run after
            n += self._len.pop(nxt)
            del self._starts[i]
        self._starts.insert(i, start)
        self._len[start] = n


MoverArg = Union[None, int, str]


class PagedKVCache:
    """Device caches + pointer tables + (optionally) a pinned, device-mapped host pool.

    Host pool layout (``pool_layout``), always seen through ``host_pool`` as
    ``[host_slots, layers, 2, block_size, kv_heads, head_dim]``:

    * ``"slot_major"`` (default): stored in that order — one slot holds every layer's K and V of a
      block contiguously, like the reference's host block that holds all layers
      (test_transfer_kernel.py:28).  Best for swaps that move all layers of a block at once.
    * ``"layer_major"``: stored ``[layers, host_slots, 2, ...]`` — a run of consecutive slots of ONE
      layer is contiguous, so a layer-wise pipeline can move a layer's blocks with one copy-engine
      transfer.  The kernels take the strides from the view, so every op works on either layout.

    ``swap_out`` / ``swap_in`` take ``mover`` = one of ``capi.MOVER_*`` (a kernel crosses the
    link) or ``"staged"`` (a packing kernel plus copy-engine transfers; needs the slot ids on
    the host, which is where a scheduler has them) or ``"hybrid[:fraction]"`` (that fraction of
    the blocks staged and the rest by the kernel, both at the same time).  ``mover=None`` decides
    per call, from what the copy engine and a kernel do on PCIe (256-byte against 128-byte
    transactions; Llama-3-8B step, 2 MiB slots): slot ids on the host in runs of
    ``STAGED_MIN_RUN`` or more consecutive slots on average (what the free list hands out) →
    staged, 55.2 GB/s against the kernels' 52.0; slot ids on the host, scattered, and at least
    ``HYBRID_MIN_BYTES`` to move → hybrid, 53.5 GB/s (the kernel's traffic fills the gaps between
    the copy engine's 2 MiB copies, which alone reach 49.7); anything else → the kernels.
    """
    STAGED_MIN_RUN = 4
    HYBRID_FRACTION = 0.4            # share of a "hybrid" swap that goes through the copy engine
    HYBRID_MIN_BYTES = 128 << 20
    # Pace of a swap-out that runs at the same time as a swap-in on the same link (1.07 GB each way on
    # Gen5 x16: unpaced 42.9 GB/s out with 34.5 in; paced to 40: 40.0 out with 42.0 in).
    BIDIR_OUT_PACE_GBS = 40.0

    def __init__(self, layers: int, num_blocks: int, block_size: int, kv_heads: int, head_dim: int,
                 dtype: torch.dtype, device: torch.device | str = "cuda", host_slots: int = 0,
                 k_caches: Optional[Sequence[torch.Tensor]] = None,
                 v_caches: Optional[Sequence[torch.Tensor]] = None,
                 host_raw: Optional[torch.Tensor] = None, pool_layout: str = "slot_major"):
        _pkg.load_ops()
        assert pool_layout in ("slot_major", "layer_major")
        self.pool_layout = pool_layout
        self.layers, self.num_blocks, self.block_size = layers, num_blocks, block_size
        self.kv_heads, self.head_dim, self.dtype = kv_heads, head_dim, dtype
        self.device = torch.device(device)
        shape = (num_blocks, block_size, kv_heads, head_dim)
        if k_caches is None:
            # one allocation per side keeps the layers adjacent; each layer is its own view
            self._k_store = torch.empty((layers,) + shape, dtype=dtype, device=self.device)
            self._v_store = torch.empty((layers,) + shape, dtype=dtype, device=self.device)
            k_caches, v_caches = list(self._k_store.unbind(0)), list(self._v_store.unbind(0))
        self.k_caches: List[torch.Tensor] = list(k_caches)
        self.v_caches: List[torch.Tensor] = list(v_caches)
        assert len(self.k_caches) == layers and len(self.v_caches) == layers
        for t in self.k_caches + self.v_caches:
            assert t.is_cuda and t.is_contiguous() and tuple(t.shape) == shape and t.dtype == dtype
        # pointer tables: built on the CPU, moved once (test_transfer_kernel.py:42-47)
        self.k_ptrs_cpu = torch.tensor([t.data_ptr() for t in self.k_caches], dtype=torch.int64)
        self.v_ptrs_cpu = torch.tensor([t.data_ptr() for t in self.v_caches], dtype=torch.int64)
        self.k_ptrs = self.k_ptrs_cpu.to(self.device)
        self.v_ptrs = self.v_ptrs_cpu.to(self.device)
        self.elt = self.k_caches[0].element_size()
        self.token_bytes = kv_heads * head_dim * self.elt
        self.block_bytes = block_size * self.token_bytes
        self.slot_bytes = layers * 2 * self.block_bytes
        self.host_slots = 0
        self.host_pool: Optional[torch.Tensor] = None
        self._host_raw: Optional[torch.Tensor] = None
        self.slot_pool: Optional[HostSlotPool] = None
        self._staging_bufs: Dict[str, torch.Tensor] = {}      # one staging buffer per direction
        self._hybrid_streams: Dict[str, Tuple[torch.cuda.Stream, torch.cuda.Stream]] = {}
        if host_raw is not None:
            self.attach_host_raw(host_raw, host_slots)
        elif host_slots > 0:
            self.attach_host_pool(host_slots)

    # -- host pool -------------------------------------------------------------
    def attach_host_pool(self, host_slots: int) -> torch.Tensor:
        with torch.cuda.device(self.device):
            raw = _pkg.memory.alloc_numa_pinned_tensor(host_slots * self.slot_bytes)
        return self.attach_host_raw(raw, host_slots)

    def attach_host_raw(self, raw: torch.Tensor, host_slots: int = 0) -> torch.Tensor:
        """Uses (a prefix of) an existing registered byte buffer — e.g. one obtained from
        ``memory.alloc_numa_pinned_tensor`` and shared by several caches in turn — as the pool."""
        fit = raw.numel() * raw.element_size() // self.slot_bytes
        host_slots = fit if host_slots <= 0 else host_slots
        assert 0 < host_slots <= fit, "the byte buffer is smaller than the pool asked for"
        self._host_raw = raw
        self.host_slots = host_slots
        flat = raw.view(torch.uint8)[:host_slots * self.slot_bytes].view(self.dtype)
        chunk = (2, self.block_size, self.kv_heads, self.head_dim)
        if self.pool_layout == "slot_major":
            self.host_pool = flat.view(host_slots, self.layers, *chunk)
        else:
            self.host_pool = flat.view(self.layers, host_slots, *chunk).transpose(0, 1)
        self.slot_pool = HostSlotPool(host_slots)
        return self.host_pool

    def swap_bytes(self, n_blocks: int) -> int:
        return n_blocks * self.layers * 2 * self.block_bytes

    # -- ops ---------------------------------------------------------------------
    def _ids(self, ids) -> torch.Tensor:
        if not torch.is_tensor(ids):
            ids = torch.tensor(list(ids), dtype=torch.int64)
        return ids.to(self.device, non_blocking=True)

    def _pick_mover(self, host_slot_ids) -> MoverArg:
        """The per-call choice of ``mover=None``: staged for host-resident slot lists made of runs."""
        if self.pool_layout != "slot_major":
            return None
        if torch.is_tensor(host_slot_ids):
            if host_slot_ids.device.type != "cpu" or host_slot_ids.numel() < self.STAGED_MIN_RUN:
                return None
            s = host_slot_ids
        else:
            if len(host_slot_ids) < self.STAGED_MIN_RUN:
                return None
            s = torch.tensor(list(host_slot_ids), dtype=torch.int64)
        runs = 1 + int((s[1:] - s[:-1] != 1).sum())
        if s.numel() >= self.STAGED_MIN_RUN * runs:
            return "staged"
        return "hybrid" if s.numel() * self.slot_bytes >= self.HYBRID_MIN_BYTES else None

    @staticmethod
    def _cpu_ids(ids) -> torch.Tensor:
        if not torch.is_tensor(ids):
            ids = torch.tensor(list(ids), dtype=torch.int64)
        return ids if ids.device.type == "cpu" else ids.cpu()

    def swap_out(self, device_block_ids, host_slot_ids=None, aiv: Optional[int] = None,
                 mover: MoverArg = None, pace_gbs: Optional[float] = None) -> torch.Tensor:
        """host_pool[slot] <- cache[block], every layer, K and V, one call, current stream.

        Without ``host_slot_ids`` the slots come from the free list (``self.slot_pool``), as runs of
        consecutive slots where possible; the slots used are returned (give them back with
        ``release`` once the blocks have been swapped in again or dropped).

        ``pace_gbs`` paces the stores of the (bulk) kernel to that many GB/s: for a swap-out that
        crosses the link at the same time as a swap-in (``BIDIR_OUT_PACE_GBS`` is the measured
        balance point); a paced swap-out always goes through the kernel."""
        n = len(device_block_ids)
        if host_slot_ids is None:
            host_slot_ids = self.slot_pool.alloc(n)
        if pace_gbs:
            torch.ops.pcie_through.swap_out(self.k_ptrs, self.v_ptrs, self.host_pool, self._ids(device_block_ids),
                                            self._ids(host_slot_ids), self.num_blocks, None, aiv,
                                            None if isinstance(mover, str) else mover, int(pace_gbs * 1000))
            return host_slot_ids
        if mover is None:
            mover = self._pick_mover(host_slot_ids)
        if mover == "staged":
            self.swap_out_staged(device_block_ids, self._cpu_ids(host_slot_ids), aiv=aiv)
        elif isinstance(mover, str) and mover.startswith("hybrid"):
            self._hybrid(True, device_block_ids, host_slot_ids, aiv,
                         float(mover.split(":")[1]) if ":" in mover else self.HYBRID_FRACTION)
        else:
            torch.ops.pcie_through.swap_out(self.k_ptrs, self.v_ptrs, self.host_pool, self._ids(device_block_ids),
                                            self._ids(host_slot_ids), self.num_blocks, None, aiv, mover)
        return host_slot_ids

    def swap_in(self, device_block_ids, host_slot_ids, aiv: Optional[int] = None,
                mover: MoverArg = None, release: bool = False) -> None:
        """cache[block] <- host_pool[slot], every layer, K and V, one call, current stream.
        ``release=True`` returns the slots to the free list (the copy is only enqueued: do not
        swap out into them again from another stream before it has run)."""
        if mover is None:
            mover = self._pick_mover(host_slot_ids)
        if mover == "staged":
            self.swap_in_staged(device_block_ids, self._cpu_ids(host_slot_ids), aiv=aiv)
        elif isinstance(mover, str) and mover.startswith("hybrid"):
            self._hybrid(False, device_block_ids, host_slot_ids, aiv,
                         float(mover.split(":")[1]) if ":" in mover else self.HYBRID_FRACTION)
        else:
            torch.ops.pcie_through.swap_in(self.k_ptrs, self.v_ptrs, self.host_pool, self._ids(device_block_ids),
                                           self._ids(host_slot_ids), self.num_blocks, None, aiv, mover)
        if release:
            self.release(host_slot_ids)

    def release(self, host_slot_ids) -> None:
        self.slot_pool.free(self._cpu_ids(host_slot_ids))

    def _staging(self, direction: str, staging_bytes: int) -> torch.Tensor:
        """The staging buffer of one direction ("out" / "in").  Swap-outs and swap-ins may run at the same
        time (each has its own buffer); two staged or hybrid swaps of the SAME direction share one and
        must be ordered by the caller (one stream, or events)."""
        want = max(self.slot_bytes, staging_bytes)
        buf = self._staging_bufs.get(direction)
        if buf is None or buf.numel() < want:
            buf = self._staging_bufs[direction] = torch.empty(want, dtype=torch.uint8, device=self.device)
        return buf

    def _hybrid(self, out: bool, device_block_ids, host_slot_ids, aiv: Optional[int], fraction: float) -> None:
        """One swap split between the two ways across the link, running at the same time: the first
        `fraction` of the blocks through the staged mover (copy engine) on one internal stream, the rest
        through the kernel on another; both fork from the current stream and join it again."""
        cur = torch.cuda.current_stream(self.device)
        direction = "out" if out else "in"
        if direction not in self._hybrid_streams:
            self._hybrid_streams[direction] = (torch.cuda.Stream(self.device), torch.cuda.Stream(self.device))
        s_copy, s_kernel = self._hybrid_streams[direction]
        slots_cpu = self._cpu_ids(host_slot_ids)
        dev_ids, slots_dev = self._ids(device_block_ids), self._ids(host_slot_ids)
        n = dev_ids.numel()
        k = max(0, min(n, int(round(n * fraction))))
        fork = torch.cuda.Event()
        fork.record(cur)
        if k > 0:
            s_copy.wait_event(fork)
            with torch.cuda.stream(s_copy):
                (self.swap_out_staged if out else self.swap_in_staged)(dev_ids[:k], slots_cpu[:k], aiv=aiv)
            cur.wait_stream(s_copy)
        if k < n:
            s_kernel.wait_event(fork)
            op = torch.ops.pcie_through.swap_out if out else torch.ops.pcie_through.swap_in
            with torch.cuda.stream(s_kernel):
                op(self.k_ptrs, self.v_ptrs, self.host_pool, dev_ids[k:], slots_dev[k:], self.num_blocks, None, aiv, None)
            cur.wait_stream(s_kernel)
        for t in (dev_ids, slots_dev):
            t.record_stream(s_copy)
            t.record_stream(s_kernel)

    def swap_out_staged(self, device_block_ids, host_slot_ids_cpu: torch.Tensor, staging_bytes: int = 256 << 20,
                        aiv: Optional[int] = None) -> None:
        """Swap-out through the copy engine: a packing kernel into a staging buffer, then one
        cudaMemcpyAsync per run of consecutive host slots (256-byte PCIe transactions instead of a
        kernel's 128-byte ones)."""
        torch.ops.pcie_through.swap_out_staged(self.k_ptrs, self.v_ptrs, self.host_pool, self._ids(device_block_ids),
                                               host_slot_ids_cpu, self._staging("out", staging_bytes), self.num_blocks,
                                               None, aiv)

    def swap_in_staged(self, device_block_ids, host_slot_ids_cpu: torch.Tensor, staging_bytes: int = 256 << 20,
                       aiv: Optional[int] = None) -> None:
        torch.ops.pcie_through.swap_in_staged(self.k_ptrs, self.v_ptrs, self.host_pool, self._ids(device_block_ids),
                                              host_slot_ids_cpu, self._staging("in", staging_bytes), self.num_blocks,
                                              None, aiv)

    def swap_out_copy_engine(self, device_block_ids: torch.Tensor, host_slot_ids: torch.Tensor) -> None:
        torch.ops.pcie_through.swap_out_copy_engine(self.k_ptrs_cpu, self.v_ptrs_cpu, self.host_pool,
                                                    device_block_ids.cpu(), host_slot_ids.cpu(), self.num_blocks)

    def swap_in_copy_engine(self, device_block_ids: torch.Tensor, host_slot_ids: torch.Tensor) -> None:
        torch.ops.pcie_through.swap_in_copy_engine(self.k_ptrs_cpu, self.v_ptrs_cpu, self.host_pool,
                                                   device_block_ids.cpu(), host_slot_ids.cpu(), self.num_blocks)

    def paged_gather(self, block_tables: torch.Tensor, seq_lens: torch.Tensor,
                     k_out: Optional[torch.Tensor] = None, v_out: Optional[torch.Tensor] = None,
                     total_tokens: Optional[int] = None, aiv: Optional[int] = None,
                     mover: Optional[int] = None):
        """Gathers every layer's pages of the batch into [layers, total_tokens, kv_heads, head_dim]."""
        if k_out is None:
            if total_tokens is None:
                total_tokens = int(seq_lens.sum().item())
            shape = (self.layers, total_tokens, self.kv_heads, self.head_dim)
            k_out = torch.empty(shape, dtype=self.dtype, device=self.device)
            v_out = torch.empty(shape, dtype=self.dtype, device=self.device)
        torch.ops.pcie_through.paged_gather(self.k_ptrs, self.v_ptrs, k_out, v_out,
                                            block_tables.to(self.device), seq_lens.to(self.device),
                                            self.block_size, self.num_blocks, None, aiv, mover)
        return k_out, v_out

    def migrate_to(self, other: "PagedKVCache", src_block_ids, dst_block_ids, aiv: Optional[int] = None,
                   run_on: str = "dst") -> None:
        """other.cache[dst_block] <- self.cache[src_block], every layer, K and V, one launch.

        ``other`` may be this cache (a copy between blocks), another cache on the same GPU, or a
        cache on a peer GPU; then one side of each copy crosses NVLink.  ``run_on`` picks the GPU that
        runs the kernel: "dst" pulls (peer loads), "src" pushes (peer stores).  The launch goes to the
        current stream of that GPU."""
        assert other.layers == self.layers and other.block_bytes == self.block_bytes
        dev = other.device if run_on == "dst" else self.device
        key = (id(other), dev)
        cached = getattr(self, "_migrate_tabs", None)
        if cached is None:
            cached = self._migrate_tabs = {}
        if key not in cached:   # first migration towards this cache from this GPU: peer access + pointer tables
            if dev != self.device or dev != other.device:
                with torch.cuda.device(dev):
                    peer = self.device if dev == other.device else other.device
                    _pkg.capi.check(_pkg.capi.lib().hfk_enable_peer_access(peer.index), "hfk_enable_peer_access")
            cached[key] = [t.to(dev) for t in (self.k_ptrs_cpu, self.v_ptrs_cpu, other.k_ptrs_cpu, other.v_ptrs_cpu)]
        tabs = cached[key]
        src = (src_block_ids if torch.is_tensor(src_block_ids) else torch.tensor(list(src_block_ids))).to(dev)
        dst = (dst_block_ids if torch.is_tensor(dst_block_ids) else torch.tensor(list(dst_block_ids))).to(dev)
        with torch.cuda.device(dev):
            torch.ops.pcie_through.migrate_blocks(tabs[0], tabs[1], tabs[2], tabs[3], src, dst, self.block_bytes,
                                                  self.num_blocks, other.num_blocks, None, None, aiv)

    def status(self) -> int:
        """Reads and clears the device status word (bits HFK_DEV_* of hfk_b200.h).  The word is per
        GPU, not per cache or stream: quiesce side streams first."""
        with torch.cuda.device(self.device):
            return int(torch.ops.pcie_through.device_status())


LayerArg = Union[int, Tuple[int, int], range]


class LayerwisePrefetcher:
    """Layer-wise prefetch pipeline: while layer l computes on the caller's stream,
    the blocks of the next layer(s) are swapped in on a side stream and other blocks are
    swapped out on a second one.

    Ordering.  A swap on a side stream starts only after the work the caller had already enqueued
    on its own stream (``after=None``: the side stream waits for the caller's current stream at the
    moment of the call; pass an event to wait for exactly that, or ``False`` to take over the ordering
    yourself).  So an ``evict`` issued right after the kernel that wrote the blocks reads finished
    blocks, and a ``prefetch`` cannot overwrite blocks an earlier kernel still reads.  In the other
    direction ``wait(layer)`` makes the caller's stream wait for that layer's swap-in, and
    ``wait_evicted(layer)`` for its swap-out (before the blocks are reused).  Id tensors are kept alive
    for the side stream (``record_stream``).

    Layers.  ``layer`` is one index or a range ``(first, last_exclusive)``: a range moves several
    layers in one launch through slices of the pointer tables and of the pool, which amortises the
    launch cost of these small (a few MB) transfers; the events of every layer of the range are
    recorded after the launch.

    Movers.  ``mover`` is one of ``capi.MOVER_*`` (a kernel crosses the link) or ``"staged"``: per
    layer a packing kernel plus copy-engine transfers through a staging buffer of the prefetcher
    (one per direction).  With a ``"layer_major"`` pool and slots that form runs (what
    ``HostSlotPool`` hands out) a layer's blocks cross the link in ONE transfer that occupies no SM,
    which is what a layer-wise pipeline next to compute wants; the slot ids must then also be given
    on the host (``host_slot_ids_cpu``).

    Defaults: the library's mover for small launches — the bulk mover with a 2 KiB x 4 ring and 64
    single-warp CTAs, whose CTAs fit next to a GEMM's on an SM — four layers per launch (pass a range;
    one layer per launch loses about 15 % to the launch itself), and TWO side streams with the
    swap-out's stores paced to ``EVICT_PACE_GBS``.  Measured next to a bf16 GEMM that fills the device
    (fp8 cache, 256 blocks per layer and direction, four layers per launch): 38.8 GB/s in and 38.9 out
    AT THE SAME TIME (76.8 together) with the GEMM 0.7 % slower.  Unpaced, the swap-out crowds the
    swap-in's read requests out of the upstream lanes: 28.6 in / 43.6 out (56.8 together).  One side
    stream (``one_stream=True``) runs the directions one after the other, each at the link's
    one-direction rate: 48.3 in, then 46.9 out (47.3 for the pair), GEMM 4 % slower.
    """
    DEFAULT_AIV = None      # library default of the mover
    DEFAULT_MOVER = None    # HFK_MOVER_AUTO
    RECOMMENDED_LAYERS_PER_LAUNCH = 4
    EVICT_PACE_GBS = PagedKVCache.BIDIR_OUT_PACE_GBS

    def __init__(self, cache: PagedKVCache, one_stream: bool = False, evict_pace_gbs: Optional[float] = None):
        """``one_stream=True`` issues swap-ins and swap-outs on ONE side stream, so the two directions never
        cross the link at the same time.  ``evict_pace_gbs``: pace of the swap-outs when there are two side
        streams (``None`` = ``EVICT_PACE_GBS``, 0 = unpaced); with one stream swap-outs are never paced."""
        self.evict_pace_gbs = 0.0 if one_stream else (self.EVICT_PACE_GBS if evict_pace_gbs is None else evict_pace_gbs)
        self.cache = cache
        self.in_stream = torch.cuda.Stream(device=cache.device, priority=-1)
        self.out_stream = self.in_stream if one_stream else torch.cuda.Stream(device=cache.device, priority=-1)
        self.ready = [torch.cuda.Event() for _ in range(cache.layers)]
        self.evicted = [torch.cuda.Event() for _ in range(cache.layers)]
        self._staging: Dict[str, torch.Tensor] = {}
        self._views: Dict[Tuple[int, int], Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}

    def _span(self, layer: LayerArg) -> Tuple[int, int]:
        if isinstance(layer, int):
            first, last = layer, layer + 1
        elif isinstance(layer, range):
            assert layer.step == 1
            first, last = layer.start, layer.stop
        else:
            first, last = layer
        assert 0 <= first < last <= self.cache.layers, f"layer range {first}:{last} outside the cache"
        return first, last

    def _view(self, first: int, last: int):
        """Pointer-table and pool slices of layers [first, last): a cache of last-first layers."""
        key = (first, last)
        if key not in self._views:
            c = self.cache
            self._views[key] = (c.k_ptrs[first:last], c.v_ptrs[first:last], c.host_pool[:, first:last])
        return self._views[key]

    def _order(self, side: torch.cuda.Stream, after) -> None:
        if after is None:
            side.wait_stream(torch.cuda.current_stream(self.cache.device))
        elif after is not False:
            side.wait_event(after)

    def _staging_for(self, direction: str, n_blocks: int) -> torch.Tensor:
        want = max(1, n_blocks) * 2 * self.cache.block_bytes      # one layer's K and V of every listed block
        buf = self._staging.get(direction)
        if buf is None or buf.numel() < want:
            buf = torch.empty(want, dtype=torch.uint8, device=self.cache.device)
            self._staging[direction] = buf
        return buf

    def _staged(self, op, direction: str, first: int, last: int, device_block_ids, host_slot_ids_cpu, aiv) -> None:
        assert host_slot_ids_cpu is not None and host_slot_ids_cpu.device.type == "cpu", \
            "the staged mover addresses its copies on the host: pass host_slot_ids_cpu"
        staging = self._staging_for(direction, device_block_ids.numel())
        for l in range(first, last):       # one layer per call: its slots are dense in a layer-major pool
            k_ptrs, v_ptrs, pool = self._view(l, l + 1)
            op(k_ptrs, v_ptrs, pool, device_block_ids, host_slot_ids_cpu, staging, self.cache.num_blocks, None, aiv)

    def prefetch(self, layer: LayerArg, device_block_ids: torch.Tensor, host_slot_ids: torch.Tensor,
                 aiv: Optional[int] = None, mover: MoverArg = None, after=None,
                 host_slot_ids_cpu: Optional[torch.Tensor] = None) -> torch.cuda.Event:
        """Swap-in of the listed blocks of ``layer`` (an index or a range) on the swap-in stream.
        Returns the event of the last layer of the range."""
        first, last = self._span(layer)
        k_ptrs, v_ptrs, pool = self._view(first, last)
        self._order(self.in_stream, after)
        with torch.cuda.stream(self.in_stream):
            if mover == "staged":
                self._staged(torch.ops.pcie_through.swap_in_staged, "in", first, last, device_block_ids,
                             host_slot_ids_cpu, aiv)
            else:
                torch.ops.pcie_through.swap_in(k_ptrs, v_ptrs, pool, device_block_ids, host_slot_ids,
                                               self.cache.num_blocks, None,
                                               self.DEFAULT_AIV if aiv is None else aiv,
                                               self.DEFAULT_MOVER if mover is None else mover)
            for l in range(first, last):
                self.ready[l].record()
        device_block_ids.record_stream(self.in_stream)
        host_slot_ids.record_stream(self.in_stream)
        return self.ready[last - 1]

    def evict(self, layer: LayerArg, device_block_ids: torch.Tensor, host_slot_ids: torch.Tensor,
              aiv: Optional[int] = None, mover: MoverArg = None, after=None,
              host_slot_ids_cpu: Optional[torch.Tensor] = None, pace_gbs: Optional[float] = None) -> torch.cuda.Event:
        """Swap-out of the listed blocks of ``layer`` (an index or a range) on the swap-out stream.
        Returns the event to wait for before the blocks are reused.  ``pace_gbs`` paces the kernel's
        stores (two side streams: keeps the swap-in of the other stream from starving)."""
        first, last = self._span(layer)
        k_ptrs, v_ptrs, pool = self._view(first, last)
        pace = self.evict_pace_gbs if pace_gbs is None else pace_gbs
        self._order(self.out_stream, after)
        with torch.cuda.stream(self.out_stream):
            if mover == "staged":
                self._staged(torch.ops.pcie_through.swap_out_staged, "out", first, last, device_block_ids,
                             host_slot_ids_cpu, aiv)
            else:
                torch.ops.pcie_through.swap_out(k_ptrs, v_ptrs, pool, device_block_ids, host_slot_ids,
                                                self.cache.num_blocks, None,
                                                self.DEFAULT_AIV if aiv is None else aiv,
                                                self.DEFAULT_MOVER if mover is None else mover,
                                                int(pace * 1000) if pace and mover != _pkg.capi.MOVER_VECTOR else None)
            for l in range(first, last):
                self.evicted[l].record()
        device_block_ids.record_stream(self.out_stream)
        host_slot_ids.record_stream(self.out_stream)
        return self.evicted[last - 1]

    def wait(self, layer: int) -> None:
        """The caller's stream waits until ``layer``'s swap-in has finished."""
        torch.cuda.current_stream(self.cache.device).wait_event(self.ready[layer])

    def wait_evicted(self, layer: int) -> None:
        """The caller's stream waits until ``layer``'s swap-out has read its blocks."""
        torch.cuda.current_stream(self.cache.device).wait_event(self.evicted[layer])

    def quiesce(self) -> None:
        """The caller's stream waits for both side streams (e.g. before reading the status word)."""
        cur = torch.cuda.current_stream(self.cache.device)
        cur.wait_stream(self.in_stream)
        cur.wait_stream(self.out_stream)
