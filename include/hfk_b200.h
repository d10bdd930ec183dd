/*
 * hfk_b200.h — C ABI of the B200-native KV-cache data path (libhfk_b200.so).
 *
 * This is the drop-in boundary: plain pointers and sizes, a CUDA stream handle
 * and an int status.  No torch types, no C++ types and no exceptions cross it.
 * The torch operator library `pcie_through` and the pybind module
 * `heterofusedkernels.memory` are thin shims over these functions.
 *
 * The model for the shape of this ABI is the launch ABI of the reference,
 *   extern "C" uint32_t aclrtlaunch_<kernel>(uint32_t blockDim, aclrtStream, args...)
 * (pcieThrough/csrc/include/aclrtlaunch_kernels.h:9-10): a core count, a
 * stream, raw addresses.  Here `ctas` plays the role of `blockDim`/`aiv`
 * ("how many cores to spend"): it is the number of CUDA thread blocks that
 * the persistent kernel is launched with; `ctas <= 0` selects the default of
 * the entry point.
 *
 * Conventions
 *  - Every compute entry point enqueues work on `stream` and returns without
 *    synchronising, like the reference's EXEC_KERNEL_CMD
 *    (pcieThrough/csrc/host/launch_utils.h:26-38).  Unlike the reference it
 *    checks the launch status and returns it.
 *  - "device-accessible" means: a device allocation, or the device alias of a
 *    host range registered through hfk_register_ptr / hfk_alloc_pinned_numa_ptr.
 *  - Return value: HFK_OK (0) or a negative HFK_ERR_* code;
 *    hfk_last_error_message() gives the detail for the calling thread.
 *  - Ids that are out of range are detected ON THE DEVICE: the kernel skips the
 *    block, sets a bit in a per-device status word and never forms the bad
 *    address.  hfk_device_status() reads and clears that word.
 */
#ifndef HFK_B200_H_
#define HFK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cudaStream_t without including the CUDA headers. */
typedef struct CUstream_st *hfk_stream_t;

/* ---- status codes ------------------------------------------------------- */
#define HFK_OK 0
#define HFK_ERR_INVALID_ARG (-1)    /* null pointer, non-positive count, bad enum */
#define HFK_ERR_ALIGNMENT (-2)      /* address or byte count not a multiple of 16 */
#define HFK_ERR_NOT_REGISTERED (-3) /* host pointer outside every registered range */
#define HFK_ERR_CUDA (-4)           /* a CUDA runtime call failed */
#define HFK_ERR_TOO_LARGE (-5)      /* size beyond a stated maximum */
#define HFK_ERR_NO_MEMORY (-6)      /* mmap / mbind / registration failed */
#define HFK_ERR_UNSUPPORTED (-7)    /* combination not implemented */

/* bits of the device status word (hfk_device_status) */
#define HFK_DEV_BAD_DEVICE_BLOCK_ID 0x1u /* device block id outside [0, num_device_blocks) */
#define HFK_DEV_BAD_HOST_SLOT_ID 0x2u    /* host slot id outside [0, num_host_slots) */
#define HFK_DEV_BAD_ROW_ID 0x4u          /* gather row id outside [0, num_rows) */
#define HFK_DEV_BAD_SEQ_LEN 0x8u         /* sequence longer than its block table row */
#define HFK_DEV_WAIT_TIMEOUT 0x10u       /* a bounded mbarrier wait gave up; the destination of that call is undefined */
#define HFK_DEV_BAD_LAYER_PTR 0x20u      /* a layer base in a device pointer table is null or not 16-byte aligned */

const char *hfk_strerror(int code);
const char *hfk_last_error_message(void);
/* Library version, "major.minor.patch". */
const char *hfk_version(void);

/* Reads the status word of the current device into *status_bits and clears it, in one atomic
 * exchange executed on `stream` (so it sees every kernel enqueued on `stream` before it), then
 * synchronises `stream`: not for the hot loop.
 * The word is per DEVICE, not per stream or per caller: every kernel of this library on that GPU
 * ORs into the same word, and a read clears it for everybody.  A caller that runs kernels on
 * several streams must quiesce them (or make `stream` wait on them) before reading, and two
 * independent users of one GPU see each other's bits. */
int hfk_device_status(unsigned int *status_bits, hfk_stream_t stream);

/* Self-test of the kernels' bounded waits: a one-warp kernel waits on a barrier that nothing
 * completes, gives up after limit_us microseconds (1..1000000), sets HFK_DEV_WAIT_TIMEOUT in the
 * status word and returns normally.  The data-path kernels use the same wait with a 2 s limit. */
int hfk_selftest_wait_timeout(unsigned int limit_us, hfk_stream_t stream);

/* Tuning knobs, process-wide, meant for benchmarking.  Ring of the bulk mover:
 * stage_bytes (multiple of 128) x n_stages of shared memory per CTA; vector
 * mover: threads per CTA x 16-byte loads in flight per thread (only a few
 * combinations are compiled).  0 restores the default. */
int hfk_set_bulk_geometry(int stage_bytes, int n_stages);
/* Of the ring's stages, how many may hold stores that are still draining (the rest hold
 * loads in flight); compiled values 1, 2, 3, 4, 6, 8; 0 restores the default. */
int hfk_set_bulk_lag(int lag);
int hfk_set_vector_geometry(int threads, int unroll);
/* Process-wide default pace of the bulk mover's swap-outs in MB/s for calls that give none
 * (hfk_swap_out, or hfk_swap_out_paced with 0); 0 = unpaced.  See hfk_swap_out_paced. */
int hfk_set_swap_out_pace(int megabytes_per_second);
/* Measurement knob: unused dynamic shared memory added to every CTA of the vector swap kernels
 * (multiple of 128, up to 200 KiB; 0 = none).  With enough of it a compute kernel's CTAs can no
 * longer share an SM with a swap CTA, which is how the cost of sharing is measured. */
int hfk_set_vector_smem_pad(int bytes);
/* Bulk paged gather: l2_hints bit 0 / bit 1 = loads / stores carry an L2 evict-first policy;
 * blocked = 1 gives every CTA one contiguous run of pages instead of every grid-th page.
 * -1 restores the default of either. */
int hfk_set_gather_tuning(int l2_hints, int blocked);
/* Staged swap: how many internal copy streams ("lanes") the per-slot copies are dealt to
 * (1 = all on the caller's stream; up to 4; 0 restores the default). */
int hfk_set_staged_copy_lanes(int lanes);

/* Diagnostics: per-CTA time stamps.  With a device buffer installed, thread 0 of every CTA of
 * the swap / migrate kernels appends {tag << 32 | SM id, CTA index, start ns, end ns}
 * (4 x uint64, %globaltimer) after the record counter in word 0; records beyond the capacity
 * are counted but not written.  hfk_debug_stamp_marker enqueues a one-thread kernel that
 * appends a record with tag 0, to mark a point of a stream on the same clock.  Passing NULL
 * removes the buffer.  The setting is per device (the current one) and is meant for
 * measurements, not for production: the caller zeroes and reads the buffer. */
int hfk_debug_set_stamps(void *device_buffer, size_t buffer_bytes);
int hfk_debug_stamp_marker(hfk_stream_t stream);

/* ======================================================================== *
 *  Host-memory registry and NUMA-local pinned allocation
 * ======================================================================== */

/* Registers [ptr, ptr+size) with the current CUDA device as mapped, portable
 * pinned memory and records host ptr -> device alias.  Registering a base that
 * is already recorded returns the existing alias.  Returns the device alias,
 * NULL on failure.
 * Replaces register_ptr (common/csrc/managed_memory/managed_mem.cpp:305-323)
 * and HostRegisteredMemoryManager::registerHostPtr (:45-66). */
void *hfk_register_ptr(void *ptr, size_t size);

/* Removes the record whose base is `ptr` and unregisters the range.  Unknown
 * pointers are not an error (returns 0), as in the reference.
 * Replaces unregister_ptr (managed_mem.cpp:325-334) / aclUnregisterHostPtr (:105-119). */
int hfk_unregister_ptr(void *ptr);

/* Device alias of a host address that lies inside a registered range, 0 if it
 * lies in none.  Replaces get_device_ptr (managed_mem.cpp:372-375) and
 * HostRegisteredMemoryManager::getDevicePtr (:139-160). */
uintptr_t hfk_get_device_ptr(uintptr_t host_ptr);

/* Size of the registered range that contains `ptr`, 0 if none.
 * Replaces HostRegisteredMemoryManager::getRecordSize (managed_mem.cpp:163-179). */
size_t hfk_get_record_size(void *ptr);

/* Number of live records. */
int hfk_registry_count(void);

/* Unregisters everything (the reference does this in the singleton's
 * destructor, managed_mem.cpp:26-41). */
void hfk_unregister_all(void);

/* Test hook: with `on` != 0 the registry stops calling the CUDA driver and
 * hands out the host address itself as the alias, so that the bookkeeping
 * (range lookup, duplicates, removal) can be tested on a machine without a
 * GPU.  No compute entry point consults this switch. */
void hfk_registry_set_test_driver(int on);

/* NUMA node of CUDA device `device` (-1 = current device), read from
 * /sys/bus/pci/devices/<bdf>/numa_node; -1 when the platform reports none.
 * Returns HFK_ERR_* (< -1) on failure.
 * Replaces the DCMI + sysfs lookup in alloc_numa_pinned_tensor
 * (common/csrc/mem_alloc.cpp:18-38, common/csrc/dcmi_management.cpp:27-39). */
int hfk_device_numa_node(int device);

/* PCI bus id of CUDA device `device` (-1 = current) as lower-case
 * "dddd:bb:dd.f" into buf.  Returns HFK_OK or an error. */
int hfk_device_pci_bus_id(int device, char *buf, size_t buf_len);

/* mmap + mbind(MPOL_BIND) to `node` (skipped when node == -1) + zero fill +
 * register.  Returns the host address, NULL on failure.
 * Replaces alloc_pinned_numa_ptr (common/csrc/mem_alloc.cpp:79-115). */
void *hfk_alloc_pinned_numa_ptr(size_t size, int node);

/* Unregister + munmap of a pointer obtained from hfk_alloc_pinned_numa_ptr.
 * Replaces free_pinned_numa_ptr (common/csrc/mem_alloc.cpp:66-77). */
int hfk_free_pinned_numa_ptr(void *ptr);

/* ======================================================================== *
 *  Group R — operators whose semantics are fixed by the reference
 * ======================================================================== */

/* dst[i, 0:row_bytes] = table[ids[i], 0:row_bytes] for i < num_ids.
 * table: device-accessible (host-registered alias or device memory);
 * dst, ids: device memory.  ids are int64 (ids_are_int64 != 0) or int32.
 * num_rows > 0 enables the on-device range check of the ids.
 * Replaces gather_kernel (pcieThrough/csrc/kernel/gather.cpp:7-48,
 * gather.h:35-134) and its launch (pcieThrough/csrc/host/gather_torch.cpp:53). */
int hfk_gather(const void *table, void *dst, const void *ids, int ids_are_int64,
               size_t num_ids, size_t row_bytes, size_t num_rows, int ctas,
               hfk_stream_t stream);

/* One KV block, all layers, with re-layout:
 *   for t < block_size, l < layers, h < heads:
 *     device_layer_ptrs[l][h][t][0:head_dim] = src_block[t][l][h][0:head_dim]
 * device_layer_ptrs: DEVICE array of `layers` pointers, each to an
 * [heads, block_size, head_dim] buffer; src_block: device-accessible
 * [block_size, layers, heads, head_dim].  head_dim*elt_size must be a
 * multiple of 16 bytes.
 * Replaces the kernel multi_layer_block_transfer
 * (pcieThrough/csrc/kernel/multi_layer_block_transfer_kernel.cpp:8-29,
 * multi_layer_block_transfer_kernel.h:42-82) and its tiling
 * (pcieThrough/csrc/host/tiling/multi_layer_block_transfer.cpp:19-56). */
int hfk_multi_layer_block_transfer(void *const *device_layer_ptrs, const void *src_block,
                                   int64_t block_size, int64_t layers, int64_t heads,
                                   int64_t head_dim, int64_t elt_size, int ctas,
                                   hfk_stream_t stream);

/* Staged twin: cudaMemcpyAsync(staging <- host_block) on the copy engine, then
 * the kernel above reading `staging` (device memory of the same size).
 * Replaces fused_memcpy_multi_layer_block_transfer
 * (pcieThrough/csrc/host/multi_layer_block_transfer_torch.cpp:82-106). */
int hfk_fused_memcpy_multi_layer_block_transfer(void *const *device_layer_ptrs,
                                                const void *host_block, void *staging,
                                                int64_t block_size, int64_t layers,
                                                int64_t heads, int64_t head_dim,
                                                int64_t elt_size, int ctas,
                                                hfk_stream_t stream);

/* Capacity of the staging block built into the library (8 MiB: the reference test's
 * largest block, [1024, 64, 1, 128] int8 — pcieThrough/tests/test_transfer_kernel.py:15-24). */
#define HFK_STATIC_STAGING_BYTES (8u * 1024u * 1024u)

/* The staged transfer above for callers that cannot allocate device memory.  It has
 * no counterpart in the reference.
 *
 * Meant for two kinds of caller: a KV-offload connector inside a serving engine that
 * gave nearly all HBM to the KV cache at start-up (a cudaMalloc in its scheduling loop
 * may fail, and always synchronises the device, stalling the compute the transfer
 * should overlap), and FFI hosts (cgo, JNI, ctypes) that hold pointers to the cache and
 * the pinned pool but own no CUDA allocator to make a staging tensor from.
 *
 * Same arguments and result as hfk_fused_memcpy_multi_layer_block_transfer without
 * `staging`: the staging block is a device array of HFK_STATIC_STAGING_BYTES inside the
 * library.  Every GPU the library runs on holds that memory until the process exits.
 * A block larger than that (block_size*layers*heads*head_dim*elt_size) is rejected with
 * HFK_ERR_TOO_LARGE.  The call allocates nothing: no cudaMalloc, cudaFree or other
 * allocating routine.
 *
 * The first call on each device looks the array's device address up (with that device
 * current) and caches it; make that first call before any stream capture begins.
 * All calls on a device share the one staging block, which still holds the previous
 * call's block: calls must not overlap on the GPU — issue them on one stream, or order
 * them with events — otherwise they race on the staging bytes.  Nothing in the block
 * needs clearing between calls: each call overwrites the bytes it then reads. */
int hfk_fused_memcpy_multi_layer_block_transfer_static(void *const *device_layer_ptrs,
                                                       const void *host_block,
                                                       int64_t block_size, int64_t layers,
                                                       int64_t heads, int64_t head_dim,
                                                       int64_t elt_size, int ctas,
                                                       hfk_stream_t stream);

/* ======================================================================== *
 *  Group N — multi-block, all-layer K/V swap and paged gather
 *  (no counterpart function in the reference; conventions follow
 *   pcieThrough/README.md:25-27 for pointer tables and
 *   pcieThrough/csrc/host/gather_torch.cpp:38,44-46 for id tensors)
 * ======================================================================== */

/* Which data mover a swap uses. */
#define HFK_MOVER_AUTO 0   /* the bulk mover; its ring and CTA count follow the bytes of the launch */
#define HFK_MOVER_VECTOR 1 /* 16-byte ld/st loops, whole CTA */
#define HFK_MOVER_BULK 2   /* one thread per CTA pumping cp.async.bulk through shared memory */

typedef struct hfk_swap_desc {
  /* DEVICE arrays of `layers` pointers: base of layer l's K (resp. V) cache,
   * laid out [num_device_blocks][block_bytes (+ padding up to device_block_stride)]. */
  void *const *k_layer_ptrs;
  void *const *v_layer_ptrs;
  /* Device alias of the host pool.  Chunk (slot s, layer l, kv) starts at
   * host_pool + s*host_slot_stride + l*host_layer_stride + kv*host_kv_stride. */
  void *host_pool;
  /* DEVICE arrays of n_blocks ids; int64 when ids_are_int64 != 0, else int32. */
  const void *device_block_ids;
  const void *host_slot_ids;
  int ids_are_int64;
  int layers;
  int64_t n_blocks;
  int64_t block_bytes;         /* bytes of one (block, layer, K|V) chunk; multiple of 16 */
  int64_t device_block_stride; /* bytes between consecutive device blocks (>= block_bytes) */
  int64_t host_slot_stride;
  int64_t host_layer_stride;
  int64_t host_kv_stride;
  int64_t num_device_blocks;   /* range check of device_block_ids */
  int64_t num_host_slots;      /* range check of host_slot_ids */
} hfk_swap_desc;

/* Swap-out: for every i < n_blocks, layer l, kv in {K,V}:
 *   host chunk(host_slot_ids[i], l, kv) = device chunk(device_block_ids[i], l, kv)
 * one launch for all layers.  host slots must be distinct. */
int hfk_swap_out(const hfk_swap_desc *desc, int mover, int ctas, hfk_stream_t stream);

/* Swap-out whose stores are paced to about `megabytes_per_second` (1 MB = 1e6 bytes; 0 = unpaced, the
 * same as hfk_swap_out; bulk mover only).  For a swap-out that shares the link with a swap-in: the
 * upstream lanes carry the swap-out's write TLPs AND the swap-in's read requests, and an unpaced
 * swap-out crowds the requests out (one B200 on Gen5 x16, 1.07 GB each way at once: 42.9 GB/s out with
 * 34.5 in unpaced; 40.0 out with 42.0 in when paced to 40 000 MB/s). */
int hfk_swap_out_paced(const hfk_swap_desc *desc, int mover, int ctas, int megabytes_per_second,
                       hfk_stream_t stream);

/* Swap-in: the inverse copy; device block ids must be distinct. */
int hfk_swap_in(const hfk_swap_desc *desc, int mover, int ctas, hfk_stream_t stream);

/* Copy-engine alternative: one cudaMemcpyAsync per chunk.  All five arrays of
 * the descriptor (pointer tables and id lists) are HOST arrays here, and
 * host_pool is the HOST address of the pinned pool.  to_host != 0 = swap-out. */
int hfk_swap_copy_engine(const hfk_swap_desc *desc_with_host_arrays, int to_host,
                         hfk_stream_t stream);

/* Multi-block swap in the reference's host block format: host slot = one KV block
 * [block_size][layers][heads][head_dim] (pcieThrough/README.md:25-29), layer l of the device
 * cache = [num_device_blocks][heads][block_size][head_dim].  K and V are separate tensor
 * families here as in the reference (call once per family, or list them as 2*layers layers). */
/* Staged swap through the copy engine.  Kernel-issued PCIe traffic moves in 128-byte
 * transactions and tops out near 92 % of what cudaMemcpyAsync reaches with 256-byte ones, so
 * this mover lets the copy engine cross the link: a short kernel packs the listed device
 * chunks into `staging` (HBM to HBM, slot-contiguous) and one cudaMemcpyAsync per RUN of
 * consecutive host slots (cut at 64 MiB) moves [slots][layers][K|V][block_bytes] at once
 * (swap-in: the copies first, then the kernel unpacks).  It pays off when the copies are
 * 8 MiB or larger, i.e. when the slots of a call come in runs.  It is the multi-block form of
 * the reference's staged transfer
 * (pcieThrough/csrc/host/multi_layer_block_transfer_torch.cpp:82-106).
 *
 * desc: as for hfk_swap_out, except that desc->host_slot_ids is not used and the pool must
 * be slot-contiguous (host_kv_stride == block_bytes, host_layer_stride == 2*block_bytes).
 * host_slot_ids_host: HOST array of desc->n_blocks ids (same width as the device ids);
 * host_pool_host: HOST address of the pinned pool; staging: device buffer of staging_bytes
 * >= one slot (layers*2*block_bytes); larger buffers mean fewer rounds.  With one copy lane
 * (the default) everything is enqueued on `stream`; with more (hfk_set_staged_copy_lanes) the
 * copies run on internal streams that fork from `stream` and join it again.  A one-layer view
 * of a layer-major pool (layers == 1, any layer stride) counts as slot-contiguous.  Nothing is
 * allocated per call. */
int hfk_swap_staged(const hfk_swap_desc *desc, const void *host_slot_ids_host, void *host_pool_host,
                    void *staging, size_t staging_bytes, int to_host, int ctas, hfk_stream_t stream);

typedef struct hfk_relayout_desc {
  void *const *layer_ptrs;      /* DEVICE array of `layers` cache bases */
  void *host_pool;              /* device alias; slot s at host_pool + s*host_slot_stride */
  const void *device_block_ids; /* DEVICE arrays of n_blocks ids */
  const void *host_slot_ids;
  int ids_are_int64;
  int layers;
  int64_t n_blocks;
  int64_t block_size;
  int64_t heads;
  int64_t head_bytes;           /* head_dim*elt_size; multiple of 16 */
  int64_t device_block_stride;  /* >= heads*block_size*head_bytes */
  int64_t host_slot_stride;     /* >= block_size*layers*heads*head_bytes */
  int64_t num_device_blocks;
  int64_t num_host_slots;
} hfk_relayout_desc;

/* to_host == 0: for every i, t, l, h:
 *   layer_ptrs[l][device_block_ids[i]][h][t][:] = host slot(host_slot_ids[i])[t][l][h][:]
 * (with n_blocks == 1 this is hfk_multi_layer_block_transfer); to_host != 0: the inverse copy.
 * Generalises multi_layer_block_transfer
 * (pcieThrough/csrc/kernel/multi_layer_block_transfer_kernel.h:42-82) to id lists and to the
 * device->host direction. */
int hfk_swap_relayout(const hfk_relayout_desc *desc, int to_host, int ctas, hfk_stream_t stream);

/* ---- block migration between two caches (one GPU, or two GPUs over NVLink) ----------------
 * No counterpart function in the reference, whose transfers are host<->device only; it is the
 * step next to the swap path: moving KV blocks between the caches of two GPUs (or inside one)
 * without a detour through the host. */
typedef struct hfk_migrate_desc {
  /* DEVICE arrays (in the memory of the GPU that runs the kernel) of `layers` cache bases.
   * The source bases, the destination bases, or neither may point into a peer GPU's memory
   * (peer access enabled, see hfk_enable_peer_access). */
  void *const *src_k_layer_ptrs;
  void *const *src_v_layer_ptrs;
  void *const *dst_k_layer_ptrs;
  void *const *dst_v_layer_ptrs;
  /* DEVICE arrays of n_blocks ids (int64 when ids_are_int64 != 0, else int32). */
  const void *src_block_ids;
  const void *dst_block_ids;
  int ids_are_int64;
  int layers;
  int64_t n_blocks;
  int64_t block_bytes;       /* multiple of 16 */
  int64_t src_block_stride;  /* >= block_bytes */
  int64_t dst_block_stride;
  int64_t num_src_blocks;    /* range checks */
  int64_t num_dst_blocks;
} hfk_migrate_desc;

/* For every i < n_blocks, layer l, kv: dst chunk(dst_block_ids[i], l, kv) = src chunk(src_block_ids[i], l, kv),
 * one launch on the current device.  Launched on the destination GPU it pulls (peer loads,
 * local stores); launched on the source GPU it pushes.  Only 16-byte vector loads and stores
 * touch peer memory.  Destination ids must be distinct. */
int hfk_migrate_blocks(const hfk_migrate_desc *desc, int ctas, hfk_stream_t stream);

/* Copy-engine alternative: one cudaMemcpyPeerAsync (cudaMemcpyAsync when src_device ==
 * dst_device) per chunk.  All arrays of the descriptor are HOST arrays here. */
int hfk_migrate_blocks_copy_engine(const hfk_migrate_desc *desc_with_host_arrays, int src_device,
                                   int dst_device, hfk_stream_t stream);

/* Lets the current device address `peer_device`'s memory (cudaDeviceEnablePeerAccess; already
 * enabled is not an error). */
int hfk_enable_peer_access(int peer_device);

typedef struct hfk_paged_gather_desc {
  void *const *k_layer_ptrs; /* DEVICE arrays of `layers` cache bases, as in hfk_swap_desc */
  void *const *v_layer_ptrs;
  void *k_out; /* [layers][total_tokens][token_bytes], layer l at k_out + l*out_layer_stride */
  void *v_out;
  int64_t out_layer_stride;
  /* DEVICE int32/int64 array [num_seqs][max_blocks_per_seq] (row stride in elements
   * = block_table_stride) and DEVICE array [num_seqs] of sequence lengths in tokens. */
  const void *block_tables;
  const void *seq_lens;
  int ids_are_int64;
  int layers;
  int64_t num_seqs;           /* batches above HFK_MAX_SEQS are split into several launches */
  int64_t max_blocks_per_seq;
  int64_t block_table_stride;
  int64_t block_size;         /* tokens per block */
  int64_t token_bytes;        /* kv_heads*head_dim*elt_size; multiple of 16 */
  int64_t device_block_stride;/* bytes between cache blocks (>= block_size*token_bytes) */
  int64_t num_device_blocks;  /* range check of the table entries */
  int64_t total_tokens;       /* capacity of k_out/v_out in tokens (range check) */
} hfk_paged_gather_desc;

#define HFK_MAX_SEQS 1024

/* Paged gather: sequence s owns output tokens [cu(s), cu(s)+seq_lens[s]) where cu
 * is the exclusive prefix sum of seq_lens; its j-th page is copied from
 * cache block block_tables[s][j] (the last page partially).  All layers, K and V,
 * one launch. */
int hfk_paged_gather(const hfk_paged_gather_desc *desc, int mover, int ctas,
                     hfk_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* HFK_B200_H_ */
