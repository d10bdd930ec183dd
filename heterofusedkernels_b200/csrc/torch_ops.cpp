// torch operator library `pcie_through` for CUDA: a thin shim that unpacks
// tensors into the C ABI of libhfk_b200.so.
//
// Group R keeps the reference's schemas verbatim
//   gather(Tensor gmEmbed, Tensor gmEmbedDst, Tensor gmIds, int? aiv=None) -> ()
//       (pcieThrough/csrc/host/gather_torch.cpp:60)
//   multi_layer_block_transfer(Tensor deviceBlockCachePtrs, Tensor hostBlockCache, int? aiv=None) -> ()
//   fused_memcpy_multi_layer_block_transfer(Tensor deviceBlockCachePtrs, Tensor hostBlockCache,
//                                           Tensor stagingBlockCache, int? aiv=None) -> ()
//       (pcieThrough/csrc/host/multi_layer_block_transfer_torch.cpp:113-114)
// registered for the CUDA dispatch key where the reference uses PrivateUse1
// (gather_torch.cpp:65-68, multi_layer_block_transfer_torch.cpp:119-122).  Ops
// mutate their destination in place, return nothing and run asynchronously on
// the current stream (pcieThrough/csrc/host/launch_utils.h:28).
//
// Differences that are deliberate: a host tensor outside every registered range
// raises instead of handing a null alias to the kernel
// (multi_layer_block_transfer_torch.cpp:77-78 passes it on unchecked); a table
// that already lives in device memory is used directly (pcieThrough/README.md:18
// promises this, gather_torch.cpp:50-51 breaks it); launch errors are reported.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime_api.h>
#include <torch/library.h>

#include <string>

#include "../../include/hfk_b200.h"

namespace pciethrough {

static void check_rc(int rc, const char *op) {
  TORCH_CHECK(rc == HFK_OK, op, ": ", hfk_strerror(rc), " — ", hfk_last_error_message());
}

static int cores_from(const c10::optional<int64_t> &aiv) {
  // "aiv" keeps its meaning of "how many cores to spend"
  // (multi_layer_block_transfer_torch.cpp:59-64); None selects the tuned default.
  if (!aiv.has_value()) return 0;
  TORCH_CHECK(aiv.value() > 0, "Number of AIV blocks should be positive.");
  return static_cast<int>(aiv.value());
}

// Address a kernel can dereference for `t`: device tensors as they are, host
// tensors through the registry.
static void *device_accessible(const at::Tensor &t, const char *what) {
  if (t.is_cuda()) return t.data_ptr();
  TORCH_CHECK(t.device().is_cpu(), what, ": tensor must live on CPU (registered) or CUDA");
  const uintptr_t alias = hfk_get_device_ptr(reinterpret_cast<uintptr_t>(t.data_ptr()));
  TORCH_CHECK(alias != 0, what,
              ": host tensor is not inside a range registered with heterofusedkernels.memory "
              "(alloc_numa_pinned_tensor / host_register)");
  return reinterpret_cast<void *>(alias);
}

static int ids_are_int64(const at::Tensor &ids, const char *what) {
  TORCH_CHECK(ids.scalar_type() == at::kLong || ids.scalar_type() == at::kInt, what,
              ": ids must be int64 or int32, got ", c10::toString(ids.scalar_type()));
  TORCH_CHECK(ids.dim() == 1 && ids.is_contiguous(), what, ": ids must be 1-D and contiguous");
  return ids.scalar_type() == at::kLong ? 1 : 0;
}

static void check_ptr_table(const at::Tensor &t, int64_t layers, const char *what, bool on_device) {
  TORCH_CHECK(t.scalar_type() == at::kLong && t.dim() == 1 && t.is_contiguous(), what,
              ": pointer table must be a contiguous 1-D int64 tensor");
  TORCH_CHECK(t.is_cuda() == on_device, what, on_device ? ": pointer table must be on the device"
                                                        : ": pointer table must be on the CPU");
  if (layers >= 0)
    TORCH_CHECK(t.numel() == layers, what, ": pointer table has ", t.numel(), " entries, expected ",
                layers, " (one per layer)");
}

// ---------------------------------------------------------------- Group R ---
void gather(const at::Tensor &gmEmbed, const at::Tensor &gmEmbedDst, const at::Tensor &gmIds,
            c10::optional<int64_t> aiv) {
  const int ctas = cores_from(aiv);
  TORCH_CHECK(gmEmbed.dim() == 2 && gmEmbed.is_contiguous(), "gather: gmEmbed must be a contiguous 2-D tensor");
  TORCH_CHECK(gmEmbedDst.is_cuda() && gmEmbedDst.is_contiguous(), "gather: gmEmbedDst must be a contiguous device tensor");
  const int is64 = ids_are_int64(gmIds, "gather");
  const size_t numIds = static_cast<size_t>(gmIds.size(0));
  const size_t rowBytes = static_cast<size_t>(gmEmbed.element_size()) * gmEmbed.size(1);
  TORCH_CHECK(static_cast<size_t>(gmEmbedDst.nbytes()) >= numIds * rowBytes,
              "gather: gmEmbedDst holds fewer than numIds rows");
  const c10::cuda::CUDAGuard guard(gmEmbedDst.device());
  check_rc(hfk_gather(device_accessible(gmEmbed, "gather(gmEmbed)"), gmEmbedDst.data_ptr(),
                      device_accessible(gmIds, "gather(gmIds)"), is64, numIds, rowBytes,
                      static_cast<size_t>(gmEmbed.size(0)), ctas,
                      at::cuda::getCurrentCUDAStream().stream()),
           "gather");
}

struct BlockGeometry {
  int64_t B, L, H, D, elt;
};
static BlockGeometry geometry_of(const at::Tensor &hostBlockCache, const char *op) {
  // the shape comes from the HOST tensor [BlockSize, Layers, Heads, HeadDim]
  // (multi_layer_block_transfer_torch.cpp:67-71)
  TORCH_CHECK(hostBlockCache.dim() == 4 && hostBlockCache.is_contiguous(), op,
              ": hostBlockCache must be a contiguous [BlockSize, Layers, Heads, HeadDim] tensor");
  return {hostBlockCache.size(0), hostBlockCache.size(1), hostBlockCache.size(2),
          hostBlockCache.size(3), static_cast<int64_t>(hostBlockCache.element_size())};
}

void multi_layer_block_transfer(const at::Tensor &deviceBlockCachePtrs,
                                const at::Tensor &hostBlockCache, c10::optional<int64_t> aiv) {
  const int ctas = cores_from(aiv);
  const BlockGeometry g = geometry_of(hostBlockCache, "multi_layer_block_transfer");
  check_ptr_table(deviceBlockCachePtrs, g.L, "multi_layer_block_transfer(deviceBlockCachePtrs)", true);
  const c10::cuda::CUDAGuard guard(deviceBlockCachePtrs.device());
  check_rc(hfk_multi_layer_block_transfer(
               reinterpret_cast<void *const *>(deviceBlockCachePtrs.data_ptr()),
               device_accessible(hostBlockCache, "multi_layer_block_transfer(hostBlockCache)"), g.B,
               g.L, g.H, g.D, g.elt, ctas, at::cuda::getCurrentCUDAStream().stream()),
           "multi_layer_block_transfer");
}

void fused_memcpy_multi_layer_block_transfer(const at::Tensor &deviceBlockCachePtrs,
                                             const at::Tensor &hostBlockCache,
                                             const at::Tensor &stagingBlockCache,
                                             c10::optional<int64_t> aiv) {
  const int ctas = cores_from(aiv);
  const BlockGeometry g = geometry_of(hostBlockCache, "fused_memcpy_multi_layer_block_transfer");
  check_ptr_table(deviceBlockCachePtrs, g.L, "fused_memcpy_multi_layer_block_transfer(deviceBlockCachePtrs)", true);
  TORCH_CHECK(hostBlockCache.device().is_cpu(), "fused_memcpy_multi_layer_block_transfer: hostBlockCache must be a CPU tensor");
  TORCH_CHECK(stagingBlockCache.is_cuda() && stagingBlockCache.is_contiguous() &&
                  stagingBlockCache.nbytes() >= hostBlockCache.nbytes(),
              "fused_memcpy_multi_layer_block_transfer: stagingBlockCache must be a contiguous device "
              "tensor at least as large as hostBlockCache");
  const c10::cuda::CUDAGuard guard(stagingBlockCache.device());
  check_rc(hfk_fused_memcpy_multi_layer_block_transfer(
               reinterpret_cast<void *const *>(deviceBlockCachePtrs.data_ptr()),
               hostBlockCache.data_ptr(), stagingBlockCache.data_ptr(), g.B, g.L, g.H, g.D, g.elt,
               ctas, at::cuda::getCurrentCUDAStream().stream()),
           "fused_memcpy_multi_layer_block_transfer");
}

// ---------------------------------------------------------------- Group N ---
// hostPool is a CPU tensor [slots, layers, 2, ...] whose trailing dimensions are
// contiguous and form one chunk; slot / layer / K|V strides are taken from the
// tensor, so a layer-major pool can be passed as a permuted view.
static hfk_swap_desc swap_desc(const at::Tensor &kLayerPtrs, const at::Tensor &vLayerPtrs,
                               const at::Tensor &hostPool, const at::Tensor &deviceBlockIds,
                               const at::Tensor &hostSlotIds, int64_t numDeviceBlocks,
                               c10::optional<int64_t> deviceBlockStride, bool arrays_on_device,
                               const char *op) {
  TORCH_CHECK(hostPool.device().is_cpu() && hostPool.dim() >= 4, op,
              ": hostPool must be a CPU tensor [slots, layers, 2, ...chunk dims]");
  TORCH_CHECK(hostPool.size(2) == 2, op, ": hostPool dimension 2 must have size 2 (K, V)");
  const int64_t elt = hostPool.element_size();
  int64_t chunk_elems = 1;
  for (int64_t d = hostPool.dim() - 1; d >= 3; --d) {
    TORCH_CHECK(hostPool.stride(d) == chunk_elems, op, ": the chunk dimensions of hostPool must be contiguous");
    chunk_elems *= hostPool.size(d);
  }
  hfk_swap_desc d;
  d.layers = static_cast<int>(hostPool.size(1));
  check_ptr_table(kLayerPtrs, d.layers, op, arrays_on_device);
  check_ptr_table(vLayerPtrs, d.layers, op, arrays_on_device);
  d.ids_are_int64 = ids_are_int64(deviceBlockIds, op);
  TORCH_CHECK(ids_are_int64(hostSlotIds, op) == d.ids_are_int64, op, ": both id lists must have the same dtype");
  TORCH_CHECK(deviceBlockIds.numel() == hostSlotIds.numel(), op, ": id lists differ in length");
  TORCH_CHECK(deviceBlockIds.is_cuda() == arrays_on_device && hostSlotIds.is_cuda() == arrays_on_device,
              op, arrays_on_device ? ": id lists must be device tensors" : ": id lists must be CPU tensors");
  d.k_layer_ptrs = reinterpret_cast<void *const *>(kLayerPtrs.data_ptr());
  d.v_layer_ptrs = reinterpret_cast<void *const *>(vLayerPtrs.data_ptr());
  d.host_pool = arrays_on_device ? device_accessible(hostPool, op) : hostPool.data_ptr();
  d.device_block_ids = deviceBlockIds.data_ptr();
  d.host_slot_ids = hostSlotIds.data_ptr();
  d.n_blocks = deviceBlockIds.numel();
  d.block_bytes = chunk_elems * elt;
  d.device_block_stride = deviceBlockStride.has_value() ? deviceBlockStride.value() : d.block_bytes;
  d.host_slot_stride = hostPool.stride(0) * elt;
  d.host_layer_stride = hostPool.stride(1) * elt;
  d.host_kv_stride = hostPool.stride(2) * elt;
  d.num_device_blocks = numDeviceBlocks;
  d.num_host_slots = hostPool.size(0);
  return d;
}

static int mover_from(const c10::optional<int64_t> &mover) {
  return mover.has_value() ? static_cast<int>(mover.value()) : HFK_MOVER_AUTO;
}

void swap_out(const at::Tensor &kLayerPtrs, const at::Tensor &vLayerPtrs, const at::Tensor &hostPool,
              const at::Tensor &deviceBlockIds, const at::Tensor &hostSlotIds,
              int64_t numDeviceBlocks, c10::optional<int64_t> deviceBlockStride,
              c10::optional<int64_t> aiv, c10::optional<int64_t> mover, c10::optional<int64_t> paceMBs) {
  const int ctas = cores_from(aiv);
  const hfk_swap_desc d = swap_desc(kLayerPtrs, vLayerPtrs, hostPool, deviceBlockIds, hostSlotIds,
                                    numDeviceBlocks, deviceBlockStride, true, "swap_out");
  const c10::cuda::CUDAGuard guard(kLayerPtrs.device());
  // paceMBs: stores paced to that many MB/s (for a swap-out that shares the link with a swap-in)
  check_rc(hfk_swap_out_paced(&d, mover_from(mover), ctas, paceMBs.has_value() ? static_cast<int>(paceMBs.value()) : 0,
                              at::cuda::getCurrentCUDAStream().stream()),
           "swap_out");
}

void swap_in(const at::Tensor &kLayerPtrs, const at::Tensor &vLayerPtrs, const at::Tensor &hostPool,
             const at::Tensor &deviceBlockIds, const at::Tensor &hostSlotIds, int64_t numDeviceBlocks,
             c10::optional<int64_t> deviceBlockStride, c10::optional<int64_t> aiv,
             c10::optional<int64_t> mover) {
  const int ctas = cores_from(aiv);
  const hfk_swap_desc d = swap_desc(kLayerPtrs, vLayerPtrs, hostPool, deviceBlockIds, hostSlotIds,
                                    numDeviceBlocks, deviceBlockStride, true, "swap_in");
  const c10::cuda::CUDAGuard guard(kLayerPtrs.device());
  check_rc(hfk_swap_in(&d, mover_from(mover), ctas, at::cuda::getCurrentCUDAStream().stream()), "swap_in");
}

// Staged movers: a packing kernel plus one copy-engine transfer per host slot.  hostSlotIds is a
// CPU tensor here (the copies are addressed on the host); staging is a device byte buffer of at
// least one slot.
static void swap_staged(const at::Tensor &kLayerPtrs, const at::Tensor &vLayerPtrs, const at::Tensor &hostPool,
                        const at::Tensor &deviceBlockIds, const at::Tensor &hostSlotIds, const at::Tensor &staging,
                        int64_t numDeviceBlocks, c10::optional<int64_t> deviceBlockStride,
                        c10::optional<int64_t> aiv, int to_host, const char *op) {
  const int ctas = cores_from(aiv);
  TORCH_CHECK(hostSlotIds.device().is_cpu(), op, ": hostSlotIds must be a CPU tensor");
  TORCH_CHECK(staging.is_cuda() && staging.is_contiguous(), op, ": staging must be a contiguous device tensor");
  // build the descriptor with the device id list standing in for both lists, then attach the host list
  hfk_swap_desc d = swap_desc(kLayerPtrs, vLayerPtrs, hostPool, deviceBlockIds, deviceBlockIds, numDeviceBlocks,
                              deviceBlockStride, true, op);
  TORCH_CHECK(ids_are_int64(hostSlotIds, op) == d.ids_are_int64 && hostSlotIds.numel() == deviceBlockIds.numel(),
              op, ": hostSlotIds must match deviceBlockIds in dtype and length");
  const c10::cuda::CUDAGuard guard(kLayerPtrs.device());
  check_rc(hfk_swap_staged(&d, hostSlotIds.data_ptr(), hostPool.data_ptr(), staging.data_ptr(),
                           static_cast<size_t>(staging.nbytes()), to_host, ctas,
                           at::cuda::getCurrentCUDAStream().stream()),
           op);
}

void swap_out_staged(const at::Tensor &kLayerPtrs, const at::Tensor &vLayerPtrs, const at::Tensor &hostPool,
                     const at::Tensor &deviceBlockIds, const at::Tensor &hostSlotIds, const at::Tensor &staging,
                     int64_t numDeviceBlocks, c10::optional<int64_t> deviceBlockStride, c10::optional<int64_t> aiv) {
  swap_staged(kLayerPtrs, vLayerPtrs, hostPool, deviceBlockIds, hostSlotIds, staging, numDeviceBlocks,
              deviceBlockStride, aiv, 1, "swap_out_staged");
}

void swap_in_staged(const at::Tensor &kLayerPtrs, const at::Tensor &vLayerPtrs, const at::Tensor &hostPool,
                    const at::Tensor &deviceBlockIds, const at::Tensor &hostSlotIds, const at::Tensor &staging,
                    int64_t numDeviceBlocks, c10::optional<int64_t> deviceBlockStride, c10::optional<int64_t> aiv) {
  swap_staged(kLayerPtrs, vLayerPtrs, hostPool, deviceBlockIds, hostSlotIds, staging, numDeviceBlocks,
              deviceBlockStride, aiv, 0, "swap_in_staged");
}

// Device that owns the memory a raw device address points into (the first entry of a CPU-resident
// pointer table); falls back to the current device when the driver does not know the address.
static c10::Device device_of_address(int64_t address) {
  cudaPointerAttributes attr;
  if (address != 0 && cudaPointerGetAttributes(&attr, reinterpret_cast<const void *>(address)) == cudaSuccess &&
      attr.type == cudaMemoryTypeDevice)
    return c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(attr.device));
  cudaGetLastError();
  return c10::Device(c10::kCUDA, c10::cuda::current_device());
}

// Copy-engine twins: every tensor argument lives on the CPU (the addresses are
// formed on the host); the copies run on the current stream of the device that
// owns the cache (taken from the first layer pointer).
void swap_out_copy_engine(const at::Tensor &kLayerPtrs, const at::Tensor &vLayerPtrs,
                          const at::Tensor &hostPool, const at::Tensor &deviceBlockIds,
                          const at::Tensor &hostSlotIds, int64_t numDeviceBlocks,
                          c10::optional<int64_t> deviceBlockStride) {
  const hfk_swap_desc d = swap_desc(kLayerPtrs, vLayerPtrs, hostPool, deviceBlockIds, hostSlotIds,
                                    numDeviceBlocks, deviceBlockStride, false, "swap_out_copy_engine");
  const c10::cuda::CUDAGuard guard(device_of_address(kLayerPtrs.numel() ? kLayerPtrs[0].item<int64_t>() : 0));
  check_rc(hfk_swap_copy_engine(&d, 1, at::cuda::getCurrentCUDAStream().stream()), "swap_out_copy_engine");
}

void swap_in_copy_engine(const at::Tensor &kLayerPtrs, const at::Tensor &vLayerPtrs,
                         const at::Tensor &hostPool, const at::Tensor &deviceBlockIds,
                         const at::Tensor &hostSlotIds, int64_t numDeviceBlocks,
                         c10::optional<int64_t> deviceBlockStride) {
  const hfk_swap_desc d = swap_desc(kLayerPtrs, vLayerPtrs, hostPool, deviceBlockIds, hostSlotIds,
                                    numDeviceBlocks, deviceBlockStride, false, "swap_in_copy_engine");
  const c10::cuda::CUDAGuard guard(device_of_address(kLayerPtrs.numel() ? kLayerPtrs[0].item<int64_t>() : 0));
  check_rc(hfk_swap_copy_engine(&d, 0, at::cuda::getCurrentCUDAStream().stream()), "swap_in_copy_engine");
}

// Multi-block swap in the reference's host block format.  hostPool: registered CPU tensor
// [slots, BlockSize, Layers, Heads, HeadDim] (each slot laid out like hostBlockCache of
// multi_layer_block_transfer); layerPtrs: device int64 [Layers], layer l's cache being
// [numDeviceBlocks, Heads, BlockSize, HeadDim].
static hfk_relayout_desc relayout_desc(const at::Tensor &layerPtrs, const at::Tensor &hostPool,
                                       const at::Tensor &deviceBlockIds, const at::Tensor &hostSlotIds,
                                       int64_t numDeviceBlocks, c10::optional<int64_t> deviceBlockStride,
                                       const char *op) {
  TORCH_CHECK(hostPool.device().is_cpu() && hostPool.dim() == 5, op,
              ": hostPool must be a CPU tensor [slots, BlockSize, Layers, Heads, HeadDim]");
  TORCH_CHECK(hostPool[0].is_contiguous(), op, ": every host slot must be contiguous");
  const int64_t elt = hostPool.element_size();
  hfk_relayout_desc d;
  d.layers = static_cast<int>(hostPool.size(2));
  check_ptr_table(layerPtrs, d.layers, op, true);
  d.ids_are_int64 = ids_are_int64(deviceBlockIds, op);
  TORCH_CHECK(ids_are_int64(hostSlotIds, op) == d.ids_are_int64, op, ": both id lists must have the same dtype");
  TORCH_CHECK(deviceBlockIds.numel() == hostSlotIds.numel(), op, ": id lists differ in length");
  TORCH_CHECK(deviceBlockIds.is_cuda() && hostSlotIds.is_cuda(), op, ": id lists must be device tensors");
  d.layer_ptrs = reinterpret_cast<void *const *>(layerPtrs.data_ptr());
  d.host_pool = device_accessible(hostPool, op);
  d.device_block_ids = deviceBlockIds.data_ptr();
  d.host_slot_ids = hostSlotIds.data_ptr();
  d.n_blocks = deviceBlockIds.numel();
  d.block_size = hostPool.size(1);
  d.heads = hostPool.size(3);
  d.head_bytes = hostPool.size(4) * elt;
  d.device_block_stride = deviceBlockStride.has_value() ? deviceBlockStride.value()
                                                        : d.heads * d.block_size * d.head_bytes;
  d.host_slot_stride = hostPool.stride(0) * elt;
  d.num_device_blocks = numDeviceBlocks;
  d.num_host_slots = hostPool.size(0);
  return d;
}

void swap_in_relayout(const at::Tensor &layerPtrs, const at::Tensor &hostPool, const at::Tensor &deviceBlockIds,
                      const at::Tensor &hostSlotIds, int64_t numDeviceBlocks,
                      c10::optional<int64_t> deviceBlockStride, c10::optional<int64_t> aiv) {
  const int ctas = cores_from(aiv);
  const hfk_relayout_desc d = relayout_desc(layerPtrs, hostPool, deviceBlockIds, hostSlotIds, numDeviceBlocks,
                                            deviceBlockStride, "swap_in_relayout");
  const c10::cuda::CUDAGuard guard(layerPtrs.device());
  check_rc(hfk_swap_relayout(&d, 0, ctas, at::cuda::getCurrentCUDAStream().stream()), "swap_in_relayout");
}

void swap_out_relayout(const at::Tensor &layerPtrs, const at::Tensor &hostPool, const at::Tensor &deviceBlockIds,
                       const at::Tensor &hostSlotIds, int64_t numDeviceBlocks,
                       c10::optional<int64_t> deviceBlockStride, c10::optional<int64_t> aiv) {
  const int ctas = cores_from(aiv);
  const hfk_relayout_desc d = relayout_desc(layerPtrs, hostPool, deviceBlockIds, hostSlotIds, numDeviceBlocks,
                                            deviceBlockStride, "swap_out_relayout");
  const c10::cuda::CUDAGuard guard(layerPtrs.device());
  check_rc(hfk_swap_relayout(&d, 1, ctas, at::cuda::getCurrentCUDAStream().stream()), "swap_out_relayout");
}

// kOut / vOut: [layers, total_tokens, ...token dims]; blockTables: [num_seqs, max_blocks];
// seqLens: [num_seqs].
void paged_gather(const at::Tensor &kLayerPtrs, const at::Tensor &vLayerPtrs, const at::Tensor &kOut,
                  const at::Tensor &vOut, const at::Tensor &blockTables, const at::Tensor &seqLens,
                  int64_t blockSize, int64_t numDeviceBlocks, c10::optional<int64_t> deviceBlockStride,
                  c10::optional<int64_t> aiv, c10::optional<int64_t> mover) {
  const int ctas = cores_from(aiv);
  TORCH_CHECK(kOut.is_cuda() && vOut.is_cuda() && kOut.dim() >= 3 && kOut.sizes() == vOut.sizes() &&
                  kOut.is_contiguous() && vOut.is_contiguous(),
              "paged_gather: kOut and vOut must be contiguous device tensors [layers, total_tokens, ...] of equal shape");
  TORCH_CHECK(blockTables.is_cuda() && blockTables.dim() == 2 && blockTables.stride(1) == 1,
              "paged_gather: blockTables must be a device tensor [num_seqs, max_blocks] with unit inner stride");
  TORCH_CHECK(seqLens.is_cuda() && seqLens.dim() == 1 && seqLens.is_contiguous() &&
                  seqLens.scalar_type() == blockTables.scalar_type() &&
                  seqLens.size(0) == blockTables.size(0),
              "paged_gather: seqLens must be a device tensor [num_seqs] of the same dtype as blockTables");
  TORCH_CHECK(blockTables.scalar_type() == at::kLong || blockTables.scalar_type() == at::kInt,
              "paged_gather: blockTables must be int64 or int32");
  hfk_paged_gather_desc d;
  d.layers = static_cast<int>(kOut.size(0));
  check_ptr_table(kLayerPtrs, d.layers, "paged_gather(kLayerPtrs)", true);
  check_ptr_table(vLayerPtrs, d.layers, "paged_gather(vLayerPtrs)", true);
  d.k_layer_ptrs = reinterpret_cast<void *const *>(kLayerPtrs.data_ptr());
  d.v_layer_ptrs = reinterpret_cast<void *const *>(vLayerPtrs.data_ptr());
  d.k_out = kOut.data_ptr();
  d.v_out = vOut.data_ptr();
  d.total_tokens = kOut.size(1);
  d.token_bytes = kOut.stride(1) * kOut.element_size();
  d.out_layer_stride = kOut.stride(0) * kOut.element_size();
  d.block_tables = blockTables.data_ptr();
  d.seq_lens = seqLens.data_ptr();
  d.ids_are_int64 = blockTables.scalar_type() == at::kLong ? 1 : 0;
  d.num_seqs = blockTables.size(0);
  d.max_blocks_per_seq = blockTables.size(1);
  d.block_table_stride = blockTables.stride(0);
  d.block_size = blockSize;
  d.device_block_stride =
      deviceBlockStride.has_value() ? deviceBlockStride.value() : blockSize * d.token_bytes;
  d.num_device_blocks = numDeviceBlocks;
  const c10::cuda::CUDAGuard guard(kOut.device());
  check_rc(hfk_paged_gather(&d, mover_from(mover), ctas, at::cuda::getCurrentCUDAStream().stream()),
           "paged_gather");
}

// Block migration between two caches.  The four pointer tables and the two id lists are device
// tensors on the GPU that runs the kernel (the current device of the tables); the addresses in
// the tables may belong to a peer GPU whose access has been enabled (torch enables it on the
// first cross-device copy; hfk_enable_peer_access does it explicitly).
void migrate_blocks(const at::Tensor &srcKLayerPtrs, const at::Tensor &srcVLayerPtrs,
                    const at::Tensor &dstKLayerPtrs, const at::Tensor &dstVLayerPtrs,
                    const at::Tensor &srcBlockIds, const at::Tensor &dstBlockIds, int64_t blockBytes,
                    int64_t numSrcBlocks, int64_t numDstBlocks, c10::optional<int64_t> srcBlockStride,
                    c10::optional<int64_t> dstBlockStride, c10::optional<int64_t> aiv) {
  const int ctas = cores_from(aiv);
  hfk_migrate_desc d;
  d.layers = static_cast<int>(srcKLayerPtrs.numel());
  check_ptr_table(srcKLayerPtrs, d.layers, "migrate_blocks(srcKLayerPtrs)", true);
  check_ptr_table(srcVLayerPtrs, d.layers, "migrate_blocks(srcVLayerPtrs)", true);
  check_ptr_table(dstKLayerPtrs, d.layers, "migrate_blocks(dstKLayerPtrs)", true);
  check_ptr_table(dstVLayerPtrs, d.layers, "migrate_blocks(dstVLayerPtrs)", true);
  d.ids_are_int64 = ids_are_int64(srcBlockIds, "migrate_blocks");
  TORCH_CHECK(ids_are_int64(dstBlockIds, "migrate_blocks") == d.ids_are_int64,
              "migrate_blocks: both id lists must have the same dtype");
  TORCH_CHECK(srcBlockIds.numel() == dstBlockIds.numel(), "migrate_blocks: id lists differ in length");
  TORCH_CHECK(srcBlockIds.is_cuda() && dstBlockIds.is_cuda(), "migrate_blocks: id lists must be device tensors");
  const auto dev = srcKLayerPtrs.device();
  TORCH_CHECK(srcVLayerPtrs.device() == dev && dstKLayerPtrs.device() == dev && dstVLayerPtrs.device() == dev &&
                  srcBlockIds.device() == dev && dstBlockIds.device() == dev,
              "migrate_blocks: pointer tables and id lists must live on the GPU that runs the kernel");
  d.src_k_layer_ptrs = reinterpret_cast<void *const *>(srcKLayerPtrs.data_ptr());
  d.src_v_layer_ptrs = reinterpret_cast<void *const *>(srcVLayerPtrs.data_ptr());
  d.dst_k_layer_ptrs = reinterpret_cast<void *const *>(dstKLayerPtrs.data_ptr());
  d.dst_v_layer_ptrs = reinterpret_cast<void *const *>(dstVLayerPtrs.data_ptr());
  d.src_block_ids = srcBlockIds.data_ptr();
  d.dst_block_ids = dstBlockIds.data_ptr();
  d.n_blocks = srcBlockIds.numel();
  d.block_bytes = blockBytes;
  d.src_block_stride = srcBlockStride.has_value() ? srcBlockStride.value() : blockBytes;
  d.dst_block_stride = dstBlockStride.has_value() ? dstBlockStride.value() : blockBytes;
  d.num_src_blocks = numSrcBlocks;
  d.num_dst_blocks = numDstBlocks;
  const c10::cuda::CUDAGuard guard(dev);
  check_rc(hfk_migrate_blocks(&d, ctas, at::cuda::getCurrentCUDAStream().stream()), "migrate_blocks");
}

// Reads and clears the device status word of the current device (bits HFK_DEV_*).
int64_t device_status() {
  unsigned int bits = 0;
  check_rc(hfk_device_status(&bits, at::cuda::getCurrentCUDAStream().stream()), "device_status");
  return static_cast<int64_t>(bits);
}

}  // namespace pciethrough

// The library is declared once and the schemas are added as fragments, as in the
// reference (pcieThrough/csrc/host/pcie_through_torchlib.cpp:4-5).
TORCH_LIBRARY(pcie_through, m) {}

TORCH_LIBRARY_FRAGMENT(pcie_through, m) {
  m.def("gather(Tensor gmEmbed, Tensor gmEmbedDst, Tensor gmIds, int? aiv=None) -> ()");
  m.def("multi_layer_block_transfer(Tensor deviceBlockCachePtrs, Tensor hostBlockCache, int? aiv=None) -> ()");
  m.def("fused_memcpy_multi_layer_block_transfer(Tensor deviceBlockCachePtrs, Tensor hostBlockCache, Tensor stagingBlockCache, int? aiv=None) -> ()");
  m.def("swap_out(Tensor kLayerPtrs, Tensor vLayerPtrs, Tensor hostPool, Tensor deviceBlockIds, Tensor hostSlotIds, int numDeviceBlocks, int? deviceBlockStride=None, int? aiv=None, int? mover=None, int? paceMBs=None) -> ()");
  m.def("swap_in(Tensor kLayerPtrs, Tensor vLayerPtrs, Tensor hostPool, Tensor deviceBlockIds, Tensor hostSlotIds, int numDeviceBlocks, int? deviceBlockStride=None, int? aiv=None, int? mover=None) -> ()");
  m.def("swap_out_copy_engine(Tensor kLayerPtrs, Tensor vLayerPtrs, Tensor hostPool, Tensor deviceBlockIds, Tensor hostSlotIds, int numDeviceBlocks, int? deviceBlockStride=None) -> ()");
  m.def("swap_in_copy_engine(Tensor kLayerPtrs, Tensor vLayerPtrs, Tensor hostPool, Tensor deviceBlockIds, Tensor hostSlotIds, int numDeviceBlocks, int? deviceBlockStride=None) -> ()");
  m.def("paged_gather(Tensor kLayerPtrs, Tensor vLayerPtrs, Tensor kOut, Tensor vOut, Tensor blockTables, Tensor seqLens, int blockSize, int numDeviceBlocks, int? deviceBlockStride=None, int? aiv=None, int? mover=None) -> ()");
  m.def("swap_out_staged(Tensor kLayerPtrs, Tensor vLayerPtrs, Tensor hostPool, Tensor deviceBlockIds, Tensor hostSlotIds, Tensor staging, int numDeviceBlocks, int? deviceBlockStride=None, int? aiv=None) -> ()");
  m.def("swap_in_staged(Tensor kLayerPtrs, Tensor vLayerPtrs, Tensor hostPool, Tensor deviceBlockIds, Tensor hostSlotIds, Tensor staging, int numDeviceBlocks, int? deviceBlockStride=None, int? aiv=None) -> ()");
  m.def("swap_in_relayout(Tensor layerPtrs, Tensor hostPool, Tensor deviceBlockIds, Tensor hostSlotIds, int numDeviceBlocks, int? deviceBlockStride=None, int? aiv=None) -> ()");
  m.def("swap_out_relayout(Tensor layerPtrs, Tensor hostPool, Tensor deviceBlockIds, Tensor hostSlotIds, int numDeviceBlocks, int? deviceBlockStride=None, int? aiv=None) -> ()");
  m.def("migrate_blocks(Tensor srcKLayerPtrs, Tensor srcVLayerPtrs, Tensor dstKLayerPtrs, Tensor dstVLayerPtrs, Tensor srcBlockIds, Tensor dstBlockIds, int blockBytes, int numSrcBlocks, int numDstBlocks, int? srcBlockStride=None, int? dstBlockStride=None, int? aiv=None) -> ()");
  m.def("device_status() -> int");
}

TORCH_LIBRARY_IMPL(pcie_through, CUDA, m) {
  m.impl("gather", TORCH_FN(pciethrough::gather));
  m.impl("multi_layer_block_transfer", TORCH_FN(pciethrough::multi_layer_block_transfer));
  m.impl("fused_memcpy_multi_layer_block_transfer", TORCH_FN(pciethrough::fused_memcpy_multi_layer_block_transfer));
  m.impl("swap_out", TORCH_FN(pciethrough::swap_out));
  m.impl("swap_in", TORCH_FN(pciethrough::swap_in));
  m.impl("paged_gather", TORCH_FN(pciethrough::paged_gather));
  m.impl("swap_out_staged", TORCH_FN(pciethrough::swap_out_staged));
  m.impl("swap_in_staged", TORCH_FN(pciethrough::swap_in_staged));
  m.impl("swap_in_relayout", TORCH_FN(pciethrough::swap_in_relayout));
  m.impl("swap_out_relayout", TORCH_FN(pciethrough::swap_out_relayout));
  m.impl("migrate_blocks", TORCH_FN(pciethrough::migrate_blocks));
}

// all-CPU argument lists dispatch here; there is no CPU implementation of any
// kernel, these two only enqueue copy-engine transfers
TORCH_LIBRARY_IMPL(pcie_through, CPU, m) {
  m.impl("swap_out_copy_engine", TORCH_FN(pciethrough::swap_out_copy_engine));
  m.impl("swap_in_copy_engine", TORCH_FN(pciethrough::swap_in_copy_engine));
}

TORCH_LIBRARY_IMPL(pcie_through, CompositeExplicitAutograd, m) {
  m.impl("device_status", TORCH_FN(pciethrough::device_status));
}
