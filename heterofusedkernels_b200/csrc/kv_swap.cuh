// Multi-block, all-layer K/V swap between the paged device cache and a pinned,
// device-mapped host pool: one launch covers every (block, layer, K|V) chunk.
//
// The single-block, host->device ancestor of this in the reference is
// KVTransfer::MultiLayerBlockTransfer (pcieThrough/csrc/kernel/
// multi_layer_block_transfer_kernel.h:42-82); the id-list convention follows
// gather's gmIds (pcieThrough/csrc/host/gather_torch.cpp:38,44-46) and the
// per-layer pointer table follows deviceBlockCachePtrs (pcieThrough/README.md:25-27).
#pragma once

#include "common.cuh"

namespace hfk {

struct SwapArgs {
  void *const *k_layer_ptrs;
  void *const *v_layer_ptrs;
  unsigned char *host_pool;
  const void *device_block_ids;
  const void *host_slot_ids;
  int ids_are_int64;
  int layers;
  int64_t n_blocks;
  int64_t block_bytes;
  int64_t device_block_stride;
  int64_t host_slot_stride;
  int64_t host_layer_stride;
  int64_t host_kv_stride;
  int64_t num_device_blocks;
  int64_t num_host_slots;
};

// Ids are staged kSwapIdTile at a time into shared memory, already converted to
// byte offsets and range-checked (-1 = skip), so the copy loops never touch the
// id lists in global memory again.
constexpr int kSwapIdTile = 1024;

__device__ __forceinline__ int64_t load_id(const void *ids, int is64, int64_t i) {
  return is64 ? reinterpret_cast<const int64_t *>(ids)[i]
              : (int64_t) reinterpret_cast<const int32_t *>(ids)[i];
}

// Shared-memory image common to both movers: id_tile device offsets, id_tile host offsets, then
// 2*layers pointers (K then V).  id_tile = min(n_blocks, kSwapIdTile), so a small launch has a
// small footprint and its CTAs fit next to a compute kernel's on an SM.
struct SwapTables {
  int64_t *dev_off;
  int64_t *host_off;
  unsigned char **layer_ptrs;
};
__host__ __device__ inline size_t swap_tables_bytes(int id_tile, int layers) {
  return (size_t)id_tile * 2 * sizeof(int64_t) + (size_t)layers * 2 * sizeof(void *);
}
__device__ __forceinline__ SwapTables carve_swap_tables(unsigned char *base, int id_tile) {
  SwapTables t;
  t.dev_off = reinterpret_cast<int64_t *>(base);
  t.host_off = t.dev_off + id_tile;
  t.layer_ptrs = reinterpret_cast<unsigned char **>(t.host_off + id_tile);
  return t;
}

// Copies the two pointer tables into shared memory.  An entry that is null or not 16-byte
// aligned is stored as null and reported; the copy loops skip every chunk of such a layer, so
// a bad table entry never becomes an address.
__device__ __forceinline__ unsigned char *checked_layer_ptr(void *p) {
  if (layer_ptr_ok(p)) return static_cast<unsigned char *>(p);
  raise_status(HFK_DEV_BAD_LAYER_PTR);
  return nullptr;
}
__device__ __forceinline__ void stage_layer_ptrs(const SwapArgs &a, unsigned char **lp) {
  for (int l = threadIdx.x; l < a.layers; l += blockDim.x) {
    lp[l] = checked_layer_ptr(a.k_layer_ptrs[l]);
    lp[a.layers + l] = checked_layer_ptr(a.v_layer_ptrs[l]);
  }
}

__device__ __forceinline__ void stage_ids(const SwapArgs &a, const SwapTables *t, int64_t tile0, int tn) {
  for (int i = threadIdx.x; i < tn; i += blockDim.x) {
    const int64_t d = load_id(a.device_block_ids, a.ids_are_int64, tile0 + i);
    // a null slot list means "slot = position in the list" (dense staging buffer)
    const int64_t h = a.host_slot_ids ? load_id(a.host_slot_ids, a.ids_are_int64, tile0 + i) : tile0 + i;
    const bool d_ok = d >= 0 && d < a.num_device_blocks;
    const bool h_ok = h >= 0 && h < a.num_host_slots;
    if (!d_ok) raise_status(HFK_DEV_BAD_DEVICE_BLOCK_ID);
    if (!h_ok) raise_status(HFK_DEV_BAD_HOST_SLOT_ID);
    const bool ok = d_ok && h_ok;
    t->dev_off[i] = ok ? d * a.device_block_stride : -1;
    t->host_off[i] = ok ? h * a.host_slot_stride : -1;
  }
}

// ---- mover 1: whole-CTA 16-byte vector loops ------------------------------
// Work item w = (block i, layer l, kv); CTA c takes items c, c+grid, ... so that
// with a block-major host pool the grid as a whole streams the host memory of a
// slot front to back.
template <bool kToHost, int kThreads, int kUnroll>
__global__ void __launch_bounds__(kThreads) kv_swap_vector_kernel(SwapArgs a, int id_tile) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const SwapTables tables = carve_swap_tables(smem_raw, id_tile);
  const SwapTables *t = &tables;
  unsigned char **lp = tables.layer_ptrs;
  CtaStamp stamp;
  stamp.begin(kStampSwapVector);
  stage_layer_ptrs(a, lp);
  const int per_block = 2 * a.layers;
  const int64_t n16 = a.block_bytes >> 4;
  for (int64_t tile0 = 0; tile0 < a.n_blocks; tile0 += id_tile) {
    const int tn = (int)min((int64_t)id_tile, a.n_blocks - tile0);
    __syncthreads();  // previous tile fully consumed
    stage_ids(a, t, tile0, tn);
    __syncthreads();
    const int64_t items = (int64_t)tn * per_block;
    for (int64_t w = blockIdx.x; w < items; w += gridDim.x) {
      const int i = (int)(w / per_block);
      const int r = (int)(w - (int64_t)i * per_block);
      const int l = r >> 1, kv = r & 1;
      const int64_t doff = t->dev_off[i];
      unsigned char *base = lp[kv * a.layers + l];
      if (doff < 0 || base == nullptr) continue;
      unsigned char *d = base + doff;
      unsigned char *h =
          a.host_pool + t->host_off[i] + (int64_t)l * a.host_layer_stride + kv * a.host_kv_stride;
      if (kToHost)
        cta_copy16<kThreads, kUnroll>(reinterpret_cast<uint4 *>(h),
                                      reinterpret_cast<const uint4 *>(d), n16);
      else
        cta_copy16<kThreads, kUnroll>(reinterpret_cast<uint4 *>(d),
                                      reinterpret_cast<const uint4 *>(h), n16);
    }
  }
  stamp.end();
}

// ---- mover 2: one warp per CTA pumping bulk copies -------------------------
// Unit = one piece (<= stage_bytes) of one chunk.  Shared memory: stages, then
// PumpSmem, then SwapTables, then the layer pointers.
// pace_ns_per_kib: 0, or the pacing of this CTA's stores (see run_pump); used for swap-outs.
template <bool kToHost, int kLag>
__global__ void __launch_bounds__(32) kv_swap_bulk_kernel(SwapArgs a, int stage_bytes,
                                                          int n_stages, int id_tile,
                                                          float pace_ns_per_kib) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char *stages = smem_raw;
  PumpSmem *ps = reinterpret_cast<PumpSmem *>(smem_raw + (size_t)stage_bytes * n_stages);
  const SwapTables tables = carve_swap_tables(reinterpret_cast<unsigned char *>(ps) + sizeof(PumpSmem), id_tile);
  const SwapTables *t = &tables;
  unsigned char **lp = tables.layer_ptrs;
  CtaStamp stamp;
  stamp.begin(kStampSwapBulk);
  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) mbar_init(&ps->full[s], 1);
    mbar_fence_init();
  }
  stage_layer_ptrs(a, lp);
  __syncwarp();
  const int per_block = 2 * a.layers;
  const int pieces = (int)((a.block_bytes + stage_bytes - 1) / stage_bytes);
  uint32_t seq = 0;
  const uint64_t pace_t0 = pace_ns_per_kib > 0.f ? global_timer_ns() : 0;
  uint64_t paced_bytes = 0;
  for (int64_t tile0 = 0; tile0 < a.n_blocks; tile0 += id_tile) {
    const int tn = (int)min((int64_t)id_tile, a.n_blocks - tile0);
    __syncwarp();
    stage_ids(a, t, tile0, tn);
    __syncwarp();
    const int64_t units = (int64_t)tn * per_block * pieces;
    // this CTA's units are g = blockIdx.x + k*gridDim.x
    const int64_t mine = units > blockIdx.x ? (units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const bool ok = run_pump<kLag>(ps, stages, stage_bytes, n_stages, mine, seq, [&](int64_t k) {
      const int64_t g = blockIdx.x + k * (int64_t)gridDim.x;
      const int64_t w = g / pieces;
      const int piece = (int)(g - w * pieces);
      const int i = (int)(w / per_block);
      const int r = (int)(w - (int64_t)i * per_block);
      const int l = r >> 1, kv = r & 1;
      CopyDesc d;
      d.src = nullptr; d.dst = nullptr; d.bytes = 0;
      const int64_t doff = t->dev_off[i];
      unsigned char *base = lp[kv * a.layers + l];
      if (doff < 0 || base == nullptr) return d;
      const int64_t off = (int64_t)piece * stage_bytes;
      unsigned char *dp = base + doff + off;
      unsigned char *hp = a.host_pool + t->host_off[i] + (int64_t)l * a.host_layer_stride +
                          kv * a.host_kv_stride + off;
      d.bytes = (uint32_t)min((int64_t)stage_bytes, a.block_bytes - off);
      d.src = kToHost ? dp : hp;
      d.dst = kToHost ? hp : dp;
      return d;
    }, 0, pace_ns_per_kib, pace_t0, &paced_bytes);
    if (!ok) break;  // a wait ran out: the barriers are out of step, issue nothing more
  }
  stamp.end();
}

}  // namespace hfk
