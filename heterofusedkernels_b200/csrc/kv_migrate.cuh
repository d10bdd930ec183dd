// Block migration between two paged K/V caches: for every listed pair,
//   dst cache block dst_ids[i]  <-  src cache block src_ids[i],  every layer, K and V,
// in one launch.  The two caches may live on one GPU (a block copy inside a cache, or between
// two caches) or on two GPUs with peer access enabled: then one side of every copy crosses
// NVLink.  The kernel runs on whichever GPU it is launched on and uses plain 16-byte vector
// loads and stores only — no bulk (TMA) copy and no cluster feature ever touches the peer's
// memory — and the data lands directly in the destination cache.
//
// The reference has no counterpart: its transfers are host<->device only
// (pcieThrough/csrc/kernel/multi_layer_block_transfer_kernel.h:42-82); the pointer-table and
// id-list conventions are the ones of the swap kernels in kv_swap.cuh.
#pragma once

#include "common.cuh"
#include "kv_swap.cuh"  // load_id, checked_layer_ptr, kSwapIdTile

namespace hfk {

struct MigrateArgs {
  void *const *src_k_layer_ptrs;
  void *const *src_v_layer_ptrs;
  void *const *dst_k_layer_ptrs;
  void *const *dst_v_layer_ptrs;
  const void *src_block_ids;
  const void *dst_block_ids;
  int ids_are_int64;
  int layers;
  int64_t n_blocks;
  int64_t block_bytes;
  int64_t src_block_stride;
  int64_t dst_block_stride;
  int64_t num_src_blocks;
  int64_t num_dst_blocks;
};

__host__ __device__ inline size_t migrate_tables_bytes(int id_tile, int layers) {
  return (size_t)id_tile * 2 * sizeof(int64_t) + (size_t)layers * 4 * sizeof(void *);
}

// Shared memory: id_tile source offsets, id_tile destination offsets, then 4*layers pointers
// (source K, source V, destination K, destination V).  Work item = (block, layer, K|V), items
// strided over the grid; the whole CTA copies one chunk with kUnroll loads in flight per thread.
template <int kThreads, int kUnroll>
__global__ void __launch_bounds__(kThreads) kv_migrate_vector_kernel(MigrateArgs a, int id_tile) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  int64_t *src_off = reinterpret_cast<int64_t *>(smem_raw);
  int64_t *dst_off = src_off + id_tile;
  unsigned char **lp = reinterpret_cast<unsigned char **>(dst_off + id_tile);
  CtaStamp stamp;
  stamp.begin(kStampMigrate);
  for (int l = threadIdx.x; l < a.layers; l += kThreads) {
    lp[l] = checked_layer_ptr(a.src_k_layer_ptrs[l]);
    lp[a.layers + l] = checked_layer_ptr(a.src_v_layer_ptrs[l]);
    lp[2 * a.layers + l] = checked_layer_ptr(a.dst_k_layer_ptrs[l]);
    lp[3 * a.layers + l] = checked_layer_ptr(a.dst_v_layer_ptrs[l]);
  }
  const int per_block = 2 * a.layers;
  const int64_t n16 = a.block_bytes >> 4;
  for (int64_t tile0 = 0; tile0 < a.n_blocks; tile0 += id_tile) {
    const int tn = (int)min((int64_t)id_tile, a.n_blocks - tile0);
    __syncthreads();
    for (int i = threadIdx.x; i < tn; i += kThreads) {
      const int64_t s = load_id(a.src_block_ids, a.ids_are_int64, tile0 + i);
      const int64_t d = load_id(a.dst_block_ids, a.ids_are_int64, tile0 + i);
      const bool s_ok = s >= 0 && s < a.num_src_blocks;
      const bool d_ok = d >= 0 && d < a.num_dst_blocks;
      if (!s_ok || !d_ok) raise_status(HFK_DEV_BAD_DEVICE_BLOCK_ID);
      src_off[i] = (s_ok && d_ok) ? s * a.src_block_stride : -1;
      dst_off[i] = (s_ok && d_ok) ? d * a.dst_block_stride : -1;
    }
    __syncthreads();
    const int64_t items = (int64_t)tn * per_block;
    for (int64_t w = blockIdx.x; w < items; w += gridDim.x) {
      const int i = (int)(w / per_block);
      const int r = (int)(w - (int64_t)i * per_block);
      const int l = r >> 1, kv = r & 1;
      const int64_t so = src_off[i];
      const unsigned char *sb = lp[kv * a.layers + l];
      unsigned char *db = lp[(2 + kv) * a.layers + l];
      if (so < 0 || sb == nullptr || db == nullptr) continue;
      cta_copy16<kThreads, kUnroll>(reinterpret_cast<uint4 *>(db + dst_off[i]),
                                    reinterpret_cast<const uint4 *>(sb + so), n16);
    }
  }
  stamp.end();
}

}  // namespace hfk
