// Multi-block swap in the reference's own host format: a host slot holds one KV block
// token-major, [block_size, layers, heads, head_dim], and layer l of the device cache holds
// it head-major, [heads, block_size, head_dim] — the re-layout of
// MultiLayerBlockTransfer::blockTransposeCopy
// (pcieThrough/csrc/kernel/multi_layer_block_transfer_kernel.h:59-68: per-token source index
// (l*H+h)*D, destination index h*B*D + t*D), generalised to a list of blocks and to both
// directions.  The reference moves one block host->device per call
// (pcieThrough/csrc/host/multi_layer_block_transfer_torch.cpp:58-80).
//
// The walk is linear in HOST order in 16-byte vectors, so the PCIe side of either direction is
// one contiguous, fully coalesced stream per block; the HBM side sees head_dim runs (>= 16 B,
// 128-256 B in practice).
#pragma once

#include "common.cuh"
#include "kv_swap.cuh"  // load_id, kSwapIdTile

namespace hfk {

struct RelayoutArgs {
  void *const *layer_ptrs;  // device array [layers]: cache of layer l, [num_blocks][H][B][D]
  unsigned char *host_pool; // slot s at host_pool + s*host_slot_stride, [B][L][H][D]
  const void *device_block_ids;
  const void *host_slot_ids;
  int ids_are_int64;
  int layers;
  int64_t n_blocks;
  int64_t block_size, heads, d16;  // d16 = head_dim*elt_size/16
  int64_t device_block_stride;     // bytes between blocks in a layer's cache (>= H*B*D*elt)
  int64_t host_slot_stride;
  int64_t num_device_blocks;
  int64_t num_host_slots;
};

struct RelayoutTables {
  int64_t dev_off[kSwapIdTile];
  int64_t host_off[kSwapIdTile];
  // followed by `layers` pointers
};

template <bool kToHost, int kThreads, int kUnroll>
__global__ void __launch_bounds__(kThreads) kv_relayout_swap_kernel(RelayoutArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  RelayoutTables *t = reinterpret_cast<RelayoutTables *>(smem_raw);
  unsigned char **lp = reinterpret_cast<unsigned char **>(smem_raw + sizeof(RelayoutTables));
  for (int l = threadIdx.x; l < a.layers; l += kThreads)
    lp[l] = checked_layer_ptr(a.layer_ptrs[l]);  // null when the entry is unusable (reported)
  const int64_t per_block = a.block_size * a.layers * a.heads * a.d16;  // 16-byte vectors per block
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  // one 16-byte vector: v = (block i of the tile, offset r in host order)
  auto locate = [&](int64_t v, const uint4 *&host, uint4 *&dev) -> bool {
    const int i = (int)(v / per_block);
    const int64_t r = v - (int64_t)i * per_block;
    const int64_t doff = t->dev_off[i];
    if (doff < 0) return false;
    const int64_t dv = r % a.d16;
    int64_t q = r / a.d16;
    const int64_t h = q % a.heads;
    q /= a.heads;
    const int64_t l = q % a.layers;
    const int64_t tok = q / a.layers;
    if (lp[l] == nullptr) return false;
    host = reinterpret_cast<const uint4 *>(a.host_pool + t->host_off[i]) + r;
    dev = reinterpret_cast<uint4 *>(lp[l] + doff) + (h * a.block_size + tok) * a.d16 + dv;
    return true;
  };
  for (int64_t tile0 = 0; tile0 < a.n_blocks; tile0 += kSwapIdTile) {
    const int tn = (int)min((int64_t)kSwapIdTile, a.n_blocks - tile0);
    __syncthreads();
    for (int i = threadIdx.x; i < tn; i += kThreads) {
      const int64_t d = load_id(a.device_block_ids, a.ids_are_int64, tile0 + i);
      const int64_t h = load_id(a.host_slot_ids, a.ids_are_int64, tile0 + i);
      const bool d_ok = d >= 0 && d < a.num_device_blocks;
      const bool h_ok = h >= 0 && h < a.num_host_slots;
      if (!d_ok) raise_status(HFK_DEV_BAD_DEVICE_BLOCK_ID);
      if (!h_ok) raise_status(HFK_DEV_BAD_HOST_SLOT_ID);
      t->dev_off[i] = (d_ok && h_ok) ? d * a.device_block_stride : -1;
      t->host_off[i] = (d_ok && h_ok) ? h * a.host_slot_stride : -1;
    }
    __syncthreads();
    const int64_t total = (int64_t)tn * per_block;
    int64_t v0 = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    for (; v0 + (kUnroll - 1) * stride < total; v0 += kUnroll * stride) {
      uint4 x[kUnroll];
      const uint4 *hp[kUnroll];
      uint4 *dp[kUnroll];
      bool ok[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        ok[u] = locate(v0 + u * stride, hp[u], dp[u]);
        if (ok[u]) x[u] = ld_stream16(kToHost ? dp[u] : hp[u]);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (ok[u]) st_stream16(kToHost ? const_cast<uint4 *>(hp[u]) : dp[u], x[u]);
    }
    for (; v0 < total; v0 += stride) {
      const uint4 *hp;
      uint4 *dp;
      if (locate(v0, hp, dp)) {
        if (kToHost) st_stream16(const_cast<uint4 *>(hp), ld_stream16(dp));
        else st_stream16(dp, ld_stream16(hp));
      }
    }
  }
}

}  // namespace hfk
