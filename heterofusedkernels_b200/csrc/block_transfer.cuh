// One KV block, all layers, host (or staging) -> device with the re-layout
//   src [block_size, layers, heads, head_dim]  ->  layers x [heads, block_size, head_dim].
// Restates MultiLayerBlockTransfer::blockTransposeCopy
// (pcieThrough/csrc/kernel/multi_layer_block_transfer_kernel.h:42-72): the
// reference reads n tokens x (L*H*D) contiguous bytes into on-chip memory and
// issues L*H strided stores of D elements per token (:59-69, src index
// (l*H+h)*D in the per-token image, dst index h*B*D + t*D).
//
// Here the source is walked linearly in 16-byte vectors, so the PCIe (or HBM)
// reads are one contiguous stream; each vector's destination is computed from
// its (t, l, h, d) coordinates.  A head_dim run is >= 128 bytes in every
// supported layout, so a warp's 512-byte read lands as at most four full,
// aligned runs in HBM: no staging through shared memory is needed.
#pragma once

#include "common.cuh"

namespace hfk {

struct TransferArgs {
  void *const *layer_ptrs;   // device array [layers]
  const unsigned char *src;  // [B, L, H, D] contiguous
  int64_t block_size, layers, heads;
  int64_t d16;               // head_dim*elt_size/16
};

template <int kThreads, int kUnroll>
__global__ void __launch_bounds__(kThreads) block_transfer_kernel(TransferArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char **lp = reinterpret_cast<unsigned char **>(smem_raw);
  // a null or misaligned layer base is reported and its vectors are skipped
  for (int l = threadIdx.x; l < a.layers; l += kThreads) {
    void *p = a.layer_ptrs[l];
    if (!layer_ptr_ok(p)) {
      raise_status(HFK_DEV_BAD_LAYER_PTR);
      p = nullptr;
    }
    lp[l] = static_cast<unsigned char *>(p);
  }
  __syncthreads();
  const int64_t total = a.block_size * a.layers * a.heads * a.d16;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  const uint4 *src = reinterpret_cast<const uint4 *>(a.src);
  auto dst_of = [&](int64_t v) -> uint4 * {
    const int64_t dv = v % a.d16;
    int64_t r = v / a.d16;
    const int64_t h = r % a.heads;
    r /= a.heads;
    const int64_t l = r % a.layers;
    const int64_t t = r / a.layers;
    if (lp[l] == nullptr) return nullptr;
    return reinterpret_cast<uint4 *>(lp[l]) + (h * a.block_size + t) * a.d16 + dv;
  };
  int64_t v0 = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  for (; v0 + (kUnroll - 1) * stride < total; v0 += kUnroll * stride) {
    uint4 x[kUnroll];
    uint4 *dp[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      dp[u] = dst_of(v0 + u * stride);
      if (dp[u]) x[u] = ld_stream16(src + v0 + u * stride);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (dp[u]) st_stream16(dp[u], x[u]);
  }
  for (; v0 < total; v0 += stride) {
    uint4 *dp = dst_of(v0);
    if (dp) st_stream16(dp, ld_stream16(src + v0));
  }
}

}  // namespace hfk
