// Row gather dst[i,:] = table[ids[i],:], the table being device memory or the
// device alias of a registered host range (then every row is a PCIe read).
// Restates Gather::MteCopy (pcieThrough/csrc/kernel/gather.h:35-134): the
// reference splits the ids evenly over cores and stages rows through on-chip
// memory; here small rows are taken four at a time by a warp (all loads of the
// four rows in flight before the first store) and large rows by a whole CTA.
#pragma once

#include "common.cuh"
#include "kv_swap.cuh"  // load_id

namespace hfk {

struct RowGatherArgs {
  const unsigned char *table;
  unsigned char *dst;
  const void *ids;
  int ids_are_int64;
  int64_t num_ids;
  int64_t row_bytes;
  int64_t num_rows;  // 0 = no range check
};

__device__ __forceinline__ bool row_id_ok(const RowGatherArgs &a, int64_t id) {
  if (id < 0 || (a.num_rows > 0 && id >= a.num_rows)) {
    raise_status(HFK_DEV_BAD_ROW_ID);
    return false;
  }
  return true;
}

constexpr int kRowsPerWarp = 4;

// rows of up to 1 KiB: two 16-byte vectors per lane per row, four rows per warp
template <int kThreads>
__global__ void __launch_bounds__(kThreads) row_gather_small_kernel(RowGatherArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * (kThreads / 32);
  const int n16 = (int)(a.row_bytes >> 4);  // <= 64
  for (int64_t i0 = warp * kRowsPerWarp; i0 < a.num_ids; i0 += n_warps * kRowsPerWarp) {
    uint4 v[kRowsPerWarp][2];
    bool ok[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      ok[r] = false;
      if (i0 + r < a.num_ids) {
        const int64_t id = load_id(a.ids, a.ids_are_int64, i0 + r);
        ok[r] = row_id_ok(a, id);
        if (ok[r]) {
          const uint4 *src = reinterpret_cast<const uint4 *>(a.table + id * a.row_bytes);
          if (lane < n16) v[r][0] = ld_stream16(src + lane);
          if (lane + 32 < n16) v[r][1] = ld_stream16(src + lane + 32);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      if (ok[r]) {
        uint4 *d = reinterpret_cast<uint4 *>(a.dst + (i0 + r) * a.row_bytes);
        if (lane < n16) st_stream16(d + lane, v[r][0]);
        if (lane + 32 < n16) st_stream16(d + lane + 32, v[r][1]);
      }
    }
  }
}

// rows above 1 KiB (multiple of 16 bytes): one row per CTA step
template <int kThreads, int kUnroll>
__global__ void __launch_bounds__(kThreads) row_gather_large_kernel(RowGatherArgs a) {
  const int64_t n16 = a.row_bytes >> 4;
  for (int64_t i = blockIdx.x; i < a.num_ids; i += gridDim.x) {
    const int64_t id = load_id(a.ids, a.ids_are_int64, i);
    if (!row_id_ok(a, id)) continue;
    cta_copy16<kThreads, kUnroll>(reinterpret_cast<uint4 *>(a.dst + i * a.row_bytes),
                                  reinterpret_cast<const uint4 *>(a.table + id * a.row_bytes), n16);
  }
}

// rows whose size or addresses are not multiples of 16 bytes: warp per row,
// 4-byte words when everything is 4-byte aligned, else bytes
template <int kThreads, typename Word>
__global__ void __launch_bounds__(kThreads) row_gather_words_kernel(RowGatherArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * (kThreads / 32);
  const int64_t nw = a.row_bytes / (int64_t)sizeof(Word);
  for (int64_t i = warp; i < a.num_ids; i += n_warps) {
    const int64_t id = load_id(a.ids, a.ids_are_int64, i);
    if (!row_id_ok(a, id)) continue;
    const Word *src = reinterpret_cast<const Word *>(a.table + id * a.row_bytes);
    Word *d = reinterpret_cast<Word *>(a.dst + i * a.row_bytes);
    for (int64_t c = lane; c < nw; c += 32) d[c] = src[c];
  }
}

}  // namespace hfk
