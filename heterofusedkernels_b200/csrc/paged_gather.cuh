// Paged gather: the pages a batch of sequences owns in the paged K/V cache are
// copied, for every layer and for K and V, into contiguous per-sequence token
// ranges of an output buffer — one launch.  HBM -> HBM, so the bound is HBM
// bandwidth (each byte is read once and written once).
//
// The reference's ancestor is the row gather Gather::MteCopy
// (pcieThrough/csrc/kernel/gather.h:79-134): dst[i,:] = table[ids[i],:] with
// row = one page.  What is added here is the block-table walk: ids come from a
// [num_seqs][max_blocks] table, the destination offset from the prefix sum of
// the sequence lengths, and the last page of a sequence is partial.
#pragma once

#include "common.cuh"
#include "kv_swap.cuh"  // load_id

namespace hfk {

struct GatherArgs {
  void *const *k_layer_ptrs;
  void *const *v_layer_ptrs;
  unsigned char *k_out;
  unsigned char *v_out;
  int64_t out_layer_stride;
  const void *block_tables;
  const void *seq_lens;
  int ids_are_int64;
  int layers;
  int num_seqs;     // sequences handled by this launch (<= HFK_MAX_SEQS)
  int seq_offset;   // index of the first of them in block_tables / seq_lens
  int64_t max_blocks_per_seq;
  int64_t block_table_stride;
  int64_t block_size;
  int64_t token_bytes;
  int64_t device_block_stride;
  int64_t num_device_blocks;
  int64_t total_tokens;
  int hints;    // L2 hints of the bulk mover (run_pump)
  int blocked;  // 0: CTA c takes units c, c+grid, ...; 1: CTA c takes one contiguous run of units
};

// Per-CTA shared-memory walk tables: exclusive prefix sums over the sequences of
// their page counts and of their token counts.
struct GatherTables {
  int64_t cu_tok[HFK_MAX_SEQS + 1];
  int32_t cu_blk[HFK_MAX_SEQS + 1];
};

// Warp 0 builds the prefix sums with shuffle scans, 32 sequences per step.
__device__ __forceinline__ void build_walk_tables(const GatherArgs &a, GatherTables *t) {
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  const int64_t cap = a.max_blocks_per_seq * a.block_size;
  // output offset of this launch's first sequence: the (clamped) lengths of all earlier ones
  int64_t carry_tok = 0;
  for (int base = 0; base < a.seq_offset; base += 32) {
    const int s = base + lane;
    int64_t len = s < a.seq_offset ? load_id(a.seq_lens, a.ids_are_int64, s) : 0;
    len = len < 0 ? 0 : (len > cap ? cap : len);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) len += __shfl_xor_sync(0xffffffffu, len, d);
    carry_tok += len;
  }
  int32_t carry_blk = 0;
  for (int base = 0; base < a.num_seqs; base += 32) {
    const int s = base + lane;
    int64_t len = s < a.num_seqs ? load_id(a.seq_lens, a.ids_are_int64, a.seq_offset + s) : 0;
    if (len < 0 || len > cap) {
      raise_status(HFK_DEV_BAD_SEQ_LEN);
      len = len < 0 ? 0 : cap;
    }
    int32_t nb = (int32_t)((len + a.block_size - 1) / a.block_size);
    int64_t inc_tok = len;
    int32_t inc_blk = nb;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int64_t vt = __shfl_up_sync(0xffffffffu, inc_tok, d);
      const int32_t vb = __shfl_up_sync(0xffffffffu, inc_blk, d);
      if (lane >= d) {
        inc_tok += vt;
        inc_blk += vb;
      }
    }
    if (s < a.num_seqs) {
      t->cu_tok[s] = carry_tok + inc_tok - len;
      t->cu_blk[s] = carry_blk + inc_blk - nb;
    }
    carry_tok += __shfl_sync(0xffffffffu, inc_tok, 31);
    carry_blk += __shfl_sync(0xffffffffu, inc_blk, 31);
  }
  if (lane == 0) {
    t->cu_tok[a.num_seqs] = carry_tok;
    t->cu_blk[a.num_seqs] = carry_blk;
  }
}

// Page p of the batch -> (source offset in a layer's cache, destination offset in
// a layer's output, bytes).  bytes == 0 when the page must be skipped.
struct PageCopy {
  int64_t src_off;
  int64_t dst_off;
  int64_t bytes;
};

__device__ __forceinline__ PageCopy locate_page(const GatherArgs &a, const GatherTables *t,
                                                int32_t p) {
  // s = number of entries of cu_blk[1..num_seqs] that are <= p
  int lo = 0, hi = a.num_seqs;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (t->cu_blk[mid + 1] <= p) lo = mid + 1; else hi = mid;
  }
  const int s = lo;
  const int64_t j = p - t->cu_blk[s];
  const int64_t len = t->cu_tok[s + 1] - t->cu_tok[s];
  const int64_t ntok = min(a.block_size, len - j * a.block_size);
  const int64_t blk =
      load_id(a.block_tables, a.ids_are_int64, (int64_t)(a.seq_offset + s) * a.block_table_stride + j);
  const int64_t tok0 = t->cu_tok[s] + j * a.block_size;
  PageCopy c;
  c.src_off = 0; c.dst_off = 0; c.bytes = 0;
  if (blk < 0 || blk >= a.num_device_blocks) {
    raise_status(HFK_DEV_BAD_DEVICE_BLOCK_ID);
    return c;
  }
  if (tok0 + ntok > a.total_tokens) {
    raise_status(HFK_DEV_BAD_SEQ_LEN);
    return c;
  }
  c.src_off = blk * a.device_block_stride;
  c.dst_off = tok0 * a.token_bytes;
  c.bytes = ntok * a.token_bytes;
  return c;
}

// ---- mover 1: whole-CTA vector loops --------------------------------------
// Item w = (layer-and-kv lk, page p), lk-major: consecutive CTAs write
// consecutive pages of one layer's output, i.e. the grid streams the output.
template <int kThreads, int kUnroll>
__global__ void __launch_bounds__(kThreads) paged_gather_vector_kernel(GatherArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  GatherTables *t = reinterpret_cast<GatherTables *>(smem_raw);
  build_walk_tables(a, t);
  __syncthreads();
  const int64_t pages = t->cu_blk[a.num_seqs];
  const int64_t items = pages * 2 * a.layers;
  for (int64_t w = blockIdx.x; w < items; w += gridDim.x) {
    const int lk = (int)(w / pages);
    const int32_t p = (int32_t)(w - (int64_t)lk * pages);
    const int l = lk >> 1, kv = lk & 1;
    const PageCopy c = locate_page(a, t, p);
    if (c.bytes == 0) continue;
    const unsigned char *base = checked_layer_ptr(kv ? a.v_layer_ptrs[l] : a.k_layer_ptrs[l]);
    if (base == nullptr) continue;
    const unsigned char *src = base + c.src_off;
    unsigned char *dst = (kv ? a.v_out : a.k_out) + (int64_t)l * a.out_layer_stride + c.dst_off;
    cta_copy16<kThreads, kUnroll>(reinterpret_cast<uint4 *>(dst),
                                  reinterpret_cast<const uint4 *>(src), c.bytes >> 4);
  }
}

// ---- mover 2: one warp per CTA pumping bulk copies -------------------------
template <int kLag>
__global__ void __launch_bounds__(32) paged_gather_bulk_kernel(GatherArgs a, int stage_bytes,
                                                               int n_stages) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char *stages = smem_raw;
  PumpSmem *ps = reinterpret_cast<PumpSmem *>(smem_raw + (size_t)stage_bytes * n_stages);
  GatherTables *t = reinterpret_cast<GatherTables *>(reinterpret_cast<unsigned char *>(ps) +
                                                     sizeof(PumpSmem));
  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) mbar_init(&ps->full[s], 1);
    mbar_fence_init();
  }
  build_walk_tables(a, t);
  __syncwarp();
  const int64_t pages = t->cu_blk[a.num_seqs];
  const int64_t page_bytes = a.block_size * a.token_bytes;
  const int pieces = (int)((page_bytes + stage_bytes - 1) / stage_bytes);
  const int64_t units = pages * 2 * a.layers * pieces;
  int64_t mine = units > blockIdx.x ? (units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  int64_t first_unit = 0;
  if (a.blocked) {
    const int64_t per = (units + gridDim.x - 1) / gridDim.x;
    first_unit = per * blockIdx.x;
    mine = first_unit < units ? min(per, units - first_unit) : 0;
  }
  uint32_t seq = 0;
  run_pump<kLag>(ps, stages, stage_bytes, n_stages, mine, seq, [&](int64_t k) {
    const int64_t g = a.blocked ? first_unit + k : blockIdx.x + k * (int64_t)gridDim.x;
    const int64_t w = g / pieces;
    const int piece = (int)(g - w * pieces);
    const int lk = (int)(w / pages);
    const int32_t p = (int32_t)(w - (int64_t)lk * pages);
    const int l = lk >> 1, kv = lk & 1;
    CopyDesc d;
    d.src = nullptr; d.dst = nullptr; d.bytes = 0;
    const PageCopy c = locate_page(a, t, p);
    const int64_t off = (int64_t)piece * stage_bytes;
    if (c.bytes <= off) return d;  // skipped page, or a piece beyond a partial page
    const unsigned char *base = checked_layer_ptr(kv ? a.v_layer_ptrs[l] : a.k_layer_ptrs[l]);
    if (base == nullptr) return d;  // null or misaligned layer base: reported, never dereferenced
    d.src = base + c.src_off + off;
    d.dst = (kv ? a.v_out : a.k_out) + (int64_t)l * a.out_layer_stride + c.dst_off + off;
    d.bytes = (uint32_t)min((int64_t)stage_bytes, c.bytes - off);
    return d;
  }, a.hints);
}

}  // namespace hfk
