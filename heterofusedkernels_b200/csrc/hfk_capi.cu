// C ABI of libhfk_b200.so: argument validation, launch planning and kernel
// launches.  The reference's counterpart is its host op layer
// (pcieThrough/csrc/host/gather_torch.cpp:30-54,
//  pcieThrough/csrc/host/multi_layer_block_transfer_torch.cpp:58-106) together
// with the tiling planner (pcieThrough/csrc/host/tiling/multi_layer_block_transfer.cpp:19-56);
// on CUDA the plan travels as kernel parameters, so nothing is uploaded per call.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>
#include <string>
#include <type_traits>

#include "block_transfer.cuh"
#include "common.cuh"
#include "host_util.h"
#include "kv_migrate.cuh"
#include "kv_swap.cuh"
#include "paged_gather.cuh"
#include "relayout_swap.cuh"
#include "row_gather.cuh"

namespace hfk {

thread_local std::string t_last_error;

int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  t_last_error = buf;
  return code;
}

int cuda_fail(cudaError_t e, const char *what) {
  return fail(HFK_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

// ---- status word ------------------------------------------------------------
// hfk_device_status() snapshots the word with an atomic exchange into one of a few slots (one
// per concurrent reader) and copies that slot back.
constexpr unsigned int kStatusSnapshots = 64;
__device__ unsigned int g_status_snapshot[kStatusSnapshots];
std::atomic<unsigned int> g_status_ticket{0};
__global__ void status_exchange_kernel(unsigned int slot) {
  g_status_snapshot[slot] = atomicExch(&g_status_word, 0u);
}

// ---- tuning state ----------------------------------------------------------
std::atomic<int> g_stage_bytes{0}, g_n_stages{0}, g_bulk_lag{0}, g_vec_threads{0}, g_vec_unroll{0};
std::atomic<int> g_gather_hints{-1}, g_gather_blocked{-1};
std::atomic<int> g_staged_lanes{0};
std::atomic<int> g_swap_out_pace_mbs{0};  // pacing of bulk swap-outs in MB/s, 0 = unpaced (hfk_set_swap_out_pace)
std::atomic<int> g_vec_smem_pad{0};  // extra dynamic shared memory of the vector swap kernels (see hfk_set_vector_smem_pad)

// ---- copy lanes of the staged mover -------------------------------------------
// The staged swap hands the link to the copy engines.  One stream executes its copies back to
// back with a gap after each; B200 has several copy engines per direction, so the slot copies
// are dealt round-robin to a few internal streams ("lanes") that fork from the caller's stream
// and join it again (events), which keeps the link busy across the gaps.  Lanes and events are
// created once per device on first use; a per-device mutex keeps two host threads from
// interleaving their fork/join sequences on the shared events.
constexpr int kMaxLanes = 4;
constexpr int kMaxDevicesLanes = 64;
struct CopyLanes {
  std::mutex mu;
  bool ready = false;
  cudaStream_t lane[kMaxLanes];
  cudaEvent_t fork;
  cudaEvent_t join[kMaxLanes];
};
static CopyLanes g_lanes[kMaxDevicesLanes];

static int lanes_for_current_device(CopyLanes **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevicesLanes)
    return fail(HFK_ERR_UNSUPPORTED, "staged swap: device ordinal %d beyond %d", dev, kMaxDevicesLanes);
  CopyLanes *l = &g_lanes[dev];
  std::lock_guard<std::mutex> g(l->mu);
  if (!l->ready) {
    for (int i = 0; i < kMaxLanes; ++i) {
      if ((e = cudaStreamCreateWithFlags(&l->lane[i], cudaStreamNonBlocking)) != cudaSuccess)
        return cuda_fail(e, "cudaStreamCreateWithFlags(copy lane)");
      if ((e = cudaEventCreateWithFlags(&l->join[i], cudaEventDisableTiming)) != cudaSuccess)
        return cuda_fail(e, "cudaEventCreateWithFlags(copy lane)");
    }
    if ((e = cudaEventCreateWithFlags(&l->fork, cudaEventDisableTiming)) != cudaSuccess)
      return cuda_fail(e, "cudaEventCreateWithFlags(copy lane)");
    l->ready = true;
  }
  *out = l;
  return HFK_OK;
}

constexpr int kMaxDynSmem = 227 * 1024;

// SM count of the current device (148 on B200), cached per device ordinal.
static int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int v = cached[dev].load();
  if (v > 0) return v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
  cached[dev] = v;
  return v;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct BulkPlan {
  int stage_bytes, n_stages, lag;
  size_t smem;
};
// Ring geometry of the bulk mover for a copy unit of `unit_bytes`, leaving
// `tables_bytes` of shared memory for the id / prefix tables.
static BulkPlan plan_bulk(int64_t unit_bytes, size_t tables_bytes, int def_stage_bytes, int def_stages,
                          int def_lag) {
  BulkPlan p;
  p.stage_bytes = g_stage_bytes.load() > 0 ? g_stage_bytes.load() : def_stage_bytes;
  if (unit_bytes < p.stage_bytes) p.stage_bytes = (int)((unit_bytes + 127) / 128 * 128);
  p.n_stages = g_n_stages.load() > 0 ? g_n_stages.load() : def_stages;
  const size_t fixed = sizeof(PumpSmem) + tables_bytes + 256;
  while (p.n_stages > 2 && (size_t)p.stage_bytes * p.n_stages + fixed > kMaxDynSmem) --p.n_stages;
  if (p.n_stages > 32) p.n_stages = 32;
  p.lag = g_bulk_lag.load() > 0 ? g_bulk_lag.load() : def_lag;
  if (p.lag > p.n_stages - 1) p.lag = p.n_stages - 1;  // at least one load in flight
  if (p.lag == 5) p.lag = 4;                            // compiled: 1, 2, 3, 4, 6, 8
  if (p.lag == 7) p.lag = 6;
  if (p.lag > kPumpLagMax) p.lag = kPumpLagMax;
  p.smem = (size_t)p.stage_bytes * p.n_stages + fixed;
  return p;
}

// Calls f(std::integral_constant<int, lag>) for the compiled lag values.
template <typename F>
static cudaError_t launch_by_lag(int lag, F f) {
  switch (lag) {
    case 1: return f(std::integral_constant<int, 1>{});
    case 2: return f(std::integral_constant<int, 2>{});
    case 3: return f(std::integral_constant<int, 3>{});
    case 4: return f(std::integral_constant<int, 4>{});
    case 6: return f(std::integral_constant<int, 6>{});
    case 8: return f(std::integral_constant<int, 8>{});
    default: return cudaErrorInvalidValue;
  }
}

template <typename K>
static cudaError_t allow_smem(K kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return cudaSuccess;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

// ---- swap ------------------------------------------------------------------
static int validate_swap(const hfk_swap_desc *d) {
  if (!d) return fail(HFK_ERR_INVALID_ARG, "swap: descriptor is null");
  if (!d->k_layer_ptrs || !d->v_layer_ptrs || !d->host_pool)
    return fail(HFK_ERR_INVALID_ARG, "swap: null pointer table or host pool");
  if (d->n_blocks < 0 || d->layers <= 0)
    return fail(HFK_ERR_INVALID_ARG, "swap: n_blocks=%lld layers=%d", (long long)d->n_blocks,
                d->layers);
  if (d->n_blocks > 0 && (!d->device_block_ids || !d->host_slot_ids))
    return fail(HFK_ERR_INVALID_ARG, "swap: null id list");
  if (d->block_bytes <= 0 || d->num_device_blocks <= 0 || d->num_host_slots <= 0)
    return fail(HFK_ERR_INVALID_ARG, "swap: block_bytes, num_device_blocks and num_host_slots must be positive");
  if (d->device_block_stride < d->block_bytes)
    return fail(HFK_ERR_INVALID_ARG, "swap: device_block_stride %lld < block_bytes %lld",
                (long long)d->device_block_stride, (long long)d->block_bytes);
  if ((d->block_bytes | d->device_block_stride | d->host_slot_stride | d->host_layer_stride |
       d->host_kv_stride) & 15)
    return fail(HFK_ERR_ALIGNMENT, "swap: block_bytes and all strides must be multiples of 16 bytes");
  if (!aligned16(d->host_pool)) return fail(HFK_ERR_ALIGNMENT, "swap: host pool is not 16-byte aligned");
  if (d->layers > 4096) return fail(HFK_ERR_TOO_LARGE, "swap: more than 4096 layers");
  if (d->host_slot_stride < 0 || d->host_layer_stride < 0 || d->host_kv_stride < 0)
    return fail(HFK_ERR_INVALID_ARG, "swap: negative host stride");
  // chunks of the pool must not overlap: the strides have to nest around the chunk (an expanded
  // or overlapping view of a pool would make distinct (slot, layer, K|V) chunks share bytes)
  if (!strides_nest(d->block_bytes, {d->host_kv_stride, 2}, {d->host_layer_stride, d->layers},
                    {d->host_slot_stride, d->num_host_slots}))
    return fail(HFK_ERR_INVALID_ARG,
                "swap: host strides (slot %lld, layer %lld, K|V %lld) let chunks of %lld bytes overlap",
                (long long)d->host_slot_stride, (long long)d->host_layer_stride,
                (long long)d->host_kv_stride, (long long)d->block_bytes);
  return HFK_OK;
}

static SwapArgs to_args(const hfk_swap_desc *d) {
  SwapArgs a;
  a.k_layer_ptrs = d->k_layer_ptrs;
  a.v_layer_ptrs = d->v_layer_ptrs;
  a.host_pool = static_cast<unsigned char *>(d->host_pool);
  a.device_block_ids = d->device_block_ids;
  a.host_slot_ids = d->host_slot_ids;
  a.ids_are_int64 = d->ids_are_int64;
  a.layers = d->layers;
  a.n_blocks = d->n_blocks;
  a.block_bytes = d->block_bytes;
  a.device_block_stride = d->device_block_stride;
  a.host_slot_stride = d->host_slot_stride;
  a.host_layer_stride = d->host_layer_stride;
  a.host_kv_stride = d->host_kv_stride;
  a.num_device_blocks = d->num_device_blocks;
  a.num_host_slots = d->num_host_slots;
  return a;
}

static int swap_id_tile(int64_t n_blocks, int cap = kSwapIdTile) {
  return (int)std::min<int64_t>(std::max<int64_t>(n_blocks, 1), cap);
}

template <bool kToHost, int kThreads, int kUnroll>
static cudaError_t launch_swap_vector(const SwapArgs &a, int ctas, size_t smem, cudaStream_t s) {
  auto k = kv_swap_vector_kernel<kToHost, kThreads, kUnroll>;
  cudaError_t e = allow_smem(k, smem);
  if (e != cudaSuccess) return e;
  k<<<ctas, kThreads, smem, s>>>(a, swap_id_tile(a.n_blocks));
  return cudaGetLastError();
}

template <bool kToHost>
static int swap_impl(const hfk_swap_desc *d, int mover, int ctas, cudaStream_t stream, int pace_mbs_arg = 0) {
  int rc = validate_swap(d);
  if (rc != HFK_OK) return rc;
  if (d->n_blocks == 0) return HFK_OK;
  const SwapArgs a = to_args(d);
  const int64_t items = d->n_blocks * 2 * d->layers;
  if (mover == HFK_MOVER_AUTO) mover = kToHost ? kDefaultMoverOut : kDefaultMoverIn;
  if (mover == HFK_MOVER_VECTOR) {
    const size_t tables = swap_tables_bytes(swap_id_tile(d->n_blocks), d->layers);
    if (ctas <= 0) ctas = kDefaultSwapCtasVector;
    if (ctas > items) ctas = (int)items;
    const int th = g_vec_threads.load(), un = g_vec_unroll.load();
    const size_t vsmem = tables + (size_t)g_vec_smem_pad.load();
    cudaError_t e;
    if (th == 0 || (th == 512 && un == 4)) e = launch_swap_vector<kToHost, 512, 4>(a, ctas, vsmem, stream);
    else if (th == 256 && un == 8) e = launch_swap_vector<kToHost, 256, 8>(a, ctas, vsmem, stream);
    else if (th == 256 && un == 4) e = launch_swap_vector<kToHost, 256, 4>(a, ctas, vsmem, stream);
    else if (th == 1024 && un == 2) e = launch_swap_vector<kToHost, 1024, 2>(a, ctas, vsmem, stream);
    else if (th == 128 && un == 8) e = launch_swap_vector<kToHost, 128, 8>(a, ctas, vsmem, stream);
    else return fail(HFK_ERR_UNSUPPORTED, "swap: vector geometry %dx%d is not compiled", th, un);
    if (e != cudaSuccess) return cuda_fail(e, "kv_swap_vector_kernel launch");
    return HFK_OK;
  }
  if (mover == HFK_MOVER_BULK) {
    // Two rings, chosen by the bytes of the launch.  A launch of a few MB (a layer-wise swap next to
    // a running compute kernel) gets many CTAs with a ring small enough to share an SM with a compute
    // CTA (a bf16 GEMM of cuBLAS leaves about 19 KB of shared memory and 22 K registers per SM): they
    // start within 10 us where a CTA that needs an SM of its own waits about 140 us for one to drain.
    // A large launch gets 4 CTAs with a 128 KiB ring each: the wait is nothing against 20 ms, and the
    // whole transfer costs 4 warps.
    const bool small = items * d->block_bytes < kAutoBulkMinBytes;
    const int id_tile = swap_id_tile(d->n_blocks, small ? kSwapSmallIdTile : kSwapIdTile);
    const size_t tables = swap_tables_bytes(id_tile, d->layers);
    const BulkPlan p = small ? plan_bulk(d->block_bytes, tables, kSwapSmallStageBytes, kSwapSmallStages, kSwapLag)
                             : plan_bulk(d->block_bytes, tables, kSwapStageBytes, kSwapStages, kSwapLag);
    if (ctas <= 0) ctas = small ? kDefaultSwapCtasBulkSmall : kDefaultSwapCtasBulk;
    const int64_t pieces = (d->block_bytes + p.stage_bytes - 1) / p.stage_bytes;
    if (ctas > items * pieces) ctas = (int)(items * pieces);
    // pacing (swap-out only): every CTA moves an equal share, so its stores are spaced for rate / ctas
    float pace_ns_per_kib = 0.f;
    const int pace_mbs = pace_mbs_arg > 0 ? pace_mbs_arg : g_swap_out_pace_mbs.load();
    if (kToHost && pace_mbs > 0) pace_ns_per_kib = 1024.0f * 1000.0f * (float)ctas / (float)pace_mbs;
    cudaError_t e = launch_by_lag(p.lag, [&](auto lag) {
      auto k = kv_swap_bulk_kernel<kToHost, decltype(lag)::value>;
      cudaError_t err = allow_smem(k, p.smem);
      if (err != cudaSuccess) return err;
      k<<<ctas, 32, p.smem, stream>>>(a, p.stage_bytes, p.n_stages, id_tile, pace_ns_per_kib);
      return cudaGetLastError();
    });
    if (e != cudaSuccess) return cuda_fail(e, "kv_swap_bulk_kernel launch");
    return HFK_OK;
  }
  return fail(HFK_ERR_INVALID_ARG, "swap: unknown mover %d", mover);
}

// ---- paged gather ----------------------------------------------------------
static int validate_gather(const hfk_paged_gather_desc *d) {
  if (!d) return fail(HFK_ERR_INVALID_ARG, "paged_gather: descriptor is null");
  if (!d->k_layer_ptrs || !d->v_layer_ptrs || !d->k_out || !d->v_out)
    return fail(HFK_ERR_INVALID_ARG, "paged_gather: null pointer table or output");
  if (d->layers <= 0 || d->num_seqs < 0 || d->block_size <= 0 || d->token_bytes <= 0 ||
      d->max_blocks_per_seq < 0 || d->num_device_blocks <= 0 || d->total_tokens < 0)
    return fail(HFK_ERR_INVALID_ARG, "paged_gather: non-positive geometry");
  if (d->num_seqs >= (int64_t)1 << 30) return fail(HFK_ERR_TOO_LARGE, "paged_gather: too many sequences");
  if (d->num_seqs > 0 && (!d->block_tables || !d->seq_lens))
    return fail(HFK_ERR_INVALID_ARG, "paged_gather: null block table or sequence lengths");
  if (d->block_table_stride < d->max_blocks_per_seq)
    return fail(HFK_ERR_INVALID_ARG, "paged_gather: block_table_stride < max_blocks_per_seq");
  if (d->device_block_stride < d->block_size * d->token_bytes)
    return fail(HFK_ERR_INVALID_ARG, "paged_gather: device_block_stride smaller than one block");
  if ((d->token_bytes | d->device_block_stride | d->out_layer_stride) & 15)
    return fail(HFK_ERR_ALIGNMENT, "paged_gather: token_bytes and strides must be multiples of 16 bytes");
  if (!aligned16(d->k_out) || !aligned16(d->v_out))
    return fail(HFK_ERR_ALIGNMENT, "paged_gather: outputs are not 16-byte aligned");
  if (d->num_seqs * d->max_blocks_per_seq >= (int64_t)1 << 31)
    return fail(HFK_ERR_TOO_LARGE, "paged_gather: more than 2^31 pages");
  if (d->layers > 1 && d->out_layer_stride < d->total_tokens * d->token_bytes)
    return fail(HFK_ERR_INVALID_ARG, "paged_gather: out_layer_stride smaller than one layer's output");
  return HFK_OK;
}

template <int kThreads, int kUnroll>
static cudaError_t launch_gather_vector(const GatherArgs &a, int ctas, cudaStream_t s) {
  auto k = paged_gather_vector_kernel<kThreads, kUnroll>;
  const size_t smem = sizeof(GatherTables);
  cudaError_t e = allow_smem(k, smem);
  if (e != cudaSuccess) return e;
  k<<<ctas, kThreads, smem, s>>>(a);
  return cudaGetLastError();
}

static int gather_launch(const GatherArgs &a, const hfk_paged_gather_desc *d, int mover, int ctas,
                         cudaStream_t stream);

static int gather_impl(const hfk_paged_gather_desc *d, int mover, int ctas, cudaStream_t stream) {
  int rc = validate_gather(d);
  if (rc != HFK_OK) return rc;
  if (d->num_seqs == 0 || d->max_blocks_per_seq == 0) return HFK_OK;
  GatherArgs a;
  a.k_layer_ptrs = d->k_layer_ptrs;
  a.v_layer_ptrs = d->v_layer_ptrs;
  a.k_out = static_cast<unsigned char *>(d->k_out);
  a.v_out = static_cast<unsigned char *>(d->v_out);
  a.out_layer_stride = d->out_layer_stride;
  a.block_tables = d->block_tables;
  a.seq_lens = d->seq_lens;
  a.ids_are_int64 = d->ids_are_int64;
  a.layers = d->layers;
  a.num_seqs = 0;
  a.seq_offset = 0;
  a.hints = g_gather_hints.load() >= 0 ? g_gather_hints.load() : kGatherHints;
  a.blocked = g_gather_blocked.load() >= 0 ? g_gather_blocked.load() : kGatherBlocked;
  a.max_blocks_per_seq = d->max_blocks_per_seq;
  a.block_table_stride = d->block_table_stride;
  a.block_size = d->block_size;
  a.token_bytes = d->token_bytes;
  a.device_block_stride = d->device_block_stride;
  a.num_device_blocks = d->num_device_blocks;
  a.total_tokens = d->total_tokens;
  if (mover == HFK_MOVER_AUTO) mover = kDefaultMoverGather;
  // The per-CTA walk tables hold HFK_MAX_SEQS sequences; larger batches go out as several launches,
  // each of which derives its output offset from the lengths of the sequences before it.
  for (int64_t first = 0; first < d->num_seqs; first += HFK_MAX_SEQS) {
    a.seq_offset = (int)first;
    a.num_seqs = (int)std::min<int64_t>(HFK_MAX_SEQS, d->num_seqs - first);
    rc = gather_launch(a, d, mover, ctas, stream);
    if (rc != HFK_OK) return rc;
  }
  return HFK_OK;
}

static int gather_launch(const GatherArgs &a, const hfk_paged_gather_desc *d, int mover, int ctas,
                         cudaStream_t stream) {
  if (mover == HFK_MOVER_VECTOR) {
    if (ctas <= 0) ctas = sm_count() * kGatherVectorCtasPerSm;
    const int th = g_vec_threads.load(), un = g_vec_unroll.load();
    cudaError_t e;
    if (th == 0 || (th == 256 && un == 8)) e = launch_gather_vector<256, 8>(a, ctas, stream);
    else if (th == 512 && un == 4) e = launch_gather_vector<512, 4>(a, ctas, stream);
    else if (th == 256 && un == 4) e = launch_gather_vector<256, 4>(a, ctas, stream);
    else if (th == 1024 && un == 2) e = launch_gather_vector<1024, 2>(a, ctas, stream);
    else if (th == 128 && un == 8) e = launch_gather_vector<128, 8>(a, ctas, stream);
    else return fail(HFK_ERR_UNSUPPORTED, "paged_gather: vector geometry %dx%d is not compiled", th, un);
    if (e != cudaSuccess) return cuda_fail(e, "paged_gather_vector_kernel launch");
    return HFK_OK;
  }
  if (mover == HFK_MOVER_BULK) {
    const BulkPlan p = plan_bulk(d->block_size * d->token_bytes, sizeof(GatherTables), kGatherStageBytes, kGatherStages,
                                kGatherLag);
    if (ctas <= 0) ctas = sm_count();
    cudaError_t e = launch_by_lag(p.lag, [&](auto lag) {
      auto k = paged_gather_bulk_kernel<decltype(lag)::value>;
      cudaError_t err = allow_smem(k, p.smem);
      if (err != cudaSuccess) return err;
      k<<<ctas, 32, p.smem, stream>>>(a, p.stage_bytes, p.n_stages);
      return cudaGetLastError();
    });
    if (e != cudaSuccess) return cuda_fail(e, "paged_gather_bulk_kernel launch");
    return HFK_OK;
  }
  return fail(HFK_ERR_INVALID_ARG, "paged_gather: unknown mover %d", mover);
}

// ---- staged swap through the copy engine ---------------------------------------
static int swap_staged_impl(const hfk_swap_desc *d, const void *slots_host, void *pool_host, void *staging,
                            size_t staging_bytes, int to_host, int ctas, cudaStream_t stream) {
  if (!d) return fail(HFK_ERR_INVALID_ARG, "swap_staged: descriptor is null");
  hfk_swap_desc probe = *d;
  probe.host_slot_ids = slots_host;  // only for the null check of the common validation
  probe.host_pool = pool_host;
  int rc = validate_swap(&probe);
  if (rc != HFK_OK) return rc;
  if (!staging) return fail(HFK_ERR_INVALID_ARG, "swap_staged: staging buffer is null");
  if (!aligned16(staging)) return fail(HFK_ERR_ALIGNMENT, "swap_staged: staging buffer is not 16-byte aligned");
  const int64_t slot_bytes = (int64_t)d->layers * 2 * d->block_bytes;
  // (a dimension of size 1 never advances, so a one-layer view may carry any layer stride)
  if (d->host_kv_stride != d->block_bytes || (d->layers > 1 && d->host_layer_stride != 2 * d->block_bytes))
    return fail(HFK_ERR_UNSUPPORTED,
                "swap_staged: the host pool must be slot-contiguous ([slot][layer][K|V][block])");
  if (d->host_slot_stride < slot_bytes)
    return fail(HFK_ERR_INVALID_ARG, "swap_staged: host_slot_stride %lld is smaller than one slot (%lld bytes)",
                (long long)d->host_slot_stride, (long long)slot_bytes);
  if ((int64_t)staging_bytes < slot_bytes)
    return fail(HFK_ERR_TOO_LARGE, "swap_staged: staging buffer of %zu bytes holds less than one slot (%lld bytes)",
                staging_bytes, (long long)slot_bytes);
  if (d->n_blocks == 0) return HFK_OK;
  auto slot_at = [&](int64_t i) -> int64_t {
    return d->ids_are_int64 ? static_cast<const int64_t *>(slots_host)[i]
                            : (int64_t) static_cast<const int32_t *>(slots_host)[i];
  };
  for (int64_t i = 0; i < d->n_blocks; ++i)
    if (slot_at(i) < 0 || slot_at(i) >= d->num_host_slots)
      return fail(HFK_ERR_INVALID_ARG, "swap_staged: host slot id %lld out of range at %lld",
                  (long long)slot_at(i), (long long)i);
  const int64_t per_round = (int64_t)(staging_bytes / (size_t)slot_bytes);
  const size_t id_width = d->ids_are_int64 ? 8 : 4;
  // The packing kernel is HBM to HBM.  A large call spreads it over the device (one CTA per SM, the
  // gather's ring); a small one (a layer-wise swap next to running compute) takes the small ring whose
  // CTAs share SMs with a compute kernel's instead of waiting for SMs to drain.
  const bool small_pack = d->n_blocks * slot_bytes < kAutoBulkMinBytes;
  if (ctas <= 0) ctas = small_pack ? kDefaultSwapCtasBulkSmall : sm_count();
  int n_lanes = g_staged_lanes.load() > 0 ? g_staged_lanes.load() : kDefaultStagedLanes;
  if (n_lanes > kMaxLanes) n_lanes = kMaxLanes;
  CopyLanes *lanes = nullptr;
  if (n_lanes > 1 && (rc = lanes_for_current_device(&lanes)) != HFK_OK) return rc;
  std::unique_lock<std::mutex> lanes_guard;
  if (lanes) lanes_guard = std::unique_lock<std::mutex>(lanes->mu);
  unsigned char *pool = static_cast<unsigned char *>(pool_host);
  unsigned char *stg = static_cast<unsigned char *>(staging);
  for (int64_t i0 = 0; i0 < d->n_blocks; i0 += per_round) {
    const int64_t n = std::min(per_round, d->n_blocks - i0);
    // the packing kernel sees the staging buffer as a dense pool: slot = position in this round
    hfk_swap_desc k = *d;
    k.host_pool = staging;
    k.device_block_ids = static_cast<const unsigned char *>(d->device_block_ids) + (size_t)i0 * id_width;
    k.host_slot_ids = nullptr;
    k.n_blocks = n;
    k.host_slot_stride = slot_bytes;
    k.num_host_slots = n;
    const SwapArgs a = to_args(&k);
    const int pack_tile = swap_id_tile(n, small_pack ? kSwapSmallIdTile : kSwapIdTile);
    const size_t tables = swap_tables_bytes(pack_tile, d->layers);
    const BulkPlan p = small_pack ? plan_bulk(d->block_bytes, tables, kSwapSmallStageBytes, kSwapSmallStages, kSwapLag)
                                  : plan_bulk(d->block_bytes, tables, kGatherStageBytes, kGatherStages, kGatherLag);
    auto pack = [&](bool to_staging) -> cudaError_t {
      return launch_by_lag(p.lag, [&](auto lag) {
        cudaError_t err;
        if (to_staging) {
          auto kern = kv_swap_bulk_kernel<true, decltype(lag)::value>;
          if ((err = allow_smem(kern, p.smem)) != cudaSuccess) return err;
          kern<<<ctas, 32, p.smem, stream>>>(a, p.stage_bytes, p.n_stages, pack_tile, 0.f);
        } else {
          auto kern = kv_swap_bulk_kernel<false, decltype(lag)::value>;
          if ((err = allow_smem(kern, p.smem)) != cudaSuccess) return err;
          kern<<<ctas, 32, p.smem, stream>>>(a, p.stage_bytes, p.n_stages, pack_tile, 0.f);
        }
        return cudaGetLastError();
      });
    };
    cudaError_t e;
    if (to_host && (e = pack(true)) != cudaSuccess) return cuda_fail(e, "staging pack kernel");
    // fork: the lanes start after everything enqueued on `stream` so far (the pack kernel, or
    // for a swap-in whatever the caller ordered before this call)
    if (lanes) {
      if ((e = cudaEventRecord(lanes->fork, stream)) != cudaSuccess) return cuda_fail(e, "cudaEventRecord(fork)");
      for (int q = 0; q < n_lanes; ++q)
        if ((e = cudaStreamWaitEvent(lanes->lane[q], lanes->fork, 0)) != cudaSuccess)
          return cuda_fail(e, "cudaStreamWaitEvent(fork)");
    }
    // one copy-engine transfer per run of consecutive slots; a long run is cut into pieces of at
    // most kStagedMaxCopyBytes so that every lane gets a share
    const bool dense_pool = d->host_slot_stride == slot_bytes;
    const int64_t max_run = std::max<int64_t>(1, kStagedMaxCopyBytes / slot_bytes);
    int copy_no = 0;
    for (int64_t i = 0; i < n;) {
      int64_t j = i + 1;
      if (dense_pool)
        while (j < n && j - i < max_run && slot_at(i0 + j) == slot_at(i0 + j - 1) + 1) ++j;
      unsigned char *h = pool + slot_at(i0 + i) * d->host_slot_stride;
      unsigned char *s = stg + i * slot_bytes;
      const size_t nb = (size_t)(j - i) * (size_t)slot_bytes;
      cudaStream_t cs = lanes ? lanes->lane[copy_no % n_lanes] : stream;
      e = to_host ? cudaMemcpyAsync(h, s, nb, cudaMemcpyDeviceToHost, cs)
                  : cudaMemcpyAsync(s, h, nb, cudaMemcpyHostToDevice, cs);
      if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(slot)");
      ++copy_no;
      i = j;
    }
    // join: `stream` continues after every lane has finished its copies
    if (lanes) {
      for (int q = 0; q < n_lanes; ++q) {
        if ((e = cudaEventRecord(lanes->join[q], lanes->lane[q])) != cudaSuccess)
          return cuda_fail(e, "cudaEventRecord(join)");
        if ((e = cudaStreamWaitEvent(stream, lanes->join[q], 0)) != cudaSuccess)
          return cuda_fail(e, "cudaStreamWaitEvent(join)");
      }
    }
    if (!to_host && (e = pack(false)) != cudaSuccess) return cuda_fail(e, "staging unpack kernel");
  }
  return HFK_OK;
}

// ---- re-layout swap ----------------------------------------------------------
template <bool kToHost>
static cudaError_t launch_relayout(const RelayoutArgs &a, int ctas, size_t smem, cudaStream_t s) {
  auto k = kv_relayout_swap_kernel<kToHost, 512, 4>;
  cudaError_t e = allow_smem(k, smem);
  if (e != cudaSuccess) return e;
  k<<<ctas, 512, smem, s>>>(a);
  return cudaGetLastError();
}

static int relayout_impl(const hfk_relayout_desc *d, int to_host, int ctas, cudaStream_t stream) {
  if (!d) return fail(HFK_ERR_INVALID_ARG, "swap_relayout: descriptor is null");
  if (!d->layer_ptrs || !d->host_pool)
    return fail(HFK_ERR_INVALID_ARG, "swap_relayout: null pointer table or host pool");
  if (d->n_blocks < 0 || d->layers <= 0 || d->block_size <= 0 || d->heads <= 0 || d->head_bytes <= 0 ||
      d->num_device_blocks <= 0 || d->num_host_slots <= 0)
    return fail(HFK_ERR_INVALID_ARG, "swap_relayout: non-positive geometry");
  if (d->n_blocks > 0 && (!d->device_block_ids || !d->host_slot_ids))
    return fail(HFK_ERR_INVALID_ARG, "swap_relayout: null id list");
  if ((d->head_bytes | d->device_block_stride | d->host_slot_stride) & 15)
    return fail(HFK_ERR_ALIGNMENT, "swap_relayout: head_bytes and strides must be multiples of 16 bytes");
  if (!aligned16(d->host_pool)) return fail(HFK_ERR_ALIGNMENT, "swap_relayout: host pool is not 16-byte aligned");
  if (d->device_block_stride < d->heads * d->block_size * d->head_bytes)
    return fail(HFK_ERR_INVALID_ARG, "swap_relayout: device_block_stride smaller than one block");
  if (d->host_slot_stride < d->block_size * d->layers * d->heads * d->head_bytes)
    return fail(HFK_ERR_INVALID_ARG, "swap_relayout: host_slot_stride smaller than one block");
  if (d->layers > 4096) return fail(HFK_ERR_TOO_LARGE, "swap_relayout: more than 4096 layers");
  if (d->n_blocks == 0) return HFK_OK;
  RelayoutArgs a;
  a.layer_ptrs = d->layer_ptrs;
  a.host_pool = static_cast<unsigned char *>(d->host_pool);
  a.device_block_ids = d->device_block_ids;
  a.host_slot_ids = d->host_slot_ids;
  a.ids_are_int64 = d->ids_are_int64;
  a.layers = d->layers;
  a.n_blocks = d->n_blocks;
  a.block_size = d->block_size;
  a.heads = d->heads;
  a.d16 = d->head_bytes / 16;
  a.device_block_stride = d->device_block_stride;
  a.host_slot_stride = d->host_slot_stride;
  a.num_device_blocks = d->num_device_blocks;
  a.num_host_slots = d->num_host_slots;
  if (ctas <= 0) ctas = kDefaultRelayoutCtas;
  const int64_t total = d->n_blocks * d->block_size * d->layers * d->heads * a.d16;
  const int64_t max_ctas = (total + 511) / 512;
  if (ctas > max_ctas) ctas = (int)max_ctas;
  const size_t smem = sizeof(RelayoutTables) + sizeof(void *) * (size_t)d->layers;
  cudaError_t e = to_host ? launch_relayout<true>(a, ctas, smem, stream)
                          : launch_relayout<false>(a, ctas, smem, stream);
  if (e != cudaSuccess) return cuda_fail(e, "kv_relayout_swap_kernel launch");
  return HFK_OK;
}

// ---- block migration between two caches ----------------------------------------
static int validate_migrate(const hfk_migrate_desc *d, const char *op) {
  if (!d) return fail(HFK_ERR_INVALID_ARG, "%s: descriptor is null", op);
  if (!d->src_k_layer_ptrs || !d->src_v_layer_ptrs || !d->dst_k_layer_ptrs || !d->dst_v_layer_ptrs)
    return fail(HFK_ERR_INVALID_ARG, "%s: null pointer table", op);
  if (d->n_blocks < 0 || d->layers <= 0 || d->block_bytes <= 0 || d->num_src_blocks <= 0 || d->num_dst_blocks <= 0)
    return fail(HFK_ERR_INVALID_ARG, "%s: non-positive geometry", op);
  if (d->n_blocks > 0 && (!d->src_block_ids || !d->dst_block_ids))
    return fail(HFK_ERR_INVALID_ARG, "%s: null id list", op);
  if (d->src_block_stride < d->block_bytes || d->dst_block_stride < d->block_bytes)
    return fail(HFK_ERR_INVALID_ARG, "%s: block stride smaller than block_bytes", op);
  if ((d->block_bytes | d->src_block_stride | d->dst_block_stride) & 15)
    return fail(HFK_ERR_ALIGNMENT, "%s: block_bytes and strides must be multiples of 16 bytes", op);
  if (d->layers > 2048) return fail(HFK_ERR_TOO_LARGE, "%s: more than 2048 layers", op);
  return HFK_OK;
}

static int migrate_impl(const hfk_migrate_desc *d, int ctas, cudaStream_t stream) {
  int rc = validate_migrate(d, "migrate_blocks");
  if (rc != HFK_OK) return rc;
  if (d->n_blocks == 0) return HFK_OK;
  MigrateArgs a;
  a.src_k_layer_ptrs = d->src_k_layer_ptrs;
  a.src_v_layer_ptrs = d->src_v_layer_ptrs;
  a.dst_k_layer_ptrs = d->dst_k_layer_ptrs;
  a.dst_v_layer_ptrs = d->dst_v_layer_ptrs;
  a.src_block_ids = d->src_block_ids;
  a.dst_block_ids = d->dst_block_ids;
  a.ids_are_int64 = d->ids_are_int64;
  a.layers = d->layers;
  a.n_blocks = d->n_blocks;
  a.block_bytes = d->block_bytes;
  a.src_block_stride = d->src_block_stride;
  a.dst_block_stride = d->dst_block_stride;
  a.num_src_blocks = d->num_src_blocks;
  a.num_dst_blocks = d->num_dst_blocks;
  const int tile = swap_id_tile(d->n_blocks);
  const size_t smem = migrate_tables_bytes(tile, d->layers);
  const int64_t items = d->n_blocks * 2 * d->layers;
  if (ctas <= 0) ctas = sm_count() * kMigrateCtasPerSm;
  if (ctas > items) ctas = (int)items;
  auto k = kv_migrate_vector_kernel<512, 4>;
  cudaError_t e = allow_smem(k, smem);
  if (e != cudaSuccess) return cuda_fail(e, "kv_migrate_vector_kernel attribute");
  k<<<ctas, 512, smem, stream>>>(a, tile);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "kv_migrate_vector_kernel launch");
  return HFK_OK;
}

// ---- Group R ---------------------------------------------------------------
static int row_gather_impl(const void *table, void *dst, const void *ids, int ids64, size_t num_ids,
                           size_t row_bytes, size_t num_rows, int ctas, cudaStream_t stream) {
  if (!table || !dst || (!ids && num_ids))
    return fail(HFK_ERR_INVALID_ARG, "gather: null table, destination or id list");
  if (row_bytes == 0) return fail(HFK_ERR_INVALID_ARG, "gather: row_bytes is 0");
  if (num_ids == 0) return HFK_OK;
  if (ctas <= 0) ctas = kDefaultRowGatherCtas;
  // the reference clamps the core count to the number of ids (gather_torch.cpp:48)
  if ((size_t)ctas > num_ids) ctas = (int)num_ids;
  RowGatherArgs a;
  a.table = static_cast<const unsigned char *>(table);
  a.dst = static_cast<unsigned char *>(dst);
  a.ids = ids;
  a.ids_are_int64 = ids64;
  a.num_ids = (int64_t)num_ids;
  a.row_bytes = (int64_t)row_bytes;
  a.num_rows = (int64_t)num_rows;
  const bool vec = (row_bytes & 15) == 0 && aligned16(table) && aligned16(dst);
  if (vec && row_bytes <= 1024) {
    row_gather_small_kernel<256><<<ctas, 256, 0, stream>>>(a);
  } else if (vec) {
    row_gather_large_kernel<512, 4><<<ctas, 512, 0, stream>>>(a);
  } else if ((row_bytes & 3) == 0 && ((uintptr_t)table & 3) == 0 && ((uintptr_t)dst & 3) == 0) {
    row_gather_words_kernel<256, uint32_t><<<ctas, 256, 0, stream>>>(a);
  } else {
    row_gather_words_kernel<256, unsigned char><<<ctas, 256, 0, stream>>>(a);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "row gather launch");
  return HFK_OK;
}

// Every argument check of the block transfer; nothing is enqueued before it passes.
static int validate_transfer(void *const *layer_ptrs, const void *src, int64_t B, int64_t L, int64_t H,
                             int64_t D, int64_t elt) {
  if (!layer_ptrs || !src)
    return fail(HFK_ERR_INVALID_ARG, "multi_layer_block_transfer: null pointer table or source block");
  if (B <= 0 || L <= 0 || H <= 0 || D <= 0 || elt <= 0)
    return fail(HFK_ERR_INVALID_ARG, "multi_layer_block_transfer: non-positive geometry");
  if ((D * elt) & 15)
    return fail(HFK_ERR_ALIGNMENT,
                "multi_layer_block_transfer: head_dim*elt_size=%lld is not a multiple of 16 bytes",
                (long long)(D * elt));
  if (!aligned16(src)) return fail(HFK_ERR_ALIGNMENT, "multi_layer_block_transfer: source is not 16-byte aligned");
  if (L > 4096) return fail(HFK_ERR_TOO_LARGE, "multi_layer_block_transfer: more than 4096 layers");
  return HFK_OK;
}

static int transfer_impl(void *const *layer_ptrs, const void *src, int64_t B, int64_t L, int64_t H,
                         int64_t D, int64_t elt, int ctas, cudaStream_t stream) {
  const int rc = validate_transfer(layer_ptrs, src, B, L, H, D, elt);
  if (rc != HFK_OK) return rc;
  TransferArgs a;
  a.layer_ptrs = layer_ptrs;
  a.src = static_cast<const unsigned char *>(src);
  a.block_size = B;
  a.layers = L;
  a.heads = H;
  a.d16 = D * elt / 16;
  if (ctas <= 0) ctas = kDefaultTransferCtas;
  const int64_t total = B * L * H * a.d16;
  const int64_t max_ctas = (total + 511) / 512;
  if (ctas > max_ctas) ctas = (int)max_ctas;
  block_transfer_kernel<512, 4><<<ctas, 512, (size_t)L * sizeof(void *), stream>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "block_transfer_kernel launch");
  return HFK_OK;
}

}  // namespace hfk

using namespace hfk;

extern "C" {

const char *hfk_strerror(int code) {
  switch (code) {
    case HFK_OK: return "ok";
    case HFK_ERR_INVALID_ARG: return "invalid argument";
    case HFK_ERR_ALIGNMENT: return "address or size is not a multiple of 16 bytes";
    case HFK_ERR_NOT_REGISTERED: return "host pointer is not inside a registered range";
    case HFK_ERR_CUDA: return "CUDA runtime error";
    case HFK_ERR_TOO_LARGE: return "size beyond the supported maximum";
    case HFK_ERR_NO_MEMORY: return "host allocation or registration failed";
    case HFK_ERR_UNSUPPORTED: return "unsupported combination";
    default: return "unknown error";
  }
}

const char *hfk_last_error_message(void) { return t_last_error.c_str(); }
const char *hfk_version(void) { return "0.1.0"; }

int hfk_device_status(unsigned int *status_bits, hfk_stream_t stream) {
  if (!status_bits) return fail(HFK_ERR_INVALID_ARG, "device_status: null output");
  // read and clear in ONE atomic exchange on the device, so a bit raised by a kernel on another
  // stream is either in this snapshot or stays for the next read, never lost in between
  const unsigned int slot = g_status_ticket.fetch_add(1) % kStatusSnapshots;
  status_exchange_kernel<<<1, 1, 0, stream>>>(slot);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "status_exchange_kernel launch");
  unsigned int v = 0;
  e = cudaMemcpyFromSymbolAsync(&v, g_status_snapshot, sizeof(v), slot * sizeof(unsigned int),
                                cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyFromSymbolAsync(status)");
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
  *status_bits = v;
  return HFK_OK;
}

int hfk_selftest_wait_timeout(unsigned int limit_us, hfk_stream_t stream) {
  if (limit_us == 0 || limit_us > 1000000u)
    return fail(HFK_ERR_INVALID_ARG, "selftest_wait_timeout: limit must be 1..1000000 microseconds");
  wait_timeout_selftest_kernel<<<1, 32, 0, stream>>>((uint64_t)limit_us * 1000ull);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "wait_timeout_selftest_kernel launch");
  return HFK_OK;
}

int hfk_set_gather_tuning(int l2_hints, int blocked) {
  if (l2_hints < -1 || l2_hints > 3 || blocked < -1 || blocked > 1)
    return fail(HFK_ERR_INVALID_ARG, "gather tuning: l2_hints -1..3, blocked -1..1");
  g_gather_hints = l2_hints;
  g_gather_blocked = blocked;
  return HFK_OK;
}

int hfk_set_bulk_lag(int lag) {
  if (lag < 0 || lag > kPumpLagMax)
    return fail(HFK_ERR_INVALID_ARG, "bulk lag: 0 (default) .. %d", kPumpLagMax);
  g_bulk_lag = lag;
  return HFK_OK;
}

int hfk_set_bulk_geometry(int stage_bytes, int n_stages) {
  if (stage_bytes < 0 || n_stages < 0 || (stage_bytes & 127) || n_stages > 32 ||
      (n_stages > 0 && n_stages < 2))
    return fail(HFK_ERR_INVALID_ARG, "bulk geometry: stage_bytes %% 128 == 0, 2 <= n_stages <= 32");
  if ((size_t)stage_bytes * (n_stages > 0 ? n_stages : 2) > (size_t)kMaxDynSmem - 20480)
    return fail(HFK_ERR_TOO_LARGE, "bulk geometry: ring does not fit shared memory");
  g_stage_bytes = stage_bytes;
  g_n_stages = n_stages;
  return HFK_OK;
}

int hfk_set_vector_geometry(int threads, int unroll) {
  const bool compiled = (threads == 0 && unroll == 0) || (threads == 512 && unroll == 4) ||
                        (threads == 256 && unroll == 8) || (threads == 256 && unroll == 4) ||
                        (threads == 1024 && unroll == 2) || (threads == 128 && unroll == 8);
  if (!compiled)
    return fail(HFK_ERR_UNSUPPORTED,
                "vector geometry %dx%d is not compiled (512x4, 256x8, 256x4, 1024x2, 128x8; 0x0 = default)",
                threads, unroll);
  g_vec_threads = threads;
  g_vec_unroll = unroll;
  return HFK_OK;
}

int hfk_swap_out(const hfk_swap_desc *desc, int mover, int ctas, hfk_stream_t stream) {
  return swap_impl<true>(desc, mover, ctas, stream);
}
int hfk_swap_out_paced(const hfk_swap_desc *desc, int mover, int ctas, int megabytes_per_second,
                       hfk_stream_t stream) {
  if (megabytes_per_second < 0 || megabytes_per_second > 1000000)
    return fail(HFK_ERR_INVALID_ARG, "swap_out_paced: pace 0 (unpaced) .. 1000000 MB/s");
  if (megabytes_per_second > 0 && mover == HFK_MOVER_VECTOR)
    return fail(HFK_ERR_UNSUPPORTED, "swap_out_paced: only the bulk mover can be paced");
  return swap_impl<true>(desc, mover, ctas, stream, megabytes_per_second);
}
int hfk_swap_in(const hfk_swap_desc *desc, int mover, int ctas, hfk_stream_t stream) {
  return swap_impl<false>(desc, mover, ctas, stream);
}

int hfk_swap_copy_engine(const hfk_swap_desc *d, int to_host, hfk_stream_t stream) {
  int rc = validate_swap(d);
  if (rc != HFK_OK) return rc;
  // Every array of the descriptor is a host array here: the addresses are
  // formed on the CPU and each chunk becomes one copy-engine transfer.
  for (int64_t i = 0; i < d->n_blocks; ++i) {
    const int64_t dev = d->ids_are_int64 ? static_cast<const int64_t *>(d->device_block_ids)[i]
                                         : static_cast<const int32_t *>(d->device_block_ids)[i];
    const int64_t slot = d->ids_are_int64 ? static_cast<const int64_t *>(d->host_slot_ids)[i]
                                          : static_cast<const int32_t *>(d->host_slot_ids)[i];
    if (dev < 0 || dev >= d->num_device_blocks)
      return fail(HFK_ERR_INVALID_ARG, "swap_copy_engine: device block id %lld out of range at %lld",
                  (long long)dev, (long long)i);
    if (slot < 0 || slot >= d->num_host_slots)
      return fail(HFK_ERR_INVALID_ARG, "swap_copy_engine: host slot id %lld out of range at %lld",
                  (long long)slot, (long long)i);
  }
  for (int64_t i = 0; i < d->n_blocks; ++i) {
    const int64_t dev = d->ids_are_int64 ? static_cast<const int64_t *>(d->device_block_ids)[i]
                                         : static_cast<const int32_t *>(d->device_block_ids)[i];
    const int64_t slot = d->ids_are_int64 ? static_cast<const int64_t *>(d->host_slot_ids)[i]
                                          : static_cast<const int32_t *>(d->host_slot_ids)[i];
    for (int l = 0; l < d->layers; ++l) {
      for (int kv = 0; kv < 2; ++kv) {
        unsigned char *dp = static_cast<unsigned char *>(kv ? d->v_layer_ptrs[l] : d->k_layer_ptrs[l]) +
                            dev * d->device_block_stride;
        unsigned char *hp = static_cast<unsigned char *>(d->host_pool) + slot * d->host_slot_stride +
                            (int64_t)l * d->host_layer_stride + kv * d->host_kv_stride;
        cudaError_t e = to_host ? cudaMemcpyAsync(hp, dp, (size_t)d->block_bytes, cudaMemcpyDeviceToHost, stream)
                                : cudaMemcpyAsync(dp, hp, (size_t)d->block_bytes, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(chunk)");
      }
    }
  }
  return HFK_OK;
}

int hfk_swap_staged(const hfk_swap_desc *desc, const void *host_slot_ids_host, void *host_pool_host,
                    void *staging, size_t staging_bytes, int to_host, int ctas, hfk_stream_t stream) {
  return swap_staged_impl(desc, host_slot_ids_host, host_pool_host, staging, staging_bytes, to_host, ctas,
                          stream);
}

int hfk_swap_relayout(const hfk_relayout_desc *desc, int to_host, int ctas, hfk_stream_t stream) {
  return relayout_impl(desc, to_host, ctas, stream);
}

int hfk_paged_gather(const hfk_paged_gather_desc *desc, int mover, int ctas, hfk_stream_t stream) {
  return gather_impl(desc, mover, ctas, stream);
}

int hfk_gather(const void *table, void *dst, const void *ids, int ids_are_int64, size_t num_ids,
               size_t row_bytes, size_t num_rows, int ctas, hfk_stream_t stream) {
  return row_gather_impl(table, dst, ids, ids_are_int64, num_ids, row_bytes, num_rows, ctas, stream);
}

int hfk_multi_layer_block_transfer(void *const *device_layer_ptrs, const void *src_block,
                                   int64_t block_size, int64_t layers, int64_t heads,
                                   int64_t head_dim, int64_t elt_size, int ctas,
                                   hfk_stream_t stream) {
  return transfer_impl(device_layer_ptrs, src_block, block_size, layers, heads, head_dim, elt_size,
                       ctas, stream);
}

int hfk_fused_memcpy_multi_layer_block_transfer(void *const *device_layer_ptrs,
                                                const void *host_block, void *staging,
                                                int64_t block_size, int64_t layers, int64_t heads,
                                                int64_t head_dim, int64_t elt_size, int ctas,
                                                hfk_stream_t stream) {
  if (!host_block || !staging)
    return fail(HFK_ERR_INVALID_ARG, "fused_memcpy_multi_layer_block_transfer: null host block or staging");
  if (block_size <= 0 || layers <= 0 || heads <= 0 || head_dim <= 0 || elt_size <= 0)
    return fail(HFK_ERR_INVALID_ARG, "fused_memcpy_multi_layer_block_transfer: non-positive geometry");
  const size_t bytes = (size_t)block_size * layers * heads * head_dim * elt_size;
  // all checks first: an error return leaves nothing in the stream and the staging bytes untouched
  const int rc = validate_transfer(device_layer_ptrs, staging, block_size, layers, heads, head_dim, elt_size);
  if (rc != HFK_OK) return rc;
  // stage 1 on the copy engine (multi_layer_block_transfer_torch.cpp:97-100) ...
  cudaError_t e = cudaMemcpyAsync(staging, host_block, bytes, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(staging)");
  // ... stage 2: the same kernel, reading the staging buffer (:105)
  return transfer_impl(device_layer_ptrs, staging, block_size, layers, heads, head_dim, elt_size,
                       ctas, stream);
}

int hfk_migrate_blocks(const hfk_migrate_desc *desc, int ctas, hfk_stream_t stream) {
  return migrate_impl(desc, ctas, stream);
}

int hfk_migrate_blocks_copy_engine(const hfk_migrate_desc *d, int src_device, int dst_device,
                                   hfk_stream_t stream) {
  int rc = validate_migrate(d, "migrate_blocks_copy_engine");
  if (rc != HFK_OK) return rc;
  auto id_at = [&](const void *ids, int64_t i) -> int64_t {
    return d->ids_are_int64 ? static_cast<const int64_t *>(ids)[i] : (int64_t) static_cast<const int32_t *>(ids)[i];
  };
  // every array of the descriptor is a HOST array here; the ids are checked before anything is enqueued
  for (int64_t i = 0; i < d->n_blocks; ++i) {
    const int64_t s = id_at(d->src_block_ids, i), t = id_at(d->dst_block_ids, i);
    if (s < 0 || s >= d->num_src_blocks || t < 0 || t >= d->num_dst_blocks)
      return fail(HFK_ERR_INVALID_ARG, "migrate_blocks_copy_engine: block id pair (%lld, %lld) out of range at %lld",
                  (long long)s, (long long)t, (long long)i);
  }
  for (int l = 0; l < d->layers; ++l)
    if (!layer_ptr_ok(d->src_k_layer_ptrs[l]) || !layer_ptr_ok(d->src_v_layer_ptrs[l]) ||
        !layer_ptr_ok(d->dst_k_layer_ptrs[l]) || !layer_ptr_ok(d->dst_v_layer_ptrs[l]))
      return fail(HFK_ERR_ALIGNMENT, "migrate_blocks_copy_engine: layer %d has a null or misaligned base", l);
  for (int64_t i = 0; i < d->n_blocks; ++i) {
    const int64_t s = id_at(d->src_block_ids, i), t = id_at(d->dst_block_ids, i);
    for (int l = 0; l < d->layers; ++l)
      for (int kv = 0; kv < 2; ++kv) {
        const unsigned char *sp = static_cast<const unsigned char *>(kv ? d->src_v_layer_ptrs[l] : d->src_k_layer_ptrs[l]) +
                                  s * d->src_block_stride;
        unsigned char *dp = static_cast<unsigned char *>(kv ? d->dst_v_layer_ptrs[l] : d->dst_k_layer_ptrs[l]) +
                            t * d->dst_block_stride;
        cudaError_t e = src_device == dst_device
                            ? cudaMemcpyAsync(dp, sp, (size_t)d->block_bytes, cudaMemcpyDeviceToDevice, stream)
                            : cudaMemcpyPeerAsync(dp, dst_device, sp, src_device, (size_t)d->block_bytes, stream);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyPeerAsync(chunk)");
      }
  }
  return HFK_OK;
}

int hfk_enable_peer_access(int peer_device) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (peer_device == dev) return HFK_OK;
  int can = 0;
  e = cudaDeviceCanAccessPeer(&can, dev, peer_device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceCanAccessPeer");
  if (!can) return fail(HFK_ERR_UNSUPPORTED, "device %d cannot access device %d as a peer", dev, peer_device);
  e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return HFK_OK;
  }
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceEnablePeerAccess");
  return HFK_OK;
}

int hfk_set_swap_out_pace(int megabytes_per_second) {
  if (megabytes_per_second < 0 || megabytes_per_second > 1000000)
    return fail(HFK_ERR_INVALID_ARG, "swap-out pace: 0 (unpaced) .. 1000000 MB/s");
  g_swap_out_pace_mbs = megabytes_per_second;
  return HFK_OK;
}

int hfk_set_vector_smem_pad(int bytes) {
  if (bytes < 0 || bytes > 200 * 1024 || (bytes & 127))
    return fail(HFK_ERR_INVALID_ARG, "vector smem pad: 0 .. 204800 bytes, multiple of 128");
  g_vec_smem_pad = bytes;
  return HFK_OK;
}

int hfk_set_staged_copy_lanes(int lanes) {
  if (lanes < 0 || lanes > kMaxLanes)
    return fail(HFK_ERR_INVALID_ARG, "staged copy lanes: 0 (default) .. %d", kMaxLanes);
  g_staged_lanes = lanes;
  return HFK_OK;
}

// ---- diagnostics: per-CTA time stamps ----------------------------------------------
__global__ void stamp_marker_kernel() {
  CtaStamp st;
  st.begin(kStampMarker);
  st.end();
}

int hfk_debug_set_stamps(void *device_buffer, size_t buffer_bytes) {
  unsigned long long *buf = static_cast<unsigned long long *>(device_buffer);
  unsigned int cap = 0;
  if (buf != nullptr) {
    if (buffer_bytes < 8 + 32 || (reinterpret_cast<uintptr_t>(buf) & 7))
      return fail(HFK_ERR_INVALID_ARG, "debug stamps: buffer must be 8-byte aligned and hold at least one record");
    cap = (unsigned int)std::min<size_t>((buffer_bytes - 8) / 32, 1u << 30);
  }
  cudaError_t e = cudaMemcpyToSymbol(g_stamp_cap, &cap, sizeof(cap));
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyToSymbol(stamp capacity)");
  e = cudaMemcpyToSymbol(g_stamp_buf, &buf, sizeof(buf));
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyToSymbol(stamp buffer)");
  return HFK_OK;
}

int hfk_debug_stamp_marker(hfk_stream_t stream) {
  stamp_marker_kernel<<<1, 1, 0, stream>>>();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "stamp_marker_kernel launch");
  return HFK_OK;
}

// ---- staged transfer for callers that cannot allocate -------------------------
//
// Who this is for.  A KV-offload connector runs inside a serving engine that handed
// nearly all free HBM to the paged KV cache at start-up and calls the transfer from
// its scheduling loop: a cudaMalloc there can fail for lack of memory, and even when
// it succeeds it synchronises the whole device and so stalls the layer compute the
// transfer is meant to overlap.  Hosts that bind this library over an FFI (cgo, JNI,
// ctypes) are in the same position for a different reason: they hold pointers to the
// cache and to the pinned pool, but they own no CUDA allocator from which a staging
// tensor could come.  For them the staging block lives inside the library.
//
// The staging block is one file-scope device array of HFK_STATIC_STAGING_BYTES.
// Every GPU on which this library runs a kernel holds that much memory until the
// process exits.  In host code the array's name only stands for the symbol — it is
// not an address the device can use — so the address is looked up once per device
// with cudaGetSymbolAddress, with that device current, and cached.
static __device__ __align__(256) unsigned char g_static_staging[HFK_STATIC_STAGING_BYTES];

namespace hfk {
constexpr int kMaxDevices = 64;
static std::mutex g_staging_mu;
static void *g_staging_addr[kMaxDevices];  // device address of g_static_staging, per device ordinal

// Address of the staging array on the current device; looked up on first use.
static int static_staging_for_current_device(void **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices)
    return fail(HFK_ERR_UNSUPPORTED, "static staging: device ordinal %d beyond %d", dev, kMaxDevices);
  std::lock_guard<std::mutex> g(g_staging_mu);
  if (g_staging_addr[dev] == nullptr) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_staging);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static staging)");
    if (p == nullptr) return fail(HFK_ERR_CUDA, "static staging: symbol address is null");
    g_staging_addr[dev] = p;
  }
  *out = g_staging_addr[dev];
  return HFK_OK;
}
}  // namespace hfk

int hfk_fused_memcpy_multi_layer_block_transfer_static(void *const *device_layer_ptrs,
                                                       const void *host_block, int64_t block_size,
                                                       int64_t layers, int64_t heads,
                                                       int64_t head_dim, int64_t elt_size, int ctas,
                                                       hfk_stream_t stream) {
  if (!host_block)
    return fail(HFK_ERR_INVALID_ARG, "fused_memcpy_multi_layer_block_transfer_static: null host block");
  if (block_size <= 0 || layers <= 0 || heads <= 0 || head_dim <= 0 || elt_size <= 0)
    return fail(HFK_ERR_INVALID_ARG, "fused_memcpy_multi_layer_block_transfer_static: non-positive geometry");
  // overflow-safe size check against the fixed capacity
  const uint64_t cap = HFK_STATIC_STAGING_BYTES;
  uint64_t bytes = 1;
  const int64_t dims[5] = {block_size, layers, heads, head_dim, elt_size};
  for (int i = 0; i < 5; ++i) {
    if ((uint64_t)dims[i] > cap || bytes * (uint64_t)dims[i] > cap)
      return fail(HFK_ERR_TOO_LARGE,
                  "fused_memcpy_multi_layer_block_transfer_static: block of [%lld,%lld,%lld,%lld] x %lld bytes "
                  "exceeds the built-in staging block of %llu bytes; use "
                  "hfk_fused_memcpy_multi_layer_block_transfer with a staging buffer of your own",
                  (long long)block_size, (long long)layers, (long long)heads, (long long)head_dim,
                  (long long)elt_size, (unsigned long long)cap);
    bytes *= (uint64_t)dims[i];
  }
  void *staging = nullptr;
  int rc = static_staging_for_current_device(&staging);
  if (rc != HFK_OK) return rc;
  // all checks first: an error return leaves nothing in the stream and the shared block untouched
  rc = validate_transfer(device_layer_ptrs, staging, block_size, layers, heads, head_dim, elt_size);
  if (rc != HFK_OK) return rc;
  // Nothing in the staging block has to start at zero: the first `bytes` bytes are
  // overwritten by this copy before the kernel reads exactly those bytes.
  cudaError_t e = cudaMemcpyAsync(staging, host_block, (size_t)bytes, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(static staging)");
  return transfer_impl(device_layer_ptrs, staging, block_size, layers, heads, head_dim, elt_size, ctas,
                       stream);
}

}  // extern "C"
