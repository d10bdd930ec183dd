// Shared device-side primitives of the KV-cache data path: 16-byte streaming
// loads/stores, the bulk-copy (TMA, untiled) PTX wrappers with bounded waits,
// and the per-device status word that kernels raise instead of faulting.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hfk_b200.h"
#include "ptr_check.h"

namespace hfk {

// Per-device status word.  Kernels OR bits into it (HFK_DEV_*) when they skip
// work because an id is out of range or a bounded wait ran out; the host reads
// and clears it through hfk_device_status().
__device__ unsigned int g_status_word;

__device__ __forceinline__ void raise_status(unsigned int bit) { atomicOr(&g_status_word, bit); }

// ---- optional per-CTA time stamps (diagnostics) ---------------------------
// When a stamp buffer is installed (hfk_debug_set_stamps), thread 0 of every CTA of the data
// movers appends one record {tag << 32 | SM id, CTA index, start ns, end ns} taken from
// %globaltimer.  Word 0 of the buffer counts the records.  With no buffer installed the cost
// is one load of a __device__ pointer per CTA.
__device__ unsigned long long *g_stamp_buf;
__device__ unsigned int g_stamp_cap;

__device__ __forceinline__ unsigned int sm_id() {
  unsigned int v;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(v));
  return v;
}
__device__ __forceinline__ unsigned long long stamp_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
struct CtaStamp {
  unsigned long long *rec;
  __device__ __forceinline__ void begin(unsigned int tag) {
    rec = nullptr;
    if (threadIdx.x != 0) return;
    unsigned long long *buf = g_stamp_buf;
    if (buf == nullptr) return;
    const unsigned long long i = atomicAdd(buf, 1ull);
    if (i >= g_stamp_cap) return;
    rec = buf + 1 + 4 * i;
    rec[0] = ((unsigned long long)tag << 32) | sm_id();
    rec[1] = blockIdx.x;
    rec[2] = stamp_now();
    rec[3] = 0;
  }
  __device__ __forceinline__ void end() {
    if (threadIdx.x == 0 && rec != nullptr) rec[3] = stamp_now();
  }
};
// tags of the stamp records
constexpr unsigned int kStampMarker = 0, kStampSwapVector = 1, kStampSwapBulk = 2, kStampGatherBulk = 3,
                       kStampGatherVector = 4, kStampMigrate = 5;

// ---- 16-byte streaming accesses ------------------------------------------
// Every byte on this path is touched exactly once, so both sides use the
// evict-first (.cs) policy and never allocate in L1.
__device__ __forceinline__ uint4 ld_stream16(const uint4 *p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream16(uint4 *p, const uint4 &v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// Whole-CTA copy of n16 16-byte vectors.  Each thread keeps kUnroll independent
// loads in flight before the first store; a warp touches 512 contiguous bytes
// per instruction, so every PCIe/HBM transaction is a full, aligned line.
template <int kThreads, int kUnroll>
__device__ __forceinline__ void cta_copy16(uint4 *__restrict__ dst, const uint4 *__restrict__ src,
                                           int64_t n16) {
  const int tid = threadIdx.x;
  int64_t base = 0;
  for (; base + (int64_t)kThreads * kUnroll <= n16; base += (int64_t)kThreads * kUnroll) {
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) v[u] = ld_stream16(src + base + u * kThreads + tid);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) st_stream16(dst + base + u * kThreads + tid, v[u]);
  }
  for (int64_t i = base + tid; i < n16; i += kThreads) st_stream16(dst + i, ld_stream16(src + i));
}

// ---- mbarrier + bulk copy (cp.async.bulk, untiled) -----------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Waits for the phase with the given parity, for at most kWaitLimitNs.  Returns
// false when it gave up; the caller raises HFK_DEV_WAIT_TIMEOUT and leaves.
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity,
                                                  uint64_t limit_ns = kWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  while (!mbar_try_wait(bar, parity)) {
    if (global_timer_ns() - t0 > limit_ns) return false;
  }
  return true;
}

// Self-test of the bounded wait: one warp waits on a barrier that nothing ever completes, gives
// up after limit_ns, raises HFK_DEV_WAIT_TIMEOUT and returns — the context stays usable.
__global__ void __launch_bounds__(32) wait_timeout_selftest_kernel(uint64_t limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    if (!mbar_wait_bounded(&bar, 0, limit_ns)) raise_status(HFK_DEV_WAIT_TIMEOUT);
  }
}
// global -> this CTA's shared memory, completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gsrc, uint32_t bytes,
                                          uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_addr(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}
// this CTA's shared memory -> global, tracked by the thread's bulk group.
__device__ __forceinline__ void bulk_store(void *gdst, const void *smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
               "r"(smem_addr(smem_src)), "r"(bytes)
               : "memory");
}
// The same two copies with an L2 eviction-priority hint (policy from make_evict_first_policy()).
__device__ __forceinline__ uint64_t make_evict_first_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_load_hint(void *smem_dst, const void *gsrc, uint32_t bytes,
                                               uint64_t *bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_addr(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_addr(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void bulk_store_hint(void *gdst, const void *smem_src, uint32_t bytes,
                                                uint64_t policy) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;" ::"l"(gdst),
               "r"(smem_addr(smem_src)), "r"(bytes), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int kPending>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void fence_async_proxy() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- the descriptor pump --------------------------------------------------
// One warp per CTA.  All 32 lanes compute copy descriptors (source, destination,
// byte count) 32 at a time; lane 0 then drives a ring of kStages shared-memory
// stages: bulk load into a stage, wait on the stage's mbarrier, bulk store out
// of it, and reuse the stage once the store has finished reading it.  No data
// passes through registers and 31 of the 32 lanes only do address arithmetic,
// so the kernel leaves the SM's issue slots and register file to whatever
// compute kernel shares the SM.
struct CopyDesc {
  const void *src;
  void *dst;
  uint32_t bytes;  // 0 = nothing to do (skipped unit)
};

// kLag (template parameter of the pump) = how many of the most recent stores may still be
// reading their stage when the next load is issued; the remaining n_stages - kLag stages hold
// loads in flight.  Compiled values:
constexpr int kPumpLagMax = 8;

struct PumpSmem {
  uint64_t full[32];      // one mbarrier per stage (kStages <= 32)
  CopyDesc desc[64];      // two batches of 32 descriptors
};

// make_desc(k) returns the descriptor of this CTA's k-th unit, k < total.
// Returns false when a bounded wait ran out: HFK_DEV_WAIT_TIMEOUT is raised, the loads that
// were still in flight get one more (short) bounded wait each so that no copy is outstanding
// into this CTA's shared memory when it exits, and the caller must stop issuing work.  After
// a timeout the destination of the whole call is undefined.
constexpr uint64_t kDrainLimitNs = 100000000ull;  // 0.1 s per stage that still has a load in flight
//
// pace_ns_per_kib > 0 paces the STORES of this CTA: the k-th KiB is not stored before
// t_start + k * pace_ns_per_kib (on %globaltimer).  A swap-out paced a little below the link's
// write rate leaves room on the upstream lanes for the read requests of a swap-in that runs at
// the same time.  The pacing wait ends at a computed time and is bounded in iterations as well.
constexpr int kPaceSpinLimit = 1 << 20;
template <int kPumpLag, typename MakeDesc>
__device__ __forceinline__ bool run_pump(PumpSmem *ps, unsigned char *stages, int stage_bytes,
                                         int n_stages, int64_t total, uint32_t &seq,
                                         MakeDesc make_desc, int hints = 0, float pace_ns_per_kib = 0.f,
                                         uint64_t pace_t0 = 0, uint64_t *paced_bytes = nullptr) {
  // hints: bit 0 = loads carry an L2 evict-first policy, bit 1 = stores do
  const int lane = threadIdx.x & 31;
  const uint64_t policy = hints ? make_evict_first_policy() : 0;
  const int in_flight = n_stages - kPumpLag;  // loads kept in flight
  int64_t issued = 0, done = 0;
  bool ok = true;
  auto fill_batch = [&](int64_t first) {
    const int64_t k = first + lane;
    CopyDesc d;
    d.src = nullptr; d.dst = nullptr; d.bytes = 0;
    if (k < total) d = make_desc(k);
    ps->desc[(first & 32) + lane] = d;
    __syncwarp();
  };
  auto issue_load = [&](int64_t k) {
    const CopyDesc d = ps->desc[k & 63];
    const uint32_t q = seq + (uint32_t)k;
    const int slot = q % n_stages;
    if (lane == 0) {
      if (d.bytes != 0) {
        mbar_expect_tx(&ps->full[slot], d.bytes);
        if (hints & 1)
          bulk_load_hint(stages + (size_t)slot * stage_bytes, d.src, d.bytes, &ps->full[slot], policy);
        else
          bulk_load(stages + (size_t)slot * stage_bytes, d.src, d.bytes, &ps->full[slot]);
      } else {
        mbar_arrive(&ps->full[slot]);  // a skipped unit still completes its phase
      }
    }
  };
  while (done < total && ok) {
    while (issued < total && issued < done + in_flight) {
      if ((issued & 31) == 0) fill_batch(issued);
      if (issued >= n_stages) {
        // stage reuse: the store of unit (issued - n_stages) must have read its stage
        if (lane == 0) bulk_wait_read<kPumpLag>();
      }
      issue_load(issued);
      ++issued;
    }
    const CopyDesc d = ps->desc[done & 63];
    const uint32_t q = seq + (uint32_t)done;
    const int slot = q % n_stages;
    const uint32_t parity = (q / n_stages) & 1u;
    if (d.bytes != 0) {
      if (lane == 0) {
        ok = mbar_wait_bounded(&ps->full[slot], parity);
        if (ok) {
          if (pace_ns_per_kib > 0.f) {
            const uint64_t due = pace_t0 + (uint64_t)((float)(*paced_bytes >> 10) * pace_ns_per_kib);
            for (int spin = 0; spin < kPaceSpinLimit && global_timer_ns() < due; ++spin) {
            }
            *paced_bytes += d.bytes;
          }
          fence_async_proxy();
          if (hints & 2)
            bulk_store_hint(d.dst, stages + (size_t)slot * stage_bytes, d.bytes, policy);
          else
            bulk_store(d.dst, stages + (size_t)slot * stage_bytes, d.bytes);
        }
      }
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
    }
    if (lane == 0) bulk_commit();  // one group per unit, empty for skipped units
    ++done;
  }
  if (!ok && lane == 0) {
    raise_status(HFK_DEV_WAIT_TIMEOUT);
    // unit done-1 is the one that timed out; it and the units up to issued-1 may still have a
    // load in flight
    for (int64_t k = done - 1; k < issued; ++k) {
      if (ps->desc[k & 63].bytes == 0) continue;
      const uint32_t q = seq + (uint32_t)k;
      mbar_wait_bounded(&ps->full[q % n_stages], (q / n_stages) & 1u, kDrainLimitNs);
    }
  }
  if (lane == 0) bulk_wait_all();
  seq += (uint32_t)total;
  __syncwarp();
  return ok;
}

}  // namespace hfk
