// Host-side helpers shared by the translation units of libhfk_b200.so.
#pragma once

#include <cuda_runtime_api.h>

namespace hfk {

// Records a printf-style message for hfk_last_error_message() and returns `code`.
int fail(int code, const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

// Launch defaults when the caller passes ctas <= 0 / HFK_MOVER_AUTO ("aiv=None"
// in the torch ops).  The swap defaults are sized to fill one PCIe Gen5 x16
// link while occupying a small part of the 148 SMs; the gather defaults to fill
// HBM.
//
// Measured on a B200 behind PCIe Gen5 x16 (cudaMemcpyAsync peak 55.5 GB/s h2d, 57.2 GB/s d2h):
// the bulk mover reaches the link's plateau for kernel-issued traffic (51.5 GB/s in,
// 52.7 GB/s out) from 2 single-warp CTAs with a 16 KiB x 8 ring, the vector mover needs 4-8
// CTAs of 512 threads; 4 CTAs leave a margin.  The paged gather reaches the device's copy
// bandwidth (6.67 TB/s) with one single-warp CTA per SM and a 32 KiB x 4 ring; more stages in
// flight were slower (6.2 TB/s with 6), and the best vector geometry gave 6.2 TB/s.
constexpr int kDefaultMoverOut = 2;      // HFK_MOVER_BULK
constexpr int kDefaultMoverIn = 2;       // HFK_MOVER_BULK
constexpr int kDefaultMoverGather = 2;   // HFK_MOVER_BULK
// Bulk swap launches below this many bytes use the small ring (see swap_impl): 2 KiB x 4 stages, 64
// single-warp CTAs, at most 256 ids staged at a time = 14 KB of shared memory per CTA.  Measured for
// the layer-wise fp8 pipeline (4 layers = 16.8 MB per launch, one side stream) next to a bf16 GEMM that
// fills the device: 48.3 GB/s in / 49.5 out with the GEMM 1.8 % slower; alone 48.6 / 50.1.
constexpr long long kAutoBulkMinBytes = 256ll << 20;
constexpr int kSwapSmallStageBytes = 2048, kSwapSmallStages = 4, kSwapSmallIdTile = 256;
constexpr int kDefaultSwapCtasBulkSmall = 64;
constexpr int kDefaultSwapCtasVector = 16;
constexpr int kDefaultSwapCtasBulk = 4;
constexpr int kSwapStageBytes = 16384, kSwapStages = 8, kSwapLag = 2;
constexpr int kGatherStageBytes = 32768, kGatherStages = 4, kGatherLag = 2;
constexpr int kGatherHints = 0, kGatherBlocked = 0;  // bulk gather: no L2 hints (see below), interleaved units
// L2 evict-first hints on the gather's bulk copies measured 6.70 TB/s when an un-hinted launch had run
// before in the same process and 6.50 TB/s in a fresh process (un-hinted: 6.67 TB/s either way), so
// they stay off by default.
constexpr int kGatherVectorCtasPerSm = 2;  // vector mover: 256 threads x 8 loads, 2 CTAs per SM
constexpr int kDefaultRowGatherCtas = 32;
constexpr int kDefaultTransferCtas = 32;
constexpr int kDefaultRelayoutCtas = 32;
// Staged swap: copy-engine lanes the slot copies are dealt to, and the largest single copy (a run of
// consecutive slots is cut at this size so that every lane gets work).  Measured on the Llama-3-8B
// step (512 slots of 2 MiB): 1, 2, 3 and 4 lanes all give 50.2 GB/s out / 49.0 in with random slots
// and 55.7-56.0 / 54.0-54.3 with slots in one run, so the copies stay on the caller's stream.
constexpr int kDefaultStagedLanes = 1;
constexpr long long kStagedMaxCopyBytes = 64ll << 20;
// Block migration: 512-thread CTAs per SM (peer loads over NVLink need megabytes in flight).
constexpr int kMigrateCtasPerSm = 2;

}  // namespace hfk
