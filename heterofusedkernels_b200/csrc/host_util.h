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
constexpr int kDefaultMoverOut = 1;      // HFK_MOVER_VECTOR
constexpr int kDefaultMoverIn = 1;       // HFK_MOVER_VECTOR
constexpr int kDefaultMoverGather = 1;   // HFK_MOVER_VECTOR
constexpr int kDefaultSwapCtasVector = 32;
constexpr int kDefaultSwapCtasBulk = 16;
constexpr int kDefaultGatherCtasVector = 148 * 8;
constexpr int kDefaultGatherCtasBulk = 148;
constexpr int kDefaultRowGatherCtas = 32;
constexpr int kDefaultTransferCtas = 32;

}  // namespace hfk
