// Predicates on addresses that arrive in device-resident tables (per-layer cache
// bases).  The host cannot look at those tables without a synchronisation, so
// the kernels test every entry when they stage it: an entry that fails is never
// added to an offset or dereferenced, its work is skipped and
// HFK_DEV_BAD_LAYER_PTR is raised in the status word.  The same functions
// compile as plain C++ so that they can be unit-tested without a GPU.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define HFK_HD __host__ __device__ __forceinline__
#else
#define HFK_HD inline
#endif

namespace hfk {

// Every mover on this path works in 16-byte units (ld/st.global.v4, cp.async.bulk).
constexpr uintptr_t kVectorAlignMask = 15u;

// A layer base is usable when it is non-null and 16-byte aligned.
HFK_HD bool layer_ptr_ok(const void *p) {
  const uintptr_t v = reinterpret_cast<uintptr_t>(p);
  return v != 0 && (v & kVectorAlignMask) == 0;
}

// Three-level strided layout check used for the host pool: with the chunk at the
// bottom, the (stride, count) pairs sorted by stride must nest — every stride is
// at least the extent of everything below it — so that no two chunks overlap.
// Dimensions of count 1 never advance and are ignored.
struct StridedDim {
  int64_t stride;
  int64_t count;
};
HFK_HD bool strides_nest(int64_t chunk_bytes, StridedDim a, StridedDim b, StridedDim c) {
  StridedDim d[3] = {a, b, c};
  for (int i = 0; i < 3; ++i)
    for (int j = i + 1; j < 3; ++j)
      if (d[j].stride < d[i].stride) {
        const StridedDim t = d[i];
        d[i] = d[j];
        d[j] = t;
      }
  int64_t extent = chunk_bytes;
  for (int i = 0; i < 3; ++i) {
    if (d[i].count <= 1) continue;
    if (d[i].stride < extent) return false;
    // extent of this level: (count-1) strides plus what lies below
    extent = d[i].stride * (d[i].count - 1) + extent;
  }
  return true;
}

}  // namespace hfk
