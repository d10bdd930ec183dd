// Host-memory side of the data path: the registry of device-mapped host ranges
// and the NUMA-local pinned allocator.
//
// Registry: restates HostRegisteredMemoryManager
// (common/csrc/managed_memory/managed_mem.h:20-59, managed_mem.cpp:45-66,
// 105-119, 139-179) on cudaHostRegister / cudaHostGetDevicePointer — a map
// base -> {base, alias, size, device} under a shared_mutex, range lookup by
// linear scan (few records), duplicate registration returns the first record.
//
// Allocator: restates alloc_pinned_numa_ptr / free_pinned_numa_ptr
// (common/csrc/mem_alloc.cpp:66-115): anonymous mmap, mbind(MPOL_BIND) to the
// GPU's NUMA node, zero fill (first touch on that node), register.  The node
// comes from cudaDeviceGetPCIBusId + sysfs instead of DCMI
// (common/csrc/dcmi_management.cpp:27-39, mem_alloc.cpp:25-38).  There is no
// libnuma on the target image, so mbind is issued as a raw syscall.
#include <cuda_runtime_api.h>
#include <errno.h>
#include <sys/mman.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <mutex>
#include <shared_mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/hfk_b200.h"
#include "host_util.h"

namespace hfk {

struct HostRecord {
  uintptr_t host;
  uintptr_t alias;
  size_t size;
  int device;
  bool by_driver;  // false when recorded under the test driver
};

class HostRegistry {
 public:
  static HostRegistry &instance() {
    static HostRegistry r;
    return r;
  }
  ~HostRegistry() { unregister_all(); }

  void *add(void *ptr, size_t size) {
    if (ptr == nullptr || size == 0) {
      fail(HFK_ERR_INVALID_ARG, "register_ptr: pointer is null or size is 0");
      return nullptr;
    }
    std::unique_lock<std::shared_mutex> guard(mu_);
    auto it = map_.find(reinterpret_cast<uintptr_t>(ptr));
    if (it != map_.end()) return reinterpret_cast<void *>(it->second.alias);
    HostRecord rec{reinterpret_cast<uintptr_t>(ptr), 0, size, -1, !test_driver_};
    if (test_driver_) {
      rec.alias = rec.host;
    } else {
      cudaError_t e = cudaHostRegister(ptr, size, cudaHostRegisterMapped | cudaHostRegisterPortable);
      if (e != cudaSuccess) {
        cudaGetLastError();
        cuda_fail(e, "cudaHostRegister");
        return nullptr;
      }
      void *alias = nullptr;
      e = cudaHostGetDevicePointer(&alias, ptr, 0);
      if (e != cudaSuccess) {
        cudaHostUnregister(ptr);
        cudaGetLastError();
        cuda_fail(e, "cudaHostGetDevicePointer");
        return nullptr;
      }
      rec.alias = reinterpret_cast<uintptr_t>(alias);
      cudaGetDevice(&rec.device);
    }
    map_.emplace(rec.host, rec);
    return reinterpret_cast<void *>(rec.alias);
  }

  int remove(void *ptr) {
    if (ptr == nullptr) return fail(HFK_ERR_INVALID_ARG, "unregister_ptr: pointer is null");
    std::unique_lock<std::shared_mutex> guard(mu_);
    auto it = map_.find(reinterpret_cast<uintptr_t>(ptr));
    if (it == map_.end()) return HFK_OK;  // never registered: nothing to do
    int rc = HFK_OK;
    if (it->second.by_driver) {
      cudaError_t e = cudaHostUnregister(ptr);
      if (e != cudaSuccess) {
        cudaGetLastError();
        rc = cuda_fail(e, "cudaHostUnregister");
      }
    }
    map_.erase(it);
    return rc;
  }

  bool find(uintptr_t p, HostRecord *out) const {
    if (p == 0) return false;
    std::shared_lock<std::shared_mutex> guard(mu_);
    // records do not overlap, so the candidate is the last base <= p
    auto it = map_.upper_bound(p);
    if (it == map_.begin()) return false;
    --it;
    const HostRecord &r = it->second;
    if (p >= r.host && p < r.host + r.size) {
      *out = r;
      return true;
    }
    return false;
  }

  int count() const {
    std::shared_lock<std::shared_mutex> guard(mu_);
    return (int)map_.size();
  }

  void unregister_all() {
    std::unique_lock<std::shared_mutex> guard(mu_);
    for (auto &kv : map_) {
      if (kv.second.by_driver) {
        // at process exit the context may already be gone; ignore the status
        cudaHostUnregister(reinterpret_cast<void *>(kv.first));
        cudaGetLastError();
      }
    }
    map_.clear();
  }

  void set_test_driver(bool on) {
    std::unique_lock<std::shared_mutex> guard(mu_);
    test_driver_ = on;
  }

 private:
  HostRegistry() = default;
  HostRegistry(const HostRegistry &) = delete;
  HostRegistry &operator=(const HostRegistry &) = delete;
  std::map<uintptr_t, HostRecord> map_;
  mutable std::shared_mutex mu_;
  bool test_driver_ = false;
};

// sizes of the mappings handed out by hfk_alloc_pinned_numa_ptr, for munmap
static std::mutex g_alloc_mu;
static std::map<uintptr_t, size_t> g_alloc_sizes;

static long raw_mbind(void *addr, unsigned long len, int mode, const unsigned long *mask,
                      unsigned long maxnode, unsigned flags) {
  return syscall(SYS_mbind, addr, len, mode, mask, maxnode, flags);
}
constexpr int kMpolBind = 2;            // MPOL_BIND
constexpr unsigned kMpolMfStrict = 1u;  // MPOL_MF_STRICT
constexpr unsigned kMpolMfMove = 2u;    // MPOL_MF_MOVE

// First touch with several threads: the pools are tens of GB and a single
// memset would take longer than the registration itself.
static void parallel_zero(void *p, size_t size) {
  const size_t kChunk = (size_t)256 << 20;
  unsigned n = std::thread::hardware_concurrency();
  n = std::max(1u, std::min(n, 16u));
  if (size < 2 * kChunk || n == 1) {
    memset(p, 0, size);
    return;
  }
  std::vector<std::thread> th;
  const size_t per = (size / n + 4095) & ~(size_t)4095;
  for (unsigned i = 0; i < n; ++i) {
    const size_t b = std::min(size, (size_t)i * per), e = std::min(size, b + per);
    if (e > b) th.emplace_back([=] { memset(static_cast<char *>(p) + b, 0, e - b); });
  }
  for (auto &t : th) t.join();
}

}  // namespace hfk

using namespace hfk;

extern "C" {

void *hfk_register_ptr(void *ptr, size_t size) { return HostRegistry::instance().add(ptr, size); }

int hfk_unregister_ptr(void *ptr) { return HostRegistry::instance().remove(ptr); }

uintptr_t hfk_get_device_ptr(uintptr_t host_ptr) {
  HostRecord r;
  if (!HostRegistry::instance().find(host_ptr, &r)) return 0;
  return r.alias + (host_ptr - r.host);
}

size_t hfk_get_record_size(void *ptr) {
  HostRecord r;
  if (!HostRegistry::instance().find(reinterpret_cast<uintptr_t>(ptr), &r)) return 0;
  return r.size;
}

int hfk_registry_count(void) { return HostRegistry::instance().count(); }
void hfk_unregister_all(void) { HostRegistry::instance().unregister_all(); }
void hfk_registry_set_test_driver(int on) { HostRegistry::instance().set_test_driver(on != 0); }

int hfk_device_pci_bus_id(int device, char *buf, size_t buf_len) {
  if (!buf || buf_len < 13) return fail(HFK_ERR_INVALID_ARG, "pci_bus_id: buffer too small");
  if (device < 0) {
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  }
  cudaError_t e = cudaDeviceGetPCIBusId(buf, (int)buf_len, device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetPCIBusId");
  for (char *c = buf; *c; ++c) *c = (char)tolower((unsigned char)*c);  // sysfs names are lower case
  return HFK_OK;
}

int hfk_device_numa_node(int device) {
  char bdf[32];
  int rc = hfk_device_pci_bus_id(device, bdf, sizeof(bdf));
  if (rc != HFK_OK) return rc < -1 ? rc : HFK_ERR_CUDA;
  const std::string path = std::string("/sys/bus/pci/devices/") + bdf + "/numa_node";
  std::ifstream f(path);
  if (!f.is_open()) return -1;  // no sysfs entry (container): treat as "no NUMA information"
  int node = -1;
  f >> node;
  if (f.fail()) return -1;
  return node < 0 ? -1 : node;
}

void *hfk_alloc_pinned_numa_ptr(size_t size, int node) {
  if (size == 0) {
    fail(HFK_ERR_INVALID_ARG, "alloc_pinned_numa_ptr: size is 0");
    return nullptr;
  }
  void *p = mmap(nullptr, size, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (p == MAP_FAILED) {
    fail(HFK_ERR_NO_MEMORY, "mmap(%zu) failed: %s", size, strerror(errno));
    return nullptr;
  }
  if (node >= 0) {
    // up to 1024 nodes; the reference limits itself to one 64-bit word (mem_alloc.cpp:90-92)
    unsigned long mask[16] = {0};
    if (node < 1024) {
      mask[node / 64] = 1ul << (node % 64);
      if (raw_mbind(p, size, kMpolBind, mask, 1024 + 1, kMpolMfMove | kMpolMfStrict) != 0) {
        const int err = errno;
        munmap(p, size);
        fail(HFK_ERR_NO_MEMORY, "mbind(node %d) failed: %s", node, strerror(err));
        return nullptr;
      }
    }
  }
  madvise(p, size, MADV_HUGEPAGE);
  parallel_zero(p, size);
  if (hfk_register_ptr(p, size) == nullptr) {
    munmap(p, size);  // the registry has already recorded the reason
    return nullptr;
  }
  std::lock_guard<std::mutex> g(g_alloc_mu);
  g_alloc_sizes[reinterpret_cast<uintptr_t>(p)] = size;
  return p;
}

int hfk_free_pinned_numa_ptr(void *ptr) {
  if (!ptr) return fail(HFK_ERR_INVALID_ARG, "free_pinned_numa_ptr: pointer is null");
  size_t size = 0;
  {
    std::lock_guard<std::mutex> g(g_alloc_mu);
    auto it = g_alloc_sizes.find(reinterpret_cast<uintptr_t>(ptr));
    if (it == g_alloc_sizes.end())
      return fail(HFK_ERR_INVALID_ARG, "free_pinned_numa_ptr: pointer was not allocated here");
    size = it->second;
    g_alloc_sizes.erase(it);
  }
  const int rc = hfk_unregister_ptr(ptr);
  if (munmap(ptr, size) != 0) return fail(HFK_ERR_NO_MEMORY, "munmap failed: %s", strerror(errno));
  return rc;
}

}  // extern "C"
