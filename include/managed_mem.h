/*
 * managed_mem.h — source-compatible view of the reference's registry header for C++ consumers.
 *
 * The reference ships common/csrc/managed_memory/managed_mem.h inside the heterofusedkernels
 * package and pcie_through compiles against it (pcieThrough/CMakeLists.txt:79-81): free
 * functions register_ptr / unregister_ptr / register_tensor / unregister_tensor /
 * get_device_ptr (managed_mem.h:75-88) and the singleton
 * managed_memory::HostRegisteredMemoryManager with getDevicePtr / getRecordSize /
 * unregisterAll (managed_mem.h:33-59).  Code written against those names compiles unchanged
 * against this header; every call forwards to the C ABI of libhfk_b200.so (hfk_b200.h), whose
 * registry is the one the kernels and torch ops consult.  Link with -lhfk_b200.
 *
 * Differences: the driver-version split (aclrtHostRegister vs halHostRegister,
 * managed_mem.cpp:305-334) does not exist on CUDA, so both register paths are
 * cudaHostRegister; register_tensor is a template and does not require an already pinned
 * tensor (cudaHostRegister pins in place).
 */
#ifndef HFK_MANAGED_MEM_H_
#define HFK_MANAGED_MEM_H_

#include <cstddef>
#include <cstdint>
#include <stdexcept>

#include "hfk_b200.h"

namespace managed_memory {

/* managed_mem.h:9-14 */
struct RegisteredMemoryRecord {
  uintptr_t ptr;
  uintptr_t devptr;
  size_t buffSize;
  int32_t device;
};

/* Facade over the registry inside libhfk_b200.so (managed_mem.h:20-59). */
class HostRegisteredMemoryManager {
 public:
  static HostRegisteredMemoryManager &GetInstance() {
    static HostRegisteredMemoryManager instance;
    return instance;
  }
  HostRegisteredMemoryManager(const HostRegisteredMemoryManager &) = delete;
  HostRegisteredMemoryManager &operator=(const HostRegisteredMemoryManager &) = delete;

  /* device alias of a host address inside a registered range, nullptr otherwise (managed_mem.cpp:139-160) */
  void *getDevicePtr(void *hostPtr) {
    return reinterpret_cast<void *>(hfk_get_device_ptr(reinterpret_cast<uintptr_t>(hostPtr)));
  }
  /* size of the registered range containing hostPtr, 0 if none (managed_mem.cpp:163-179) */
  size_t getRecordSize(void *hostPtr) { return hfk_get_record_size(hostPtr); }
  int aclUnregisterHostPtr(void *hostPtr) { return hfk_unregister_ptr(hostPtr); }
  int halUnregisterHostPtr(void *hostPtr) { return hfk_unregister_ptr(hostPtr); }
  void unregisterAll() { hfk_unregister_all(); }

 private:
  HostRegisteredMemoryManager() = default;
};

}  // namespace managed_memory

/* managed_mem.cpp:305-323; the caller checks for nullptr */
inline void *register_ptr(void *ptr, size_t size) {
  if (ptr == nullptr) throw std::invalid_argument("ptr is a nullptr.");
  return hfk_register_ptr(ptr, size);
}

/* managed_mem.cpp:325-334 */
inline int unregister_ptr(void *ptr) {
  if (ptr == nullptr) throw std::invalid_argument("ptr is a nullptr.");
  return hfk_unregister_ptr(ptr);
}

/* managed_mem.cpp:336-364 — any tensor type with device().is_cpu(), data_ptr() and nbytes() */
template <class Tensor>
inline void *register_tensor(Tensor &tensor) {
  if (!tensor.device().is_cpu()) throw std::invalid_argument("Invalid device. Device must be CPU.");
  return hfk_register_ptr(tensor.data_ptr(), static_cast<size_t>(tensor.nbytes()));
}

/* managed_mem.cpp:366-370 */
template <class Tensor>
inline void unregister_tensor(Tensor &tensor) {
  hfk_unregister_ptr(tensor.data_ptr());
}

/* managed_mem.cpp:372-375 */
inline uintptr_t get_device_ptr(uintptr_t ptr) { return hfk_get_device_ptr(ptr); }

#endif /* HFK_MANAGED_MEM_H_ */
