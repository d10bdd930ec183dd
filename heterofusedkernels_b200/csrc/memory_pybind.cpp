// pybind11 module `memory` — the Python surface of the reference's
// heterofusedkernels.memory (common/csrc/pybind.cpp:7-11): the same three
// names with the same meaning, over the C ABI of libhfk_b200.so.
#include <torch/extension.h>

#include <iostream>

#include "../../include/hfk_b200.h"

namespace {

// NUMA-local, zero-filled, device-mapped host buffer as a 1-D int8 CPU tensor of
// `size` bytes; users .view(dtype).view(shape) it (common/README.md:39-40).  The
// tensor owns the mapping: its deleter unregisters and unmaps and never throws
// (common/csrc/mem_alloc.cpp:17-64).
torch::Tensor alloc_numa_pinned_tensor(std::size_t size) {
  const int node = hfk_device_numa_node(-1);
  TORCH_CHECK(node >= -1, "Unable to obtain the NUMA node of the current device: ", hfk_last_error_message());
  void *ptr = hfk_alloc_pinned_numa_ptr(size, node);
  if (ptr == nullptr)
    throw std::runtime_error(std::string("unable to allocate NUMA-pinned host memory: ") + hfk_last_error_message());
  auto deleter = [](void *p) {
    if (hfk_free_pinned_numa_ptr(p) != HFK_OK)
      std::cerr << "free of NUMA-pinned host memory failed: " << hfk_last_error_message() << std::endl;
  };
  auto opts = torch::TensorOptions().dtype(torch::kInt8).device(torch::kCPU).pinned_memory(true);
  return torch::from_blob(ptr, {static_cast<int64_t>(size)}, deleter, opts);
}

// Registers the storage bytes of an existing CPU tensor with the current device
// and returns the device alias of its first element
// (register_tensor, common/csrc/managed_memory/managed_mem.cpp:336-364).  The
// reference insists on an already pinned tensor; cudaHostRegister pins pageable
// memory in place, so any CPU tensor is accepted here.
std::uintptr_t host_register(torch::Tensor &tensor) {
  TORCH_CHECK(tensor.device().is_cpu(), "Invalid device. Device must be CPU.");
  TORCH_CHECK(tensor.is_contiguous(), "host_register: tensor must be contiguous");
  void *alias = hfk_register_ptr(tensor.data_ptr(), tensor.nbytes());
  TORCH_CHECK(alias != nullptr, "Failed to register memory: ", hfk_last_error_message());
  return reinterpret_cast<std::uintptr_t>(alias);
}

// unregister_tensor (managed_mem.cpp:366-370)
void host_unregister(torch::Tensor &tensor) {
  const int rc = hfk_unregister_ptr(tensor.data_ptr());
  TORCH_CHECK(rc == HFK_OK, "host_unregister: ", hfk_last_error_message());
}

}  // namespace

PYBIND11_MODULE(memory, m) {
  m.def("alloc_numa_pinned_tensor", &alloc_numa_pinned_tensor);
  m.def("host_register", &host_register);
  m.def("get_device_ptr", [](std::uintptr_t p) { return hfk_get_device_ptr(p); });
  m.def("host_unregister", &host_unregister);
  m.def("device_numa_node", []() { return hfk_device_numa_node(-1); });
  m.def("registry_count", []() { return hfk_registry_count(); });
}
