"""``from heterofusedkernels import memory`` — the reference's pybind module
(common/csrc/pybind.cpp:7-11) re-exported from the in-tree build."""
import heterofusedkernels_b200 as _pkg

_m = _pkg.memory
alloc_numa_pinned_tensor = _m.alloc_numa_pinned_tensor
host_register = _m.host_register
get_device_ptr = _m.get_device_ptr
host_unregister = _m.host_unregister
device_numa_node = _m.device_numa_node
registry_count = _m.registry_count
