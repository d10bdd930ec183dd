// CPU-only checks compiled and run by tests/test_cpp_host.py:
//  * the address and stride predicates the kernels and the host validation share (ptr_check.h);
//  * a consumer written against the reference's managed_mem.h names compiles against
//    include/managed_mem.h and reaches the registry of libhfk_b200.so (test driver: no GPU).
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "managed_mem.h"
#include "ptr_check.h"

#define CHECK(cond)                                                       \
  do {                                                                    \
    if (!(cond)) {                                                        \
      std::printf("FAILED %s:%d %s\n", __FILE__, __LINE__, #cond);        \
      return 1;                                                           \
    }                                                                     \
  } while (0)

struct FakeDevice {
  bool is_cpu() const { return true; }
};
struct FakeTensor {  // the three members register_tensor needs
  std::vector<char> bytes;
  FakeDevice device() const { return {}; }
  void *data_ptr() { return bytes.data(); }
  size_t nbytes() const { return bytes.size(); }
};

int main() {
  using namespace hfk;
  // layer bases
  CHECK(!layer_ptr_ok(nullptr));
  CHECK(layer_ptr_ok(reinterpret_cast<void *>(0x7f0000000000ull)));
  CHECK(layer_ptr_ok(reinterpret_cast<void *>(0x10)));
  for (int off = 1; off < 16; ++off) CHECK(!layer_ptr_ok(reinterpret_cast<void *>(0x7f0000000000ull + off)));
  // host pool strides: [slot][layer][K|V][chunk], chunk 4096
  CHECK(strides_nest(4096, {4096, 2}, {8192, 4}, {32768, 100}));
  CHECK(strides_nest(4096, {4096, 2}, {8192, 4}, {65536, 100}));            // padded slots
  CHECK(!strides_nest(4096, {4096, 2}, {8192, 4}, {16384, 100}));           // slots overlap layers
  CHECK(!strides_nest(4096, {2048, 2}, {8192, 4}, {32768, 100}));           // K overlaps V
  CHECK(!strides_nest(4096, {0, 2}, {8192, 4}, {32768, 100}));              // expanded K|V dimension
  CHECK(strides_nest(4096, {0, 1}, {8192, 4}, {32768, 100}));               // size-1 dimension: stride ignored
  // layer-major pool [layer][K|V][slot][chunk]
  CHECK(strides_nest(4096, {4096 * 100, 2}, {4096 * 200, 4}, {4096, 100}));
  CHECK(!strides_nest(4096, {4096 * 50, 2}, {4096 * 200, 4}, {4096, 100}));
  // single-layer view of a slot-major pool (what a layer-wise prefetcher passes)
  CHECK(strides_nest(8192, {8192, 2}, {16384, 1}, {16384 * 28, 1000}));
  // three-layer view
  CHECK(strides_nest(8192, {8192, 2}, {16384, 3}, {16384 * 28, 1000}));

  // the reference's C++ names over the C ABI, without a GPU
  hfk_registry_set_test_driver(1);
  std::vector<char> buf(1 << 16);
  void *alias = register_ptr(buf.data(), buf.size());
  CHECK(alias != nullptr);
  auto &hmm = managed_memory::HostRegisteredMemoryManager::GetInstance();
  CHECK(hmm.getDevicePtr(buf.data() + 100) == static_cast<char *>(alias) + 100);
  CHECK(hmm.getRecordSize(buf.data() + 5) == buf.size());
  CHECK(get_device_ptr(reinterpret_cast<uintptr_t>(buf.data()) + 4096) == reinterpret_cast<uintptr_t>(alias) + 4096);
  CHECK(get_device_ptr(reinterpret_cast<uintptr_t>(buf.data()) + buf.size()) == 0);
  FakeTensor t;
  t.bytes.resize(4096);
  CHECK(register_tensor(t) != nullptr);
  CHECK(hfk_registry_count() == 2);
  unregister_tensor(t);
  CHECK(unregister_ptr(buf.data()) == 0);
  CHECK(hmm.getDevicePtr(buf.data()) == nullptr);
  bool threw = false;
  try {
    register_ptr(nullptr, 16);
  } catch (const std::invalid_argument &) {
    threw = true;
  }
  CHECK(threw);
  hmm.unregisterAll();
  hfk_registry_set_test_driver(0);
  std::printf("host checks ok\n");
  return 0;
}
