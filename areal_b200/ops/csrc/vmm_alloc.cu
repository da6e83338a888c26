// Pausable device memory: allocations whose virtual address survives while their physical memory is
// given back to the driver and taken again later.
//
// A buffer is a reserved virtual address range (cuMemAddressReserve) with physical memory mapped
// behind it (cuMemCreate + cuMemMap). pause() optionally saves the contents to host memory, unmaps
// and releases the physical memory; resume() creates and maps new physical memory at the SAME
// address and optionally restores the contents. Pointers held by tensors, kernels' argument lists
// and captured CUDA graphs stay valid across a pause, which is what lets a trainer and a rollout
// engine time-share one GPU (weights and KV cache of the idle side leave the device without
// tearing the engine down).
//
// Role of torch_memory_saver in the reference (areal/utils/offload.py:29-50,
// areal/engine/fsdp_engine.py:928-959), which interposes cudaMalloc with LD_PRELOAD; here the
// owners of the large buffers (KV pool, flat parameter / optimizer buffers) ask for pausable memory
// explicitly. Driver entry points are resolved at run time (no link-time libcuda dependency).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <stdint.h>

#include <map>
#include <mutex>

namespace {

struct Api {
  PFN_cuMemCreate_v10020 create = nullptr;
  PFN_cuMemRelease_v10020 release = nullptr;
  PFN_cuMemAddressReserve_v10020 reserve = nullptr;
  PFN_cuMemAddressFree_v10020 addr_free = nullptr;
  PFN_cuMemMap_v10020 map = nullptr;
  PFN_cuMemUnmap_v10020 unmap = nullptr;
  PFN_cuMemSetAccess_v10020 set_access = nullptr;
  PFN_cuMemGetAllocationGranularity_v10020 granularity = nullptr;
  bool ok = false;
};

Api g_api;
std::once_flag g_api_once;

template <typename T>
bool load(const char* name, T* out) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return false;
  *out = reinterpret_cast<T>(fn);
  return true;
}

void load_api() {
  bool ok = load("cuMemCreate", &g_api.create);
  ok = load("cuMemRelease", &g_api.release) && ok;
  ok = load("cuMemAddressReserve", &g_api.reserve) && ok;
  ok = load("cuMemAddressFree", &g_api.addr_free) && ok;
  ok = load("cuMemMap", &g_api.map) && ok;
  ok = load("cuMemUnmap", &g_api.unmap) && ok;
  ok = load("cuMemSetAccess", &g_api.set_access) && ok;
  ok = load("cuMemGetAllocationGranularity", &g_api.granularity) && ok;
  g_api.ok = ok;
}

struct Buffer {
  CUdeviceptr va = 0;
  size_t size = 0;           // mapped size (multiple of the granularity)
  size_t requested = 0;
  int device = 0;
  CUmemGenericAllocationHandle handle = 0;
  bool mapped = false;
};

std::map<uintptr_t, Buffer> g_buffers;
std::mutex g_mu;

CUmemAllocationProp prop_for(int device) {
  CUmemAllocationProp p = {};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  return p;
}

int map_physical(Buffer& b) {
  CUmemAllocationProp p = prop_for(b.device);
  if (g_api.create(&b.handle, b.size, &p, 0) != CUDA_SUCCESS) return 3;    // out of device memory: the caller may retry later
  if (g_api.map(b.va, b.size, 0, b.handle, 0) != CUDA_SUCCESS) {
    g_api.release(b.handle);
    return 4;
  }
  CUmemAccessDesc acc = {};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = b.device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (g_api.set_access(b.va, b.size, &acc, 1) != CUDA_SUCCESS) {
    g_api.unmap(b.va, b.size);
    g_api.release(b.handle);
    return 5;
  }
  b.mapped = true;
  return 0;
}

}  // namespace

extern "C" {

// 0 when the virtual-memory API is available on this driver.
int ab2_vmm_available() {
  cudaFree(0);
  std::call_once(g_api_once, load_api);
  return g_api.ok ? 0 : 1;
}

// Reserves an address range and maps `bytes` (rounded up to the allocation granularity) of the
// current device's memory behind it. Returns the device pointer or 0.
void* ab2_vmm_alloc(size_t bytes) {
  if (ab2_vmm_available() != 0 || bytes == 0) return nullptr;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  CUmemAllocationProp p = prop_for(dev);
  size_t gran = 0;
  if (g_api.granularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0) return nullptr;
  Buffer b;
  b.requested = bytes;
  b.size = (bytes + gran - 1) / gran * gran;
  b.device = dev;
  if (g_api.reserve(&b.va, b.size, gran, 0, 0) != CUDA_SUCCESS) return nullptr;
  if (map_physical(b) != 0) {
    g_api.addr_free(b.va, b.size);
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  g_buffers[(uintptr_t)b.va] = b;
  return reinterpret_cast<void*>(b.va);
}

// Gives the physical memory back. host_backup (pinned host memory of at least the requested size, or
// null to discard the contents) receives a copy first, on `stream`, which is synchronised before the
// memory is unmapped: no kernel may use the buffer while it is paused.
int ab2_vmm_pause(void* ptr, void* host_backup, void* stream) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_buffers.find((uintptr_t)ptr);
  if (it == g_buffers.end()) return 1;
  Buffer& b = it->second;
  if (!b.mapped) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (host_backup != nullptr && cudaMemcpyAsync(host_backup, ptr, b.requested, cudaMemcpyDeviceToHost, s) != cudaSuccess) return 2;
  if (cudaStreamSynchronize(s) != cudaSuccess) return 2;
  if (cudaDeviceSynchronize() != cudaSuccess) return 2;      // other streams may still read the buffer
  if (g_api.unmap(b.va, b.size) != CUDA_SUCCESS) return 4;
  if (g_api.release(b.handle) != CUDA_SUCCESS) return 5;
  b.mapped = false;
  b.handle = 0;
  return 0;
}

// Maps fresh physical memory at the same address; restores from host_backup when given (on `stream`,
// asynchronously: stream order protects later kernels of that stream). Returns 3 when the device has no room.
int ab2_vmm_resume(void* ptr, const void* host_backup, void* stream) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_buffers.find((uintptr_t)ptr);
  if (it == g_buffers.end()) return 1;
  Buffer& b = it->second;
  if (!b.mapped) {
    const int rc = map_physical(b);
    if (rc != 0) return rc;
  }
  if (host_backup != nullptr &&
      cudaMemcpyAsync(ptr, host_backup, b.requested, cudaMemcpyHostToDevice, reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess)
    return 2;
  return 0;
}

int ab2_vmm_is_paused(void* ptr) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_buffers.find((uintptr_t)ptr);
  if (it == g_buffers.end()) return -1;
  return it->second.mapped ? 0 : 1;
}

int ab2_vmm_free(void* ptr) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_buffers.find((uintptr_t)ptr);
  if (it == g_buffers.end()) return 1;
  Buffer& b = it->second;
  cudaDeviceSynchronize();
  if (b.mapped) {
    g_api.unmap(b.va, b.size);
    g_api.release(b.handle);
  }
  g_api.addr_free(b.va, b.size);
  g_buffers.erase(it);
  return 0;
}
}
