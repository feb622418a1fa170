// Fixed-address device memory arena for buffers that must give their physical memory back and later return at the
// SAME virtual address: the paged KV cache of a sleeping generation engine.  A CUDA graph captured against the cache
// stays valid across sleep / wake, because only the physical backing is released; the address range is kept.
//
// The reference obtains this from vLLM's cumem allocator (sleep mode: `sleep(level)` / `wake_up(tags)`,
// skyrl/backends/skyrl_train/inference_servers/vllm_worker.py); here it is a small wrapper over the virtual memory
// management driver API: cuMemAddressReserve once, then cuMemCreate + cuMemMap + cuMemSetAccess on wake and
// cuMemUnmap + cuMemRelease on sleep.  The driver entry points are resolved through the runtime
// (cudaGetDriverEntryPoint), so the library has no link-time dependency on libcuda.
//
// Not thread-safe per arena (one engine owns one arena); every call returns an SB_* code.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <mutex>

#include "host_common.h"

namespace sb {

struct VmmApi {
  CUresult (*AddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*AddressFree)(CUdeviceptr, size_t);
  CUresult (*Create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*Release)(CUmemGenericAllocationHandle);
  CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*Unmap)(CUdeviceptr, size_t);
  CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*GetGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  bool ok;
};

static const VmmApi& vmm_api() {
  static VmmApi api = {};
  static std::once_flag once;
  std::call_once(once, [] {
    auto get = [](const char* name, void** out) {
      cudaDriverEntryPointQueryResult q;
      return cudaGetDriverEntryPoint(name, out, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess &&
             *out != nullptr;
    };
    bool ok = true;
    ok &= get("cuMemAddressReserve", reinterpret_cast<void**>(&api.AddressReserve));
    ok &= get("cuMemAddressFree", reinterpret_cast<void**>(&api.AddressFree));
    ok &= get("cuMemCreate", reinterpret_cast<void**>(&api.Create));
    ok &= get("cuMemRelease", reinterpret_cast<void**>(&api.Release));
    ok &= get("cuMemMap", reinterpret_cast<void**>(&api.Map));
    ok &= get("cuMemUnmap", reinterpret_cast<void**>(&api.Unmap));
    ok &= get("cuMemSetAccess", reinterpret_cast<void**>(&api.SetAccess));
    ok &= get("cuMemGetAllocationGranularity", reinterpret_cast<void**>(&api.GetGranularity));
    api.ok = ok;
  });
  return api;
}

struct VmmArena {
  CUdeviceptr base = 0;
  size_t bytes = 0;  // reserved (and, when mapped, backed) size: a multiple of the granularity
  int device = 0;
  bool mapped = false;
  CUmemGenericAllocationHandle handle = 0;
};

static CUmemAllocationProp vmm_prop(int device) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  return prop;
}

}  // namespace sb

extern "C" {

int sb_vmm_arena_wake(void* arena);

// Reserve an address range of at least `bytes` on the current device and back it with physical memory.
// *arena_out receives an opaque handle, *ptr_out the device address, *bytes_out the rounded-up size.
int sb_vmm_arena_create(size_t bytes, void** arena_out, unsigned long long* ptr_out, size_t* bytes_out) {
  using namespace sb;
  if (bytes == 0 || !arena_out || !ptr_out) return SB_ERR_ARG;
  const VmmApi& api = vmm_api();
  if (!api.ok) return SB_ERR_CUDA;
  if (cudaFree(nullptr) != cudaSuccess) return SB_ERR_CUDA;  // make sure the primary context exists
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SB_ERR_CUDA;
  const CUmemAllocationProp prop = vmm_prop(dev);
  size_t gran = 0;
  if (api.GetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0) return SB_ERR_CUDA;
  auto* a = new VmmArena();
  a->device = dev;
  a->bytes = (bytes + gran - 1) / gran * gran;
  if (api.AddressReserve(&a->base, a->bytes, gran, 0, 0) != CUDA_SUCCESS) {
    delete a;
    return SB_ERR_CUDA;
  }
  *arena_out = a;
  *ptr_out = static_cast<unsigned long long>(a->base);
  if (bytes_out) *bytes_out = a->bytes;
  // back it right away; a failure here leaves a valid, unmapped arena that the caller may wake later or destroy
  return sb_vmm_arena_wake(a);
}

// Give the physical memory back; the address range stays reserved.  The caller must have synchronised every stream
// that touches the arena.  Contents are lost.
int sb_vmm_arena_sleep(void* arena) {
  using namespace sb;
  auto* a = static_cast<VmmArena*>(arena);
  if (!a) return SB_ERR_ARG;
  if (!a->mapped) return SB_OK;
  const VmmApi& api = vmm_api();
  if (api.Unmap(a->base, a->bytes) != CUDA_SUCCESS) return SB_ERR_CUDA;
  a->mapped = false;
  if (api.Release(a->handle) != CUDA_SUCCESS) return SB_ERR_CUDA;
  a->handle = 0;
  return SB_OK;
}

// Back the reserved range with fresh physical memory (contents undefined) at the same address.
int sb_vmm_arena_wake(void* arena) {
  using namespace sb;
  auto* a = static_cast<VmmArena*>(arena);
  if (!a) return SB_ERR_ARG;
  if (a->mapped) return SB_OK;
  const VmmApi& api = vmm_api();
  const CUmemAllocationProp prop = vmm_prop(a->device);
  if (api.Create(&a->handle, a->bytes, &prop, 0) != CUDA_SUCCESS) return SB_ERR_TOO_LARGE;  // typically out of memory
  if (api.Map(a->base, a->bytes, 0, a->handle, 0) != CUDA_SUCCESS) {
    api.Release(a->handle);
    a->handle = 0;
    return SB_ERR_CUDA;
  }
  CUmemAccessDesc acc = {};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = a->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (api.SetAccess(a->base, a->bytes, &acc, 1) != CUDA_SUCCESS) {
    api.Unmap(a->base, a->bytes);
    api.Release(a->handle);
    a->handle = 0;
    return SB_ERR_CUDA;
  }
  a->mapped = true;
  return SB_OK;
}

int sb_vmm_arena_is_mapped(void* arena) { return arena && static_cast<sb::VmmArena*>(arena)->mapped ? 1 : 0; }

int sb_vmm_arena_destroy(void* arena) {
  using namespace sb;
  auto* a = static_cast<VmmArena*>(arena);
  if (!a) return SB_OK;
  int rc = sb_vmm_arena_sleep(a);
  if (vmm_api().AddressFree(a->base, a->bytes) != CUDA_SUCCESS) rc = SB_ERR_CUDA;
  delete a;
  return rc;
}

}  // extern "C"
