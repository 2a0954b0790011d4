#include "vmm.hpp"

#include <string>

namespace dfb {

template <typename F>
static bool entry(const char* name, F*& fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || !p) return false;
  fn = reinterpret_cast<F*>(p);
  return true;
}

bool CudaVmSpace::resolve() {
  return entry("cuMemAddressReserve", memAddressReserve_) && entry("cuMemAddressFree", memAddressFree_) &&
         entry("cuMemCreate", memCreate_) && entry("cuMemRelease", memRelease_) && entry("cuMemMap", memMap_) &&
         entry("cuMemUnmap", memUnmap_) && entry("cuMemSetAccess", memSetAccess_) &&
         entry("cuMemGetAllocationGranularity", memGetGranularity_);
}

static CUmemAllocationProp device_prop(int device) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  return prop;
}

CudaVmSpace::CudaVmSpace(int device, size_t va_bytes, size_t phys_bytes) : device_(device) {
  if (cudaSetDevice(device) != cudaSuccess) throw EngineError("AllocError", "cudaSetDevice failed");
  cudaFree(nullptr);   // make sure the primary context exists
  if (!resolve()) throw EngineError("AllocError", "the driver exposes no virtual-memory management API");
  CUmemAllocationProp prop = device_prop(device);
  size_t g = 0;
  if (memGetGranularity_(&g, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM) != CUDA_SUCCESS || g == 0)
    throw EngineError("AllocError", "cuMemGetAllocationGranularity failed");
  init(g, va_bytes, phys_bytes);
  reserved_ = this->va_bytes();
  if (memAddressReserve_(&base_, reserved_, g, 0, 0) != CUDA_SUCCESS)
    throw EngineError("AllocError", "cuMemAddressReserve of " + std::to_string(reserved_) + " bytes failed");
  ++driver_calls;
  handle_of_.assign(reserved_ / g, 0);
}

CudaVmSpace::~CudaVmSpace() {
  if (!base_) return;
  for (size_t p = 0; p < handle_of_.size(); ++p) {
    if (!handle_of_[p]) continue;
    memUnmap_(base_ + p * page(), page());
    memRelease_(handle_of_[p]);
  }
  for (auto h : parked_) memRelease_(h);
  memAddressFree_(base_, reserved_);
}

bool CudaVmSpace::map_page(size_t p) {
  CUmemGenericAllocationHandle h = 0;
  if (!parked_.empty()) {
    h = parked_.back();
    parked_.pop_back();
  } else {
    CUmemAllocationProp prop = device_prop(device_);
    ++driver_calls;
    if (memCreate_(&h, page(), &prop, 0) != CUDA_SUCCESS) return false;          // the device itself is out of memory
  }
  ++driver_calls;
  if (memMap_(base_ + p * page(), page(), 0, h, 0) != CUDA_SUCCESS) {
    parked_.push_back(h);
    return false;
  }
  handle_of_[p] = h;
  return true;
}

void CudaVmSpace::unmap_page(size_t p) {
  if (!handle_of_[p]) return;
  ++driver_calls;
  memUnmap_(base_ + p * page(), page());
  parked_.push_back(handle_of_[p]);
  handle_of_[p] = 0;
}

void CudaVmSpace::grant(size_t p0, size_t count) {
  CUmemAccessDesc acc = {};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device_;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  ++driver_calls;
  if (memSetAccess_(base_ + p0 * page(), count * page(), &acc, 1) != CUDA_SUCCESS)
    throw EngineError("AllocError", "cuMemSetAccess failed");
}

}  // namespace dfb
