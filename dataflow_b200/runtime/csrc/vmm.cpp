#include "vmm.hpp"

#include <stdexcept>
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

bool VmmArena::resolve() {
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

VmmArena::VmmArena(int device, size_t va_bytes) : device_(device) {
  if (cudaSetDevice(device) != cudaSuccess) return;
  cudaFree(nullptr);   // make sure the primary context exists
  if (!resolve()) return;
  CUmemAllocationProp prop = device_prop(device);
  size_t g = 0;
  if (memGetGranularity_(&g, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM) != CUDA_SUCCESS || g == 0) return;
  granule_ = g;
  va_bytes_ = (va_bytes + g - 1) / g * g;
  if (memAddressReserve_(&base_, va_bytes_, g, 0, 0) != CUDA_SUCCESS) return;
  driver_calls_++;
  ok_ = true;
}

VmmArena::~VmmArena() {
  if (!ok_) return;
  for (auto& kv : mapped_) {
    memUnmap_(base_ + kv.first * granule_, granule_);
    memRelease_(kv.second);
  }
  for (auto h : parked_) memRelease_(h);
  memAddressFree_(base_, va_bytes_);
}

uint64_t VmmArena::map(size_t offset, size_t bytes) {
  if (!ok_) throw std::runtime_error("VMM arena unavailable");
  if (offset % granule_) throw std::runtime_error("VMM map offset is not granule aligned");
  size_t first = offset / granule_, count = (bytes + granule_ - 1) / granule_;
  if ((first + count) * granule_ > va_bytes_) throw std::runtime_error("VMM map exceeds the reserved range");
  CUmemAllocationProp prop = device_prop(device_);
  CUmemAccessDesc acc = {};
  acc.location = prop.location;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (size_t g = first; g < first + count; ++g) {
    if (mapped_.count(g)) continue;
    CUmemGenericAllocationHandle h;
    if (!parked_.empty()) { h = parked_.back(); parked_.pop_back(); }
    else {
      if (memCreate_(&h, granule_, &prop, 0) != CUDA_SUCCESS) throw std::runtime_error("cuMemCreate failed");
      driver_calls_++;
    }
    CUdeviceptr at = base_ + g * granule_;
    if (memMap_(at, granule_, 0, h, 0) != CUDA_SUCCESS) { parked_.push_back(h); throw std::runtime_error("cuMemMap failed"); }
    if (memSetAccess_(at, granule_, &acc, 1) != CUDA_SUCCESS) throw std::runtime_error("cuMemSetAccess failed");
    driver_calls_ += 2;
    mapped_[g] = h;
  }
  return static_cast<uint64_t>(base_ + offset);
}

void VmmArena::unmap(size_t offset, size_t bytes) {
  if (!ok_) return;
  size_t first = offset / granule_, count = (bytes + granule_ - 1) / granule_;
  for (size_t g = first; g < first + count; ++g) {
    auto it = mapped_.find(g);
    if (it == mapped_.end()) continue;
    memUnmap_(base_ + g * granule_, granule_);
    driver_calls_++;
    parked_.push_back(it->second);
    mapped_.erase(it);
  }
}

void VmmArena::trim() {
  for (auto h : parked_) { memRelease_(h); driver_calls_++; }
  parked_.clear();
}

}  // namespace dfb
