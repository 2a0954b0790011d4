#pragma once
#include <cuda_runtime_api.h>

#include <deque>
#include <map>
#include <vector>

#include "backend.hpp"

namespace dfb {

// CUDA streams backend: non-blocking streams, pooled timing events, cudaMalloc
// for the fast tier, mmap + cudaHostRegister for the pinned backing tier, async
// copies on the caller's stream, completion by event polling or host callbacks.
// Role parity: reference src/dataflow/runtime/device/cuda.py:109-529.
class CudaBackend : public Backend {
 public:
  explicit CudaBackend(int device, const char* completion_mode);
  ~CudaBackend() override;
  const char* name() const override { return "cuda"; }
  int create_stream(const char* label, int priority) override;
  uint64_t stream_handle(int stream) const override { return reinterpret_cast<uint64_t>(streams_[stream]); }
  int record_event(int stream) override;
  void stream_wait_event(int stream, int event) override;
  void release_event(int event) override;
  double event_time_us(int event) override;
  void mark_epoch() override;
  void* alloc(Location loc, size_t bytes) override;
  void free(Location loc, void* p, size_t bytes) override;
  std::unique_ptr<VmSpace> create_vm_space(size_t va_bytes, size_t phys_bytes) override;
  void memcpy_async(void* dst, const void* src, size_t bytes, int stream, double) override;
  void memset_async(void* dst, int value, size_t bytes, int stream) override;
  void busy(int stream, double us) override;
  void notify_after(int event, uint64_t token, int prio) override;
  Completion next_completion(bool block) override;
  size_t pending() const override { return waiting_.size(); }
  void drain_aborted() override;
  void synchronize() override;

  // pinned host regions (also used by the service store)
  void* pin_region(size_t bytes, bool populate);
  void unpin_region(void* p, size_t bytes);
  // bandwidth probe: returns GB/s for h2d, d2h, and both at once
  void measure_pcie(size_t bytes, int repeats, double out[4]);
  int device() const { return device_; }
  int64_t device_allocs = 0, host_allocs = 0;

 private:
  struct Waiting { cudaEvent_t ev; uint64_t token; int prio; uint64_t seq; };
  void check(cudaError_t e, const char* what) const;
  int device_;
  bool hostfn_mode_;
  std::vector<cudaStream_t> streams_;
  std::vector<cudaEvent_t> events_;
  std::vector<int> free_events_;
  cudaEvent_t epoch_ = nullptr;
  std::deque<Waiting> waiting_;
  uint64_t seq_ = 0;
  std::map<void*, size_t> pinned_;
};

// defined in spin.cu
void launch_spin_us(double us, cudaStream_t stream);

}  // namespace dfb
