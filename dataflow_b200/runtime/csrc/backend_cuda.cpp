#include "backend_cuda.hpp"
#include "vmm.hpp"

#include <sched.h>
#include <sys/mman.h>

#include <algorithm>
#include <string>

namespace dfb {

void CudaBackend::check(cudaError_t e, const char* what) const {
  if (e != cudaSuccess)
    throw EngineError("CudaError", std::string(what) + ": " + cudaGetErrorString(e));
}

CudaBackend::CudaBackend(int device, const char* completion_mode)
    : device_(device), hostfn_mode_(completion_mode && std::string(completion_mode) == "hostfn") {
  check(cudaSetDevice(device_), "cudaSetDevice");
  check(cudaEventCreate(&epoch_), "cudaEventCreate");
}

CudaBackend::~CudaBackend() {
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  for (auto e : events_) cudaEventDestroy(e);
  if (epoch_) cudaEventDestroy(epoch_);
  for (auto s : streams_) cudaStreamDestroy(s);
  for (auto& kv : pinned_) { cudaHostUnregister(kv.first); munmap(kv.first, kv.second); }
}

int CudaBackend::create_stream(const char*, int priority) {
  cudaStream_t s;
  int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);
  int pr = std::max(hi, std::min(lo, priority));
  check(cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, pr), "cudaStreamCreateWithPriority");
  streams_.push_back(s);
  return static_cast<int>(streams_.size()) - 1;
}

int CudaBackend::record_event(int stream) {
  int id;
  if (!free_events_.empty()) { id = free_events_.back(); free_events_.pop_back(); }
  else {
    cudaEvent_t e;
    check(cudaEventCreate(&e), "cudaEventCreate");
    events_.push_back(e);
    id = static_cast<int>(events_.size()) - 1;
  }
  check(cudaEventRecord(events_[id], streams_[stream]), "cudaEventRecord");
  return id;
}

void CudaBackend::stream_wait_event(int stream, int event) {
  check(cudaStreamWaitEvent(streams_[stream], events_[event], 0), "cudaStreamWaitEvent");
}

void CudaBackend::release_event(int event) { free_events_.push_back(event); }

double CudaBackend::event_time_us(int event) {
  float ms = 0.f;
  check(cudaEventSynchronize(events_[event]), "cudaEventSynchronize");
  check(cudaEventElapsedTime(&ms, epoch_, events_[event]), "cudaEventElapsedTime");
  return static_cast<double>(ms) * 1000.0;
}

void CudaBackend::mark_epoch() {
  // the epoch rides the compute stream (stream 0) after everything already queued there
  check(cudaEventRecord(epoch_, streams_.empty() ? nullptr : streams_[0]), "cudaEventRecord(epoch)");
}

void* CudaBackend::pin_region(size_t bytes, bool populate) {
  size_t len = (bytes + (2u << 20) - 1) / (2u << 20) * (2u << 20);
  int flags = MAP_PRIVATE | MAP_ANONYMOUS | (populate ? MAP_POPULATE : 0);
  void* p = mmap(nullptr, len, PROT_READ | PROT_WRITE, flags, -1, 0);
  if (p == MAP_FAILED) throw EngineError("AllocError", "mmap of " + std::to_string(len) + " bytes failed");
  cudaError_t e = cudaHostRegister(p, len, cudaHostRegisterPortable | cudaHostRegisterMapped);
  if (e != cudaSuccess) {
    munmap(p, len);
    check(e, "cudaHostRegister");
  }
  pinned_[p] = len;
  host_allocs++;
  return p;
}

void CudaBackend::unpin_region(void* p, size_t) {
  auto it = pinned_.find(p);
  if (it == pinned_.end()) return;
  cudaHostUnregister(p);
  munmap(p, it->second);
  pinned_.erase(it);
}

void* CudaBackend::alloc(Location loc, size_t bytes) {
  if (loc == FAST) {
    void* p = nullptr;
    check(cudaMalloc(&p, bytes ? bytes : 1), "cudaMalloc");
    device_allocs++;
    return p;
  }
  return pin_region(bytes ? bytes : 1, true);
}

std::unique_ptr<VmSpace> CudaBackend::create_vm_space(size_t va_bytes, size_t phys_bytes) {
  check(cudaSetDevice(device_), "cudaSetDevice");
  return std::make_unique<CudaVmSpace>(device_, va_bytes, phys_bytes);
}

void CudaBackend::free(Location loc, void* p, size_t bytes) {
  if (loc == FAST) cudaFree(p);
  else unpin_region(p, bytes);
}

void CudaBackend::memcpy_async(void* dst, const void* src, size_t bytes, int stream, double) {
  if (!bytes) return;
  check(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, streams_[stream]), "cudaMemcpyAsync");
}

void CudaBackend::memset_async(void* dst, int value, size_t bytes, int stream) {
  if (!bytes) return;
  check(cudaMemsetAsync(dst, value, bytes, streams_[stream]), "cudaMemsetAsync");
}

void CudaBackend::busy(int stream, double us) { launch_spin_us(us, streams_[stream]); }

void CudaBackend::notify_after(int event, uint64_t token, int prio) {
  waiting_.push_back({events_[event], token, prio, seq_++});
}

Completion CudaBackend::next_completion(bool block) {
  Completion c;
  if (waiting_.empty()) return c;
  for (;;) {
    // among the events that have completed, the lowest (priority, seq) wins
    int best = -1;
    for (size_t i = 0; i < waiting_.size(); ++i) {
      cudaError_t q = cudaEventQuery(waiting_[i].ev);
      if (q == cudaSuccess) {
        if (best < 0 || waiting_[i].prio < waiting_[best].prio) best = static_cast<int>(i);
      } else if (q != cudaErrorNotReady) {
        check(q, "cudaEventQuery");
      }
    }
    if (best >= 0) {
      c.valid = true; c.token = waiting_[best].token; c.prio = waiting_[best].prio;
      waiting_.erase(waiting_.begin() + best);
      return c;
    }
    if (!block) return c;
    sched_yield();
  }
}

void CudaBackend::drain_aborted() {
  for (auto s : streams_) cudaStreamSynchronize(s);
  waiting_.clear();
}

void CudaBackend::synchronize() {
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
}

void CudaBackend::measure_pcie(size_t bytes, int repeats, double out[4]) {
  void* h0 = pin_region(bytes, true);
  void* h1 = pin_region(bytes, true);
  void *d0 = nullptr, *d1 = nullptr;
  check(cudaMalloc(&d0, bytes), "cudaMalloc");
  check(cudaMalloc(&d1, bytes), "cudaMalloc");
  cudaStream_t a, b;
  cudaStreamCreateWithFlags(&a, cudaStreamNonBlocking);
  cudaStreamCreateWithFlags(&b, cudaStreamNonBlocking);
  cudaEvent_t e0, e1, f0, f1;
  cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventCreate(&f0); cudaEventCreate(&f1);
  auto gbs = [&](float ms, double n) { return n * bytes / (ms * 1e-3) / 1e9; };
  float ms;
  cudaMemcpyAsync(d0, h0, bytes, cudaMemcpyDefault, a); cudaStreamSynchronize(a);   // warm
  cudaEventRecord(e0, a);
  for (int i = 0; i < repeats; ++i) cudaMemcpyAsync(d0, h0, bytes, cudaMemcpyDefault, a);
  cudaEventRecord(e1, a); cudaEventSynchronize(e1); cudaEventElapsedTime(&ms, e0, e1);
  out[0] = gbs(ms, repeats);
  cudaEventRecord(e0, a);
  for (int i = 0; i < repeats; ++i) cudaMemcpyAsync(h1, d1, bytes, cudaMemcpyDefault, a);
  cudaEventRecord(e1, a); cudaEventSynchronize(e1); cudaEventElapsedTime(&ms, e0, e1);
  out[1] = gbs(ms, repeats);
  cudaEventRecord(e0, a); cudaEventRecord(f0, b);
  for (int i = 0; i < repeats; ++i) {
    cudaMemcpyAsync(d0, h0, bytes, cudaMemcpyDefault, a);
    cudaMemcpyAsync(h1, d1, bytes, cudaMemcpyDefault, b);
  }
  cudaEventRecord(e1, a); cudaEventRecord(f1, b);
  cudaEventSynchronize(e1); cudaEventSynchronize(f1);
  cudaEventElapsedTime(&ms, e0, e1); out[2] = gbs(ms, repeats);
  cudaEventElapsedTime(&ms, f0, f1); out[3] = gbs(ms, repeats);
  cudaEventDestroy(e0); cudaEventDestroy(e1); cudaEventDestroy(f0); cudaEventDestroy(f1);
  cudaStreamDestroy(a); cudaStreamDestroy(b);
  cudaFree(d0); cudaFree(d1);
  unpin_region(h0, bytes); unpin_region(h1, bytes);
}

}  // namespace dfb
