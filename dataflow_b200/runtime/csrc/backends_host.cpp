// Host-only backends: FakeBackend (virtual clock, no memory) and CpuBackend
// (real host memory, synchronous copies).  Role parity: reference
// src/dataflow/runtime/device/fake.py:18-118 for the virtual-time model; the CPU
// backend has no counterpart there (it exists so that a whole training step can
// run without a GPU).
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <queue>
#include <tuple>
#include <vector>

#include "backends_host.hpp"

namespace dfb {

// ----------------------------------------------------------------------------- Fake
int FakeBackend::create_stream(const char*, int) {
  clocks_.push_back(0.0);
  return static_cast<int>(clocks_.size()) - 1;
}

int FakeBackend::record_event(int stream) {
  double t = std::max(clocks_[stream], now_);
  int id;
  if (!free_events_.empty()) { id = free_events_.back(); free_events_.pop_back(); event_time_[id] = t; }
  else { id = static_cast<int>(event_time_.size()); event_time_.push_back(t); }
  return id;
}

void FakeBackend::stream_wait_event(int stream, int event) {
  clocks_[stream] = std::max(clocks_[stream], event_time_[event]);
}

void FakeBackend::release_event(int event) { free_events_.push_back(event); }
double FakeBackend::event_time_us(int event) { return event_time_[event]; }

void FakeBackend::mark_epoch() {
  now_ = 0.0;
  for (auto& c : clocks_) c = 0.0;
  while (!heap_.empty()) heap_.pop();
  seq_ = 0;
}

void* FakeBackend::alloc(Location, size_t bytes) {
  uintptr_t p = next_addr_;
  next_addr_ += (bytes + 4095) / 4096 * 4096 + 4096;
  return reinterpret_cast<void*>(p);
}

void FakeBackend::free(Location, void*, size_t) {}

HostVmSpace::HostVmSpace(size_t va_bytes, size_t phys_bytes, bool real, uintptr_t fake_base, size_t page) : real_(real) {
  init(page, va_bytes, phys_bytes);
  if (real) {
    if (posix_memalign(&base_, 4096, this->va_bytes()) != 0) throw EngineError("AllocError", "host range of " + std::to_string(va_bytes) + " bytes failed");
  } else {
    base_ = reinterpret_cast<void*>(fake_base);
  }
}
HostVmSpace::~HostVmSpace() {
  if (real_) std::free(base_);
}

std::unique_ptr<VmSpace> FakeBackend::create_vm_space(size_t va_bytes, size_t phys_bytes) {
  uintptr_t p = next_addr_;
  next_addr_ += (va_bytes + (2u << 20)) / 4096 * 4096 + 4096;
  return std::make_unique<HostVmSpace>(va_bytes, phys_bytes, false, p);
}

void FakeBackend::memcpy_async(void*, const void*, size_t, int stream, double planned_us) {
  busy(stream, planned_us * transfer_time_scale);
}

void FakeBackend::memset_async(void*, int, size_t, int) {}

void FakeBackend::busy(int stream, double us) {
  clocks_[stream] = std::max(clocks_[stream], now_) + us * (stream == 0 ? compute_time_scale : 1.0);
}

void FakeBackend::notify_after(int event, uint64_t token, int prio) {
  heap_.push(Item{event_time_[event], prio, seq_++, token});
}

Completion FakeBackend::next_completion(bool) {
  Completion c;
  if (heap_.empty()) return c;
  Item it = heap_.top();
  heap_.pop();
  now_ = std::max(now_, it.t);
  c.valid = true; c.token = it.token; c.prio = it.prio;
  return c;
}

void FakeBackend::drain_aborted() { while (!heap_.empty()) heap_.pop(); }

// ----------------------------------------------------------------------------- Cpu
static inline double steady_us() {
  using namespace std::chrono;
  return duration<double, std::micro>(steady_clock::now().time_since_epoch()).count();
}

int CpuBackend::create_stream(const char*, int) { return n_streams_++; }

int CpuBackend::record_event(int) {
  double t = steady_us() - epoch_;
  int id;
  if (!free_events_.empty()) { id = free_events_.back(); free_events_.pop_back(); event_time_[id] = t; }
  else { id = static_cast<int>(event_time_.size()); event_time_.push_back(t); }
  return id;
}

void CpuBackend::release_event(int event) { free_events_.push_back(event); }
double CpuBackend::event_time_us(int event) { return event_time_[event]; }
void CpuBackend::mark_epoch() { epoch_ = steady_us(); }

void* CpuBackend::alloc(Location, size_t bytes) {
  void* p = nullptr;
  if (posix_memalign(&p, 4096, bytes ? (bytes + 4095) / 4096 * 4096 : 4096) != 0)
    throw EngineError("AllocError", "host allocation of " + std::to_string(bytes) + " bytes failed");
  return p;
}

void CpuBackend::free(Location, void* p, size_t) { std::free(p); }

std::unique_ptr<VmSpace> CpuBackend::create_vm_space(size_t va_bytes, size_t phys_bytes) {
  return std::make_unique<HostVmSpace>(va_bytes, phys_bytes, true, 0);
}

void CpuBackend::memcpy_async(void* dst, const void* src, size_t bytes, int, double) {
  if (bytes) std::memcpy(dst, src, bytes);
}

void CpuBackend::memset_async(void* dst, int value, size_t bytes, int) { std::memset(dst, value, bytes); }

void CpuBackend::busy(int, double us) {
  if (!spin_busy) return;
  double t0 = steady_us();
  while (steady_us() - t0 < us) {}
}

void CpuBackend::notify_after(int, uint64_t token, int prio) { done_.push_back({token, prio}); }

Completion CpuBackend::next_completion(bool) {
  Completion c;
  if (done_.empty()) return c;
  // everything has already happened; among the finished items honour the priority order
  size_t best = 0;
  for (size_t i = 1; i < done_.size(); ++i)
    if (done_[i].second < done_[best].second) best = i;
  c.valid = true; c.token = done_[best].first; c.prio = done_[best].second;
  done_.erase(done_.begin() + best);
  return c;
}

}  // namespace dfb
