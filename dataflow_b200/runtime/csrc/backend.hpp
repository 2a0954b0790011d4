// Device backend interface of the task executor.
//
// A backend owns streams, events, raw allocations, async copies and the
// completion-token queue.  The executor never touches a vendor API directly, so
// the same dispatch loop runs on virtual time (FakeBackend), on host memory
// (CpuBackend) and on CUDA streams (CudaBackend).  Protocol parity: reference
// src/dataflow/runtime/device/base.py:35-163 (priorities, notify_after,
// next_completion, drain_aborted, event_time_us).
#pragma once
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace dfb {

enum Location : int { FAST = 0, BACKING = 1 };

// completion priorities: lower value is handled first at equal times
constexpr int PRIO_H2D_DONE = 0;
constexpr int PRIO_D2H_DONE = 1;
constexpr int PRIO_TASK = 2;

struct Completion {
  bool valid = false;
  uint64_t token = 0;
  int prio = 0;
};

struct EngineError : std::runtime_error {
  std::string kind;
  EngineError(const std::string& k, const std::string& msg) : std::runtime_error(msg), kind(k) {}
};

class Backend {
 public:
  virtual ~Backend() = default;
  virtual const char* name() const = 0;
  virtual bool is_virtual() const { return false; }

  // streams are small integer handles; 0 = compute, 1 = h2d, 2 = d2h are created by the session
  virtual int create_stream(const char* label, int priority) = 0;
  virtual uint64_t stream_handle(int stream) const { return 0; }   // raw vendor handle (cudaStream_t)

  // events
  virtual int record_event(int stream) = 0;            // returns an event handle
  virtual void stream_wait_event(int stream, int event) = 0;
  virtual void release_event(int event) = 0;
  virtual double event_time_us(int event) = 0;          // time since the epoch event; valid once complete
  virtual void mark_epoch() = 0;

  // memory
  virtual void* alloc(Location loc, size_t bytes) = 0;
  virtual void free(Location loc, void* p, size_t bytes) = 0;
  virtual void memcpy_async(void* dst, const void* src, size_t bytes, int stream, double planned_us) = 0;
  virtual void memset_async(void* dst, int value, size_t bytes, int stream) = 0;

  // synthetic work: make ``stream`` busy for ``us`` (virtual clock or a spin kernel)
  virtual void busy(int stream, double us) = 0;

  // completion tokens
  virtual void notify_after(int event, uint64_t token, int prio) = 0;
  virtual Completion next_completion(bool block) = 0;   // invalid when nothing is pending
  virtual size_t pending() const = 0;
  virtual void drain_aborted() = 0;                      // wait for everything in flight, drop tokens
  virtual void synchronize() = 0;
};

}  // namespace dfb
