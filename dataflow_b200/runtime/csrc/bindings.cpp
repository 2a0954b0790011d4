// Python bindings of the native runtime (pybind11): backends, session, executor,
// slab allocator.  The module never imports torch.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <atomic>
#include <cstring>

#include "backends_host.hpp"
#include "engine.hpp"
#ifdef DFB_WITH_CUDA
#include <nvtx3/nvToolsExt.h>

#include "backend_cuda.hpp"
#endif

namespace py = pybind11;
using namespace dfb;

static std::atomic<bool> g_nvtx{false};

static py::dict result_to_py(const RunResult& r) {
  py::dict d;
  d["outcome"] = r.outcome;
  d["message"] = r.message;
  d["failed_task"] = r.failed_task;
  d["error_kind"] = r.error_kind;
  py::list iv;
  for (auto& i : r.intervals) iv.append(py::make_tuple(i.name, i.track, i.start, i.end));
  d["intervals"] = iv;
  py::list ev;
  for (auto& e : r.events) ev.append(py::make_tuple(e.kind, e.what, e.fast_bytes));
  d["events"] = ev;
  py::list al;
  for (auto& a : r.allocs) al.append(py::make_tuple(a.obj, a.size, a.ptr, a.kind));
  d["allocs"] = al;
  py::dict s;
  s["makespan_us"] = r.stats.makespan_us;
  s["peak_fast_bytes"] = r.stats.peak_fast;
  s["peak_backing_bytes"] = r.stats.peak_backing;
  s["slab_overflows"] = r.stats.slab_overflows;
  s["vendor_allocs"] = r.stats.vendor_allocs;
  s["pressure_evictions"] = r.stats.pressure_evictions;
  s["placement_escapes"] = r.stats.placement_escapes;
  s["h2d_bytes"] = r.stats.h2d_bytes;
  s["d2h_bytes"] = r.stats.d2h_bytes;
  s["h2d_count"] = r.stats.h2d_count;
  s["d2h_count"] = r.stats.d2h_count;
  s["dispatch_us_total"] = r.stats.dispatch_us_total;
  s["wait_us_total"] = r.stats.wait_us_total;
  d["stats"] = s;
  py::dict f;
  for (auto& b : r.finals) f[py::str(b.id)] = py::make_tuple(b.loc, b.ptr, b.size, b.external);
  d["finals"] = f;
  return d;
}

static py::dict pool_stats(BufferPool& pool) {
  py::dict d;
  d["mode"] = pool.vm_active() ? "vmm" : "slab";
  d["capacity"] = pool.slab_capacity();
  d["overflows"] = pool.slab_overflows;
  d["vendor_allocs"] = pool.vendor_allocs;
  d["used"] = pool.slab_used();
  d["peak"] = pool.slab_peak();
  d["largest_free"] = pool.slab_largest_free();
  py::list log;
  for (auto& o : pool.overflow_log) log.append(py::make_tuple(o.asked, o.used, o.largest_free));
  d["overflow_log"] = log;
  if (const VmSpace* vm = pool.vm()) {
    d["page"] = vm->page();
    d["va_bytes"] = vm->va_bytes();
    d["phys_pages"] = vm->phys_pages();
    d["held_pages"] = vm->held_pages();
    d["mapped_pages"] = vm->mapped_pages();
    d["maps"] = vm->maps;
    d["reclaims"] = vm->reclaims;
  }
  return d;
}

PYBIND11_MODULE(_runtime, m) {
  m.doc() = "dataflow_b200 native runtime: backends, session, task executor";
  m.attr("PRIO_H2D_DONE") = PRIO_H2D_DONE;
  m.attr("PRIO_D2H_DONE") = PRIO_D2H_DONE;
  m.attr("PRIO_TASK") = PRIO_TASK;
#ifdef DFB_WITH_CUDA
  m.attr("with_cuda") = true;
#else
  m.attr("with_cuda") = false;
#endif

  py::class_<Backend, std::shared_ptr<Backend>>(m, "Backend")
      .def("name", &Backend::name)
      .def("is_virtual", &Backend::is_virtual)
      .def("synchronize", &Backend::synchronize)
      .def("pending", &Backend::pending)
      .def("create_stream", &Backend::create_stream)
      .def("stream_handle", &Backend::stream_handle)
      .def("record_event", &Backend::record_event)
      .def("release_event", &Backend::release_event)
      .def("event_time_us", &Backend::event_time_us)
      .def("mark_epoch", &Backend::mark_epoch)
      .def("busy", &Backend::busy)
      .def("alloc", [](Backend& b, int loc, size_t n) { return reinterpret_cast<uint64_t>(b.alloc(static_cast<Location>(loc), n)); })
      .def("free", [](Backend& b, int loc, uint64_t p, size_t n) { b.free(static_cast<Location>(loc), reinterpret_cast<void*>(p), n); })
      .def("memcpy_async", [](Backend& b, uint64_t dst, uint64_t src, size_t n, int stream) {
        b.memcpy_async(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), n, stream, 0.0);
      })
      .def("memset_async", [](Backend& b, uint64_t dst, int v, size_t n, int stream) {
        b.memset_async(reinterpret_cast<void*>(dst), v, n, stream);
      });

  py::class_<FakeBackend, Backend, std::shared_ptr<FakeBackend>>(m, "FakeBackend")
      .def(py::init<>())
      .def_readwrite("transfer_time_scale", &FakeBackend::transfer_time_scale)
      .def_readwrite("compute_time_scale", &FakeBackend::compute_time_scale)
      .def("now", &FakeBackend::now);

  py::class_<CpuBackend, Backend, std::shared_ptr<CpuBackend>>(m, "CpuBackend")
      .def(py::init<>())
      .def_readwrite("spin_busy", &CpuBackend::spin_busy);

#ifdef DFB_WITH_CUDA
  py::class_<CudaBackend, Backend, std::shared_ptr<CudaBackend>>(m, "CudaBackend")
      .def(py::init<int, const char*>(), py::arg("device") = 0, py::arg("completion") = "poll")
      .def("device", &CudaBackend::device)
      .def_readonly("device_allocs", &CudaBackend::device_allocs)
      .def_readonly("host_allocs", &CudaBackend::host_allocs)
      .def("pin_region", [](CudaBackend& b, size_t n, bool populate) {
        py::gil_scoped_release rel;
        return reinterpret_cast<uint64_t>(b.pin_region(n, populate));
      }, py::arg("bytes"), py::arg("populate") = true)
      .def("unpin_region", [](CudaBackend& b, uint64_t p, size_t n) { b.unpin_region(reinterpret_cast<void*>(p), n); })
      .def("ipc_handle", [](CudaBackend&, uint64_t ptr) {
        cudaIpcMemHandle_t h;
        cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(ptr));
        if (e != cudaSuccess) throw std::runtime_error(std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
        return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
      })
      .def("ipc_open", [](CudaBackend&, py::bytes handle) {
        std::string s = handle;
        if (s.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("bad IPC handle size");
        cudaIpcMemHandle_t h;
        std::memcpy(&h, s.data(), sizeof(h));
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) throw std::runtime_error(std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
        return reinterpret_cast<uint64_t>(p);
      })
      .def("ipc_close", [](CudaBackend&, uint64_t ptr) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); })
      .def("device_alloc_zeroed", [](CudaBackend&, size_t n) {
        void* p = nullptr;
        if (cudaMalloc(&p, n) != cudaSuccess) throw std::runtime_error("cudaMalloc failed");
        cudaMemset(p, 0, n);
        cudaDeviceSynchronize();
        return reinterpret_cast<uint64_t>(p);
      })
      .def("device_free", [](CudaBackend&, uint64_t p) { cudaFree(reinterpret_cast<void*>(p)); })
      .def("measure_pcie", [](CudaBackend& b, size_t bytes, int repeats) {
        double out[4];
        {
          py::gil_scoped_release rel;
          b.measure_pcie(bytes, repeats, out);
        }
        py::dict d;
        d["h2d_gbs"] = out[0]; d["d2h_gbs"] = out[1]; d["h2d_bidi_gbs"] = out[2]; d["d2h_bidi_gbs"] = out[3];
        return d;
      }, py::arg("bytes") = (256u << 20), py::arg("repeats") = 4);

  // One buffer pool on its own (tests of the pool modes; the engine owns its pools through Session).
  struct PoolProbe {
    std::shared_ptr<Backend> be;
    BufferPool pool;
    std::map<int, BufferRef> live;
    int next = 0;
    PoolProbe(std::shared_ptr<Backend> b, size_t capacity, bool vm, double va_factor) : be(std::move(b)), pool(be.get(), FAST) {
      pool.set_vm_mode(vm, va_factor);
      pool.ensure_slab(capacity);
    }
  };
  py::class_<PoolProbe>(m, "PoolProbe")
      .def(py::init<std::shared_ptr<Backend>, size_t, bool, double>(), py::arg("backend"), py::arg("capacity"), py::arg("vm") = false,
           py::arg("va_factor") = 2.0)
      .def("get", [](PoolProbe& p, size_t bytes) {
        BufferRef b = p.pool.get(bytes);
        int h = p.next++;
        p.live[h] = b;
        return py::make_tuple(h, reinterpret_cast<uint64_t>(b.ptr), b.overflow);
      })
      .def("put", [](PoolProbe& p, int h) {
        auto it = p.live.find(h);
        if (it == p.live.end()) throw std::runtime_error("unknown pool handle");
        p.pool.put(it->second);
        p.live.erase(it);
      })
      .def("stats", [](PoolProbe& p) { return pool_stats(p.pool); });
  m.def("set_nvtx", [](bool on) { g_nvtx.store(on); });
  m.def("nvtx_mark", [](const std::string& s) { if (g_nvtx.load()) nvtxMarkA(s.c_str()); });
  m.def("nvtx_push", [](const std::string& s) { nvtxRangePushA(s.c_str()); });
  m.def("nvtx_pop", []() { nvtxRangePop(); });
#else
  m.def("set_nvtx", [](bool) {});
  m.def("nvtx_mark", [](const std::string&) {});
  m.def("nvtx_push", [](const std::string&) {});
  m.def("nvtx_pop", []() {});
#endif

  py::class_<SlabAllocator>(m, "SlabAllocator")
      .def(py::init<size_t, size_t>(), py::arg("capacity"), py::arg("align") = 512)
      .def("allocate", [](SlabAllocator& s, size_t n) -> py::object {
        size_t off = s.allocate(n);
        if (off == SlabAllocator::kNone) return py::none();
        return py::int_(off);
      })
      .def("allocate_at", &SlabAllocator::allocate_at)
      .def("release", &SlabAllocator::release)
      .def("capacity", &SlabAllocator::capacity)
      .def("used", &SlabAllocator::used)
      .def("peak", &SlabAllocator::peak)
      .def("largest_free", &SlabAllocator::largest_free)
      .def("live_blocks", &SlabAllocator::live_blocks)
      .def("block_size", &SlabAllocator::block_size);

  py::class_<ObjIR>(m, "ObjIR").def(py::init<>())
      .def_readwrite("id", &ObjIR::id).def_readwrite("size", &ObjIR::size)
      .def_readwrite("init_fast", &ObjIR::init_fast).def_readwrite("init_backing", &ObjIR::init_backing)
      .def_readwrite("final_loc", &ObjIR::final_loc).def_readwrite("last_ref", &ObjIR::last_ref);
  py::class_<TaskIR>(m, "TaskIR").def(py::init<>())
      .def_readwrite("id", &TaskIR::id).def_readwrite("inputs", &TaskIR::inputs)
      .def_readwrite("mutates", &TaskIR::mutates).def_readwrite("releases", &TaskIR::releases)
      .def_readwrite("runtime_us", &TaskIR::runtime_us).def_readwrite("workspace", &TaskIR::workspace)
      .def("add_output", [](TaskIR& t, int obj, int loc) { t.outputs.push_back({obj, loc}); })
      .def("add_offload", [](TaskIR& t, int obj, double us) { t.offloads.push_back({obj, us}); })
      .def("add_prefetch", [](TaskIR& t, int obj, double us) { t.prefetches.push_back({obj, us}); });
  py::class_<ProgramIR, std::shared_ptr<ProgramIR>>(m, "ProgramIR").def(py::init<>())
      .def_readwrite("name", &ProgramIR::name)
      .def_readwrite("fast_cap", &ProgramIR::fast_cap).def_readwrite("backing_cap", &ProgramIR::backing_cap)
      .def_readwrite("bw_from", &ProgramIR::bw_from).def_readwrite("bw_to", &ProgramIR::bw_to)
      .def("add_obj", [](ProgramIR& p, const ObjIR& o) { p.objs.push_back(o); return p.objs.size() - 1; })
      .def("add_task", [](ProgramIR& p, const TaskIR& t) { p.tasks.push_back(t); return p.tasks.size() - 1; })
      .def("num_tasks", [](ProgramIR& p) { return p.tasks.size(); })
      .def("num_objs", [](ProgramIR& p) { return p.objs.size(); });

  py::class_<Session, std::shared_ptr<Session>>(m, "Session")
      .def(py::init<std::shared_ptr<Backend>>())
      .def_readonly("compute_stream", &Session::compute_stream)
      .def_readonly("h2d_stream", &Session::h2d_stream)
      .def_readonly("d2h_stream", &Session::d2h_stream)
      .def("ensure_pools", &Session::ensure_pools, py::arg("fast_cap"), py::arg("backing_cap"), py::arg("headroom") = 0.0,
           py::arg("fast_vm") = false)
      .def("fast_pool_stats", [](Session& s) { return pool_stats(s.fast_pool); })
      .def("backing_pool_stats", [](Session& s) { return pool_stats(s.backing_pool); })
      .def("set_fast_policy", [](Session& s, size_t large_div, bool best_fit) { s.fast_pool.set_policy(large_div, best_fit); },
           py::arg("large_div") = 48, py::arg("best_fit") = false)
      .def("fast_slab", [](Session& s) { return py::make_tuple(reinterpret_cast<uint64_t>(s.fast_pool.slab_base()), s.fast_pool.slab_capacity()); })
      .def("set_fast_tail", [](Session& s, size_t bytes) { s.fast_pool.set_tail(bytes); })
      .def("fast_tail", [](Session& s) { return s.fast_pool.slab_tail(); })
      .def("backing_slab", [](Session& s) { return py::make_tuple(reinterpret_cast<uint64_t>(s.backing_pool.slab_base()), s.backing_pool.slab_capacity()); })
      .def("vendor_allocs", [](Session& s) { return s.fast_pool.vendor_allocs + s.backing_pool.vendor_allocs; })
      .def("trim", [](Session& s) { s.fast_pool.trim(); s.backing_pool.trim(); })
      .def("resident", [](Session& s) {
        py::dict d;
        for (auto& kv : s.resident) d[py::str(kv.first)] = py::make_tuple(reinterpret_cast<uint64_t>(kv.second.ptr), kv.second.size);
        return d;
      })
      .def("drop_resident", [](Session& s) { s.drop_resident(); });

  py::class_<std::atomic<bool>, std::shared_ptr<std::atomic<bool>>>(m, "CancelFlag")
      .def(py::init([]() { return std::make_shared<std::atomic<bool>>(false); }))
      .def("set", [](std::atomic<bool>& f) { f.store(true); })
      .def("clear", [](std::atomic<bool>& f) { f.store(false); })
      .def("is_set", [](std::atomic<bool>& f) { return f.load(); });

  py::class_<Engine>(m, "Engine")
      .def(py::init<std::shared_ptr<Session>>())
      .def("execute",
           [](Engine& e, std::shared_ptr<ProgramIR> p, py::object launch, py::dict initial,
              bool strict_final, bool poison, bool record_events, double headroom,
              std::shared_ptr<std::atomic<bool>> cancel, bool manage_pools, bool keep_resident, int dispatch_ahead,
              bool record_allocs, std::vector<std::vector<int64_t>> placement, py::object annotate) {
             std::unordered_map<std::string, InitialBuffer> init;
             for (auto kv : initial) {
               auto t = kv.second.cast<py::tuple>();
               init[kv.first.cast<std::string>()] = {t[0].cast<uint64_t>(), t[1].cast<size_t>(), t[2].cast<int>()};
             }
             ExecOptions opt;
             opt.strict_final_locations = strict_final;
             opt.poison_on_free = poison;
             opt.record_events = record_events;
             opt.slab_headroom = headroom;
             opt.cancel = cancel ? cancel.get() : nullptr;
             opt.manage_pools = manage_pools;
             opt.keep_resident = keep_resident;
             opt.dispatch_ahead = dispatch_ahead;
             opt.record_allocs = record_allocs;
             if (!placement.empty()) opt.placement = &placement;
             LaunchFn fn;
             if (!launch.is_none()) {
               fn = [launch](const LaunchArgs& a) {
                 py::gil_scoped_acquire gil;
                 launch(a.task_index, a.input_ptrs, a.output_ptrs, a.stream_handle);
               };
             }
             RangeFn range;
             if (!annotate.is_none()) {
               // a Python annotator (recording, renaming, or NVTX through nvtx_push / nvtx_pop): called with the GIL
               range = [annotate](const std::string& name, bool push) {
                 py::gil_scoped_acquire gil;
                 annotate(name, push);
               };
             }
#ifdef DFB_WITH_CUDA
             else if (g_nvtx.load()) {
               range = [](const std::string& name, bool push) {
                 if (push) nvtxRangePushA(name.c_str()); else nvtxRangePop();
               };
             }
#endif
             RunResult r;
             {
               py::gil_scoped_release rel;
               r = e.execute(*p, fn, init, opt, range);
             }
             return result_to_py(r);
           },
           py::arg("program"), py::arg("launch") = py::none(), py::arg("initial") = py::dict(),
           py::arg("strict_final_locations") = true, py::arg("poison_on_free") = false,
           py::arg("record_events") = false, py::arg("slab_headroom") = 0.0,
           py::arg("cancel") = std::shared_ptr<std::atomic<bool>>(), py::arg("manage_pools") = true,
           py::arg("keep_resident") = false, py::arg("dispatch_ahead") = 0, py::arg("record_allocs") = false,
           py::arg("placement") = std::vector<std::vector<int64_t>>(), py::arg("annotate") = py::none());
}
