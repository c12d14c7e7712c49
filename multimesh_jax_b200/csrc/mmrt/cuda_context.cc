#include "cuda_context.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <sstream>
#include <stdexcept>

namespace mmrt {

// ---------------------------------------------------------------------------
// The CUDA runtime behind GpuApi
// ---------------------------------------------------------------------------
namespace {

class RuntimeApi : public GpuApi {
 public:
  RuntimeApi() {
    // NVTX ranges are optional: the tools library is looked up at run time, never linked
    for (const char* name : {"libnvToolsExt.so.1", "libnvToolsExt.so"}) {
      void* h = dlopen(name, RTLD_LAZY | RTLD_LOCAL);
      if (!h) continue;
      push_ = reinterpret_cast<int (*)(const char*)>(dlsym(h, "nvtxRangePushA"));
      pop_ = reinterpret_cast<int (*)()>(dlsym(h, "nvtxRangePop"));
      mark_ = reinterpret_cast<void (*)(const char*)>(dlsym(h, "nvtxMarkA"));
      if (push_ && pop_) break;
    }
  }
  bool SetDevice(int ordinal) override { return Ok(cudaSetDevice(ordinal)); }
  void PriorityRange(int* least, int* greatest) override {
    if (!Ok(cudaDeviceGetStreamPriorityRange(least, greatest))) *least = *greatest = 0;
  }
  // Streams are cached for the life of the process (the reference keeps a stream cache too,
  // src/pjrt_client/mm_utils.cc:44-70): a context that shuts down parks its side streams here
  // and the next context on that device takes them over. They are never destroyed, because
  // memory blocks of the caching allocator may still carry them as "used on this stream"
  // marks and would record an event on them when they are freed.
  void* CreateStream(int priority) override {
    int dev = 0;
    cudaGetDevice(&dev);
    auto& parked = parked_[{dev, priority}];
    if (!parked.empty()) {
      void* s = parked.back();
      parked.pop_back();
      where_[s] = {dev, priority};
      return s;
    }
    cudaStream_t s = nullptr;
    if (!Ok(cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, priority))) return nullptr;
    where_[s] = {dev, priority};
    return s;
  }
  void DestroyStream(void* stream) override {
    auto it = where_.find(stream);
    if (it != where_.end()) parked_[it->second].push_back(stream);
  }
  void* CreateEvent(bool timing) override {
    cudaEvent_t e = nullptr;
    return Ok(cudaEventCreateWithFlags(&e, timing ? cudaEventDefault : cudaEventDisableTiming)) ? e : nullptr;
  }
  void DestroyEvent(void* event) override { cudaEventDestroy(static_cast<cudaEvent_t>(event)); }
  bool RecordEvent(void* event, void* stream) override {
    return Ok(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
  }
  bool StreamWaitEvent(void* stream, void* event) override {
    return Ok(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
  }
  bool EventSynchronize(void* event) override { return Ok(cudaEventSynchronize(static_cast<cudaEvent_t>(event))); }
  bool EventDone(void* event) override {
    const cudaError_t e = cudaEventQuery(static_cast<cudaEvent_t>(event));
    if (e == cudaErrorNotReady) { cudaGetLastError(); return false; }
    return Ok(e);
  }
  float ElapsedMs(void* start, void* stop) override {
    float ms = 0.f;
    return Ok(cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop))) ? ms : -1.f;
  }
  bool StreamSynchronize(void* stream) override { return Ok(cudaStreamSynchronize(static_cast<cudaStream_t>(stream))); }
  void* Malloc(size_t bytes) override {
    void* p = nullptr;
    return Ok(cudaMalloc(&p, bytes)) ? p : nullptr;
  }
  void Free(void* ptr) override { cudaFree(ptr); }
  void RangePush(const std::string& name) override { if (push_) push_(name.c_str()); }
  void RangePop() override { if (pop_) pop_(); }
  void Mark(const std::string& name) override { if (mark_) mark_(name.c_str()); }
  std::string LastError() override { return last_; }

 private:
  bool Ok(cudaError_t e) {
    if (e == cudaSuccess) return true;
    last_ = cudaGetErrorString(e);
    cudaGetLastError();
    return false;
  }
  std::string last_;
  std::map<std::pair<int, int>, std::vector<void*>> parked_;   // (device, priority) -> idle streams
  std::map<void*, std::pair<int, int>> where_;
  int (*push_)(const char*) = nullptr;
  int (*pop_)() = nullptr;
  void (*mark_)(const char*) = nullptr;
};

std::string S(void* p) { return std::to_string(reinterpret_cast<intptr_t>(p)); }

}  // namespace

GpuApi* CudaRuntimeApi() {
  static RuntimeApi api;
  return &api;
}

// ---------------------------------------------------------------------------
// FakeGpuApi
// ---------------------------------------------------------------------------
bool FakeGpuApi::SetDevice(int ordinal) { trace.push_back("device " + std::to_string(ordinal)); return true; }
void* FakeGpuApi::CreateStream(int priority) {
  stream_priorities.push_back(priority);
  trace.push_back("stream s" + std::to_string(next_stream_) + " priority " + std::to_string(priority));
  return reinterpret_cast<void*>(next_stream_++);
}
void* FakeGpuApi::CreateEvent(bool) { return reinterpret_cast<void*>(next_event_++); }
bool FakeGpuApi::RecordEvent(void* event, void* stream) { trace.push_back("record e" + S(event) + " s" + S(stream)); return true; }
bool FakeGpuApi::StreamWaitEvent(void* stream, void* event) { trace.push_back("wait s" + S(stream) + " e" + S(event)); return true; }
bool FakeGpuApi::EventSynchronize(void* event) { trace.push_back("sync e" + S(event)); return true; }
bool FakeGpuApi::StreamSynchronize(void* stream) { trace.push_back("sync s" + S(stream)); return true; }
void* FakeGpuApi::Malloc(size_t bytes) {
  const intptr_t p = next_ptr_;
  next_ptr_ += static_cast<intptr_t>((bytes + 4095) / 4096 * 4096) + 4096;
  allocations_[p] = bytes;
  bytes_allocated += static_cast<int64_t>(bytes);
  trace.push_back("malloc " + std::to_string(bytes));
  return reinterpret_cast<void*>(p);
}
void FakeGpuApi::Free(void* ptr) {
  auto it = allocations_.find(reinterpret_cast<intptr_t>(ptr));
  if (it == allocations_.end()) return;
  bytes_allocated -= static_cast<int64_t>(it->second);
  allocations_.erase(it);
  trace.push_back("free");
}

// ---------------------------------------------------------------------------
// CudaContext
// ---------------------------------------------------------------------------
CudaContext::Event::~Event() {
  if (!handle || !owner) return;
  (timing ? owner->free_timing_events_ : owner->free_events_).push_back(handle);
}

CudaContext::CudaContext(std::vector<int> local_devices, std::vector<int> ordinals, std::vector<uintptr_t> compute_streams,
                         GpuApi* api, bool record_submissions)
    : api_(api), record_(record_submissions), epoch_(Clock::now()) {
  if (local_devices.size() != ordinals.size() || local_devices.size() != compute_streams.size())
    throw std::runtime_error("mmrt: one CUDA ordinal and one compute stream per local device");
  for (size_t i = 0; i < local_devices.size(); ++i) {
    Device d;
    d.id = local_devices[i];
    d.ordinal = ordinals[i];
    if (!api_->SetDevice(d.ordinal)) throw std::runtime_error("mmrt: cannot select CUDA device: " + api_->LastError());
    int least = 0, greatest = 0;
    api_->PriorityRange(&least, &greatest);   // numerically lower = higher priority
    d.stream[kComputeStream] = reinterpret_cast<void*>(compute_streams[i]);
    d.stream[kCommStream] = api_->CreateStream(greatest);
    d.stream[kAuxStream] = api_->CreateStream(least);
    d.owned[kCommStream] = d.owned[kAuxStream] = true;
    if (!d.stream[kCommStream] || !d.stream[kAuxStream])
      throw std::runtime_error("mmrt: stream creation failed: " + api_->LastError());
    devices_.push_back(d);
  }
}

CudaContext::~CudaContext() {
  Shutdown();
}

void CudaContext::Shutdown() {
  if (shutdown_) return;
  shutdown_ = true;
  Synchronize();
  tiles_.clear();
  timers_.clear();
  window_events_.clear();
  for (auto& d : devices_) {
    d.last_strict = Access{};
    for (auto& e : d.last_event) e = nullptr;
    api_->SetDevice(d.ordinal);
    for (int k = 0; k < kNumStreamKinds; ++k)
      if (d.owned[k] && d.stream[k]) { api_->DestroyStream(d.stream[k]); d.stream[k] = nullptr; }
    if (d.scratch) { api_->Free(d.scratch); d.scratch = nullptr; d.scratch_bytes = 0; }
  }
  for (void* e : free_events_) api_->DestroyEvent(e);
  for (void* e : free_timing_events_) api_->DestroyEvent(e);
  free_events_.clear();
  free_timing_events_.clear();
}

double CudaContext::NowUs() const { return std::chrono::duration<double, std::micro>(Clock::now() - epoch_).count(); }

CudaContext::Device& CudaContext::DeviceOf(int device) {
  for (auto& d : devices_) if (d.id == device) return d;
  throw std::runtime_error("mmrt: device " + std::to_string(device) + " is not local to this process");
}
const CudaContext::Device& CudaContext::DeviceOf(int device) const {
  for (auto& d : devices_) if (d.id == device) return d;
  throw std::runtime_error("mmrt: device " + std::to_string(device) + " is not local to this process");
}

uintptr_t CudaContext::StreamHandle(int device, int kind) const {
  if (kind < 0 || kind >= kNumStreamKinds) throw std::runtime_error("mmrt: unknown stream kind");
  return reinterpret_cast<uintptr_t>(DeviceOf(device).stream[kind]);
}

CudaContext::EventPtr CudaContext::NewEvent(bool timing) {
  auto& pool = timing ? free_timing_events_ : free_events_;
  void* h = nullptr;
  if (!pool.empty()) { h = pool.back(); pool.pop_back(); }
  else h = api_->CreateEvent(timing);
  if (!h) throw std::runtime_error("mmrt: event creation failed: " + api_->LastError());
  auto e = std::make_shared<Event>();
  e->handle = h;
  e->owner = this;
  e->timing = timing;
  return e;
}

void CudaContext::Fail(Status status, const std::string& message, int step) {
  if (error_ != Status::kOk) return;
  error_ = status;
  error_message_ = message;
  failed_step_ = step;
}

uint64_t CudaContext::CreateExecuteTask(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes,
                                        Body body, const ExecuteOptions& options) {
  return Submit(device, reads, writes, std::move(body), options);
}
uint64_t CudaContext::Reshard(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes, Body body,
                              const ExecuteOptions& options) {
  ExecuteOptions o = options;
  o.kind = 1;
  return Submit(device, reads, writes, std::move(body), o);
}

uint64_t CudaContext::Submit(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes, Body body,
                             ExecuteOptions options) {
  if (shutdown_) throw std::runtime_error("mmrt: submit after shutdown");
  Device& dev = DeviceOf(device);
  const int kind = std::min(std::max(options.stream, 0), kNumStreamKinds - 1);
  void* stream = dev.stream[kind];
  const uint64_t id = next_id_++;
  const double submit_us = NowUs();

  // ---- the tasks this one must be ordered behind
  std::map<uint64_t, Access> deps;
  for (const TileRef& r : reads) {
    const TileState& st = tiles_[r];
    if (st.last_writer.task) deps.emplace(st.last_writer.task, st.last_writer);      // read after write
  }
  for (const TileRef& w : writes) {
    const TileState& st = tiles_[w];
    if (st.last_writer.task) deps.emplace(st.last_writer.task, st.last_writer);      // write after write
    for (const Access& rd : st.readers_since_write) deps.emplace(rd.task, rd);       // write after read
  }
  if (options.strict_ordering && dev.last_strict.task) deps.emplace(dev.last_strict.task, dev.last_strict);
  std::vector<uint64_t> dep_ids;
  api_->SetDevice(dev.ordinal);
  for (auto& kv : deps) {
    const Access& a = kv.second;
    dep_ids.push_back(a.task);
    // tasks on one stream run in submission order; every other pair needs the event
    if (a.device == device && a.stream == kind) continue;
    if (!a.event) continue;
    if (!api_->StreamWaitEvent(stream, a.event->handle))
      throw std::runtime_error("mmrt: cudaStreamWaitEvent failed: " + api_->LastError());
    edges_.push_back(EventEdge{a.task, id, device, a.stream, kind, a.name, options.name});
    if (edges_.size() > (1u << 20)) edges_.erase(edges_.begin(), edges_.begin() + (edges_.size() >> 1));
  }
  if (record_) submissions_.push_back(SubmittedTask{id, reads, writes, dep_ids, options.name});

  // ---- run the body: it launches the task's kernels onto `stream`
  bool skip = error_ != Status::kOk && options.step == failed_step_ && options.kind != 3;
  bool failed = false;
  FaultSpec fault;
  bool has_fault = false;
  for (auto& f : faults_) {
    if (f.remaining <= 0) continue;
    if (f.device >= 0 && f.device != device) continue;
    if (options.name.find(f.name_substring) == std::string::npos) continue;
    --f.remaining;
    fault = f;
    has_fault = true;
    break;
  }
  const double start_us = NowUs();
  if (!skip) {
    if (task_ranges_) api_->RangePush(options.name + " device " + std::to_string(device));
    try {
      if (has_fault && fault.kind == FaultSpec::kDelay)
        std::this_thread::sleep_for(std::chrono::milliseconds(fault.delay_ms));
      if (has_fault && fault.kind == FaultSpec::kThrow)
        throw std::runtime_error("injected fault in task '" + options.name + "'");
      if (!(has_fault && fault.kind == FaultSpec::kDrop) && body) body();
    } catch (const std::exception& e) {
      failed = true;
      Fail(has_fault ? Status::kInjectedFault : Status::kTaskFailed, e.what(), options.step);
    } catch (...) {
      failed = true;
      Fail(Status::kTaskFailed, "unknown exception in task '" + options.name + "'", options.step);
    }
    if (task_ranges_) api_->RangePop();
  }
  body = nullptr;

  // ---- the event later tasks on other streams wait for
  Access me;
  me.task = id;
  me.device = device;
  me.stream = kind;
  me.name = options.name;
  me.event = NewEvent(false);
  api_->SetDevice(dev.ordinal);
  if (!api_->RecordEvent(me.event->handle, stream))
    throw std::runtime_error("mmrt: cudaEventRecord failed: " + api_->LastError());
  dev.last_event[kind] = me.event;
  for (const TileRef& r : reads) tiles_[r].readers_since_write.push_back(me);
  for (const TileRef& w : writes) {
    TileState& st = tiles_[w];
    st.last_writer = me;
    st.readers_since_write.clear();
  }
  if (options.strict_ordering) dev.last_strict = me;
  log_.push_back(TaskRecord{id, options.name, device, options.kind, options.step, submit_us, start_us, NowUs(), skip, failed});
  if (log_.size() > (1u << 20)) log_.erase(log_.begin(), log_.begin() + (log_.size() >> 1));
  return id;
}

void CudaContext::CreateStore(int buffer, int device, int64_t bytes, bool host) {
  auto key = std::make_pair(buffer, device);
  if (store_bytes_.count(key)) return;
  store_bytes_[key] = bytes;
  if (!host) {
    device_bytes_ += bytes;
    device_hwm_ = std::max(device_hwm_, device_bytes_);
  }
}
void CudaContext::FreeStore(int buffer, int device) {
  auto it = store_bytes_.find({buffer, device});
  if (it == store_bytes_.end()) return;
  device_bytes_ -= it->second;
  store_bytes_.erase(it);
  tiles_.erase(TileRef{buffer, device});
}

// A step's window stays open until the device has finished the step. Opening the ninth window
// waits - on the host, the only place where the host waits at all - for the oldest open step.
void CudaContext::OpenWindow() {
  while (static_cast<int>(window_events_.size()) >= kMaxOpenWindows) {
    for (auto& e : window_events_.front())
      if (e && !api_->EventDone(e->handle)) {
        ++host_blocks_;
        api_->EventSynchronize(e->handle);
      }
    window_events_.pop_front();
  }
  // steps that have already finished on the device leave the window without any waiting
  while (!window_events_.empty()) {
    bool done = true;
    for (auto& e : window_events_.front()) done = done && (!e || api_->EventDone(e->handle));
    if (!done) break;
    window_events_.pop_front();
  }
  ++windows_opened_;
}

// Joins the side streams into the compute stream (results handed to the caller are ordered
// behind every message and collective of the step) and marks the end of the step there.
void CudaContext::CloseWindow() {
  std::vector<EventPtr> ends;
  for (auto& d : devices_) {
    api_->SetDevice(d.ordinal);
    for (int k = 1; k < kNumStreamKinds; ++k)
      if (d.last_event[k]) {
        api_->StreamWaitEvent(d.stream[kComputeStream], d.last_event[k]->handle);
        d.last_event[k] = nullptr;
      }
    EventPtr end = NewEvent(false);
    api_->RecordEvent(end->handle, d.stream[kComputeStream]);
    ends.push_back(end);
  }
  window_events_.push_back(std::move(ends));
}

void CudaContext::RunAfterAllTasks(Body body) {
  // bodies run at submission, so every task submitted so far has been launched
  if (body) body();
}

void CudaContext::StartTimer(const std::string& name) {
  if (devices_.empty()) return;
  Device& d = devices_[0];
  api_->SetDevice(d.ordinal);
  Timer t;
  t.start = NewEvent(true);
  api_->RecordEvent(t.start->handle, d.stream[kComputeStream]);
  timers_[name] = t;
}
void CudaContext::StopTimer(const std::string& name) {
  auto it = timers_.find(name);
  if (it == timers_.end() || devices_.empty()) return;
  Device& d = devices_[0];
  api_->SetDevice(d.ordinal);
  it->second.stop = NewEvent(true);
  api_->RecordEvent(it->second.stop->handle, d.stream[kComputeStream]);
}
std::map<std::string, double> CudaContext::TimerResultsMs() {
  for (auto it = timers_.begin(); it != timers_.end();) {
    Timer& t = it->second;
    if (t.start && t.stop && api_->EventDone(t.stop->handle)) {
      timer_ms_[it->first] = api_->ElapsedMs(t.start->handle, t.stop->handle);
      it = timers_.erase(it);
    } else {
      ++it;
    }
  }
  return timer_ms_;
}
void CudaContext::MarkProfile(const std::string& name) {
  api_->Mark(name);
  const double t = NowUs();
  log_.push_back(TaskRecord{0, name, -1, 3, 0, t, t, t, false, false});
}

Status CudaContext::WaitAll(std::string* message) {
  // every body has run by the time its submission returns; device completion is a matter of
  // stream order (or of Synchronize)
  if (message) *message = error_message_;
  return error_;
}
void CudaContext::ResetError() {
  error_ = Status::kOk;
  error_message_.clear();
  failed_step_ = -1;
}

bool CudaContext::Synchronize() {
  bool ok = true;
  for (auto& d : devices_) {
    api_->SetDevice(d.ordinal);
    for (int k = 0; k < kNumStreamKinds; ++k)
      if (d.stream[k] || k == kComputeStream) ok = api_->StreamSynchronize(d.stream[k]) && ok;
  }
  return ok;
}

uintptr_t CudaContext::ReserveScratch(int device, int64_t bytes) {
  Device& d = DeviceOf(device);
  if (bytes <= d.scratch_bytes) return reinterpret_cast<uintptr_t>(d.scratch);
  api_->SetDevice(d.ordinal);
  if (d.scratch) {
    // kernels of earlier tasks may still use the old tile
    for (int k = 0; k < kNumStreamKinds; ++k) api_->StreamSynchronize(d.stream[k]);
    api_->Free(d.scratch);
    d.scratch = nullptr;
    d.scratch_bytes = 0;
  }
  const int64_t rounded = (bytes + (1 << 21) - 1) / (1 << 21) * (1 << 21);
  d.scratch = api_->Malloc(static_cast<size_t>(rounded));
  if (!d.scratch) return 0;
  d.scratch_bytes = rounded;
  return reinterpret_cast<uintptr_t>(d.scratch);
}
int64_t CudaContext::ScratchBytes(int device) const { return DeviceOf(device).scratch_bytes; }

}  // namespace mmrt
