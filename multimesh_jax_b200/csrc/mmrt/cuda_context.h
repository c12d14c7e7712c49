// CudaContext: the task-graph runtime of a process that drives CUDA devices.
//
// Every local device gets three streams: `compute` (the stream the caller already works on, so
// results are ordered with the caller's own kernels), `comm` (cross-submesh reshards and
// collectives that are tasks of their own; highest stream priority, their small kernels unblock
// other GPUs) and `aux` (non-critical work such as weight-gradient halves of a split backward
// task; lowest priority). Tasks are submitted in plan order by one host thread and their bodies
// run at submission, launching kernels onto the stream the task was given. Ordering between
// streams is what the dependence analysis says and nothing more: every read-after-write,
// write-after-read and write-after-write pair on a (buffer, device) tile whose two tasks sit on
// different streams becomes a CUDA event wait (`cudaStreamWaitEvent`), as does the strict-order
// chain of tasks with collectives; pairs on one stream are ordered by the stream itself. The
// host never blocks inside a step, except in `OpenWindow` when `kMaxOpenWindows` steps are in
// flight. This is the part the external task runtime plays for the reference
// (src/pjrt_client/zuku_execute_context_impl.cc:302-345: `across().after().priority()
// .stream_ordered().defer()`; stream cache src/pjrt_client/mm_utils.cc:44-70; event record after
// launch src/pjrt_client/mm_computation.cc:886-889).
//
// The context also owns the per-device scratch tile of the native task launcher
// (src/pjrt_client/mm_pjrt_executable.cc:549-590: one cached scratch buffer sized for the
// largest task, handed out by a bump allocator - src/pjrt_client/allocator.h:10-24).
//
// All CUDA calls go through `GpuApi`, so that the ordering logic can be exercised on a machine
// without a GPU against `FakeGpuApi`, which records the calls it receives.
#pragma once
#include <deque>

#include "runtime.h"

namespace mmrt {

class GpuApi {
 public:
  virtual ~GpuApi() = default;
  virtual bool SetDevice(int ordinal) = 0;
  virtual void PriorityRange(int* least, int* greatest) = 0;
  virtual void* CreateStream(int priority) = 0;
  virtual void DestroyStream(void* stream) = 0;
  virtual void* CreateEvent(bool timing) = 0;
  virtual void DestroyEvent(void* event) = 0;
  virtual bool RecordEvent(void* event, void* stream) = 0;
  virtual bool StreamWaitEvent(void* stream, void* event) = 0;
  virtual bool EventSynchronize(void* event) = 0;
  virtual bool EventDone(void* event) = 0;
  virtual float ElapsedMs(void* start, void* stop) = 0;
  virtual bool StreamSynchronize(void* stream) = 0;
  virtual void* Malloc(size_t bytes) = 0;
  virtual void Free(void* ptr) = 0;
  virtual void RangePush(const std::string& name) = 0;
  virtual void RangePop() = 0;
  virtual void Mark(const std::string& name) = 0;
  virtual std::string LastError() = 0;
};

// The CUDA runtime (and NVTX when the tools library can be loaded).
GpuApi* CudaRuntimeApi();

// Stand-in without a GPU: streams and events are small integers, every call is appended to
// `trace` ("wait s2 e7", "record e7 s1", ...), events complete when they are recorded.
class FakeGpuApi : public GpuApi {
 public:
  bool SetDevice(int ordinal) override;
  void PriorityRange(int* least, int* greatest) override { *least = 0; *greatest = -5; }
  void* CreateStream(int priority) override;
  void DestroyStream(void*) override {}
  void* CreateEvent(bool timing) override;
  void DestroyEvent(void*) override {}
  bool RecordEvent(void* event, void* stream) override;
  bool StreamWaitEvent(void* stream, void* event) override;
  bool EventSynchronize(void* event) override;
  bool EventDone(void*) override { return true; }
  float ElapsedMs(void*, void*) override { return 1.0f; }
  bool StreamSynchronize(void* stream) override;
  void* Malloc(size_t bytes) override;
  void Free(void* ptr) override;
  void RangePush(const std::string& name) override { trace.push_back("push " + name); }
  void RangePop() override { trace.push_back("pop"); }
  void Mark(const std::string& name) override { trace.push_back("mark " + name); }
  std::string LastError() override { return ""; }

  std::vector<std::string> trace;
  std::vector<int> stream_priorities;   // by stream number (1-based)
  int64_t bytes_allocated = 0;

 private:
  intptr_t next_stream_ = 1, next_event_ = 1, next_ptr_ = 4096;
  std::map<intptr_t, size_t> allocations_;
};

enum StreamKind : int { kComputeStream = 0, kCommStream = 1, kAuxStream = 2, kNumStreamKinds = 3 };

// One cross-stream ordering edge that the context enforced with an event wait.
struct EventEdge {
  uint64_t from_task, to_task;
  int device;
  int from_stream, to_stream;   // StreamKind
  std::string from_name, to_name;
};

class CudaContext : public ExecuteContext {
 public:
  // `local_devices`: global device ids driven by this process; `ordinals`: their CUDA ordinals;
  // `compute_streams`: for each, the handle of the stream the caller computes on (0 = the
  // default stream). `api` is not owned.
  CudaContext(std::vector<int> local_devices, std::vector<int> ordinals, std::vector<uintptr_t> compute_streams,
              GpuApi* api, bool record_submissions = false);
  ~CudaContext() override;

  uint64_t CreateExecuteTask(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes,
                             Body body, const ExecuteOptions& options) override;
  uint64_t Reshard(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes, Body body,
                   const ExecuteOptions& options) override;
  void CreateStore(int buffer, int device, int64_t bytes, bool host) override;
  void FreeStore(int buffer, int device) override;
  void OffloadDtoH(int, int) override {}
  void OffloadHtoD(int, int) override {}
  void OpenWindow() override;
  void CloseWindow() override;
  void RunAfterAllTasks(Body body) override;
  void FenceCompilation() override {}
  void StartTimer(const std::string& name) override;
  void StopTimer(const std::string& name) override;
  void MarkProfile(const std::string& name) override;
  Status WaitAll(std::string* message) override;
  Status WaitTask(uint64_t, std::string* message) override { return WaitAll(message); }
  void Shutdown() override;
  std::vector<TaskRecord> EventLog() const override { return log_; }
  void ClearEventLog() override { log_.clear(); edges_.clear(); }

  // Stream of `device` for tasks of kind `kind`; the body of a task submitted with
  // ExecuteOptions::stream == kind must launch its kernels there.
  uintptr_t StreamHandle(int device, int kind) const;
  // Blocks until every stream of every local device is idle.
  bool Synchronize();
  void InjectFault(const FaultSpec& spec) { faults_.push_back(spec); }
  void ResetError();
  std::vector<SubmittedTask> Submissions() const { return submissions_; }
  std::vector<EventEdge> Edges() const { return edges_; }
  // Device-timed durations (CUDA events on the compute stream) of the timers whose stop event
  // has completed; a timer that is still running on the device is left out.
  std::map<std::string, double> TimerResultsMs();
  void set_task_ranges(bool on) { task_ranges_ = on; }
  int64_t device_bytes_high_water() const { return device_hwm_; }
  int open_windows() const { return static_cast<int>(window_events_.size()); }
  int host_blocks() const { return host_blocks_; }   // how often the host had to wait for the device

  // Scratch tile of `device`: grows to the largest size ever asked for (the device is
  // synchronised before an old tile is released). Returns the base address, 0 on failure.
  uintptr_t ReserveScratch(int device, int64_t bytes);
  int64_t ScratchBytes(int device) const;

 private:
  struct Event {
    void* handle = nullptr;
    CudaContext* owner = nullptr;
    bool timing = false;
    ~Event();
  };
  using EventPtr = std::shared_ptr<Event>;
  struct Access {
    uint64_t task = 0;
    int device = -1;       // device whose stream the task ran on
    int stream = 0;        // StreamKind
    EventPtr event;        // recorded behind the task's kernels
    std::string name;
  };
  struct TileState {
    Access last_writer;
    std::vector<Access> readers_since_write;
  };
  struct Device {
    int id = -1, ordinal = 0;
    void* stream[kNumStreamKinds] = {nullptr, nullptr, nullptr};
    bool owned[kNumStreamKinds] = {false, false, false};
    Access last_strict;
    EventPtr last_event[kNumStreamKinds];   // behind the most recent task of each stream
    void* scratch = nullptr;
    int64_t scratch_bytes = 0;
  };
  uint64_t Submit(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes, Body body,
                  ExecuteOptions options);
  Device& DeviceOf(int device);
  const Device& DeviceOf(int device) const;
  EventPtr NewEvent(bool timing);
  void Fail(Status status, const std::string& message, int step);
  double NowUs() const;

  GpuApi* api_;
  std::vector<Device> devices_;
  std::map<TileRef, TileState> tiles_;
  std::vector<void*> free_events_, free_timing_events_;
  uint64_t next_id_ = 1;
  bool shutdown_ = false;
  bool record_;
  bool task_ranges_ = false;
  Status error_ = Status::kOk;
  std::string error_message_;
  int failed_step_ = -1;
  std::vector<TaskRecord> log_;
  std::vector<SubmittedTask> submissions_;
  std::vector<EventEdge> edges_;
  std::vector<FaultSpec> faults_;
  std::deque<std::vector<EventPtr>> window_events_;   // per open step: its end event on every device
  int windows_opened_ = 0;
  int host_blocks_ = 0;
  struct Timer { EventPtr start, stop; };
  std::map<std::string, Timer> timers_;
  std::map<std::string, double> timer_ms_;
  std::map<std::pair<int, int>, int64_t> store_bytes_;
  int64_t device_bytes_ = 0, device_hwm_ = 0;
  Clock::time_point epoch_;
};

}  // namespace mmrt
