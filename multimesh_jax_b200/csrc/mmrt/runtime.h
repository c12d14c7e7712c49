// mmrt: the task-graph runtime.
//
// The compiler's plan is a linear list of operations over stores. At run time
// every operation is *submitted* (never executed inline by the submitter): the
// runtime derives dependencies from the read / write sets on (buffer, device)
// tiles - read-after-write, write-after-read, write-after-write - adds a
// strict-order chain per device for tasks that contain collectives, and hands
// ready tasks to one worker thread per local device, highest priority first.
// Task bodies are opaque callables (they launch CUDA kernels on the device's
// stream, or run CPU tensor code). This is the role the external task runtime
// plays for the reference (src/pjrt_client/zuku_execute_context_impl.cc:213-486);
// the abstract interface mirrors src/pjrt_client/zuku_execute_context.h:38-133.
//
// Three implementations share the interface:
//   ThreadedContext - real execution (CPU virtual devices or CUDA devices)
//   MockContext     - records an operation hash, simulates device / host memory
//                     high-water marks and checks protocol invariants; runs nothing
// Failures are status codes, not aborts: a body that throws marks its step as
// failed, later tasks of that step are skipped, and Wait() reports the error.
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <queue>
#include <set>
#include <string>
#include <thread>
#include <vector>

namespace mmrt {

using Clock = std::chrono::steady_clock;

// A (buffer, device) tile: the unit of dependence analysis.
struct TileRef {
  int buffer = -1;  // id of the physical buffer (stores that share a scheduling name share it)
  int device = -1;  // global device id
  bool operator<(const TileRef& o) const { return buffer != o.buffer ? buffer < o.buffer : device < o.device; }
};

struct ExecuteOptions {
  std::string name;
  bool strict_ordering = false;
  int priority = 0;
  int kind = 0;  // 0 task, 1 reshard, 2 host callback, 3 marker
  int step = 0;
  int stream = 0;  // contexts with several streams per device: 0 compute, 1 communication, 2 auxiliary
};

struct TaskRecord {  // one entry of the event log
  uint64_t id;
  std::string name;
  int device;
  int kind;
  int step;
  double submit_us, start_us, end_us;
  bool skipped;
  bool failed;
};

enum class Status : int { kOk = 0, kTaskFailed = 1, kInjectedFault = 2, kProtocolViolation = 3, kShutdown = 4 };

using Body = std::function<void()>;

class ExecuteContext {
 public:
  virtual ~ExecuteContext() = default;
  // Submits `body` to run on local device `device` after its dependencies. Returns the task id.
  virtual uint64_t CreateExecuteTask(int device, const std::vector<TileRef>& reads,
                                     const std::vector<TileRef>& writes, Body body,
                                     const ExecuteOptions& options) = 0;
  // A reshard is a task whose body moves data; kept separate so contexts can account for it.
  virtual uint64_t Reshard(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes,
                           Body body, const ExecuteOptions& options) = 0;
  // Store bookkeeping (allocation itself is done by the owner of the tensors).
  virtual void CreateStore(int buffer, int device, int64_t bytes, bool host) = 0;
  virtual void FreeStore(int buffer, int device) = 0;
  virtual void OffloadDtoH(int buffer, int device) = 0;
  virtual void OffloadHtoD(int buffer, int device) = 0;
  // Bounds the number of steps in flight (blocks when kMaxOpenWindows are open).
  virtual void OpenWindow() = 0;
  virtual void CloseWindow() = 0;
  virtual void RunAfterAllTasks(Body body) = 0;
  virtual void FenceCompilation() = 0;
  virtual void StartTimer(const std::string& name) = 0;
  virtual void StopTimer(const std::string& name) = 0;
  virtual void MarkProfile(const std::string& name) = 0;
  // Blocks until everything submitted so far has finished; returns the first error status.
  virtual Status WaitAll(std::string* message) = 0;
  virtual Status WaitTask(uint64_t id, std::string* message) = 0;
  virtual void Shutdown() = 0;
  virtual std::vector<TaskRecord> EventLog() const = 0;
  virtual void ClearEventLog() = 0;
  static constexpr int kMaxOpenWindows = 8;
};

// ---------------------------------------------------------------------------
// Dependence analysis shared by all contexts
// ---------------------------------------------------------------------------
class DependenceTracker {
 public:
  // Returns ids of the tasks that `task` must wait for and updates the tables.
  std::vector<uint64_t> Register(uint64_t task, int device, const std::vector<TileRef>& reads,
                                 const std::vector<TileRef>& writes, bool strict);
  void Forget(int buffer, int device);
  void Clear();

 private:
  struct TileState {
    uint64_t last_writer = 0;
    std::vector<uint64_t> readers_since_write;
  };
  std::map<TileRef, TileState> tiles_;
  std::map<int, uint64_t> last_strict_;  // device -> last strictly ordered task
};

// Replays a submitted task list and checks that every RAW / WAR / WAW pair on a tile is
// ordered by the recorded dependency edges (transitively). Returns a description of the
// first unordered pair, or "" when the schedule is race free.
struct SubmittedTask {
  uint64_t id;
  std::vector<TileRef> reads, writes;
  std::vector<uint64_t> deps;
  std::string name;
};
std::string CheckHazards(const std::vector<SubmittedTask>& tasks);

// ---------------------------------------------------------------------------
// Fault injection (host side only)
// ---------------------------------------------------------------------------
struct FaultSpec {
  enum Kind { kThrow = 0, kDrop = 1, kDelay = 2 } kind = kThrow;
  std::string name_substring;  // matches ExecuteOptions::name
  int device = -1;             // -1 = any
  int remaining = 1;           // how many matching tasks to hit
  int delay_ms = 0;
};

// ---------------------------------------------------------------------------
// Real execution
// ---------------------------------------------------------------------------
class ThreadedContext : public ExecuteContext {
 public:
  // `local_devices`: global ids of the devices this process drives (one worker each).
  // With `inline_execution` bodies run on the submitting thread as soon as their dependencies
  // are met (single-device processes: no hand-off, stream order is program order).
  explicit ThreadedContext(std::vector<int> local_devices, bool inline_execution = false,
                           bool record_submissions = false);
  ~ThreadedContext() override;

  uint64_t CreateExecuteTask(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes,
                             Body body, const ExecuteOptions& options) override;
  uint64_t Reshard(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes, Body body,
                   const ExecuteOptions& options) override;
  void CreateStore(int buffer, int device, int64_t bytes, bool host) override;
  void FreeStore(int buffer, int device) override;
  void OffloadDtoH(int buffer, int device) override;
  void OffloadHtoD(int buffer, int device) override;
  void OpenWindow() override;
  void CloseWindow() override;
  void RunAfterAllTasks(Body body) override;
  void FenceCompilation() override {}
  void StartTimer(const std::string& name) override;
  void StopTimer(const std::string& name) override;
  void MarkProfile(const std::string& name) override;
  Status WaitAll(std::string* message) override;
  Status WaitTask(uint64_t id, std::string* message) override;
  void Shutdown() override;
  std::vector<TaskRecord> EventLog() const override;
  // One line per task that has been submitted and not finished: "id name device state" where
  // state is "running or ready" or "waits for: <unfinished predecessors>". For diagnosing a step
  // that does not end (a task body blocked in a collective its partners never reach).
  std::vector<std::string> PendingReport() const;
  void ClearEventLog() override;

  void InjectFault(const FaultSpec& spec);
  std::vector<SubmittedTask> Submissions() const;
  std::map<std::string, double> TimerResultsMs() const;
  void ResetError();
  int64_t device_bytes_high_water() const { return device_hwm_; }

 private:
  struct Task {
    uint64_t id = 0;
    int device = -1;
    Body body;
    ExecuteOptions options;
    int pending = 0;
    std::vector<uint64_t> successors;
    bool done = false;
    double submit_us = 0;
  };
  struct Worker {
    std::thread thread;
    // (priority, -id): highest priority first, then submission order
    std::priority_queue<std::pair<int, int64_t>> ready;
    std::condition_variable cv;
  };
  Worker& WorkerOf(const Task& task);
  uint64_t Submit(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes, Body body,
                  ExecuteOptions options);
  void WorkerLoop(Worker& worker);
  void RunTask(std::shared_ptr<Task> task);
  void Finish(const std::shared_ptr<Task>& task, bool skipped, bool failed, double start_us);
  double NowUs() const;

  std::vector<int> local_devices_;
  bool inline_;
  bool record_;
  mutable std::mutex mu_;
  std::condition_variable done_cv_;
  std::map<int, std::unique_ptr<Worker>> workers_;        // task bodies, one thread per device
  std::map<int, std::unique_ptr<Worker>> comm_workers_;   // reshard bodies, one thread per device
  std::map<uint64_t, std::shared_ptr<Task>> tasks_;  // live (unfinished) tasks
  DependenceTracker deps_;
  uint64_t next_id_ = 1;
  uint64_t outstanding_ = 0;
  bool shutdown_ = false;
  Status error_ = Status::kOk;
  std::string error_message_;
  int failed_step_ = -1;
  std::vector<TaskRecord> log_;
  std::vector<SubmittedTask> submissions_;
  std::vector<FaultSpec> faults_;
  std::map<std::string, double> timer_start_us_, timer_ms_;
  std::map<std::pair<int, int>, int64_t> store_bytes_;
  int64_t device_bytes_ = 0, device_hwm_ = 0;
  int open_windows_ = 0;
  Clock::time_point epoch_;
};

// ---------------------------------------------------------------------------
// Mock: verifies the protocol, measures memory, executes nothing
// ---------------------------------------------------------------------------
class MockContext : public ExecuteContext {
 public:
  explicit MockContext(int num_devices);
  uint64_t CreateExecuteTask(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes,
                             Body body, const ExecuteOptions& options) override;
  uint64_t Reshard(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes, Body body,
                   const ExecuteOptions& options) override;
  void CreateStore(int buffer, int device, int64_t bytes, bool host) override;
  void FreeStore(int buffer, int device) override;
  void OffloadDtoH(int buffer, int device) override;
  void OffloadHtoD(int buffer, int device) override;
  void OpenWindow() override { Mix("open"); ++open_windows_; }
  void CloseWindow() override { Mix("close"); --open_windows_; }
  void RunAfterAllTasks(Body body) override { Mix("after_all"); if (body) body(); }
  void FenceCompilation() override { Mix("fence"); }
  void StartTimer(const std::string& name) override { Mix("start_timer " + name); }
  void StopTimer(const std::string& name) override { Mix("stop_timer " + name); }
  void MarkProfile(const std::string& name) override { Mix("mark " + name); }
  Status WaitAll(std::string* message) override;
  Status WaitTask(uint64_t, std::string* message) override { return WaitAll(message); }
  void Shutdown() override {}
  std::vector<TaskRecord> EventLog() const override { return log_; }
  void ClearEventLog() override { log_.clear(); }

  uint64_t operation_hash() const { return hash_; }
  int64_t device_high_water(int device) const;
  int64_t host_high_water() const { return host_hwm_; }
  int64_t max_device_high_water() const;
  int num_tasks() const { return num_tasks_; }
  int num_reshards() const { return num_reshards_; }
  std::string violation() const { return violation_; }
  std::string hazard_report() const { return CheckHazards(submissions_); }

 private:
  void Mix(const std::string& s);
  void Violation(const std::string& s);
  uint64_t Record(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes,
                  const ExecuteOptions& options, bool reshard);
  struct Tile { int64_t bytes = 0; bool host = false; bool reshard_pending = false; };
  int num_devices_;
  std::map<TileRef, Tile> tiles_;
  std::map<int, int64_t> device_bytes_, device_hwm_;
  int64_t host_bytes_ = 0, host_hwm_ = 0;
  uint64_t hash_ = 1469598103934665603ull;
  uint64_t next_id_ = 1;
  int num_tasks_ = 0, num_reshards_ = 0, open_windows_ = 0;
  std::string violation_;
  DependenceTracker deps_;
  std::vector<SubmittedTask> submissions_;
  std::vector<TaskRecord> log_;
};

}  // namespace mmrt
