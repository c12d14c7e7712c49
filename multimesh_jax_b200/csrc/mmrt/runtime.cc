#include "runtime.h"

#include <algorithm>
#include <sstream>
#include <stdexcept>

namespace mmrt {

// ---------------------------------------------------------------------------
// DependenceTracker
// ---------------------------------------------------------------------------
std::vector<uint64_t> DependenceTracker::Register(uint64_t task, int device, const std::vector<TileRef>& reads,
                                                  const std::vector<TileRef>& writes, bool strict) {
  std::set<uint64_t> deps;
  for (const TileRef& r : reads) {
    TileState& st = tiles_[r];
    if (st.last_writer) deps.insert(st.last_writer);  // read after write
  }
  for (const TileRef& w : writes) {
    TileState& st = tiles_[w];
    if (st.last_writer) deps.insert(st.last_writer);                      // write after write
    for (uint64_t rd : st.readers_since_write) deps.insert(rd);           // write after read
  }
  if (strict) {
    auto it = last_strict_.find(device);
    if (it != last_strict_.end()) deps.insert(it->second);
    last_strict_[device] = task;
  }
  for (const TileRef& r : reads) tiles_[r].readers_since_write.push_back(task);
  for (const TileRef& w : writes) {
    TileState& st = tiles_[w];
    st.last_writer = task;
    st.readers_since_write.clear();
  }
  deps.erase(task);
  return std::vector<uint64_t>(deps.begin(), deps.end());
}
void DependenceTracker::Forget(int buffer, int device) { tiles_.erase(TileRef{buffer, device}); }
void DependenceTracker::Clear() { tiles_.clear(); last_strict_.clear(); }

std::string CheckHazards(const std::vector<SubmittedTask>& tasks) {
  // ancestors via recorded deps (tasks are in submission order, deps point backwards)
  std::map<uint64_t, size_t> index;
  for (size_t i = 0; i < tasks.size(); ++i) index[tasks[i].id] = i;
  std::vector<std::set<size_t>> anc(tasks.size());
  for (size_t i = 0; i < tasks.size(); ++i)
    for (uint64_t d : tasks[i].deps) {
      auto it = index.find(d);
      if (it == index.end()) continue;  // finished long ago
      anc[i].insert(it->second);
      anc[i].insert(anc[it->second].begin(), anc[it->second].end());
    }
  auto conflicts = [](const SubmittedTask& a, const SubmittedTask& b, TileRef* tile) {
    for (auto& w : a.writes) {
      for (auto& x : b.writes) if (!(w < x) && !(x < w)) { *tile = w; return true; }
      for (auto& x : b.reads) if (!(w < x) && !(x < w)) { *tile = w; return true; }
    }
    for (auto& r : a.reads)
      for (auto& x : b.writes) if (!(r < x) && !(x < r)) { *tile = r; return true; }
    return false;
  };
  for (size_t j = 0; j < tasks.size(); ++j)
    for (size_t i = 0; i < j; ++i) {
      TileRef tile;
      if (!conflicts(tasks[i], tasks[j], &tile)) continue;
      if (anc[j].count(i)) continue;
      std::ostringstream os;
      os << "unordered conflicting accesses to buffer " << tile.buffer << " on device " << tile.device
         << " by '" << tasks[i].name << "' and '" << tasks[j].name << "'";
      return os.str();
    }
  return "";
}

// ---------------------------------------------------------------------------
// ThreadedContext
// ---------------------------------------------------------------------------
ThreadedContext::ThreadedContext(std::vector<int> local_devices, bool inline_execution, bool record_submissions)
    : local_devices_(std::move(local_devices)), inline_(inline_execution), record_(record_submissions),
      epoch_(Clock::now()) {
  if (!inline_) {
    for (int d : local_devices_) {
      workers_[d] = std::make_unique<Worker>();
      comm_workers_[d] = std::make_unique<Worker>();
    }
    for (int d : local_devices_) {
      workers_[d]->thread = std::thread([this, d] { WorkerLoop(*workers_[d]); });
      comm_workers_[d]->thread = std::thread([this, d] { WorkerLoop(*comm_workers_[d]); });
    }
  }
}

// Reshards run on a thread of their own per device (the counterpart of the communication stream
// of the CUDA context). A task body may block in a collective until its partners on other devices
// reach it, and a partner may be unable to start before a reshard has read the tile it is about
// to overwrite; with reshards queued behind the blocked task on the same thread, two such chains
// close into a cycle (seen with interleaved stages whose tasks exchange data inside).
ThreadedContext::Worker& ThreadedContext::WorkerOf(const Task& task) {
  return task.options.kind == 1 ? *comm_workers_[task.device] : *workers_[task.device];
}

ThreadedContext::~ThreadedContext() { Shutdown(); }

double ThreadedContext::NowUs() const {
  return std::chrono::duration<double, std::micro>(Clock::now() - epoch_).count();
}

void ThreadedContext::Shutdown() {
  {
    std::unique_lock<std::mutex> lock(mu_);
    if (shutdown_) return;
    done_cv_.wait(lock, [&] { return outstanding_ == 0; });
    shutdown_ = true;
    for (auto& kv : workers_) kv.second->cv.notify_all();
    for (auto& kv : comm_workers_) kv.second->cv.notify_all();
  }
  for (auto& kv : workers_) if (kv.second->thread.joinable()) kv.second->thread.join();
  for (auto& kv : comm_workers_) if (kv.second->thread.joinable()) kv.second->thread.join();
}

uint64_t ThreadedContext::CreateExecuteTask(int device, const std::vector<TileRef>& reads,
                                            const std::vector<TileRef>& writes, Body body,
                                            const ExecuteOptions& options) {
  return Submit(device, reads, writes, std::move(body), options);
}
uint64_t ThreadedContext::Reshard(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes,
                                  Body body, const ExecuteOptions& options) {
  ExecuteOptions o = options;
  o.kind = 1;
  return Submit(device, reads, writes, std::move(body), o);
}

uint64_t ThreadedContext::Submit(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes,
                                 Body body, ExecuteOptions options) {
  std::shared_ptr<Task> task = std::make_shared<Task>();
  bool run_now = false;
  {
    std::unique_lock<std::mutex> lock(mu_);
    if (shutdown_) throw std::runtime_error("mmrt: submit after shutdown");
    if (!inline_ && !workers_.count(device)) throw std::runtime_error("mmrt: device is not local to this process");
    task->id = next_id_++;
    task->device = device;
    task->body = std::move(body);
    task->options = std::move(options);
    task->submit_us = NowUs();
    std::vector<uint64_t> deps = deps_.Register(task->id, device, reads, writes, task->options.strict_ordering);
    if (record_) submissions_.push_back(SubmittedTask{task->id, reads, writes, deps, task->options.name});
    for (uint64_t d : deps) {
      auto it = tasks_.find(d);
      if (it == tasks_.end() || it->second->done) continue;  // already finished
      it->second->successors.push_back(task->id);
      ++task->pending;
    }
    tasks_[task->id] = task;
    ++outstanding_;
    if (task->pending == 0) {
      if (inline_) run_now = true;
      else {
        Worker& w = WorkerOf(*task);
        w.ready.emplace(task->options.priority, -static_cast<int64_t>(task->id));
        w.cv.notify_one();
      }
    }
  }
  if (run_now) RunTask(task);
  return task->id;
}

void ThreadedContext::WorkerLoop(Worker& w) {
  while (true) {
    std::shared_ptr<Task> task;
    {
      std::unique_lock<std::mutex> lock(mu_);
      w.cv.wait(lock, [&] { return shutdown_ || !w.ready.empty(); });
      if (w.ready.empty()) return;
      const uint64_t id = static_cast<uint64_t>(-w.ready.top().second);
      w.ready.pop();
      task = tasks_[id];
    }
    RunTask(task);
  }
}

void ThreadedContext::RunTask(std::shared_ptr<Task> task) {
  bool skip = false, failed = false;
  FaultSpec fault;
  bool has_fault = false;
  {
    std::unique_lock<std::mutex> lock(mu_);
    // once a step has failed, its remaining tasks are skipped (status-code propagation)
    if (error_ != Status::kOk && task->options.step == failed_step_ && task->options.kind != 3) skip = true;
    for (auto& f : faults_) {
      if (f.remaining <= 0) continue;
      if (f.device >= 0 && f.device != task->device) continue;
      if (task->options.name.find(f.name_substring) == std::string::npos) continue;
      --f.remaining;
      fault = f;
      has_fault = true;
      break;
    }
  }
  const double start = NowUs();
  if (!skip) {
    try {
      if (has_fault && fault.kind == FaultSpec::kDelay)
        std::this_thread::sleep_for(std::chrono::milliseconds(fault.delay_ms));
      if (has_fault && fault.kind == FaultSpec::kThrow)
        throw std::runtime_error("injected fault in task '" + task->options.name + "'");
      if (has_fault && fault.kind == FaultSpec::kDrop) {
        // the task silently does not run: downstream results are wrong, which the caller's checks must catch
      } else if (task->body) {
        task->body();
      }
    } catch (const std::exception& e) {
      failed = true;
      std::unique_lock<std::mutex> lock(mu_);
      if (error_ == Status::kOk) {
        error_ = has_fault ? Status::kInjectedFault : Status::kTaskFailed;
        error_message_ = e.what();
        failed_step_ = task->options.step;
      }
    } catch (...) {
      failed = true;
      std::unique_lock<std::mutex> lock(mu_);
      if (error_ == Status::kOk) {
        error_ = Status::kTaskFailed;
        error_message_ = "unknown exception in task '" + task->options.name + "'";
        failed_step_ = task->options.step;
      }
    }
  }
  // drop the callable here, outside the runtime lock: its destructor may need other locks
  task->body = nullptr;
  Finish(task, skip, failed, start);
}

void ThreadedContext::Finish(const std::shared_ptr<Task>& task, bool skipped, bool failed, double start_us) {
  std::vector<std::shared_ptr<Task>> run_inline;
  {
    std::unique_lock<std::mutex> lock(mu_);
    task->done = true;
    log_.push_back(TaskRecord{task->id, task->options.name, task->device, task->options.kind, task->options.step,
                              task->submit_us, start_us, NowUs(), skipped, failed});
    if (log_.size() > (1u << 20)) log_.erase(log_.begin(), log_.begin() + (log_.size() >> 1));
    for (uint64_t sid : task->successors) {
      auto it = tasks_.find(sid);
      if (it == tasks_.end()) continue;
      if (--it->second->pending == 0) {
        if (inline_) run_inline.push_back(it->second);
        else {
          Worker& w = WorkerOf(*it->second);
          w.ready.emplace(it->second->options.priority, -static_cast<int64_t>(sid));
          w.cv.notify_one();
        }
      }
    }
    tasks_.erase(task->id);
    --outstanding_;
    done_cv_.notify_all();
  }
  for (auto& t : run_inline) RunTask(t);
}

std::vector<std::string> ThreadedContext::PendingReport() const {
  std::unique_lock<std::mutex> lock(mu_);
  std::map<uint64_t, std::vector<uint64_t>> waits_for;
  for (auto& kv : tasks_)
    if (!kv.second->done)
      for (uint64_t succ : kv.second->successors) waits_for[succ].push_back(kv.first);
  std::vector<std::string> out;
  for (auto& kv : tasks_) {
    const Task& t = *kv.second;
    if (t.done) continue;
    std::string line = std::to_string(t.id) + " " + t.options.name + " dev " + std::to_string(t.device) + " ";
    if (t.pending == 0) {
      line += "running or ready";
    } else {
      line += "waits for:";
      for (uint64_t p : waits_for[t.id]) {
        auto it = tasks_.find(p);
        line += " " + std::to_string(p) + (it != tasks_.end() ? "(" + it->second->options.name + "@" + std::to_string(it->second->device) + ")" : "");
      }
    }
    out.push_back(line);
  }
  return out;
}

void ThreadedContext::CreateStore(int buffer, int device, int64_t bytes, bool host) {
  std::unique_lock<std::mutex> lock(mu_);
  auto key = std::make_pair(buffer, device);
  if (store_bytes_.count(key)) return;
  store_bytes_[key] = bytes;
  if (!host) {
    device_bytes_ += bytes;
    device_hwm_ = std::max(device_hwm_, device_bytes_);
  }
}
void ThreadedContext::FreeStore(int buffer, int device) {
  std::unique_lock<std::mutex> lock(mu_);
  auto it = store_bytes_.find({buffer, device});
  if (it == store_bytes_.end()) return;
  device_bytes_ -= it->second;
  store_bytes_.erase(it);
  deps_.Forget(buffer, device);
}
void ThreadedContext::OffloadDtoH(int, int) {}
void ThreadedContext::OffloadHtoD(int, int) {}

void ThreadedContext::OpenWindow() {
  std::unique_lock<std::mutex> lock(mu_);
  done_cv_.wait(lock, [&] { return open_windows_ < kMaxOpenWindows; });
  ++open_windows_;
}
void ThreadedContext::CloseWindow() {
  // the window closes when everything submitted so far has run
  RunAfterAllTasks([this] {
    std::unique_lock<std::mutex> lock(mu_);
    --open_windows_;
    done_cv_.notify_all();
  });
}

void ThreadedContext::RunAfterAllTasks(Body body) {
  // a marker task that depends on every live task
  std::shared_ptr<Task> task = std::make_shared<Task>();
  bool run_now = false;
  {
    std::unique_lock<std::mutex> lock(mu_);
    task->id = next_id_++;
    task->device = local_devices_.empty() ? 0 : local_devices_[0];
    task->body = std::move(body);
    task->options.name = "after_all";
    task->options.kind = 3;
    task->options.priority = 1 << 20;
    task->submit_us = NowUs();
    for (auto& kv : tasks_) {
      if (kv.second->done) continue;
      kv.second->successors.push_back(task->id);
      ++task->pending;
    }
    tasks_[task->id] = task;
    ++outstanding_;
    if (task->pending == 0) {
      if (inline_) run_now = true;
      else {
        Worker& w = *workers_[task->device];
        w.ready.emplace(task->options.priority, -static_cast<int64_t>(task->id));
        w.cv.notify_one();
      }
    }
  }
  if (run_now) RunTask(task);
}

void ThreadedContext::StartTimer(const std::string& name) {
  RunAfterAllTasks([this, name] {
    std::unique_lock<std::mutex> lock(mu_);
    timer_start_us_[name] = NowUs();
  });
}
void ThreadedContext::StopTimer(const std::string& name) {
  RunAfterAllTasks([this, name] {
    std::unique_lock<std::mutex> lock(mu_);
    auto it = timer_start_us_.find(name);
    if (it != timer_start_us_.end()) timer_ms_[name] = (NowUs() - it->second) / 1000.0;
  });
}
void ThreadedContext::MarkProfile(const std::string& name) {
  std::unique_lock<std::mutex> lock(mu_);
  const double t = NowUs();
  log_.push_back(TaskRecord{0, name, -1, 3, 0, t, t, t, false, false});
}

Status ThreadedContext::WaitAll(std::string* message) {
  std::unique_lock<std::mutex> lock(mu_);
  done_cv_.wait(lock, [&] { return outstanding_ == 0; });
  if (message) *message = error_message_;
  return error_;
}
Status ThreadedContext::WaitTask(uint64_t id, std::string* message) {
  std::unique_lock<std::mutex> lock(mu_);
  done_cv_.wait(lock, [&] { return tasks_.find(id) == tasks_.end(); });
  if (message) *message = error_message_;
  return error_;
}
void ThreadedContext::ResetError() {
  std::unique_lock<std::mutex> lock(mu_);
  error_ = Status::kOk;
  error_message_.clear();
  failed_step_ = -1;
}
std::vector<TaskRecord> ThreadedContext::EventLog() const {
  std::unique_lock<std::mutex> lock(mu_);
  return log_;
}
void ThreadedContext::ClearEventLog() {
  std::unique_lock<std::mutex> lock(mu_);
  log_.clear();
}
void ThreadedContext::InjectFault(const FaultSpec& spec) {
  std::unique_lock<std::mutex> lock(mu_);
  faults_.push_back(spec);
}
std::vector<SubmittedTask> ThreadedContext::Submissions() const {
  std::unique_lock<std::mutex> lock(mu_);
  return submissions_;
}
std::map<std::string, double> ThreadedContext::TimerResultsMs() const {
  std::unique_lock<std::mutex> lock(mu_);
  return timer_ms_;
}

// ---------------------------------------------------------------------------
// MockContext
// ---------------------------------------------------------------------------
MockContext::MockContext(int num_devices) : num_devices_(num_devices) {}

void MockContext::Mix(const std::string& s) {
  for (unsigned char c : s) { hash_ ^= c; hash_ *= 1099511628211ull; }
  hash_ ^= 0xff;
  hash_ *= 1099511628211ull;
}
void MockContext::Violation(const std::string& s) { if (violation_.empty()) violation_ = s; }

uint64_t MockContext::Record(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes,
                             const ExecuteOptions& options, bool reshard) {
  const uint64_t id = next_id_++;
  std::ostringstream os;
  os << (reshard ? "reshard " : "task ") << options.name << " dev " << device << " in";
  for (auto& r : reads) os << " " << r.buffer << "@" << r.device;
  os << " out";
  for (auto& w : writes) os << " " << w.buffer << "@" << w.device;
  Mix(os.str());
  if (device < 0 || device >= num_devices_) Violation("task '" + options.name + "' submitted for an unknown device");
  for (auto& r : reads) {
    auto it = tiles_.find(r);
    if (it == tiles_.end()) { Violation("task '" + options.name + "' reads a tile that does not exist"); continue; }
    if (it->second.host && !reshard) Violation("task '" + options.name + "' reads an offloaded input");
  }
  for (auto& w : writes) {
    auto it = tiles_.find(w);
    if (it == tiles_.end()) { Violation("task '" + options.name + "' writes a tile that does not exist"); continue; }
    if (!reshard && w.device != device) Violation("task '" + options.name + "' writes a tile of another device");
    it->second.reshard_pending = false;
  }
  std::vector<uint64_t> deps = deps_.Register(id, device, reads, writes, options.strict_ordering);
  submissions_.push_back(SubmittedTask{id, reads, writes, deps, options.name});
  log_.push_back(TaskRecord{id, options.name, device, reshard ? 1 : 0, options.step, 0, 0, 0, false, false});
  return id;
}
uint64_t MockContext::CreateExecuteTask(int device, const std::vector<TileRef>& reads,
                                        const std::vector<TileRef>& writes, Body, const ExecuteOptions& options) {
  ++num_tasks_;
  return Record(device, reads, writes, options, false);
}
uint64_t MockContext::Reshard(int device, const std::vector<TileRef>& reads, const std::vector<TileRef>& writes,
                              Body, const ExecuteOptions& options) {
  ++num_reshards_;
  return Record(device, reads, writes, options, true);
}
void MockContext::CreateStore(int buffer, int device, int64_t bytes, bool host) {
  TileRef t{buffer, device};
  if (tiles_.count(t)) return;
  tiles_[t] = Tile{bytes, host, false};
  std::ostringstream os;
  os << "create " << buffer << "@" << device << " " << bytes;
  Mix(os.str());
  if (host) { host_bytes_ += bytes; host_hwm_ = std::max(host_hwm_, host_bytes_); }
  else { device_bytes_[device] += bytes; device_hwm_[device] = std::max(device_hwm_[device], device_bytes_[device]); }
}
void MockContext::FreeStore(int buffer, int device) {
  auto it = tiles_.find(TileRef{buffer, device});
  if (it == tiles_.end()) { Violation("free of a tile that does not exist"); return; }
  if (it->second.host) host_bytes_ -= it->second.bytes;
  else device_bytes_[device] -= it->second.bytes;
  tiles_.erase(it);
  deps_.Forget(buffer, device);
  std::ostringstream os;
  os << "free " << buffer << "@" << device;
  Mix(os.str());
}
void MockContext::OffloadDtoH(int buffer, int device) {
  auto it = tiles_.find(TileRef{buffer, device});
  if (it == tiles_.end()) { Violation("offload of a tile that does not exist"); return; }
  if (it->second.reshard_pending) Violation("offload before the reshard into the tile finished");
  if (it->second.host) return;
  it->second.host = true;
  device_bytes_[device] -= it->second.bytes;
  host_bytes_ += it->second.bytes;
  host_hwm_ = std::max(host_hwm_, host_bytes_);
  Mix("d2h");
}
void MockContext::OffloadHtoD(int buffer, int device) {
  auto it = tiles_.find(TileRef{buffer, device});
  if (it == tiles_.end()) { Violation("prefetch of a tile that does not exist"); return; }
  if (!it->second.host) return;
  it->second.host = false;
  host_bytes_ -= it->second.bytes;
  device_bytes_[device] += it->second.bytes;
  device_hwm_[device] = std::max(device_hwm_[device], device_bytes_[device]);
  Mix("h2d");
}
Status MockContext::WaitAll(std::string* message) {
  if (!violation_.empty()) {
    if (message) *message = violation_;
    return Status::kProtocolViolation;
  }
  return Status::kOk;
}
int64_t MockContext::device_high_water(int device) const {
  auto it = device_hwm_.find(device);
  return it == device_hwm_.end() ? 0 : it->second;
}
int64_t MockContext::max_device_high_water() const {
  int64_t m = 0;
  for (auto& kv : device_hwm_) m = std::max(m, kv.second);
  return m;
}

}  // namespace mmrt
