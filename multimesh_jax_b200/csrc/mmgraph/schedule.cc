#include "schedule.h"

#include <algorithm>
#include <map>
#include <queue>
#include <set>
#include <stdexcept>
#include <tuple>

namespace mmg {

bool EnforceBijectiveTasks(const std::string& schedule) {
  return schedule == "custom" || schedule == "zero-bubble-h2";
}

ScheduleResult ScheduleFillDrain(const std::vector<std::vector<SchedTask>>& tasks) {
  ScheduleResult r;
  r.orders.emplace_back();
  if (tasks.empty()) return r;
  const int stages = static_cast<int>(tasks[0].size());
  for (int s = 0; s < stages; ++s)
    for (size_t it = 0; it < tasks.size(); ++it) r.orders[0].emplace_back(static_cast<int>(it), s);
  return r;
}

static int NumGroups(const std::vector<SchedTask>& row) {
  std::set<DeviceRange> lists;
  for (auto& t : row) if (!t.on_full_mesh) lists.insert(t.devices);
  return std::max<int>(1, static_cast<int>(lists.size()));
}

ScheduleResult ScheduleWavefront(const LoopConfig& cfg, const std::vector<std::vector<SchedTask>>& tasks,
                                 bool prefetch) {
  ScheduleResult r;
  r.orders.emplace_back();
  if (tasks.empty()) return r;
  auto& order = r.orders[0];
  const int num_iters = static_cast<int>(tasks.size());
  // prefetch tasks (loop counter updates, round-robin embeddings ...) go first for all iterations
  std::vector<int> stages;
  for (size_t s = 0; s < tasks[0].size(); ++s) {
    if (prefetch && tasks[0][s].prefetch) {
      for (int it = 0; it < num_iters; ++it) order.emplace_back(it, static_cast<int>(s));
    } else {
      stages.push_back(static_cast<int>(s));
    }
  }
  const int pipeline_tasks = static_cast<int>(stages.size());
  if (pipeline_tasks <= 1) {  // a single-task body degenerates to fill-drain
    for (int s : stages) for (int it = 0; it < num_iters; ++it) order.emplace_back(it, s);
    return r;
  }
  std::vector<SchedTask> row;
  for (int s : stages) row.push_back(tasks[0][s]);
  const int minibatch_size = NumGroups(row);
  // a minibatch needs at least one tick per member, whatever the caller asked for
  const int delay = std::max(minibatch_size, cfg.num_stages > 0 ? cfg.num_stages : std::max(1, (pipeline_tasks + 1) / 2));
  const int num_minibatches = (num_iters + minibatch_size - 1) / minibatch_size;
  const int last_wf = pipeline_tasks + num_minibatches * delay;
  for (int wf = 0; wf < last_wf; ++wf) {
    for (int si = pipeline_tasks - 1; si >= 0; --si) {
      const int tick = wf - si;
      if (tick < 0) continue;
      const int minibatch = tick / delay;
      const int off = tick % delay;
      if (off >= minibatch_size) continue;
      const int it = minibatch * minibatch_size + off;
      if (it >= num_iters) continue;
      order.emplace_back(it, stages[si]);
    }
  }
  return r;
}

ScheduleResult ScheduleZeroBubbleH2(const LoopConfig& cfg, const std::vector<std::vector<SchedTask>>& tasks) {
  ScheduleResult r;
  r.orders.emplace_back();
  if (tasks.empty()) return r;
  const int num_iters = static_cast<int>(tasks.size());
  // Row order: critical tasks as they are, then non-critical ones, the consumer of the
  // latest critical stage first (so the weight gradient of the last backward runs first).
  std::vector<int> crit, noncrit;
  for (size_t s = 0; s < tasks[0].size(); ++s) (tasks[0][s].noncritical ? noncrit : crit).push_back(static_cast<int>(s));
  std::stable_sort(noncrit.begin(), noncrit.end(), [&](int a, int b) {
    return tasks[0][a].consumes_stage > tasks[0][b].consumes_stage;
  });
  std::vector<int> row = crit;
  row.insert(row.end(), noncrit.begin(), noncrit.end());
  const int n = static_cast<int>(row.size());
  std::vector<SchedTask> group_row;
  for (int s : row) group_row.push_back(tasks[0][s]);
  const int minibatch_size = NumGroups(group_row);
  const int delay = cfg.num_stages > 0 ? cfg.num_stages : std::max(1, (static_cast<int>(crit.size()) + 1) / 2);
  using Key = std::tuple<int, int, int>;  // (wavefront, microbatch, position in row)
  std::priority_queue<Key, std::vector<Key>, std::greater<Key>> heap;
  for (int it = 0; it < num_iters; ++it) {
    const int minibatch = it / minibatch_size, in_mb = it % minibatch_size;
    for (int p = 0; p < n; ++p) heap.emplace(minibatch * delay + in_mb + p, it, p);
  }
  // unit-cost simulation: one clock per device list and per microbatch, +0.1 per mesh change
  std::map<DeviceRange, double> device_clock;
  std::vector<double> mb_clock(num_iters, 0.0);
  std::vector<DeviceRange> mb_last(num_iters);
  std::vector<bool> mb_seen(num_iters, false);
  while (!heap.empty()) {
    auto [wf, it, p] = heap.top();
    heap.pop();
    (void)wf;
    const SchedTask& t = tasks[it][row[p]];
    r.orders[0].emplace_back(it, row[p]);
    double start = device_clock[t.devices];
    if (!t.noncritical) {
      double ready = mb_clock[it];
      if (mb_seen[it] && mb_last[it] != t.devices) ready += 0.1;
      start = std::max(start, ready);
    }
    const double end = start + 1.0;
    device_clock[t.devices] = end;
    if (!t.noncritical) {
      mb_clock[it] = end;
      mb_last[it] = t.devices;
      mb_seen[it] = true;
    }
    r.simulated_makespan = std::max(r.simulated_makespan, end);
  }
  return r;
}

ScheduleResult ScheduleCustom(const LoopConfig& cfg, const std::vector<std::vector<SchedTask>>& tasks) {
  ScheduleResult r;
  if (tasks.empty()) return r;
  const int num_iters = static_cast<int>(tasks.size());
  if (cfg.custom_schedule.empty()) throw std::runtime_error("custom schedule: no rows given");
  std::map<std::string, int> name_count;
  std::set<std::pair<int, int>> seen;
  for (auto& row : cfg.custom_schedule) {
    r.orders.emplace_back();
    for (auto& entry : row) {
      const int it = entry.first;
      const std::string& name = entry.second;
      if (it < 0 || it >= num_iters)
        throw std::runtime_error("custom schedule: microbatch index out of range for task '" + name + "'");
      int found = -1;
      for (size_t s = 0; s < tasks[it].size(); ++s) {
        if (tasks[it][s].color.find(name) == std::string::npos) continue;
        if (found >= 0)
          throw std::runtime_error("custom schedule: name '" + name + "' matches more than one task of a microbatch");
        found = static_cast<int>(s);
      }
      if (found < 0) throw std::runtime_error("custom schedule: no task matches '" + name + "'");
      if (!seen.insert({it, found}).second)
        throw std::runtime_error("custom schedule: task '" + name + "' scheduled twice for one microbatch");
      ++name_count[name];
      r.orders.back().emplace_back(it, found);
    }
  }
  for (auto& kv : name_count)
    if (kv.second != num_iters)
      throw std::runtime_error("custom schedule: task '" + kv.first + "' appears " + std::to_string(kv.second) +
                               " times, expected " + std::to_string(num_iters));
  if (static_cast<int>(seen.size()) != num_iters * static_cast<int>(tasks[0].size()))
    throw std::runtime_error("custom schedule: not every loop task is scheduled");
  return r;
}

ScheduleResult ScheduleLoops(const LoopConfig& cfg, const std::vector<std::vector<SchedTask>>& tasks) {
  const std::string& s = cfg.schedule;
  if (s.empty() || s == "gpipe" || s == "fill-drain" || s == "breadth-first") return ScheduleFillDrain(tasks);
  if (s == "1f1b" || s == "wavefront") return ScheduleWavefront(cfg, tasks, /*prefetch=*/false);
  if (s == "prefetch-wavefront") return ScheduleWavefront(cfg, tasks, /*prefetch=*/true);
  if (s == "zero-bubble-h2") return ScheduleZeroBubbleH2(cfg, tasks);
  if (s == "custom") return ScheduleCustom(cfg, tasks);
  throw std::runtime_error("unknown microbatch schedule '" + s + "'");
}

}  // namespace mmg
