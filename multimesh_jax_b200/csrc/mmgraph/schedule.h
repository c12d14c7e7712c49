// Pipeline schedules for the unrolled microbatch loop.
//
// Input: tasks[iteration][stage] in loop-body order. Output: one or more
// orders of (iteration, stage) pairs; consecutive tasks of an order that run
// on identical device lists are later chained by control dependencies
// (behaviour of src/pjrt_client/loop_scheduler.cc:69-533 and
// src/pjrt_client/mpmd_loop_unroll.cc:334-350).
#pragma once
#include <string>
#include <utility>
#include <vector>

#include "graph.h"

namespace mmg {

struct SchedTask {
  int iteration = 0;
  int stage = 0;              // index in the loop body
  std::string color;          // unique colour (matched by substring in custom schedules)
  DeviceRange devices;
  bool noncritical = false;   // weight-gradient half of a split backward task
  bool on_full_mesh = false;  // runs on every device of the executable
  bool prefetch = false;      // coloured `loop_increment`: emitted ahead of the pipeline
  int consumes_stage = -1;    // for non-critical tasks: latest critical stage they read from
};

using SchedEntry = std::pair<int, int>;  // (iteration, stage)
struct ScheduleResult {
  // One global order, or (custom schedules) one order per mesh.
  std::vector<std::vector<SchedEntry>> orders;
  // Simulated makespan in task units (zero-bubble only; 0 otherwise).
  double simulated_makespan = 0;
};

ScheduleResult ScheduleFillDrain(const std::vector<std::vector<SchedTask>>& tasks);
ScheduleResult ScheduleWavefront(const LoopConfig& cfg, const std::vector<std::vector<SchedTask>>& tasks,
                                 bool prefetch);
ScheduleResult ScheduleZeroBubbleH2(const LoopConfig& cfg, const std::vector<std::vector<SchedTask>>& tasks);
ScheduleResult ScheduleCustom(const LoopConfig& cfg, const std::vector<std::vector<SchedTask>>& tasks);
// Dispatch on cfg.schedule ("gpipe", "1f1b", "wavefront", "prefetch-wavefront", "zero-bubble-h2", "custom").
ScheduleResult ScheduleLoops(const LoopConfig& cfg, const std::vector<std::vector<SchedTask>>& tasks);

// Schedules that need tasks to stay one-to-one with schedule entries
// (no device-based fusion of loop tasks).
bool EnforceBijectiveTasks(const std::string& schedule);

}  // namespace mmg
