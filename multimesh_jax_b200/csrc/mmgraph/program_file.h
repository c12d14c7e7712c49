// Stored programs and the offline compile entry point (see program_file.cc).
#pragma once
#include <memory>

#include "passes.h"

namespace mmg {

Json GraphToJson(const Graph& g);
Graph GraphFromJson(const Json& j);
// Throws std::runtime_error when an id, a producer / result link, a loop reference or a shape of
// a graph read from a file is inconsistent (GraphFromJson calls it before anything follows an id).
void ValidateStoredGraph(const Graph& g);

struct StoredProgram {
  std::shared_ptr<Graph> graph;
  std::shared_ptr<Partition> partition;
  PartitionConfig config;
};

// Serialises a captured step *before* it is partitioned (the pipeline rewrites the graph in place).
std::string ProgramToJson(const Graph& g, Partition& part, const PartitionConfig& cfg);
StoredProgram ProgramFromJson(const std::string& text);
void SaveProgram(const std::string& path, const Graph& g, Partition& part, const PartitionConfig& cfg);
StoredProgram LoadProgram(const std::string& path);

struct OfflineResult {
  int status = 0;                 // mmrt::Status of the mock run
  std::string message;            // protocol violation, if any
  std::string hazards;            // first unordered conflicting pair of the submission log, "" when race free
  uint64_t plan_hash = 0;         // hash of the plan's operation list
  uint64_t operation_hash = 0;    // hash of what the mock runtime was asked to do
  int templates = 0, stores = 0, tasks = 0, reshards = 0;
  int64_t reshard_bytes = 0;
  int64_t temp_bytes_per_device_max = 0;
  int64_t device_high_water_max = 0;
  std::vector<int64_t> device_high_water;
  bool fits = true;               // device_high_water_max <= the fake device-memory size (always true for size 0)
  std::map<std::string, std::string> stats;
  std::vector<std::string> template_names;
};

// Replays `plan` for `steps` steps on the mock runtime.
OfflineResult MockExecutePlan(const Plan& plan, int device_start, int num_devices, int64_t device_memory_bytes, int steps);
// Loads a stored program, partitions it and replays the plan on the mock runtime.
OfflineResult CompileProgramFile(const std::string& path, int64_t device_memory_bytes, Plan* plan_out = nullptr,
                                 std::vector<std::string>* log = nullptr);

}  // namespace mmg
