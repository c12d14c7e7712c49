// Pass interfaces of the MPMD compiler. Each pass is a free function over a
// CompileState; MpmdPartition() (pipeline.cc) runs them in order, validates
// the graph after each one and optionally dumps it.
//
// Pass order follows src/pjrt_client/mpmd_partition.cc:872-961. XLA-specific
// steps collapse: optimisation-barrier pack/unpack and the cross-task barrier
// remover have no counterpart because torch.fx captures carry no barriers;
// iota sanitising is unnecessary because shardings are stored submesh-relative
// from the start; reorder-shard-map-transpose is folded into the layout flags
// of the GEMM kernels.
#pragma once
#include <string>
#include <vector>

#include "graph.h"
#include "schedule.h"

namespace mmg {

// A group of same-colour nodes that will execute as one task.
struct TaskGroup {
  int id = -1;
  std::string color;
  int region = 0;  // 0 = before the microbatch loop, 1 = loop body, 2 = after it
  std::vector<int> nodes;
  bool noncritical = false;
};

struct CompileState {
  Graph* graph = nullptr;
  Partition* partition = nullptr;
  PartitionConfig config;
  std::vector<TaskGroup> groups;  // in execution order
  std::vector<std::string> log;   // human-readable notes from passes
  void Note(const std::string& s) { log.push_back(s); }
};

// ---- op classification ------------------------------------------------------
bool IsMarker(const Node& n);
bool IsElementwise(const Node& n);
bool IsAliasOp(const Node& n);      // view-like: output shares the input's data
bool IsFactory(const Node& n);      // no tensor operands
bool IsDot(const Node& n);          // matmul-like contraction
bool IsReduce(const Node& n);
bool IsConvert(const Node& n);      // dtype cast
bool IsCollective(const Node& n);
bool IsExpensive(const Node& n);    // dot / attention / custom kernels: never recomputed
int64_t NodeFlops(const Graph& g, const Node& n);

// Per-node facts derived from the whole graph (the role of InstructionProperties,
// src/pjrt_client/mpmd_utils.h:69-189).
struct ValueProperties {
  std::vector<bool> derived_constant;   // per node: computed from constants only
  std::vector<bool> derived_parameter;  // per node: cheap function of graph inputs only
  std::vector<int> depth;               // per node: longest path from an input
  std::vector<int> topo_index;          // per node: position in graph.order
  std::vector<int> region;              // per node: 0 pre-loop, 1 loop, 2 post-loop
  static ValueProperties Compute(const Graph& g);
};

// ---- passes (return value: whether the graph changed) ------------------------
void ValidateCircularDependencies(const CompileState& s, const std::string& after_pass);
bool ConstantOutputCopy(CompileState& s);
bool RepeatedOutputCopy(CompileState& s);
bool MicrobatchLoopCanonicalizer(CompileState& s);
bool SimpleLoopIncrementColoring(CompileState& s);
bool UnusedLoopOutputRemover(CompileState& s);
bool Coloring(CompileState& s);
bool LogicalShardingPropagation(CompileState& s);
bool HoistLoopConvert(CompileState& s);
bool ParameterReplication(CompileState& s);
bool ReplicateUncolored(CompileState& s);
bool ComputationGrouper(CompileState& s);
enum class FusionMode { kMatchingColor, kOriginalColor, kMatchingDevices };
bool ComputationFusion(CompileState& s, FusionMode mode);
bool UniquifyColors(CompileState& s);
bool InstructionDelayRecolor(CompileState& s);
bool ArgumentRecompute(CompileState& s);
bool CutSizeMinimizer(CompileState& s);
bool SplitCriticalPath(CompileState& s);
bool LogicalToPhysicalSharding(CompileState& s);
enum class PropagationMode { kForwardInputOutput, kBackwardInputOutput, kForwardFull };
bool ShardingPropagation(CompileState& s, PropagationMode mode);
bool SpmdLowering(CompileState& s);         // contracting-dim dots -> local op + collective
bool HoistShardMapReduce(CompileState& s);  // gradient reductions once per step, after the loop
bool ReduceScatterCreator(CompileState& s); // all-reduce + slice -> reduce-scatter; tags all-gathers
bool SplitUpdateByReduction(CompileState& s);  // optimizer task cut into pieces behind the hoisted reductions
bool UnusedParamOutputRemover(CompileState& s);

// Final stage: unroll + schedule + reshard + buffers -> Plan.
Plan BuildPlan(CompileState& s);

// Whole pipeline.
Plan MpmdPartition(Graph& g, Partition& p, const PartitionConfig& cfg, std::vector<std::string>* log = nullptr);

// Per-task sharding helpers shared by passes.
ShardedShape DefaultSharding(const Value& v, const ColorConfig& c);

}  // namespace mmg
