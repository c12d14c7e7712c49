// The compiler driver: runs the passes in order over one captured step, validates
// after each pass and optionally dumps the graph (the role of MpmdPartition,
// src/pjrt_client/mpmd_partition.cc:791-986).
#include <fstream>
#include <stdexcept>

#include "passes.h"

namespace mmg {

void ReleaseShardingTables(const CompileState& s);

namespace {

void Dump(const CompileState& s, const std::string& stage, int* counter) {
  if (s.config.dump_dir.empty()) return;
  char buf[16];
  snprintf(buf, sizeof(buf), "%02d", (*counter)++);
  std::ofstream f(s.config.dump_dir + "/" + buf + "_" + stage + ".txt");
  f << "# " << stage << "\n" << s.graph->Dump();
  if (!s.groups.empty()) {
    f << "# tasks\n";
    for (auto& grp : s.groups) {
      f << "task " << grp.id << " color=" << grp.color << " region=" << grp.region << " nodes=";
      for (int id : grp.nodes) f << id << " ";
      f << "\n";
    }
  }
}

template <class F>
void RunPass(CompileState& s, const char* name, F&& fn, int* counter) {
  const bool changed = fn();
  ValidateCircularDependencies(s, name);
  if (s.config.dump_all_passes || changed) {
    if (s.config.dump_all_passes) Dump(s, std::string("after_") + name, counter);
  }
}

}  // namespace

Plan MpmdPartition(Graph& g, Partition& part, const PartitionConfig& cfg, std::vector<std::string>* log) {
  CompileState s;
  s.graph = &g;
  s.partition = &part;
  s.config = cfg;
  int counter = 0;
  g.Toposort();
  g.DeadCodeElimination();
  Dump(s, "before_mpmd_preprocess", &counter);

  RunPass(s, "constant_output_copy", [&] { return ConstantOutputCopy(s); }, &counter);
  RunPass(s, "repeated_output_copy", [&] { return RepeatedOutputCopy(s); }, &counter);
  RunPass(s, "microbatch_loop_canonicalizer", [&] { return MicrobatchLoopCanonicalizer(s); }, &counter);
  Dump(s, "after_mpmd_preprocess", &counter);
  RunPass(s, "simple_loop_increment_coloring", [&] { return SimpleLoopIncrementColoring(s); }, &counter);
  RunPass(s, "coloring", [&] { return Coloring(s); }, &counter);
  RunPass(s, "unused_loop_output_remover", [&] { return UnusedLoopOutputRemover(s); }, &counter);
  RunPass(s, "logical_sharding_propagation", [&] { return LogicalShardingPropagation(s); }, &counter);
  RunPass(s, "hoist_loop_convert", [&] { return HoistLoopConvert(s); }, &counter);
  RunPass(s, "parameter_replication", [&] { return ParameterReplication(s); }, &counter);
  RunPass(s, "replicate_uncolored", [&] { return ReplicateUncolored(s); }, &counter);

  // first grouping: gives the recolouring optimisations a task order to reason about
  RunPass(s, "computation_grouper", [&] { return ComputationGrouper(s); }, &counter);
  RunPass(s, "computation_fusion_matching_color", [&] { return ComputationFusion(s, FusionMode::kMatchingColor); }, &counter);
  bool recolored = false;
  RunPass(s, "instruction_delay_recolor", [&] { bool c = InstructionDelayRecolor(s); recolored |= c; return c; }, &counter);
  RunPass(s, "argument_recompute", [&] { bool c = ArgumentRecompute(s); recolored |= c; return c; }, &counter);
  RunPass(s, "cut_size_minimizer", [&] { bool c = CutSizeMinimizer(s); recolored |= c; return c; }, &counter);
  if (recolored) {
    s.groups.clear();
    RunPass(s, "computation_grouper_2", [&] { return ComputationGrouper(s); }, &counter);
  }
  // after the regrouping: call sites that descend from the same user task fuse again where the
  // dependencies allow it (src/pjrt_client/mpmd_partition.cc:946)
  RunPass(s, "computation_fusion_original_color", [&] { return ComputationFusion(s, FusionMode::kOriginalColor); }, &counter);
  RunPass(s, "split_critical_path", [&] { return SplitCriticalPath(s); }, &counter);
  std::string schedule = g.loops.empty() ? "" : g.loops[0].schedule;
  if (!EnforceBijectiveTasks(schedule))
    RunPass(s, "computation_fusion_matching_devices", [&] { return ComputationFusion(s, FusionMode::kMatchingDevices); }, &counter);
  RunPass(s, "uniquify_colors", [&] { return UniquifyColors(s); }, &counter);
  Dump(s, "global_mpmd", &counter);

  RunPass(s, "logical_to_physical_sharding", [&] { return LogicalToPhysicalSharding(s); }, &counter);
  RunPass(s, "sharding_propagation_forward_io", [&] { return ShardingPropagation(s, PropagationMode::kForwardInputOutput); }, &counter);
  RunPass(s, "sharding_propagation_backward_io", [&] { return ShardingPropagation(s, PropagationMode::kBackwardInputOutput); }, &counter);
  RunPass(s, "sharding_propagation_forward_full", [&] { return ShardingPropagation(s, PropagationMode::kForwardFull); }, &counter);
  RunPass(s, "spmd_lowering", [&] { return SpmdLowering(s); }, &counter);
  RunPass(s, "hoist_shard_map_reduce", [&] { return HoistShardMapReduce(s); }, &counter);
  RunPass(s, "reduce_scatter_creator", [&] { return ReduceScatterCreator(s); }, &counter);
  RunPass(s, "split_update_by_reduction", [&] { return SplitUpdateByReduction(s); }, &counter);
  RunPass(s, "unused_param_output_remover", [&] { return UnusedParamOutputRemover(s); }, &counter);
  Dump(s, "after_mpmd_partitioning", &counter);

  Plan plan = BuildPlan(s);
  if (!cfg.dump_dir.empty()) {
    std::ofstream f(cfg.dump_dir + "/plan.txt");
    f << plan.Dump(g);
  }
  for (auto& grp : s.groups) (void)grp;
  if (log) *log = s.log;
  ReleaseShardingTables(s);
  return plan;
}

}  // namespace mmg
