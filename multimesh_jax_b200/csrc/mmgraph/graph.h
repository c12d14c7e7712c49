// mmgraph: the graph IR of the MPMD compiler, the colour table ("Partition"),
// the compile configuration and the resulting execution plan.
//
// A captured training step arrives from torch.fx as a flat list of nodes over
// SSA values. Passes annotate nodes with a *colour* (task id string) and
// values with logical axes / physical shardings, group nodes into tasks,
// unroll the microbatch loop at task granularity, schedule it, insert
// cross-submesh reshards and plan buffers. The result is a linear list of
// operations (task / reshard / create-store / free-store) over stores, the
// same shape of output as the reference's MpmdPartition
// (src/pjrt_client/mpmd_partition.h:30-92).
#pragma once
#include <functional>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "json.h"
#include "sharding.h"

namespace mmg {

// ---------------------------------------------------------------------------
// IR
// ---------------------------------------------------------------------------
struct Value {
  int id = -1;
  std::string name;
  std::vector<int64_t> shape;
  DType dtype = DType::F32;
  int producer = -1;    // node id, or -1 for a graph input
  int out_index = 0;    // which output of the producer
  int input_index = -1; // position among graph inputs (if producer == -1)
  std::vector<std::vector<std::string>> axes;  // logical axis names per dim
  bool has_axes = false;
  bool axes_logical = true;   // false: names are mesh axes (fixed sharding)
  ShardedShape sharding;      // physical sharding on the owning task's submesh
  bool has_sharding = false;
  bool partial = false;       // holds a partial sum over `partial_axes` mesh axes
  std::vector<int> partial_axes;
  int64_t Elements() const { int64_t n = 1; for (auto s : shape) n *= s; return n; }
  int64_t Bytes() const { return Elements() * static_cast<int64_t>(DTypeSize(dtype)); }
};

struct Node {
  int id = -1;
  std::string op;              // e.g. "aten.mm.default", "mm.marker", "mm.reshard"
  std::vector<int> inputs;     // tensor operands (value ids)
  std::vector<int> outputs;    // tensor results (value ids)
  std::map<std::string, std::string> attrs;  // "args" (JSON of non-tensor args), marker kind/payload ...
  std::string scope;           // name stack at creation ("a/b/c")
  bool backprop = false;       // created while running the backward pass
  int loop = -1;               // id of the enclosing microbatch loop, or -1
  std::string explicit_task;   // JSON payload of an explicit task(), or ""
  std::string color;           // task colour; "" = not (yet) coloured
  int task = -1;               // task (group) id after grouping
  bool dead = false;
  std::string Attr(const std::string& k, const std::string& dflt = "") const {
    auto it = attrs.find(k);
    return it == attrs.end() ? dflt : it->second;
  }
};

struct LoopConfig {
  int id = 0;
  int num_microbatches = 1;
  int slice_dim = 0;
  int64_t size = 0;
  int batch_dim = 0;
  int interleave = 1;
  int unrolling = 0;
  int num_stages = 0;            // 0 = derive
  std::string schedule = "gpipe";
  // rows = meshes, entries = (microbatch index, task-name substring)
  std::vector<std::vector<std::pair<int, std::string>>> custom_schedule;
  std::string accumulate_dtype;  // "" = dtype of the summed value
  static LoopConfig FromJson(const Json& j);
};

class Graph {
 public:
  std::vector<Value> values;
  std::vector<Node> nodes;
  std::vector<int> order;    // node ids in a valid topological order
  std::vector<int> inputs;   // value ids
  std::vector<int> outputs;  // value ids
  std::vector<LoopConfig> loops;
  std::vector<int> donated_inputs;  // indices of graph inputs whose buffers may be reused

  int AddInput(const std::string& name, std::vector<int64_t> shape, DType dtype);
  // Adds a node with fresh output values; returns the node id.
  int AddNode(const std::string& op, const std::vector<int>& inputs,
              const std::vector<std::vector<int64_t>>& out_shapes, const std::vector<DType>& out_dtypes,
              const std::map<std::string, std::string>& attrs = {});
  void SetOutputs(const std::vector<int>& value_ids) { outputs = value_ids; }

  const Node& node(int id) const { return nodes[id]; }
  Node& node(int id) { return nodes[id]; }
  const Value& value(int id) const { return values[id]; }
  Value& value(int id) { return values[id]; }

  // Users of a value (node ids, live nodes only), recomputed on demand.
  std::vector<std::vector<int>> ComputeUsers() const;
  // Recomputes `order` (stable w.r.t. the previous order); throws on a cycle.
  void Toposort();
  // Marks nodes that do not reach an output as dead. Returns #removed.
  int DeadCodeElimination();
  // Replaces every use of `from` by `to` (also among graph outputs).
  void ReplaceAllUses(int from, int to);
  bool IsLive(int node_id) const { return !nodes[node_id].dead; }
  std::string Dump() const;  // human-readable listing (one node per line)
};

// ---------------------------------------------------------------------------
// Colour table
// ---------------------------------------------------------------------------
struct TaskOptions {
  std::string name;
  std::vector<int> devices;
  std::vector<int> dims;
  std::vector<std::string> device_axes;
  std::vector<std::pair<std::string, std::string>> logical_axes;
  std::vector<std::string> split_backprop;                 // {} or {critical sfx, noncritical sfx}
  std::vector<std::vector<int>> loop_dependent_devices;    // per microbatch, or {}
  static TaskOptions FromJson(const Json& j);
  Json ToJson() const;
};

struct ColorConfig {
  std::string name;
  DeviceRange devices;
  bool backprop = false;
  bool noncritical = false;
  TaskOptions options;
  std::string original;  // colour before uniquification
};

// callback(matched_group, backprop) -> JSON text of a TaskOptions record.
using TaskFactory = std::function<std::string(const std::string&, bool)>;

class Partition {
 public:
  explicit Partition(DeviceRange global) : global_(global) {
    ColorConfig g;
    g.name = kGlobalColor;
    g.devices = global;
    g.options.name = kGlobalColor;
    g.options.devices = global.ToList();
    g.options.dims = {global.n};
    g.options.device_axes = {"x"};
    colors_[kGlobalColor] = g;
  }
  static constexpr const char* kGlobalColor = "global";
  static constexpr const char* kLoopIncrementColor = "loop_increment";

  DeviceRange global() const { return global_; }
  bool Has(const std::string& color) const { return colors_.count(color) > 0; }
  const ColorConfig& Get(const std::string& color) const;
  ColorConfig& GetMutable(const std::string& color);
  // Registers a colour; the same name may not map to two device lists.
  const ColorConfig& Add(const TaskOptions& opts, bool backprop, const std::string& color_name = "");
  // Gives `color` a new unique name; the original colour is remembered.
  std::string Recolor(const std::string& color, const std::string& new_name);
  std::string Clone(const std::string& color, const std::string& new_name, DeviceRange devices);

  // Regex contexts, innermost first.
  void RegisterFactory(const std::string& regex, TaskFactory factory);
  void ClearFactories() { factories_.clear(); cache_.clear(); }
  // Resolves the colour of an operator from its name stack; "" when nothing matches.
  std::string ComputeScopeColor(const std::string& scope, bool backprop);
  // Fixes the colour of one name stack (stored programs carry the resolved table instead of
  // the regex contexts, which are callbacks of the process that captured the step).
  void PinScopeColor(const std::string& scope, bool backprop, const std::string& color) {
    pinned_[{scope, backprop}] = color;
  }
  const std::map<std::string, ColorConfig>& colors() const { return colors_; }

 private:
  DeviceRange global_;
  std::map<std::string, ColorConfig> colors_;
  std::vector<std::pair<std::string, TaskFactory>> factories_;
  std::map<std::pair<std::string, bool>, std::string> cache_;
  std::map<std::pair<std::string, bool>, std::string> pinned_;
};

// ---------------------------------------------------------------------------
// Configuration (per-call struct + environment options)
// ---------------------------------------------------------------------------
struct PartitionConfig {
  bool use_task_fusion = true;
  int64_t replicated_parameter_num_elements_cutoff = 0;
  bool run_simplification_passes = true;
  bool only_fuse_loop_tasks = false;
  bool hoist_loop_convert = false;
  bool remove_hoisted_reduces = false;
  int64_t recompute_from_arguments_if_cost_less_than = 1 << 20;
  bool argument_recompute = true;
  bool minimize_cut_size = true;
  bool loop_increment_color = false;
  bool enable_recomputation = true;
  // hoisted parameter casts produce zeros (debugging aid: isolates the cost / effect of the casts)
  bool zero_arguments = false;
  // tasks outside the microbatch loop that contain no collective may overtake one another;
  // false = every task keeps its submission order on its device
  bool dynamic_schedule_post_loop_tasks = true;
  std::string color_propagation_priority = "WEIGHT";  // WEIGHT | DEPTH | TOPOLOGICAL
  std::string dump_dir;
  bool dump_all_passes = false;
  // Reads the MULTIMESH_* environment variables on top of the defaults.
  static PartitionConfig FromEnv();
};
bool GetEnvBool(const char* name, bool dflt);
int64_t GetEnvInt(const char* name, int64_t dflt);
std::string GetEnvString(const char* name, const std::string& dflt);

// ---------------------------------------------------------------------------
// Plan (output of the compiler)
// ---------------------------------------------------------------------------
struct TaskTemplate {
  int id = -1;
  std::string name;            // unique colour, e.g. "3.stage1_bwd" (+"_loop" for loop bodies)
  std::string original_color;
  DeviceRange devices;
  std::vector<int> mesh_dims;
  std::vector<std::string> mesh_axes;
  std::vector<int> nodes;      // node ids in execution order
  std::vector<int> inputs;     // value ids consumed from outside the task
  std::vector<int> outputs;    // value ids visible outside the task
  bool in_loop = false;
  bool backprop = false;
  bool noncritical = false;
  bool has_collectives = false;
  int64_t flops = 0;
};

struct Store {
  enum Kind { PARAM = 0, ROOT = 1, TEMP = 2 };
  int id = -1;
  Kind kind = TEMP;
  int index = -1;          // parameter / root index, or temp ordinal
  std::string name;        // scheduling name == physical buffer identity
  bool scalar = false;
  ShardedShape shape;
  int value = -1;          // IR value this store materialises
  int iteration = -1;      // microbatch, or -1
  int alias_of = -1;       // store id whose buffer this one reuses (donation / in-place), or -1
};

struct PlanOp {
  enum Kind { TASK = 0, RESHARD = 1, CREATE_STORE = 2, FREE_STORE = 3 };
  Kind kind = TASK;
  // TASK
  int task_template = -1;
  std::string name;
  DeviceRange devices;
  std::vector<int> inputs;     // store ids, aligned with TaskTemplate::inputs
  std::vector<int> outputs;    // store ids, aligned with TaskTemplate::outputs
  std::vector<int> accumulate; // per output: 0 plain write, 1 "first write of an accumulator", 2 "+="
  std::vector<int64_t> scalars;  // microbatch slice offsets etc.
  bool loop = false;
  int iteration = -1;
  int priority = 0;
  bool strict_ordering = false;
  // RESHARD
  int src_store = -1;
  int dst_store = -1;
  // CREATE_STORE / FREE_STORE
  int store = -1;
};

struct Plan {
  std::vector<TaskTemplate> templates;
  std::vector<Store> stores;
  std::vector<PlanOp> ops;
  std::vector<int> param_stores;   // graph input i  -> store id (-1 if unused)
  std::vector<int> root_stores;    // graph output j -> store id
  std::vector<int> unused_params;
  std::vector<std::pair<int, int>> aliases;  // (param store, root store) sharing a buffer
  int64_t temp_bytes_per_device_max = 0;
  std::map<std::string, std::string> stats;
  std::string Dump(const Graph& g) const;
  // Order-sensitive hash of the operation list (for determinism checks).
  uint64_t Hash() const;
};

}  // namespace mmg
