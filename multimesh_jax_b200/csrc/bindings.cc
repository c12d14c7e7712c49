// pybind11 module `_mm_C`: graph ingest from torch.fx, the colour table and task-factory
// registry, the compiler entry points (whole pipeline and single passes), sharding
// algebra, loop schedulers and the task-graph runtime. This is the counterpart of the
// reference's native binding layer (src/plugin/multimesh_jax_impl.cc:96-177).
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "mmgraph/graph.h"
#include "mmgraph/passes.h"
#include "mmgraph/program_file.h"
#include "mmgraph/schedule.h"
#include "mmgraph/sharding.h"
#include "mmrt/cuda_context.h"
#include "mmrt/launcher.h"
#include "mmrt/runtime.h"

namespace py = pybind11;
using namespace mmg;

namespace mmg { void ReleaseShardingTables(const CompileState& s); const ShardedShape* InputShardingOf(const CompileState& s, int group, int value); }

namespace {

py::dict ShardedShapeToDict(const ShardedShape& s) {
  py::dict d;
  d["dtype"] = DTypeName(s.dtype);
  d["sizes"] = s.sizes;
  d["dim_axes"] = s.dim_axes;
  d["mesh_dims"] = s.mesh_dims;
  d["device_start"] = s.devices.start;
  d["num_devices"] = s.devices.n;
  d["shard_size"] = s.ShardSize();
  d["key"] = s.Key();
  return d;
}
ShardedShape ShardedShapeFromDict(const py::dict& d) {
  ShardedShape s;
  s.dtype = DTypeFromName(d["dtype"].cast<std::string>());
  s.sizes = d["sizes"].cast<std::vector<int64_t>>();
  s.dim_axes = d["dim_axes"].cast<std::vector<std::vector<int>>>();
  s.mesh_dims = d["mesh_dims"].cast<std::vector<int>>();
  s.devices = DeviceRange{d["device_start"].cast<int>(), d["num_devices"].cast<int>()};
  std::string why;
  if (!s.Valid(&why)) throw std::runtime_error("invalid sharded shape: " + why);
  return s;
}

py::dict PlanToDict(const Plan& plan) {
  py::dict out;
  py::list templates;
  for (auto& t : plan.templates) {
    py::dict d;
    d["id"] = t.id;
    d["name"] = t.name;
    d["original_color"] = t.original_color;
    d["device_start"] = t.devices.start;
    d["num_devices"] = t.devices.n;
    d["mesh_dims"] = t.mesh_dims;
    d["mesh_axes"] = t.mesh_axes;
    d["nodes"] = t.nodes;
    d["inputs"] = t.inputs;
    d["outputs"] = t.outputs;
    d["in_loop"] = t.in_loop;
    d["backprop"] = t.backprop;
    d["noncritical"] = t.noncritical;
    d["has_collectives"] = t.has_collectives;
    d["flops"] = t.flops;
    templates.append(d);
  }
  out["templates"] = templates;
  py::list stores;
  for (auto& s : plan.stores) {
    py::dict d;
    d["id"] = s.id;
    d["kind"] = s.kind == Store::PARAM ? "PARAM" : (s.kind == Store::ROOT ? "ROOT" : "TEMP");
    d["index"] = s.index;
    d["name"] = s.name;
    d["scalar"] = s.scalar;
    d["shape"] = ShardedShapeToDict(s.shape);
    d["value"] = s.value;
    d["iteration"] = s.iteration;
    d["alias_of"] = s.alias_of;
    stores.append(d);
  }
  out["stores"] = stores;
  py::list ops;
  for (auto& op : plan.ops) {
    py::dict d;
    static const char* kinds[] = {"task", "reshard", "create_store", "free_store"};
    d["kind"] = kinds[op.kind];
    d["template"] = op.task_template;
    d["name"] = op.name;
    d["device_start"] = op.devices.start;
    d["num_devices"] = op.devices.n;
    d["inputs"] = op.inputs;
    d["outputs"] = op.outputs;
    d["accumulate"] = op.accumulate;
    d["scalars"] = op.scalars;
    d["loop"] = op.loop;
    d["iteration"] = op.iteration;
    d["priority"] = op.priority;
    d["strict_ordering"] = op.strict_ordering;
    d["src_store"] = op.src_store;
    d["dst_store"] = op.dst_store;
    d["store"] = op.store;
    ops.append(d);
  }
  out["ops"] = ops;
  out["param_stores"] = plan.param_stores;
  out["root_stores"] = plan.root_stores;
  out["unused_params"] = plan.unused_params;
  out["aliases"] = plan.aliases;
  out["temp_bytes_per_device_max"] = plan.temp_bytes_per_device_max;
  out["stats"] = plan.stats;
  out["hash"] = plan.Hash();
  return out;
}

// Keeps Graph + Partition + CompileState alive together so that single passes can be
// run and inspected from Python (pass-level golden tests).
struct Compiler {
  std::shared_ptr<Graph> graph;
  std::shared_ptr<Partition> partition;
  CompileState state;
  Compiler(std::shared_ptr<Graph> g, std::shared_ptr<Partition> p, const PartitionConfig& cfg)
      : graph(std::move(g)), partition(std::move(p)) {
    state.graph = graph.get();
    state.partition = partition.get();
    state.config = cfg;
    graph->Toposort();
  }
  ~Compiler() { ReleaseShardingTables(state); }
  bool Run(const std::string& name) {
    CompileState& s = state;
    bool changed;
    if (name == "constant_output_copy") changed = ConstantOutputCopy(s);
    else if (name == "repeated_output_copy") changed = RepeatedOutputCopy(s);
    else if (name == "microbatch_loop_canonicalizer") changed = MicrobatchLoopCanonicalizer(s);
    else if (name == "simple_loop_increment_coloring") changed = SimpleLoopIncrementColoring(s);
    else if (name == "coloring") changed = Coloring(s);
    else if (name == "unused_loop_output_remover") changed = UnusedLoopOutputRemover(s);
    else if (name == "logical_sharding_propagation") changed = LogicalShardingPropagation(s);
    else if (name == "hoist_loop_convert") changed = HoistLoopConvert(s);
    else if (name == "parameter_replication") changed = ParameterReplication(s);
    else if (name == "replicate_uncolored") changed = ReplicateUncolored(s);
    else if (name == "computation_grouper") changed = ComputationGrouper(s);
    else if (name == "computation_fusion_matching_color") changed = ComputationFusion(s, FusionMode::kMatchingColor);
    else if (name == "computation_fusion_original_color") changed = ComputationFusion(s, FusionMode::kOriginalColor);
    else if (name == "computation_fusion_matching_devices") changed = ComputationFusion(s, FusionMode::kMatchingDevices);
    else if (name == "uniquify_colors") changed = UniquifyColors(s);
    else if (name == "instruction_delay_recolor") changed = InstructionDelayRecolor(s);
    else if (name == "argument_recompute") changed = ArgumentRecompute(s);
    else if (name == "cut_size_minimizer") changed = CutSizeMinimizer(s);
    else if (name == "split_critical_path") changed = SplitCriticalPath(s);
    else if (name == "logical_to_physical_sharding") changed = LogicalToPhysicalSharding(s);
    else if (name == "sharding_propagation_forward_io") changed = ShardingPropagation(s, PropagationMode::kForwardInputOutput);
    else if (name == "sharding_propagation_backward_io") changed = ShardingPropagation(s, PropagationMode::kBackwardInputOutput);
    else if (name == "sharding_propagation_forward_full") changed = ShardingPropagation(s, PropagationMode::kForwardFull);
    else if (name == "spmd_lowering") changed = SpmdLowering(s);
    else if (name == "hoist_shard_map_reduce") changed = HoistShardMapReduce(s);
    else if (name == "reduce_scatter_creator") changed = ReduceScatterCreator(s);
    else if (name == "split_update_by_reduction") changed = SplitUpdateByReduction(s);
    else if (name == "unused_param_output_remover") changed = UnusedParamOutputRemover(s);
    else throw std::runtime_error("unknown pass '" + name + "'");
    ValidateCircularDependencies(s, name);
    return changed;
  }
  py::list Groups() const {
    py::list out;
    for (auto& grp : state.groups) {
      py::dict d;
      d["id"] = grp.id;
      d["color"] = grp.color;
      d["region"] = grp.region;
      d["nodes"] = grp.nodes;
      d["noncritical"] = grp.noncritical;
      out.append(d);
    }
    return out;
  }
  py::dict BuildPlanDict() { return PlanToDict(BuildPlan(state)); }
  py::object InputSharding(int group, int value) const {
    const ShardedShape* s = InputShardingOf(state, group, value);
    if (!s) return py::none();
    return ShardedShapeToDict(*s);
  }
};

py::dict NodeToDict(const Graph& g, int id) {
  const Node& n = g.node(id);
  py::dict d;
  d["id"] = n.id;
  d["op"] = n.op;
  d["inputs"] = n.inputs;
  d["outputs"] = n.outputs;
  d["attrs"] = n.attrs;
  d["scope"] = n.scope;
  d["backprop"] = n.backprop;
  d["loop"] = n.loop;
  d["color"] = n.color;
  d["task"] = n.task;
  d["dead"] = n.dead;
  return d;
}
py::dict ValueToDict(const Graph& g, int id) {
  const Value& v = g.value(id);
  py::dict d;
  d["id"] = v.id;
  d["name"] = v.name;
  d["shape"] = v.shape;
  d["dtype"] = DTypeName(v.dtype);
  d["producer"] = v.producer;
  d["out_index"] = v.out_index;
  d["input_index"] = v.input_index;
  d["axes"] = v.axes;
  d["has_axes"] = v.has_axes;
  d["partial"] = v.partial;
  if (v.has_sharding) d["sharding"] = ShardedShapeToDict(v.sharding);
  else d["sharding"] = py::none();
  return d;
}

// Wraps a Python callable so that it is invoked and destroyed with the GIL held and
// Python exceptions surface as C++ exceptions carrying the message.
mmrt::Body WrapBody(py::object fn) {
  if (fn.is_none()) return nullptr;
  auto holder = std::shared_ptr<py::object>(new py::object(std::move(fn)), [](py::object* p) {
    py::gil_scoped_acquire gil;
    delete p;
  });
  return [holder]() {
    py::gil_scoped_acquire gil;
    try {
      (*holder)();
    } catch (py::error_already_set& e) {
      std::string msg = e.what();
      e.restore();
      PyErr_Clear();
      throw std::runtime_error(msg);
    }
  };
}

std::vector<mmrt::TileRef> Tiles(const std::vector<std::pair<int, int>>& v) {
  std::vector<mmrt::TileRef> out;
  for (auto& p : v) out.push_back(mmrt::TileRef{p.first, p.second});
  return out;
}

py::list LogToList(const std::vector<mmrt::TaskRecord>& log) {
  py::list out;
  for (auto& r : log) {
    py::dict d;
    d["id"] = r.id;
    d["name"] = r.name;
    d["device"] = r.device;
    d["kind"] = r.kind;
    d["step"] = r.step;
    d["submit_us"] = r.submit_us;
    d["start_us"] = r.start_us;
    d["end_us"] = r.end_us;
    d["skipped"] = r.skipped;
    d["failed"] = r.failed;
    out.append(d);
  }
  return out;
}

mmrt::ExecuteOptions Options(const std::string& name, bool strict, int priority, int step) {
  mmrt::ExecuteOptions o;
  o.name = name;
  o.strict_ordering = strict;
  o.priority = priority;
  o.step = step;
  return o;
}

}  // namespace

PYBIND11_MODULE(_mm_C, m) {
  m.doc() = "MPMD graph compiler and task-graph runtime (native)";

  // ------------------------------------------------------------------ graph
  py::class_<Graph, std::shared_ptr<Graph>>(m, "Graph")
      .def(py::init<>())
      .def("add_input", [](Graph& g, const std::string& name, std::vector<int64_t> shape, const std::string& dtype) {
        return g.AddInput(name, std::move(shape), DTypeFromName(dtype));
      })
      .def("add_node",
           [](Graph& g, const std::string& op, const std::vector<int>& inputs,
              const std::vector<std::vector<int64_t>>& out_shapes, const std::vector<std::string>& out_dtypes,
              const std::map<std::string, std::string>& attrs, const std::string& scope, bool backprop, int loop,
              const std::string& explicit_task, const std::string& color) {
             std::vector<DType> dts;
             for (auto& d : out_dtypes) dts.push_back(DTypeFromName(d));
             const int id = g.AddNode(op, inputs, out_shapes, dts, attrs);
             Node& n = g.node(id);
             n.scope = scope;
             n.backprop = backprop;
             n.loop = loop;
             n.explicit_task = explicit_task;
             n.color = color;
             return std::make_pair(id, n.outputs);
           },
           py::arg("op"), py::arg("inputs"), py::arg("out_shapes"), py::arg("out_dtypes"),
           py::arg("attrs") = std::map<std::string, std::string>{}, py::arg("scope") = "", py::arg("backprop") = false,
           py::arg("loop") = -1, py::arg("explicit_task") = "", py::arg("color") = "")
      .def("set_outputs", &Graph::SetOutputs)
      .def("add_loop", [](Graph& g, const std::string& json) { g.loops.push_back(LoopConfig::FromJson(Json::parse(json))); })
      .def("set_donated_inputs", [](Graph& g, std::vector<int> idx) { g.donated_inputs = std::move(idx); })
      .def("set_value_axes", [](Graph& g, int value, std::vector<std::vector<std::string>> axes, bool logical) {
        Value& v = g.value(value);
        v.axes = std::move(axes);
        v.has_axes = true;
        v.axes_logical = logical;
      })
      .def("node", [](const Graph& g, int id) { return NodeToDict(g, id); })
      .def("value", [](const Graph& g, int id) { return ValueToDict(g, id); })
      .def_property_readonly("num_nodes", [](const Graph& g) { return g.nodes.size(); })
      .def_property_readonly("num_values", [](const Graph& g) { return g.values.size(); })
      .def_property_readonly("order", [](const Graph& g) { return g.order; })
      .def_property_readonly("inputs", [](const Graph& g) { return g.inputs; })
      .def_property_readonly("outputs", [](const Graph& g) { return g.outputs; })
      .def("toposort", &Graph::Toposort)
      .def("dce", &Graph::DeadCodeElimination)
      .def("dump", &Graph::Dump);

  // -------------------------------------------------------------- partition
  py::class_<Partition, std::shared_ptr<Partition>>(m, "Partition")
      .def(py::init([](int start, int n) { return std::make_shared<Partition>(DeviceRange{start, n}); }))
      .def("register_task_factory",
           [](Partition& p, const std::string& regex, py::function cb) {
             p.RegisterFactory(regex, [cb](const std::string& matched, bool backprop) {
               py::gil_scoped_acquire gil;
               return cb(matched, backprop).cast<std::string>();
             });
           })
      .def("clear_tasks", &Partition::ClearFactories)
      .def("add_task", [](Partition& p, const std::string& json, bool backprop) {
        return p.Add(TaskOptions::FromJson(Json::parse(json)), backprop).name;
      })
      .def("recolor", &Partition::Recolor)
      .def("compute_scope_color", &Partition::ComputeScopeColor)
      .def("has", &Partition::Has)
      .def("color", [](const Partition& p, const std::string& name) {
        const ColorConfig& c = p.Get(name);
        py::dict d;
        d["name"] = c.name;
        d["device_start"] = c.devices.start;
        d["num_devices"] = c.devices.n;
        d["backprop"] = c.backprop;
        d["noncritical"] = c.noncritical;
        d["original"] = c.original;
        d["dims"] = c.options.dims;
        d["device_axes"] = c.options.device_axes;
        d["logical_axes"] = c.options.logical_axes;
        return d;
      })
      .def("colors", [](const Partition& p) {
        std::vector<std::string> names;
        for (auto& kv : p.colors()) names.push_back(kv.first);
        return names;
      });

  py::class_<PartitionConfig>(m, "PartitionConfig")
      .def(py::init<>())
      .def_static("from_env", &PartitionConfig::FromEnv)
      .def_readwrite("use_task_fusion", &PartitionConfig::use_task_fusion)
      .def_readwrite("replicated_parameter_num_elements_cutoff", &PartitionConfig::replicated_parameter_num_elements_cutoff)
      .def_readwrite("run_simplification_passes", &PartitionConfig::run_simplification_passes)
      .def_readwrite("only_fuse_loop_tasks", &PartitionConfig::only_fuse_loop_tasks)
      .def_readwrite("hoist_loop_convert", &PartitionConfig::hoist_loop_convert)
      .def_readwrite("remove_hoisted_reduces", &PartitionConfig::remove_hoisted_reduces)
      .def_readwrite("recompute_from_arguments_if_cost_less_than", &PartitionConfig::recompute_from_arguments_if_cost_less_than)
      .def_readwrite("argument_recompute", &PartitionConfig::argument_recompute)
      .def_readwrite("minimize_cut_size", &PartitionConfig::minimize_cut_size)
      .def_readwrite("zero_arguments", &PartitionConfig::zero_arguments)
      .def_readwrite("dynamic_schedule_post_loop_tasks", &PartitionConfig::dynamic_schedule_post_loop_tasks)
      .def_readwrite("loop_increment_color", &PartitionConfig::loop_increment_color)
      .def_readwrite("enable_recomputation", &PartitionConfig::enable_recomputation)
      .def_readwrite("color_propagation_priority", &PartitionConfig::color_propagation_priority)
      .def_readwrite("dump_dir", &PartitionConfig::dump_dir)
      .def_readwrite("dump_all_passes", &PartitionConfig::dump_all_passes);

  m.def("mpmd_partition",
        [](std::shared_ptr<Graph> g, std::shared_ptr<Partition> p, const PartitionConfig& cfg) {
          std::vector<std::string> log;
          Plan plan = MpmdPartition(*g, *p, cfg, &log);
          py::dict d = PlanToDict(plan);
          d["log"] = log;
          d["dump"] = plan.Dump(*g);
          return d;
        },
        "Runs the whole MPMD pipeline on a captured step and returns the execution plan.");

  m.def("save_program",
        [](std::shared_ptr<Graph> g, std::shared_ptr<Partition> p, const PartitionConfig& cfg, const std::string& path) {
          SaveProgram(path, *g, *p, cfg);
        },
        "Writes a captured, not yet partitioned step (graph, resolved task table, loop settings, partition "
        "options) to one JSON file.");
  m.def("load_program",
        [](const std::string& path) {
          StoredProgram sp = LoadProgram(path);
          return py::make_tuple(sp.graph, sp.partition, sp.config);
        },
        "Reads a stored program back: (Graph, Partition, PartitionConfig).");
  m.def("compile_program_file",
        [](const std::string& path, int64_t device_memory_bytes, bool want_plan) {
          Plan plan;
          std::vector<std::string> log;
          OfflineResult r;
          {
            py::gil_scoped_release rel;
            r = CompileProgramFile(path, device_memory_bytes, &plan, &log);
          }
          py::dict d;
          d["status"] = r.status;
          d["message"] = r.message;
          d["hazards"] = r.hazards;
          d["plan_hash"] = r.plan_hash;
          d["operation_hash"] = r.operation_hash;
          d["templates"] = r.templates;
          d["template_names"] = r.template_names;
          d["stores"] = r.stores;
          d["tasks"] = r.tasks;
          d["reshards"] = r.reshards;
          d["reshard_bytes"] = r.reshard_bytes;
          d["temp_bytes_per_device_max"] = r.temp_bytes_per_device_max;
          d["device_high_water_max"] = r.device_high_water_max;
          d["device_high_water"] = r.device_high_water;
          d["fits"] = r.fits;
          d["stats"] = r.stats;
          d["log"] = log;
          if (want_plan) d["plan"] = PlanToDict(plan);
          return d;
        },
        py::arg("path"), py::arg("device_memory_bytes") = 0, py::arg("want_plan") = false,
        "Offline compile: loads a stored program, runs the MPMD pipeline and replays the plan on the mock "
        "runtime against a made-up device-memory size. No tensor is allocated and no device is needed.");

  py::class_<Compiler>(m, "Compiler")
      .def(py::init<std::shared_ptr<Graph>, std::shared_ptr<Partition>, const PartitionConfig&>())
      .def("run", &Compiler::Run)
      .def("groups", &Compiler::Groups)
      .def("build_plan", &Compiler::BuildPlanDict)
      .def("input_sharding", &Compiler::InputSharding)
      .def("log", [](const Compiler& c) { return c.state.log; });

  // ---------------------------------------------------------------- sharding
  m.def("logical_to_physical",
        [](const std::string& dtype, std::vector<int64_t> sizes, std::vector<std::vector<std::string>> axes,
           std::vector<std::pair<std::string, std::string>> logical_axes, std::vector<std::string> mesh_axis_names,
           std::vector<int> mesh_dims, int device_start) {
          int n = 1;
          for (int d : mesh_dims) n *= d;
          return ShardedShapeToDict(LogicalToPhysical(DTypeFromName(dtype), sizes, axes, logical_axes, mesh_axis_names,
                                                      mesh_dims, DeviceRange{device_start, n}));
        });
  m.def("resize_sharding", [](const py::dict& s, int start, int n) {
    bool ok = true;
    ShardedShape r = ResizeSharding(ShardedShapeFromDict(s), DeviceRange{start, n}, &ok);
    return std::make_pair(ShardedShapeToDict(r), ok);
  });
  m.def("replicate_dims", [](const py::dict& s, std::vector<int> dims) {
    return ShardedShapeToDict(ReplicateDims(ShardedShapeFromDict(s), dims));
  });
  m.def("mesh_equivalent", [](const py::dict& a, const py::dict& b) {
    return MeshEquivalent(ShardedShapeFromDict(a), ShardedShapeFromDict(b));
  });
  m.def("needs_reshard", [](const py::dict& a, const py::dict& b) {
    return NeedsReshard(ShardedShapeFromDict(a), ShardedShapeFromDict(b));
  });
  m.def("tile_box", [](const py::dict& s, int ordinal) {
    Box b = ShardedShapeFromDict(s).TileBox(ordinal);
    return std::make_pair(b.lo, b.hi);
  });
  m.def("sharded_shape", [](const std::string& dtype, std::vector<int64_t> sizes, std::vector<std::vector<int>> dim_axes,
                            std::vector<int> mesh_dims, int start) {
    ShardedShape s;
    s.dtype = DTypeFromName(dtype);
    s.sizes = std::move(sizes);
    s.dim_axes = std::move(dim_axes);
    s.mesh_dims = std::move(mesh_dims);
    int n = 1;
    for (int d : s.mesh_dims) n *= d;
    s.devices = DeviceRange{start, n};
    std::string why;
    if (!s.Valid(&why)) throw std::runtime_error("invalid sharded shape: " + why);
    return ShardedShapeToDict(s);
  });
  m.def("sharded_shape_to_json", [](const py::dict& s) { return ShardedShapeFromDict(s).ToJson().dump(); });
  m.def("sharded_shape_from_json", [](const std::string& j) { return ShardedShapeToDict(ShardedShape::FromJson(Json::parse(j))); });
  m.def("plan_reshard", [](const py::dict& src, const py::dict& dst) {
    ReshardPlan plan = PlanReshard(ShardedShapeFromDict(src), ShardedShapeFromDict(dst));
    py::list chunks;
    for (auto& c : plan.chunks) {
      py::dict d;
      d["src_device"] = c.src_device;
      d["dst_device"] = c.dst_device;
      d["lo"] = c.box.lo;
      d["hi"] = c.box.hi;
      d["src_offset"] = c.src_offset;
      d["dst_offset"] = c.dst_offset;
      chunks.append(d);
    }
    py::dict out;
    out["chunks"] = chunks;
    out["bytes_over_links"] = plan.BytesOverLinks();
    out["bytes_total"] = plan.BytesTotal();
    return out;
  });

  // --------------------------------------------------------------- schedules
  m.def("schedule_loops",
        [](const std::string& cfg_json, const std::vector<std::vector<py::dict>>& tasks) {
          LoopConfig cfg = LoopConfig::FromJson(Json::parse(cfg_json));
          std::vector<std::vector<SchedTask>> rows;
          for (size_t it = 0; it < tasks.size(); ++it) {
            rows.emplace_back();
            for (size_t st = 0; st < tasks[it].size(); ++st) {
              const py::dict& d = tasks[it][st];
              SchedTask t;
              t.iteration = static_cast<int>(it);
              t.stage = static_cast<int>(st);
              t.color = d["color"].cast<std::string>();
              t.devices = DeviceRange{d["device_start"].cast<int>(), d["num_devices"].cast<int>()};
              if (d.contains("noncritical")) t.noncritical = d["noncritical"].cast<bool>();
              if (d.contains("on_full_mesh")) t.on_full_mesh = d["on_full_mesh"].cast<bool>();
              if (d.contains("prefetch")) t.prefetch = d["prefetch"].cast<bool>();
              if (d.contains("consumes_stage")) t.consumes_stage = d["consumes_stage"].cast<int>();
              rows.back().push_back(t);
            }
          }
          ScheduleResult r = ScheduleLoops(cfg, rows);
          py::dict out;
          out["orders"] = r.orders;
          out["simulated_makespan"] = r.simulated_makespan;
          return out;
        });
  m.def("enforce_bijective_tasks", &EnforceBijectiveTasks);
  m.def("get_env_bool", &GetEnvBool);

  // ----------------------------------------------------------------- runtime
  py::enum_<mmrt::Status>(m, "Status")
      .value("OK", mmrt::Status::kOk)
      .value("TASK_FAILED", mmrt::Status::kTaskFailed)
      .value("INJECTED_FAULT", mmrt::Status::kInjectedFault)
      .value("PROTOCOL_VIOLATION", mmrt::Status::kProtocolViolation)
      .value("SHUTDOWN", mmrt::Status::kShutdown);

  py::class_<mmrt::ThreadedContext>(m, "ThreadedContext")
      .def(py::init<std::vector<int>, bool, bool>(), py::arg("local_devices"), py::arg("inline_execution") = false,
           py::arg("record_submissions") = false)
      .def("create_execute_task",
           [](mmrt::ThreadedContext& c, int device, const std::vector<std::pair<int, int>>& reads,
              const std::vector<std::pair<int, int>>& writes, py::object body, const std::string& name, bool strict,
              int priority, int step) {
             mmrt::Body b = WrapBody(std::move(body));
             py::gil_scoped_release rel;
             return c.CreateExecuteTask(device, Tiles(reads), Tiles(writes), std::move(b), Options(name, strict, priority, step));
           },
           py::arg("device"), py::arg("reads"), py::arg("writes"), py::arg("body"), py::arg("name") = "",
           py::arg("strict_ordering") = false, py::arg("priority") = 0, py::arg("step") = 0)
      .def("reshard",
           [](mmrt::ThreadedContext& c, int device, const std::vector<std::pair<int, int>>& reads,
              const std::vector<std::pair<int, int>>& writes, py::object body, const std::string& name, int step) {
             mmrt::Body b = WrapBody(std::move(body));
             py::gil_scoped_release rel;
             return c.Reshard(device, Tiles(reads), Tiles(writes), std::move(b), Options(name, false, 0, step));
           },
           py::arg("device"), py::arg("reads"), py::arg("writes"), py::arg("body"), py::arg("name") = "reshard",
           py::arg("step") = 0)
      .def("create_store", &mmrt::ThreadedContext::CreateStore)
      .def("free_store", &mmrt::ThreadedContext::FreeStore)
      .def("open_window", &mmrt::ThreadedContext::OpenWindow, py::call_guard<py::gil_scoped_release>())
      .def("close_window", &mmrt::ThreadedContext::CloseWindow, py::call_guard<py::gil_scoped_release>())
      .def("run_after_all_tasks", [](mmrt::ThreadedContext& c, py::object body) {
        mmrt::Body b = WrapBody(std::move(body));
        py::gil_scoped_release rel;
        c.RunAfterAllTasks(std::move(b));
      })
      .def("start_timer", &mmrt::ThreadedContext::StartTimer, py::call_guard<py::gil_scoped_release>())
      .def("stop_timer", &mmrt::ThreadedContext::StopTimer, py::call_guard<py::gil_scoped_release>())
      .def("mark_profile", &mmrt::ThreadedContext::MarkProfile)
      .def("wait_all", [](mmrt::ThreadedContext& c) {
        std::string msg;
        mmrt::Status st;
        {
          py::gil_scoped_release rel;
          st = c.WaitAll(&msg);
        }
        return std::make_pair(st, msg);
      })
      .def("wait_task", [](mmrt::ThreadedContext& c, uint64_t id) {
        std::string msg;
        mmrt::Status st;
        {
          py::gil_scoped_release rel;
          st = c.WaitTask(id, &msg);
        }
        return std::make_pair(st, msg);
      })
      .def("reset_error", &mmrt::ThreadedContext::ResetError)
      .def("shutdown", &mmrt::ThreadedContext::Shutdown, py::call_guard<py::gil_scoped_release>())
      .def("event_log", [](const mmrt::ThreadedContext& c) { return LogToList(c.EventLog()); })
      .def("clear_event_log", &mmrt::ThreadedContext::ClearEventLog)
      .def("timer_results_ms", &mmrt::ThreadedContext::TimerResultsMs)
      .def("inject_fault",
           [](mmrt::ThreadedContext& c, const std::string& kind, const std::string& name, int device, int count, int delay_ms) {
             mmrt::FaultSpec f;
             f.kind = kind == "drop" ? mmrt::FaultSpec::kDrop : (kind == "delay" ? mmrt::FaultSpec::kDelay : mmrt::FaultSpec::kThrow);
             f.name_substring = name;
             f.device = device;
             f.remaining = count;
             f.delay_ms = delay_ms;
             c.InjectFault(f);
           },
           py::arg("kind"), py::arg("name"), py::arg("device") = -1, py::arg("count") = 1, py::arg("delay_ms") = 0)
      .def("hazard_report", [](const mmrt::ThreadedContext& c) { return mmrt::CheckHazards(c.Submissions()); })
      .def("pending_report", &mmrt::ThreadedContext::PendingReport)
      .def_property_readonly("device_bytes_high_water", &mmrt::ThreadedContext::device_bytes_high_water);

  // CUDA streams, events and the scratch tile behind the same submission interface. With
  // `fake=True` every CUDA call goes to a recording stand-in (no GPU needed): `fake_trace()`
  // returns what was called.
  struct PyCudaContext {
    std::unique_ptr<mmrt::FakeGpuApi> fake;
    std::unique_ptr<mmrt::CudaContext> ctx;
  };
  py::class_<PyCudaContext>(m, "CudaContext")
      .def(py::init([](std::vector<int> local_devices, std::vector<int> ordinals, std::vector<uintptr_t> compute_streams,
                       bool fake, bool record_submissions) {
             auto p = std::make_unique<PyCudaContext>();
             if (fake) p->fake = std::make_unique<mmrt::FakeGpuApi>();
             mmrt::GpuApi* api = fake ? static_cast<mmrt::GpuApi*>(p->fake.get()) : mmrt::CudaRuntimeApi();
             p->ctx = std::make_unique<mmrt::CudaContext>(std::move(local_devices), std::move(ordinals),
                                                          std::move(compute_streams), api, record_submissions);
             return p;
           }),
           py::arg("local_devices"), py::arg("ordinals"), py::arg("compute_streams"), py::arg("fake") = false,
           py::arg("record_submissions") = false)
      .def("create_execute_task",
           [](PyCudaContext& c, int device, const std::vector<std::pair<int, int>>& reads,
              const std::vector<std::pair<int, int>>& writes, py::object body, const std::string& name, bool strict,
              int priority, int step, int stream) {
             mmrt::Body b = WrapBody(std::move(body));
             mmrt::ExecuteOptions o = Options(name, strict, priority, step);
             o.stream = stream;
             py::gil_scoped_release rel;
             return c.ctx->CreateExecuteTask(device, Tiles(reads), Tiles(writes), std::move(b), o);
           },
           py::arg("device"), py::arg("reads"), py::arg("writes"), py::arg("body"), py::arg("name") = "",
           py::arg("strict_ordering") = false, py::arg("priority") = 0, py::arg("step") = 0, py::arg("stream") = 0)
      .def("reshard",
           [](PyCudaContext& c, int device, const std::vector<std::pair<int, int>>& reads,
              const std::vector<std::pair<int, int>>& writes, py::object body, const std::string& name, int step,
              int stream) {
             mmrt::Body b = WrapBody(std::move(body));
             mmrt::ExecuteOptions o = Options(name, false, 0, step);
             o.stream = stream;
             py::gil_scoped_release rel;
             return c.ctx->Reshard(device, Tiles(reads), Tiles(writes), std::move(b), o);
           },
           py::arg("device"), py::arg("reads"), py::arg("writes"), py::arg("body"), py::arg("name") = "reshard",
           py::arg("step") = 0, py::arg("stream") = 1)
      .def("create_store", [](PyCudaContext& c, int b, int d, int64_t bytes, bool host) { c.ctx->CreateStore(b, d, bytes, host); })
      .def("free_store", [](PyCudaContext& c, int b, int d) { c.ctx->FreeStore(b, d); })
      .def("open_window", [](PyCudaContext& c) { py::gil_scoped_release rel; c.ctx->OpenWindow(); })
      .def("close_window", [](PyCudaContext& c) { c.ctx->CloseWindow(); })
      .def("run_after_all_tasks", [](PyCudaContext& c, py::object body) {
        mmrt::Body b = WrapBody(std::move(body));
        py::gil_scoped_release rel;
        c.ctx->RunAfterAllTasks(std::move(b));
      })
      .def("start_timer", [](PyCudaContext& c, const std::string& n) { c.ctx->StartTimer(n); })
      .def("stop_timer", [](PyCudaContext& c, const std::string& n) { c.ctx->StopTimer(n); })
      .def("mark_profile", [](PyCudaContext& c, const std::string& n) { c.ctx->MarkProfile(n); })
      .def("wait_all", [](PyCudaContext& c) {
        std::string msg;
        mmrt::Status st = c.ctx->WaitAll(&msg);
        return std::make_pair(st, msg);
      })
      .def("reset_error", [](PyCudaContext& c) { c.ctx->ResetError(); })
      .def("shutdown", [](PyCudaContext& c) { py::gil_scoped_release rel; c.ctx->Shutdown(); })
      .def("synchronize", [](PyCudaContext& c) { py::gil_scoped_release rel; return c.ctx->Synchronize(); })
      .def("event_log", [](const PyCudaContext& c) { return LogToList(c.ctx->EventLog()); })
      .def("clear_event_log", [](PyCudaContext& c) { c.ctx->ClearEventLog(); })
      .def("timer_results_ms", [](PyCudaContext& c) { return c.ctx->TimerResultsMs(); })
      .def("stream_handle", [](const PyCudaContext& c, int device, int kind) { return c.ctx->StreamHandle(device, kind); })
      .def("set_task_ranges", [](PyCudaContext& c, bool on) { c.ctx->set_task_ranges(on); })
      .def("reserve_scratch", [](PyCudaContext& c, int device, int64_t bytes) { return c.ctx->ReserveScratch(device, bytes); })
      .def("scratch_bytes", [](const PyCudaContext& c, int device) { return c.ctx->ScratchBytes(device); })
      .def("edges", [](const PyCudaContext& c) {
        py::list out;
        for (auto& e : c.ctx->Edges()) {
          py::dict d;
          d["from_task"] = e.from_task;
          d["to_task"] = e.to_task;
          d["device"] = e.device;
          d["from_stream"] = e.from_stream;
          d["to_stream"] = e.to_stream;
          d["from_name"] = e.from_name;
          d["to_name"] = e.to_name;
          out.append(d);
        }
        return out;
      })
      .def("inject_fault",
           [](PyCudaContext& c, const std::string& kind, const std::string& name, int device, int count, int delay_ms) {
             mmrt::FaultSpec f;
             f.kind = kind == "drop" ? mmrt::FaultSpec::kDrop : (kind == "delay" ? mmrt::FaultSpec::kDelay : mmrt::FaultSpec::kThrow);
             f.name_substring = name;
             f.device = device;
             f.remaining = count;
             f.delay_ms = delay_ms;
             c.ctx->InjectFault(f);
           },
           py::arg("kind"), py::arg("name"), py::arg("device") = -1, py::arg("count") = 1, py::arg("delay_ms") = 0)
      .def("hazard_report", [](const PyCudaContext& c) { return mmrt::CheckHazards(c.ctx->Submissions()); })
      .def("fake_trace", [](const PyCudaContext& c) { return c.fake ? c.fake->trace : std::vector<std::string>(); })
      .def("fake_stream_priorities", [](const PyCudaContext& c) { return c.fake ? c.fake->stream_priorities : std::vector<int>(); })
      .def_property_readonly("open_windows", [](const PyCudaContext& c) { return c.ctx->open_windows(); })
      .def_property_readonly("host_blocks", [](const PyCudaContext& c) { return c.ctx->host_blocks(); })
      .def_property_readonly("device_bytes_high_water", [](const PyCudaContext& c) { return c.ctx->device_bytes_high_water(); });

  // ------------------------------------------------------------ native task launcher
  py::class_<mmrt::KernelProgram>(m, "KernelProgram")
      .def(py::init<>())
      // args: list of tuples ("p", slot, offset[, scalar, scale]) | ("i", value) | ("f", value) | ("s",)
      .def("add_call",
           [](mmrt::KernelProgram& p, uintptr_t fn, const std::string& name, const py::list& args) {
             std::vector<mmrt::LaunchArg> out;
             for (auto item : args) {
               py::tuple t = item.cast<py::tuple>();
               const std::string kind = t[0].cast<std::string>();
               mmrt::LaunchArg a;
               if (kind == "p") {
                 a.kind = mmrt::LaunchArg::kPtr;
                 a.slot = t[1].cast<int>();
                 a.value = t.size() > 2 ? t[2].cast<int64_t>() : 0;
                 if (t.size() > 4) {
                   a.scalar = t[3].cast<int>();
                   a.scalar_scale = t[4].cast<int64_t>();
                 }
               } else if (kind == "i") {
                 a.kind = mmrt::LaunchArg::kInt;
                 a.value = t[1].cast<int64_t>();
               } else if (kind == "f") {
                 a.kind = mmrt::LaunchArg::kFloat;
                 a.fvalue = t[1].cast<double>();
               } else if (kind == "s") {
                 a.kind = mmrt::LaunchArg::kStream;
               } else {
                 throw std::runtime_error("unknown launch argument kind '" + kind + "'");
               }
               out.push_back(a);
             }
             p.AddCall(fn, name, std::move(out));
           })
      .def("launch",
           [](const mmrt::KernelProgram& p, const std::vector<uintptr_t>& bases, const std::vector<int64_t>& scalars,
              uintptr_t stream) {
             std::string err;
             int rc;
             {
               py::gil_scoped_release rel;
               rc = p.Launch(bases, scalars, stream, &err);
             }
             if (rc != 0) throw std::runtime_error("native task launch failed: " + err);
           })
      .def("__len__", &mmrt::KernelProgram::size)
      .def("describe", &mmrt::KernelProgram::Describe)
      .def_property_readonly("launches", &mmrt::KernelProgram::launches);
  m.def("selftest_kernel_address", [] { return reinterpret_cast<uintptr_t>(&mmrt::mmrt_selftest_axpy); });

  py::class_<mmrt::MockContext>(m, "MockContext")
      .def(py::init<int>())
      .def("create_execute_task",
           [](mmrt::MockContext& c, int device, const std::vector<std::pair<int, int>>& reads,
              const std::vector<std::pair<int, int>>& writes, py::object, const std::string& name, bool strict,
              int priority, int step) {
             return c.CreateExecuteTask(device, Tiles(reads), Tiles(writes), nullptr, Options(name, strict, priority, step));
           },
           py::arg("device"), py::arg("reads"), py::arg("writes"), py::arg("body") = py::none(), py::arg("name") = "",
           py::arg("strict_ordering") = false, py::arg("priority") = 0, py::arg("step") = 0)
      .def("reshard",
           [](mmrt::MockContext& c, int device, const std::vector<std::pair<int, int>>& reads,
              const std::vector<std::pair<int, int>>& writes, py::object, const std::string& name, int step) {
             return c.Reshard(device, Tiles(reads), Tiles(writes), nullptr, Options(name, false, 0, step));
           },
           py::arg("device"), py::arg("reads"), py::arg("writes"), py::arg("body") = py::none(),
           py::arg("name") = "reshard", py::arg("step") = 0)
      .def("create_store", &mmrt::MockContext::CreateStore)
      .def("free_store", &mmrt::MockContext::FreeStore)
      .def("offload_d2h", &mmrt::MockContext::OffloadDtoH)
      .def("offload_h2d", &mmrt::MockContext::OffloadHtoD)
      .def("open_window", &mmrt::MockContext::OpenWindow)
      .def("close_window", &mmrt::MockContext::CloseWindow)
      .def("run_after_all_tasks", [](mmrt::MockContext& c, py::object body) {
        c.RunAfterAllTasks([body]() { if (!body.is_none()) body(); });
      })
      .def("start_timer", &mmrt::MockContext::StartTimer)
      .def("stop_timer", &mmrt::MockContext::StopTimer)
      .def("mark_profile", &mmrt::MockContext::MarkProfile)
      .def("wait_all", [](mmrt::MockContext& c) {
        std::string msg;
        mmrt::Status st = c.WaitAll(&msg);
        return std::make_pair(st, msg);
      })
      .def("reset_error", [](mmrt::MockContext&) {})
      .def("shutdown", &mmrt::MockContext::Shutdown)
      .def("event_log", [](const mmrt::MockContext& c) { return LogToList(c.EventLog()); })
      .def("clear_event_log", &mmrt::MockContext::ClearEventLog)
      .def("hazard_report", &mmrt::MockContext::hazard_report)
      .def_property_readonly("operation_hash", &mmrt::MockContext::operation_hash)
      .def_property_readonly("max_device_high_water", &mmrt::MockContext::max_device_high_water)
      .def_property_readonly("host_high_water", &mmrt::MockContext::host_high_water)
      .def_property_readonly("num_tasks", &mmrt::MockContext::num_tasks)
      .def_property_readonly("num_reshards", &mmrt::MockContext::num_reshards)
      .def_property_readonly("violation", &mmrt::MockContext::violation)
      .def("device_high_water", &mmrt::MockContext::device_high_water);
}
