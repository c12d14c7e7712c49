// Stored programs: a captured step (graph, task table, loop settings, partition options) written
// to one JSON file, and an offline compile entry point that reads such a file, runs the whole
// MPMD pipeline, and replays the resulting plan on the mock runtime with a made-up device-memory
// size - no tensors, no devices. This is how real-model graphs become regression fixtures
// (the reference keeps 50 HLO text files under src/pjrt_client/testdata/ and compiles them with
// `CompileHloModuleFromFile`, src/pjrt_client/mm_pjrt_client.cc:702-771, which takes the path, the
// number of devices and a fake memory size).
#include "program_file.h"

#include <fstream>
#include <set>
#include <sstream>

#include "../mmrt/runtime.h"

namespace mmg {

namespace {

Json IntArray(const std::vector<int>& v) {
  Json a = Json::array();
  for (int x : v) a.push(Json::number(x));
  return a;
}
Json Int64Array(const std::vector<int64_t>& v) {
  Json a = Json::array();
  for (int64_t x : v) a.push(Json::number(static_cast<double>(x)));
  return a;
}
std::vector<int> ToInts(const Json& j) {
  std::vector<int> out;
  for (auto v : j.as_int_vector()) out.push_back(static_cast<int>(v));
  return out;
}

Json LoopToJson(const LoopConfig& c) {
  Json j = Json::object();
  j.set("id", Json::number(c.id));
  j.set("num_microbatches", Json::number(c.num_microbatches));
  j.set("slice_dim", Json::number(c.slice_dim));
  j.set("size", Json::number(static_cast<double>(c.size)));
  j.set("batch_dim", Json::number(c.batch_dim));
  j.set("interleave", Json::number(c.interleave));
  j.set("unrolling", Json::number(c.unrolling));
  j.set("num_stages", Json::number(c.num_stages));
  j.set("schedule", Json::string(c.schedule));
  j.set("accumulate_dtype", Json::string(c.accumulate_dtype));
  Json rows = Json::array();
  for (auto& row : c.custom_schedule) {
    Json r = Json::array();
    for (auto& e : row) {
      Json p = Json::array();
      p.push(Json::number(e.first));
      p.push(Json::string(e.second));
      r.push(p);
    }
    rows.push(r);
  }
  j.set("custom_schedule", rows);
  return j;
}

Json ConfigToJson(const PartitionConfig& c) {
  Json j = Json::object();
  j.set("use_task_fusion", Json::boolean(c.use_task_fusion));
  j.set("replicated_parameter_num_elements_cutoff",
        Json::number(static_cast<double>(c.replicated_parameter_num_elements_cutoff)));
  j.set("run_simplification_passes", Json::boolean(c.run_simplification_passes));
  j.set("only_fuse_loop_tasks", Json::boolean(c.only_fuse_loop_tasks));
  j.set("hoist_loop_convert", Json::boolean(c.hoist_loop_convert));
  j.set("remove_hoisted_reduces", Json::boolean(c.remove_hoisted_reduces));
  j.set("recompute_from_arguments_if_cost_less_than",
        Json::number(static_cast<double>(c.recompute_from_arguments_if_cost_less_than)));
  j.set("argument_recompute", Json::boolean(c.argument_recompute));
  j.set("minimize_cut_size", Json::boolean(c.minimize_cut_size));
  j.set("loop_increment_color", Json::boolean(c.loop_increment_color));
  j.set("enable_recomputation", Json::boolean(c.enable_recomputation));
  j.set("zero_arguments", Json::boolean(c.zero_arguments));
  j.set("dynamic_schedule_post_loop_tasks", Json::boolean(c.dynamic_schedule_post_loop_tasks));
  j.set("color_propagation_priority", Json::string(c.color_propagation_priority));
  return j;
}

PartitionConfig ConfigFromJson(const Json& j) {
  PartitionConfig c;
  auto flag = [&](const char* k, bool* dst) { if (j.has(k)) *dst = j.at(k).as_bool(); };
  flag("use_task_fusion", &c.use_task_fusion);
  flag("run_simplification_passes", &c.run_simplification_passes);
  flag("only_fuse_loop_tasks", &c.only_fuse_loop_tasks);
  flag("hoist_loop_convert", &c.hoist_loop_convert);
  flag("remove_hoisted_reduces", &c.remove_hoisted_reduces);
  flag("argument_recompute", &c.argument_recompute);
  flag("minimize_cut_size", &c.minimize_cut_size);
  flag("loop_increment_color", &c.loop_increment_color);
  flag("enable_recomputation", &c.enable_recomputation);
  flag("zero_arguments", &c.zero_arguments);
  flag("dynamic_schedule_post_loop_tasks", &c.dynamic_schedule_post_loop_tasks);
  if (j.has("replicated_parameter_num_elements_cutoff"))
    c.replicated_parameter_num_elements_cutoff = j.at("replicated_parameter_num_elements_cutoff").as_int();
  if (j.has("recompute_from_arguments_if_cost_less_than"))
    c.recompute_from_arguments_if_cost_less_than = j.at("recompute_from_arguments_if_cost_less_than").as_int();
  if (j.has("color_propagation_priority")) c.color_propagation_priority = j.at("color_propagation_priority").str;
  return c;
}

}  // namespace

// ------------------------------------------------------------------------------ graph
Json GraphToJson(const Graph& g) {
  Json j = Json::object();
  Json values = Json::array();
  for (const Value& v : g.values) {
    Json e = Json::object();
    e.set("name", Json::string(v.name));
    e.set("shape", Int64Array(v.shape));
    e.set("dtype", Json::string(DTypeName(v.dtype)));
    e.set("producer", Json::number(v.producer));
    e.set("out_index", Json::number(v.out_index));
    e.set("input_index", Json::number(v.input_index));
    if (v.has_axes) {
      Json axes = Json::array();
      for (auto& dim : v.axes) {
        Json d = Json::array();
        for (auto& a : dim) d.push(Json::string(a));
        axes.push(d);
      }
      e.set("axes", axes);
      e.set("axes_logical", Json::boolean(v.axes_logical));
    }
    values.push(e);
  }
  j.set("values", values);
  Json nodes = Json::array();
  for (const Node& n : g.nodes) {
    Json e = Json::object();
    e.set("op", Json::string(n.op));
    e.set("inputs", IntArray(n.inputs));
    e.set("outputs", IntArray(n.outputs));
    Json attrs = Json::object();
    for (auto& kv : n.attrs) attrs.set(kv.first, Json::string(kv.second));
    e.set("attrs", attrs);
    e.set("scope", Json::string(n.scope));
    e.set("backprop", Json::boolean(n.backprop));
    e.set("loop", Json::number(n.loop));
    e.set("explicit_task", Json::string(n.explicit_task));
    if (n.dead) e.set("dead", Json::boolean(true));
    nodes.push(e);
  }
  j.set("nodes", nodes);
  j.set("order", IntArray(g.order));
  j.set("inputs", IntArray(g.inputs));
  j.set("outputs", IntArray(g.outputs));
  j.set("donated_inputs", IntArray(g.donated_inputs));
  Json loops = Json::array();
  for (auto& l : g.loops) loops.push(LoopToJson(l));
  j.set("loops", loops);
  return j;
}

Graph GraphFromJson(const Json& j) {
  Graph g;
  for (const Json& e : j.at("values").arr) {
    Value v;
    v.id = static_cast<int>(g.values.size());
    v.name = e.at("name").str;
    v.shape = e.at("shape").as_int_vector();
    v.dtype = DTypeFromName(e.at("dtype").str);
    v.producer = static_cast<int>(e.at("producer").as_int());
    v.out_index = static_cast<int>(e.at("out_index").as_int());
    v.input_index = static_cast<int>(e.at("input_index").as_int());
    if (e.has("axes")) {
      v.has_axes = true;
      for (const Json& dim : e.at("axes").arr) v.axes.push_back(dim.as_string_vector());
      v.axes_logical = e.at("axes_logical").as_bool();
    }
    g.values.push_back(std::move(v));
  }
  for (const Json& e : j.at("nodes").arr) {
    Node n;
    n.id = static_cast<int>(g.nodes.size());
    n.op = e.at("op").str;
    n.inputs = ToInts(e.at("inputs"));
    n.outputs = ToInts(e.at("outputs"));
    for (auto& kv : e.at("attrs").obj) n.attrs[kv.first] = kv.second.str;
    n.scope = e.at("scope").str;
    n.backprop = e.at("backprop").as_bool();
    n.loop = static_cast<int>(e.at("loop").as_int());
    n.explicit_task = e.at("explicit_task").str;
    n.dead = e.has("dead") && e.at("dead").as_bool();
    g.nodes.push_back(std::move(n));
  }
  g.order = ToInts(j.at("order"));
  g.inputs = ToInts(j.at("inputs"));
  g.outputs = ToInts(j.at("outputs"));
  g.donated_inputs = ToInts(j.at("donated_inputs"));
  for (const Json& l : j.at("loops").arr) g.loops.push_back(LoopConfig::FromJson(l));
  ValidateStoredGraph(g);
  g.Toposort();
  return g;
}

// A file is input from outside: every id is checked against the tables it indexes and every
// producer / result link against its mirror image before a pass follows it.
void ValidateStoredGraph(const Graph& g) {
  auto fail = [](const std::string& what) { throw std::runtime_error("stored program: " + what); };
  const int nv = static_cast<int>(g.values.size()), nn = static_cast<int>(g.nodes.size());
  auto check_value = [&](int v) { if (v < 0 || v >= nv) fail("value id out of range"); };
  std::set<int> loop_ids;
  for (const LoopConfig& l : g.loops) {
    if (l.num_microbatches < 1 || l.num_microbatches > 65536) fail("number of microbatches out of range");
    if (l.size < 0 || l.interleave < 1 || l.num_stages < 0 || l.slice_dim < 0 || l.batch_dim < 0)
      fail("loop setting out of range");
    if (!loop_ids.insert(l.id).second) fail("loop id used twice");
  }
  for (const Node& n : g.nodes) {
    for (int v : n.inputs) check_value(v);
    for (size_t i = 0; i < n.outputs.size(); ++i) {
      check_value(n.outputs[i]);
      const Value& v = g.values[n.outputs[i]];
      if (v.producer != n.id || v.out_index != static_cast<int>(i)) fail("result does not name its producer");
    }
    if (n.loop != -1 && !loop_ids.count(n.loop)) fail("operator in an unknown loop");
  }
  for (const Value& v : g.values) {
    if (v.producer < -1 || v.producer >= nn) fail("producer id out of range");
    if (v.producer >= 0) {
      const Node& n = g.nodes[v.producer];
      if (v.out_index < 0 || v.out_index >= static_cast<int>(n.outputs.size()) || n.outputs[v.out_index] != v.id)
        fail("value is not a result of its producer");
    } else if (v.input_index < 0 || v.input_index >= static_cast<int>(g.inputs.size()) ||
               g.inputs[v.input_index] != v.id) {
      fail("value without a producer is not a graph input");
    }
    if (v.shape.size() > 8) fail("rank above 8");
    int64_t elements = 1;
    for (int64_t d : v.shape) {
      if (d < 0 || d > (int64_t{1} << 40)) fail("dimension out of range");
      if (d > 0 && elements > (int64_t{1} << 50) / d) fail("tensor too large");
      elements *= std::max<int64_t>(d, 1);
    }
    if (v.has_axes && v.axes.size() != v.shape.size()) fail("axis annotation does not match the rank");
  }
  std::vector<char> seen(nn, 0);
  for (int id : g.order) {
    if (id < 0 || id >= nn) fail("operator id out of range");
    if (seen[id]++) fail("operator listed twice");
  }
  for (int v : g.inputs) {
    check_value(v);
    if (g.values[v].producer != -1) fail("graph input has a producer");
  }
  for (int v : g.outputs) check_value(v);
  for (int i : g.donated_inputs)
    if (i < 0 || i >= static_cast<int>(g.inputs.size())) fail("donated input index out of range");
}

// ------------------------------------------------------------------------------ program
std::string ProgramToJson(const Graph& g, Partition& part, const PartitionConfig& cfg) {
  Json j = Json::object();
  j.set("format", Json::string("multimesh_jax_b200.program/1"));
  j.set("device_start", Json::number(part.global().start));
  j.set("num_devices", Json::number(part.global().n));
  j.set("graph", GraphToJson(g));
  j.set("config", ConfigToJson(cfg));
  // The task table: regex contexts are callbacks of the capturing process, so what is stored is
  // their result for every name stack that occurs in the graph.
  Json scopes = Json::array();
  std::set<std::pair<std::string, bool>> seen;
  std::set<std::string> used;
  for (const Node& n : g.nodes) {
    if (n.dead || n.scope.empty() || !n.explicit_task.empty()) continue;
    if (!seen.insert({n.scope, n.backprop}).second) continue;
    const std::string color = part.ComputeScopeColor(n.scope, n.backprop);
    if (color.empty()) continue;
    Json e = Json::array();
    e.push(Json::string(n.scope));
    e.push(Json::boolean(n.backprop));
    e.push(Json::string(color));
    scopes.push(e);
    used.insert(color);
  }
  j.set("scopes", scopes);
  Json colors = Json::array();
  for (auto& kv : part.colors()) {
    if (!used.count(kv.first)) continue;
    Json e = Json::object();
    e.set("options", kv.second.options.ToJson());
    e.set("backprop", Json::boolean(kv.second.backprop));
    colors.push(e);
  }
  j.set("colors", colors);
  return j.dump();
}

StoredProgram ProgramFromJson(const std::string& text) {
  const Json j = Json::parse(text);
  if (!j.has("format") || j.at("format").str != "multimesh_jax_b200.program/1")
    throw std::runtime_error("stored program: unknown format");
  StoredProgram p;
  p.graph = std::make_shared<Graph>(GraphFromJson(j.at("graph")));
  const int64_t dev_start = j.at("device_start").as_int(), dev_count = j.at("num_devices").as_int();
  if (dev_start < 0 || dev_count < 1 || dev_start + dev_count > 65536)
    throw std::runtime_error("stored program: device range out of bounds");
  p.partition = std::make_shared<Partition>(
      DeviceRange::Create(static_cast<int>(j.at("device_start").as_int()), static_cast<int>(j.at("num_devices").as_int())));
  p.config = ConfigFromJson(j.at("config"));
  for (const Json& e : j.at("colors").arr)
    p.partition->Add(TaskOptions::FromJson(e.at("options")), e.at("backprop").as_bool());
  for (const Json& e : j.at("scopes").arr)
    p.partition->PinScopeColor(e.arr[0].str, e.arr[1].as_bool(), e.arr[2].str);
  return p;
}

void SaveProgram(const std::string& path, const Graph& g, Partition& part, const PartitionConfig& cfg) {
  std::ofstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot write " + path);
  f << ProgramToJson(g, part, cfg);
}

StoredProgram LoadProgram(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot read " + path);
  std::ostringstream ss;
  ss << f.rdbuf();
  return ProgramFromJson(ss.str());
}

// ------------------------------------------------------------------------------ offline compile
namespace {

int64_t TileBytes(const Store& st) {
  int64_t n = static_cast<int64_t>(DTypeSize(st.shape.dtype));
  for (auto s : st.shape.ShardSize()) n *= s;
  return n;
}

}  // namespace

OfflineResult MockExecutePlan(const Plan& plan, int device_start, int num_devices, int64_t device_memory_bytes, int steps) {
  OfflineResult r;
  // stores that share a scheduling name share a physical buffer
  std::map<std::string, int> buffer_id;
  std::vector<int> buffer_of(plan.stores.size(), -1);
  for (const Store& st : plan.stores) {
    auto it = buffer_id.find(st.name);
    if (it == buffer_id.end()) it = buffer_id.emplace(st.name, static_cast<int>(buffer_id.size())).first;
    buffer_of[st.id] = it->second;
  }
  mmrt::MockContext ctx(device_start + num_devices);
  for (int step = 0; step < steps; ++step) {
    ctx.OpenWindow();
    ctx.StartTimer("step");
    if (step == 0) {
      for (const Store& st : plan.stores)
        for (int d = st.shape.devices.start; d < st.shape.devices.stop(); ++d)
          ctx.CreateStore(buffer_of[st.id], d, TileBytes(st), false);
    }
    for (const PlanOp& op : plan.ops) {
      mmrt::ExecuteOptions eo;
      eo.name = op.name;
      eo.step = step;
      eo.priority = op.priority;
      eo.strict_ordering = op.strict_ordering;
      if (op.kind == PlanOp::TASK) {
        for (int d = op.devices.start; d < op.devices.stop(); ++d) {
          std::vector<mmrt::TileRef> reads, writes;
          for (int s : op.inputs) reads.push_back({buffer_of[s], d});
          for (size_t k = 0; k < op.outputs.size(); ++k) {
            writes.push_back({buffer_of[op.outputs[k]], d});
            if (k < op.accumulate.size() && op.accumulate[k] == 2) reads.push_back({buffer_of[op.outputs[k]], d});
          }
          ctx.CreateExecuteTask(d, reads, writes, nullptr, eo);
          ++r.tasks;
        }
      } else if (op.kind == PlanOp::RESHARD) {
        const Store& src = plan.stores[op.src_store];
        const Store& dst = plan.stores[op.dst_store];
        const ReshardPlan rp = PlanReshard(src.shape, dst.shape);
        eo.kind = 1;
        eo.name = "reshard S" + std::to_string(op.src_store) + "->S" + std::to_string(op.dst_store);
        for (int d = dst.shape.devices.start; d < dst.shape.devices.stop(); ++d) {
          std::set<int> from;
          for (auto& c : rp.chunks) if (c.dst_device == d) from.insert(c.src_device);
          if (from.empty()) continue;
          std::vector<mmrt::TileRef> reads;
          for (int s : from) reads.push_back({buffer_of[op.src_store], s});
          ctx.Reshard(d, reads, {{buffer_of[op.dst_store], d}}, nullptr, eo);
          ++r.reshards;
          r.reshard_bytes += TileBytes(dst);
        }
      }
    }
    ctx.StopTimer("step");
    ctx.CloseWindow();
  }
  std::string msg;
  const mmrt::Status st = ctx.WaitAll(&msg);
  r.status = static_cast<int>(st);
  r.message = msg.empty() ? ctx.violation() : msg;
  r.hazards = ctx.hazard_report();
  r.operation_hash = ctx.operation_hash();
  r.device_high_water_max = ctx.max_device_high_water();
  for (int d = device_start; d < device_start + num_devices; ++d) r.device_high_water.push_back(ctx.device_high_water(d));
  r.fits = device_memory_bytes <= 0 || r.device_high_water_max <= device_memory_bytes;
  return r;
}

OfflineResult CompileProgramFile(const std::string& path, int64_t device_memory_bytes, Plan* plan_out,
                                 std::vector<std::string>* log) {
  StoredProgram p = LoadProgram(path);
  Plan plan = MpmdPartition(*p.graph, *p.partition, p.config, log);
  OfflineResult r = MockExecutePlan(plan, p.partition->global().start, p.partition->global().n, device_memory_bytes, 2);
  r.plan_hash = plan.Hash();
  r.templates = static_cast<int>(plan.templates.size());
  r.stores = static_cast<int>(plan.stores.size());
  r.temp_bytes_per_device_max = plan.temp_bytes_per_device_max;
  r.stats = plan.stats;
  for (auto& t : plan.templates) r.template_names.push_back(t.name);
  if (plan_out) *plan_out = std::move(plan);
  return r;
}

}  // namespace mmg
