#include "graph.h"

#include <algorithm>
#include <cstdlib>
#include <queue>
#include <regex>
#include <sstream>
#include <stdexcept>

namespace mmg {

// ------------------------------------------------------------------ LoopConfig
LoopConfig LoopConfig::FromJson(const Json& j) {
  LoopConfig c;
  if (j.has("id")) c.id = static_cast<int>(j.at("id").as_int());
  if (j.has("num_microbatches")) c.num_microbatches = static_cast<int>(j.at("num_microbatches").as_int());
  if (j.has("slice_dim")) c.slice_dim = static_cast<int>(j.at("slice_dim").as_int());
  if (j.has("size")) c.size = j.at("size").as_int();
  c.batch_dim = j.has("batch_dim") ? static_cast<int>(j.at("batch_dim").as_int()) : c.slice_dim;
  if (j.has("interleave")) c.interleave = static_cast<int>(j.at("interleave").as_int());
  if (j.has("unrolling")) c.unrolling = static_cast<int>(j.at("unrolling").as_int());
  if (j.has("num_stages")) c.num_stages = static_cast<int>(j.at("num_stages").as_int());
  if (j.has("schedule")) c.schedule = j.at("schedule").str;
  if (j.has("accumulate_dtype")) c.accumulate_dtype = j.at("accumulate_dtype").str;
  if (j.has("custom_schedule")) {
    for (auto& row : j.at("custom_schedule").arr) {
      std::vector<std::pair<int, std::string>> r;
      for (auto& e : row.arr) r.emplace_back(static_cast<int>(e.arr[0].as_int()), e.arr[1].str);
      c.custom_schedule.push_back(std::move(r));
    }
  }
  return c;
}

// ----------------------------------------------------------------------- Graph
int Graph::AddInput(const std::string& name, std::vector<int64_t> shape, DType dtype) {
  Value v;
  v.id = static_cast<int>(values.size());
  v.name = name;
  v.shape = std::move(shape);
  v.dtype = dtype;
  v.input_index = static_cast<int>(inputs.size());
  values.push_back(v);
  inputs.push_back(v.id);
  return v.id;
}

int Graph::AddNode(const std::string& op, const std::vector<int>& ins,
                   const std::vector<std::vector<int64_t>>& out_shapes,
                   const std::vector<DType>& out_dtypes, const std::map<std::string, std::string>& attrs) {
  Node n;
  n.id = static_cast<int>(nodes.size());
  n.op = op;
  n.inputs = ins;
  n.attrs = attrs;
  for (size_t i = 0; i < out_shapes.size(); ++i) {
    Value v;
    v.id = static_cast<int>(values.size());
    v.name = op + "." + std::to_string(n.id) + (out_shapes.size() > 1 ? "." + std::to_string(i) : "");
    v.shape = out_shapes[i];
    v.dtype = out_dtypes[i];
    v.producer = n.id;
    v.out_index = static_cast<int>(i);
    values.push_back(v);
    n.outputs.push_back(v.id);
  }
  nodes.push_back(n);
  order.push_back(n.id);
  return n.id;
}

std::vector<std::vector<int>> Graph::ComputeUsers() const {
  std::vector<std::vector<int>> users(values.size());
  for (int id : order) {
    const Node& n = nodes[id];
    if (n.dead) continue;
    for (int v : n.inputs) {
      if (users[v].empty() || users[v].back() != id) users[v].push_back(id);
    }
  }
  return users;
}

void Graph::Toposort() {
  std::vector<int> pos(nodes.size(), 1 << 30);
  for (size_t i = 0; i < order.size(); ++i) pos[order[i]] = static_cast<int>(i);
  std::vector<int> indeg(nodes.size(), 0);
  std::vector<std::vector<int>> succ(nodes.size());
  int live = 0;
  for (auto& n : nodes) {
    if (n.dead) continue;
    ++live;
    std::set<int> preds;
    for (int v : n.inputs) {
      int p = values[v].producer;
      if (p >= 0 && !nodes[p].dead) preds.insert(p);
    }
    indeg[n.id] = static_cast<int>(preds.size());
    for (int p : preds) succ[p].push_back(n.id);
  }
  auto cmp = [&](int a, int b) { return pos[a] != pos[b] ? pos[a] > pos[b] : a > b; };
  std::priority_queue<int, std::vector<int>, decltype(cmp)> ready(cmp);
  for (auto& n : nodes) if (!n.dead && indeg[n.id] == 0) ready.push(n.id);
  std::vector<int> out;
  while (!ready.empty()) {
    int id = ready.top();
    ready.pop();
    out.push_back(id);
    for (int s : succ[id]) if (--indeg[s] == 0) ready.push(s);
  }
  if (static_cast<int>(out.size()) != live) throw std::runtime_error("mmgraph: circular dependency between nodes");
  order = std::move(out);
}

int Graph::DeadCodeElimination() {
  std::vector<bool> live_value(values.size(), false);
  for (int v : outputs) live_value[v] = true;
  int removed = 0;
  for (auto it = order.rbegin(); it != order.rend(); ++it) {
    Node& n = nodes[*it];
    if (n.dead) continue;
    bool used = false;
    for (int o : n.outputs) used = used || live_value[o];
    if (!used) {
      n.dead = true;
      ++removed;
      continue;
    }
    for (int v : n.inputs) live_value[v] = true;
  }
  if (removed) {
    std::vector<int> keep;
    for (int id : order) if (!nodes[id].dead) keep.push_back(id);
    order = std::move(keep);
  }
  return removed;
}

void Graph::ReplaceAllUses(int from, int to) {
  for (auto& n : nodes) {
    if (n.dead) continue;
    for (int& v : n.inputs) if (v == from) v = to;
  }
  for (int& v : outputs) if (v == from) v = to;
}

std::string Graph::Dump() const {
  std::ostringstream os;
  auto vname = [&](int v) {
    std::ostringstream s;
    s << "%" << v << ":" << DTypeName(values[v].dtype) << "[";
    for (size_t i = 0; i < values[v].shape.size(); ++i) s << (i ? "," : "") << values[v].shape[i];
    s << "]";
    if (values[v].has_sharding) s << "{" << values[v].sharding.Key() << "}";
    return s.str();
  };
  os << "inputs:";
  for (int v : inputs) os << " " << vname(v);
  os << "\n";
  for (int id : order) {
    const Node& n = nodes[id];
    if (n.dead) continue;
    os << "  ";
    for (size_t i = 0; i < n.outputs.size(); ++i) os << (i ? ", " : "") << vname(n.outputs[i]);
    os << " = " << n.op << "(";
    for (size_t i = 0; i < n.inputs.size(); ++i) os << (i ? ", " : "") << "%" << n.inputs[i];
    os << ")";
    if (!n.color.empty()) os << " color=" << n.color;
    if (n.task >= 0) os << " task=" << n.task;
    if (n.loop >= 0) os << " loop=" << n.loop;
    if (!n.scope.empty()) os << " scope=" << n.scope;
    if (n.backprop) os << " bwd";
    os << "\n";
  }
  os << "outputs:";
  for (int v : outputs) os << " %" << v;
  os << "\n";
  return os.str();
}

// ------------------------------------------------------------------ TaskOptions
TaskOptions TaskOptions::FromJson(const Json& j) {
  TaskOptions o;
  if (j.has("name") && j.at("name").is_string()) o.name = j.at("name").str;
  if (j.has("devices")) for (auto v : j.at("devices").as_int_vector()) o.devices.push_back(static_cast<int>(v));
  if (j.has("dims")) for (auto v : j.at("dims").as_int_vector()) o.dims.push_back(static_cast<int>(v));
  if (j.has("device_axes")) o.device_axes = j.at("device_axes").as_string_vector();
  if (j.has("logical_axes"))
    for (auto& e : j.at("logical_axes").arr) o.logical_axes.emplace_back(e.arr[0].str, e.arr[1].str);
  if (j.has("split_backprop")) o.split_backprop = j.at("split_backprop").as_string_vector();
  if (j.has("loop_dependent_devices"))
    for (auto& row : j.at("loop_dependent_devices").arr) {
      std::vector<int> r;
      for (auto v : row.as_int_vector()) r.push_back(static_cast<int>(v));
      o.loop_dependent_devices.push_back(std::move(r));
    }
  return o;
}
Json TaskOptions::ToJson() const {
  Json j = Json::object();
  j.set("name", Json::string(name));
  Json d = Json::array();
  for (int v : devices) d.push(Json::number(v));
  j.set("devices", d);
  Json dm = Json::array();
  for (int v : dims) dm.push(Json::number(v));
  j.set("dims", dm);
  Json ax = Json::array();
  for (auto& a : device_axes) ax.push(Json::string(a));
  j.set("device_axes", ax);
  Json la = Json::array();
  for (auto& p : logical_axes) {
    Json e = Json::array();
    e.push(Json::string(p.first));
    e.push(Json::string(p.second));
    la.push(e);
  }
  j.set("logical_axes", la);
  Json sb = Json::array();
  for (auto& x : split_backprop) sb.push(Json::string(x));
  j.set("split_backprop", sb);
  Json ld = Json::array();
  for (auto& row : loop_dependent_devices) {
    Json r = Json::array();
    for (int v : row) r.push(Json::number(v));
    ld.push(r);
  }
  j.set("loop_dependent_devices", ld);
  return j;
}

// -------------------------------------------------------------------- Partition
const ColorConfig& Partition::Get(const std::string& color) const {
  auto it = colors_.find(color);
  if (it == colors_.end()) throw std::runtime_error("unknown task colour '" + color + "'");
  return it->second;
}
ColorConfig& Partition::GetMutable(const std::string& color) {
  auto it = colors_.find(color);
  if (it == colors_.end()) throw std::runtime_error("unknown task colour '" + color + "'");
  return it->second;
}

const ColorConfig& Partition::Add(const TaskOptions& in, bool backprop, const std::string& color_name) {
  TaskOptions opts = in;
  if (opts.devices.empty()) {  // default placement: every device, one axis "x"
    opts.devices = global_.ToList();
    opts.dims = {global_.n};
    opts.device_axes = {"x"};
  }
  if (opts.dims.empty()) {
    opts.dims = {static_cast<int>(opts.devices.size())};
    if (opts.device_axes.empty()) opts.device_axes = {"x"};
  }
  int mesh = 1;
  for (int d : opts.dims) mesh *= d;
  if (mesh != static_cast<int>(opts.devices.size()))
    throw std::runtime_error("task '" + opts.name + "': mesh shape does not match its device count");
  DeviceRange devs = DeviceRange::FromList(opts.devices);
  if (!global_.Contains(devs))
    throw std::runtime_error("task '" + opts.name + "': devices " + devs.ToString() +
                             " are outside the executable's devices " + global_.ToString());
  const std::string name = color_name.empty() ? opts.name : color_name;
  auto it = colors_.find(name);
  if (it != colors_.end()) {
    if (it->second.devices != devs)
      throw std::runtime_error("task colour '" + name + "' is mapped to two different device lists");
    return it->second;
  }
  ColorConfig c;
  c.name = name;
  c.devices = devs;
  c.backprop = backprop;
  c.options = opts;
  c.original = name;
  return colors_[name] = c;
}

std::string Partition::Recolor(const std::string& color, const std::string& new_name) {
  ColorConfig c = Get(color);
  if (c.original.empty()) c.original = color;
  c.name = new_name;
  colors_[new_name] = c;
  return new_name;
}
std::string Partition::Clone(const std::string& color, const std::string& new_name, DeviceRange devices) {
  ColorConfig c = Get(color);
  c.name = new_name;
  c.devices = devices;
  c.options.devices = devices.ToList();
  colors_[new_name] = c;
  return new_name;
}

void Partition::RegisterFactory(const std::string& regex, TaskFactory factory) {
  factories_.emplace_back(regex, std::move(factory));
}

std::string Partition::ComputeScopeColor(const std::string& scope, bool backprop) {
  if (scope.empty()) return "";
  auto pin = pinned_.find({scope, backprop});
  if (pin != pinned_.end()) return pin->second;
  for (auto& f : factories_) {
    std::smatch m;
    std::regex re(f.first);
    if (!std::regex_search(scope, m, re)) continue;
    const std::string matched = m.size() > 1 ? m[1].str() : m[0].str();
    auto key = std::make_pair(f.first + "\x01" + matched, backprop);
    auto hit = cache_.find(key);
    if (hit != cache_.end()) return hit->second;
    TaskOptions opts = TaskOptions::FromJson(Json::parse(f.second(matched, backprop)));
    std::string name = opts.name.empty() ? matched : opts.name;
    if (opts.name.empty() && backprop) name += "_bwd";
    opts.name = name;
    const ColorConfig& c = Add(opts, backprop);
    cache_[key] = c.name;
    return c.name;
  }
  return "";
}

// ----------------------------------------------------------------------- config
bool GetEnvBool(const char* name, bool dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  std::string s(v);
  return !(s == "0" || s == "false" || s == "False" || s == "off");
}
int64_t GetEnvInt(const char* name, int64_t dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  return std::atoll(v);
}
std::string GetEnvString(const char* name, const std::string& dflt) {
  const char* v = std::getenv(name);
  return (v && *v) ? std::string(v) : dflt;
}
PartitionConfig PartitionConfig::FromEnv() {
  PartitionConfig c;
  c.hoist_loop_convert = GetEnvBool("MULTIMESH_HOIST_CONVERT", false);
  c.remove_hoisted_reduces = GetEnvBool("MULTIMESH_REMOVE_HOISTED_REDUCE", false);
  c.loop_increment_color = GetEnvBool("MULTIMESH_LOOP_INCREMENT_COLOR", false);
  c.argument_recompute = GetEnvBool("MULTIMESH_ARGUMENT_RECOMPUTE", true);
  c.minimize_cut_size = GetEnvBool("MULTIMESH_MINIMIZE_CUT_SIZE", true);
  c.zero_arguments = GetEnvBool("MULTIMESH_ZERO_ARGUMENTS", false);
  c.dynamic_schedule_post_loop_tasks = GetEnvBool("MULTIMESH_DYNAMIC_SCHEDULE_POST_LOOP_TASKS", true);
  c.color_propagation_priority = GetEnvString("MULTIMESH_COLOR_PROPAGATION_PRIORITY", "WEIGHT");
  return c;
}

// ------------------------------------------------------------------------- Plan
std::string Plan::Dump(const Graph& g) const {
  std::ostringstream os;
  os << "templates:\n";
  for (auto& t : templates) {
    os << "  T" << t.id << " " << t.name << " devices=" << t.devices.ToString() << " nodes=" << t.nodes.size()
       << (t.in_loop ? " loop" : "") << (t.backprop ? " bwd" : "") << (t.noncritical ? " noncritical" : "")
       << (t.has_collectives ? " collectives" : "") << "\n";
  }
  os << "stores:\n";
  for (auto& s : stores) {
    static const char* kinds[] = {"PARAM", "ROOT", "TEMP"};
    os << "  S" << s.id << " " << kinds[s.kind] << "#" << s.index << " name=" << s.name << " " << s.shape.Key();
    if (s.alias_of >= 0) os << " alias_of=S" << s.alias_of;
    os << "\n";
  }
  os << "ops:\n";
  for (auto& op : ops) {
    switch (op.kind) {
      case PlanOp::TASK:
        os << "  task " << op.name << " T" << op.task_template << " it=" << op.iteration << " dev="
           << op.devices.ToString() << " in=";
        for (int s : op.inputs) os << "S" << s << " ";
        os << "out=";
        for (int s : op.outputs) os << "S" << s << " ";
        os << "\n";
        break;
      case PlanOp::RESHARD: os << "  reshard S" << op.src_store << " -> S" << op.dst_store << "\n"; break;
      case PlanOp::CREATE_STORE: os << "  create S" << op.store << "\n"; break;
      case PlanOp::FREE_STORE: os << "  free S" << op.store << "\n"; break;
    }
  }
  (void)g;
  return os.str();
}

uint64_t Plan::Hash() const {
  uint64_t h = 1469598103934665603ull;
  auto mix = [&](uint64_t v) { h ^= v; h *= 1099511628211ull; };
  for (auto& op : ops) {
    mix(static_cast<uint64_t>(op.kind));
    mix(static_cast<uint64_t>(op.task_template + 1));
    mix(static_cast<uint64_t>(op.iteration + 1));
    mix(static_cast<uint64_t>(op.devices.start));
    mix(static_cast<uint64_t>(op.devices.n));
    for (int s : op.inputs) mix(static_cast<uint64_t>(s));
    for (int s : op.outputs) mix(static_cast<uint64_t>(s));
    mix(static_cast<uint64_t>(op.src_store + 1));
    mix(static_cast<uint64_t>(op.dst_store + 1));
    mix(static_cast<uint64_t>(op.store + 1));
  }
  return h;
}

}  // namespace mmg
