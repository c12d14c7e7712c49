// Per-task sharding: logical -> physical mapping, propagation through an
// index-class ("einsum-like") rule table, SPMD lowering (insert local
// reshards and reductions of partial results) and hoisting of gradient
// reductions out of the microbatch loop.
//
// The reference delegates propagation and partitioning to XLA
// (src/pjrt_client/mpmd_sharding_propagation.cc:198-206,
//  src/pjrt_client/mpmd_shard_map_loop_reduce.cc:137-147); here the rule table is ours.
#include <algorithm>
#include <map>
#include <set>
#include <stdexcept>

#include "passes.h"

namespace mmg {

namespace {

std::string BaseOp(const std::string& op) {
  size_t first = op.find('.');
  if (first == std::string::npos) return op;
  size_t second = op.find('.', first + 1);
  return second == std::string::npos ? op : op.substr(0, second);
}

// One tensor index shared by several operand / result dimensions.
struct IndexClass {
  std::vector<std::pair<int, int>> members;  // (slot, dim); slot < #inputs: input, else output
  bool no_shard = false;                     // must stay unsharded (softmax dim, conv window ...)
  std::set<int> reduced_outputs;             // outputs (by index) in which this index is summed away
  bool shares_axes = false;                  // may use a mesh axis that another class of the node uses
                                             // (experts and tokens of an expert-parallel layer)
};

struct Rule {
  std::vector<IndexClass> classes;
  bool known = true;
  double partial_scale = 1.0;  // e.g. mean: multiply after the reduction
};

Json ArgsOf(const Node& n) {
  try { return Json::parse(n.Attr("args", "[]")); } catch (...) { return Json::array(); }
}
int NormDim(int64_t d, size_t rank) { return static_cast<int>(d < 0 ? d + static_cast<int64_t>(rank) : d); }

void AddIdentity(Rule& r, const Graph& g, const Node& n, int in_slot, int out_idx) {
  const auto& a = g.value(n.inputs[in_slot]).shape;
  const auto& o = g.value(n.outputs[out_idx]).shape;
  const int nin = static_cast<int>(n.inputs.size());
  // right-aligned broadcasting
  for (size_t k = 0; k < o.size(); ++k) {
    const int od = static_cast<int>(o.size() - 1 - k);
    if (k >= a.size()) continue;
    const int ad = static_cast<int>(a.size() - 1 - k);
    if (a[ad] != o[od] || a[ad] == 1) continue;
    // find the class that already holds (out, od)
    IndexClass* found = nullptr;
    for (auto& c : r.classes)
      for (auto& m : c.members) if (m.first == nin + out_idx && m.second == od) found = &c;
    if (!found) { r.classes.emplace_back(); found = &r.classes.back(); found->members.emplace_back(nin + out_idx, od); }
    found->members.emplace_back(in_slot, ad);
  }
}

Rule ElementwiseRule(const Graph& g, const Node& n) {
  Rule r;
  for (size_t o = 0; o < n.outputs.size(); ++o)
    for (size_t i = 0; i < n.inputs.size(); ++i) AddIdentity(r, g, n, static_cast<int>(i), static_cast<int>(o));
  // several same-shaped outputs share classes through their common inputs only; merge by dim
  return r;
}

IndexClass Cls(std::initializer_list<std::pair<int, int>> m) { IndexClass c; c.members.assign(m.begin(), m.end()); return c; }

Rule GetRule(const Graph& g, const Node& n) {
  Rule r;
  const std::string b = BaseOp(n.op);
  const int nin = static_cast<int>(n.inputs.size());
  auto in_rank = [&](int i) { return static_cast<int>(g.value(n.inputs[i]).shape.size()); };
  auto out_rank = [&](int i) { return static_cast<int>(g.value(n.outputs[i]).shape.size()); };
  const Json args = ArgsOf(n);

  if (IsElementwise(n) || b == "aten.detach" || b == "aten.alias" || b == "aten.contiguous" ||
      b == "aten.lift_fresh" || n.op == "mm.all_reduce") {
    return ElementwiseRule(g, n);
  }
  if (b == "aten.mm" && nin == 2) {
    r.classes = {Cls({{0, 0}, {2, 0}}), Cls({{1, 1}, {2, 1}})};
    IndexClass k = Cls({{0, 1}, {1, 0}});
    k.reduced_outputs = {0};
    r.classes.push_back(k);
    return r;
  }
  if (b == "aten.addmm" && nin == 3) {
    r.classes = {Cls({{1, 0}, {3, 0}}), Cls({{2, 1}, {3, 1}})};
    IndexClass k = Cls({{1, 1}, {2, 0}});
    k.reduced_outputs = {0};
    r.classes.push_back(k);
    const auto& bias = g.value(n.inputs[0]).shape;
    if (bias.size() == 1 && bias[0] != 1) r.classes[1].members.emplace_back(0, 0);
    return r;
  }
  if (b == "aten.bmm" && nin == 2) {
    r.classes = {Cls({{0, 0}, {1, 0}, {2, 0}}), Cls({{0, 1}, {2, 1}}), Cls({{1, 2}, {2, 2}})};
    IndexClass k = Cls({{0, 2}, {1, 1}});
    k.reduced_outputs = {0};
    r.classes.push_back(k);
    return r;
  }
  if (b == "mm_ops.linear" && nin >= 2) {  // x[..., K], w[N, K] -> [..., N]
    const int xr = in_rank(0);
    for (int d = 0; d + 1 < xr; ++d) r.classes.push_back(Cls({{0, d}, {nin, d}}));
    r.classes.push_back(Cls({{1, 0}, {nin, xr - 1}}));
    IndexClass k = Cls({{0, xr - 1}, {1, 1}});
    k.reduced_outputs = {0};
    r.classes.push_back(k);
    return r;
  }
  if (b == "mm_ops.linear_dgrad" && nin >= 2) {  // dy[..., N], w[N, K] -> [..., K]
    const int xr = in_rank(0);
    for (int d = 0; d + 1 < xr; ++d) r.classes.push_back(Cls({{0, d}, {nin, d}}));
    r.classes.push_back(Cls({{1, 1}, {nin, xr - 1}}));
    IndexClass k = Cls({{0, xr - 1}, {1, 0}});
    k.reduced_outputs = {0};
    r.classes.push_back(k);
    return r;
  }
  if (b == "mm_ops.linear_wgrad" && nin >= 2) {  // dy[..., N], x[..., K] -> [N, K]
    const int xr = in_rank(0);
    for (int d = 0; d + 1 < xr; ++d) {
      IndexClass k = Cls({{0, d}, {1, d}});
      k.reduced_outputs = {0};
      r.classes.push_back(k);
    }
    r.classes.push_back(Cls({{0, xr - 1}, {nin, 0}}));
    r.classes.push_back(Cls({{1, xr - 1}, {nin, 1}}));
    return r;
  }
  if (b == "aten.t" && in_rank(0) == 2) {
    r.classes = {Cls({{0, 0}, {1, 1}}), Cls({{0, 1}, {1, 0}})};
    return r;
  }
  if (b == "aten.transpose" && args.arr.size() >= 2) {
    const int rank = in_rank(0);
    const int d0 = NormDim(args.arr[0].as_int(), rank), d1 = NormDim(args.arr[1].as_int(), rank);
    for (int d = 0; d < rank; ++d) r.classes.push_back(Cls({{0, d}, {1, d == d0 ? d1 : (d == d1 ? d0 : d)}}));
    return r;
  }
  if (b == "aten.permute" && args.arr.size() >= 1 && args.arr[0].is_array()) {
    const auto perm = args.arr[0].as_int_vector();
    const int rank = in_rank(0);
    for (size_t od = 0; od < perm.size(); ++od)
      r.classes.push_back(Cls({{0, NormDim(perm[od], rank)}, {1, static_cast<int>(od)}}));
    return r;
  }
  if (b == "aten.view" || b == "aten.reshape" || b == "aten._unsafe_view" || b == "aten.flatten" ||
      b == "aten.unflatten") {
    // match groups of dims with equal products; only the major dim of a group carries sharding
    const auto& a = g.value(n.inputs[0]).shape;
    const auto& o = g.value(n.outputs[0]).shape;
    size_t i = 0, j = 0;
    while (i < a.size() && j < o.size()) {
      size_t i0 = i, j0 = j;
      int64_t pa = a[i++], po = o[j++];
      while (pa != po) {
        if (pa < po) { if (i >= a.size()) break; pa *= a[i++]; }
        else { if (j >= o.size()) break; po *= o[j++]; }
      }
      if (pa != po) { r.known = false; return r; }
      // skip leading size-1 dims on either side
      size_t ia = i0, jo = j0;
      while (ia + 1 < i && a[ia] == 1) ++ia;
      while (jo + 1 < j && o[jo] == 1) ++jo;
      IndexClass c = Cls({{0, static_cast<int>(ia)}, {1, static_cast<int>(jo)}});
      // If the group is not 1:1, the shard count must divide both major dims; checked when assigning.
      r.classes.push_back(c);
      for (size_t d = i0; d < i; ++d) if (d != ia) { IndexClass z = Cls({{0, static_cast<int>(d)}}); z.no_shard = true; r.classes.push_back(z); }
      for (size_t d = j0; d < j; ++d) if (d != jo) { IndexClass z = Cls({{1, static_cast<int>(d)}}); z.no_shard = true; r.classes.push_back(z); }
    }
    return r;
  }
  if (b == "aten.unsqueeze" && args.arr.size() >= 1) {
    const int rank = out_rank(0);
    const int at = NormDim(args.arr[0].as_int(), rank);
    for (int d = 0, s = 0; d < rank; ++d) { if (d == at) continue; r.classes.push_back(Cls({{0, s}, {1, d}})); ++s; }
    return r;
  }
  if (b == "aten.squeeze") {
    const auto& a = g.value(n.inputs[0]).shape;
    const auto& o = g.value(n.outputs[0]).shape;
    size_t j = 0;
    for (size_t d = 0; d < a.size(); ++d) {
      if (j < o.size() && a[d] == o[j]) { r.classes.push_back(Cls({{0, static_cast<int>(d)}, {1, static_cast<int>(j)}})); ++j; }
    }
    return r;
  }
  if (b == "aten.expand") { AddIdentity(r, g, n, 0, 0); return r; }
  if ((b == "aten.sum" || b == "aten.mean") ) {
    const int rank = in_rank(0);
    std::set<int> red;
    bool keepdim = false;
    if (args.arr.size() >= 1 && args.arr[0].is_array()) {
      for (auto d : args.arr[0].as_int_vector()) red.insert(NormDim(d, rank));
      if (args.arr.size() >= 2 && args.arr[1].kind == Json::Bool) keepdim = args.arr[1].b;
    } else {
      for (int d = 0; d < rank; ++d) red.insert(d);
    }
    int od = 0;
    for (int d = 0; d < rank; ++d) {
      if (red.count(d)) {
        IndexClass k = Cls({{0, d}});
        k.reduced_outputs = {0};
        r.classes.push_back(k);
        if (keepdim) ++od;
      } else {
        r.classes.push_back(Cls({{0, d}, {1, od}}));
        ++od;
      }
    }
    if (b == "aten.mean") r.partial_scale = -1.0;  // scale by 1/#shards after the reduction
    return r;
  }
  if (b == "aten._softmax" || b == "aten._log_softmax" || b == "aten._softmax_backward_data" ||
      b == "aten._log_softmax_backward_data" || b == "aten.softmax" || b == "aten.log_softmax") {
    Rule e = ElementwiseRule(g, n);
    const int rank = out_rank(0);
    int dim = rank - 1;
    for (auto& a : args.arr) if (a.is_number()) { dim = NormDim(a.as_int(), rank); break; }
    for (auto& c : e.classes) for (auto& m : c.members) if (m.first == nin && m.second == dim) c.no_shard = true;
    return e;
  }
  if (b == "aten.slice" || b == "aten.narrow" || b == "aten.select" || b == "aten.cat" || b == "aten.index_select") {
    if (b == "aten.cat") { r.known = false; return r; }
    const int rank = in_rank(0);
    const int dim = args.arr.size() >= 1 && args.arr[0].is_number() ? NormDim(args.arr[0].as_int(), rank) : 0;
    int od = 0;
    for (int d = 0; d < rank; ++d) {
      if (d == dim) {
        IndexClass z = Cls({{0, d}});
        z.no_shard = true;
        if (b != "aten.select") { z.members.emplace_back(1, od); ++od; }
        r.classes.push_back(z);
      } else {
        r.classes.push_back(Cls({{0, d}, {1, od}}));
        ++od;
      }
    }
    return r;
  }
  if (n.op == "mm.dynamic_slice" || n.op == "mm.copy" || n.op == "mm.accumulate") {
    // same rank, dimension by dimension; a sliced dimension keeps its sharding (every
    // shard contributes its own rows to each microbatch) unless the slices of the loop would
    // be cut differently (`exact_rows`, see MarkExactMicrobatchSlices): then the sliced
    // dimension stays whole and microbatch i is rows [i * size, (i + 1) * size) exactly
    const int rank = in_rank(0);
    const int exact = n.op == "mm.dynamic_slice" && n.Attr("exact_rows") == "1" ? std::atoi(n.Attr("dim", "0").c_str()) : -1;
    for (int d = 0; d < rank; ++d) {
      IndexClass c = Cls({{0, d}, {nin, d}});
      c.no_shard = d == exact;
      r.classes.push_back(c);
    }
    return r;
  }
  r.known = false;
  return r;
}

// Rules supplied by the front end for custom operators: attrs["shard_rule"] =
// {"classes":[{"members":[[slot,dim],...],"no_shard":bool,"reduced_outputs":[i,...]}], "partial_scale": x}
bool RuleFromAttr(const Node& n, Rule* out) {
  auto it = n.attrs.find("shard_rule");
  if (it == n.attrs.end()) return false;
  const Json j = Json::parse(it->second);
  Rule r;
  for (auto& c : j.at("classes").arr) {
    IndexClass ic;
    for (auto& m : c.at("members").arr)
      ic.members.emplace_back(static_cast<int>(m.arr[0].as_int()), static_cast<int>(m.arr[1].as_int()));
    if (c.has("no_shard")) ic.no_shard = c.at("no_shard").as_bool();
    if (c.has("shares_axes")) ic.shares_axes = c.at("shares_axes").as_bool();
    if (c.has("reduced_outputs"))
      for (auto v : c.at("reduced_outputs").as_int_vector()) ic.reduced_outputs.insert(static_cast<int>(v));
    r.classes.push_back(ic);
  }
  if (j.has("partial_scale")) r.partial_scale = j.at("partial_scale").num;
  *out = r;
  return true;
}

Rule RuleFor(const Graph& g, const Node& n) {
  Rule r;
  if (RuleFromAttr(n, &r)) return r;
  return GetRule(g, n);
}

struct TaskMeshInfo {
  std::vector<int> dims;
  std::vector<std::string> names;
  std::vector<std::pair<std::string, std::string>> logical_axes;
  DeviceRange devices;
};

TaskMeshInfo MeshOf(const Partition& part, const std::string& color) {
  const ColorConfig& c = part.Get(color);
  TaskMeshInfo m;
  m.dims = c.options.dims.empty() ? std::vector<int>{c.devices.n} : c.options.dims;
  m.names = c.options.device_axes;
  while (m.names.size() < m.dims.size()) m.names.push_back("axis" + std::to_string(m.names.size()));
  m.logical_axes = c.options.logical_axes;
  m.devices = c.devices;
  return m;
}

ShardedShape ReplicatedOn(const Value& v, const TaskMeshInfo& m) {
  ShardedShape s;
  s.dtype = v.dtype;
  s.sizes = v.shape;
  s.dim_axes.assign(v.shape.size(), {});
  s.mesh_dims = m.dims;
  s.devices = m.devices;
  return s;
}

// Sharding implied by the value's axis-name annotation on mesh `m`.
ShardedShape FromAxes(const Value& v, const TaskMeshInfo& m) {
  if (v.axes_logical)
    return LogicalToPhysical(v.dtype, v.shape, v.axes, m.logical_axes, m.names, m.dims, m.devices);
  ShardedShape s = ReplicatedOn(v, m);
  std::vector<bool> used(m.dims.size(), false);
  for (size_t d = 0; d < v.axes.size(); ++d)
    for (auto& name : v.axes[d])
      for (size_t a = 0; a < m.names.size(); ++a)
        if (m.names[a] == name && !used[a] && m.dims[a] > 1 &&
            v.shape[d] % (static_cast<int64_t>(s.Shards(static_cast<int>(d))) * m.dims[a]) == 0) {
          s.dim_axes[d].push_back(static_cast<int>(a));
          used[a] = true;
        }
  return s;
}

// Re-expresses `src` (sharded on another submesh) on mesh `m`: equal meshes copy the
// assignment; otherwise shard counts are matched to mesh axes, with the first sharded
// dimension rescaled when the device counts differ (ResizeSharding semantics).
ShardedShape AdoptSharding(const ShardedShape& src, const Value& v, const TaskMeshInfo& m) {
  if (src.mesh_dims == m.dims) {
    ShardedShape s = src;
    s.devices = m.devices;
    return s;
  }
  bool ok = true;
  ShardedShape resized = src.devices.n == m.devices.n ? src : ResizeSharding(src, m.devices, &ok);
  ShardedShape s = ReplicatedOn(v, m);
  if (!ok) return s;
  std::vector<bool> used(m.dims.size(), false);
  for (int d = 0; d < resized.rank(); ++d) {
    int want = resized.Shards(d);
    if (want == 1) continue;
    // greedily take unused mesh axes, major first, whose product equals the shard count
    std::vector<int> pick;
    int prod = 1;
    for (size_t a = 0; a < m.dims.size() && prod < want; ++a) {
      if (used[a] || m.dims[a] == 1) continue;
      if (want % (prod * m.dims[a]) == 0) { pick.push_back(static_cast<int>(a)); prod *= m.dims[a]; }
    }
    if (prod == want) {
      for (int a : pick) used[a] = true;
      s.dim_axes[d] = pick;
    }
  }
  return s;
}

int AxesProduct(const std::vector<int>& axes, const std::vector<int>& dims) {
  int p = 1;
  for (int a : axes) p *= dims[a];
  return p;
}

}  // namespace

// ---------------------------------------------------------------------------
// Shared state of the sharding passes, kept on the side of CompileState
// ---------------------------------------------------------------------------
struct ShardingTables {
  // sharding with which task `group` reads external value `value`
  std::map<std::pair<int, int>, ShardedShape> input_sharding;
  std::set<int> fixed_values;  // values whose sharding comes from an annotation
};
static std::map<const CompileState*, ShardingTables> g_tables;
ShardingTables& TablesOf(const CompileState& s) { return g_tables[&s]; }
void ReleaseShardingTables(const CompileState& s) { g_tables.erase(&s); }
const ShardedShape* InputShardingOf(const CompileState& s, int group, int value) {
  auto& t = TablesOf(s);
  auto it = t.input_sharding.find({group, value});
  return it == t.input_sharding.end() ? nullptr : &it->second;
}

void SetInputSharding(const CompileState& s, int group, int value, const ShardedShape& sh) {
  TablesOf(s).input_sharding[{group, value}] = sh;
}

namespace {

const ShardedShape* Available(CompileState& s, const TaskGroup& grp, int value) {
  const Graph& g = *s.graph;
  const int p = g.value(value).producer;
  if (p >= 0 && g.node(p).task == grp.id) return g.value(value).has_sharding ? &g.value(value).sharding : nullptr;
  return InputShardingOf(s, grp.id, value);
}

void SetAvailable(CompileState& s, const TaskGroup& grp, int value, const ShardedShape& sh) {
  Graph& g = *s.graph;
  const int p = g.value(value).producer;
  if (p >= 0 && g.node(p).task == grp.id) {
    g.value(value).sharding = sh;
    g.value(value).has_sharding = true;
  } else {
    TablesOf(s).input_sharding[{grp.id, value}] = sh;
  }
}

// Evaluates one node: derives per-class mesh axes from the shardings that are known and
// writes them to members that have none. Returns true when something was assigned.
bool EvalNode(CompileState& s, const TaskGroup& grp, const TaskMeshInfo& mesh, Node& n, bool to_outputs,
              bool to_inputs, bool assign_trivial) {
  Graph& g = *s.graph;
  const int nin = static_cast<int>(n.inputs.size());
  auto slot_value = [&](int slot) { return slot < nin ? n.inputs[slot] : n.outputs[slot - nin]; };
  Rule rule = RuleFor(g, n);
  bool changed = false;
  if (!rule.known) {
    if (assign_trivial) {
      for (int slot = 0; slot < nin + static_cast<int>(n.outputs.size()); ++slot) {
        const int v = slot_value(slot);
        if ((slot < nin ? to_inputs : to_outputs) && !Available(s, grp, v)) {
          SetAvailable(s, grp, v, ReplicatedOn(g.value(v), mesh));
          changed = true;
        }
      }
    }
    return changed;
  }
  // candidate axes per class
  std::vector<std::vector<int>> class_axes(rule.classes.size());
  for (size_t c = 0; c < rule.classes.size(); ++c) {
    const IndexClass& ic = rule.classes[c];
    if (ic.no_shard) continue;
    int best = 1;
    for (auto& m : ic.members) {
      const ShardedShape* sh = Available(s, grp, slot_value(m.first));
      if (!sh || sh->mesh_dims != mesh.dims || m.second >= sh->rank()) continue;
      const int prod = AxesProduct(sh->dim_axes[m.second], mesh.dims);
      if (prod > best) { best = prod; class_axes[c] = sh->dim_axes[m.second]; }
    }
    // every member must be divisible
    for (auto& m : ic.members) {
      const Value& v = g.value(slot_value(m.first));
      if (m.second >= static_cast<int>(v.shape.size()) || v.shape[m.second] % best) { class_axes[c].clear(); break; }
    }
  }
  // a mesh axis may serve only one class of a node (unless the class says otherwise)
  std::set<int> used;
  for (size_t c = 0; c < class_axes.size(); ++c) {
    if (rule.classes[c].shares_axes) continue;
    std::vector<int> keep;
    for (int a : class_axes[c]) if (used.insert(a).second) keep.push_back(a);
    class_axes[c] = keep;
  }
  // write to members without sharding
  const int nslots = nin + static_cast<int>(n.outputs.size());
  for (int slot = 0; slot < nslots; ++slot) {
    const bool is_in = slot < nin;
    if (is_in ? !to_inputs : !to_outputs) continue;
    const int v = slot_value(slot);
    if (Available(s, grp, v)) continue;
    ShardedShape sh = ReplicatedOn(g.value(v), mesh);
    bool nontrivial = false;
    for (size_t c = 0; c < rule.classes.size(); ++c)
      for (auto& m : rule.classes[c].members)
        if (m.first == slot && m.second < sh.rank() && !class_axes[c].empty()) {
          sh.dim_axes[m.second] = class_axes[c];
          nontrivial = true;
        }
    if (!nontrivial && !assign_trivial) continue;
    SetAvailable(s, grp, v, sh);
    changed = true;
  }
  return changed;
}

}  // namespace

// ---------------------------------------------------------------------------
// Logical -> physical
// ---------------------------------------------------------------------------
bool LogicalToPhysicalSharding(CompileState& s) {
  Graph& g = *s.graph;
  Partition& part = *s.partition;
  ShardingTables& tables = TablesOf(s);
  tables.input_sharding.clear();
  tables.fixed_values.clear();
  for (auto& v : g.values) { v.has_sharding = false; v.partial = false; v.partial_axes.clear(); }
  bool changed = false;
  for (auto& grp : s.groups) {
    const TaskMeshInfo mesh = MeshOf(part, grp.color);
    if (mesh.devices.n == 1) continue;  // single-device tasks carry no sharding at all
    for (int id : grp.nodes) {
      const Node& n = g.node(id);
      for (int o : n.outputs) {
        Value& v = g.value(o);
        if (!v.has_axes) continue;
        v.sharding = FromAxes(v, mesh);
        v.has_sharding = true;
        tables.fixed_values.insert(o);
        changed = true;
      }
      for (int in : n.inputs) {
        const Value& v = g.value(in);
        const int p = v.producer;
        if ((p >= 0 && g.node(p).task == grp.id) || !v.has_axes) continue;
        tables.input_sharding[{grp.id, in}] = FromAxes(v, mesh);
        changed = true;
      }
    }
  }
  return changed;
}

// ---------------------------------------------------------------------------
// Propagation
// ---------------------------------------------------------------------------
bool ShardingPropagation(CompileState& s, PropagationMode mode) {
  Graph& g = *s.graph;
  Partition& part = *s.partition;
  bool changed_any = false;
  const bool full = mode == PropagationMode::kForwardFull;
  const bool forward = mode != PropagationMode::kBackwardInputOutput;
  for (int round = 0; round < 4; ++round) {
    bool changed = false;
    // Layout that some task already chose for an argument of the step (a parameter, its
    // optimizer state): other tasks on the same mesh read the argument in that layout too
    // instead of each settling on its own (a replicated reader of a sharded weight would
    // pay a gather of the weight and redundant math every step).
    std::map<int, ShardedShape> argument_layout;
    for (auto& kv : TablesOf(s).input_sharding) {
      const int value = kv.first.second;
      if (g.value(value).producer >= 0 || kv.second.IsReplicated()) continue;
      argument_layout.emplace(value, kv.second);
    }
    auto do_group = [&](TaskGroup& grp) {
      const TaskMeshInfo mesh = MeshOf(part, grp.color);
      if (mesh.devices.n == 1) return;
      if (forward) {
        // adopt producer shardings for external inputs
        for (int id : grp.nodes)
          for (int in : g.node(id).inputs) {
            const Value& v = g.value(in);
            const int p = v.producer;
            if (p < 0) {
              auto al = argument_layout.find(in);
              if (al == argument_layout.end() || InputShardingOf(s, grp.id, in)) continue;
              if (al->second.mesh_dims != mesh.dims || !(al->second.devices == mesh.devices)) continue;
              TablesOf(s).input_sharding[{grp.id, in}] = al->second;
              changed = true;
              continue;
            }
            if (g.node(p).task == grp.id || !v.has_sharding) continue;
            if (InputShardingOf(s, grp.id, in)) continue;
            ShardedShape adopted = AdoptSharding(v.sharding, v, mesh);
            if (adopted.IsReplicated() && !full) continue;
            TablesOf(s).input_sharding[{grp.id, in}] = adopted;
            changed = true;
          }
        for (int id : grp.nodes) changed |= EvalNode(s, grp, mesh, g.node(id), true, full, full);
      } else {
        for (auto it = grp.nodes.rbegin(); it != grp.nodes.rend(); ++it)
          changed |= EvalNode(s, grp, mesh, g.node(*it), false, true, false);
        // hand input shardings back to producers that have none (same mesh only)
        for (int id : grp.nodes)
          for (int in : g.node(id).inputs) {
            Value& v = g.value(in);
            const int p = v.producer;
            if (p < 0 || g.node(p).task == grp.id || v.has_sharding) continue;
            const ShardedShape* want = InputShardingOf(s, grp.id, in);
            if (!want || want->IsReplicated()) continue;
            const TaskMeshInfo pm = MeshOf(part, g.node(p).color);
            if (pm.devices.n == 1) continue;
            v.sharding = AdoptSharding(*want, v, pm);
            v.has_sharding = true;
            changed = true;
          }
      }
    };
    if (forward) for (auto& grp : s.groups) do_group(grp);
    else for (auto it = s.groups.rbegin(); it != s.groups.rend(); ++it) do_group(*it);
    changed_any |= changed;
    if (!changed) break;
  }
  return changed_any;
}

// ---------------------------------------------------------------------------
// SPMD lowering
// ---------------------------------------------------------------------------
namespace {

// Number of ways the sliced dimension of every microbatch slice is cut, per loop.
std::map<int, std::vector<std::pair<int, int>>> MicrobatchSliceCuts(CompileState& s, bool skip_exact) {
  Graph& g = *s.graph;
  std::map<int, std::vector<std::pair<int, int>>> cuts;   // loop -> (node, parts)
  for (auto& grp : s.groups) {
    const TaskMeshInfo mesh = MeshOf(*s.partition, grp.color);
    for (int id : grp.nodes) {
      const Node& n = g.node(id);
      if (n.dead || n.op != "mm.dynamic_slice" || n.loop < 0 || n.inputs.empty()) continue;
      if (skip_exact && n.Attr("exact_rows") == "1") continue;
      int parts = 1;
      if (mesh.devices.n > 1) {
        const Value& out = g.value(n.outputs[0]);
        const ShardedShape* sh = out.has_sharding ? &out.sharding : Available(s, grp, n.inputs[0]);
        const int dim = std::atoi(n.Attr("dim", "0").c_str());
        if (sh && dim >= 0 && dim < sh->rank()) parts = AxesProduct(sh->dim_axes[dim], mesh.dims);
      }
      cuts[n.loop].emplace_back(id, parts);
    }
  }
  return cuts;
}

// A microbatch slice along a sharded dimension is taken shard by shard: with the batch cut p
// ways, microbatch i is made of every shard's own rows [i * size / p, (i + 1) * size / p), not of
// the global rows [i * size, (i + 1) * size). That regrouping of rows is harmless - results of the
// loop are sums over all microbatches - as long as every sliced value of the loop is regrouped the
// same way. Where the slices of one loop would be cut differently (the samples split over two
// devices, the labels replicated; stages with different data-parallel widths), all of them are
// marked `exact_rows`: the sliced dimension stays whole, each device slices the global rows and a
// consumer that wants them split takes its part afterwards.
bool MarkExactMicrobatchSlices(CompileState& s) {
  bool marked = false;
  for (auto& kv : MicrobatchSliceCuts(s, false)) {
    bool same = true;
    for (auto& e : kv.second) same = same && e.second == kv.second.front().second;
    if (same) continue;
    for (auto& e : kv.second) s.graph->node(e.first).attrs["exact_rows"] = "1";
    s.Note("microbatch slices of loop " + std::to_string(kv.first) + " are cut differently: exact rows for all " +
           std::to_string(kv.second.size()) + " of them");
    marked = true;
  }
  return marked;
}

}  // namespace

bool SpmdLowering(CompileState& s) {
  Graph& g = *s.graph;
  Partition& part = *s.partition;
  bool changed = MarkExactMicrobatchSlices(s);
  for (auto& grp : s.groups) {
    const TaskMeshInfo mesh = MeshOf(part, grp.color);
    if (mesh.devices.n == 1) continue;
    std::vector<int> new_nodes;
    std::set<int> settled;  // external inputs whose layout some node of this task already relies on
    for (int id : std::vector<int>(grp.nodes)) {
      Node& n0 = g.node(id);
      const int nin = static_cast<int>(n0.inputs.size());
      if (n0.op == "mm.relayout") {
        // identity between two layouts: the result keeps the layout it was given (replicated
        // if none), the operand is converted to it right here
        const int in = n0.inputs[0], out = n0.outputs[0];
        ShardedShape target = g.value(out).has_sharding ? g.value(out).sharding : ReplicatedOn(g.value(out), mesh);
        g.value(out).sharding = target;
        g.value(out).has_sharding = true;
        const ShardedShape* have = Available(s, grp, in);
        // a value that another task produced is asked for in the target layout, so that the
        // layout changes while the value crosses between the tasks (one reshard, not two)
        const int in_prod = g.value(in).producer;
        if (in_prod >= 0 && g.node(in_prod).task != grp.id && !settled.count(in)) {
          TablesOf(s).input_sharding[{grp.id, in}] = target;
          settled.insert(in);
          continue;
        }
        settled.insert(in);
        if (!have) { SetAvailable(s, grp, in, target); continue; }
        if (have->mesh_dims == target.mesh_dims && have->dim_axes == target.dim_axes) continue;
        const ShardedShape from = *have;
        const int rid = g.AddNode("mm.spmd_reshard", {in}, {g.value(in).shape}, {g.value(in).dtype},
                                  {{"from", from.ToJson().dump()}, {"to", target.ToJson().dump()}});
        Node& rn = g.node(rid);
        rn.color = grp.color;
        rn.task = grp.id;
        rn.loop = g.node(id).loop;
        rn.backprop = g.node(id).backprop;
        g.value(rn.outputs[0]).sharding = target;
        g.value(rn.outputs[0]).has_sharding = true;
        g.node(id).inputs[0] = rn.outputs[0];
        new_nodes.push_back(rid);
        changed = true;
        continue;
      }
      Rule rule = RuleFor(g, n0);
      auto slot_value = [&](int slot) { return slot < nin ? g.node(id).inputs[slot] : g.node(id).outputs[slot - nin]; };
      // class axes: from outputs first (they are final), else from the most-sharded input
      std::vector<std::vector<int>> class_axes(rule.classes.size());
      if (rule.known) {
        std::set<int> used;
        for (int pass = 0; pass < 2; ++pass)
          for (size_t c = 0; c < rule.classes.size(); ++c) {
            if (rule.classes[c].no_shard || !class_axes[c].empty()) continue;
            std::vector<int> best;
            int best_p = 1;
            for (auto& m : rule.classes[c].members) {
              const bool is_out = m.first >= nin;
              if ((pass == 0) != is_out) continue;
              const ShardedShape* sh = Available(s, grp, slot_value(m.first));
              if (!sh || m.second >= sh->rank()) continue;
              const int p = AxesProduct(sh->dim_axes[m.second], mesh.dims);
              if (p > best_p) { best_p = p; best = sh->dim_axes[m.second]; }
            }
            bool ok = !best.empty();
            const bool shares = rule.classes[c].shares_axes;
            for (int a : best) ok = ok && (shares || !used.count(a));
            for (auto& m : rule.classes[c].members) {
              const Value& v = g.value(slot_value(m.first));
              if (m.second >= static_cast<int>(v.shape.size()) || v.shape[m.second] % best_p) ok = false;
            }
            if (ok) { class_axes[c] = best; if (!shares) for (int a : best) used.insert(a); }
          }
      }
      // operators whose per-device form exchanges data over a shared axis learn which axes
      if (rule.known)
        for (size_t c = 0; c < rule.classes.size(); ++c)
          if (rule.classes[c].shares_axes) {
            Json axes = Json::array();
            for (int a : class_axes[c]) axes.push(Json::number(a));
            g.node(id).attrs["shared_axes"] = axes.dump();
          }
      // required sharding of every input
      for (int slot = 0; slot < nin; ++slot) {
        const int v = g.node(id).inputs[slot];
        ShardedShape want = ReplicatedOn(g.value(v), mesh);
        if (rule.known)
          for (size_t c = 0; c < rule.classes.size(); ++c)
            for (auto& m : rule.classes[c].members)
              if (m.first == slot && m.second < want.rank()) want.dim_axes[m.second] = class_axes[c];
        const ShardedShape* have = Available(s, grp, v);
        if (!have) { SetAvailable(s, grp, v, want); settled.insert(v); continue; }
        if (have->mesh_dims == want.mesh_dims && have->dim_axes == want.dim_axes) { settled.insert(v); continue; }
        const int prod = g.value(v).producer;
        if (prod < 0 || g.node(prod).task != grp.id) {
          // external input: ask for it in the wanted layout unless another node of this task
          // already fixed a different one; then convert locally
          bool conflicting = TablesOf(s).fixed_values.count(v) > 0;
          conflicting = conflicting || settled.count(v) > 0;
          if (!conflicting) { TablesOf(s).input_sharding[{grp.id, v}] = want; settled.insert(v); continue; }
        }
        const int rid = g.AddNode("mm.spmd_reshard", {v}, {g.value(v).shape}, {g.value(v).dtype},
                                  {{"from", have->ToJson().dump()}, {"to", want.ToJson().dump()}});
        Node& rn = g.node(rid);
        rn.color = grp.color;
        rn.task = grp.id;
        rn.loop = g.node(id).loop;
        rn.backprop = g.node(id).backprop;
        g.value(rn.outputs[0]).sharding = want;
        g.value(rn.outputs[0]).has_sharding = true;
        g.node(id).inputs[slot] = rn.outputs[0];
        new_nodes.push_back(rid);
        changed = true;
      }
      // final sharding and partial-sum state of every output
      for (size_t o = 0; o < g.node(id).outputs.size(); ++o) {
        const int v = g.node(id).outputs[o];
        ShardedShape sh = ReplicatedOn(g.value(v), mesh);
        std::vector<int> partial;
        if (rule.known)
          for (size_t c = 0; c < rule.classes.size(); ++c) {
            for (auto& m : rule.classes[c].members)
              if (m.first == nin + static_cast<int>(o) && m.second < sh.rank()) sh.dim_axes[m.second] = class_axes[c];
            if (rule.classes[c].reduced_outputs.count(static_cast<int>(o)))
              partial.insert(partial.end(), class_axes[c].begin(), class_axes[c].end());
          }
        g.value(v).sharding = sh;
        g.value(v).has_sharding = true;
        if (partial.empty()) continue;
        std::sort(partial.begin(), partial.end());
        Json axes = Json::array();
        int shards = 1;
        for (int a : partial) { axes.push(Json::number(a)); shards *= mesh.dims[a]; }
        const double scale = rule.partial_scale < 0 ? 1.0 / shards : rule.partial_scale;
        const int rid = g.AddNode("mm.all_reduce", {v}, {g.value(v).shape}, {g.value(v).dtype},
                                  {{"axes", axes.dump()}, {"scale", std::to_string(scale)}});
        Node& rn = g.node(rid);
        rn.color = grp.color;
        rn.task = grp.id;
        rn.loop = g.node(id).loop;
        rn.backprop = g.node(id).backprop;
        const int reduced = rn.outputs[0];
        g.value(reduced).sharding = sh;
        g.value(reduced).has_sharding = true;
        g.value(reduced).axes = g.value(v).axes;
        g.value(reduced).has_axes = g.value(v).has_axes;
        g.value(v).partial = true;
        g.value(v).partial_axes = partial;
        // every other user reads the reduced value
        for (auto& m : g.nodes) {
          if (m.dead || m.id == rid) continue;
          for (int& in : m.inputs) if (in == v) in = reduced;
        }
        for (int& out : g.outputs) if (out == v) out = reduced;
        new_nodes.push_back(rid);
        changed = true;
      }
    }
    grp.nodes.insert(grp.nodes.end(), new_nodes.begin(), new_nodes.end());
  }
  if (changed) {
    g.Toposort();
    std::vector<int> pos(g.nodes.size(), 0);
    for (size_t i = 0; i < g.order.size(); ++i) pos[g.order[i]] = static_cast<int>(i);
    std::vector<int> order;
    for (auto& grp : s.groups) {
      std::sort(grp.nodes.begin(), grp.nodes.end(), [&](int a, int b) { return pos[a] < pos[b]; });
      order.insert(order.end(), grp.nodes.begin(), grp.nodes.end());
    }
    g.order = order;
  }
  // the layouts are final now: slices that regroup rows must all regroup them alike
  for (auto& kv : MicrobatchSliceCuts(s, true))
    for (auto& e : kv.second)
      if (e.second != kv.second.front().second)
        throw std::runtime_error("spmd_lowering: microbatch slices of loop " + std::to_string(kv.first) + " are cut " +
                                 std::to_string(kv.second.front().second) + " and " + std::to_string(e.second) +
                                 " ways; their rows would be paired wrongly");
  return changed;
}

// ---------------------------------------------------------------------------
// Collective folding: all-reduce followed by a slice over the same mesh axes becomes a
// reduce-scatter, and layout changes that only drop mesh axes from one dimension are tagged as
// all-gathers (the role of AllReduceFolder / ReduceScatterCreator behind
// src/pjrt_client/mpmd_shard_map_loop_reduce.cc:137-147, and of the splice at :234-301). The
// lowering can then fuse either one into the tensor-core GEMM next to it.
// ---------------------------------------------------------------------------
namespace {

// `to` equals `from` except that dimension *dim additionally carries exactly `axes` (appended
// after the axes it already has, i.e. every `from` tile is cut into |axes| consecutive parts).
bool IsScatterOf(const ShardedShape& from, const ShardedShape& to, const std::vector<int>& axes, int* dim) {
  if (from.mesh_dims != to.mesh_dims || from.rank() != to.rank() || axes.empty()) return false;
  int found = -1;
  for (int d = 0; d < from.rank(); ++d) {
    if (from.dim_axes[d] == to.dim_axes[d]) continue;
    if (found >= 0) return false;
    std::vector<int> want = from.dim_axes[d];
    want.insert(want.end(), axes.begin(), axes.end());
    if (to.dim_axes[d] != want) return false;
    found = d;
  }
  if (found < 0) return false;
  for (int d = 0; d < from.rank(); ++d)
    for (int a : from.dim_axes[d])
      if (std::find(axes.begin(), axes.end(), a) != axes.end()) return false;
  *dim = found;
  return true;
}

std::vector<int> IntList(const std::string& json) {
  std::vector<int> out;
  for (auto v : Json::parse(json).as_int_vector()) out.push_back(static_cast<int>(v));
  return out;
}

}  // namespace

bool ReduceScatterCreator(CompileState& s) {
  Graph& g = *s.graph;
  const auto users = g.ComputeUsers();
  std::set<int> graph_outputs(g.outputs.begin(), g.outputs.end());
  int scatters = 0, gathers = 0;
  for (int id : std::vector<int>(g.order)) {
    Node& n = g.node(id);
    if (n.dead) continue;
    if (n.op == "mm.spmd_reshard" && !n.attrs.count("gather_dim")) {
      // pure all-gather: the target drops trailing mesh axes of one dimension
      const ShardedShape from = ShardedShape::FromJson(Json::parse(n.attrs.at("from")));
      const ShardedShape to = ShardedShape::FromJson(Json::parse(n.attrs.at("to")));
      if (from.mesh_dims == to.mesh_dims && from.rank() == to.rank()) {
        int dim = -1;
        bool ok = true;
        std::vector<int> dropped;
        for (int d = 0; d < from.rank() && ok; ++d) {
          if (from.dim_axes[d] == to.dim_axes[d]) continue;
          if (dim >= 0 || to.dim_axes[d].size() >= from.dim_axes[d].size()) { ok = false; break; }
          for (size_t k = 0; k < to.dim_axes[d].size(); ++k) ok = ok && to.dim_axes[d][k] == from.dim_axes[d][k];
          dropped.assign(from.dim_axes[d].begin() + to.dim_axes[d].size(), from.dim_axes[d].end());
          dim = d;
        }
        if (ok && dim >= 0) {
          Json axes = Json::array();
          for (int a : dropped) axes.push(Json::number(a));
          n.attrs["gather_dim"] = std::to_string(dim);
          n.attrs["gather_axes"] = axes.dump();
          ++gathers;
        }
      }
      continue;
    }
    if (n.op != "mm.all_reduce") continue;
    const int out = n.outputs[0];
    if (graph_outputs.count(out) || !g.value(out).has_sharding) continue;
    const std::vector<int> axes = IntList(n.Attr("axes", "[]"));
    const ShardedShape from = g.value(out).sharding;
    // (a) the only reader is a local slice of the reduced value, in the same task
    if (users[out].size() == 1) {
      Node& u = g.node(users[out][0]);
      if (u.op == "mm.spmd_reshard" && u.task == n.task && !u.dead) {
        const ShardedShape to = ShardedShape::FromJson(Json::parse(u.attrs.at("to")));
        int dim = -1;
        if (IsScatterOf(from, to, axes, &dim)) {
          n.op = "mm.reduce_scatter";
          n.attrs["dim"] = std::to_string(dim);
          n.attrs["from"] = from.ToJson().dump();
          n.attrs["to"] = to.ToJson().dump();
          g.value(out).sharding = to;
          const int sliced = u.outputs[0];
          g.value(out).axes = g.value(sliced).axes;
          g.value(out).has_axes = g.value(sliced).has_axes;
          g.value(out).axes_logical = g.value(sliced).axes_logical;
          g.ReplaceAllUses(sliced, out);
          u.dead = true;
          ++scatters;
          continue;
        }
      }
    }
    // (b) a reduction that runs once per step in a task of its own (a hoisted gradient sum) and
    // whose readers, in other tasks, all ask for the same finer layout: the FSDP case, where
    // every data-parallel rank only needs the gradient of the parameter shard it owns
    if (n.Attr("hoisted") == "1" && !users[out].empty()) {
      const ShardedShape* want = nullptr;
      bool same = true;
      for (int u : users[out]) {
        const Node& un = g.node(u);
        if (un.task == n.task) { same = false; break; }
        const ShardedShape* w = InputShardingOf(s, un.task, out);
        if (!w) { same = false; break; }
        if (want && !(*want == *w)) { same = false; break; }
        want = w;
      }
      int dim = -1;
      if (same && want && IsScatterOf(from, *want, axes, &dim)) {
        n.op = "mm.reduce_scatter";
        n.attrs["dim"] = std::to_string(dim);
        n.attrs["from"] = from.ToJson().dump();
        n.attrs["to"] = want->ToJson().dump();
        g.value(out).sharding = *want;
        ++scatters;
        continue;
      }
      // (c) the readers take the reduced value as it is and slice it themselves, all to the same
      // finer layout (the reader's task had already settled on the coarse layout when the slice
      // was inserted): reduce-scatter here, and the slices become the identity
      bool all_slices = true;
      std::string to_json;
      for (int u : users[out]) {
        const Node& un = g.node(u);
        if (un.dead || un.op != "mm.spmd_reshard" || un.task == n.task) { all_slices = false; break; }
        if (to_json.empty()) to_json = un.attrs.at("to");
        else if (to_json != un.attrs.at("to")) { all_slices = false; break; }
      }
      if (all_slices && !to_json.empty()) {
        const ShardedShape to = ShardedShape::FromJson(Json::parse(to_json));
        if (IsScatterOf(from, to, axes, &dim)) {
          n.op = "mm.reduce_scatter";
          n.attrs["dim"] = std::to_string(dim);
          n.attrs["from"] = from.ToJson().dump();
          n.attrs["to"] = to.ToJson().dump();
          g.value(out).sharding = to;
          for (int u : std::vector<int>(users[out])) {
            Node& un = g.node(u);
            SetInputSharding(s, un.task, out, to);
            g.ReplaceAllUses(un.outputs[0], out);
            un.dead = true;
          }
          ++scatters;
        }
      }
    }
  }
  if (!scatters && !gathers) return false;
  if (scatters) {
    std::vector<int> keep;
    for (int id : g.order) if (!g.node(id).dead) keep.push_back(id);
    g.order = keep;
    for (auto& grp : s.groups) {
      std::vector<int> nodes;
      for (int id : grp.nodes) if (!g.node(id).dead) nodes.push_back(id);
      grp.nodes = nodes;
    }
  }
  s.Note("collective folding: " + std::to_string(scatters) + " reduce-scatters, " + std::to_string(gathers) +
         " all-gathers");
  return true;
}

// ---------------------------------------------------------------------------
// Hoist reductions of gradient accumulators out of the loop
// (src/pjrt_client/mpmd_hoist_shard_map_reduce.cc:49-189): an all-reduce whose only
// consumer is the loop-carried sum runs once after the loop on the accumulated value.
// ---------------------------------------------------------------------------
bool HoistShardMapReduce(CompileState& s) {
  Graph& g = *s.graph;
  const auto users = g.ComputeUsers();
  bool changed = false;
  for (int id : std::vector<int>(g.order)) {
    Node& ar = g.node(id);
    if (ar.dead || ar.op != "mm.all_reduce" || ar.loop < 0) continue;
    // The reduced value must end in exactly one microbatch accumulator, directly or through
    // view-like operators (the detach autograd puts on a returned loss); any other user may
    // only look at its shape (the ones_like that seeds the backward pass).
    const auto& us = users[ar.outputs[0]];
    int acc_id = -1, chain_head = -1;
    std::vector<int> shape_only;
    bool ok = !us.empty();
    for (int u : us) {
      const Node& un = g.node(u);
      if (un.op == "mm.accumulate" && acc_id < 0) {
        acc_id = u;
      } else if (un.op == "aten.ones_like.default" || un.op == "aten.zeros_like.default" ||
                 un.op == "aten.empty_like.default") {
        shape_only.push_back(u);
      } else if (IsAliasOp(un) && acc_id < 0 && un.loop == ar.loop) {
        int cur = u;
        while (true) {   // follow the chain of single-user views down to the accumulator
          const auto& cu = users[g.node(cur).outputs[0]];
          if (cu.size() != 1) { ok = false; break; }
          const Node& next = g.node(cu[0]);
          if (next.op == "mm.accumulate") { acc_id = cu[0]; chain_head = u; break; }
          if (!IsAliasOp(next) || next.loop != ar.loop) { ok = false; break; }
          cur = cu[0];
        }
      } else {
        ok = false;
      }
      if (!ok) break;
    }
    if (!ok || acc_id < 0) continue;
    // accumulate the partial value; reduce its sum once, after the loop
    const int partial = ar.inputs[0];
    if (chain_head >= 0) {
      for (int& in : g.node(chain_head).inputs) if (in == ar.outputs[0]) in = partial;
    } else {
      g.node(acc_id).inputs[0] = partial;
    }
    for (int u : shape_only)
      for (int& in : g.node(u).inputs) if (in == ar.outputs[0]) in = partial;
    const int acc_out = g.node(acc_id).outputs[0];
    if (s.config.remove_hoisted_reduces) {  // performance upper-bound experiment: drop it entirely
      ar.dead = true;
      changed = true;
      continue;
    }
    const std::map<std::string, std::string> ar_attrs = ar.attrs;
    const std::string acc_color = g.node(acc_id).color;
    const bool acc_backprop = g.node(acc_id).backprop;
    const int rid = g.AddNode("mm.all_reduce", {acc_out}, {g.value(acc_out).shape}, {g.value(acc_out).dtype}, ar_attrs);
    Node& rn = g.node(rid);
    rn.color = acc_color;
    rn.loop = -1;
    rn.backprop = acc_backprop;
    rn.attrs["hoisted"] = "1";
    g.value(rn.outputs[0]).sharding = g.value(acc_out).sharding;
    g.value(rn.outputs[0]).has_sharding = g.value(acc_out).has_sharding;
    const int reduced = rn.outputs[0];
    for (auto& m : g.nodes) {
      if (m.dead || m.id == rid) continue;
      for (int& in : m.inputs) if (in == acc_out) in = reduced;
    }
    for (int& out : g.outputs) if (out == acc_out) out = reduced;
    // tasks that asked for the accumulated value in some layout now read the reduced one
    {
      auto& table = TablesOf(s).input_sharding;
      std::vector<std::pair<int, ShardedShape>> moved;
      for (auto& kv : table) if (kv.first.second == acc_out) moved.emplace_back(kv.first.first, kv.second);
      for (auto& mv : moved) table[{mv.first, reduced}] = mv.second;
    }
    g.node(id).dead = true;
    changed = true;
  }
  if (changed) {
    std::vector<int> keep;
    for (int id : g.order) if (!g.node(id).dead) keep.push_back(id);
    g.order = keep;
    g.Toposort();
    s.Note("hoisted gradient reductions out of the microbatch loop");
    // hoisted reductions live after the loop: each gets a task of its own, with the colour and
    // devices of the accumulator it reduces, placed right after the last loop task
    Partition& part = *s.partition;
    for (auto& n : g.nodes) {
      if (n.dead || n.Attr("hoisted") != "1" || n.task >= 0) continue;
      const Node& src = g.node(g.value(n.inputs[0]).producer);
      TaskGroup grp;
      int max_id = 0;
      for (auto& x : s.groups) max_id = std::max(max_id, x.id + 1);
      grp.id = max_id;
      const ColorConfig& cc = part.Get(src.color);
      grp.color = part.Recolor(src.color, std::to_string(grp.id) + "." + (cc.original.empty() ? src.color : cc.original) + "_reduce");
      grp.region = 2;
      grp.nodes = {n.id};
      n.task = grp.id;
      n.color = grp.color;
      // the reduction reads the accumulator in the layout the loop tasks left it in
      if (g.value(n.inputs[0]).has_sharding) SetInputSharding(s, grp.id, n.inputs[0], g.value(n.inputs[0]).sharding);
      size_t pos = s.groups.size();
      for (size_t i = 0; i < s.groups.size(); ++i) if (s.groups[i].region == 2) { pos = i; break; }
      s.groups.insert(s.groups.begin() + pos, grp);
    }
    std::vector<int> order;
    for (auto& grp : s.groups) order.insert(order.end(), grp.nodes.begin(), grp.nodes.end());
    g.order = order;
  }
  return changed;
}

// ---------------------------------------------------------------------------
// Update splitting: the task that consumes the once-per-step gradient reductions (the
// optimizer) is cut into pieces, each holding the update operators of one bucket of
// reduced gradients, in the order in which the reductions are issued. The reductions run
// on the communication stream; with one update task the optimizer waits for the last of
// them, with pieces the update of bucket i runs under the reduction of bucket i + 1.
// Only tasks whose operators are independent of one another are cut (an optimizer whose
// per-tensor updates share an intermediate, e.g. a global gradient norm, is left whole).
// The reference gets the same overlap from its runtime's data-flow scheduling of the
// operations XLA emits per parameter (src/pjrt_client/mpmd_hoist_shard_map_reduce.cc:70-189
// hoists the reductions; nothing forces the update into one region).
// ---------------------------------------------------------------------------
bool SplitUpdateByReduction(CompileState& s) {
  Graph& g = *s.graph;
  Partition& part = *s.partition;
  // bucket size: MULTIMESH_UPDATE_BUCKET_MB (default 256; 0 keeps the update in one task), or in
  // bytes with MULTIMESH_UPDATE_BUCKET_BYTES (small models, tests)
  const int64_t bucket_bytes = GetEnvInt("MULTIMESH_UPDATE_BUCKET_BYTES", GetEnvInt("MULTIMESH_UPDATE_BUCKET_MB", 256) << 20);
  if (bucket_bytes <= 0) return false;
  bool changed = false;
  std::map<int, size_t> group_pos;
  for (size_t i = 0; i < s.groups.size(); ++i) group_pos[s.groups[i].id] = i;
  auto is_reduce_node = [&](const Node& n) { return !n.dead && n.Attr("hoisted") == "1"; };
  std::vector<TaskGroup> result;
  int next_id = 0;
  for (auto& grp : s.groups) next_id = std::max(next_id, grp.id + 1);
  for (const TaskGroup& grp : s.groups) {
    bool cut = grp.region == 2 && grp.nodes.size() >= 2;
    // every node: no operand produced inside the group; at most one reduced operand, its own
    std::vector<std::pair<size_t, int>> keyed;   // (position of the feeding reduction, node)
    std::vector<int> free_nodes;                 // nodes without a reduced operand
    std::set<int> produced;
    if (cut) for (int id : grp.nodes) for (int v : g.node(id).outputs) produced.insert(v);
    for (int id : grp.nodes) {
      if (!cut) break;
      const Node& n = g.node(id);
      if (is_reduce_node(n)) { cut = false; break; }
      size_t latest = 0;
      bool fed = false;
      for (int v : n.inputs) {
        if (produced.count(v)) { cut = false; break; }
        const int p = g.value(v).producer;
        if (p >= 0 && is_reduce_node(g.node(p))) {
          fed = true;
          latest = std::max(latest, group_pos[g.node(p).task]);
        }
      }
      if (!cut) break;
      if (fed) keyed.emplace_back(latest, id); else free_nodes.push_back(id);
    }
    if (!cut || keyed.size() < 2) { result.push_back(grp); continue; }
    std::stable_sort(keyed.begin(), keyed.end(), [](const std::pair<size_t, int>& a, const std::pair<size_t, int>& b) {
      return a.first < b.first;
    });
    // buckets by bytes of reduced input
    std::vector<std::vector<int>> pieces(1);
    int64_t filled = 0;
    for (auto& kn : keyed) {
      int64_t bytes = 0;
      for (int v : g.node(kn.second).inputs) {
        const int p = g.value(v).producer;
        if (p >= 0 && is_reduce_node(g.node(p))) {
          const Value& val = g.value(v);
          int64_t b = static_cast<int64_t>(DTypeSize(val.dtype));
          for (auto e : (val.has_sharding ? val.sharding.ShardSize() : val.shape)) b *= e;
          bytes += b;
        }
      }
      if (filled > 0 && filled + bytes > bucket_bytes) { pieces.emplace_back(); filled = 0; }
      pieces.back().push_back(kn.second);
      filled += bytes;
    }
    if (pieces.size() < 2) { result.push_back(grp); continue; }
    pieces.back().insert(pieces.back().end(), free_nodes.begin(), free_nodes.end());
    const ColorConfig& cc = part.Get(grp.color);
    const std::string base = cc.original.empty() ? grp.color : cc.original;
    // inputs with a layout on record for the whole task keep it in the piece that reads them
    std::vector<std::pair<int, ShardedShape>> layouts;
    for (auto& kv : TablesOf(s).input_sharding) if (kv.first.first == grp.id) layouts.emplace_back(kv.first.second, kv.second);
    for (size_t k = 0; k < pieces.size(); ++k) {
      TaskGroup piece = grp;
      piece.nodes = pieces[k];
      std::sort(piece.nodes.begin(), piece.nodes.end(), [&](int a, int b) {
        return std::find(grp.nodes.begin(), grp.nodes.end(), a) < std::find(grp.nodes.begin(), grp.nodes.end(), b);
      });
      if (k > 0) {
        piece.id = next_id++;
        piece.color = part.Clone(grp.color, std::to_string(piece.id) + "." + base + "_update", cc.devices);
        part.GetMutable(piece.color).original = base;
        part.GetMutable(piece.color).backprop = cc.backprop;
        part.GetMutable(piece.color).noncritical = cc.noncritical;
        std::set<int> reads;
        for (int id : piece.nodes) for (int v : g.node(id).inputs) reads.insert(v);
        for (auto& lv : layouts) if (reads.count(lv.first)) SetInputSharding(s, piece.id, lv.first, lv.second);
      }
      for (int id : piece.nodes) {
        g.node(id).task = piece.id;
        g.node(id).color = piece.color;
      }
      result.push_back(std::move(piece));
    }
    s.Note("update task " + grp.color + " cut into " + std::to_string(pieces.size()) + " pieces behind its gradient reductions");
    changed = true;
  }
  if (changed) {
    s.groups = std::move(result);
    std::vector<int> order;
    for (auto& grp : s.groups) order.insert(order.end(), grp.nodes.begin(), grp.nodes.end());
    g.order = order;
    g.Toposort();
  }
  return changed;
}

}  // namespace mmg
