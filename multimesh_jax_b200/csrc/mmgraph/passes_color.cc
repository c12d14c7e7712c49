// Op classification, graph-wide value properties, loop canonicalisation,
// task colouring and logical-axis propagation.
#include <algorithm>
#include <map>
#include <set>
#include <stdexcept>

#include "passes.h"

namespace mmg {

// ---------------------------------------------------------------------------
// Op classification
// ---------------------------------------------------------------------------
static bool StartsWith(const std::string& s, const char* p) { return s.rfind(p, 0) == 0; }
static std::string BaseOp(const std::string& op) {
  // "aten.add.Tensor" -> "aten.add"
  size_t first = op.find('.');
  if (first == std::string::npos) return op;
  size_t second = op.find('.', first + 1);
  return second == std::string::npos ? op : op.substr(0, second);
}

static const std::set<std::string>& ElementwiseOps() {
  static const std::set<std::string> s = {
      "aten.add", "aten.sub", "aten.mul", "aten.div", "aten.neg", "aten.exp", "aten.log", "aten.tanh",
      "aten.gelu", "aten.relu", "aten.silu", "aten.sigmoid", "aten.rsqrt", "aten.sqrt", "aten.pow",
      "aten.gelu_backward", "aten.threshold_backward", "aten.silu_backward", "aten.tanh_backward",
      "aten.sigmoid_backward", "aten.where", "aten.maximum", "aten.minimum", "aten.abs", "aten.clone",
      "aten._to_copy", "aten.to", "aten.masked_fill", "aten.reciprocal", "aten.square", "aten.cos",
      "aten.sin", "aten.erf", "aten.ge", "aten.gt", "aten.le", "aten.lt", "aten.eq", "aten.ne",
      "aten.zeros_like", "aten.ones_like", "aten.full_like", "aten.fill", "aten.copy", "aten.addcmul",
      "aten.addcdiv", "aten.lerp", "aten.clamp", "aten.clamp_min", "aten.clamp_max", "aten.sign",
      "aten.native_dropout", "aten.mul_", "aten.add_", "mm.copy", "mm.accumulate", "aten.lift_fresh_copy",
      "aten.nan_to_num", "aten.logical_not", "aten.logical_and", "aten.bitwise_and", "aten.isnan"};
  return s;
}
static const std::set<std::string>& AliasOps() {
  static const std::set<std::string> s = {
      "aten.view", "aten.reshape", "aten._unsafe_view", "aten.t", "aten.transpose", "aten.permute",
      "aten.unsqueeze", "aten.squeeze", "aten.expand", "aten.detach", "aten.alias", "aten.slice",
      "aten.select", "aten.narrow", "aten.flatten", "aten.contiguous", "aten.view_as", "aten.unflatten",
      "aten.lift_fresh", "aten.split", "aten.split_with_sizes", "aten.unbind", "aten.chunk"};
  return s;
}
static const std::set<std::string>& DotOps() {
  static const std::set<std::string> s = {"aten.mm", "aten.bmm", "aten.addmm", "aten.matmul", "aten.linear",
                                          "aten.baddbmm", "mm_ops.linear", "mm_ops.linear_dgrad",
                                          "mm_ops.linear_wgrad", "aten.einsum", "aten.dot", "aten.mv"};
  return s;
}
static const std::set<std::string>& ReduceOps() {
  static const std::set<std::string> s = {"aten.sum", "aten.mean", "aten.amax", "aten.amin", "aten.max",
                                          "aten.min", "aten.prod", "aten.logsumexp", "aten.var", "aten.norm"};
  return s;
}

bool IsMarker(const Node& n) { return n.op == "mm.marker.default" || n.op == "mm.marker"; }
bool IsElementwise(const Node& n) { return ElementwiseOps().count(BaseOp(n.op)) > 0; }
bool IsAliasOp(const Node& n) { return AliasOps().count(BaseOp(n.op)) > 0; }
bool IsFactory(const Node& n) { return n.inputs.empty() && !StartsWith(n.op, "mm."); }
bool IsDot(const Node& n) { return DotOps().count(BaseOp(n.op)) > 0; }
bool IsReduce(const Node& n) { return ReduceOps().count(BaseOp(n.op)) > 0; }
bool IsConvert(const Node& n) { const std::string b = BaseOp(n.op); return b == "aten._to_copy" || b == "aten.to"; }
bool IsCollective(const Node& n) {
  return n.op == "mm.all_reduce" || n.op == "mm.all_gather" || n.op == "mm.reduce_scatter" ||
         n.op == "mm.all_to_all" || n.op == "mm.spmd_reshard" || StartsWith(n.op, "mm_ops.moe_dispatch") ||
         StartsWith(n.op, "mm_ops.moe_combine") || StartsWith(n.op, "mm_ops.moe_ffn");
}
bool IsExpensive(const Node& n) {
  if (IsDot(n)) return true;
  if (StartsWith(n.op, "mm_ops.")) return true;
  const std::string b = BaseOp(n.op);
  return b == "aten._scaled_dot_product_flash_attention" || b == "aten.convolution" ||
         b == "aten._scaled_dot_product_efficient_attention" || b == "aten.scaled_dot_product_attention";
}
int64_t NodeFlops(const Graph& g, const Node& n) {
  if (n.outputs.empty()) return 0;
  const Value& out = g.value(n.outputs[0]);
  if (IsDot(n) && n.inputs.size() >= 2) {
    const Value& a = g.value(n.inputs[BaseOp(n.op) == "aten.addmm" ? 1 : 0]);
    int64_t k = a.shape.empty() ? 1 : a.shape.back();
    if (BaseOp(n.op) == "mm_ops.linear_wgrad") k = a.shape.empty() ? 1 : a.shape.front();
    return 2 * out.Elements() * k;
  }
  return out.Elements();
}

// ---------------------------------------------------------------------------
// Value properties
// ---------------------------------------------------------------------------
ValueProperties ValueProperties::Compute(const Graph& g) {
  ValueProperties p;
  const size_t n = g.nodes.size();
  p.derived_constant.assign(n, false);
  p.derived_parameter.assign(n, false);
  p.depth.assign(n, 0);
  p.topo_index.assign(n, -1);
  p.region.assign(n, 0);
  std::vector<bool> after_loop(n, false);
  int idx = 0;
  for (int id : g.order) {
    const Node& node = g.node(id);
    if (node.dead) continue;
    p.topo_index[id] = idx++;
    bool all_const = true, all_param = true;
    int depth = 0;
    bool post = false;
    for (int v : node.inputs) {
      const int prod = g.value(v).producer;
      if (prod < 0) {
        all_const = false;  // a graph input
      } else {
        all_const = all_const && p.derived_constant[prod];
        all_param = all_param && (p.derived_parameter[prod] || p.derived_constant[prod]);
        depth = std::max(depth, p.depth[prod] + 1);
        post = post || after_loop[prod] || g.node(prod).loop >= 0;
      }
    }
    const bool cheap = IsElementwise(node) || IsAliasOp(node) || IsFactory(node);
    p.derived_constant[id] = cheap && all_const && !IsMarker(node) && node.loop < 0 &&
                             node.op.rfind("mm.", 0) != 0;
    p.derived_parameter[id] = cheap && all_param && !node.inputs.empty() && !p.derived_constant[id] &&
                              node.op.rfind("mm.", 0) != 0;
    p.depth[id] = depth;
    after_loop[id] = node.loop < 0 && post;
    p.region[id] = node.loop >= 0 ? 1 : (after_loop[id] ? 2 : 0);
  }
  return p;
}

void ValidateCircularDependencies(const CompileState& s, const std::string& after_pass) {
  // Node-level order must be topological, and the quotient graph over tasks acyclic.
  const Graph& g = *s.graph;
  std::vector<int> pos(g.nodes.size(), -1);
  int i = 0;
  for (int id : g.order) pos[id] = i++;
  for (int id : g.order) {
    const Node& n = g.node(id);
    if (n.dead) continue;
    for (int v : n.inputs) {
      const int p = g.value(v).producer;
      if (p >= 0 && (g.node(p).dead || pos[p] < 0 || pos[p] >= pos[id]))
        throw std::runtime_error("circular or dangling dependency after pass " + after_pass + " at node " +
                                 std::to_string(id) + " (" + n.op + ")");
    }
  }
  if (s.groups.empty()) return;
  std::map<int, int> group_pos;
  for (size_t k = 0; k < s.groups.size(); ++k) group_pos[s.groups[k].id] = static_cast<int>(k);
  for (auto& grp : s.groups)
    for (int id : grp.nodes)
      for (int v : g.node(id).inputs) {
        const int p = g.value(v).producer;
        if (p < 0) continue;
        const int pt = g.node(p).task;
        if (pt >= 0 && pt != grp.id && group_pos[pt] > group_pos[grp.id])
          throw std::runtime_error("task-level circular dependency after pass " + after_pass + ": task " +
                                   grp.color + " reads from a later task");
      }
}

// ---------------------------------------------------------------------------
// Output copies
// ---------------------------------------------------------------------------
static int InsertCopy(Graph& g, int value, const Node* like) {
  const Value v = g.value(value);
  // AddNode may reallocate the node table: copy what is needed from `like` first
  const std::string color = like ? like->color : "";
  const std::string scope = like ? like->scope : "";
  const int loop = like ? like->loop : -1;
  int id = g.AddNode("mm.copy", {value}, {v.shape}, {v.dtype});
  g.node(id).color = color;
  g.node(id).scope = scope;
  g.node(id).loop = loop;
  return g.node(id).outputs[0];
}

bool ConstantOutputCopy(CompileState& s) {
  Graph& g = *s.graph;
  ValueProperties props = ValueProperties::Compute(g);
  bool changed = false;
  for (size_t i = 0; i < g.outputs.size(); ++i) {
    const int v = g.outputs[i];
    const int p = g.value(v).producer;
    // outputs that are inputs, constants or pure views of inputs must own a buffer
    bool needs = p < 0 || props.derived_constant[p];
    if (!needs && p >= 0 && IsAliasOp(g.node(p))) {
      int cur = v;
      while (g.value(cur).producer >= 0 && IsAliasOp(g.node(g.value(cur).producer)))
        cur = g.node(g.value(cur).producer).inputs[0];
      needs = g.value(cur).producer < 0;
    }
    if (needs) {
      g.outputs[i] = InsertCopy(g, v, p >= 0 ? &g.node(p) : nullptr);
      changed = true;
    }
  }
  if (changed) g.Toposort();
  return changed;
}

bool RepeatedOutputCopy(CompileState& s) {
  Graph& g = *s.graph;
  std::set<int> seen;
  bool changed = false;
  for (size_t i = 0; i < g.outputs.size(); ++i) {
    const int v = g.outputs[i];
    if (seen.insert(v).second) continue;
    const int p = g.value(v).producer;
    g.outputs[i] = InsertCopy(g, v, p >= 0 ? &g.node(p) : nullptr);
    changed = true;
  }
  if (changed) g.Toposort();
  return changed;
}

// ---------------------------------------------------------------------------
// Microbatch loop canonicalisation
// ---------------------------------------------------------------------------
bool MicrobatchLoopCanonicalizer(CompileState& s) {
  Graph& g = *s.graph;
  bool changed = false;
  std::set<int> loops;
  for (auto& n : g.nodes) {
    if (n.dead) continue;
    if (n.op == "mm.microbatch_slice.default") {
      n.op = "mm.dynamic_slice";  // offset supplied by the runtime as a host scalar
      const Json args = Json::parse(n.Attr("args", "[]"));
      n.attrs["dim"] = std::to_string(args.arr.at(0).as_int());
      n.attrs["size"] = std::to_string(args.arr.at(1).as_int());
      n.loop = static_cast<int>(args.arr.at(2).as_int());
      loops.insert(n.loop);
      changed = true;
    } else if (n.op == "mm.microbatch_out.default") {
      n.op = "mm.accumulate";  // value after the loop = sum over iterations
      const Json args = Json::parse(n.Attr("args", "[]"));
      n.loop = static_cast<int>(args.arr.at(0).as_int());
      loops.insert(n.loop);
      changed = true;
    }
  }
  if (loops.size() > 1) throw std::runtime_error("only one microbatch loop per step is supported");
  for (int l : loops) {
    bool found = false;
    for (auto& c : g.loops) found = found || c.id == l;
    if (!found) throw std::runtime_error("microbatch loop without a configuration record");
  }
  // A loop value may leave the loop only through an accumulate node.
  for (auto& n : g.nodes) {
    if (n.dead || n.loop >= 0) continue;
    for (int v : n.inputs) {
      const int p = g.value(v).producer;
      if (p >= 0 && g.node(p).loop >= 0 && g.node(p).op != "mm.accumulate")
        throw std::runtime_error("value produced inside the microbatch loop is used outside of it (node " +
                                 n.op + "); only summed outputs may leave the loop");
    }
  }
  for (int v : g.outputs) {
    const int p = g.value(v).producer;
    if (p >= 0 && g.node(p).loop >= 0 && g.node(p).op != "mm.accumulate")
      throw std::runtime_error("a microbatch loop value is returned without accumulation");
  }
  return changed;
}

// Loop-carried sums that nobody reads after the loop (a gradient the optimizer ignores, an
// auxiliary output the caller drops) are removed together with the loop work that only fed
// them (src/pjrt_client/mpmd_unused_loop_output_remover.cc:39). It runs after colouring, as
// in the reference: colouring may have cloned or rewired users, so an accumulator that had a
// reader at capture time can be dead by now.
bool UnusedLoopOutputRemover(CompileState& s) {
  Graph& g = *s.graph;
  const auto users = g.ComputeUsers();
  std::set<int> outputs(g.outputs.begin(), g.outputs.end());
  int removed_outputs = 0;
  for (auto& n : g.nodes) {
    if (n.dead || n.op != "mm.accumulate" || n.loop < 0) continue;
    bool used = false;
    for (int o : n.outputs) used = used || outputs.count(o) || !users[o].empty();
    if (used) continue;
    n.dead = true;
    ++removed_outputs;
  }
  if (!removed_outputs) return false;
  std::vector<int> keep;
  for (int id : g.order) if (!g.node(id).dead) keep.push_back(id);
  g.order = keep;
  const int swept = g.DeadCodeElimination();
  s.log.push_back("unused_loop_output_remover: dropped " + std::to_string(removed_outputs) + " loop outputs and " +
                  std::to_string(swept) + " operators that only fed them");
  return true;
}

bool SimpleLoopIncrementColoring(CompileState& s) {
  if (!s.config.loop_increment_color) return false;
  Graph& g = *s.graph;
  bool changed = false;
  TaskOptions opts;
  opts.name = Partition::kLoopIncrementColor;
  for (auto& n : g.nodes) {
    if (n.dead || n.loop < 0 || !n.color.empty()) continue;
    if (n.scope.find("loop_increment") == std::string::npos) continue;
    if (!s.partition->Has(opts.name)) s.partition->Add(opts, false);
    n.color = opts.name;
    changed = true;
  }
  return changed;
}

// ---------------------------------------------------------------------------
// Colouring
// ---------------------------------------------------------------------------
static void ApplyAssignedColors(CompileState& s) {
  Graph& g = *s.graph;
  Partition& part = *s.partition;
  for (int id : g.order) {
    Node& n = g.node(id);
    if (n.dead || !n.color.empty()) continue;
    if (!n.explicit_task.empty()) {
      TaskOptions opts = TaskOptions::FromJson(Json::parse(n.explicit_task));
      std::string name = opts.name + (n.backprop ? "_bwd" : "");
      opts.name = name;
      n.color = part.Add(opts, n.backprop).name;
      continue;
    }
    std::string c = part.ComputeScopeColor(n.scope, n.backprop);
    if (!c.empty()) n.color = c;
  }
}

static int64_t EdgeWeight(const Graph& g, const Node& n, int value) {
  // bytes moved if the edge is cut; a broadcast is weighed by its (small) operand
  (void)n;
  return std::max<int64_t>(1, g.value(value).Bytes());
}

bool Coloring(CompileState& s) {
  Graph& g = *s.graph;
  ApplyAssignedColors(s);
  const ValueProperties props = ValueProperties::Compute(g);
  const auto users = g.ComputeUsers();
  auto votes = [&](int id) { return !props.derived_constant[id] && !props.derived_parameter[id]; };
  const std::string prio = s.config.color_propagation_priority;

  // (1) inside the loop body: forward, favouring the most recent coloured operand; then backward.
  //     A node of the backward pass takes its colour only from operands whose colour itself comes
  //     from the backward pass (a gradient), never from a saved forward value: otherwise an
  //     activation derivative written outside every scope would land in the forward task of its
  //     layer and split the backward task around it.
  std::vector<char> from_bwd(g.nodes.size(), 0);
  for (int id : g.order) {
    const Node& n = g.node(id);
    if (!n.dead && n.backprop && !n.color.empty()) from_bwd[id] = 1;
  }
  for (int id : g.order) {
    Node& n = g.node(id);
    if (n.dead || n.loop < 0 || !n.color.empty() || !votes(id)) continue;
    int best = -1;
    for (int v : n.inputs) {
      const int p = g.value(v).producer;
      if (p < 0 || g.node(p).loop < 0 || g.node(p).color.empty()) continue;
      if (n.backprop && !from_bwd[p]) continue;
      if (best < 0 || props.topo_index[p] > props.topo_index[best]) best = p;
    }
    if (best >= 0) {
      n.color = g.node(best).color;
      from_bwd[id] = from_bwd[best];
    }
  }
  for (auto it = g.order.rbegin(); it != g.order.rend(); ++it) {
    Node& n = g.node(*it);
    if (n.dead || n.loop < 0 || !n.color.empty() || !votes(*it)) continue;
    int best = -1;
    for (int o : n.outputs)
      for (int u : users[o]) {
        if (g.node(u).loop < 0 || g.node(u).color.empty()) continue;
        if (best < 0 || props.topo_index[u] < props.topo_index[best]) best = u;
      }
    if (best >= 0) {
      n.color = g.node(best).color;
      from_bwd[*it] = from_bwd[best];
    }
  }

  // (2) neighbour voting, three widening filters, to a fixed point
  auto passes_filter = [&](const Node& n, int level) {
    if (level >= 2) return true;
    if (level == 1) {
      for (int o : n.outputs) if (!g.value(o).shape.empty()) return true;
      return false;
    }
    return IsElementwise(n) || IsReduce(n) || IsAliasOp(n) || n.op == "mm.dynamic_slice" || IsMarker(n);
  };
  for (int level = 0; level < 3; ++level) {
    bool changed = true;
    while (changed) {
      changed = false;
      for (int id : g.order) {
        Node& n = g.node(id);
        if (n.dead || !n.color.empty() || !votes(id) || !passes_filter(n, level)) continue;
        std::map<std::string, double> score;
        auto vote = [&](int neighbour, int via_value) {
          const Node& m = g.node(neighbour);
          if (m.color.empty()) return;
          // a loop node is never coloured from outside the loop (the reverse is fine: work that
          // consumes a summed gradient runs where that gradient lives)
          if (n.loop >= 0 && m.loop < 0) return;
          double w = 1;
          if (prio == "WEIGHT") w = static_cast<double>(EdgeWeight(g, n, via_value));
          else if (prio == "DEPTH") w = 1.0 + props.depth[neighbour];
          else w = 1.0 / (1.0 + std::abs(props.topo_index[neighbour] - props.topo_index[id]));
          score[m.color] += w;
        };
        for (int v : n.inputs) {
          const int p = g.value(v).producer;
          if (p >= 0) vote(p, v);
        }
        for (int o : n.outputs) for (int u : users[o]) vote(u, o);
        if (score.empty()) continue;
        std::string best;
        double best_w = -1;
        for (auto& kv : score) if (kv.second > best_w) { best_w = kv.second; best = kv.first; }
        n.color = best;
        changed = true;
      }
    }
  }

  // (3) whatever is still uncoloured and feeds an output (or nothing) gets the global colour,
  //     then colours backwards.
  for (auto it = g.order.rbegin(); it != g.order.rend(); ++it) {
    Node& n = g.node(*it);
    if (n.dead || !n.color.empty() || !votes(*it)) continue;
    std::string c;
    for (int o : n.outputs) for (int u : users[o]) if (c.empty() && !g.node(u).color.empty() &&
                                                       !(n.loop >= 0 && g.node(u).loop < 0)) c = g.node(u).color;
    n.color = c.empty() ? Partition::kGlobalColor : c;
  }
  return true;
}

// ---------------------------------------------------------------------------
// Logical sharding propagation
// ---------------------------------------------------------------------------
static void SetAxes(Value& v, const std::vector<std::vector<std::string>>& axes, bool logical) {
  if (v.has_axes) return;  // first annotation wins
  if (axes.size() != v.shape.size()) return;
  v.axes = axes;
  v.has_axes = true;
  v.axes_logical = logical;
}

bool LogicalShardingPropagation(CompileState& s) {
  Graph& g = *s.graph;
  bool changed = false;
  // (1) consume AutoSharding markers: annotate operand and result, then drop the marker
  for (int id : std::vector<int>(g.order)) {
    Node& n = g.node(id);
    if (n.dead || !IsMarker(n)) continue;
    const Json args = Json::parse(n.Attr("args", "[]"));
    const std::string kind = args.arr.size() > 0 ? args.arr[0].str : "";
    const std::string payload = args.arr.size() > 1 ? args.arr[1].str : "";
    if (kind == "AutoSharding") {
      const Json p = Json::parse(payload);
      std::vector<std::vector<std::string>> axes;
      for (auto& d : p.at("axes").arr) axes.push_back(d.as_string_vector());
      const bool logical = !p.has("logical") || p.at("logical").as_bool();
      SetAxes(g.value(n.inputs[0]), axes, logical);
    }
    if (kind == "Relayout") {
      // a layout change point: the node stays (as an identity whose result has the given
      // layout while its operand keeps its own), so the lowering gathers or slices here
      const Json p = Json::parse(payload);
      std::vector<std::vector<std::string>> axes;
      for (auto& d : p.at("axes").arr) axes.push_back(d.as_string_vector());
      const bool logical = !p.has("logical") || p.at("logical").as_bool();
      SetAxes(g.value(n.outputs[0]), axes, logical);
      n.op = "mm.relayout";
      changed = true;
      continue;
    }
    // every marker is an identity: forward its operand and delete it
    g.ReplaceAllUses(n.outputs[0], n.inputs[0]);
    n.dead = true;
    changed = true;
  }
  if (changed) {
    std::vector<int> keep;
    for (int id : g.order) if (!g.node(id).dead) keep.push_back(id);
    g.order = keep;
  }
  // (2) push names through aliases / elementwise ops and the dot rule, to a fixed point
  bool progress = true;
  int rounds = 0;
  while (progress && rounds++ < 8) {
    progress = false;
    for (int id : g.order) {
      Node& n = g.node(id);
      if (n.dead || n.outputs.empty()) continue;
      Value& out = g.value(n.outputs[0]);
      if (IsElementwise(n) || IsConvert(n) || n.op == "mm.accumulate" || n.op == "aten.detach.default") {
        // same-shape operands and result share names (both directions)
        for (int v : n.inputs) {
          Value& in = g.value(v);
          if (in.shape != out.shape) continue;
          if (in.has_axes && !out.has_axes) { SetAxes(out, in.axes, in.axes_logical); progress = true; }
          if (out.has_axes && !in.has_axes) { SetAxes(in, out.axes, out.axes_logical); progress = true; }
        }
      } else if (n.attrs.count("shard_rule")) {
        // Operators that describe their index structure: a result dimension inherits the
        // names of the operand dimensions that carry the same index (right operand first,
        // as in the dot rule below); a name is never used twice in one tensor.
        const Json rule = Json::parse(n.attrs.at("shard_rule"));
        const int nin = static_cast<int>(n.inputs.size());
        for (size_t o = 0; o < n.outputs.size(); ++o) {
          Value& ov = g.value(n.outputs[o]);
          if (ov.has_axes) continue;
          std::vector<std::vector<std::string>> axes(ov.shape.size());
          std::set<std::string> used;
          bool any = false, logical = true;
          for (auto& c : rule.at("classes").arr) {
            int out_dim = -1;
            for (auto& m : c.at("members").arr)
              if (m.arr[0].as_int() == nin + static_cast<int>(o)) out_dim = static_cast<int>(m.arr[1].as_int());
            if (out_dim < 0 || out_dim >= static_cast<int>(axes.size())) continue;
            for (int pass = nin - 1; pass >= 0; --pass)
              for (auto& m : c.at("members").arr) {
                if (m.arr[0].as_int() != pass) continue;
                const Value& iv = g.value(n.inputs[pass]);
                const int d = static_cast<int>(m.arr[1].as_int());
                if (!iv.has_axes || d >= static_cast<int>(iv.axes.size())) continue;
                for (auto& a : iv.axes[d]) if (used.insert(a).second) { axes[out_dim].push_back(a); any = true; }
                logical = iv.axes_logical;
              }
          }
          if (any) { SetAxes(ov, axes, logical); progress = true; }
        }
      } else if (IsDot(n) && n.inputs.size() >= 2 && !out.has_axes) {
        // Dot rule: result names come from the right operand's free dims first, then the
        // left operand's; a name is never used twice
        // (src/pjrt_client/mpmd_logical_sharding_propagation.cc:91-175).
        const std::string b = BaseOp(n.op);
        const int ai = b == "aten.addmm" ? 1 : 0;
        const Value& lhs = g.value(n.inputs[ai]);
        const Value& rhs = g.value(n.inputs[ai + 1]);
        if (!(lhs.has_axes || rhs.has_axes) || out.shape.size() < 2) continue;
        std::vector<std::vector<std::string>> axes(out.shape.size());
        std::set<std::string> used;
        auto take = [&](const std::vector<std::string>& names, size_t dim) {
          for (auto& a : names) if (used.insert(a).second) axes[dim].push_back(a);
        };
        const size_t r = out.shape.size();
        // result dim r-1 <- rhs free dim; result dims 0..r-2 <- lhs leading dims
        if (rhs.has_axes) {
          size_t free_dim = b == "mm_ops.linear" ? 0 : rhs.shape.size() - 1;
          if (b == "mm_ops.linear_dgrad") free_dim = 1;
          if (free_dim < rhs.axes.size()) take(rhs.axes[free_dim], r - 1);
        }
        if (lhs.has_axes)
          for (size_t d = 0; d + 1 < r && d < lhs.axes.size(); ++d) take(lhs.axes[d], d);
        bool any = false;
        for (auto& a : axes) any = any || !a.empty();
        if (any) { SetAxes(out, axes, lhs.has_axes ? lhs.axes_logical : rhs.axes_logical); progress = true; }
      }
    }
  }
  return changed;
}

// ---------------------------------------------------------------------------
// Loop-invariant convert hoisting and parameter replication
// ---------------------------------------------------------------------------
bool HoistLoopConvert(CompileState& s) {
  if (!s.config.hoist_loop_convert) return false;
  Graph& g = *s.graph;
  bool changed = false;
  for (int id : g.order) {
    Node& n = g.node(id);
    if (n.dead || n.loop < 0 || n.op == "mm.dynamic_slice" || n.op == "mm.accumulate") continue;
    if (!(IsConvert(n) || IsAliasOp(n))) continue;
    bool invariant = !n.inputs.empty();
    for (int v : n.inputs) {
      const int p = g.value(v).producer;
      invariant = invariant && (p < 0 || g.node(p).loop < 0);
    }
    if (invariant) {
      n.loop = -1;  // cast weights once per step, not once per microbatch
      if (s.config.zero_arguments && IsConvert(n)) n.attrs["zero_result"] = "1";
      changed = true;
    }
  }
  return changed;
}

bool ParameterReplication(CompileState& s) {
  const int64_t cutoff = s.config.replicated_parameter_num_elements_cutoff;
  if (cutoff <= 0) return false;
  Graph& g = *s.graph;
  bool changed = false;
  for (int v : g.inputs) {
    Value& val = g.value(v);
    if (val.Elements() <= cutoff && val.has_axes) {
      for (auto& a : val.axes) a.clear();  // explicit "replicated" annotation
      changed = true;
    }
  }
  return changed;
}

ShardedShape DefaultSharding(const Value& v, const ColorConfig& c) {
  ShardedShape s = ShardedShape::Replicated(v.dtype, v.shape, c.devices);
  s.mesh_dims = c.options.dims.empty() ? std::vector<int>{c.devices.n} : c.options.dims;
  return s;
}

}  // namespace mmg
