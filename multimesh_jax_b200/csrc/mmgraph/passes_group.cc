// Grouping coloured nodes into tasks, fusing tasks, and the recolouring
// optimisations that move work between tasks.
#include <algorithm>
#include <functional>
#include <map>
#include <queue>
#include <set>
#include <stdexcept>
#include <tuple>

#include "passes.h"

namespace mmg {

// ---------------------------------------------------------------------------
// Replicate uncoloured producers into every consumer colour
// (src/pjrt_client/mpmd_computation_grouper.cc:72-88: uncoloured, constant-derived
// and parameter-derived instructions are recomputed, not communicated).
// ---------------------------------------------------------------------------
static int CloneNode(Graph& g, int id, const std::string& color, int loop) {
  const Node src = g.node(id);
  std::vector<std::vector<int64_t>> shapes;
  std::vector<DType> dtypes;
  for (int o : src.outputs) {
    shapes.push_back(g.value(o).shape);
    dtypes.push_back(g.value(o).dtype);
  }
  const int nid = g.AddNode(src.op, src.inputs, shapes, dtypes, src.attrs);
  Node& n = g.node(nid);
  n.scope = src.scope;
  n.backprop = src.backprop;
  n.loop = loop;
  n.color = color;
  n.attrs["cloned_from"] = std::to_string(id);
  for (size_t i = 0; i < src.outputs.size(); ++i) {
    Value& nv = g.value(n.outputs[i]);
    const Value& ov = g.value(src.outputs[i]);
    nv.axes = ov.axes;
    nv.has_axes = ov.has_axes;
    nv.axes_logical = ov.axes_logical;
  }
  return nid;
}

bool ReplicateUncolored(CompileState& s) {
  Graph& g = *s.graph;
  bool changed = false;
  // reverse topological order so that chains of uncoloured nodes are cloned consumer-first
  std::vector<int> rev(g.order.rbegin(), g.order.rend());
  for (int id : rev) {
    if (g.node(id).dead || !g.node(id).color.empty()) continue;
    // consumers grouped by (colour, loop)
    std::map<std::pair<std::string, int>, std::vector<int>> by_color;
    bool feeds_output = false;
    for (int o : g.node(id).outputs) {
      for (int out : g.outputs) feeds_output = feeds_output || out == o;
    }
    for (auto& m : g.nodes) {
      if (m.dead || m.id == id) continue;
      bool uses = false;
      for (int v : m.inputs) for (int o : g.node(id).outputs) uses = uses || v == o;
      if (uses) by_color[{m.color, m.loop}].push_back(m.id);
    }
    if (by_color.empty() || feeds_output) {
      g.node(id).color = by_color.empty() ? Partition::kGlobalColor : by_color.begin()->first.first;
      if (feeds_output) g.node(id).color = Partition::kGlobalColor;
      changed = true;
      continue;
    }
    bool first = true;
    for (auto& kv : by_color) {
      if (kv.first.first.empty()) continue;  // consumer itself still uncoloured: handled when visited
      if (first) {
        g.node(id).color = kv.first.first;
        g.node(id).loop = kv.first.second;
        first = false;
        continue;
      }
      const int clone = CloneNode(g, id, kv.first.first, kv.first.second);
      for (int user : kv.second) {
        Node& u = g.node(user);
        for (int& v : u.inputs)
          for (size_t i = 0; i < g.node(id).outputs.size(); ++i)
            if (v == g.node(id).outputs[i]) v = g.node(clone).outputs[i];
      }
    }
    if (first) g.node(id).color = Partition::kGlobalColor;
    changed = true;
  }
  if (changed) g.Toposort();
  return changed;
}

// ---------------------------------------------------------------------------
// Grouper: colour-sticky topological order, consecutive same-colour runs = tasks
// ---------------------------------------------------------------------------
bool ComputationGrouper(CompileState& s) {
  Graph& g = *s.graph;
  g.Toposort();
  const ValueProperties props = ValueProperties::Compute(g);
  s.groups.clear();
  for (auto& n : g.nodes) n.task = -1;
  std::vector<int> new_order;
  for (int region = 0; region < 3; ++region) {
    std::vector<int> ids;
    for (int id : g.order) if (!g.node(id).dead && props.region[id] == region) ids.push_back(id);
    if (ids.empty()) continue;
    std::set<int> in_region(ids.begin(), ids.end());
    std::map<int, int> indeg;
    std::map<int, std::vector<int>> succ;
    for (int id : ids) {
      std::set<int> preds;
      for (int v : g.node(id).inputs) {
        const int p = g.value(v).producer;
        if (p >= 0 && in_region.count(p)) preds.insert(p);
      }
      indeg[id] = static_cast<int>(preds.size());
      for (int p : preds) succ[p].push_back(id);
    }
    // ready sets per colour, ordered by original topological position
    auto by_pos = [&](int a, int b) { return props.topo_index[a] < props.topo_index[b]; };
    std::map<std::string, std::set<int, decltype(by_pos)>> ready;
    auto push_ready = [&](int id) {
      auto it = ready.find(g.node(id).color);
      if (it == ready.end()) it = ready.emplace(g.node(id).color, std::set<int, decltype(by_pos)>(by_pos)).first;
      it->second.insert(id);
    };
    for (int id : ids) if (indeg[id] == 0) push_ready(id);
    std::string current;
    size_t emitted = 0;
    while (emitted < ids.size()) {
      auto cur = ready.find(current);
      if (cur == ready.end() || cur->second.empty()) {
        // switch to the colour owning the earliest ready node
        int best = -1;
        for (auto& kv : ready)
          if (!kv.second.empty() && (best < 0 || by_pos(*kv.second.begin(), best))) best = *kv.second.begin();
        if (best < 0) throw std::runtime_error("grouper: dependency cycle inside a region");
        current = g.node(best).color;
        cur = ready.find(current);
        TaskGroup grp;
        grp.id = static_cast<int>(s.groups.size());
        grp.color = current;
        grp.region = region;
        s.groups.push_back(grp);
      }
      const int id = *cur->second.begin();
      cur->second.erase(cur->second.begin());
      g.node(id).task = s.groups.back().id;
      s.groups.back().nodes.push_back(id);
      new_order.push_back(id);
      ++emitted;
      for (int nx : succ[id]) if (--indeg[nx] == 0) push_ready(nx);
    }
  }
  g.order = new_order;
  return true;
}

// ---------------------------------------------------------------------------
// Fusion of tasks that can be made adjacent
// ---------------------------------------------------------------------------
static std::vector<std::set<int>> GroupPreds(const CompileState& s) {
  const Graph& g = *s.graph;
  std::map<int, int> index;
  for (size_t i = 0; i < s.groups.size(); ++i) index[s.groups[i].id] = static_cast<int>(i);
  std::vector<std::set<int>> preds(s.groups.size());
  for (size_t i = 0; i < s.groups.size(); ++i)
    for (int id : s.groups[i].nodes)
      for (int v : g.node(id).inputs) {
        const int p = g.value(v).producer;
        if (p < 0 || g.node(p).task < 0 || g.node(p).task == s.groups[i].id) continue;
        preds[i].insert(index[g.node(p).task]);
      }
  return preds;
}

bool ComputationFusion(CompileState& s, FusionMode mode) {
  if (!s.config.use_task_fusion) return false;
  Graph& g = *s.graph;
  Partition& part = *s.partition;
  bool changed_any = false;
  bool changed = true;
  while (changed) {
    changed = false;
    const size_t n = s.groups.size();
    auto preds = GroupPreds(s);
    // reach[i] = set of groups from which i is reachable (transitive predecessors)
    std::vector<std::set<int>> reach(n);
    for (size_t i = 0; i < n; ++i)
      for (int p : preds[i]) {
        reach[i].insert(p);
        reach[i].insert(reach[p].begin(), reach[p].end());
      }
    auto match = [&](const TaskGroup& a, const TaskGroup& b) {
      if (a.region != b.region || a.noncritical != b.noncritical) return false;
      if (s.config.only_fuse_loop_tasks && a.region != 1) return false;
      const ColorConfig& ca = part.Get(a.color);
      const ColorConfig& cb = part.Get(b.color);
      switch (mode) {
        case FusionMode::kMatchingColor: return a.color == b.color;
        case FusionMode::kOriginalColor:
          // colours that descend from one user-visible task (recolouring and regrouping split it);
          // descendants always share the parent's devices, the test only guards against a table
          // that was edited by hand
          return (ca.original.empty() ? ca.name : ca.original) == (cb.original.empty() ? cb.name : cb.original) &&
                 ca.devices == cb.devices && ca.backprop == cb.backprop;
        case FusionMode::kMatchingDevices:
          return a.region == 1 && ca.devices == cb.devices && ca.backprop == cb.backprop;
      }
      return false;
    };
    for (size_t i = 0; i < n && !changed; ++i) {
      for (size_t j = i + 1; j < n && !changed; ++j) {
        if (!match(s.groups[i], s.groups[j])) continue;
        // legal iff no group strictly between depends on i and is depended on by j
        bool legal = true;
        for (size_t k = i + 1; k < j && legal; ++k)
          if ((reach[k].count(static_cast<int>(i))) && (reach[j].count(static_cast<int>(k)))) legal = false;
        if (!legal) continue;
        // Merge j into i. Groups between them that j depends on move before the merged
        // group; that is only valid if they do not depend on i (checked above).
        TaskGroup merged = s.groups[i];
        merged.nodes.insert(merged.nodes.end(), s.groups[j].nodes.begin(), s.groups[j].nodes.end());
        std::vector<TaskGroup> before, after;
        for (size_t k = i + 1; k < j; ++k)
          (reach[j].count(static_cast<int>(k)) ? before : after).push_back(s.groups[k]);
        std::vector<TaskGroup> out(s.groups.begin(), s.groups.begin() + i);
        out.insert(out.end(), before.begin(), before.end());
        out.push_back(merged);
        out.insert(out.end(), after.begin(), after.end());
        out.insert(out.end(), s.groups.begin() + j + 1, s.groups.end());
        for (int id : s.groups[j].nodes) g.node(id).task = merged.id;
        if (mode != FusionMode::kMatchingColor)
          for (int id : s.groups[j].nodes) g.node(id).color = merged.color;
        s.groups = out;
        changed = true;
        changed_any = true;
      }
    }
  }
  if (changed_any) {
    // keep node order consistent with group order; inside a merged group keep topological order
    std::vector<int> pos(g.nodes.size(), 0);
    for (size_t i = 0; i < g.order.size(); ++i) pos[g.order[i]] = static_cast<int>(i);
    std::vector<int> order;
    for (auto& grp : s.groups) {
      std::sort(grp.nodes.begin(), grp.nodes.end(), [&](int a, int b) { return pos[a] < pos[b]; });
      order.insert(order.end(), grp.nodes.begin(), grp.nodes.end());
    }
    g.order = order;
    // a merged group may now contain a consumer placed before its producer: fix with a local sort
    g.Toposort();
    std::vector<int> pos2(g.nodes.size(), 0);
    for (size_t i = 0; i < g.order.size(); ++i) pos2[g.order[i]] = static_cast<int>(i);
    order.clear();
    for (auto& grp : s.groups) {
      std::sort(grp.nodes.begin(), grp.nodes.end(), [&](int a, int b) { return pos2[a] < pos2[b]; });
      order.insert(order.end(), grp.nodes.begin(), grp.nodes.end());
    }
    g.order = order;
  }
  return changed_any;
}

bool UniquifyColors(CompileState& s) {
  Graph& g = *s.graph;
  Partition& part = *s.partition;
  int counter = 0;
  for (auto& grp : s.groups) {
    const std::string fresh = std::to_string(counter++) + "." + grp.color + (grp.region == 1 ? "_loop" : "");
    part.Recolor(grp.color, fresh);
    ColorConfig& cc = part.GetMutable(fresh);
    cc.noncritical = grp.noncritical;
    for (int id : grp.nodes) g.node(id).color = fresh;
    grp.color = fresh;
  }
  return true;
}

// ---------------------------------------------------------------------------
// Recolouring optimisations (operate on colours before the final grouping)
// ---------------------------------------------------------------------------

// Move single-consumer producer sub-trees into a later task on the same devices when
// at least two other tasks run in between (src/pjrt_client/mpmd_instruction_delay_recolor.cc:30-353):
// work that nobody needs yet should not delay the pipeline's critical path.
bool InstructionDelayRecolor(CompileState& s) {
  Graph& g = *s.graph;
  Partition& part = *s.partition;
  if (s.groups.empty()) return false;
  std::map<int, int> group_pos;
  for (size_t i = 0; i < s.groups.size(); ++i) group_pos[s.groups[i].id] = static_cast<int>(i);
  const auto users = g.ComputeUsers();
  bool changed = false;
  std::vector<int> rev(g.order.rbegin(), g.order.rend());
  for (int id : rev) {
    Node& n = g.node(id);
    if (n.dead || n.task < 0 || IsExpensive(n) || n.op.rfind("mm.", 0) == 0) continue;
    // all users in exactly one other, later task
    int user_task = -1;
    bool ok = !n.outputs.empty();
    for (int o : n.outputs) {
      for (int out : g.outputs) if (out == o) ok = false;
      for (int u : users[o]) {
        const int t = g.node(u).task;
        if (t == n.task) ok = false;
        else if (user_task < 0) user_task = t;
        else if (user_task != t) ok = false;
      }
    }
    if (!ok || user_task < 0) continue;
    if (group_pos[user_task] - group_pos[n.task] < 2) continue;
    const TaskGroup& from = s.groups[group_pos[n.task]];
    const TaskGroup& to = s.groups[group_pos[user_task]];
    if (from.region != to.region) continue;
    if (part.Get(from.color).devices != part.Get(to.color).devices) continue;
    // operands must be available to the later task anyway (inputs or values from earlier tasks)
    n.color = to.color;
    n.task = to.id;
    changed = true;
  }
  if (changed) {
    // keep the groups' member lists in step with the nodes' new tasks (in graph order)
    for (auto& grp : s.groups) grp.nodes.clear();
    for (int id : g.order) {
      const Node& n = g.node(id);
      if (n.dead || n.task < 0) continue;
      auto it = group_pos.find(n.task);
      if (it != group_pos.end()) s.groups[it->second].nodes.push_back(id);
    }
    s.Note("delay-recolor moved instructions to later tasks");
  }
  return changed;
}

// Clone cheap producer trees into the consumer's colour instead of communicating their
// result (src/pjrt_client/mpmd_argument_recompute.cc:20-336).
bool ArgumentRecompute(CompileState& s) {
  if (!s.config.argument_recompute || !s.config.enable_recomputation) return false;
  const int64_t user_cutoff = s.config.recompute_from_arguments_if_cost_less_than;
  if (user_cutoff <= 0) return false;
  Graph& g = *s.graph;
  Partition& part = *s.partition;
  bool changed = false;
  std::map<std::tuple<int, std::string, int>, int> shared_clones;
  for (int id : std::vector<int>(g.order)) {
    if (g.node(id).dead || g.node(id).color.empty()) continue;
    for (size_t ii = 0; ii < g.node(id).inputs.size(); ++ii) {
      const int v = g.node(id).inputs[ii];
      const int p = g.value(v).producer;
      if (p < 0) continue;
      const Node prod = g.node(p);  // by value: cloning below grows the node table
      if (prod.color.empty() || prod.color == g.node(id).color || prod.loop != g.node(id).loop) continue;
      // DFS the producer tree back to graph inputs
      std::vector<int> tree;
      std::set<int> seen;
      int64_t cost = 0;
      bool ok = true;
      std::function<void(int)> dfs = [&](int nid) {
        if (!ok || seen.count(nid)) return;
        seen.insert(nid);
        const Node& m = g.node(nid);
        if (IsExpensive(m) || IsCollective(m) || m.op.rfind("mm.", 0) == 0 || m.loop != prod.loop) { ok = false; return; }
        for (int o : m.outputs) cost += g.value(o).Elements();
        for (int in : m.inputs) {
          const int q = g.value(in).producer;
          if (q >= 0) dfs(q);
        }
        tree.push_back(nid);  // post-order: operands first
      };
      dfs(p);
      if (!ok) continue;
      const int64_t bytes = g.value(v).Bytes();
      const bool cross_mesh = part.Get(prod.color).devices != part.Get(g.node(id).color).devices;
      int64_t limit = std::max<int64_t>(bytes * 100, user_cutoff);
      if (cross_mesh && bytes > (8 << 20)) limit = std::max<int64_t>(limit, bytes * 1000);
      if (cost > limit) continue;
      // the tree's graph-input leaves must be cheap to have on the consumer: require that the
      // recomputation reads less than it saves when crossing meshes
      std::map<int, int> remap;  // old value -> new value
      const std::string color = g.node(id).color;
      const int loop = g.node(id).loop;
      // consumers of one colour share a single clone of the tree
      auto shared_key = std::make_tuple(v, color, loop);
      auto shared_hit = shared_clones.find(shared_key);
      if (shared_hit != shared_clones.end()) {
        g.node(id).inputs[ii] = shared_hit->second;
        changed = true;
        continue;
      }
      for (int nid : tree) {
        const int clone = CloneNode(g, nid, color, loop);
        Node& c = g.node(clone);
        for (int& in : c.inputs) { auto it = remap.find(in); if (it != remap.end()) in = it->second; }
        for (size_t k = 0; k < c.outputs.size(); ++k) remap[g.node(nid).outputs[k]] = c.outputs[k];
      }
      g.node(id).inputs[ii] = remap[v];
      shared_clones[shared_key] = remap[v];
      changed = true;
    }
  }
  if (changed) {
    g.Toposort();
    g.DeadCodeElimination();
    s.Note("argument-recompute cloned producer trees into consumer tasks");
  }
  return changed;
}

// If an instruction (through up to three unary ops) is bigger than its operands and has a
// single consumer colour on an equivalent mesh, move it to the consumer so that the smaller
// tensor is sent (src/pjrt_client/mpmd_cut_size_minimizer.cc:16-156).
bool CutSizeMinimizer(CompileState& s) {
  if (!s.config.minimize_cut_size) return false;
  Graph& g = *s.graph;
  Partition& part = *s.partition;
  const auto users = g.ComputeUsers();
  bool changed = false;
  std::vector<int> rev(g.order.rbegin(), g.order.rend());
  for (int id : rev) {
    Node& n = g.node(id);
    if (n.dead || n.color.empty() || n.outputs.size() != 1 || n.inputs.empty()) continue;
    if (IsExpensive(n) && !IsDot(n)) continue;
    if (n.op.rfind("mm.", 0) == 0) continue;
    const int out = n.outputs[0];
    bool is_output = false;
    for (int o : g.outputs) is_output = is_output || o == out;
    if (is_output) continue;
    // follow up to three unary ops of the same colour
    int tail = id;
    std::vector<int> chain = {id};
    for (int hop = 0; hop < 3; ++hop) {
      const auto& us = users[g.node(tail).outputs[0]];
      if (us.size() != 1) break;
      const Node& u = g.node(us[0]);
      if (u.color != n.color || u.inputs.size() != 1 || u.outputs.size() != 1 || IsExpensive(u)) break;
      tail = u.id;
      chain.push_back(tail);
    }
    std::string consumer_color;
    int consumer_loop = -1;
    bool single = true;
    for (int u : users[g.node(tail).outputs[0]]) {
      const Node& un = g.node(u);
      if (consumer_color.empty()) { consumer_color = un.color; consumer_loop = un.loop; }
      else if (consumer_color != un.color) single = false;
    }
    if (!single || consumer_color.empty() || consumer_color == n.color || consumer_loop != n.loop) continue;
    if (part.Get(consumer_color).devices.n != part.Get(n.color).devices.n) continue;
    int64_t operand_bytes = 0;
    for (int v : n.inputs) operand_bytes += g.value(v).Bytes();
    if (g.value(g.node(tail).outputs[0]).Bytes() <= operand_bytes) continue;
    // a contraction qualifies like anything else: with an output larger than both operands
    // together its contracted extent is tiny, so it is the result, not the math, that is heavy
    for (int c : chain) g.node(c).color = consumer_color;
    changed = true;
  }
  if (changed) s.Note("cut-size minimiser moved expanding instructions to their consumers");
  return changed;
}

// ---------------------------------------------------------------------------
// Split backward tasks into activation-gradient (critical) and weight-gradient halves
// (src/pjrt_client/mpmd_split_critical_path.cc:33-131, task_splitter.cc:35-188,
//  critical_path_finder.cc:20-71).
// ---------------------------------------------------------------------------
bool SplitCriticalPath(CompileState& s) {
  Graph& g = *s.graph;
  Partition& part = *s.partition;
  bool changed = false;
  std::map<int, int> group_pos;
  for (size_t i = 0; i < s.groups.size(); ++i) group_pos[s.groups[i].id] = static_cast<int>(i);
  const auto users = g.ComputeUsers();
  std::vector<TaskGroup> out_groups;
  int next_id = 0;
  for (auto& grp : s.groups) next_id = std::max(next_id, grp.id + 1);
  for (auto& grp : s.groups) {
    const ColorConfig& cc = part.Get(grp.color);
    if (cc.options.split_backprop.size() != 2 || !cc.backprop) { out_groups.push_back(grp); continue; }
    // critical output = the one whose first consumer task comes earliest (the activation gradient)
    int critical_value = -1, earliest = 1 << 30;
    for (int id : grp.nodes)
      for (int o : g.node(id).outputs)
        for (int u : users[o]) {
          const int t = g.node(u).task;
          if (t == grp.id || t < 0) continue;
          if (group_pos[t] < earliest) { earliest = group_pos[t]; critical_value = o; }
        }
    if (critical_value < 0) { out_groups.push_back(grp); continue; }
    // everything the critical output depends on (inside the task) is critical
    std::set<int> critical;
    std::function<void(int)> mark = [&](int nid) {
      if (critical.count(nid) || g.node(nid).task != grp.id) return;
      critical.insert(nid);
      for (int v : g.node(nid).inputs) { const int p = g.value(v).producer; if (p >= 0) mark(p); }
    };
    // every value handed to that first consumer is on the critical path (a stage boundary may
    // carry several activation gradients), not only the first one found
    for (int id : grp.nodes)
      for (int o : g.node(id).outputs)
        for (int u : users[o]) {
          const int t = g.node(u).task;
          if (t != grp.id && t >= 0 && group_pos[t] == earliest) mark(id);
        }
    mark(g.value(critical_value).producer);
    if (critical.size() == grp.nodes.size()) { out_groups.push_back(grp); continue; }
    const std::string base = cc.original.empty() ? grp.color : cc.original;
    const std::string ca = base + cc.options.split_backprop[0];
    const std::string cb = base + cc.options.split_backprop[1];
    TaskOptions oa = cc.options, ob = cc.options;
    oa.name = ca;
    ob.name = cb;
    oa.split_backprop.clear();
    ob.split_backprop.clear();
    part.Add(oa, true);
    part.Add(ob, true);
    part.GetMutable(cb).noncritical = true;
    TaskGroup a = grp, b = grp;
    a.color = ca;
    a.nodes.clear();
    b.id = next_id++;
    b.color = cb;
    b.nodes.clear();
    b.noncritical = true;
    for (int id : grp.nodes) {
      if (critical.count(id)) { a.nodes.push_back(id); g.node(id).color = ca; }
      else { b.nodes.push_back(id); g.node(id).color = cb; g.node(id).task = b.id; }
    }
    out_groups.push_back(a);
    out_groups.push_back(b);
    changed = true;
  }
  if (changed) {
    s.groups = out_groups;
    std::vector<int> order;
    for (auto& grp : s.groups) order.insert(order.end(), grp.nodes.begin(), grp.nodes.end());
    g.order = order;
    s.Note("split-critical-path separated weight-gradient work from activation gradients");
  }
  return changed;
}

bool UnusedParamOutputRemover(CompileState& s) {
  Graph& g = *s.graph;
  const int removed = g.DeadCodeElimination();
  // drop dead nodes (from this or earlier passes) from the task groups, and empty groups
  bool pruned = false;
  for (auto& grp : s.groups) {
    std::vector<int> keep;
    for (int id : grp.nodes) if (!g.node(id).dead) keep.push_back(id);
    pruned = pruned || keep.size() != grp.nodes.size();
    grp.nodes = keep;
  }
  std::vector<TaskGroup> keep_groups;
  for (auto& grp : s.groups) if (!grp.nodes.empty()) keep_groups.push_back(grp);
  pruned = pruned || keep_groups.size() != s.groups.size();
  s.groups = keep_groups;
  return removed > 0 || pruned;
}

}  // namespace mmg
