// From task groups to an executable plan: task templates, task-level loop
// unrolling, pipeline scheduling, cross-submesh reshard insertion (deduplicated
// per producer and target layout), liveness-based buffer pooling, donation
// aliasing and the final linear list of operations.
//
// Counterparts in the reference: mpmd_loop_unroll.cc:147-356 (unroll, control
// edges), mpmd_insert_reshard.cc:51-220, mpmd_buffer_scheduling_name.cc:94-229,
// mpmd_input_output_buffer_alias.cc and MpmdScheduler in mpmd_partition.cc:242-640.
// The loop is unrolled at task granularity: every iteration reuses the same
// task template (one compiled body per unique task), only its store bindings
// and scalar slice offsets differ.
#include <algorithm>
#include <map>
#include <queue>
#include <set>
#include <stdexcept>

#include "passes.h"

namespace mmg {

const ShardedShape* InputShardingOf(const CompileState& s, int group, int value);

namespace {

struct Instance {
  int group_index;  // index into s.groups
  int iteration;    // -1 outside the loop
  DeviceRange devices;
};

struct StoreKey {
  int value;
  int iteration;
  bool operator<(const StoreKey& o) const { return value != o.value ? value < o.value : iteration < o.iteration; }
};

ShardedShape OnDevices(ShardedShape s, DeviceRange devices) {
  s.devices = devices;
  int mesh = 1;
  for (int m : s.mesh_dims) mesh *= m;
  if (mesh != devices.n) {  // mesh no longer fits (loop-dependent placement keeps the size, so this is rare)
    s.mesh_dims = {devices.n};
    for (auto& a : s.dim_axes) a.clear();
  }
  return s;
}

}  // namespace

Plan BuildPlan(CompileState& s) {
  Graph& g = *s.graph;
  Partition& part = *s.partition;
  Plan plan;
  const auto users = g.ComputeUsers();
  std::set<int> graph_outputs(g.outputs.begin(), g.outputs.end());

  // ---------------------------------------------------------------- templates
  std::map<int, int> group_index;  // group id -> index
  for (size_t i = 0; i < s.groups.size(); ++i) group_index[s.groups[i].id] = static_cast<int>(i);
  for (size_t gi = 0; gi < s.groups.size(); ++gi) {
    const TaskGroup& grp = s.groups[gi];
    const ColorConfig& cc = part.Get(grp.color);
    TaskTemplate t;
    t.id = static_cast<int>(gi);
    t.name = grp.color;
    t.original_color = cc.original.empty() ? grp.color : cc.original;
    t.devices = cc.devices;
    t.mesh_dims = cc.options.dims.empty() ? std::vector<int>{cc.devices.n} : cc.options.dims;
    t.mesh_axes = cc.options.device_axes;
    t.nodes = grp.nodes;
    t.in_loop = grp.region == 1;
    t.backprop = cc.backprop;
    t.noncritical = grp.noncritical || cc.noncritical;
    std::set<int> seen_in, seen_out;
    for (int id : grp.nodes) {
      const Node& n = g.node(id);
      t.has_collectives = t.has_collectives || IsCollective(n);
      t.flops += NodeFlops(g, n);
      for (int v : n.inputs) {
        const int p = g.value(v).producer;
        if ((p < 0 || g.node(p).task != grp.id) && seen_in.insert(v).second) t.inputs.push_back(v);
      }
      for (int o : n.outputs) {
        bool external = graph_outputs.count(o) > 0;
        for (int u : users[o]) external = external || g.node(u).task != grp.id;
        if (external && seen_out.insert(o).second) t.outputs.push_back(o);
      }
    }
    plan.templates.push_back(t);
  }

  // ---------------------------------------------------------------- loop config
  LoopConfig loop;
  bool has_loop = false;
  for (auto& grp : s.groups) has_loop = has_loop || grp.region == 1;
  if (has_loop) {
    if (g.loops.empty()) throw std::runtime_error("loop tasks without a loop configuration");
    loop = g.loops[0];
  }
  const int num_iters = has_loop ? loop.num_microbatches : 0;

  // ---------------------------------------------------------------- instances
  auto devices_of = [&](int gi, int iteration) {
    const ColorConfig& cc = part.Get(s.groups[gi].color);
    if (iteration >= 0 && !cc.options.loop_dependent_devices.empty()) {
      const auto& lists = cc.options.loop_dependent_devices;
      return DeviceRange::FromList(lists[iteration % lists.size()]);
    }
    return cc.devices;
  };
  std::vector<Instance> order;  // final execution order
  std::vector<int> loop_groups;
  for (size_t gi = 0; gi < s.groups.size(); ++gi) {
    if (s.groups[gi].region == 0) order.push_back({static_cast<int>(gi), -1, devices_of(static_cast<int>(gi), -1)});
    if (s.groups[gi].region == 1) loop_groups.push_back(static_cast<int>(gi));
  }
  if (has_loop && !loop_groups.empty()) {
    // schedule input: tasks[iteration][stage]
    std::map<int, int> stage_of;  // group index -> stage
    for (size_t st = 0; st < loop_groups.size(); ++st) stage_of[loop_groups[st]] = static_cast<int>(st);
    // stage-level data dependencies inside one iteration
    std::vector<std::set<int>> stage_preds(loop_groups.size());
    for (size_t st = 0; st < loop_groups.size(); ++st)
      for (int id : s.groups[loop_groups[st]].nodes)
        for (int v : g.node(id).inputs) {
          const int p = g.value(v).producer;
          if (p < 0) continue;
          auto it = group_index.find(g.node(p).task);
          if (it == group_index.end()) continue;
          auto ps = stage_of.find(it->second);
          if (ps != stage_of.end() && ps->second != static_cast<int>(st)) stage_preds[st].insert(ps->second);
        }
    std::vector<std::vector<SchedTask>> tasks(num_iters);
    for (int it = 0; it < num_iters; ++it)
      for (size_t st = 0; st < loop_groups.size(); ++st) {
        const int gi = loop_groups[st];
        const ColorConfig& cc = part.Get(s.groups[gi].color);
        SchedTask t;
        t.iteration = it;
        t.stage = static_cast<int>(st);
        t.color = s.groups[gi].color;
        t.devices = devices_of(gi, it);
        t.noncritical = plan.templates[gi].noncritical;
        t.on_full_mesh = t.devices == part.global() && part.global().n > 1;
        t.prefetch = (cc.original.empty() ? cc.name : cc.original) == Partition::kLoopIncrementColor;
        for (int p : stage_preds[st])
          if (!plan.templates[loop_groups[p]].noncritical) t.consumes_stage = std::max(t.consumes_stage, p);
        tasks[it].push_back(t);
      }
    ScheduleResult sched = ScheduleLoops(loop, tasks);
    plan.stats["schedule"] = loop.schedule;
    if (sched.simulated_makespan > 0) plan.stats["simulated_makespan"] = std::to_string(sched.simulated_makespan);

    // linearise: data deps + iteration order per stage + control edges between consecutive
    // same-device tasks of each order
    const int S = static_cast<int>(loop_groups.size());
    auto idx = [&](int it, int st) { return it * S + st; };
    std::vector<std::set<int>> preds(num_iters * S);
    std::vector<std::pair<int, int>> prio(num_iters * S, {1 << 30, 0});
    for (int it = 0; it < num_iters; ++it)
      for (int st = 0; st < S; ++st) {
        for (int p : stage_preds[st]) preds[idx(it, st)].insert(idx(it, p));
        if (it > 0) preds[idx(it, st)].insert(idx(it - 1, st));
      }
    for (size_t o = 0; o < sched.orders.size(); ++o) {
      std::map<DeviceRange, int> last_on_devices;
      for (size_t k = 0; k < sched.orders[o].size(); ++k) {
        const auto [it, st] = sched.orders[o][k];
        const int me = idx(it, st);
        prio[me] = {static_cast<int>(k), static_cast<int>(o)};
        const DeviceRange dev = tasks[it][st].devices;
        auto last = last_on_devices.find(dev);
        if (last != last_on_devices.end() && last->second != me) preds[me].insert(last->second);
        last_on_devices[dev] = me;
      }
    }
    std::vector<int> indeg(num_iters * S, 0);
    std::vector<std::vector<int>> succ(num_iters * S);
    for (int i = 0; i < num_iters * S; ++i) {
      indeg[i] = static_cast<int>(preds[i].size());
      for (int p : preds[i]) succ[p].push_back(i);
    }
    auto cmp = [&](int a, int b) { return prio[a] != prio[b] ? prio[a] > prio[b] : a > b; };
    std::priority_queue<int, std::vector<int>, decltype(cmp)> ready(cmp);
    for (int i = 0; i < num_iters * S; ++i) if (indeg[i] == 0) ready.push(i);
    int emitted = 0;
    while (!ready.empty()) {
      const int i = ready.top();
      ready.pop();
      ++emitted;
      const int it = i / S, st = i % S;
      order.push_back({loop_groups[st], it, tasks[it][st].devices});
      for (int nx : succ[i]) if (--indeg[nx] == 0) ready.push(nx);
    }
    if (emitted != num_iters * S)
      throw std::runtime_error("the requested pipeline schedule contradicts the data dependencies of the loop body");
  }
  for (size_t gi = 0; gi < s.groups.size(); ++gi)
    if (s.groups[gi].region == 2) order.push_back({static_cast<int>(gi), -1, devices_of(static_cast<int>(gi), -1)});

  // ---------------------------------------------------------------- stores
  std::map<StoreKey, int> store_of;
  auto new_store = [&](Store::Kind kind, int index, int value, int iteration, const ShardedShape& shape) {
    Store st;
    st.id = static_cast<int>(plan.stores.size());
    st.kind = kind;
    st.index = index;
    st.value = value;
    st.iteration = iteration;
    st.shape = shape;
    st.scalar = shape.IsScalar();
    plan.stores.push_back(st);
    return st.id;
  };
  auto sharding_in_group = [&](int gi, int value, DeviceRange devices) {
    // layout with which group gi wants to read `value`
    if (const ShardedShape* sh = InputShardingOf(s, s.groups[gi].id, value)) return OnDevices(*sh, devices);
    const Value& v = g.value(value);
    ShardedShape rep = ShardedShape::Replicated(v.dtype, v.shape, devices);
    const ColorConfig& cc = part.Get(s.groups[gi].color);
    if (!cc.options.dims.empty() && cc.devices.n == devices.n) rep.mesh_dims = cc.options.dims;
    return rep;
  };
  auto produced_sharding = [&](int gi, int value, DeviceRange devices) {
    const Value& v = g.value(value);
    if (v.has_sharding) return OnDevices(v.sharding, devices);
    ShardedShape rep = ShardedShape::Replicated(v.dtype, v.shape, devices);
    const ColorConfig& cc = part.Get(s.groups[gi].color);
    if (!cc.options.dims.empty() && cc.devices.n == devices.n) rep.mesh_dims = cc.options.dims;
    return rep;
  };

  // parameters: placed where their first consumer runs, in the layout it wants
  plan.param_stores.assign(g.inputs.size(), -1);
  for (size_t i = 0; i < g.inputs.size(); ++i) {
    const int v = g.inputs[i];
    int first = -1;
    for (size_t k = 0; k < order.size() && first < 0; ++k) {
      const auto& ins = plan.templates[order[k].group_index].inputs;
      if (std::find(ins.begin(), ins.end(), v) != ins.end()) first = static_cast<int>(k);
    }
    if (first < 0) {
      plan.unused_params.push_back(static_cast<int>(i));
      if (!graph_outputs.count(v)) continue;
    }
    const int gi = first >= 0 ? order[first].group_index : 0;
    const DeviceRange dev = first >= 0 ? part.Get(s.groups[gi].color).devices : part.global();
    const int sid = new_store(Store::PARAM, static_cast<int>(i), v, -1,
                              first >= 0 ? sharding_in_group(gi, v, dev)
                                         : ShardedShape::Replicated(g.value(v).dtype, g.value(v).shape, dev));
    plan.stores[sid].name = "param" + std::to_string(i);
    plan.param_stores[i] = sid;
    store_of[{v, -1}] = sid;
  }

  // ---------------------------------------------------------------- ops
  std::map<int, int> root_index;  // value -> first root position
  for (size_t j = 0; j < g.outputs.size(); ++j) root_index.emplace(g.outputs[j], static_cast<int>(j));
  std::map<std::pair<int, std::string>, int> reshard_cache;  // (src store, target key) -> dst store
  std::map<int, int> accumulate_writes;                      // store id -> number of writes so far
  int temp_counter = 0;

  auto emit_reshard = [&](int src_store, const ShardedShape& want) {
    auto key = std::make_pair(src_store, want.Key());
    auto hit = reshard_cache.find(key);
    if (hit != reshard_cache.end()) return hit->second;
    // by value: new_store() grows the store table and would leave a reference dangling
    const int src_value = plan.stores[src_store].value;
    const int src_iteration = plan.stores[src_store].iteration;
    const DeviceRange src_devices = plan.stores[src_store].shape.devices;
    const int dst = new_store(Store::TEMP, temp_counter++, src_value, src_iteration, want);
    PlanOp op;
    op.kind = PlanOp::RESHARD;
    op.src_store = src_store;
    op.dst_store = dst;
    op.name = "reshard";
    op.iteration = src_iteration;
    // every device of either layout takes part
    const int lo = std::min(src_devices.start, want.devices.start);
    const int hi = std::max(src_devices.stop(), want.devices.stop());
    op.devices = DeviceRange{lo, hi - lo};
    plan.ops.push_back(op);
    reshard_cache[key] = dst;
    return dst;
  };

  for (const Instance& inst : order) {
    const TaskTemplate& t = plan.templates[inst.group_index];
    PlanOp op;
    op.kind = PlanOp::TASK;
    op.task_template = t.id;
    op.name = t.name;
    op.devices = inst.devices;
    op.loop = t.in_loop;
    op.iteration = inst.iteration;
    op.priority = t.in_loop ? 10 : 0;
    op.strict_ordering = t.in_loop || t.has_collectives || !s.config.dynamic_schedule_post_loop_tasks;
    if (t.in_loop) op.scalars.push_back(static_cast<int64_t>(inst.iteration) * loop.size);
    // inputs
    for (int v : t.inputs) {
      const int p = g.value(v).producer;
      int src = -1;
      if (p < 0) {
        src = store_of.at({v, -1});
      } else {
        const Node& pn = g.node(p);
        const bool loop_value = pn.loop >= 0 && pn.op != "mm.accumulate";
        auto it = store_of.find({v, loop_value ? inst.iteration : -1});
        if (it == store_of.end())
          throw std::runtime_error("plan: task " + t.name + " reads a value that has not been produced yet (" +
                                   g.value(v).name + ")");
        src = it->second;
      }
      const ShardedShape want = sharding_in_group(inst.group_index, v, inst.devices);
      int bound = src;
      if (NeedsReshard(plan.stores[src].shape, want)) bound = emit_reshard(src, want);
      op.inputs.push_back(bound);
    }
    // outputs
    for (int v : t.outputs) {
      const Node& pn = g.node(g.value(v).producer);
      const bool is_acc = pn.op == "mm.accumulate" && pn.loop >= 0;
      const int iteration = (t.in_loop && !is_acc) ? inst.iteration : -1;
      int sid;
      auto it = store_of.find({v, iteration});
      if (it != store_of.end()) {
        sid = it->second;
      } else {
        auto root = root_index.find(v);
        const ShardedShape shape = produced_sharding(inst.group_index, v, inst.devices);
        if (root != root_index.end()) {
          sid = new_store(Store::ROOT, root->second, v, iteration, shape);
          plan.stores[sid].name = "root" + std::to_string(root->second);
        } else {
          sid = new_store(Store::TEMP, temp_counter++, v, iteration, shape);
        }
        store_of[{v, iteration}] = sid;
      }
      if (is_acc) {
        if (plan.stores[sid].shape.devices != inst.devices)
          throw std::runtime_error("a summed microbatch output must be produced on the same devices in every iteration");
        op.accumulate.push_back(accumulate_writes[sid]++ == 0 ? 1 : 2);
      } else {
        op.accumulate.push_back(0);
      }
      op.outputs.push_back(sid);
    }
    plan.ops.push_back(op);
  }

  // roots: outputs that are graph inputs passed through were copied by ConstantOutputCopy, so
  // every root has a producer; scalars living on a submesh are broadcast to the global mesh
  plan.root_stores.assign(g.outputs.size(), -1);
  for (size_t j = 0; j < g.outputs.size(); ++j) {
    const int v = g.outputs[j];
    auto it = store_of.find({v, -1});
    if (it == store_of.end()) throw std::runtime_error("plan: graph output " + std::to_string(j) + " is never produced");
    int sid = it->second;
    const Store& st = plan.stores[sid];
    if (st.shape.IsScalar() && st.shape.devices != part.global()) {
      const ShardedShape want = ShardedShape::Replicated(st.shape.dtype, st.shape.sizes, part.global());
      const int dst = emit_reshard(sid, want);
      plan.stores[dst].kind = Store::ROOT;
      plan.stores[dst].index = static_cast<int>(j);
      plan.stores[dst].name = "root" + std::to_string(j) + "_global";
      sid = dst;
    }
    plan.root_stores[j] = sid;
  }

  // ---------------------------------------------------------------- hoist reshards
  // A reshard runs right after the operation that (last) produced its source, so the
  // transfer overlaps whatever the schedule runs next; reshards of parameters go first.
  {
    std::vector<int> anchor(plan.ops.size(), -2);
    for (size_t k = 0; k < plan.ops.size(); ++k) {
      if (plan.ops[k].kind != PlanOp::RESHARD) continue;
      anchor[k] = -1;
      for (int j = static_cast<int>(k) - 1; j >= 0; --j) {
        const PlanOp& w = plan.ops[j];
        if (w.kind != PlanOp::TASK) continue;
        if (std::find(w.outputs.begin(), w.outputs.end(), plan.ops[k].src_store) != w.outputs.end()) {
          anchor[k] = j;
          break;
        }
      }
    }
    std::vector<PlanOp> reordered;
    for (size_t k = 0; k < plan.ops.size(); ++k) if (anchor[k] == -1) reordered.push_back(plan.ops[k]);
    for (size_t k = 0; k < plan.ops.size(); ++k) {
      if (plan.ops[k].kind == PlanOp::RESHARD) continue;
      reordered.push_back(plan.ops[k]);
      for (size_t r = k + 1; r < plan.ops.size(); ++r) if (anchor[r] == static_cast<int>(k)) reordered.push_back(plan.ops[r]);
    }
    plan.ops = reordered;
  }

  // ---------------------------------------------------------------- in-place collectives
  // A task outside the loop that is nothing but an all-reduce of one of its inputs (the
  // once-per-step reduction of a gradient accumulator) writes its result over that input when
  // nothing else reads the input: the output store reuses the input's buffer and the runtime
  // reduces in place (src/pjrt_client/mpmd_inplace_collectives.cc:20-76).
  {
    std::vector<int> readers(plan.stores.size(), 0), writers(plan.stores.size(), 0);
    for (const PlanOp& op : plan.ops) {
      if (op.kind == PlanOp::TASK) {
        for (int sid : op.inputs) ++readers[sid];
        for (int sid : op.outputs) ++writers[sid];
      } else if (op.kind == PlanOp::RESHARD) {
        ++readers[op.src_store];
        ++writers[op.dst_store];
      }
    }
    int count = 0;
    for (const PlanOp& op : plan.ops) {
      if (op.kind != PlanOp::TASK || op.loop) continue;
      const TaskTemplate& t = plan.templates[op.task_template];
      int reduce = -1, others = 0;
      for (int id : t.nodes) {
        const Node& n = g.node(id);
        if (n.op == "mm.all_reduce") reduce = reduce < 0 ? id : -2;
        else if (n.op != "mm.accumulate" && n.op != "mm.relayout" && n.op.rfind("mm.marker", 0) != 0) ++others;
      }
      if (reduce < 0 || others > 0 || t.inputs.size() != 1 || t.outputs.size() != 1) continue;
      const int in_sid = op.inputs[0], out_sid = op.outputs[0];
      const Store& in = plan.stores[in_sid];
      Store& out = plan.stores[out_sid];
      if (in.kind != Store::TEMP || out.kind != Store::TEMP || in.alias_of >= 0 || out.alias_of >= 0) continue;
      if (readers[in_sid] != 1 || writers[out_sid] != 1 || !(in.shape == out.shape)) continue;
      out.alias_of = in_sid;
      g.node(reduce).attrs["in_place"] = "1";
      ++count;
    }
    plan.stats["in_place_collectives"] = std::to_string(count);
  }

  // ---------------------------------------------------------------- buffer names
  // last use of every store in op order; reshards tick the clock twice so that a buffer
  // released by a reshard is not handed out again immediately
  std::vector<int> first_def(plan.stores.size(), -1), last_use(plan.stores.size(), -1);
  std::vector<int> clock_at(plan.ops.size(), 0);
  int clock = 0;
  for (size_t k = 0; k < plan.ops.size(); ++k) {
    const PlanOp& op = plan.ops[k];
    clock += op.kind == PlanOp::RESHARD ? 2 : 1;
    clock_at[k] = clock;
    auto touch = [&](int sid, bool def) {
      if (def && first_def[sid] < 0) first_def[sid] = clock;
      last_use[sid] = clock;
    };
    if (op.kind == PlanOp::TASK) {
      for (int sid : op.inputs) touch(sid, false);
      for (int sid : op.outputs) touch(sid, true);
    } else if (op.kind == PlanOp::RESHARD) {
      touch(op.src_store, false);
      touch(op.dst_store, true);
    }
  }
  for (int sid : plan.root_stores) if (sid >= 0) last_use[sid] = 1 << 30;
  // a store that reuses another temporary's buffer keeps that buffer alive for its own lifetime
  for (auto& st : plan.stores)
    if (st.kind == Store::TEMP && st.alias_of >= 0) last_use[st.alias_of] = std::max(last_use[st.alias_of], last_use[st.id]);
  {
    std::map<std::string, std::vector<std::pair<int, std::string>>> pools;  // shape key -> (free-at clock, name)
    std::vector<int> temps;
    for (auto& st : plan.stores) if (st.kind == Store::TEMP) temps.push_back(st.id);
    std::sort(temps.begin(), temps.end(), [&](int a, int b) { return first_def[a] < first_def[b]; });
    int fresh = 0;
    for (int sid : temps) {
      Store& st = plan.stores[sid];
      if (st.alias_of >= 0) {           // in-place result: the name of the buffer it overwrites
        st.name = plan.stores[st.alias_of].name;
        continue;
      }
      auto& pool = pools[st.shape.Key()];
      std::string name;
      for (size_t i = 0; i < pool.size(); ++i)
        if (pool[i].first < first_def[sid]) { name = pool[i].second; pool.erase(pool.begin() + i); break; }
      if (name.empty()) name = "temp" + std::to_string(fresh++);
      st.name = name;
      pool.emplace_back(last_use[sid], name);
    }
    plan.stats["temp_buffers"] = std::to_string(fresh);
    // high-water mark per device
    std::map<std::string, std::pair<int64_t, DeviceRange>> uniq;
    for (auto& st : plan.stores) if (st.kind == Store::TEMP) uniq[st.name] = {st.shape.ShardBytes(), st.shape.devices};
    std::map<int, int64_t> per_device;
    for (auto& kv : uniq)
      for (int d = kv.second.second.start; d < kv.second.second.stop(); ++d) per_device[d] += kv.second.first;
    for (auto& kv : per_device) plan.temp_bytes_per_device_max = std::max(plan.temp_bytes_per_device_max, kv.second);
  }

  // ---------------------------------------------------------------- donation
  {
    std::set<int> taken;
    for (int pi : g.donated_inputs) {
      if (pi < 0 || pi >= static_cast<int>(plan.param_stores.size())) continue;
      const int ps = plan.param_stores[pi];
      if (ps < 0) continue;
      for (size_t j = 0; j < plan.root_stores.size(); ++j) {
        const int rs = plan.root_stores[j];
        if (rs < 0 || taken.count(rs) || plan.stores[rs].alias_of >= 0) continue;
        if (!(plan.stores[rs].shape == plan.stores[ps].shape)) continue;
        // the parameter must not be read after the root has been written
        if (last_use[ps] > first_def[rs]) continue;
        plan.stores[rs].alias_of = ps;
        plan.aliases.emplace_back(ps, rs);
        taken.insert(rs);
        break;
      }
    }
  }

  // CREATE_STORE records for every physical buffer, ahead of the first op
  std::vector<PlanOp> creates;
  std::set<std::string> created;
  for (auto& st : plan.stores) {
    if (st.alias_of >= 0 || st.kind == Store::PARAM) continue;
    if (!created.insert(st.name + "@" + st.shape.Key()).second) continue;
    PlanOp c;
    c.kind = PlanOp::CREATE_STORE;
    c.store = st.id;
    c.devices = st.shape.devices;
    creates.push_back(c);
  }
  plan.ops.insert(plan.ops.begin(), creates.begin(), creates.end());
  plan.stats["tasks"] = std::to_string(order.size());
  plan.stats["reshards"] = std::to_string(reshard_cache.size());
  return plan;
}

}  // namespace mmg
