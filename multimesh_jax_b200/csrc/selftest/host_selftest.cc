// Stand-alone self test of the C++ compiler (mmgraph) and task runtime (mmrt), meant to be built
// with -fsanitize=address,undefined or -fsanitize=thread (no Python in the process):
//
//   1. builds a microbatched P-stage pipeline graph with forward, backward and weight-gradient
//      work, compiles it with every pipeline schedule and checks plan invariants;
//   2. executes each plan on a ThreadedContext with one worker thread per virtual device. Task
//      and reshard bodies read and write plain host buffers (one per physical buffer and device,
//      shared by every store with the same scheduling name) WITHOUT locks, so a missing
//      dependency edge is a data race the thread sanitizer reports and a wrong checksum here;
//   3. replays the submission log through the hazard checker; runs the same plan on the
//      stream-and-event context (CudaContext over the recording stand-in for the CUDA runtime) and
//      checks that it computes the same result and that its cross-stream conflicts became waits;
//   4. injects host-side faults (a task body that throws, a dropped task) and checks that the
//      error surfaces as a status and that the context stays usable;
//   5. runs 20 random task graphs (random devices, tiles, priorities, strict-order flags) on the
//      threaded runtime and compares each with the same tasks run one after the other;
//   6. for every stored-program file named on the command line (real-model training steps with
//      pipeline, tensor, sequence, data and expert parallelism): loads it, compiles it offline,
//      replays the plan on the mock runtime, writes the program back to text, reads that again
//      and compares the plans; then feeds the loader truncated and corrupted copies of the text,
//      which must be refused with an exception, never read out of bounds, and 40 randomly damaged
//      copies of the first file, which must be refused or compile.
//
//   host_selftest [repeats] [stored-program.json ...]
//
// Exit code 0 = all checks passed. The reference gets the same assurance from its ASAN build type
// (CMakeLists.txt:12-17) over the mock-runtime tests.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <string>
#include <vector>

#include "../mmgraph/graph.h"
#include "../mmgraph/passes.h"
#include "../mmgraph/program_file.h"
#include "../mmrt/cuda_context.h"
#include "../mmrt/runtime.h"

using namespace mmg;

static int g_failures = 0;
#define CHECK(cond, msg)                                                \
  do {                                                                  \
    if (!(cond)) {                                                      \
      std::fprintf(stderr, "CHECK failed (%s:%d): %s\n", __FILE__, __LINE__, msg); \
      ++g_failures;                                                     \
    }                                                                   \
  } while (0)

static std::string TaskJson(const std::string& name, int device, bool split) {
  std::string s = "{\"name\":\"" + name + "\",\"devices\":[" + std::to_string(device) + "],\"dims\":[1],"
                  "\"device_axes\":[\"x\"],\"logical_axes\":[],\"split_backprop\":[";
  if (split) s += "\"_act\",\"_wgt\"";
  s += "],\"loop_dependent_devices\":[]}";
  return s;
}

static int AddOp(Graph& g, const std::string& op, const std::vector<int>& in, std::vector<int64_t> shape, int loop,
                 const std::string& task, bool backprop) {
  const int id = g.AddNode(op, in, {shape}, {DType::F32}, {{"args", "[]"}});
  Node& n = g.node(id);
  n.loop = loop;
  n.explicit_task = task;
  n.backprop = backprop;
  return n.outputs[0];
}

// x -> P stages of (mm, tanh) -> loss; backward chain with input and weight gradients per stage.
static void BuildPipeline(Graph& g, int stages, int microbatches, const std::string& schedule, bool split) {
  const int64_t B = 4 * microbatches, D = 8;
  LoopConfig loop;
  loop.id = 0;
  loop.num_microbatches = microbatches;
  loop.slice_dim = 0;
  loop.size = 4;
  loop.schedule = schedule;
  g.loops.push_back(loop);
  const int x = g.AddInput("x", {B, D}, DType::F32);
  std::vector<int> w(stages);
  for (int s = 0; s < stages; ++s) w[s] = g.AddInput("w" + std::to_string(s), {D, D}, DType::F32);
  const int slice_node = g.AddNode("mm.microbatch_slice.default", {x}, {{4, D}}, {DType::F32}, {{"args", "[0, 4, 0]"}});
  g.node(slice_node).loop = 0;
  int h = g.node(slice_node).outputs[0];
  std::vector<int> acts;
  for (int s = 0; s < stages; ++s) {
    const std::string t = TaskJson("stage" + std::to_string(s), s, false);
    acts.push_back(h);
    h = AddOp(g, "aten.mm.default", {h, w[s]}, {4, D}, 0, t, false);
    h = AddOp(g, "aten.tanh.default", {h}, {4, D}, 0, t, false);
  }
  int grad = AddOp(g, "aten.ones_like.default", {h}, {4, D}, 0, TaskJson("stage" + std::to_string(stages - 1) + "_bwd",
                                                                          stages - 1, split), true);
  std::vector<int> outs;
  for (int s = stages - 1; s >= 0; --s) {
    const std::string t = TaskJson("stage" + std::to_string(s) + "_bwd", s, split);
    const int dw = AddOp(g, "aten.mm.default", {acts[s], grad}, {D, D}, 0, t, true);   // weight gradient
    if (s > 0) grad = AddOp(g, "aten.mm.default", {grad, w[s]}, {4, D}, 0, t, true);   // input gradient
    const int out_node = g.AddNode("mm.microbatch_out.default", {dw}, {{D, D}}, {DType::F32}, {{"args", "[0, \"\"]"}});
    g.node(out_node).loop = 0;
    outs.push_back(g.node(out_node).outputs[0]);
  }
  g.SetOutputs(outs);
}

struct RunResult {
  double checksum = 0;
  std::string hazards;
  mmrt::Status status = mmrt::Status::kOk;
};

// Executes the plan's operation list on `ctx` with synthetic bodies over unlocked host buffers.
template <class Context>
static RunResult ExecuteOn(Context& ctx, const Plan& plan, bool inject_throw) {
  std::map<std::string, int> buffer_of_name;
  auto buffer_id = [&](const Store& st) {
    const std::string key = std::to_string(static_cast<int>(st.kind)) + ":" + st.name;
    auto it = buffer_of_name.find(key);
    if (it == buffer_of_name.end()) it = buffer_of_name.emplace(key, static_cast<int>(buffer_of_name.size())).first;
    return it->second;
  };
  // one cell of payload per (buffer, device); sized up front so bodies never rehash the map
  std::map<std::pair<int, int>, double> cells;
  for (const Store& st : plan.stores)
    for (int d = st.shape.devices.start; d < st.shape.devices.stop(); ++d) cells[{buffer_id(st), d}] = 0.0;
  for (size_t i = 0; i < plan.param_stores.size(); ++i) {
    if (plan.param_stores[i] < 0) continue;
    const Store& st = plan.stores[plan.param_stores[i]];
    for (int d = st.shape.devices.start; d < st.shape.devices.stop(); ++d) cells[{buffer_id(st), d}] = 1.0 + 0.25 * i;
  }
  auto tiles = [&](int store, int device_filter) {
    std::vector<mmrt::TileRef> t;
    const Store& st = plan.stores[store];
    for (int d = st.shape.devices.start; d < st.shape.devices.stop(); ++d)
      if (device_filter < 0 || d == device_filter) t.push_back({buffer_id(st), d});
    return t;
  };
  if (inject_throw) {
    mmrt::FaultSpec f;
    f.kind = mmrt::FaultSpec::kThrow;
    f.name_substring = "_bwd";
    f.remaining = 1;
    ctx.InjectFault(f);
  }
  ctx.OpenWindow();
  int k = 0;
  for (const PlanOp& op : plan.ops) {
    ++k;
    if (op.kind == PlanOp::TASK) {
      for (int d = op.devices.start; d < op.devices.stop(); ++d) {
        std::vector<mmrt::TileRef> reads, writes;
        for (int s : op.inputs) for (auto& t : tiles(s, d)) reads.push_back(t);
        for (size_t o = 0; o < op.outputs.size(); ++o) {
          for (auto& t : tiles(op.outputs[o], d)) {
            writes.push_back(t);
            if (!op.accumulate.empty() && op.accumulate[o] == 2) reads.push_back(t);
          }
        }
        const std::vector<int> acc = op.accumulate;
        mmrt::ExecuteOptions eo;
        eo.name = op.name;
        eo.priority = op.priority;
        eo.strict_ordering = op.strict_ordering;
        ctx.CreateExecuteTask(d, reads, writes, [&cells, reads, writes, acc, k] {
          double v = 0.001 * k;
          for (auto& r : reads) v += 0.5 * cells.at({r.buffer, r.device});
          size_t o = 0;
          for (auto& wt : writes) {
            double& c = cells.at({wt.buffer, wt.device});
            c = (!acc.empty() && o < acc.size() && acc[o] == 2) ? c + std::tanh(v) : std::tanh(v);
            ++o;
          }
        }, eo);
      }
    } else if (op.kind == PlanOp::RESHARD) {
      const Store& dst = plan.stores[op.dst_store];
      for (int d = dst.shape.devices.start; d < dst.shape.devices.stop(); ++d) {
        std::vector<mmrt::TileRef> reads = tiles(op.src_store, -1), writes = tiles(op.dst_store, d);
        mmrt::ExecuteOptions eo;
        eo.name = "reshard";
        eo.kind = 1;
        ctx.Reshard(d, reads, writes, [&cells, reads, writes] {
          double v = 0;
          for (auto& r : reads) v += cells.at({r.buffer, r.device});
          for (auto& wt : writes) cells.at({wt.buffer, wt.device}) = v / static_cast<double>(reads.size());
        }, eo);
      }
    }
  }
  ctx.CloseWindow();
  RunResult res;
  std::string message;
  res.status = ctx.WaitAll(&message);
  res.hazards = mmrt::CheckHazards(ctx.Submissions());
  for (int r : plan.root_stores)
    for (auto& t : tiles(r, -1)) res.checksum += cells.at({t.buffer, t.device});
  if (inject_throw) {
    // the context must stay usable after a failed step
    ctx.ResetError();
    mmrt::ExecuteOptions eo;
    eo.name = "after_failure";
    double probe = 0;
    ctx.CreateExecuteTask(0, {}, {}, [&probe] { probe = 42.0; }, eo);
    std::string m2;
    CHECK(ctx.WaitAll(&m2) == mmrt::Status::kOk && probe == 42.0, "context unusable after an injected fault");
  }
  ctx.Shutdown();
  return res;
}

static RunResult Execute(const Plan& plan, int num_devices, bool inject_throw) {
  std::vector<int> devices(num_devices);
  for (int d = 0; d < num_devices; ++d) devices[d] = d;
  mmrt::ThreadedContext ctx(devices, /*inline_execution=*/false, /*record_submissions=*/true);
  return ExecuteOn(ctx, plan, inject_throw);
}

// The same plan on the stream-and-event context over the recording stand-in for the CUDA runtime:
// bodies run at submission, reshards are given the communication stream, and every conflicting
// pair of accesses on different streams must have become an event wait.
static RunResult ExecuteOnStreams(const Plan& plan, int num_devices, bool inject_throw, size_t* edges, size_t* waits) {
  std::vector<int> devices(num_devices);
  for (int d = 0; d < num_devices; ++d) devices[d] = d;
  mmrt::FakeGpuApi api;
  RunResult res;
  {
    mmrt::CudaContext ctx(devices, devices, std::vector<uintptr_t>(num_devices, 0), &api, /*record_submissions=*/true);
    res = ExecuteOn(ctx, plan, inject_throw);
    *edges = ctx.Edges().size();
  }
  *waits = 0;
  for (const std::string& line : api.trace) *waits += line.rfind("wait ", 0) == 0;
  return res;
}

// Random task graphs straight on the runtime: tasks on random devices read and write random tiles
// (their own device's and other devices'), with random priorities and strict-order flags. The
// bodies update unlocked cells, so the result equals the one of running the tasks one after the other
// in submission order only if every read-after-write, write-after-read and write-after-write pair
// was ordered - and an unordered pair is a data race for the thread sanitizer.
static void RandomTaskGraphs(int rounds) {
  uint64_t state = 0x2545F4914F6CDD1Dull;
  auto next = [&](uint64_t bound) {
    state ^= state << 13; state ^= state >> 7; state ^= state << 17;
    return static_cast<int>(state % bound);
  };
  for (int round = 0; round < rounds; ++round) {
    const int devices = 2 + next(5), buffers = 3 + next(10), tasks = 50 + next(200);
    std::vector<int> ids(devices);
    for (int d = 0; d < devices; ++d) ids[d] = d;
    std::map<std::pair<int, int>, double> cells, expect;
    for (int b = 0; b < buffers; ++b)
      for (int d = 0; d < devices; ++d) cells[{b, d}] = expect[{b, d}] = 1.0 + 0.01 * b + 0.1 * d;
    mmrt::ThreadedContext ctx(ids, /*inline_execution=*/false, /*record_submissions=*/true);
    ctx.OpenWindow();
    for (int k = 0; k < tasks; ++k) {
      const int device = next(devices);
      std::vector<mmrt::TileRef> reads, writes;
      for (int r = 1 + next(3); r > 0; --r) reads.push_back({next(buffers), next(4) ? device : next(devices)});
      for (int w = 1 + next(2); w > 0; --w) {
        mmrt::TileRef t{next(buffers), next(6) ? device : next(devices)};
        bool dup = false;
        for (auto& x : writes) dup = dup || (x.buffer == t.buffer && x.device == t.device);
        if (!dup) writes.push_back(t);
      }
      auto apply = [reads, writes, k](std::map<std::pair<int, int>, double>& m) {
        double v = 0.001 * k;
        for (auto& r : reads) v += 0.5 * m.at({r.buffer, r.device});
        for (auto& w : writes) m.at({w.buffer, w.device}) = std::tanh(v + 0.25 * m.at({w.buffer, w.device}));
      };
      apply(expect);                       // the sequential answer
      std::vector<mmrt::TileRef> all_reads = reads;
      for (auto& w : writes) all_reads.push_back(w);   // a written cell is also read
      mmrt::ExecuteOptions eo;
      eo.name = "t" + std::to_string(k);
      eo.priority = next(3) - 1;
      eo.strict_ordering = next(8) == 0;
      if (next(5) == 0) ctx.Reshard(device, all_reads, writes, [&cells, apply] { apply(cells); }, eo);
      else ctx.CreateExecuteTask(device, all_reads, writes, [&cells, apply] { apply(cells); }, eo);
    }
    ctx.CloseWindow();
    std::string message;
    CHECK(ctx.WaitAll(&message) == mmrt::Status::kOk, "random task graph reported an error");
    CHECK(mmrt::CheckHazards(ctx.Submissions()).empty(), "random task graph: unordered conflicting accesses");
    bool same = true;
    for (auto& kv : expect) same = same && cells.at(kv.first) == kv.second;
    CHECK(same, "random task graph: result differs from the sequential run");
    ctx.Shutdown();
    // The same kind of graph on the stream-and-event context with tasks spread over the compute,
    // communication and auxiliary streams: bodies run at submission there, so the question is
    // whether the stream order plus the event waits it issued order every conflicting pair.
    mmrt::FakeGpuApi api;
    mmrt::CudaContext streams(ids, ids, std::vector<uintptr_t>(devices, 0), &api, /*record_submissions=*/true);
    streams.OpenWindow();
    for (int k = 0; k < tasks; ++k) {
      const int device = next(devices);
      std::vector<mmrt::TileRef> reads, writes;
      for (int r = 1 + next(3); r > 0; --r) reads.push_back({next(buffers), next(4) ? device : next(devices)});
      writes.push_back({next(buffers), next(6) ? device : next(devices)});
      mmrt::ExecuteOptions eo;
      eo.name = "s" + std::to_string(k);
      eo.stream = next(3);
      eo.strict_ordering = next(8) == 0;
      streams.CreateExecuteTask(device, reads, writes, [] {}, eo);
    }
    streams.CloseWindow();
    CHECK(streams.WaitAll(&message) == mmrt::Status::kOk, "stream context: random task graph reported an error");
    CHECK(mmrt::CheckHazards(streams.Submissions()).empty(), "stream context: a conflicting pair on two streams has no event edge");
    streams.Shutdown();
  }
  std::printf("%d random task graphs match their sequential runs\n", rounds);
}

static void CheckStoredProgram(const std::string& path) {
  Plan plan;
  std::vector<std::string> log;
  OfflineResult r = CompileProgramFile(path, 0, &plan, &log);
  CHECK(r.status == 0, ("stored program did not replay cleanly: " + path + ": " + r.message).c_str());
  CHECK(r.hazards.empty(), r.hazards.c_str());
  CHECK(r.tasks > 0 && r.templates > 0 && r.device_high_water_max > 0, "degenerate offline result");
  CHECK(r.fits, "a plan cannot fail to fit without a device-memory size");
  OfflineResult tight = CompileProgramFile(path, r.device_high_water_max - 1);
  CHECK(!tight.fits && tight.plan_hash == r.plan_hash, "memory limit below the high-water mark must not fit");
  // text -> program -> text -> program: the second reading compiles to the same plan
  StoredProgram first = LoadProgram(path);
  const std::string text = ProgramToJson(*first.graph, *first.partition, first.config);
  StoredProgram second = ProgramFromJson(text);
  std::vector<std::string> log2;
  Plan plan2 = MpmdPartition(*second.graph, *second.partition, second.config, &log2);
  CHECK(plan2.Hash() == r.plan_hash, "a program written back and read again compiles to another plan");
  // damaged text must be refused, not read past its end
  int refused = 0, tried = 0;
  for (size_t cut : {text.size() / 7, text.size() / 3, text.size() / 2, text.size() - 2}) {
    ++tried;
    try { ProgramFromJson(text.substr(0, cut)); } catch (const std::exception&) { ++refused; }
  }
  CHECK(refused == tried, "a truncated program file was accepted");
  std::string wrong = text;
  const size_t at = wrong.find("\"inputs\":[");
  if (at != std::string::npos) {
    wrong.insert(at + 10, "123456789,");     // an operand id that no value has
    bool threw = false;
    try {
      StoredProgram bad = ProgramFromJson(wrong);
      MpmdPartition(*bad.graph, *bad.partition, bad.config);
    } catch (const std::exception&) { threw = true; }
    CHECK(threw, "an operand id out of range was accepted");
  }
  // an operator id that does not exist in the order list, and a result that names another producer
  for (const char* key : {"\"order\":[", "\"outputs\":["}) {
    std::string broken = text;
    const size_t k = broken.find(key);
    if (k == std::string::npos) continue;
    broken.insert(k + std::string(key).size(), "7880,");
    bool threw = false;
    try { ProgramFromJson(broken); } catch (const std::exception&) { threw = true; }
    CHECK(threw, "an inconsistent id list was accepted");
  }
  std::printf("%-60s %d templates, %d tasks, %d reshards, high water %lld bytes\n",
              path.substr(path.find_last_of('/') + 1).c_str(), r.templates, r.tasks, r.reshards,
              static_cast<long long>(r.device_high_water_max));
}

// Random small damage to the text of a stored program (a digit replaced, a few characters cut,
// a structural character overwritten): the loader and the compiler either refuse the result with
// an exception or compile it; under the sanitizers anything else shows up as a report.
static void MutateStoredProgram(const std::string& path, int rounds) {
  StoredProgram original = LoadProgram(path);
  const std::string text = ProgramToJson(*original.graph, *original.partition, original.config);
  uint64_t state = 0x9E3779B97F4A7C15ull;
  auto next = [&](uint64_t bound) {
    state = state * 6364136223846793005ull + 1442695040888963407ull;
    return static_cast<size_t>((state >> 33) % bound);
  };
  int refused = 0, compiled = 0;
  for (int r = 0; r < rounds; ++r) {
    std::string t = text;
    const int edits = 1 + static_cast<int>(next(3));
    for (int e = 0; e < edits; ++e) {
      const size_t i = next(t.size());
      if (t[i] >= '0' && t[i] <= '9') t[i] = static_cast<char>('0' + next(10));
      else if (next(2)) t.erase(i, 1 + next(6));
      else t[i] = "{}[]\",:0a-"[next(11)];
    }
    try {
      StoredProgram p = ProgramFromJson(t);
      Plan plan = MpmdPartition(*p.graph, *p.partition, p.config);
      MockExecutePlan(plan, p.partition->global().start, p.partition->global().n, 0, 1);
      ++compiled;
    } catch (const std::exception&) {
      ++refused;
    }
  }
  std::printf("%d damaged copies of %s: %d refused, %d still compiled\n", rounds,
              path.substr(path.find_last_of('/') + 1).c_str(), refused, compiled);
}

int main(int argc, char** argv) {
  const int repeats = argc > 1 ? std::atoi(argv[1]) : 3;
  const char* schedules[] = {"gpipe", "1f1b", "wavefront", "zero-bubble-h2"};
  for (const char* schedule : schedules) {
    const bool split = std::string(schedule) == "zero-bubble-h2";
    for (int stages : {2, 4}) {
      const int microbatches = 2 * stages;
      Graph g;
      BuildPipeline(g, stages, microbatches, schedule, split);
      Partition part(DeviceRange::Create(0, stages));
      PartitionConfig cfg;
      std::vector<std::string> log;
      Plan plan = MpmdPartition(g, part, cfg, &log);
      int tasks = 0, reshards = 0;
      for (const PlanOp& op : plan.ops) {
        tasks += op.kind == PlanOp::TASK;
        reshards += op.kind == PlanOp::RESHARD;
        if (op.kind == PlanOp::TASK) {
          CHECK(op.inputs.size() == plan.templates[op.task_template].inputs.size(), "task inputs do not match template");
          CHECK(op.outputs.size() == plan.templates[op.task_template].outputs.size(), "task outputs do not match template");
        }
      }
      CHECK(tasks >= 2 * stages * microbatches, "fewer tasks than forward + backward per stage and microbatch");
      CHECK(reshards > 0, "a pipeline without stage-boundary reshards");
      // determinism: compiling the same graph again gives the same plan
      Graph g2;
      BuildPipeline(g2, stages, microbatches, schedule, split);
      Partition part2(DeviceRange::Create(0, stages));
      CHECK(MpmdPartition(g2, part2, cfg).Hash() == plan.Hash(), "plan hash is not deterministic");

      double first = 0;
      for (int r = 0; r < repeats; ++r) {
        RunResult res = Execute(plan, stages, false);
        CHECK(res.status == mmrt::Status::kOk, "execution reported an error");
        CHECK(res.hazards.empty(), res.hazards.c_str());
        CHECK(std::isfinite(res.checksum) && res.checksum != 0.0, "degenerate checksum");
        if (r == 0) first = res.checksum;
        CHECK(std::fabs(res.checksum - first) < 1e-12, "results differ between runs: tasks raced");
      }
      RunResult failed = Execute(plan, stages, true);
      CHECK(failed.status != mmrt::Status::kOk, "an injected fault did not surface as a status");
      size_t edges = 0, waits = 0;
      RunResult streams = ExecuteOnStreams(plan, stages, false, &edges, &waits);
      CHECK(streams.status == mmrt::Status::kOk, "stream context reported an error");
      CHECK(streams.hazards.empty(), streams.hazards.c_str());
      CHECK(std::fabs(streams.checksum - first) < 1e-12, "stream context computed another result");
      CHECK(edges > 0 && waits >= edges, "cross-stream conflicts did not become event waits");
      RunResult streams_failed = ExecuteOnStreams(plan, stages, true, &edges, &waits);
      CHECK(streams_failed.status != mmrt::Status::kOk, "stream context: an injected fault did not surface");
      std::printf("%-15s stages=%d microbatches=%d: %d tasks, %d reshards, checksum %.9f\n", schedule, stages,
                  microbatches, tasks, reshards, first);
    }
  }
  RandomTaskGraphs(20);
  for (int a = 2; a < argc; ++a) CheckStoredProgram(argv[a]);
  if (argc > 2) MutateStoredProgram(argv[2], 40);
  if (g_failures) {
    std::fprintf(stderr, "%d check(s) failed\n", g_failures);
    return 1;
  }
  std::printf("host selftest ok\n");
  return 0;
}
