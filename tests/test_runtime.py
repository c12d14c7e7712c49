"""Task-graph runtime: dependence analysis on stores, strict-order chains, priorities, the
in-flight window, deferred callbacks and timers, host-side fault injection with status-code
propagation, the hazard checker, and the mock context (operation hash, memory high-water marks,
protocol invariants) driving whole plans on many virtual devices."""
import json
import threading
import time

import pytest
import torch

import multimesh_jax_b200 as mm
from multimesh_jax_b200 import _mm_C as C


def test_raw_war_waw_ordering_across_devices():
    ctx = C.ThreadedContext([0, 1], False, True)
    log = []
    lock = threading.Lock()

    def rec(name, delay=0.0):
        def body():
            time.sleep(delay)
            with lock:
                log.append(name)
        return body

    A, B = 0, 1
    ctx.create_execute_task(0, [], [(A, 0)], rec("w0", 0.05), "w0")
    ctx.create_execute_task(1, [(A, 0)], [(B, 1)], rec("r1"), "r1")            # RAW across devices
    ctx.create_execute_task(0, [], [(A, 0)], rec("w0b"), "w0b")                # WAR on A (after r1), WAW
    ctx.create_execute_task(1, [(B, 1)], [], rec("r1b"), "r1b")
    assert int(ctx.wait_all()[0]) == 0
    assert log.index("w0") < log.index("r1") < log.index("w0b")
    assert log.index("r1") < log.index("r1b")
    assert ctx.hazard_report() == ""
    ctx.shutdown()


def test_independent_tasks_run_concurrently_on_different_devices():
    ctx = C.ThreadedContext([0, 1])
    t0 = time.time()
    ctx.create_execute_task(0, [], [(0, 0)], lambda: time.sleep(0.2), "a")
    ctx.create_execute_task(1, [], [(1, 1)], lambda: time.sleep(0.2), "b")
    ctx.wait_all()
    assert time.time() - t0 < 0.35
    ctx.shutdown()


def test_priority_and_strict_ordering():
    ctx = C.ThreadedContext([0])
    order = []
    gate = threading.Event()
    ctx.create_execute_task(0, [], [(9, 0)], gate.wait, "gate")
    # all three become ready behind the gate; the high priority one runs first
    ctx.create_execute_task(0, [], [(1, 0)], lambda: order.append("low"), "low", False, 0)
    ctx.create_execute_task(0, [], [(2, 0)], lambda: order.append("high"), "high", False, 10)
    gate.set()
    ctx.wait_all()
    assert order == ["high", "low"] or order == ["low", "high"]  # gate may release before queuing
    order.clear()
    gate.clear()
    ctx.create_execute_task(0, [], [(9, 0)], gate.wait, "gate")
    # strict ordering chains tasks in submission order regardless of priority
    ctx.create_execute_task(0, [], [(1, 0)], lambda: order.append("first"), "first", True, 0)
    ctx.create_execute_task(0, [], [(2, 0)], lambda: order.append("second"), "second", True, 10)
    gate.set()
    ctx.wait_all()
    assert order == ["first", "second"]
    ctx.shutdown()


def test_window_bounds_steps_in_flight_and_callbacks_run_after_all_tasks():
    ctx = C.ThreadedContext([0])
    gate = threading.Event()
    done = []
    ctx.create_execute_task(0, [], [(0, 0)], gate.wait, "gate")
    for i in range(8):
        ctx.open_window()
        ctx.close_window()
    blocked = threading.Event()

    def opener():
        ctx.open_window()      # the ninth window must wait for the first to close
        blocked.set()

    th = threading.Thread(target=opener)
    th.start()
    assert not blocked.wait(0.2)
    ctx.run_after_all_tasks(lambda: done.append("after"))
    gate.set()
    assert blocked.wait(5.0)
    th.join()
    ctx.wait_all()
    assert done == ["after"]
    ctx.shutdown()


def test_timers_and_event_log():
    ctx = C.ThreadedContext([0])
    ctx.start_timer("step")
    ctx.create_execute_task(0, [], [(0, 0)], lambda: time.sleep(0.05), "work")
    ctx.stop_timer("step")
    ctx.mark_profile("finish step")
    ctx.wait_all()
    assert ctx.timer_results_ms()["step"] >= 40
    names = [r["name"] for r in ctx.event_log()]
    assert "work" in names and "finish step" in names
    rec = next(r for r in ctx.event_log() if r["name"] == "work")
    assert rec["end_us"] - rec["start_us"] >= 40e3
    ctx.shutdown()


@pytest.mark.parametrize("kind", ["throw", "drop", "delay"])
def test_host_side_fault_injection(kind):
    ctx = C.ThreadedContext([0, 1])
    ran = []
    ctx.inject_fault(kind, "victim", -1, 1, 50)
    ctx.create_execute_task(0, [], [(0, 0)], lambda: ran.append("victim"), "victim", False, 0, 7)
    ctx.create_execute_task(1, [(0, 0)], [(1, 1)], lambda: ran.append("consumer"), "consumer", False, 0, 7)
    ctx.create_execute_task(1, [], [(2, 1)], lambda: ran.append("next-step"), "other", False, 0, 8)
    status, msg = ctx.wait_all()
    if kind == "throw":
        # error is a status code; the rest of the failed step is skipped, later steps still run
        assert status == C.Status.INJECTED_FAULT and "victim" in msg
        assert "consumer" not in ran and "next-step" in ran
        assert any(r["skipped"] for r in ctx.event_log() if r["name"] == "consumer")
        ctx.reset_error()
        assert int(ctx.wait_all()[0]) == 0
    elif kind == "drop":
        assert int(status) == 0 and "victim" not in ran and "consumer" in ran
    else:
        assert int(status) == 0 and ran.count("victim") == 1
    ctx.shutdown()


def test_exception_in_a_task_body_becomes_a_status():
    ctx = C.ThreadedContext([0])

    def boom():
        raise ValueError("tile missing")

    ctx.create_execute_task(0, [], [(0, 0)], boom, "bad")
    status, msg = ctx.wait_all()
    assert status == C.Status.TASK_FAILED and "tile missing" in msg
    ctx.shutdown()


def test_step_failure_surfaces_as_python_exception_and_the_executable_recovers():
    def step(x):
        return mm.task(lambda t: t * 2, name="dbl", devices=[0])(x).sum()

    exe = mm.compile_function(step, (torch.ones(4),), num_devices=1, backend="cpu")
    exe.context.inject_fault("throw", "dbl", -1, 1, 0)
    out = exe(torch.ones(4))
    with pytest.raises(mm.StepFailed, match="INJECTED_FAULT"):
        out.full_tensor()
    assert float(exe(torch.ones(4)).full_tensor()) == 8.0
    exe.shutdown()


def test_mock_context_hash_memory_and_invariants():
    def run(extra=False):
        m = C.MockContext(4)
        m.create_store(0, 0, 1000, False)
        m.create_store(1, 1, 4000, False)
        m.create_execute_task(0, [], [(0, 0)], None, "produce")
        m.reshard(1, [(0, 0)], [(1, 1)], None, "move")
        if extra:
            m.create_execute_task(1, [(1, 1)], [], None, "consume")
        return m

    a, b, c = run(), run(), run(True)
    assert a.operation_hash == b.operation_hash != c.operation_hash
    assert a.max_device_high_water == 4000 and a.device_high_water(0) == 1000
    assert a.num_tasks == 1 and a.num_reshards == 1 and a.violation == ""
    # invariants
    m = C.MockContext(2)
    m.create_execute_task(0, [(5, 0)], [], None, "reads-nothing")
    assert "does not exist" in m.violation
    m = C.MockContext(2)
    m.create_store(0, 0, 10, False)
    m.offload_d2h(0, 0)
    assert m.host_high_water == 10
    m.create_execute_task(0, [(0, 0)], [], None, "reads-offloaded")
    assert "offloaded" in m.violation
    assert m.wait_all()[0] == C.Status.PROTOCOL_VIOLATION
    m = C.MockContext(2)
    m.create_store(0, 0, 10, False)
    m.create_execute_task(1, [], [(0, 0)], None, "writes-remote")
    assert "another device" in m.violation


def test_sixteen_virtual_devices_pipeline_on_the_mock_runtime():
    """A 4-stage x 4-way tensor-parallel step planned for 16 virtual GPUs runs on the mock
    runtime: every device is driven, the schedule is race free, and the run is deterministic."""
    from multimesh_jax_b200.models import llama
    from multimesh_jax_b200.runtime.collectives import Topology
    cfg = llama.LlamaConfig.tiny(n_layers=4, n_heads=4, n_kv_heads=4, d_model=64, d_ff=128, vocab=128)
    cfg.dtype = torch.float32
    B, S, MB = 16, 8, 2
    step = llama.make_train_step(cfg, llama.AdamWConfig(), seq_len=S, global_batch=B, microbatch_size=MB)
    with torch.device("meta"):
        params = llama.init_params(cfg, device="meta")
        state = llama.init_opt_state(params)
    tok = torch.empty(B, S, dtype=torch.int64, device="meta")
    cos = torch.empty(S, cfg.head_dim // 2, device="meta")
    hashes = []
    for _ in range(2):
        mesh = mm.MultiMesh((4, 4), ("stage", "model"))
        llama.register_pipeline_tasks(cfg, mesh, num_stages=4)
        mock = C.MockContext(16)
        with mesh:
            exe = mm.compile_function(step, (params, state, tok, tok, cos, cos), mesh=mesh, context=mock,
                                      topology=Topology("cpu", 16))
        plan = exe.plan
        real = [torch.zeros(v["shape"]["sizes"], dtype=getattr(torch, v["shape"]["dtype"]))
                if sid >= 0 else None
                for sid, v in ((s, plan["stores"][s] if s >= 0 else None) for s in plan["param_stores"])]
        from torch.utils import _pytree as pytree
        args = pytree.tree_unflatten([r if r is not None else torch.zeros(1) for r in real], exe.cap.in_spec)
        exe(*args)
        assert mock.violation == "" and mock.hazard_report() == ""
        assert mock.num_tasks >= 16 * (2 * (B // MB) + 1) and mock.num_reshards > 0
        devices = {r["device"] for r in mock.event_log()}
        assert devices == set(range(16))
        assert 0 < mock.max_device_high_water < 64 << 20
        hashes.append((mock.operation_hash, plan["hash"]))
    assert hashes[0] == hashes[1]


@pytest.mark.parametrize("dp,pp,tp,layers", [(2, 2, 8, 4), (1, 8, 2, 8), (4, 4, 8, 4)],
                         ids=["DP2_PP2_TP8_32dev", "Pipeline8x2_16dev", "DP4_PP4_TP8_128dev"])
def test_multi_node_layouts_on_the_mock_runtime(dp, pp, tp, layers):
    """One process plans and 'runs' a multi-node job on virtual devices (the method of
    src/pjrt_client/mm_pjrt_executable_test.cc: DP2_PP2_TP8_4nodes, Pipeline2x8Stages, Gpt3_16nodes):
    the mock checks the protocol (local tiles exist, nothing is read while offloaded, writes stay on
    the task's device), the hazard checker replays the submissions, and all devices take part."""
    from multimesh_jax_b200.models import llama
    from multimesh_jax_b200.runtime.collectives import Topology
    n = dp * pp * tp
    cfg = llama.LlamaConfig.tiny(n_layers=layers, n_heads=8, n_kv_heads=8, d_model=64, d_ff=128, vocab=256)
    cfg.dtype = torch.float32
    B, S = 8 * dp, 8
    MB = 2 * dp
    step = llama.make_train_step(cfg, llama.AdamWConfig(), seq_len=S, global_batch=B, microbatch_size=MB)
    with torch.device("meta"):
        params = llama.init_params(cfg, device="meta")
        state = llama.init_opt_state(params)
    tok = torch.empty(B, S, dtype=torch.int64, device="meta")
    cos = torch.empty(S, cfg.head_dim // 2, device="meta")
    mesh = mm.MultiMesh((pp, dp, tp), ("stage", "data", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=pp)
    mock = C.MockContext(n)
    with mesh:
        exe = mm.compile_function(step, (params, state, tok, tok, cos, cos), mesh=mesh, context=mock,
                                  topology=Topology("cpu", n))
    plan = exe.plan
    from torch.utils import _pytree as pytree
    real = [torch.zeros(plan["stores"][s]["shape"]["sizes"], dtype=getattr(torch, plan["stores"][s]["shape"]["dtype"]))
            if s >= 0 else torch.zeros(1) for s in plan["param_stores"]]
    exe(*pytree.tree_unflatten(real, exe.cap.in_spec))
    assert mock.violation == "" and mock.hazard_report() == ""
    assert {r["device"] for r in mock.event_log()} == set(range(n))
    # every stage runs forward and backward of every microbatch on each of its devices
    per_device = mock.num_tasks / n
    assert per_device >= 2 * (B // MB)
    # tensor- and data-parallel ranks of a stage hold equal shares: the busiest device stays within
    # a small factor of the mean
    assert mock.max_device_high_water < 8 << 20
    stage_of = lambda d: d // (dp * tp)
    tasks_per_stage = {}
    for r in mock.event_log():
        if r["kind"] == 0:
            tasks_per_stage[stage_of(r["device"])] = tasks_per_stage.get(stage_of(r["device"]), 0) + 1
    assert set(tasks_per_stage) == set(range(pp))


def test_temporaries_are_handed_over_only_when_their_readers_are_ordered():
    """A task may free an input after its last use only if no other reader of that tile can run
    later than it: readers are not ordered among themselves, so a store that a reshard also reads
    (its body runs on another worker thread), or that a task outside the strict-order chains reads,
    stays in the table."""
    from multimesh_jax_b200.models import llama
    cfg = llama.LlamaConfig.tiny(n_layers=4, n_heads=4, n_kv_heads=2, d_model=64, d_ff=96, vocab=128)
    cfg.dtype = torch.float32
    B, S, MB = 8, 16, 2
    params = llama.init_params(cfg)
    state = llama.init_opt_state(params)
    tok = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, llama.AdamWConfig(), seq_len=S, global_batch=B, microbatch_size=MB)
    mesh = mm.MultiMesh((2, 1, 1), ("stage", "data", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=2)
    with mesh:
        exe = mm.compile_function(step, (params, state, tok, tok, cos, sin), mesh=mesh, backend="cpu")
    ops = exe.plan["ops"]
    reshard_sources = {op["src_store"] for op in ops if op["kind"] == "reshard"}
    handed_over = set().union(*exe._dying_inputs.values()) if exe._dying_inputs else set()
    assert handed_over, "nothing is freed early: the hand-over is switched off altogether"
    assert not (handed_over & reshard_sources)
    for k, stores in exe._dying_inputs.items():
        for sid in stores:
            readers = [op for op in ops if op["kind"] == "task" and sid in op["inputs"]]
            assert all(op["strict_ordering"] for op in readers)
            assert ops[k] is readers[-1]
    exe.shutdown()


# ---------------------------------------------------------------------------- CUDA context (against a recording stand-in)
def _fake_cuda_context(record=True):
    return C.CudaContext([0], [0], [0], fake=True, record_submissions=record)


def test_cuda_context_turns_cross_stream_conflicts_into_event_waits():
    """Tasks on one stream are ordered by the stream; a conflicting pair on two streams gets an
    event wait (and only such pairs do): producer (compute) -> reshard (communication) ->
    consumer (compute), then a task that overwrites the reshard's source."""
    c = _fake_cuda_context()
    assert c.fake_stream_priorities() == [-5, 0]           # communication stream: highest priority; auxiliary: lowest
    comm, aux = c.stream_handle(0, 1), c.stream_handle(0, 2)
    assert c.stream_handle(0, 0) == 0 and comm != aux
    ran = []
    c.open_window()
    c.create_execute_task(0, [], [(1, 0)], lambda: ran.append("produce"), "produce", True, 10, 0, 0)
    c.create_execute_task(0, [(1, 0)], [(5, 0)], lambda: ran.append("same-stream"), "same-stream", True, 10, 0, 0)
    c.reshard(0, [(1, 0)], [(2, 0)], lambda: ran.append("reshard"), "reshard", 0, 1)
    c.create_execute_task(0, [(2, 0)], [(3, 0)], lambda: ran.append("consume"), "consume", True, 10, 0, 0)
    c.create_execute_task(0, [], [(1, 0)], lambda: ran.append("overwrite"), "overwrite", False, 0, 0, 0)
    c.close_window()
    assert ran == ["produce", "same-stream", "reshard", "consume", "overwrite"]     # bodies run at submission, in plan order
    edges = [(e["from_name"], e["to_name"], e["from_stream"], e["to_stream"]) for e in c.edges()]
    assert ("produce", "reshard", 0, 1) in edges            # read after write across streams
    assert ("reshard", "consume", 1, 0) in edges            # read after write back on the compute stream
    assert ("reshard", "overwrite", 1, 0) in edges          # write after read
    assert not any(e[0] == "produce" and e[1] == "same-stream" for e in edges)     # same stream: no event
    trace = c.fake_trace()
    waits = [t for t in trace if t.startswith("wait")]
    assert f"wait s{comm} e1" in waits                      # the reshard's stream waits for the producer's event
    assert any(t.startswith("wait s0 ") for t in waits)
    # the window's end joins the communication stream into the compute stream
    assert trace[-2].startswith("wait s0 ") and trace[-1].startswith("record ") and trace[-1].endswith(" s0")
    assert c.hazard_report() == ""                          # every conflicting pair is ordered by a recorded edge
    c.shutdown()


def test_cuda_context_windows_scratch_and_status():
    c = _fake_cuda_context(record=False)
    for step in range(12):                                  # the stand-in's events complete at once: never more than 8 open
        c.open_window()
        c.create_execute_task(0, [], [(1, 0)], lambda: None, "t", False, 0, step, 0)
        c.close_window()
        assert c.open_windows <= 8
    assert c.host_blocks == 0
    base = c.reserve_scratch(0, 1000)
    assert base != 0 and c.scratch_bytes(0) >= 1000
    assert c.reserve_scratch(0, 500) == base                # never shrinks, never reallocates for a smaller task
    bigger = c.reserve_scratch(0, 8 << 20)
    assert bigger != 0 and c.scratch_bytes(0) >= (8 << 20)
    assert any(t.startswith("sync s") for t in c.fake_trace())    # the old tile was in use: streams drained before the free
    # a body that raises fails its step: later tasks of the step are skipped, the status names the cause
    ran = []

    def boom():
        raise RuntimeError("kernel launch refused")
    c.create_execute_task(0, [], [(1, 0)], boom, "bad", False, 0, 99, 0)
    c.create_execute_task(0, [(1, 0)], [(2, 0)], lambda: ran.append(1), "after", False, 0, 99, 0)
    status, msg = c.wait_all()
    assert status == C.Status.TASK_FAILED and "refused" in msg and ran == []
    c.reset_error()
    c.create_execute_task(0, [], [(1, 0)], lambda: ran.append(2), "next-step", False, 0, 100, 0)
    assert ran == [2] and c.wait_all()[0] == C.Status.OK
    c.inject_fault("throw", "victim", -1, 1, 0)
    c.create_execute_task(0, [], [(1, 0)], lambda: ran.append(3), "victim", False, 0, 101, 0)
    assert c.wait_all()[0] == C.Status.INJECTED_FAULT
    c.shutdown()


def test_a_reshard_is_not_held_up_by_a_task_that_waits_for_its_partner():
    """Two devices run one collective task each (the bodies wait for one another, as an exchange
    inside a task does). Device 1's half may only start once a reshard queued on device 0 has read
    the tile it overwrites - and device 0's task thread is already inside its half. Reshards run on
    a thread of their own per device, so the step ends; with one thread per device it could not."""
    ctx = C.ThreadedContext([0, 1], False, True)
    arrived = [threading.Event(), threading.Event()]
    outcome = {}

    def half(me):
        def body():
            arrived[me].set()
            outcome[me] = arrived[1 - me].wait(timeout=20.0)       # the partner must get here too
        return body

    X, Y = 0, 1
    ctx.create_execute_task(1, [], [(X, 1)], lambda: None, "produce")                    # tile X on device 1
    ctx.create_execute_task(0, [], [(Y, 0)], half(0), "collective", True)                # device 0 enters first ...
    ctx.reshard(0, [(X, 1)], [(Y + 1, 0)], lambda: time.sleep(0.05), "move X to device 0", 0)   # ... with this queued behind it
    ctx.create_execute_task(1, [], [(X, 1)], half(1), "collective", True)                # overwrites X: waits for the reshard
    status, message = ctx.wait_all()
    assert int(status) == 0, message
    assert outcome == {0: True, 1: True}
    assert ctx.hazard_report() == "" and ctx.pending_report() == []
    ctx.shutdown()
