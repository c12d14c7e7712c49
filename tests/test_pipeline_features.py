"""End-to-end pipeline features on virtual CPU devices, each against the eager step: 1F1B,
zero-bubble-H2 with split backward tasks, interleaved (circular) layer placement, a custom
schedule given per mesh, loop-dependent placement (a task that moves to another sub-mesh every
microbatch), inter-task recomputation, and the fast path for tiny functions."""
import pytest
import torch

import multimesh_jax_b200 as mm

D = 16


def _params():
    g = torch.Generator().manual_seed(0)
    return [torch.randn(D, D, generator=g) / D ** 0.5 for _ in range(4)]


def _data():
    g = torch.Generator().manual_seed(1)
    return torch.randn(8, D, generator=g), torch.randn(8, D, generator=g)


def _step(schedule, **mbkw):
    def loss_fn(params, batch):
        xb, yb = batch
        h = xb
        for i, w in enumerate(params):
            with mm.named_scope(f"blk.{i}"):
                h = torch.tanh(h @ w)
        with mm.named_scope("lossfn"):
            return ((h - yb) ** 2).sum()

    def step(params, batch):
        vg = mm.microbatch(mm.value_and_grad(loss_fn), size=2, argnum=1, schedule=schedule, **mbkw)
        return vg(params, batch)
    return step


def _stage_of(matched):
    return int(matched.split(".")[1]) // 2


def _two_stage(split=None):
    def factory(matched, backprop):
        s = _stage_of(matched)
        return mm.Task(name=f"stage{s}" + ("_bwd" if backprop else ""), mesh_slice={"stage": s}, split_backprop=split)
    return factory


def _loss_task(split=None):
    return lambda m, b: mm.Task(name="stage1" + ("_bwd" if b else ""), mesh_slice={"stage": 1}, split_backprop=split)


def _compile_and_check(step, block_factory, loss_factory):
    mesh = mm.MultiMesh((2,), ("stage",))
    mesh.register_task(r"(blk\.\d+)", factory=block_factory)
    mesh.register_task("(lossfn)", factory=loss_factory)
    params, batch = _params(), _data()
    with mesh:
        exe = mm.compile_function(step, (params, batch), mesh=mesh, backend="cpu")
    with mm.ignore_transforms():
        loss_ref, grads_ref = step(params, batch)
    loss, grads = exe(params, batch)
    torch.testing.assert_close(loss.full_tensor(), loss_ref, rtol=1e-5, atol=1e-5)
    for a, b in zip(grads, grads_ref):
        torch.testing.assert_close(a.full_tensor(), b, rtol=1e-5, atol=1e-5)
    return exe


def _names(exe):
    return {t["name"].split(".", 1)[1] for t in exe.plan["templates"]}


def _order(exe, device):
    tm = {t["id"]: t["name"].split(".", 1)[1] for t in exe.plan["templates"]}
    return [(tm[op["template"]], op["scalars"][0] // 2 if op["scalars"] else -1) for op in exe.plan["ops"]
            if op["kind"] == "task" and op["device_start"] <= device < op["device_start"] + op["num_devices"]]


def test_one_forward_one_backward():
    exe = _compile_and_check(_step("1f1b"), _two_stage(), _loss_task())
    order = _order(exe, 1)      # last stage alternates forward and backward of the same microbatch
    fb = [(n, i) for n, i in order if n in ("stage1_loop", "stage1_bwd_loop")]
    assert fb[:4] == [("stage1_loop", 0), ("stage1_bwd_loop", 0), ("stage1_loop", 1), ("stage1_bwd_loop", 1)]
    exe.shutdown()


def test_zero_bubble_splits_the_backward_task():
    split = ("_act", "_wgt")
    exe = _compile_and_check(_step("zero-bubble-h2"), _two_stage(split), _loss_task(split))
    names = _names(exe)
    assert {"stage1_bwd_act_loop", "stage1_bwd_wgt_loop"} <= names
    order = _order(exe, 1)
    pos = {e: k for k, e in enumerate(order)}
    for i in range(4):   # activation gradients (critical path) run before the weight gradients of the microbatch
        assert pos[("stage1_bwd_act_loop", i)] < pos[("stage1_bwd_wgt_loop", i)]
    exe.shutdown()


def test_interleaved_layer_placement():
    def factory(matched, backprop):
        i = int(matched.split(".")[1])
        return mm.Task(name=f"v{i}" + ("_bwd" if backprop else ""), mesh_slice={"stage": i % 2})
    exe = _compile_and_check(_step("1f1b"), factory, _loss_task())
    where = {t["name"].split(".", 1)[1]: t["device_start"] for t in exe.plan["templates"]}
    assert [where[f"v{i}_loop"] for i in range(4)] == [0, 1, 0, 1]   # every microbatch visits each device twice
    exe.shutdown()


def test_custom_schedule_per_mesh():
    rows = [[(0, "stage0_loop"), (1, "stage0_loop"), (2, "stage0_loop"), (3, "stage0_loop"),
             (0, "stage0_bwd"), (1, "stage0_bwd"), (2, "stage0_bwd"), (3, "stage0_bwd")],
            [(0, "stage1_loop"), (0, "stage1_bwd"), (1, "stage1_loop"), (1, "stage1_bwd"),
             (2, "stage1_loop"), (2, "stage1_bwd"), (3, "stage1_loop"), (3, "stage1_bwd")]]
    try:
        exe = _compile_and_check(_step("custom", custom_schedule=rows), _two_stage(), _loss_task())
    except RuntimeError as e:   # names are matched against task colours: report what exists
        pytest.fail(str(e))
    # stage 0 runs fill-drain (all forwards first), stage 1 one-forward-one-backward: as written
    order0 = [n for n, _ in _order(exe, 0) if n.startswith("stage0")]
    assert order0 == ["stage0_loop"] * 4 + ["stage0_bwd_loop"] * 4
    order1 = [e for e in _order(exe, 1) if e[0] in ("stage1_loop", "stage1_bwd_loop")]
    assert order1[:4] == [("stage1_loop", 0), ("stage1_bwd_loop", 0), ("stage1_loop", 1), ("stage1_bwd_loop", 1)]
    # an order that breaks the microbatch order of a stage is refused
    bad = [list(reversed(rows[0])), rows[1]]
    with pytest.raises(RuntimeError, match="contradicts"):
        _compile_and_check(_step("custom", custom_schedule=bad), _two_stage(), _loss_task())
    exe.shutdown()


def test_loop_dependent_placement_moves_a_task_between_submeshes():
    def factory(matched, backprop):
        if matched == "blk.0" and not backprop:
            return mm.Task(name="rr", mesh_slice={"stage": 0}, loop_dependent_mesh_slice=lambda i: {"stage": i % 2})
        return _two_stage()(matched, backprop)
    exe = _compile_and_check(_step("1f1b"), factory, _loss_task())
    tm = {t["id"]: t["name"].split(".", 1)[1] for t in exe.plan["templates"]}
    starts = [op["device_start"] for op in exe.plan["ops"] if op["kind"] == "task" and tm[op["template"]] == "rr_loop"]
    assert sorted(starts) == [0, 0, 1, 1] and len(set(starts)) == 2
    exe.shutdown()


def test_recomputation_between_tasks_keeps_results():
    with mm.enable_recomputation(True):
        exe = _compile_and_check(_step("gpipe"), _two_stage(), _loss_task())
    exe.shutdown()


def test_fast_path_runs_tiny_functions_without_the_mpmd_runtime():
    """One small task without markers is dispatched to the wrapper executable: no task-graph
    context exists, nothing is submitted, and the result is the plain function's. With the fast
    path switched off the same function goes through the partitioned executable."""
    from multimesh_jax_b200.runtime.wrapper import WrapperExecutable

    def tiny(a, b):
        return a * 2 + b
    a, b = torch.ones(4), torch.arange(4.0)
    before = WrapperExecutable.total_calls
    with mm.enable_fast_path(True):
        exe = mm.compile_function(tiny, (a, b), num_devices=2, backend="cpu")
        assert isinstance(exe, WrapperExecutable) and exe.reason == "fast-path" and exe.context is None
        out = exe(a, b)
        f = mm.mjit(tiny, backend="cpu")
        out2 = f(a, b)
    assert WrapperExecutable.total_calls == before + 2
    assert isinstance(out, mm.ShardedTensor) and sorted(out.local_tiles()) == [0, 1]     # replicated on the assignment
    assert torch.equal(out.full_tensor(), a * 2 + b) and torch.equal(out2.full_tensor(), a * 2 + b)
    with mm.enable_fast_path(False):
        slow = mm.compile_function(tiny, (a, b), num_devices=2, backend="cpu")
    assert isinstance(slow, mm.Executable) and slow.context is not None
    got = slow(a, b)
    assert torch.equal(got.full_tensor(), a * 2 + b)
    assert slow.launches > 0 and WrapperExecutable.total_calls == before + 2
    slow.shutdown()


def test_single_device_programs_without_markers_bypass_the_mpmd_runtime():
    """A device assignment of one device and nothing to partition: the wrapper runs the captured
    graph even when it is larger than the fast-path limit; an explicit task, a microbatch loop
    or a donated argument keeps the partitioned executable."""
    from multimesh_jax_b200.runtime.wrapper import WrapperExecutable

    def big(x):
        for i in range(30):
            x = torch.tanh(x) + i
        return x.sum()
    x = torch.randn(8)
    exe = mm.compile_function(big, (x,), num_devices=1, backend="cpu")
    assert isinstance(exe, WrapperExecutable) and exe.reason == "single-device"
    torch.testing.assert_close(exe(x).full_tensor(), big(x))
    # the same program on two devices is partitioned (one task, replicated)
    two = mm.compile_function(big, (x,), num_devices=2, backend="cpu")
    assert isinstance(two, mm.Executable)
    torch.testing.assert_close(two(x).full_tensor(), big(x))
    two.shutdown()

    def tasked(x):
        return mm.task(lambda t: t * 2, name="dbl", devices=[0])(x).sum()
    assert isinstance(mm.compile_function(tasked, (x,), num_devices=1, backend="cpu"), mm.Executable)
    donated = mm.compile_function(big, (x,), num_devices=1, backend="cpu", donate_argnums=(0,))
    assert isinstance(donated, mm.Executable)


def test_zero_arguments_option_zeroes_hoisted_parameter_casts():
    """With hoisted parameter casts switched on and the zero-arguments debugging option set, the
    cast of a weight (done once per step, outside the microbatch loop) yields zeros: the loss of
    ``sum((x @ w.to(float64)) ** 2)`` becomes 0 while the untouched run matches eager."""
    from multimesh_jax_b200 import _mm_C

    def loss_fn(w, batch):
        with mm.named_scope("blk.0"):
            return ((batch @ w.to(torch.float64)) ** 2).sum()

    def step(w, batch):
        return mm.microbatch(loss_fn, size=2, argnum=1, schedule="gpipe")(w, batch)

    torch.manual_seed(0)
    w, x = torch.randn(D, D), torch.randn(8, D, dtype=torch.float64)
    results = {}
    for zero in (False, True):
        mesh = mm.MultiMesh((1,), ("stage",))
        mesh.register_task(r"(blk\.\d+)", task=mm.Task(mesh_slice={"stage": 0}))
        with mesh:
            exe = mm.compile_function(step, (w, x), mesh=mesh, backend="cpu",
                                      config_overrides={"hoist_loop_convert": True, "zero_arguments": zero})
        results[zero] = float(exe(w, x).full_tensor())
        g = exe.cap.graph
        casts = [g.node(n) for t in exe.plan["templates"] for n in t["nodes"] if g.node(n)["op"].startswith("aten._to_copy")]
        assert casts and all(c["loop"] < 0 for c in casts)           # hoisted out of the loop
        exe.shutdown()
    with mm.ignore_transforms():
        ref = float(step(w, x))
    assert abs(results[False] - ref) < 1e-6 * abs(ref) and results[True] == 0.0


def test_lifetime_checking_catches_two_live_stores_in_one_buffer(monkeypatch):
    """MM_CHECK_LIFETIMES=1: the compiler's buffer plan passes on a real pipeline; a plan that is
    corrupted so that a stage-boundary activation shares its buffer with a later store is caught
    when the overwritten store is read, naming both stores."""
    monkeypatch.setenv("MM_CHECK_LIFETIMES", "1")
    exe = _compile_and_check(_step("1f1b"), _two_stage(), _loss_task())      # numerics checked with the knob on
    assert exe._lifetimes and exe._owner
    plan = exe.plan
    # find two TEMP stores of equal layout that are alive at the same time: an input of some task
    # and a store written between that input's definition and the task
    ops = [op for op in plan["ops"] if op["kind"] == "task"]
    victim = None
    for k, op in enumerate(ops):
        for sid in op["inputs"]:
            st = plan["stores"][sid]
            if st["kind"] != "TEMP":
                continue
            first_def = next((j for j, o in enumerate(ops) if sid in o["outputs"]), None)
            if first_def is None:
                continue
            for j in range(first_def + 1, k):
                for other in ops[j]["outputs"]:
                    so = plan["stores"][other]
                    if (so["kind"] == "TEMP" and other != sid and so["shape"]["key"] == st["shape"]["key"]
                            and exe.buffer_of[other] != exe.buffer_of[sid]):
                        victim = (sid, other)
                        break
                if victim:
                    break
            if victim:
                break
        if victim:
            break
    assert victim is not None
    sid, other = victim
    exe.buffer_of[other] = exe.buffer_of[sid]                  # the corrupted plan: both stores in one buffer
    exe.tiles[other] = exe.tiles[sid]
    with pytest.raises(mm.StepFailed, match="buffer plan lets two live stores share a buffer"):
        loss, grads = exe(_params(), _data())
        loss.wait()
        exe.wait()
    exe.shutdown()


def test_task_and_reshard_bodies_are_built_once_and_reused_by_later_steps():
    exe = _compile_and_check(_step("1f1b"), _two_stage(), _loss_task())     # first step ran in the helper
    ops = exe.plan["ops"]
    n_tasks = sum(op["num_devices"] for op in ops if op["kind"] == "task")
    n_reshards = sum(1 for op in ops if op["kind"] == "reshard")
    assert len(exe._task_entries) == n_tasks and len(exe._reshard_entries) == n_reshards
    bodies = {key: entry[2] for key, entry in exe._task_entries.items()}
    moves = {k: [e[3] for e in entries] for k, entries in exe._reshard_entries.items()}
    params, batch = _params(), _data()
    with mm.ignore_transforms():
        loss_ref, grads_ref = _step("1f1b")(params, batch)
    for _ in range(2):                       # later steps: same closures, fresh results
        loss, grads = exe(params, batch)
        torch.testing.assert_close(loss.full_tensor(), loss_ref, rtol=1e-5, atol=1e-5)
        for a, b in zip(grads, grads_ref):
            torch.testing.assert_close(a.full_tensor(), b, rtol=1e-5, atol=1e-5)
    assert all(exe._task_entries[key][2] is body for key, body in bodies.items())
    assert all([e[3] for e in exe._reshard_entries[k]] == m for k, m in moves.items())
    # a different input gives a different result through the same bodies
    x, y = batch
    loss2, _ = exe(params, (x * 2.0, y))
    assert abs(float(loss2.full_tensor()) - float(loss_ref)) > 1e-3
    exe.shutdown()


def test_microbatches_cut_along_an_inner_dimension_feed_views():
    """Microbatches taken along dimension 1: the slice is not one block of memory, the projection
    behind it flattens its operand with a view (found by a randomised run)."""
    g = torch.Generator().manual_seed(0)
    w = torch.randn(D, D, generator=g) / D ** 0.5
    x, y = torch.randn(4, 6, D, generator=g), torch.randn(4, 6, D, generator=g)

    def loss_fn(w, batch):
        xb, yb = batch
        with mm.named_scope("blk.0"):
            h = torch.tanh(xb @ w)
        with mm.named_scope("lossfn"):
            return ((h - yb) ** 2).sum()

    def step(w, batch):
        return mm.microbatch(mm.value_and_grad(loss_fn), dim=1, size=2, argnum=1, schedule="gpipe")(w, batch)

    mesh = mm.MultiMesh((2,), ("stage",))
    mesh.register_task(r"(blk\.\d+)", task=mm.Task(name="s0", mesh_slice={"stage": 0}))
    mesh.register_task("(lossfn)", factory=lambda m, b: mm.Task(name="s1" + ("_bwd" if b else ""), mesh_slice={"stage": 1}))
    with mesh:
        exe = mm.compile_function(step, (w, (x, y)), mesh=mesh, backend="cpu")
    loss, grad = exe(w, (x, y))
    with mm.ignore_transforms():
        ref_loss, ref_grad = step(w, (x, y))
    torch.testing.assert_close(loss.full_tensor(), ref_loss, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(grad.full_tensor(), ref_grad, rtol=1e-4, atol=1e-5)
    offsets = {op["scalars"][0] for op in exe.plan["ops"] if op["kind"] == "task" and op["scalars"]}
    assert offsets == {0, 2, 4}                                   # three microbatches of two columns of dimension 1
    exe.shutdown()
