"""Passes of the sharding half of the pipeline, run one at a time on hand-built graphs, with
assertions on what each pass alone leaves behind (the method of the reference's
mpmd_simple_loop_increment_coloring_test.cc, mpmd_logical_to_gspmd_sharding_test.cc,
mpmd_hoist_shard_map_reduce_test.cc, mpmd_shard_map_loop_reduce_test.cc and
mpmd_unused_param_output_remover_test.cc; the collective folding and the update cut have no test
file of their own there)."""
import json

import pytest

from multimesh_jax_b200 import _mm_C as C
from test_passes import G, task_json

TO_TASKS = ["coloring", "logical_sharding_propagation", "replicate_uncolored", "computation_grouper",
            "uniquify_colors"]
TO_LAYOUTS = ["logical_to_physical_sharding", "sharding_propagation_forward_io",
              "sharding_propagation_backward_io", "sharding_propagation_forward_full"]


def _run(c, passes):
    return {p: c.run(p) for p in passes}


def _ops(b):
    return [b.g.node(i)["op"] for i in b.g.order if not b.g.node(i).get("dead", False)]


def _layout(b, value):
    return b.g.value(value)["sharding"]["key"]


def _row_parallel(b):
    """x[4,16] split along its columns times w[16,8] split along its rows, on two devices."""
    t = task_json("T", [0, 1], logical=[("mlp", "x")])
    x, w = b.inp("x", [4, 16]), b.inp("w", [16, 8])
    b.g.set_value_axes(x, [[], ["mlp"]], True)
    b.g.set_value_axes(w, [["mlp"], []], True)
    y = b.op("aten.mm.default", [x, w], [4, 8], task=t)
    return t, x, w, y


def test_loop_increment_nodes_get_their_own_colour_only_when_asked():
    for on in (False, True):
        b = G(1)
        b.cfg.loop_increment_color = on
        b.g.add_loop(json.dumps({"id": 0, "num_microbatches": 2, "size": 1}))
        i = b.inp("i", [])
        inc = b.op("aten.add.Tensor", [i, i], [], loop=0, scope="step/loop_increment")
        other = b.op("aten.neg.default", [i], [], loop=0, scope="step/body")
        b.g.set_outputs([inc, other])
        c = b.compiler()
        assert c.run("simple_loop_increment_coloring") is on
        assert b.color_of(inc) == ("loop_increment" if on else "")
        assert b.color_of(other) == ""
        assert b.part.has("loop_increment") is on


def test_uncoloured_producer_is_cloned_once_per_consumer_colour():
    b = G(2)
    x = b.inp("x", [4])
    shared = b.op("aten.neg.default", [x], [4])                       # no colour: nobody voted for it
    a = b.op("aten.relu.default", [shared], [4], color="A")
    c_ = b.op("aten.exp.default", [shared], [4], color="B")
    b.part.add_task(task_json("A", [0]), False)
    b.part.add_task(task_json("B", [1]), False)
    b.g.set_outputs([a, c_])
    c = b.compiler()
    assert c.run("replicate_uncolored")
    negs = [i for i in b.g.order if b.g.node(i)["op"] == "aten.neg.default"]
    assert sorted(b.g.node(i)["color"] for i in negs) == ["A", "B"]
    # each consumer reads the copy of its own colour
    for v in (a, c_):
        n = b.g.node(b.g.value(v)["producer"])
        src = b.g.node(b.g.value(n["inputs"][0])["producer"])
        assert src["color"] == n["color"]


def test_uncoloured_node_that_is_a_result_becomes_global():
    b = G(2)
    x = b.inp("x", [4])
    r = b.op("aten.neg.default", [x], [4])
    b.g.set_outputs([r])
    c = b.compiler()
    assert c.run("replicate_uncolored") and b.color_of(r) == "global"


def test_logical_to_physical_fixes_annotated_values_and_leaves_single_device_tasks_alone():
    b = G(3)
    t, x, w, y = _row_parallel(b)
    one = b.op("aten.relu.default", [y], [4, 8], task=task_json("S", [2], logical=[("mlp", "x")]))
    b.g.set_value_axes(one, [["mlp"], []], True)
    b.g.set_outputs([one])
    c = b.compiler()
    _run(c, TO_TASKS)
    assert c.run("logical_to_physical_sharding")
    by_color = {g_["color"]: g_["id"] for g_ in c.groups()}
    gid = next(v for k, v in by_color.items() if k.endswith("T"))
    sid = next(v for k, v in by_color.items() if k.endswith("S"))
    xs, ws = c.input_sharding(gid, x), c.input_sharding(gid, w)
    assert xs["dim_axes"] == [[], [0]] and xs["shard_size"] == [4, 8]
    assert ws["dim_axes"] == [[0], []] and ws["shard_size"] == [8, 8]
    assert (xs["device_start"], xs["num_devices"]) == (0, 2)
    # the task on one device carries no layouts, whatever its values are annotated with
    assert c.input_sharding(sid, y) is None


def test_contracting_dimension_becomes_a_local_product_and_an_all_reduce():
    b = G(2)
    t, x, w, y = _row_parallel(b)
    z = b.op("aten.relu.default", [y], [4, 8], task=t)
    b.g.set_outputs([z])
    c = b.compiler()
    _run(c, TO_TASKS + TO_LAYOUTS)
    assert _ops(b) == ["aten.mm.default", "aten.relu.default"]
    assert c.run("spmd_lowering")
    assert _ops(b) == ["aten.mm.default", "mm.all_reduce", "aten.relu.default"]
    ar = next(b.g.node(i) for i in b.g.order if b.g.node(i)["op"] == "mm.all_reduce")
    assert json.loads(ar["attrs"]["axes"]) == [0]
    assert _layout(b, z) == "float32[4,8]m(2)@[0,2)"          # replicated after the reduction
    assert not c.run("hoist_shard_map_reduce")                # nothing to hoist outside a loop


def test_reduce_followed_by_a_slice_folds_into_a_reduce_scatter_and_the_gather_is_tagged():
    b = G(2)
    t, x, w, y = _row_parallel(b)
    w2 = b.inp("w2", [8, 16])
    rows = b.op("mm.relayout", [y], [4, 8], task=t)
    b.g.set_value_axes(rows, [["mlp"], []], True)            # sequence-parallel region
    act = b.op("aten.relu.default", [rows], [4, 8], task=t)
    full = b.op("mm.relayout", [act], [4, 8], task=t)
    b.g.set_value_axes(full, [[], []], True)
    z = b.op("aten.mm.default", [full, w2], [4, 16], task=t)
    b.g.set_outputs([z])
    c = b.compiler()
    _run(c, TO_TASKS + TO_LAYOUTS + ["spmd_lowering"])
    assert _ops(b).count("mm.all_reduce") == 1 and _ops(b).count("mm.spmd_reshard") == 2
    assert c.run("reduce_scatter_creator")
    ops = _ops(b)
    assert "mm.all_reduce" not in ops and ops.count("mm.reduce_scatter") == 1 and ops.count("mm.spmd_reshard") == 1
    rs = next(b.g.node(i) for i in b.g.order if b.g.node(i)["op"] == "mm.reduce_scatter")
    assert rs["attrs"]["dim"] == "0" and _layout(b, rs["outputs"][0]) == "float32[4/0,8]m(2)@[0,2)"
    ag = next(b.g.node(i) for i in b.g.order if b.g.node(i)["op"] == "mm.spmd_reshard")
    assert ag["attrs"]["gather_dim"] == "0" and json.loads(ag["attrs"]["gather_axes"]) == [0]
    assert _layout(b, act) == "float32[4/0,8]m(2)@[0,2)"     # the activation stays split between the two
    assert any("1 reduce-scatters, 1 all-gathers" in line for line in c.log())


def _data_parallel_step(b):
    """Two weight gradients accumulated over two microbatches, then one update per parameter."""
    la = [("batch", "x")]
    t, u = task_json("T", [0, 1], logical=la), task_json("U", [0, 1], logical=la)
    b.g.add_loop(json.dumps({"id": 0, "num_microbatches": 2, "size": 4}))
    x, dy = b.inp("x", [8, 16]), b.inp("dy", [8, 4])
    p1, p2 = b.inp("p1", [4, 16]), b.inp("p2", [16, 4])
    xs = b.op("mm.microbatch_slice.default", [x], [4, 16], loop=0, args=[0, 4, 0], task=t)
    ds = b.op("mm.microbatch_slice.default", [dy], [4, 4], loop=0, args=[0, 4, 0], task=t)
    b.g.set_value_axes(xs, [["batch"], []], True)
    b.g.set_value_axes(ds, [["batch"], []], True)
    dyt = b.op("aten.t.default", [ds], [4, 4], loop=0, task=t)
    dw1 = b.op("aten.mm.default", [dyt, xs], [4, 16], loop=0, task=t)
    xt = b.op("aten.t.default", [xs], [16, 4], loop=0, task=t)
    dw2 = b.op("aten.mm.default", [xt, ds], [16, 4], loop=0, task=t)
    a1 = b.op("mm.microbatch_out.default", [dw1], [4, 16], loop=0, args=[0, ""])
    a2 = b.op("mm.microbatch_out.default", [dw2], [16, 4], loop=0, args=[0, ""])
    n1 = b.op("aten.sub.Tensor", [p1, a1], [4, 16], task=u)
    n2 = b.op("aten.sub.Tensor", [p2, a2], [16, 4], task=u)
    b.g.set_outputs([n1, n2])
    return n1, n2


def _groups(b, c):
    return [(g_["color"], g_["region"], [b.g.node(n)["op"] for n in g_["nodes"] if not b.g.node(n).get("dead", False)])
            for g_ in c.groups()]


def test_hoisted_reductions_get_tasks_of_their_own_between_the_loop_and_the_update():
    b = G(2)
    _data_parallel_step(b)
    c = b.compiler()
    _run(c, ["microbatch_loop_canonicalizer"] + TO_TASKS + TO_LAYOUTS + ["spmd_lowering"])
    before = _groups(b, c)
    assert [r for _, r, _ in before] == [1, 2]
    assert before[0][2].count("mm.all_reduce") == 2           # one per microbatch and gradient
    assert c.run("hoist_shard_map_reduce")
    c.run("unused_param_output_remover")
    after = _groups(b, c)
    assert [r for _, r, _ in after] == [1, 2, 2, 2]
    assert "mm.all_reduce" not in after[0][2]
    assert after[1][2] == ["mm.all_reduce"] and after[2][2] == ["mm.all_reduce"]
    assert after[1][0].endswith("T_reduce") and after[2][0].endswith("T_reduce")
    assert after[3][2] == ["aten.sub.Tensor", "aten.sub.Tensor"]
    # the reductions read the accumulated sums, the update reads the reduced values
    for color, _, _ in after[1:3]:
        ar = next(b.g.node(i) for i in b.g.order if b.g.node(i)["color"] == color)
        assert b.g.node(b.g.value(ar["inputs"][0])["producer"])["op"] == "mm.accumulate"
        assert ar["attrs"]["hoisted"] == "1" and ar["loop"] == -1


@pytest.mark.parametrize("bucket,pieces", [("1", 2), ("1000000", 1), ("0", 1)])
def test_update_task_is_cut_behind_its_reductions_by_bucket_size(monkeypatch, bucket, pieces):
    monkeypatch.setenv("MULTIMESH_UPDATE_BUCKET_BYTES", bucket)
    b = G(2)
    n1, n2 = _data_parallel_step(b)
    c = b.compiler()
    _run(c, ["microbatch_loop_canonicalizer"] + TO_TASKS + TO_LAYOUTS +
         ["spmd_lowering", "hoist_shard_map_reduce", "reduce_scatter_creator"])
    assert c.run("split_update_by_reduction") is (pieces == 2)
    c.run("unused_param_output_remover")
    updates = [g_ for g_ in _groups(b, c) if g_[2] and set(g_[2]) == {"aten.sub.Tensor"}]
    assert len(updates) == pieces
    assert sum(len(g_[2]) for g_ in updates) == 2
    if pieces == 2:
        assert b.color_of(n1) != b.color_of(n2)
        assert any("cut into 2 pieces" in line for line in c.log())
    plan = c.build_plan()
    tasks = [op["name"] for op in plan["ops"] if op["kind"] == "task"]
    assert len(tasks) == 2 + 2 + pieces                       # two loop trips, two reductions, the update


def test_unused_param_output_remover_sweeps_dead_operators_and_empty_tasks():
    b = G(2)
    x = b.inp("x", [4])
    used = b.op("aten.relu.default", [x], [4], task=task_json("A", [0]))
    unused = b.op("aten.exp.default", [x], [4], task=task_json("B", [1]))
    b.g.set_outputs([used])
    c = b.compiler()
    _run(c, ["coloring", "computation_grouper"])
    assert len(c.groups()) == 2
    assert c.run("unused_param_output_remover")
    groups = c.groups()
    assert len(groups) == 1 and [b.g.node(n)["op"] for n in groups[0]["nodes"]] == ["aten.relu.default"]
    assert not c.run("unused_param_output_remover")           # nothing left to sweep
