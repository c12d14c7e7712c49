"""Pass-level tests of the MPMD compiler on small hand-built graphs (the method of the
reference's per-pass gtest files: build a tiny module, register tasks, run one pass or the whole
pipeline on N virtual devices, assert on colours, devices, stores and the operation list)."""
import json

import pytest

from multimesh_jax_b200 import _mm_C as C

F32 = "float32"


def task_json(name, devices, dims=None, axes=None, logical=(), split=()):
    return json.dumps({"name": name, "devices": devices, "dims": dims or [len(devices)],
                       "device_axes": axes or ["x"], "logical_axes": [list(p) for p in logical],
                       "split_backprop": list(split), "loop_dependent_devices": []})


class G:
    """Small builder around the native graph."""

    def __init__(self, num_devices=2):
        self.g = C.Graph()
        self.part = C.Partition(0, num_devices)
        self.cfg = C.PartitionConfig()

    def inp(self, name, shape, dtype=F32):
        return self.g.add_input(name, shape, dtype)

    def op(self, op, inputs, shape, *, scope="", backprop=False, loop=-1, task="", color="", args=None, dtype=F32,
           attrs=None):
        a = {"args": json.dumps(args or [])}
        a.update(attrs or {})
        nid, outs = self.g.add_node(op, inputs, [shape], [dtype], a, scope, backprop, loop, task, color)
        return outs[0]

    def compiler(self):
        return C.Compiler(self.g, self.part, self.cfg)

    def colors(self):
        return {self.g.node(i)["op"] + "#" + str(i): self.g.node(i)["color"] for i in self.g.order}

    def color_of(self, value):
        return self.g.node(self.g.value(value)["producer"])["color"]


def two_stage_graph(b, loop=False):
    """x -> [stage0: relu, mm] -> [stage1: gelu, sum]"""
    x = b.inp("x", [4, 8])
    w = b.inp("w", [8, 8])
    lp = 0 if loop else -1
    if loop:
        b.g.add_loop(json.dumps({"id": 0, "num_microbatches": 2, "slice_dim": 0, "size": 2, "schedule": "gpipe"}))
        x = b.op("mm.microbatch_slice.default", [x], [2, 8], loop=0, args=[0, 2, 0])
    rows = 2 if loop else 4
    h = b.op("aten.relu.default", [x], [rows, 8], task=task_json("s0", [0]), loop=lp)
    h = b.op("aten.mm.default", [h, w], [rows, 8], task=task_json("s0", [0]), loop=lp)
    y = b.op("aten.gelu.default", [h], [rows, 8], task=task_json("s1", [1]), loop=lp)
    z = b.op("aten.sum.default", [y], [], task=task_json("s1", [1]), loop=lp)
    if loop:
        z = b.op("mm.microbatch_out.default", [z], [], loop=0, args=[0, ""])
    b.g.set_outputs([z])
    return z


# ---------------------------------------------------------------------------- colouring
def test_explicit_tasks_and_backward_suffix():
    b = G()
    x = b.inp("x", [4])
    f = b.op("aten.relu.default", [x], [4], task=task_json("layer", [0]))
    g_ = b.op("aten.threshold_backward.default", [f, f], [4], task=task_json("layer", [0]), backprop=True)
    b.g.set_outputs([g_])
    c = b.compiler()
    c.run("coloring")
    assert b.color_of(f) == "layer" and b.color_of(g_) == "layer_bwd"
    assert b.part.color("layer_bwd")["backprop"]


def test_regex_tasks_innermost_registration_wins_and_backprop_flag():
    b = G(4)
    calls = []

    def outer(matched, backprop):
        calls.append(("outer", matched, backprop))
        return task_json("", [0, 1])

    def inner(matched, backprop):
        calls.append(("inner", matched, backprop))
        return task_json(f"{matched}_{'b' if backprop else 'f'}", [2, 3])

    b.part.register_task_factory("(layer1)", inner)        # innermost first
    b.part.register_task_factory(r"(layer\d)", outer)
    x = b.inp("x", [4])
    a0 = b.op("aten.relu.default", [x], [4], scope="model/layer0/act")
    a1 = b.op("aten.relu.default", [a0], [4], scope="model/layer1/act")
    g1 = b.op("aten.neg.default", [a1], [4], scope="model/layer1/act", backprop=True)
    b.g.set_outputs([g1])
    b.compiler().run("coloring")
    assert b.color_of(a0) == "layer0" and b.color_of(a1) == "layer1_f" and b.color_of(g1) == "layer1_b"
    assert b.part.color("layer0")["num_devices"] == 2 and b.part.color("layer1_f")["device_start"] == 2
    # callbacks are cached per (matched name, backprop)
    assert sorted(calls) == [("inner", "layer1", False), ("inner", "layer1", True), ("outer", "layer0", False)]


def test_one_colour_cannot_map_to_two_device_lists():
    b = G(4)
    x = b.inp("x", [4])
    a = b.op("aten.relu.default", [x], [4], task=task_json("t", [0]))
    c_ = b.op("aten.relu.default", [a], [4], task=task_json("t", [1]))
    b.g.set_outputs([c_])
    with pytest.raises(RuntimeError, match="two different device lists"):
        b.compiler().run("coloring")


def test_noncontiguous_devices_are_rejected():
    b = G(4)
    x = b.inp("x", [4])
    a = b.op("aten.relu.default", [x], [4], task=task_json("t", [0, 2]))
    b.g.set_outputs([a])
    with pytest.raises(RuntimeError, match="contiguous"):
        b.compiler().run("coloring")


def test_neighbour_voting_colours_unannotated_nodes_and_favours_heavy_edges():
    b = G()
    x = b.inp("x", [64, 64])
    a = b.op("aten.relu.default", [x], [64, 64], task=task_json("big", [0]))
    s = b.op("aten.sum.default", [x], [], task=task_json("small", [1]))
    # uncoloured elementwise node with a heavy edge to `big` and a scalar edge to `small`
    m = b.op("aten.mul.Tensor", [a, s], [64, 64])
    out = b.op("aten.neg.default", [m], [64, 64])
    b.g.set_outputs([out])
    b.compiler().run("coloring")
    assert b.color_of(m) == "big" and b.color_of(out) == "big"


def test_forward_propagation_in_loops_favours_most_recent_operand():
    b = G()
    b.g.add_loop(json.dumps({"id": 0, "num_microbatches": 2, "size": 1}))
    x = b.inp("x", [4, 4])
    s = b.op("mm.microbatch_slice.default", [x], [2, 4], loop=0, args=[0, 2, 0])
    a = b.op("aten.relu.default", [s], [2, 4], task=task_json("early", [0]), loop=0)
    c_ = b.op("aten.gelu.default", [a], [2, 4], task=task_json("late", [1]), loop=0)
    u = b.op("aten.add.Tensor", [a, c_], [2, 4], loop=0)
    o = b.op("mm.microbatch_out.default", [u], [2, 4], loop=0, args=[0, ""])
    b.g.set_outputs([o])
    c = b.compiler()
    c.run("microbatch_loop_canonicalizer")
    c.run("coloring")
    assert b.color_of(u) == "late" and b.color_of(s) == "early" and b.color_of(o) == "late"


def test_backward_colouring_does_not_overwrite_and_roots_get_global_colour():
    b = G()
    x = b.inp("x", [4])
    a = b.op("aten.relu.default", [x], [4], task=task_json("t0", [0]))
    pre = b.op("aten.exp.default", [x], [4])              # feeds only the coloured node b2
    b2 = b.op("aten.add.Tensor", [a, pre], [4], task=task_json("t1", [1]))
    lonely = b.op("aten.cos.default", [x], [4])           # reaches an output through nothing coloured
    b.g.set_outputs([b2, lonely])
    b.compiler().run("coloring")
    assert b.color_of(a) == "t0" and b.color_of(b2) == "t1"
    assert b.color_of(pre) in ("t1", "")                  # parameter-derived: recomputed in its consumer
    assert b.color_of(lonely) in ("global", "")


# ------------------------------------------------------------------- grouping and fusion
def test_grouper_builds_one_task_per_colour_run_and_fusion_merges_split_runs():
    b = G()
    x = b.inp("x", [4])
    a1 = b.op("aten.relu.default", [x], [4], task=task_json("A", [0]))
    b1 = b.op("aten.relu.default", [x], [4], task=task_json("B", [1]))
    a2 = b.op("aten.neg.default", [a1], [4], task=task_json("A", [0]))
    b2 = b.op("aten.neg.default", [b1], [4], task=task_json("B", [1]))
    out = b.op("aten.add.Tensor", [a2, b2], [4], task=task_json("B", [1]))
    b.g.set_outputs([out])
    c = b.compiler()
    c.run("coloring")
    c.run("computation_grouper")
    groups = c.groups()
    assert [g_["color"] for g_ in groups] == ["A", "B"]      # colour-sticky order keeps runs together
    assert sum(len(g_["nodes"]) for g_ in groups) == 5


def test_fusion_does_not_merge_across_a_dependency():
    b = G()
    x = b.inp("x", [4])
    a1 = b.op("aten.relu.default", [x], [4], task=task_json("A", [0]))
    m = b.op("aten.neg.default", [a1], [4], task=task_json("B", [1]))
    a2 = b.op("aten.exp.default", [m], [4], task=task_json("A", [0]))
    b.g.set_outputs([a2])
    c = b.compiler()
    for p in ("coloring", "computation_grouper", "computation_fusion_matching_color"):
        c.run(p)
    assert [g_["color"] for g_ in c.groups()] == ["A", "B", "A"]


def test_device_fusion_merges_loop_tasks_on_the_same_devices_only():
    b = G()
    b.g.add_loop(json.dumps({"id": 0, "num_microbatches": 2, "size": 1}))
    x = b.inp("x", [2, 4])
    s = b.op("mm.microbatch_slice.default", [x], [1, 4], loop=0, args=[0, 1, 0])
    a = b.op("aten.relu.default", [s], [1, 4], task=task_json("A", [0]), loop=0)
    a2 = b.op("aten.neg.default", [a], [1, 4], task=task_json("A2", [0]), loop=0)
    c_ = b.op("aten.exp.default", [a2], [1, 4], task=task_json("C", [1]), loop=0)
    o = b.op("mm.microbatch_out.default", [c_], [1, 4], loop=0, args=[0, ""])
    b.g.set_outputs([o])
    c = b.compiler()
    for p in ("microbatch_loop_canonicalizer", "coloring", "computation_grouper", "computation_fusion_matching_devices"):
        c.run(p)
    assert [g_["color"] for g_ in c.groups()] == ["A", "C"]


def test_uniquify_gives_every_task_its_own_colour_and_remembers_the_original():
    b = G()
    z = two_stage_graph(b)
    c = b.compiler()
    for p in ("coloring", "computation_grouper", "uniquify_colors"):
        c.run(p)
    names = [g_["color"] for g_ in c.groups()]
    assert names == ["0.s0", "1.s1"]
    assert b.part.color("0.s0")["original"] == "s0"


# ------------------------------------------------------------------- whole pipeline
def test_whole_pipeline_two_stages_inserts_one_reshard():
    b = G()
    two_stage_graph(b)
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    kinds = [op["kind"] for op in plan["ops"]]
    # one reshard carries the activation to stage 1, one broadcasts the scalar result
    assert kinds.count("task") == 2 and kinds.count("reshard") == 2
    t0, t1 = [op for op in plan["ops"] if op["kind"] == "task"]
    assert (t0["device_start"], t1["device_start"]) == (0, 1)
    # parameters live where their first consumer runs; the scalar result is broadcast to all devices
    stores = plan["stores"]
    assert stores[plan["param_stores"][0]]["shape"]["device_start"] == 0
    root = stores[plan["root_stores"][0]]
    assert root["scalar"] and root["shape"]["num_devices"] == 2


def test_microbatch_loop_unrolls_per_iteration_and_accumulates():
    b = G()
    two_stage_graph(b, loop=True)
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    tasks = [op for op in plan["ops"] if op["kind"] == "task"]
    assert len(tasks) == 4 and [t["iteration"] for t in tasks] == [0, 1, 0, 1]      # gpipe: stage major
    assert [t["scalars"] for t in tasks if t["name"].endswith("s0_loop")] == [[0], [2]]
    acc = [t["accumulate"] for t in tasks if t["name"].endswith("s1_loop")]
    assert acc == [[1], [2]]                                                         # first write, then +=
    # both iterations of stage 1 write the same accumulator store
    outs = [t["outputs"] for t in tasks if t["name"].endswith("s1_loop")]
    assert outs[0] == outs[1]


def test_loop_value_escaping_without_sum_is_an_error():
    b = G()
    b.g.add_loop(json.dumps({"id": 0, "num_microbatches": 2, "size": 1}))
    x = b.inp("x", [2, 4])
    s = b.op("mm.microbatch_slice.default", [x], [1, 4], loop=0, args=[0, 1, 0])
    bad = b.op("aten.relu.default", [s], [1, 4])       # outside the loop, reads a loop value
    b.g.set_outputs([bad])
    with pytest.raises(RuntimeError, match="used outside"):
        b.compiler().run("microbatch_loop_canonicalizer")


def test_constant_and_repeated_outputs_get_their_own_buffers():
    b = G(1)
    x = b.inp("x", [4])
    y = b.op("aten.relu.default", [x], [4], task=task_json("t", [0]))
    b.g.set_outputs([x, y, y])
    c = b.compiler()
    assert c.run("constant_output_copy") and c.run("repeated_output_copy")
    outs = b.g.outputs
    assert len(set(outs)) == 3 and all(b.g.node(b.g.value(o)["producer"])["op"] == "mm.copy" for o in (outs[0], outs[2]))


def test_common_reshard_is_deduplicated_per_target_layout():
    b = G(3)
    x = b.inp("x", [4])
    a = b.op("aten.relu.default", [x], [4], task=task_json("A", [0]))
    u1 = b.op("aten.neg.default", [a], [4], task=task_json("B", [1]))
    u2 = b.op("aten.exp.default", [a], [4], task=task_json("B2", [1]))
    u3 = b.op("aten.cos.default", [a], [4], task=task_json("C", [2]))
    out = b.op("aten.add.Tensor", [u1, u2], [4], task=task_json("B2", [1]))
    b.g.set_outputs([out, u3])
    b.cfg.use_task_fusion = False
    b.cfg.argument_recompute = False
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    reshards = [op for op in plan["ops"] if op["kind"] == "reshard"]
    from_a = [r for r in reshards if plan["stores"][r["src_store"]]["value"] == a]
    assert len(from_a) == 2          # one per destination device, shared by B and B2
    # reshards are hoisted right after the producer
    ops = plan["ops"]
    first_task = next(i for i, op in enumerate(ops) if op["kind"] == "task")
    assert ops[first_task + 1]["kind"] == "reshard" and ops[first_task + 2]["kind"] == "reshard"


def test_same_devices_different_sharding_needs_a_reshard():
    b = G(2)
    la = [("rows", "x")]
    x = b.inp("x", [4, 4])
    a = b.op("aten.relu.default", [x], [4, 4], task=task_json("A", [0, 1], logical=la))
    c_ = b.op("aten.neg.default", [a], [4, 4], task=task_json("B", [0, 1], logical=[("cols", "x")]))
    b.g.set_value_axes(a, [["rows"], []], True)
    b.g.set_value_axes(c_, [[], ["cols"]], True)
    b.g.set_outputs([c_])
    b.cfg.use_task_fusion = False
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    assert any(op["kind"] == "reshard" for op in plan["ops"]) or \
        any(C.Graph.node(b.g, n)["op"] == "mm.spmd_reshard" for t in plan["templates"] for n in t["nodes"])


def test_buffer_names_are_reused_once_a_temporary_is_dead():
    b = G(1)
    x = b.inp("x", [8, 8])
    w = b.inp("w", [8, 8])
    cur = x
    for i in range(6):  # a chain of single-device tasks: only two temporaries are ever live
        cur = b.op("aten.mm.default", [cur, w], [8, 8], task=task_json(f"t{i}", [0]))
    b.g.set_outputs([cur])
    b.cfg.use_task_fusion = False
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    temp_names = {s["name"] for s in plan["stores"] if s["kind"] == "TEMP"}
    assert len([s for s in plan["stores"] if s["kind"] == "TEMP"]) == 5 and len(temp_names) <= 3


def test_donated_parameter_aliases_the_matching_output():
    b = G(1)
    p = b.inp("p", [8])
    g_ = b.inp("g", [8])
    new_p = b.op("aten.sub.Tensor", [p, g_], [8], task=task_json("opt", [0]))
    b.g.set_outputs([new_p])
    b.g.set_donated_inputs([0])
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    assert plan["aliases"] == [(plan["param_stores"][0], plan["root_stores"][0])]


def test_argument_recompute_clones_cheap_producers_into_the_consumer():
    b = G()
    x = b.inp("x", [4])
    cheap = b.op("aten.exp.default", [x], [4], task=task_json("A", [0]))
    a_out = b.op("aten.relu.default", [cheap], [4], task=task_json("A", [0]))
    use = b.op("aten.add.Tensor", [cheap, a_out], [4], task=task_json("B", [1]))
    b.g.set_outputs([use])
    c = b.compiler()
    for p in ("coloring", "computation_grouper", "argument_recompute"):
        c.run(p)
    producers = [b.g.node(b.g.value(v)["producer"]) for v in b.g.node(b.g.value(use)["producer"])["inputs"]]
    assert any(p["op"] == "aten.exp.default" and p["color"] == "B" for p in producers)
    b.cfg.argument_recompute = False


def test_recomputation_can_be_switched_off():
    b = G()
    b.cfg.enable_recomputation = False
    x = b.inp("x", [4])
    cheap = b.op("aten.exp.default", [x], [4], task=task_json("A", [0]))
    use = b.op("aten.neg.default", [cheap], [4], task=task_json("B", [1]))
    b.g.set_outputs([use])
    c = b.compiler()
    for p in ("coloring", "computation_grouper"):
        c.run(p)
    assert not c.run("argument_recompute")


def test_cut_size_minimizer_moves_expanding_ops_to_the_consumer():
    b = G()
    x = b.inp("x", [1, 8])
    small = b.op("aten.relu.default", [x], [1, 8], task=task_json("A", [0]))
    big = b.op("aten.expand.default", [small], [64, 8], task=task_json("A", [0]), args=[[64, 8]])
    use = b.op("aten.neg.default", [big], [64, 8], task=task_json("B", [1]))
    b.g.set_outputs([use])
    c = b.compiler()
    for p in ("coloring", "computation_grouper"):
        c.run(p)
    assert c.run("cut_size_minimizer")
    assert b.color_of(big) == "B" and b.color_of(small) == "A"


def test_cut_size_minimizer_moves_a_contraction_that_is_larger_than_its_operands():
    """[1024, 8] x [8, 1024] -> [1024, 1024]: the product is 64 times the size of its operands
    together, so it moves to the only task that reads it and the two small operands cross the
    cut instead - alone, and through a chain of unary operators behind it
    (src/pjrt_client/mpmd_cut_size_minimizer_test.cc: LargeDotWithSmallOperands, UnaryOperandMove)."""
    for chain in (False, True):
        b = G()
        x = b.inp("x", [1024, 8])
        y = b.inp("y", [1024, 1024])
        c0 = b.op("aten.cos.default", [x], [1024, 8], task=task_json("red", [0]))
        a0 = b.op("aten.add.Tensor", [c0, x], [1024, 8], task=task_json("red", [0]))
        c0t = b.op("aten.t.default", [c0], [8, 1024], task=task_json("red", [0]))
        dot = b.op("aten.mm.default", [a0, c0t], [1024, 1024], task=task_json("red", [0]))
        last = dot
        if chain:
            tr = b.op("aten.t.default", [dot], [1024, 1024], task=task_json("red", [0]))
            last = b.op("aten.neg.default", [tr], [1024, 1024], task=task_json("red", [0]))
        c1 = b.op("aten.cos.default", [last], [1024, 1024], task=task_json("blue", [1]))
        a1 = b.op("aten.add.Tensor", [c1, y], [1024, 1024], task=task_json("blue", [1]))
        b.g.set_outputs([a1])
        c = b.compiler()
        for p in ("coloring", "computation_grouper"):
            c.run(p)
        assert b.color_of(dot) == "red"
        assert c.run("cut_size_minimizer")
        assert b.color_of(dot) == "blue" and b.color_of(last) == "blue"
        assert b.color_of(a0) == "red" and b.color_of(c0) == "red"
    # a contraction whose result is smaller than its operands stays where it is
    b = G()
    x = b.inp("x", [64, 512])
    w = b.inp("w", [512, 64])
    dot = b.op("aten.mm.default", [x, w], [64, 64], task=task_json("red", [0]))
    use = b.op("aten.neg.default", [dot], [64, 64], task=task_json("blue", [1]))
    b.g.set_outputs([use])
    c = b.compiler()
    for p in ("coloring", "computation_grouper"):
        c.run(p)
    c.run("cut_size_minimizer")
    assert b.color_of(dot) == "red"


def test_split_critical_path_separates_weight_gradients():
    b = G()
    x = b.inp("x", [4, 4])
    w = b.inp("w", [4, 4])
    f = b.op("aten.mm.default", [x, w], [4, 4], task=task_json("s1", [1]))
    split = ("_crit", "_wgrad")
    dx = b.op("aten.mm.default", [f, w], [4, 4], task=task_json("s1", [1], split=split), backprop=True)
    dw = b.op("aten.mm.default", [x, f], [4, 4], task=task_json("s1", [1], split=split), backprop=True)
    prev = b.op("aten.neg.default", [dx], [4, 4], task=task_json("s0", [0]), backprop=True)
    b.g.set_outputs([prev, dw])
    c = b.compiler()
    for p in ("coloring", "computation_grouper"):
        c.run(p)
    assert c.run("split_critical_path")
    by_color = {g_["color"]: g_ for g_ in c.groups()}
    assert "s1_bwd_crit" in by_color and "s1_bwd_wgrad" in by_color
    assert by_color["s1_bwd_wgrad"]["noncritical"] and not by_color["s1_bwd_crit"]["noncritical"]
    assert b.color_of(dx) == "s1_bwd_crit" and b.color_of(dw) == "s1_bwd_wgrad"


def test_contracting_dimension_sharding_inserts_an_all_reduce_and_hoists_gradient_reductions():
    b = G(2)
    la = [("batch", "x")]
    b.g.add_loop(json.dumps({"id": 0, "num_microbatches": 2, "size": 4}))
    x = b.inp("x", [8, 16])
    dy = b.inp("dy", [8, 4])
    xs = b.op("mm.microbatch_slice.default", [x], [4, 16], loop=0, args=[0, 4, 0], task=task_json("T", [0, 1], logical=la))
    ds = b.op("mm.microbatch_slice.default", [dy], [4, 4], loop=0, args=[0, 4, 0], task=task_json("T", [0, 1], logical=la))
    dyt = b.op("aten.t.default", [ds], [4, 4], loop=0, task=task_json("T", [0, 1], logical=la))
    dw = b.op("aten.mm.default", [dyt, xs], [4, 16], loop=0, task=task_json("T", [0, 1], logical=la))
    acc = b.op("mm.microbatch_out.default", [dw], [4, 16], loop=0, args=[0, ""])
    b.g.set_value_axes(xs, [["batch"], []], True)
    b.g.set_value_axes(ds, [["batch"], []], True)
    b.g.set_outputs([acc])
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    ops_of = lambda t: [b.g.node(n)["op"] for n in t["nodes"]]
    loop_t = [t for t in plan["templates"] if t["in_loop"]]
    post_t = [t for t in plan["templates"] if not t["in_loop"]]
    # the data-parallel weight-gradient reduction runs once, after the loop, not per microbatch
    assert all("mm.all_reduce" not in ops_of(t) for t in loop_t)
    assert any("mm.all_reduce" in ops_of(t) for t in post_t)
    assert any("hoisted" in line for line in plan["log"])


def test_remove_hoisted_reduce_option_drops_the_reduction():
    b = G(2)
    b.cfg.remove_hoisted_reduces = True
    la = [("batch", "x")]
    b.g.add_loop(json.dumps({"id": 0, "num_microbatches": 2, "size": 4}))
    x = b.inp("x", [8, 16])
    dy = b.inp("dy", [8, 4])
    xs = b.op("mm.microbatch_slice.default", [x], [4, 16], loop=0, args=[0, 4, 0], task=task_json("T", [0, 1], logical=la))
    ds = b.op("mm.microbatch_slice.default", [dy], [4, 4], loop=0, args=[0, 4, 0], task=task_json("T", [0, 1], logical=la))
    dyt = b.op("aten.t.default", [ds], [4, 4], loop=0, task=task_json("T", [0, 1], logical=la))
    dw = b.op("aten.mm.default", [dyt, xs], [4, 16], loop=0, task=task_json("T", [0, 1], logical=la))
    acc = b.op("mm.microbatch_out.default", [dw], [4, 16], loop=0, args=[0, ""])
    b.g.set_value_axes(xs, [["batch"], []], True)
    b.g.set_value_axes(ds, [["batch"], []], True)
    b.g.set_outputs([acc])
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    assert all(b.g.node(n)["op"] != "mm.all_reduce" for t in plan["templates"] for n in t["nodes"])


def test_logical_sharding_dot_rule_prefers_right_operand_names():
    b = G(4)
    x = b.inp("x", [8, 16])
    w = b.inp("w", [16, 32])
    y = b.op("aten.mm.default", [x, w], [8, 32], task=task_json("T", [0, 1, 2, 3], dims=[2, 2], axes=["a", "b"]))
    b.g.set_value_axes(x, [["batch"], ["embed"]], True)
    b.g.set_value_axes(w, [["embed"], ["mlp"]], True)
    b.g.set_outputs([y])
    c = b.compiler()
    c.run("coloring")
    c.run("logical_sharding_propagation")
    assert b.g.value(y)["axes"] == [["batch"], ["mlp"]]


def test_parameter_replication_cutoff_clears_annotations_of_small_inputs():
    b = G(2)
    b.cfg.replicated_parameter_num_elements_cutoff = 64
    small = b.inp("small", [8])
    big = b.inp("big", [128])
    b.g.set_value_axes(small, [["batch"]], True)
    b.g.set_value_axes(big, [["batch"]], True)
    y = b.op("aten.relu.default", [small], [8], task=task_json("T", [0, 1], logical=[("batch", "x")]))
    z = b.op("aten.relu.default", [big], [128], task=task_json("T", [0, 1], logical=[("batch", "x")]))
    b.g.set_outputs([y, z])
    c = b.compiler()
    assert c.run("parameter_replication")
    assert b.g.value(small)["axes"] == [[]] and b.g.value(big)["axes"] == [["batch"]]


def test_hoist_loop_convert_moves_parameter_casts_out_of_the_loop():
    b = G(1)
    b.cfg.hoist_loop_convert = True
    b.g.add_loop(json.dumps({"id": 0, "num_microbatches": 2, "size": 1}))
    w = b.inp("w", [4, 4])
    cast = b.op("aten._to_copy.default", [w], [4, 4], loop=0, dtype="bfloat16")
    b.g.set_outputs([cast])
    c = b.compiler()
    assert c.run("hoist_loop_convert") and b.g.node(b.g.value(cast)["producer"])["loop"] == -1


def test_plan_hash_is_deterministic():
    hashes = []
    for _ in range(2):
        b = G()
        two_stage_graph(b, loop=True)
        hashes.append(C.mpmd_partition(b.g, b.part, b.cfg)["hash"])
    assert hashes[0] == hashes[1]


def test_environment_options_for_zeroed_arguments_and_static_post_loop_schedule(monkeypatch):
    monkeypatch.setenv("MULTIMESH_ZERO_ARGUMENTS", "1")
    monkeypatch.setenv("MULTIMESH_DYNAMIC_SCHEDULE_POST_LOOP_TASKS", "0")
    cfg = C.PartitionConfig.from_env()
    assert cfg.zero_arguments and not cfg.dynamic_schedule_post_loop_tasks
    monkeypatch.delenv("MULTIMESH_ZERO_ARGUMENTS")
    monkeypatch.delenv("MULTIMESH_DYNAMIC_SCHEDULE_POST_LOOP_TASKS")
    cfg = C.PartitionConfig.from_env()
    assert not cfg.zero_arguments and cfg.dynamic_schedule_post_loop_tasks


def test_static_schedule_keeps_every_task_in_submission_order():
    def plan_with(dynamic):
        b = G()
        two_stage_graph(b)
        b.cfg.dynamic_schedule_post_loop_tasks = dynamic
        return C.mpmd_partition(b.g, b.part, b.cfg)
    dyn = [op["strict_ordering"] for op in plan_with(True)["ops"] if op["kind"] == "task"]
    sta = [op["strict_ordering"] for op in plan_with(False)["ops"] if op["kind"] == "task"]
    assert dyn == [False, False]      # no loop, no collectives: free to overtake
    assert sta == [True, True]
