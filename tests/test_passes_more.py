"""More pass-level cases on hand-built graphs, after the case lists of the reference's
mpmd_insert_reshard_test.cc (ScalarReshard, RootTupleRecolor), mpmd_buffer_scheduling_name_test.cc
(SubsetDeviceSkipReshard), mpmd_argument_recompute_test.cc (RecomputeSharedClone),
mpmd_instruction_delay_recolor_test.cc (DelayInitInstructions), mpmd_computation_grouper_test.cc
(implicit nodes join a neighbouring task) and mpmd_loop_unroll_test.cc (LoopIterDependent)."""
import json

import pytest

from multimesh_jax_b200 import _mm_C as C
from test_passes import G, task_json


def _ops(plan, kind):
    return [op for op in plan["ops"] if op["kind"] == kind]


def _template_ops(b, plan):
    return {t["name"]: [b.g.node(n)["op"] for n in t["nodes"]] for t in plan["templates"]}


def test_scalar_crossing_a_task_boundary_is_resharded_as_a_scalar_store():
    b = G(2)
    x = b.inp("x", [4])
    s = b.op("aten.sum.default", [x], [], task=task_json("A", [0]))
    y = b.op("aten.mul.Tensor", [x, s], [4], task=task_json("B", [1]))
    b.g.set_outputs([y])
    b.cfg.argument_recompute = False
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    stores = plan["stores"]
    scalar_moves = [r for r in _ops(plan, "reshard") if stores[r["src_store"]]["scalar"]]
    assert len(scalar_moves) == 1 and stores[scalar_moves[0]["dst_store"]]["scalar"]
    assert stores[scalar_moves[0]["src_store"]]["shape"]["device_start"] == 0
    assert stores[scalar_moves[0]["dst_store"]]["shape"]["device_start"] == 1
    # the parameter is read by both tasks: it lives with the first and is copied once to the second
    param_moves = [r for r in _ops(plan, "reshard") if stores[r["src_store"]]["kind"] == "PARAM"]
    assert len(param_moves) == 1


def test_consumer_on_a_subset_of_the_producer_devices_reads_the_replicated_tile_in_place():
    b = G(2)
    x = b.inp("x", [4, 4])
    a = b.op("aten.relu.default", [x], [4, 4], task=task_json("A", [0, 1]))
    c = b.op("aten.neg.default", [a], [4, 4], task=task_json("B", [0]))
    b.g.set_outputs([c])
    b.cfg.use_task_fusion = False
    b.cfg.argument_recompute = False
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    assert not _ops(plan, "reshard")
    ta, tb = _ops(plan, "task")
    assert (ta["device_start"], ta["num_devices"], tb["device_start"], tb["num_devices"]) == (0, 2, 0, 1)
    assert tb["inputs"] == ta["outputs"]          # the same store, no copy in between


def test_results_of_different_tasks_stay_on_their_producers_devices():
    b = G(2)
    x = b.inp("x", [4])
    a = b.op("aten.relu.default", [x], [4], task=task_json("A", [0]))
    c = b.op("aten.neg.default", [a], [4], task=task_json("B", [1]))
    b.g.set_outputs([a, c])
    b.cfg.argument_recompute = False
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    roots = [plan["stores"][r]["shape"] for r in plan["root_stores"]]
    assert [(r["device_start"], r["num_devices"]) for r in roots] == [(0, 1), (1, 1)]


def test_unannotated_nodes_join_a_neighbouring_task_instead_of_forming_their_own():
    b = G(2)
    x, w = b.inp("x", [4, 4]), b.inp("w", [4, 4])
    a = b.op("aten.mm.default", [x, w], [4, 4], task=task_json("A", [0]))
    m = b.op("aten.neg.default", [a], [4, 4])
    m2 = b.op("aten.exp.default", [m], [4, 4])
    c = b.op("aten.mm.default", [m2, w], [4, 4], task=task_json("B", [1]))
    b.g.set_outputs([c])
    b.cfg.argument_recompute = False
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    names = _template_ops(b, plan)
    assert len(names) == 2
    assert sorted(op for ops in names.values() for op in ops) == sorted(
        ["aten.mm.default", "aten.neg.default", "aten.exp.default", "aten.mm.default"])
    # exactly one activation crosses the boundary
    stores = plan["stores"]
    assert len([r for r in _ops(plan, "reshard") if stores[r["src_store"]]["kind"] == "TEMP"]) == 1


def test_cheap_producer_read_by_two_tasks_is_cloned_into_the_second_task():
    b = G(2)
    x = b.inp("x", [4, 4])
    w = b.inp("w", [4, 4])
    cheap = b.op("aten.neg.default", [x], [4, 4], task=task_json("A", [0]))
    a = b.op("aten.mm.default", [cheap, w], [4, 4], task=task_json("A", [0]))
    c = b.op("aten.add.Tensor", [a, cheap], [4, 4], task=task_json("B", [1]))
    b.g.set_outputs([c])
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    names = _template_ops(b, plan)
    a_ops = next(v for k, v in names.items() if k.endswith("A"))
    b_ops = next(v for k, v in names.items() if k.endswith("B"))
    assert a_ops.count("aten.neg.default") == 1 and b_ops.count("aten.neg.default") == 1
    # only the matrix product crosses the boundary as a temporary; x itself is copied as a parameter
    stores = plan["stores"]
    assert len([r for r in _ops(plan, "reshard") if stores[r["src_store"]]["kind"] == "TEMP"]) == 1


def test_initialiser_without_operands_is_delayed_to_its_consumer():
    b = G(2)
    x, w = b.inp("x", [4, 4]), b.inp("w", [4, 4])
    z0 = b.op("aten.zeros.default", [], [4, 4], args=[[4, 4]])
    a = b.op("aten.mm.default", [x, w], [4, 4], task=task_json("A", [0]))
    c = b.op("aten.mm.default", [a, w], [4, 4], task=task_json("B", [1]))
    d = b.op("aten.add.Tensor", [c, z0], [4, 4], task=task_json("B", [1]))
    b.g.set_outputs([d])
    b.cfg.argument_recompute = False
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    names = _template_ops(b, plan)
    assert "aten.zeros.default" in next(v for k, v in names.items() if k.endswith("B"))
    assert "aten.zeros.default" not in next(v for k, v in names.items() if k.endswith("A"))


def test_summed_loop_output_must_not_move_between_devices():
    b = G(4)
    b.g.add_loop(json.dumps({"id": 0, "num_microbatches": 4, "slice_dim": 0, "size": 1, "schedule": "gpipe"}))
    x = b.inp("x", [4, 8])
    xs = b.op("mm.microbatch_slice.default", [x], [1, 8], loop=0, args=[0, 1, 0])
    tj = json.dumps({"name": "mover", "devices": [0, 1], "dims": [2], "device_axes": ["x"], "logical_axes": [],
                     "split_backprop": [], "loop_dependent_devices": [[0, 1], [2, 3], [0, 1], [2, 3]]})
    h = b.op("aten.relu.default", [xs], [1, 8], task=tj, loop=0)
    z = b.op("aten.sum.default", [h], [], task=tj, loop=0)
    z = b.op("mm.microbatch_out.default", [z], [], loop=0, args=[0, ""])
    b.g.set_outputs([z])
    with pytest.raises(RuntimeError, match="same devices in every iteration"):
        C.mpmd_partition(b.g, b.part, b.cfg)


def test_loop_dependent_task_alternates_between_submeshes_and_feeds_a_fixed_task():
    b = G(4)
    b.g.add_loop(json.dumps({"id": 0, "num_microbatches": 4, "slice_dim": 0, "size": 1, "schedule": "gpipe"}))
    x = b.inp("x", [4, 8])
    xs = b.op("mm.microbatch_slice.default", [x], [1, 8], loop=0, args=[0, 1, 0])
    tj = json.dumps({"name": "mover", "devices": [0, 1], "dims": [2], "device_axes": ["x"], "logical_axes": [],
                     "split_backprop": [], "loop_dependent_devices": [[0, 1], [2, 3], [0, 1], [2, 3]]})
    h = b.op("aten.relu.default", [xs], [1, 8], task=tj, loop=0)
    z = b.op("aten.sum.default", [h], [], task=task_json("fixed", [0, 1], dims=[2]), loop=0)
    z = b.op("mm.microbatch_out.default", [z], [], loop=0, args=[0, ""])
    b.g.set_outputs([z])
    b.cfg.use_task_fusion = False
    b.cfg.argument_recompute = False
    plan = C.mpmd_partition(b.g, b.part, b.cfg)
    movers = sorted((t["iteration"], t["device_start"]) for t in _ops(plan, "task") if "mover" in t["name"])
    assert movers == [(0, 0), (1, 2), (2, 0), (3, 2)]
    fixed = {t["device_start"] for t in _ops(plan, "task") if "fixed" in t["name"]}
    assert fixed == {0}
    # iterations that ran on devices 2-3 hand their activation back to devices 0-1
    stores = plan["stores"]
    back = [r for r in _ops(plan, "reshard") if stores[r["src_store"]]["shape"]["device_start"] == 2
            and stores[r["dst_store"]]["shape"]["device_start"] == 0]
    assert len(back) == 2


# ---------------------------------------------------------------------------- fusion by original colour
def test_fusion_by_original_colour_rejoins_call_sites_of_one_user_task():
    """Two call sites whose colours differ only because one was recoloured (``s0`` and its
    descendant ``s0_late``) are not fused by the matching-colour round but are by the
    original-colour round that follows the regrouping (src/pjrt_client/mpmd_partition.cc:946);
    a pair whose fusion would contradict the dependencies stays apart."""
    from test_passes import G, task_json
    b = G(2)
    x, y = b.inp("x", [4]), b.inp("y", [4])
    b.part.add_task(task_json("s0", [0]), False)
    late = b.part.recolor("s0", "s0_late")
    assert b.part.color(late)["original"] == "s0"
    a = b.op("aten.relu.default", [x], [4], task=task_json("s0", [0]))
    m = b.op("aten.gelu.default", [y], [4], task=task_json("s1", [1]))
    c = b.op("aten.neg.default", [a], [4], color=late)
    e = b.op("aten.add.Tensor", [c, m], [4], task=task_json("s1", [1]))
    b.g.set_outputs([e])
    comp = b.compiler()
    comp.run("coloring")
    comp.run("computation_grouper")
    comp.run("computation_fusion_matching_color")
    assert [(g["color"], g["nodes"]) for g in comp.groups()] == [("s0", [0]), ("s0_late", [2]), ("s1", [1, 3])]
    assert comp.run("computation_fusion_original_color")
    assert [(g["color"], g["nodes"]) for g in comp.groups()] == [("s0", [0, 2]), ("s1", [1, 3])]
    assert b.g.node(2)["color"] == "s0"

    # s0 -> s1 -> s0_late: the middle task depends on the first and feeds the last; no fusion
    b = G(2)
    x = b.inp("x", [4])
    b.part.add_task(task_json("s0", [0]), False)
    late = b.part.recolor("s0", "s0_late")
    a = b.op("aten.relu.default", [x], [4], task=task_json("s0", [0]))
    m = b.op("aten.gelu.default", [a], [4], task=task_json("s1", [1]))
    c = b.op("aten.neg.default", [m], [4], color=late)
    b.g.set_outputs([c])
    comp = b.compiler()
    comp.run("coloring")
    comp.run("computation_grouper")
    assert not comp.run("computation_fusion_original_color")
    assert len(comp.groups()) == 3


# ---------------------------------------------------------------------------- unused loop outputs
def test_unused_loop_output_is_removed_with_the_work_that_only_fed_it():
    from test_passes import G, task_json
    b = G(1)
    b.g.add_loop(json.dumps({"id": 0, "num_microbatches": 2, "slice_dim": 0, "size": 2, "schedule": "gpipe"}))
    x = b.inp("x", [4, 8])
    xs = b.op("mm.microbatch_slice.default", [x], [2, 8], loop=0, args=[0, 2, 0])
    h = b.op("aten.relu.default", [xs], [2, 8], loop=0, task=task_json("t", [0]))
    used = b.op("aten.sum.default", [h], [], loop=0, task=task_json("t", [0]))
    aux = b.op("aten.exp.default", [h], [2, 8], loop=0, task=task_json("t", [0]))       # feeds only the dropped output
    aux_sum = b.op("aten.sum.default", [aux], [], loop=0, task=task_json("t", [0]))
    out_used = b.op("mm.microbatch_out.default", [used], [], loop=0, args=[0, ""])
    out_dropped = b.op("mm.microbatch_out.default", [aux_sum], [], loop=0, args=[0, ""])
    b.g.set_outputs([out_used])
    comp = b.compiler()
    comp.run("microbatch_loop_canonicalizer")
    comp.run("coloring")
    assert comp.run("unused_loop_output_remover")
    dead = {i for i in range(7) if b.g.node(i)["dead"]}
    assert dead == {b.g.value(aux)["producer"], b.g.value(aux_sum)["producer"], b.g.value(out_dropped)["producer"]}
    assert any("dropped 1 loop outputs and 2 operators" in line for line in comp.log())
    assert not comp.run("unused_loop_output_remover")          # nothing left to drop


# ---------------------------------------------------------------------------- in-place collectives
def test_hoisted_gradient_reduction_reuses_the_accumulator_buffer():
    """The once-per-step all-reduce of a gradient accumulator is a task of its own whose only
    input dies there: its output store takes the accumulator's buffer and the all-reduce node is
    marked in-place (src/pjrt_client/mpmd_inplace_collectives.cc:20-76). Numerics are unchanged."""
    import torch
    import multimesh_jax_b200 as mm
    from multimesh_jax_b200.models import llama
    torch.manual_seed(0)
    cfg = llama.LlamaConfig.tiny(n_layers=1, n_heads=2, n_kv_heads=2, d_model=32, d_ff=48, vocab=64)
    cfg.dtype = torch.float32
    B, S = 8, 8
    params = llama.init_params(cfg)
    state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-2), seq_len=S, global_batch=B, microbatch_size=4)
    mesh = mm.MultiMesh((1, 2, 1), ("stage", "data", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=1)
    args = (params, state, tokens, tokens, cos, sin)
    with mesh:
        exe = mm.compile_function(step, args, mesh=mesh, backend="cpu")
    plan, g = exe.plan, exe.cap.graph
    n_inplace = int(plan["stats"]["in_place_collectives"])
    assert n_inplace > 0
    marked = [n for t in plan["templates"] for n in t["nodes"]
              if g.node(n)["op"] == "mm.all_reduce" and g.node(n)["attrs"].get("in_place") == "1"]
    assert len(marked) == n_inplace
    aliased = [st for st in plan["stores"] if st["kind"] == "TEMP" and st["alias_of"] >= 0]
    assert len(aliased) == n_inplace
    for st in aliased:
        src = plan["stores"][st["alias_of"]]
        assert src["name"] == st["name"] and src["shape"]["key"] == st["shape"]["key"]
        assert exe.buffer_of[st["id"]] == exe.buffer_of[src["id"]]
    with mm.ignore_transforms():
        loss_ref, p_ref, _ = step(*args)
    loss, p_mm, _ = exe(*args)
    from torch.utils import _pytree as pytree
    torch.testing.assert_close(loss.full_tensor(), loss_ref, rtol=1e-4, atol=1e-5)
    for a, r in zip(pytree.tree_leaves(p_mm), pytree.tree_leaves(p_ref)):
        torch.testing.assert_close(a.full_tensor(), r, rtol=1e-3, atol=2e-4)
    assert not exe.context.hazard_report()        # every conflicting pair of accesses is ordered
    exe.shutdown()
