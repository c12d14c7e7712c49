"""Pipeline schedulers on synthetic tasks ``fwd-i / last / bwd-i`` (the method of
src/pjrt_client/loop_scheduler_test.cc): exact orders for fill-drain, validity and shape of
wavefront (1F1B), interleaved, prefetch, zero-bubble-H2 and custom schedules."""
import json

import pytest

from multimesh_jax_b200 import _mm_C as C


def pipeline(num_stages, num_iters, split_bwd=False, embeddings=False, devices_per_stage=1):
    """tasks[iteration][stage]: fwd0..fwdP-1, bwdP-1..bwd0 (optionally split into B and W halves)."""
    names, devs, noncrit, consumes = [], [], [], []
    if embeddings:
        names.append("loop_increment")
        devs.append((0, num_stages * devices_per_stage))
        noncrit.append(False)
        consumes.append(-1)
    for s in range(num_stages):
        names.append(f"fwd{s}")
        devs.append((s * devices_per_stage, devices_per_stage))
        noncrit.append(False)
        consumes.append(-1)
    for s in reversed(range(num_stages)):
        names.append(f"bwd{s}")
        devs.append((s * devices_per_stage, devices_per_stage))
        noncrit.append(False)
        consumes.append(-1)
        if split_bwd:
            names.append(f"wgrad{s}")
            devs.append((s * devices_per_stage, devices_per_stage))
            noncrit.append(True)
            consumes.append(len(names) - 2)
    rows = []
    for _ in range(num_iters):
        rows.append([{"color": n, "device_start": d[0], "num_devices": d[1], "noncritical": nc, "consumes_stage": cs,
                      "prefetch": n == "loop_increment", "on_full_mesh": n == "loop_increment"}
                     for n, d, nc, cs in zip(names, devs, noncrit, consumes)])
    return rows, names


def run(schedule, rows, n, **extra):
    cfg = {"num_microbatches": n, "schedule": schedule, **extra}
    return C.schedule_loops(json.dumps(cfg), rows)


def check_valid(order, names, n, num_stages):
    """Every task once; forward of stage s after stage s-1, backward after forward and after
    the next stage's backward; one stage runs its own tasks in microbatch order."""
    assert len(order) == len(set(order)) == n * len(names)
    pos = {e: i for i, e in enumerate(order)}
    idx = {name: k for k, name in enumerate(names)}
    for it in range(n):
        for s in range(num_stages):
            if s > 0:
                assert pos[(it, idx[f"fwd{s}"])] > pos[(it, idx[f"fwd{s - 1}"])]
            assert pos[(it, idx[f"bwd{s}"])] > pos[(it, idx[f"fwd{s}"])]
            if s + 1 < num_stages:
                assert pos[(it, idx[f"bwd{s}"])] > pos[(it, idx[f"bwd{s + 1}"])]
            if it > 0:
                assert pos[(it, idx[f"fwd{s}"])] > pos[(it - 1, idx[f"fwd{s}"])]


def test_fill_drain_is_stage_major():
    rows, names = pipeline(2, 3)
    out = run("gpipe", rows, 3)
    assert out["orders"] == [[(it, st) for st in range(4) for it in range(3)]]


@pytest.mark.parametrize("stages,n", [(2, 4), (4, 8), (4, 16), (3, 5)])
def test_wavefront_is_valid_and_bounds_live_microbatches(stages, n):
    rows, names = pipeline(stages, n)
    order = [tuple(e) for e in run("1f1b", rows, n)["orders"][0]]
    check_valid(order, names, n, stages)
    # 1F1B property on the first stage: the number of microbatches whose forward ran but whose
    # backward did not is bounded by a constant independent of the number of microbatches
    idx = {name: k for k, name in enumerate(names)}
    live, peak = 0, 0
    for it, st in order:
        if st == idx["fwd0"]:
            live += 1
        elif st == idx["bwd0"]:
            live -= 1
        peak = max(peak, live)
    assert peak <= 2 * stages
    gp = [tuple(e) for e in run("gpipe", rows, n)["orders"][0]]
    live, gpeak = 0, 0
    for it, st in gp:
        if st == idx["fwd0"]:
            live += 1
        elif st == idx["bwd0"]:
            live -= 1
        gpeak = max(gpeak, live)
    assert gpeak == n


def test_wavefront_with_few_iterations():
    rows, names = pipeline(4, 2)
    order = [tuple(e) for e in run("wavefront", rows, 2)["orders"][0]]
    check_valid(order, names, 2, 4)


def test_wavefront_num_stages_override_changes_the_delay():
    rows, names = pipeline(2, 6)
    a = run("1f1b", rows, 6)["orders"][0]
    b = run("1f1b", rows, 6, num_stages=3)["orders"][0]
    assert a != b
    check_valid([tuple(e) for e in b], names, 6, 2)


def test_single_task_body_degenerates_to_fill_drain():
    rows = [[{"color": "only", "device_start": 0, "num_devices": 1}] for _ in range(4)]
    assert run("1f1b", rows, 4)["orders"] == [[(0, 0), (1, 0), (2, 0), (3, 0)]]


def test_prefetch_wavefront_runs_loop_increment_first():
    rows, names = pipeline(2, 4, embeddings=True)
    order = [tuple(e) for e in run("prefetch-wavefront", rows, 4)["orders"][0]]
    assert order[:4] == [(0, 0), (1, 0), (2, 0), (3, 0)]
    assert len(order) == 4 * len(names)


@pytest.mark.parametrize("stages,n", [(2, 4), (4, 8), (4, 24)])
def test_zero_bubble_defers_weight_gradients(stages, n):
    rows, names = pipeline(stages, n, split_bwd=True)
    out = run("zero-bubble-h2", rows, n)
    order = [tuple(e) for e in out["orders"][0]]
    assert len(order) == len(set(order)) == n * len(names)
    idx = {name: k for k, name in enumerate(names)}
    pos = {e: i for i, e in enumerate(order)}
    for it in range(n):
        for s in range(stages):
            # the weight-gradient half runs after the activation-gradient half it reads
            assert pos[(it, idx[f"wgrad{s}"])] > pos[(it, idx[f"bwd{s}"])]
        # critical path first: the first stage's activation gradient is not delayed by the
        # last stage's weight gradient of the same microbatch
        assert pos[(it, idx["bwd0"])] < pos[(it, idx[f"wgrad0"])]
    assert out["simulated_makespan"] > 0


def test_zero_bubble_orders_noncritical_tasks_by_descending_consumed_stage():
    rows, names = pipeline(2, 1, split_bwd=True)
    order = [tuple(e) for e in run("zero-bubble-h2", rows, 1)["orders"][0]]
    idx = {name: k for k, name in enumerate(names)}
    assert order.index((0, idx["wgrad0"])) < order.index((0, idx["wgrad1"]))


def test_custom_gpipe_and_1f1b_rows():
    rows, names = pipeline(2, 2)
    gpipe = [[[0, "fwd0"], [1, "fwd0"], [1, "bwd0"], [0, "bwd0"]], [[0, "fwd1"], [1, "fwd1"], [1, "bwd1"], [0, "bwd1"]]]
    out = run("custom", rows, 2, custom_schedule=gpipe)
    assert len(out["orders"]) == 2
    idx = {name: k for k, name in enumerate(names)}
    assert [tuple(e) for e in out["orders"][0]] == [(0, idx["fwd0"]), (1, idx["fwd0"]), (1, idx["bwd0"]), (0, idx["bwd0"])]
    f1b1 = [[[0, "fwd0"], [1, "fwd0"], [0, "bwd0"], [1, "bwd0"]], [[0, "fwd1"], [0, "bwd1"], [1, "fwd1"], [1, "bwd1"]]]
    out = run("custom", rows, 2, custom_schedule=f1b1)
    assert [tuple(e) for e in out["orders"][1]] == [(0, idx["fwd1"]), (0, idx["bwd1"]), (1, idx["fwd1"]), (1, idx["bwd1"])]


def test_custom_schedule_validation():
    rows, names = pipeline(2, 2)
    with pytest.raises(RuntimeError, match="appears"):
        run("custom", rows, 2, custom_schedule=[[[0, "fwd0"]], [[0, "fwd1"], [1, "fwd1"]]])
    with pytest.raises(RuntimeError, match="no task matches"):
        run("custom", rows, 2, custom_schedule=[[[0, "nothing"], [1, "nothing"]]])
    with pytest.raises(RuntimeError, match="twice"):
        run("custom", rows, 2, custom_schedule=[[[0, "fwd0"], [0, "fwd0"]]])
    with pytest.raises(RuntimeError, match="unknown microbatch schedule"):
        run("round-robin", rows, 2)


def test_bijective_task_requirement():
    assert C.enforce_bijective_tasks("custom") and C.enforce_bijective_tasks("zero-bubble-h2")
    assert not C.enforce_bijective_tasks("1f1b")


def interleaved(groups, rounds, num_iters, split_bwd=False):
    """Circular placement: ``groups * rounds`` virtual stages over ``groups`` device groups, stage s
    on group ``s % groups`` (the interleaved cases of src/pjrt_client/loop_scheduler_test.cc)."""
    stages = groups * rounds
    rows, names = pipeline(stages, num_iters, split_bwd=split_bwd)
    for row in rows:
        for t in row:
            s = int("".join(ch for ch in t["color"] if ch.isdigit()))
            t["device_start"] = s % groups
    return rows, names, stages


@pytest.mark.parametrize("groups,rounds,n", [(2, 2, 4), (4, 2, 8), (4, 4, 8), (2, 4, 6)])
def test_interleaved_wavefront_is_valid_and_every_group_alternates(groups, rounds, n):
    rows, names, stages = interleaved(groups, rounds, n)
    out = run("1f1b", rows, n)
    order = [tuple(e) for e in out["orders"][0]]
    check_valid(order, names, n, stages)
    # the minibatch is as wide as the number of device groups: within one group the first
    # `groups` microbatches pass the group's first virtual stage before any reaches its second
    idx = {name: k for k, name in enumerate(names)}
    pos = {e: i for i, e in enumerate(order)}
    first_second_round = min(pos[(it, idx[f"fwd{groups}"])] for it in range(n))
    assert sum(1 for it in range(n) if pos[(it, idx["fwd0"])] < first_second_round) >= min(groups, n)
    # no group ever holds all microbatches in flight: a backward of the last stage is reached
    # before the last forward of the first stage when there are more microbatches than groups
    if n > 2 * groups * rounds:
        assert pos[(0, idx[f"bwd{stages - 1}"])] < pos[(n - 1, idx["fwd0"])]


def test_interleaved_wavefront_with_embeddings_prefetches_the_full_mesh_task():
    rows, names, stages = interleaved(2, 2, 4)
    for row in rows:
        row.insert(0, {"color": "loop_increment", "device_start": 0, "num_devices": 2, "prefetch": True,
                       "on_full_mesh": True, "noncritical": False, "consumes_stage": -1})
    order = [tuple(e) for e in run("prefetch-wavefront", rows, 4)["orders"][0]]
    assert order[:4] == [(it, 0) for it in range(4)]
    assert len(order) == len(set(order)) == 4 * (len(names) + 1)


@pytest.mark.parametrize("groups,rounds,n", [(2, 2, 4), (4, 2, 8), (4, 6, 8)])
def test_zero_bubble_interleaved_keeps_dependencies_and_defers_weight_gradients(groups, rounds, n):
    rows, names, stages = interleaved(groups, rounds, n, split_bwd=True)
    order = [tuple(e) for e in run("zero-bubble-h2", rows, n)["orders"][0]]
    assert len(order) == len(set(order)) == n * len(names)
    pos = {e: i for i, e in enumerate(order)}
    idx = {name: k for k, name in enumerate(names)}
    for it in range(n):
        for s in range(stages):
            assert pos[(it, idx[f"wgrad{s}"])] > pos[(it, idx[f"bwd{s}"])]
            if s > 0:
                assert pos[(it, idx[f"fwd{s}"])] > pos[(it, idx[f"fwd{s - 1}"])]
                assert pos[(it, idx[f"bwd{s - 1}"])] > pos[(it, idx[f"bwd{s}"])]


def test_random_pipelines_are_scheduled_validly_or_refused():
    """400 seeded random cases over every schedule name, split backward halves, a full-mesh
    prefetch task, interleaving, unrolling and random custom schedules: the scheduler either
    refuses the request with an error or returns an order that keeps every dependency."""
    import random
    rng = random.Random(1234)
    valid = refused = 0
    for _ in range(400):
        stages, n = rng.randint(1, 6), rng.randint(1, 12)
        schedule = rng.choice(["gpipe", "1f1b", "wavefront", "zero-bubble-h2", "prefetch-wavefront", "custom"])
        split = schedule == "zero-bubble-h2" or rng.random() < 0.2
        rows, names = pipeline(stages, n, split_bwd=split, embeddings=rng.random() < 0.3,
                               devices_per_stage=rng.randint(1, 2))
        extra = {}
        if rng.random() < 0.3:
            extra["interleave"] = rng.randint(1, 3)
        if rng.random() < 0.2:
            extra["unrolling"] = rng.randint(0, 3)
        if schedule == "custom":
            extra["custom_schedule"] = []
            for s in range(stages):
                entries = [(it, rng.choice([f"fwd{s}", f"bwd{s}", f"wgrad{s}", "fwd", "x"])) for it in range(n) for _ in range(2)]
                rng.shuffle(entries)
                extra["custom_schedule"].append(entries[:rng.randint(0, len(entries))])
        try:
            out = run(schedule, rows, n, **extra)
        except (RuntimeError, ValueError):
            refused += 1
            continue
        if len(out["orders"]) == 1:
            check_valid([tuple(e) for e in out["orders"][0]], names, n, stages)
        valid += 1
    assert valid > 250 and refused > 10, (valid, refused)
