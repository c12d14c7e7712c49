"""Sharding algebra: logical -> physical mapping, canonical descriptors, resize across unequal
submeshes, mesh equivalence, the needs-reshard predicate and the reshard planner
(the checklist of src/pjrt_client/mm_sharding_test.cc, restated for this IR)."""
import itertools

import pytest

from multimesh_jax_b200 import _mm_C as C


def shape(dtype, sizes, dim_axes, mesh, start=0):
    return C.sharded_shape(dtype, sizes, dim_axes, mesh, start)


def test_replicated_shape_has_full_tile_on_every_device():
    s = shape("float32", [8, 6], [[], []], [4])
    assert s["shard_size"] == [8, 6]
    for o in range(4):
        assert C.tile_box(s, o) == ([0, 0], [8, 6])


def test_one_axis_tiling():
    s = shape("bfloat16", [8, 6], [[0], []], [4], start=2)
    assert s["shard_size"] == [2, 6] and s["device_start"] == 2
    assert C.tile_box(s, 3) == ([6, 0], [8, 6])


def test_two_axis_mesh_row_major_device_order():
    # mesh (2, 4): dim0 over axis 0, dim1 over axis 1; device ordinal = a0 * 4 + a1
    s = shape("float32", [4, 8], [[0], [1]], [2, 4])
    assert s["shard_size"] == [2, 2]
    assert C.tile_box(s, 5) == ([2, 2], [4, 4])


def test_transposed_assignment_and_partial_replication():
    # dim0 over the *minor* mesh axis, the major axis replicates
    s = shape("float32", [8, 2], [[1], []], [2, 4])
    assert s["shard_size"] == [2, 2]
    assert C.tile_box(s, 1) == C.tile_box(s, 5) == ([2, 0], [4, 2])


def test_two_axes_on_one_dimension():
    s = shape("float32", [16], [[0, 1]], [2, 4])
    assert s["shard_size"] == [2]
    assert [C.tile_box(s, o)[0][0] for o in range(8)] == [0, 2, 4, 6, 8, 10, 12, 14]


def test_invalid_shapes_are_rejected():
    with pytest.raises(RuntimeError):
        shape("float32", [7], [[0]], [2])          # not divisible
    with pytest.raises(RuntimeError):
        shape("float32", [8, 8], [[0], [0]], [2])  # mesh axis used twice


def test_json_round_trip_keeps_the_per_shard_layout():
    s = shape("bfloat16", [4, 8, 16], [[], [1], [0]], [2, 2], start=4)
    j = C.sharded_shape_to_json(s)
    assert '"permutation"' in j and '"sharding"' in j and '"num_devices":4' in j
    assert C.sharded_shape_from_json(j)["key"] == s["key"]


# ---------------------------------------------------------------- logical -> physical
AXES = [("batch", "x"), ("model", "y"), ("seq", "y")]


def test_logical_axes_priority_and_single_use_of_a_mesh_axis():
    s = C.logical_to_physical("float32", [8, 16, 32], [["batch"], ["seq"], ["model"]], AXES, ["x", "y"], [2, 4], 0)
    # "model" comes before "seq" in the table, so y goes to dim 2 and seq stays unsharded
    assert s["dim_axes"] == [[0], [], [1]]


def test_logical_axis_needs_divisibility():
    s = C.logical_to_physical("float32", [3, 16], [["batch"], ["model"]], AXES, ["x", "y"], [2, 4], 0)
    assert s["dim_axes"] == [[], [1]]


def test_large_parameters_not_sharded_without_names():
    s = C.logical_to_physical("float32", [1024, 1024], [[], []], AXES, ["x", "y"], [2, 4], 0)
    assert s["dim_axes"] == [[], []]


def test_several_mesh_axes_can_land_on_one_dimension():
    table = [("data", "x"), ("data", "y")]
    s = C.logical_to_physical("float32", [16, 4], [["data"], []], table, ["x", "y"], [2, 4], 0)
    assert s["dim_axes"] == [[0, 1], []] and s["shard_size"] == [2, 4]


# ---------------------------------------------------------------- resize / equivalence
def test_resize_scales_first_sharded_dimension():
    s = shape("float32", [16, 8], [[0], []], [4])
    r, ok = C.resize_sharding(s, 4, 2)
    assert ok and r["shard_size"] == [8, 8] and r["device_start"] == 4
    r, ok = C.resize_sharding(s, 0, 8)
    assert ok and r["shard_size"] == [2, 8]


def test_resize_falls_back_to_replicated():
    s = shape("float32", [4, 8], [[0], []], [4])
    r, ok = C.resize_sharding(s, 0, 3)
    assert not ok and r["shard_size"] == [4, 8]
    # transposed assignment cannot be rescaled
    t = shape("float32", [8, 8], [[1], [0]], [2, 2])
    r, ok = C.resize_sharding(t, 0, 8)
    assert not ok and r["dim_axes"] == [[], []]


def test_replicate_dims():
    s = shape("float32", [8, 8], [[0], [1]], [2, 2])
    assert C.replicate_dims(s, [1])["dim_axes"] == [[0], []]


def test_mesh_equivalence_ignores_mesh_factoring():
    a = shape("float32", [8, 4], [[0], []], [4])
    b = shape("float32", [8, 4], [[0, 1], []], [2, 2])
    assert C.mesh_equivalent(a, b)
    c = shape("float32", [8, 4], [[], [0]], [4])
    assert not C.mesh_equivalent(a, c)


def test_needs_reshard_predicate():
    rep_big = shape("float32", [4], [[]], [4], start=0)
    rep_small = shape("float32", [4], [[]], [2], start=1)
    assert not C.needs_reshard(rep_big, rep_small)        # replicated producer covers the consumer
    assert C.needs_reshard(rep_small, rep_big)
    a = shape("float32", [8, 4], [[0], []], [2], start=0)
    b = shape("float32", [8, 4], [[0], []], [2], start=2)
    assert C.needs_reshard(a, b)                           # same tiles, other devices
    c = shape("float32", [8, 4], [[], [0]], [2], start=0)
    assert C.needs_reshard(a, c)                           # same devices, other tiles
    assert not C.needs_reshard(a, a)


# ---------------------------------------------------------------- planner
CASES = [
    (shape("bfloat16", [8, 4, 16], [[0], [], []], [2], 0), shape("bfloat16", [8, 4, 16], [[], [], [0]], [2], 2)),
    (shape("bfloat16", [8, 4, 16], [[], [], [0]], [4], 0), shape("bfloat16", [8, 4, 16], [[], [], []], [2], 4)),
    (shape("bfloat16", [8, 4, 16], [[], [], []], [2], 0), shape("bfloat16", [8, 4, 16], [[0], [], []], [4], 2)),
    (shape("bfloat16", [8, 4, 16], [[0], [], [1]], [2, 2], 0), shape("bfloat16", [8, 4, 16], [[1], [0], []], [2, 2], 2)),
    (shape("bfloat16", [8, 4, 16], [[0], [], []], [4], 0), shape("bfloat16", [8, 4, 16], [[0], [], []], [2], 1)),
]


@pytest.mark.parametrize("src,dst", CASES)
def test_plan_covers_every_destination_element_exactly_once(src, dst):
    plan = C.plan_reshard(src, dst)
    sizes = src["sizes"]
    for o in range(dst["num_devices"]):
        dev = dst["device_start"] + o
        lo, hi = C.tile_box(dst, o)
        cover = {}
        for c in plan["chunks"]:
            if c["dst_device"] != dev:
                continue
            # chunk lies inside the destination tile and inside the named source tile
            s_lo, s_hi = C.tile_box(src, c["src_device"] - src["device_start"])
            for d in range(len(sizes)):
                assert lo[d] <= c["lo"][d] < c["hi"][d] <= hi[d]
                assert s_lo[d] <= c["lo"][d] and c["hi"][d] <= s_hi[d]
                assert c["src_offset"][d] == c["lo"][d] - s_lo[d]
                assert c["dst_offset"][d] == c["lo"][d] - lo[d]
            for idx in itertools.product(*[range(a, b) for a, b in zip(c["lo"], c["hi"])]):
                cover[idx] = cover.get(idx, 0) + 1
        want = set(itertools.product(*[range(a, b) for a, b in zip(lo, hi)]))
        assert set(cover) == want and all(v == 1 for v in cover.values())


def test_planner_prefers_the_local_replica_and_spreads_the_rest():
    src = shape("bfloat16", [8, 16], [[], []], [4], 0)           # replicated on 0..3
    dst = shape("bfloat16", [8, 16], [[0], []], [4], 2)          # devices 2..5
    plan = C.plan_reshard(src, dst)
    by_dst = {c["dst_device"]: c["src_device"] for c in plan["chunks"]}
    assert by_dst[2] == 2 and by_dst[3] == 3                     # overlap: no link traffic
    assert len({by_dst[4], by_dst[5]}) == 2                      # different sources serve the others
    assert plan["bytes_over_links"] == 2 * 2 * 16 * 2


def test_layout_predicates_hold_on_random_layout_pairs():
    """2,000 seeded random pairs of layouts (one to three mesh axes, several axes on one dimension,
    any device offsets): mesh-equivalent layouts have the same tiles; where no reshard is asked for,
    every destination device already holds its tile of the source; equal tiles on equal devices never
    ask for one; text round trips keep the tiles; a resized layout has the requested device count and
    covers every element once per replica."""
    import random

    def layout(rng, sizes, start):
        mesh = [rng.choice([1, 2, 2, 3, 4]) for _ in range(rng.randint(1, 3))]
        dim_axes, left = [[] for _ in sizes], list(sizes)
        order = list(range(len(mesh)))
        rng.shuffle(order)
        for axis in order:
            fits = [d for d in range(len(sizes)) if left[d] % mesh[axis] == 0 and left[d] >= mesh[axis]]
            if fits and rng.random() > 0.25:
                d = rng.choice(fits)
                dim_axes[d].append(axis)
                left[d] //= mesh[axis]
        return C.sharded_shape("float32", list(sizes), dim_axes, mesh, start)

    def boxes(s):
        return [C.tile_box(s, o) for o in range(s["num_devices"])]

    def volume(box):
        v = 1
        for lo, hi in zip(*box):
            v *= hi - lo
        return v

    equivalent = in_place = 0
    for seed in range(2000):
        rng = random.Random(seed)
        sizes = [rng.choice([2, 4, 6, 8, 12]) for _ in range(rng.randint(1, 3))]
        a, b = layout(rng, sizes, rng.randint(0, 2)), layout(rng, sizes, rng.randint(0, 2))
        same_tiles = a["num_devices"] == b["num_devices"] and boxes(a) == boxes(b)
        if C.mesh_equivalent(a, b):
            equivalent += 1
            assert same_tiles, (a["key"], b["key"])
        if not C.needs_reshard(a, b):
            in_place += 1
            for o in range(b["num_devices"]):
                pos = b["device_start"] + o - a["device_start"]
                assert 0 <= pos < a["num_devices"] and C.tile_box(a, pos) == C.tile_box(b, o), (a["key"], b["key"])
        if same_tiles and a["device_start"] == b["device_start"]:
            assert not C.needs_reshard(a, b), (a["key"], b["key"])
        again = C.sharded_shape_from_json(C.sharded_shape_to_json(a))
        assert again["key"] == a["key"] and boxes(again) == boxes(a)
        count = rng.choice([1, 2, 3, 4, 6, 8])
        resized, _ = C.resize_sharding(a, rng.randint(0, 4), count)
        assert resized["num_devices"] == count
        used = {axis for dim in resized["dim_axes"] for axis in dim}
        replicas = 1
        for axis, extent in enumerate(resized["mesh_dims"]):
            if axis not in used:
                replicas *= extent
        total = 1
        for s_ in sizes:
            total *= s_
        assert sum(volume(bx) for bx in boxes(resized)) == total * replicas, (a["key"], resized["key"])
    assert equivalent > 10 and in_place > 30
