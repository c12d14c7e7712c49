"""The records handed to the reshard pull kernel, checked on the CPU: for every planner case the
records of each destination device are executed by a few lines of numpy that follow the kernel's
addressing (base + sum(index * stride), at most four dimensions), and the destination tile must
equal the slice of the global tensor it stands for. Covers the planner, the merging of contiguous
trailing dimensions, the per-chunk tile shapes and the per-destination source rotation."""
import itertools

import numpy as np
import pytest

from multimesh_jax_b200 import _mm_C as C
from multimesh_jax_b200.parallel import symm
from test_sharding import CASES, shape

ELEM = 2        # bytes per element (bfloat16): bases are byte addresses, strides count elements


def _run_records(memory: np.ndarray, records):
    """memory: flat uint16 array addressed in elements (byte address / ELEM)."""
    for r in records:
        src_base, dst_base = r[0], r[1]
        ext, ss, ds = r[2:6], r[6:10], r[10:14]
        assert src_base % ELEM == 0 and dst_base % ELEM == 0
        for idx in itertools.product(*[range(e) for e in ext]):
            s = src_base // ELEM + sum(i * st for i, st in zip(idx, ss))
            d = dst_base // ELEM + sum(i * st for i, st in zip(idx, ds))
            memory[d] = memory[s]


EXTRA = [
    (shape("bfloat16", [4, 6, 8], [[0], [], []], [2], 0), shape("bfloat16", [4, 6, 8], [[], [], [0]], [2], 2)),
    (shape("bfloat16", [2, 4, 6, 8], [[], [0], [], []], [2], 0), shape("bfloat16", [2, 4, 6, 8], [[], [], [0], []], [2], 0)),
    (shape("bfloat16", [8, 12], [[0], [1]], [2, 2], 0), shape("bfloat16", [8, 12], [[1], [0]], [2, 2], 4)),
]


@pytest.mark.parametrize("src,dst", list(CASES) + EXTRA)
def test_records_move_every_element_to_its_place(src, dst):
    _check_case(src, dst)


def _random_layout(rng, sizes, start):
    """A random valid layout of `sizes`: a mesh of one to three axes of extent 1-4, each axis either
    unused (replication) or tiling a dimension it divides; several axes may tile one dimension."""
    mesh = [rng.choice([1, 2, 2, 3, 4]) for _ in range(rng.randint(1, 3))]
    dim_axes = [[] for _ in sizes]
    left = list(sizes)
    for axis, extent in enumerate(mesh):
        fits = [d for d in range(len(sizes)) if left[d] % extent == 0 and left[d] >= extent]
        if not fits or rng.random() < 0.25:
            continue
        d = rng.choice(fits)
        dim_axes[d].append(axis)
        left[d] //= extent
    return shape("bfloat16", list(sizes), dim_axes, mesh, start)


def test_random_layout_pairs_move_every_element_to_its_place():
    import random
    rng = random.Random(99)
    done = 0
    for _ in range(120):
        sizes = [rng.choice([2, 4, 6, 8, 12]) for _ in range(rng.randint(1, 4))]
        src = _random_layout(rng, sizes, rng.randint(0, 3))
        dst = _random_layout(rng, sizes, rng.randint(0, 9))
        _check_case(src, dst)
        done += 1
    assert done == 120


def _check_case(src, dst):
    sizes = src["sizes"]
    total = int(np.prod(sizes)) if sizes else 1
    glob = np.arange(1, total + 1, dtype=np.uint16).reshape(sizes)
    # lay the source tiles out one after another in a flat memory, then the destination tiles
    memory = np.zeros(4 * total * max(src["num_devices"], dst["num_devices"]) + 64, dtype=np.uint16)
    src_ptr, cursor = {}, 16
    for o in range(src["num_devices"]):
        lo, hi = C.tile_box(src, o)
        tile = glob[tuple(slice(a, b) for a, b in zip(lo, hi))]
        src_ptr[src["device_start"] + o] = cursor * ELEM
        memory[cursor:cursor + tile.size] = tile.reshape(-1)
        cursor += tile.size
    plan = C.plan_reshard(src, dst)
    for o in range(dst["num_devices"]):
        dev = dst["device_start"] + o
        lo, hi = C.tile_box(dst, o)
        want = glob[tuple(slice(a, b) for a, b in zip(lo, hi))]
        dst_base = cursor
        cursor += want.size
        mine = [c for c in plan["chunks"] if c["dst_device"] == dev]
        before = [dict(c, lo=list(c["lo"]), hi=list(c["hi"])) for c in mine]
        records = symm.build_pull_chunks(mine, list(src["shard_size"]), list(dst["shard_size"]),
                                         lambda d: src_ptr[d], dst_base * ELEM, ELEM)
        assert all(len(r) == 14 for r in records) and len(records) == len(mine)
        assert [c["lo"] for c in mine] == [c["lo"] for c in before]          # the plan is not modified
        _run_records(memory, records)
        got = memory[dst_base:dst_base + want.size].reshape(want.shape)
        np.testing.assert_array_equal(got, want)


def test_destinations_start_pulling_from_different_sources():
    src = shape("bfloat16", [8, 16], [[0], []], [4], 0)          # rows over devices 0..3
    dst = shape("bfloat16", [8, 16], [[], [0]], [4], 4)          # columns over devices 4..7: every pair talks
    plan = C.plan_reshard(src, dst)
    first_sources = []
    for o in range(4):
        mine = [c for c in plan["chunks"] if c["dst_device"] == 4 + o]
        recs = symm.build_pull_chunks(mine, list(src["shard_size"]), list(dst["shard_size"]),
                                      lambda d: 1000 * (d + 1) * ELEM, 0, ELEM)
        first_sources.append(recs[0][0] // (1000 * ELEM) - 1)
    assert sorted(first_sources) == [0, 1, 2, 3]                 # no two destinations begin at the same source


def test_counter_words_are_never_shared_between_launchers():
    """Every launcher of the pull kernel counts finished CTAs in a word of its own: two kernels
    that overlap on the GPU would otherwise mix their counts and raise done flags early."""
    import pytest
    words = symm.WordAllocator(1 << 14)
    owners = [f"launcher{i}" for i in range(symm.WordAllocator.NUM_COUNTERS)]
    got = [words.alloc_counter(o) for o in owners]
    assert len(set(got)) == len(got) and all(0 <= i < symm.WordAllocator.NUM_COUNTERS for i in got)
    assert words.counter_owner == dict(zip(got, owners))
    with pytest.raises(MemoryError):
        words.alloc_counter("one too many")
    # flags live behind the counter words and never overlap them
    flag = words.alloc_flag()
    assert flag >= 4 * symm.WordAllocator.NUM_COUNTERS
