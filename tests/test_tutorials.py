"""Runs the five tutorials of docs/tutorials on virtual CPU devices (the counterpart of the
reference's tutorial notebooks, which all start with ``init(cpus=8)``). Tutorial 5 doubles as the
regression test for two compiler defects it exposed: activation derivatives written outside every
scope used to be coloured into forward tasks, and a chain of instructions delayed into a later task
left stale member lists behind, which the dependency check then reported as a cycle."""
import importlib.util
import pathlib

import pytest

TUTORIALS = pathlib.Path(__file__).resolve().parent.parent / "docs" / "tutorials"


def _load(name):
    spec = importlib.util.spec_from_file_location(name, TUTORIALS / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_tutorial_1_spmd_autosharding():
    assert _load("t01_spmd_autosharding").main() > 0


def test_tutorial_2_mpmd_autosharding():
    tasks = _load("t02_mpmd_autosharding").main()
    assert [t[1] for t in tasks] == [0, 2]


def test_tutorial_3_multimesh_contexts():
    assert "stage1_bwd" in _load("t03_multimesh_contexts").main()


def test_tutorial_4_module_tasks_train():
    losses = _load("t04_mlp_pipeline_module_tasks").main(steps=3)
    assert losses[-1] < losses[0]


@pytest.mark.parametrize("stages", [2, 4])
def test_tutorial_5_registered_tasks_zero_bubble(stages):
    assert len(_load("t05_mlp_pipeline_registered_tasks").main(stages=stages)) == stages - 1
