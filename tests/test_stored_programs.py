"""Stored programs: real-model training steps kept as files and compiled offline (no model code,
no tensors, no device) - regression fixtures for the whole MPMD pipeline."""
import json
import os

import pytest
import torch

import multimesh_jax_b200 as mm
from multimesh_jax_b200 import _mm_C

DATA = os.path.join(os.path.dirname(os.path.abspath(__file__)), "testdata")
with open(os.path.join(DATA, "expected.json")) as f:
    EXPECTED = json.load(f)


@pytest.mark.parametrize("name", sorted(EXPECTED))
def test_stored_program_compiles_offline_to_the_expected_plan(name):
    want = EXPECTED[name]
    got = mm.compile_program_file(os.path.join(DATA, name + ".mmprog.json"))
    assert got["status"] == 0 and got["message"] == "" and got["hazards"] == ""
    for key in ("templates", "template_names", "stores", "tasks", "reshards", "reshard_bytes",
                "temp_bytes_per_device_max", "device_high_water_max", "device_high_water", "stats", "plan_hash"):
        assert got[key] == want[key], (name, key, got[key], want[key])
    # compiling the same file twice is deterministic down to the mock runtime's operation hash
    again = mm.compile_program_file(os.path.join(DATA, name + ".mmprog.json"))
    assert again["operation_hash"] == got["operation_hash"] and again["plan_hash"] == got["plan_hash"]


def test_fake_device_memory_size_decides_whether_the_plan_fits():
    path = os.path.join(DATA, "llama_pp4_zero_bubble.mmprog.json")
    need = mm.compile_program_file(path)["device_high_water_max"]
    assert mm.compile_program_file(path, device_memory_bytes=need)["fits"]
    assert not mm.compile_program_file(path, device_memory_bytes=need - 1)["fits"]
    assert mm.compile_program_file(path, device_memory_bytes=0)["fits"]          # 0 = no limit


def test_program_written_by_compile_function_gives_the_same_plan_when_read_back(tmp_path):
    from multimesh_jax_b200.models import llama
    from multimesh_jax_b200.runtime.collectives import Topology
    cfg = llama.LlamaConfig.tiny(n_layers=4, n_heads=4, n_kv_heads=2, d_model=64, d_ff=96, vocab=128)
    cfg.dtype = torch.float32
    B, S, MB = 8, 16, 2
    params = llama.init_params(cfg)
    opt_state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-2), seq_len=S, global_batch=B, microbatch_size=MB)
    mesh = mm.MultiMesh((2, 1, 2), ("stage", "data", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=2)
    path = tmp_path / "step.mmprog.json"
    with mesh:
        exe = mm.compile_function(step, (params, opt_state, tokens, tokens, cos, sin), mesh=mesh,
                                  context=_mm_C.MockContext(4), topology=Topology("cpu", 4), donate_argnums=(0, 1),
                                  save_program=str(path))
    got = mm.compile_program_file(str(path), want_plan=True)
    # regex task contexts were resolved when the file was written; the reader needs none of them
    assert json.dumps(got["plan"]["ops"], sort_keys=True) == json.dumps(exe.plan["ops"], sort_keys=True)
    assert [t["name"] for t in got["plan"]["templates"]] == [t["name"] for t in exe.plan["templates"]]
    assert got["plan"]["stats"] == exe.plan["stats"]
    # the graph survives a second round trip unchanged
    g, part, cfg2 = _mm_C.load_program(str(path))
    path2 = tmp_path / "again.mmprog.json"
    _mm_C.save_program(g, part, cfg2, str(path2))
    assert json.load(open(path))["graph"] == json.load(open(path2))["graph"]
    exe.shutdown()


def test_unknown_format_and_bad_ids_are_rejected(tmp_path):
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"format": "something else"}))
    with pytest.raises(RuntimeError):
        mm.compile_program_file(str(bad))
    text = open(os.path.join(DATA, "llama_tp2_sequence_parallel.mmprog.json")).read()
    for cut in (len(text) // 7, len(text) // 2, len(text) - 2):      # text that ends early is refused
        bad.write_text(text[:cut])
        with pytest.raises(RuntimeError, match="json"):
            mm.compile_program_file(str(bad))
    prog = json.loads(text)
    prog["graph"]["nodes"][0]["inputs"] = [10 ** 6]
    bad.write_text(json.dumps(prog))
    with pytest.raises(RuntimeError):
        mm.compile_program_file(str(bad))
    # every table that holds ids is checked before a pass follows one
    for damage, message in (
            (lambda g: g["order"].__setitem__(3, 7880), "operator id out of range"),
            (lambda g: g["order"].__setitem__(3, g["order"][2]), "operator listed twice"),
            (lambda g: g["values"][g["nodes"][5]["outputs"][0]].__setitem__("producer", 4), "does not name its producer"),
            (lambda g: g["nodes"][5].__setitem__("loop", 9), "unknown loop"),
            (lambda g: g["donated_inputs"].append(10 ** 6), "donated input"),
            (lambda g: g["values"][0].__setitem__("shape", [-4, 64]), "dimension out of range"),
            (lambda g: g["loops"][0].__setitem__("num_microbatches", 0), "microbatches")):
        prog = json.loads(text)
        damage(prog["graph"])
        bad.write_text(json.dumps(prog))
        with pytest.raises(RuntimeError, match=message):
            mm.compile_program_file(str(bad))
    prog = json.loads(text)
    prog["num_devices"] = 0
    bad.write_text(json.dumps(prog))
    with pytest.raises(RuntimeError, match="device range"):
        mm.compile_program_file(str(bad))
