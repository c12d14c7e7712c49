"""The C++ compiler and task runtime under AddressSanitizer + UndefinedBehaviorSanitizer and under
ThreadSanitizer (the reference has an ASAN build type for its host code, CMakeLists.txt:12-17).
``csrc/selftest/host_selftest.cc`` compiles pipelines with every schedule and executes the plans on
worker threads whose task bodies touch unlocked buffers, so a missing dependency edge is a data
race the thread sanitizer reports; it then loads the stored real-model programs of ``tests/testdata``,
compiles them offline, round-trips them through text and feeds the loader damaged copies. No Python
runs inside the instrumented process."""
import glob
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import pytest

from multimesh_jax_b200.csrc import build


@pytest.fixture(scope="module")
def programs():
    def one(kind):
        try:
            return build.build_selftest(kind)
        except build.SanitizerUnavailable as e:
            return e
    with ThreadPoolExecutor(max_workers=2) as ex:
        a, t = ex.map(one, ["address", "thread"])
    return {"address": a, "thread": t}


@pytest.mark.parametrize("sanitizer", ["address", "thread"])
def test_host_selftest_is_clean_under(sanitizer, programs):
    if isinstance(programs[sanitizer], Exception):
        pytest.skip(str(programs[sanitizer]))
    env = {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0", "UBSAN_OPTIONS": "print_stacktrace=1:halt_on_error=1",
           "TSAN_OPTIONS": "halt_on_error=1", "PATH": "/usr/bin:/bin"}
    stored = sorted(glob.glob(os.path.join(os.path.dirname(os.path.abspath(__file__)), "testdata", "*.mmprog.json")))
    assert len(stored) >= 6
    if sanitizer == "thread":
        stored = stored[:2]          # the loader is single-threaded; two files keep the slow build's run short
    proc = subprocess.run([str(programs[sanitizer]), "3", *stored], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                          timeout=600, env=env)
    out = proc.stdout
    assert proc.returncode == 0, out[-4000:]
    assert "host selftest ok" in out
    for marker in ("ERROR: AddressSanitizer", "runtime error:", "WARNING: ThreadSanitizer", "ERROR: LeakSanitizer"):
        assert marker not in out, out[-4000:]
