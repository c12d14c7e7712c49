"""The C++ compiler and task runtime under AddressSanitizer + UndefinedBehaviorSanitizer and under
ThreadSanitizer (the reference has an ASAN build type for its host code, CMakeLists.txt:12-17).
``csrc/selftest/host_selftest.cc`` compiles pipelines with every schedule and executes the plans on
worker threads whose task bodies touch unlocked buffers, so a missing dependency edge is a data
race the thread sanitizer reports. No Python runs inside the instrumented process."""
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
    proc = subprocess.run([str(programs[sanitizer]), "3"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                          timeout=600, env=env)
    out = proc.stdout
    assert proc.returncode == 0, out[-4000:]
    assert "host selftest ok" in out
    for marker in ("ERROR: AddressSanitizer", "runtime error:", "WARNING: ThreadSanitizer", "ERROR: LeakSanitizer"):
        assert marker not in out, out[-4000:]
