"""In-tree build of the native code.

Two shared libraries are produced next to the Python package:

* ``_mm_kernels.so`` - the hand-written sm_100a CUDA kernels, compiled with
  ``nvcc -gencode arch=compute_100a,code=sm_100a`` and exposed through a plain
  C ABI (loaded with ctypes, so no PyTorch headers are needed to build it).
* ``_mm_C*.so``      - the C++ graph compiler and task-graph runtime with their
  pybind11 bindings (host code only).

Both are rebuilt only when a source file is newer than the library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
PKG = HERE.parent
KERNEL_DIR = HERE / "kernels"
BUILD_DIR = HERE / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def _cuda_home() -> Path:
    return Path(_nvcc()).resolve().parent.parent


def _newer(srcs, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in srcs)


def _run(cmd, log: Path | None = None):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.write_text(" ".join(map(str, cmd)) + "\n" + proc.stdout)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        raise RuntimeError(f"build command failed: {' '.join(map(str, cmd))}")
    return proc.stdout


def kernels_lib_path(checked: bool = False) -> Path:
    return PKG / ("_mm_kernels_checked.so" if checked else "_mm_kernels.so")


def host_lib_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return PKG / f"_mm_C{suffix}"


def build_kernels(force: bool = False, verbose: bool = False, checked: bool = False) -> Path:
    """Compile every .cu file for sm_100a and link ``_mm_kernels.so``. ``checked`` builds the
    variant with ``-DMM_CHECKED`` (``_mm_kernels_checked.so``): indices derived from run-time data
    are verified before use and violations are recorded in the status word instead of trapping;
    ``MM_CHECKED=1`` makes the package load that library."""
    out_dir = BUILD_DIR / "checked" if checked else BUILD_DIR
    out_dir.mkdir(parents=True, exist_ok=True)
    cus = sorted(KERNEL_DIR.glob("*.cu"))
    hdrs = sorted(KERNEL_DIR.glob("*.cuh")) + sorted(KERNEL_DIR.glob("*.h"))
    target = kernels_lib_path(checked)
    if not force and not _newer(cus + hdrs, target):
        return target
    nvcc = _nvcc()
    extra = ["-DMM_CHECKED"] if checked else []

    def compile_one(cu: Path) -> Path:
        obj = out_dir / (cu.stem + ".o")
        if force or _newer([cu] + hdrs, obj):
            out = _run([nvcc, *NVCC_FLAGS, *extra, "-I", str(KERNEL_DIR), "-c", str(cu), "-o", str(obj)],
                       log=out_dir / (cu.stem + ".ptxas.log"))
            if verbose:
                print(out)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(cus))) as ex:
        objs = list(ex.map(compile_one, cus))
    # link beside the target and rename: a reader never sees a half-written library
    tmp = target.with_name(target.name + ".tmp")
    _run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"])
    os.replace(tmp, target)
    return target


def build_host(force: bool = False) -> Path:
    """Compile the C++ compiler/runtime and its pybind11 module ``_mm_C``."""
    import pybind11

    BUILD_DIR.mkdir(exist_ok=True)
    srcs = sorted((HERE / "mmgraph").glob("*.cc")) + sorted((HERE / "mmrt").glob("*.cc")) + [
        HERE / "bindings.cc"]
    hdrs = sorted((HERE / "mmgraph").glob("*.h")) + sorted((HERE / "mmrt").glob("*.h"))
    target = host_lib_path()
    if not force and not _newer(srcs + hdrs, target):
        return target
    cuda = _cuda_home()
    # $CXX is ignored on purpose: a toolchain that links libstdc++ statically would give this
    # module a second copy of the C++ runtime next to the one PyTorch loads.
    cxx = os.environ.get("MM_CXX") or ("/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")
    inc = ["-I", str(HERE), "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
           "-I", str(cuda / "include")]
    flags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-sign-compare",
             "-pthread"]
    extra = os.environ.get("MM_HOST_CXXFLAGS", "").split()

    def compile_one(src: Path) -> Path:
        obj = BUILD_DIR / (src.parent.name + "_" + src.stem + ".host.o")
        if force or _newer([src] + hdrs, obj):
            _run([cxx, *flags, *extra, *inc, "-c", str(src), "-o", str(obj)])
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, srcs))
    # link beside the target and rename: a process that has the old module mapped keeps its file
    tmp = target.with_name(target.name + ".tmp")
    _run([cxx, "-shared", "-o", str(tmp), *map(str, objs), *extra,
          "-L", str(cuda / "lib64"), "-lcudart", "-Wl,-rpath," + str(cuda / "lib64"), "-pthread"])
    os.replace(tmp, target)
    return target


SANITIZER_FLAGS = {
    "address": ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer"],
    "thread": ["-fsanitize=thread"],
    "none": [],
}


class SanitizerUnavailable(RuntimeError):
    """No installed C++ compiler can link with the requested sanitizer runtime."""


def _compiler_with(flags, scratch: Path) -> str:
    """First of $CXX, g++, /usr/bin/g++, clang++ that links a trivial program with ``flags``."""
    probe = scratch / "probe.cc"
    probe.write_text("int main() { return 0; }\n")
    seen = []
    for cxx in [os.environ.get("CXX"), "g++", "/usr/bin/g++", "clang++"]:
        if not cxx or cxx in seen or not shutil.which(cxx):
            continue
        seen.append(cxx)
        proc = subprocess.run([cxx, "-pthread", *flags, str(probe), "-o", str(scratch / "probe")],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
        if proc.returncode == 0:
            return cxx
    raise SanitizerUnavailable(f"no compiler among {seen} links with {' '.join(flags)}")


def build_selftest(sanitizer: str = "address", force: bool = False) -> Path:
    """Builds ``selftest/host_selftest.cc`` with the compiler and runtime sources into a
    stand-alone program instrumented by ``sanitizer`` (``address`` = ASan + UBSan, ``thread`` =
    TSan, ``none``); one object per source, compiled in parallel. Returns the program's path."""
    flags = SANITIZER_FLAGS[sanitizer]
    # outside the source tree: the instrumented objects are large and of no use to anyone else
    out_dir = Path(tempfile.gettempdir()) / f"mm_selftest_{os.getuid()}" / sanitizer
    out_dir.mkdir(parents=True, exist_ok=True)
    srcs = ([HERE / "selftest" / "host_selftest.cc"] + sorted((HERE / "mmgraph").glob("*.cc"))
            + [HERE / "mmrt" / "runtime.cc", HERE / "mmrt" / "cuda_context.cc"])
    cuda = _cuda_home()
    hdrs = sorted((HERE / "mmgraph").glob("*.h")) + sorted((HERE / "mmrt").glob("*.h"))
    target = out_dir / "host_selftest"
    if not force and not _newer(srcs + hdrs, target):
        return target
    cxx = _compiler_with(flags, out_dir)

    def compile_one(src: Path) -> Path:
        obj = out_dir / (src.stem + ".o")
        if force or _newer([src] + hdrs, obj):
            _run([cxx, "-std=c++17", "-O0", "-g1", "-pthread", *flags, "-I", str(cuda / "include"), "-c", str(src),
                  "-o", str(obj)])
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    # the stream context is driven through its recording stand-in here; the CUDA runtime is linked
    # only because the same source also holds the real adaptor
    _run([cxx, "-pthread", *flags, "-o", str(target), *map(str, objs), "-L", str(cuda / "lib64"), "-lcudart", "-ldl",
          "-Wl,-rpath," + str(cuda / "lib64")])
    return target


def build_all(force: bool = False) -> None:
    build_kernels(force=force)
    build_kernels(force=force, checked=True)
    build_host(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built", kernels_lib_path(), host_lib_path())
