"""In-tree build of the native extension ``llumnix_kv_b200/kvtransfer_ops*.so``.

The extension is one shared object holding the pybind11 module, the C++ engine and the
sm_100a kernels.  It is compiled with plain ``nvcc`` / ``g++`` (no torch headers) so that it
builds in seconds, loads on a machine without a GPU, and is found next to the package on a
GPU machine.  The reference builds its extension through CMake from ``setup.py``
(setup.py:27-142, kvtransfer/CMakeLists.txt); here the whole tree is a flat list of
translation units compiled in parallel.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
PKG = ROOT / "llumnix_kv_b200"
BUILD = ROOT / "build"
MODULE = "kvtransfer_ops"

NVCC = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")

GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]

# KVX_SANITIZE=address|thread builds the host code with that sanitizer into its own object directory (the
# reference configures none).  Run the CPU tests of such a build with the sanitizer runtime preloaded:
#   KVX_SANITIZE=address python -m llumnix_kv_b200._build -f
#   LD_PRELOAD=$(gcc -print-file-name=libasan.so) ASAN_OPTIONS=detect_leaks=0 python -m pytest tests -m "not gpu"
# KVX_SANITIZE=coverage builds the host code with gcov instrumentation instead (the reference's test build uses
# --coverage, kvtransfer/CMakeLists.txt:49-51): the .gcda files appear beside the objects in build_coverage/ when
# the test process exits.
SANITIZE = os.environ.get("KVX_SANITIZE", "")
if SANITIZE:
    BUILD = ROOT / f"build_{SANITIZE}"


def _ext_suffix() -> str:
    return sysconfig.get_config_var("EXT_SUFFIX") or ".so"


def target_path() -> Path:
    return PKG / f"{MODULE}{_ext_suffix()}"


def _includes() -> list[str]:
    import pybind11

    return [
        f"-I{CSRC}",
        f"-I{pybind11.get_include()}",
        f"-I{sysconfig.get_paths()['include']}",
        "-I/usr/local/cuda/include",
    ]


def sources() -> list[Path]:
    out: list[Path] = []
    for sub in ("core", "plan", "transport", "kernels", "naming", "topo", "store", "bind"):
        d = CSRC / sub
        if d.is_dir():
            out += sorted(d.glob("*.cpp")) + sorted(d.glob("*.cu"))
    return out


def _headers_digest() -> str:
    h = hashlib.sha1()
    for p in sorted(CSRC.rglob("*.h")) + sorted(CSRC.rglob("*.cuh")):
        h.update(p.read_bytes())
    return h.hexdigest()


def _compile_one(src: Path, hdr_digest: str, verbose: bool) -> Path:
    obj = BUILD / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
    stamp = obj.with_suffix(".stamp")
    key = hashlib.sha1(src.read_bytes() + hdr_digest.encode()).hexdigest()
    if obj.exists() and stamp.exists() and stamp.read_text() == key:
        return obj
    common = ["-O3", "-std=c++17", "-DNDEBUG"] + _includes()
    san = [f"-fsanitize={SANITIZE}", "-g", "-fno-omit-frame-pointer"] if SANITIZE else []
    if SANITIZE == "coverage":
        san = ["--coverage", "-g"]
    if src.suffix == ".cu":
        cmd = [NVCC, *GENCODE, "-lineinfo", "-Xcompiler", ",".join(["-fPIC", "-g1", "-Wall", "-Wextra", "-Wno-unused-parameter"] + san),
               "--expt-relaxed-constexpr", "-Xptxas", "-v" if verbose else "-O3", *common,
               "-c", str(src), "-o", str(obj)]
    else:
        cmd = [CXX, "-fPIC", "-g1", "-Wall", "-Wextra", "-Wshadow", "-Wno-unused-parameter", "-pthread", *san, *common,
               "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr)
    stamp.write_text(key)
    return obj


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile every translation unit for sm_100a and link the extension in-tree."""
    BUILD.mkdir(exist_ok=True)
    if force:
        for p in BUILD.glob("*.stamp"):
            p.unlink()
    srcs = sources()
    digest = _headers_digest()
    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, digest, verbose), srcs))
    target = target_path()
    newest = max(o.stat().st_mtime for o in objs)
    # every mode links to the same in-tree target: remember which one it holds
    mode_file = ROOT / "build" / ".linked_mode"
    mode_file.parent.mkdir(exist_ok=True)
    linked = mode_file.read_text() if mode_file.exists() else ""
    if not target.exists() or target.stat().st_mtime < newest or force or linked != SANITIZE:
        cmd = [NVCC, *GENCODE, "-shared", "-o", str(target), *map(str, objs), "-lpthread", "-lrt", "-ldl"]
        if SANITIZE == "coverage":
            cmd += ["-Xcompiler", "--coverage", "-lgcov"]
        elif SANITIZE:
            cmd += ["-Xcompiler", f"-fsanitize={SANITIZE}"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        mode_file.write_text(SANITIZE)
    return target


if __name__ == "__main__":
    t = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(t)
