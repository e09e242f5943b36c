"""In-tree build of the native library ``parameter_server_b200/_C*.so``.

Every ``.cu`` / ``.cpp`` under ``csrc/`` is compiled for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) and linked into one shared object that carries both
the pybind11 module ``_C`` and the plain ``extern "C"`` entry points. The role of the reference's
CMake build (CMakeLists.txt:6-44, pico-ps/CMakeLists.txt:1-46).

Usage:  python -m parameter_server_b200._build [-j N] [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
BUILD = PKG.parent / "build" / "obj"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _ext_suffix() -> str:
    return sysconfig.get_config_var("EXT_SUFFIX") or ".so"


def lib_path() -> Path:
    return PKG / ("_C" + _ext_suffix())


def node_path() -> Path:
    """The native master / pserver executable (``csrc/apps/psb_node.cpp``)."""
    return PKG / "bin" / "psb_node"


def _includes() -> list[str]:
    import pybind11

    inc = [pybind11.get_include(), sysconfig.get_paths()["include"], str(CSRC), "/usr/local/cuda/include"]
    return [f"-I{p}" for p in inc]


def _sources() -> list[Path]:
    srcs = sorted(list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cpp")))
    return srcs


def _header_digest() -> str:
    h = hashlib.sha1()
    for p in sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + [Path(__file__)]):
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def _compile_cmd(src: Path, obj: Path, verbose: bool) -> list[str]:
    common = ["-O3", "-std=c++17", *_includes()]
    if src.suffix == ".cu":
        cmd = [NVCC, *ARCH, "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden",
               "-Xcudafe", "--diag_suppress=20012", *common]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += ["-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++", "-fPIC", "-fvisibility=hidden", "-Wall", "-pthread", *common, "-c", str(src), "-o", str(obj)]
    return cmd


def build(jobs: int | None = None, force: bool = False, verbose: bool = False) -> Path:
    """Compile what changed and link. Returns the path of the shared object."""
    BUILD.mkdir(parents=True, exist_ok=True)
    digest = _header_digest()
    stamp = BUILD / "headers.sha1"
    if not stamp.exists() or stamp.read_text() != digest:
        force = True
    srcs = _sources()
    todo: list[tuple[Path, Path]] = []
    objs: list[Path] = []
    for s in srcs:
        rel = s.relative_to(CSRC)
        obj = BUILD / (str(rel).replace("/", "__") + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < s.stat().st_mtime:
            todo.append((s, obj))
    jobs = jobs or min(8, os.cpu_count() or 4)

    def run(pair: tuple[Path, Path]) -> tuple[Path, int, str]:
        src, obj = pair
        p = subprocess.run(_compile_cmd(src, obj, verbose), capture_output=True, text=True)
        return src, p.returncode, p.stdout + p.stderr

    failed = False
    if todo:
        with ThreadPoolExecutor(max_workers=jobs) as ex:
            for src, rc, out in ex.map(run, todo):
                tag = "ok" if rc == 0 else "FAILED"
                print(f"[build] {src.relative_to(PKG)}: {tag}", flush=True)
                if out.strip() and (rc != 0 or verbose):
                    print(out)
                failed |= rc != 0
    if failed:
        raise RuntimeError("native build failed")
    out = lib_path()
    # stale objects of deleted sources must not be linked
    keep = {o.name for o in objs}
    for o in BUILD.glob("*.o"):
        if o.name not in keep:
            o.unlink()
    # the shared object takes everything except the executables' mains; the node executable takes everything
    # except the Python bindings
    lib_objs = [o for o in objs if not o.name.startswith("apps__")]
    node_objs = [o for o in objs if not o.name.startswith("bindings")]
    node = node_path()
    if todo or not node.exists():
        node.parent.mkdir(parents=True, exist_ok=True)
        # --export-dynamic: operator plug-ins bind to the executable's registry accessor (psb_operator_factory)
        cmd = [NVCC, *ARCH, "-o", str(node), *[str(o) for o in node_objs], "-lpthread", "-ldl", "-lrt", "-Xlinker", "--export-dynamic"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            print(p.stdout + p.stderr)
            raise RuntimeError("link of psb_node failed")
        print(f"[build] linked {node.relative_to(PKG.parent)}", flush=True)
    if todo or not out.exists():
        cmd = [NVCC, *ARCH, "-shared", "-o", str(out), *[str(o) for o in lib_objs], "-lpthread", "-ldl", "-lrt"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            print(p.stdout + p.stderr)
            raise RuntimeError("link failed")
        print(f"[build] linked {out.relative_to(PKG.parent)}", flush=True)
    stamp.write_text(digest)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("-j", type=int, default=None)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    build(a.j, a.force, a.verbose)


if __name__ == "__main__":
    main()
