"""In-tree build of the native libraries.

Shared objects produced next to this file (plus ``libtyr_parquet.so``, see :func:`build_parquet`):

* ``libtyr_kernels.so`` - every ``csrc/*.cu`` file, compiled by nvcc for ``sm_100a`` only
  (``-gencode arch=compute_100a,code=sm_100a -lineinfo``).  The kernels are exported as plain
  ``extern "C"`` launchers that take raw device pointers and a stream, so the library does not
  depend on libtorch and compiles in seconds.
* ``libtyr_host.so`` - every ``csrc/host/*.cpp`` file (safetensors reader, token-shard loader,
  BOS finder, float ring buffer, WAV/PPM writers, parquet bridge, process-group bookkeeping),
  compiled with g++.

The reference builds one ``libTyrC`` with exactly one ``-gencode`` pair chosen by ``-Kgpu``
(cc/Makefile:112-128); here the only supported target is B200.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
CSRC = ROOT / "csrc"
OUT_DIR = Path(__file__).resolve().parent
OBJ_DIR = ROOT / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build tyr_b200 kernels")
    return cand


def _digest(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(str(p.name).encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build command failed:\n  %s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout, r.stderr))
    return r.stdout + r.stderr


def _link(cmd, out: Path):
    """Links into a sibling temporary file and renames it over ``out``, so a reader never sees a half-written library."""
    tmp = out.with_name(out.name + ".tmp")
    _run([*cmd, "-o", str(tmp)])
    os.replace(tmp, out)


CHECKED_UNITS = ("moe_nvfp4", "rope")       # translation units with index checks; the checked library holds only these


def build_kernels(verbose: bool = False, force: bool = False, checked: bool = False) -> Path:
    """``checked=True`` builds ``libtyr_kernels_checked.so``: the units listed in ``CHECKED_UNITS`` compiled with
    ``-DTYR_BOUNDS_CHECK`` (data-dependent indices are tested and violations recorded, see csrc/common.cuh)."""
    srcs = sorted(CSRC.glob("*.cu"))
    if checked:
        srcs = [s for s in srcs if s.stem in CHECKED_UNITS]
    hdrs = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    out = OUT_DIR / ("libtyr_kernels_checked.so" if checked else "libtyr_kernels.so")
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    base_flags = NVCC_FLAGS + (["-DTYR_BOUNDS_CHECK"] if checked else [])
    hdr_digest = _digest(hdrs, " ".join(base_flags))
    nvcc = _nvcc()
    jobs = []
    objs = []
    for s in srcs:
        obj = OBJ_DIR / (s.stem + (".checked.o" if checked else ".o"))
        stamp = OBJ_DIR / (s.stem + (".checked.sha" if checked else ".sha"))
        dig = _digest([s], hdr_digest)
        objs.append(obj)
        if force or not obj.exists() or not stamp.exists() or stamp.read_text() != dig:
            jobs.append((s, obj, stamp, dig))

    def compile_one(job):
        s, obj, stamp, dig = job
        flags = list(base_flags)
        if verbose:
            flags += ["-Xptxas", "-v"]
        log = _run([nvcc, *flags, "-I", str(CSRC), "-c", str(s), "-o", str(obj)])
        stamp.write_text(dig)
        return s.name, log

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for name, log in ex.map(compile_one, jobs):
                if verbose and log.strip():
                    print("[%s]\n%s" % (name, log))
    if jobs or not out.exists():
        _link([nvcc, "-shared", *map(str, objs), "-lcudart"], out)
    return out


def build_host(force: bool = False) -> Path:
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    hdrs = sorted((CSRC / "host").glob("*.h"))
    out = OUT_DIR / "libtyr_host.so"
    stamp = OBJ_DIR / "host.sha"
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    dig = _digest(srcs + hdrs, " ".join(CXX_FLAGS))
    if not force and out.exists() and stamp.exists() and stamp.read_text() == dig:
        return out
    cxx = shutil.which("g++") or "g++"
    _link([cxx, *CXX_FLAGS, "-shared", *map(str, srcs), "-ldl"], out)
    stamp.write_text(dig)
    return out


def build_parquet(force: bool = False):
    """``libtyr_parquet.so``: csrc/parquet/*.cpp against the Arrow C++ / parquet-cpp libraries inside the pyarrow wheel (the
    reference links the same ones, cc/Makefile:37-44).  Returns None when pyarrow is not installed."""
    try:
        import pyarrow as pa
    except Exception:
        return None
    srcs = sorted((CSRC / "parquet").glob("*.cpp"))
    libdir = Path(pa.get_library_dirs()[0])
    arrow = sorted(libdir.glob("libarrow.so.*"), key=lambda q: len(q.name))
    parquet = sorted(libdir.glob("libparquet.so.*"), key=lambda q: len(q.name))
    if not srcs or not arrow or not parquet:
        return None
    out = OUT_DIR / "libtyr_parquet.so"
    stamp = OBJ_DIR / "parquet.sha"
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    flags = ["-O2", "-std=c++20", "-fPIC", "-Wall", "-fvisibility=hidden"]
    dig = _digest(srcs, " ".join(flags) + pa.__version__)
    if not force and out.exists() and stamp.exists() and stamp.read_text() == dig:
        return out
    cxx = shutil.which("g++") or "g++"
    _link([cxx, *flags, "-shared", "-I", pa.get_include(), *map(str, srcs), "-L", str(libdir),
           "-l:" + parquet[0].name, "-l:" + arrow[0].name, "-Wl,-rpath," + str(libdir)], out)
    stamp.write_text(dig)
    return out


def build_all(verbose: bool = False, force: bool = False):
    build_kernels(verbose=verbose, force=force, checked=True)
    build_parquet(force=force)
    return build_kernels(verbose=verbose, force=force), build_host(force=force)


if __name__ == "__main__":
    k, h = build_all(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(k)
    print(h)
