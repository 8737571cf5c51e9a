"""Binding / export consistency (the role of the reference's generated FFI header + `nm` export check,
Tyr/GenerateFfiHeader.lean, lakefile.lean:84-133): every native symbol the Python side names must be exported by a built
library, and every exported entry point must be named by the Python side or the tests."""
import re
import subprocess
from pathlib import Path

from tyr_b200 import _native

ROOT = Path(__file__).resolve().parent.parent
SYMBOL = re.compile(r"\b(tyr_[a-z0-9_]+)\b")
OPTIONAL = set()                 # symbols probed with hasattr() that a build may leave out


def _python_names():
    names = set()
    for base in ("tyr_b200", "tests", "bench.py", "__graft_entry__.py", "baseline"):
        p = ROOT / base
        files = [p] if p.is_file() else list(p.rglob("*.py"))
        for f in files:
            if f.name == "test_native_exports.py":
                continue
            text = f.read_text()
            names.update(m for m in set(SYMBOL.findall(text))
                         if re.search(r'(?:lib\.|\(\)\.)' + re.escape(m) + r'(?![a-z0-9_])', text) or f'"{m}"' in text or f".{m}(" in text)
    return {n for n in names if not n.startswith("tyr_b200")}


def _exported(lib_name):
    out = subprocess.run(["nm", "-D", "--defined-only", str(ROOT / "tyr_b200" / "_native" / lib_name)], capture_output=True, text=True, check=True).stdout
    return {line.split()[-1] for line in out.splitlines() if " T " in line and line.split()[-1].startswith("tyr_")}


def test_every_bound_symbol_is_exported_and_every_export_is_bound():
    _native.kernels(), _native.host()          # builds the libraries when missing
    from tyr_b200._native import checked
    checked.checked()
    exported = _exported("libtyr_kernels.so") | _exported("libtyr_host.so") | _exported("libtyr_kernels_checked.so")
    if _native.parquet() is not None:
        exported |= _exported("libtyr_parquet.so")
    else:
        exported |= {n for n in _python_names() if n.startswith("tyr_parquet_")}
    named = _python_names()
    missing = sorted(n for n in named if n not in exported and n not in OPTIONAL)
    assert not missing, f"Python names native symbols that no library exports: {missing}"
    unbound = sorted(exported - named)
    assert not unbound, f"exported entry points with no Python binding or test: {unbound}"
