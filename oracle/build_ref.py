"""Recipe for oracle/_ref: the reference's own CPU implementation of the attention path, compiled
from its sources where they lie (nothing is copied into this repository).

The reference's CPU-runnable implementation of the hot path is its FP64 torch oracle,
``tests/_reference.py`` (masks :35-131, masked softmax read :134-155) and
``tests/softdelta/reference.py`` (SoftDelta :9-71).  Its CUDA extension cannot be built without the
CUTLASS checkout its build system fetches, and refuses devices other than sm_90.  This script turns
the two Python files into extension modules with Cython and gcc:

    python oracle/build_ref.py <reference root>     ->  oracle/_ref/_reference.so, oracle/_ref/reference.so

The outputs stay under oracle/_ref/, which version control ignores (the intermediate C files are deleted).
They are test infrastructure: tests/ pins the restatement in oracle/attention_oracle.py against them,
and bench.py's reference arm times them; nothing in the package imports them.
"""
from __future__ import annotations

import importlib.util
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SOURCES = {"_reference": os.path.join("tests", "_reference.py"),
           "reference": os.path.join("tests", "softdelta", "reference.py")}


def build(reference_root: str, force: bool = False) -> dict:
    """Compile whatever of SOURCES exists under ``reference_root``; returns {module name: .so path}."""
    built = {}
    os.makedirs(OUT, exist_ok=True)
    include = sysconfig.get_paths()["include"]
    for name, rel in SOURCES.items():
        src = os.path.join(reference_root, rel)
        if not os.path.exists(src):
            continue
        so = os.path.join(OUT, name + ".so")
        if not force and os.path.exists(so) and os.path.getmtime(so) >= os.path.getmtime(src):
            built[name] = so
            continue
        c_file = os.path.join(OUT, name + ".c")
        subprocess.run([sys.executable, "-m", "cython", "-3", "--module-name", name, src, "-o", c_file], check=True)
        subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-I", include, c_file, "-o", so], check=True)
        os.remove(c_file)           # only the compiled module stays
        built[name] = so
    return built


def load(name: str = "_reference"):
    """The compiled reference module, or None when oracle/_ref has not been built."""
    so = os.path.join(OUT, name + ".so")
    if not os.path.exists(so):
        return None
    spec = importlib.util.spec_from_file_location(name, so)
    module = importlib.util.module_from_spec(spec)
    # the SoftDelta oracle imports its sibling by the reference's package path
    if name == "reference":
        base = load("_reference")
        if base is None:
            return None
        import types
        try:
            pkg = importlib.import_module("tests")
        except ImportError:
            pkg = sys.modules.setdefault("tests", types.ModuleType("tests"))
        sys.modules.setdefault("tests._reference", base)
        if not hasattr(pkg, "_reference"):
            setattr(pkg, "_reference", base)
    spec.loader.exec_module(module)
    return module


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python oracle/build_ref.py <reference root> [--force]")
    print(build(sys.argv[1], force="--force" in sys.argv))
