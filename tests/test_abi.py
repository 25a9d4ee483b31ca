"""The C-ABI library loads and exports every symbol include/xattn_b200.h declares (no compute)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "xattn_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(xattn_b200_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    for required in ("xattn_b200_fwd", "xattn_b200_bwd", "xattn_b200_build_plan", "xattn_b200_build_varlen_plan"):
        assert required in names


def test_library_exports_every_declared_symbol():
    from xattn_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from xattn_b200.build import build
        build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    loaded = _lib.load()
    assert loaded.xattn_b200_abi_version() == _lib.ABI_VERSION == 2
    assert set(_lib.SYMBOLS) == set(declared_symbols())


def test_plan_bytes_layout():
    from xattn_b200 import _lib
    lib = _lib.load()
    assert lib.xattn_b200_plan_bytes(0, 1, 1) == 0
    # rows padded to 4 words twice, 4 words per query tile, 2 per key tile padded to 4
    assert lib.xattn_b200_plan_bytes(1, 130, 300) == 4 * (2 * 132 + 4 * 2 + 8 + 4)   # rows, query tiles, key tiles, key-tile order
    assert lib.xattn_b200_bwd_workspace_bytes(2, 4, 100) == 2 * 4 * 128 * (2 * 4 + 32)   # rows padded to 128
    assert lib.xattn_b200_bwd_workspace_bytes_hp(2, 4, 100) == 2 * 4 * 128 * (3 * 4 + 32)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from xattn_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(ImportError, match="no CPU fallback"):
        _lib.load()


def test_header_is_plain_c_and_structs_match_ctypes(tmp_path):
    """include/xattn_b200.h compiles as C11 on its own, and the ctypes mirrors have the C sizes."""
    import shutil
    import subprocess
    import ctypes as C
    from xattn_b200 import _lib
    if shutil.which("gcc") is None:
        pytest.skip("gcc not available")
    names = {"XattnPlanArgs": _lib.PlanArgs, "XattnVarlenPlanArgs": _lib.VarlenPlanArgs, "XattnFwdArgs": _lib.FwdArgs,
             "XattnBwdArgs": _lib.BwdArgs, "XattnGateArgs": _lib.GateArgs, "XattnConstantKeyArgs": _lib.ConstantKeyArgs,
             "XattnMergeArgs": _lib.MergeArgs}
    src = tmp_path / "sizes.c"
    body = "\n".join(f'  printf("{n} %zu\\n", sizeof({n}));' for n in names)
    src.write_text('#include <stdio.h>\n#include "xattn_b200.h"\nint main(void) {\n' + body + "\n  return 0;\n}\n")
    exe = tmp_path / "sizes"
    include = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-I", include, str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    sizes = dict(zip(out[::2], map(int, out[1::2])))
    for name, mirror in names.items():
        assert sizes[name] == C.sizeof(mirror), name
