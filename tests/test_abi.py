"""The C-ABI library loads and exports every symbol the public header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "poker2_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(p2b_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_declared_symbols():
    from poker2_b200 import _lib, build

    path = build.build()
    handle = ctypes.CDLL(path)
    declared = _declared_symbols()
    assert len(declared) >= 5
    for name in declared:
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"
    # the Python binding table covers the same set
    assert sorted(_lib.exported_symbols()) == declared
    assert handle.p2b_version() >= 1


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "poker2_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in src and "from oracle" not in src, f


def test_tree_builder_rejects_bad_arguments_without_a_gpu():
    """Argument checks come before any CUDA call: status code and message, no launch."""
    from poker2_b200 import _lib, build

    build.build()
    handle = _lib.lib()
    bins = (ctypes.c_float * 16)(*([0.5] * 16))
    dummy = (ctypes.c_int32 * 64)()
    p = ctypes.cast(dummy, ctypes.c_void_p)
    assert handle.p2b_tree_count(p, 1, bins, 14, 4, -1, p, p, None) == -1  # too many bet bins
    assert b"bet bins" in handle.p2b_last_error()
    assert handle.p2b_tree_count(p, 1, bins, 2, 64, -1, p, p, None) == -1  # depth beyond the limit
    assert b"max_depth" in handle.p2b_last_error()
    assert handle.p2b_tree_count(None, 1, bins, 2, 4, -1, p, p, None) == -1  # null roots
    assert handle.p2b_tree_records(p, None, 5, 1, bins, 2, 4, -1, p, p, p, p, p, p, None, None, None) == -1
    assert handle.p2b_tree_count(p, 0, bins, 2, 4, -1, p, p, None) == 0  # empty batch: nothing to do
