"""The C-ABI library loads and exports every symbol that include/af8.h declares.
No compute call is made, so this runs without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "af8.h")).read()
    return sorted(set(re.findall(r"AF8_API\s+[A-Za-z0-9_ ]+?\**\s*\*?(af8_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    for must in ("af8_version", "af8_last_error", "af8_fullrank_step", "af8_norm_finalize", "af8_set_qmap"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from adafactor8bit import _native
    path = _native.library_path()
    if not os.path.exists(path):
        import importlib.util
        spec = importlib.util.spec_from_file_location("af8_build", os.path.join(ROOT, "adafactor-8bit_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    handle = ctypes.CDLL(path)
    for name in declared_symbols():
        assert hasattr(handle, name), f"libaf8.so does not export {name}"
    # the Python binding knows the same set
    assert sorted(_native.PROTOTYPES) == declared_symbols()


def test_version_and_error_string():
    from adafactor8bit import _native
    assert _native.version() == 1
    assert isinstance(_native.lib().af8_last_error(), bytes)


def test_struct_sizes_match_header():
    from adafactor8bit import _native
    assert _native.FULLRANK_TENSOR.itemsize == 144
    assert _native.DYN_SCALARS.itemsize == 32
    assert _native.NORM_TENSOR.itemsize == 64
    assert _native.SCALE_TENSOR.itemsize == 64
    assert ctypes.sizeof(_native.FullrankCfg) == 48
    assert _native.APOLLO_APPLY_TENSOR.itemsize == 104


def test_bad_arguments_are_rejected_without_a_gpu():
    from adafactor8bit import _native
    lib = _native.lib()
    cfg = _native.FullrankCfg()
    cfg.block = 100   # not a multiple of 128
    rc = lib.af8_fullrank_step(ctypes.byref(cfg), None, ctypes.c_void_p(16), 1, 1, None, None, None)
    assert rc == _native.ERR_INVALID
    assert b"block" in lib.af8_last_error()
    with pytest.raises(RuntimeError):
        _native.check(rc, "af8_fullrank_step")
    assert lib.af8_fullrank_step(None, None, None, 0, 0, None, None, None) == _native.ERR_INVALID


def test_batched_entry_points_reject_empty_tables_without_a_gpu():
    """The table checks of the multi-tensor entry points run on the host before anything is enqueued."""
    import numpy as np
    from adafactor8bit import _native
    lib = _native.lib()
    assert lib.af8_apollo_apply_batch(None, None, 0, 0, _native.F32, _native.BF16, 0, None) == _native.ERR_INVALID
    t = np.zeros(2, dtype=_native.APOLLO_APPLY_TENSOR)
    for k in ("param", "grad", "sf", "scalars"):
        t[k] = 256
    t["rows"], t["cols"] = 64, 64
    t["first_chunk"] = [0, 5]                 # the second tensor starts at chunk 2, not 5
    rc = lib.af8_apollo_apply_batch(t.ctypes.data, ctypes.c_void_p(256), 2, 4, _native.F32, _native.BF16, 0, None)
    assert rc == _native.ERR_INVALID and b"first_chunk" in lib.af8_last_error()
    t["first_chunk"] = [0, 2]
    rc = lib.af8_apollo_apply_batch(t.ctypes.data, ctypes.c_void_p(256), 2, 5, _native.F32, _native.BF16, 0, None)
    assert rc == _native.ERR_INVALID and b"total_chunks" in lib.af8_last_error()
    assert lib.af8_factored_stats_boxes(None, None, None, 0, None, None, None, None) == _native.ERR_INVALID
