"""The C-ABI library loads and exports every function include/gsq.h and include/gsq_debug.h declare (no compute calls)."""

import ctypes
import os
import re

from gsq_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    src = open(os.path.join(ROOT, "include", "gsq.h")).read() + open(os.path.join(ROOT, "include", "gsq_debug.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(gsq_[a-z0-9_]+)\s*\(", src)))


def test_header_functions_are_exported():
    names = _declared()
    assert len(names) >= 14
    lib = ctypes.CDLL(_cabi.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert set(_cabi.EXPORTS) <= set(names)


def test_host_only_entry_points():
    lib = _cabi.lib
    assert lib.gsq_abi_version() >= 1
    assert [lib.gsq_type_block_bytes(t) for t in (12, 14, 21, 23, 2)] == [144, 210, 110, 136, 0]
    assert lib.gsq_strerror(0) == b"ok" and b"guard" in lib.gsq_strerror(-1)
    assert lib.gsq_q8_layout_for_type(12) == _cabi.LAYOUT_DS4 and lib.gsq_q8_layout_for_type(21) == _cabi.LAYOUT_D4
    # zero-size work returns before any CUDA call
    assert lib.gsq_mul_mat_vec_q8(None, 0, 0, 21, 1, None, 0, 5120, None, 0, 0, None) == 0
    assert lib.gsq_quantize_q8_1(None, 1, 0, 512, 512, None, None) == 0
    assert lib.gsq_iq3s_repack(None, 0, 220, 0, None) == 0
