"""CPU-side checks of the C ABI: the shared library loads without a GPU, exports every symbol
include/dualquant_b200.h declares, and the ctypes table binds all of them.  No compute call."""
import ctypes
import os
import re

import pytest

from dualquant_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "dualquant_b200.h")).read()
    return sorted(set(re.findall(r"DQ_API\s+[\w\s\*]+?\b(dq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_expected_entry_points():
    names = _declared()
    assert len(names) >= 18
    for must in ("dq_init", "dq_quant_act_int4", "dq_gemm_w4a4_int4", "dq_linear_w4a4_int4",
                 "dq_pack_w_int4", "dq_last_error_string"):
        assert must in names


def test_library_exports_every_declared_symbol():
    if not os.path.exists(_lib.LIB_PATH):
        pytest.fail(f"{_lib.LIB_PATH} missing: run python -m dualquant_b200.build")
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in _declared():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_ctypes_table_covers_the_header():
    assert sorted(_lib.SIGNATURES) == _declared()
    lib = _lib.load()
    assert lib.dq_abi_version() == 2
    assert lib.dq_packed_w_bytes(200, 256) == 2 * 2 * 8448  # 2 row tiles x 2 k groups
    assert lib.dq_linear_w4a4_int4_scratch_bytes(16, 128, 4096) == 16 * 4096 + 256


def test_calls_fail_loudly_without_init():
    # no GPU work: an op on a device that was never initialised must return an error code
    lib = _lib.load()
    rc = lib.dq_unpack_w_int4(None, 128, 128, None, None)
    assert rc != 0
    assert _lib.last_error() != ""
