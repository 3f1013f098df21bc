"""The C-ABI library builds for sm_100a on a machine without a GPU, loads, and exports every
function that ``include/neuropress_b200.h`` declares.  No compute call is made here."""

import ctypes
import re
from pathlib import Path

import pytest

from neuropress_b200 import _cabi

HEADER = Path(__file__).resolve().parents[1] / "include" / "neuropress_b200.h"


def declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(npb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_the_binding_lists():
    assert declared_functions() == sorted(_cabi.EXPORTED_SYMBOLS)


def test_library_exports_every_declared_symbol():
    if not _cabi.library_available():
        pytest.skip("library not built (run python -m neuropress_b200.build)")
    lib = ctypes.CDLL(str(_cabi.LIB_PATH))
    for name in declared_functions():
        assert hasattr(lib, name), name


def test_status_strings_and_version():
    if not _cabi.library_available():
        pytest.skip("library not built")
    lib = _cabi.load_library()
    assert lib.npb_version() >= 100
    assert lib.npb_status_string(0) == b"ok"
    texts = {lib.npb_status_string(i) for i in range(8)}
    assert len(texts) == 8 and b"unknown status" not in texts
    assert lib.npb_status_string(99) == b"unknown status"
    with pytest.raises(RuntimeError, match="alignment|aligned"):
        _cabi.check(4, "x")


def test_struct_layouts_match_the_header():
    # npb_vq_weight: 3 pointers-or-int64 + ... = 80 bytes; npb_q_weight: 32 bytes (LP64).
    assert ctypes.sizeof(_cabi.VQWeightStruct) == 80
    assert ctypes.sizeof(_cabi.QWeightStruct) == 32
    assert _cabi.VQWeightStruct.centroids.offset == 24
    assert _cabi.VQWeightStruct.res_packed.offset == 40
    assert _cabi.VQWeightStruct.row_scale.offset == 72
