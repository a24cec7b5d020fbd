"""The C-ABI library loads without a GPU and exports every declared symbol;
host-only entry points behave; argument errors are reported before any launch."""
import ctypes as C
import re
from pathlib import Path

from gemmallm_b200 import _cabi
from gemmallm_b200._cabi import lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "moe_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(moe_b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 14
    raw = C.CDLL(str(_cabi.LIB_PATH))
    for n in names:
        assert hasattr(raw, n), f"{n} declared in moe_b200.h but not exported"
        assert n in _cabi.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_cabi.SIGNATURES) == set(names)


def test_version_and_sizes():
    assert lib.moe_b200_version() == 1
    n = _cabi.workspace_bytes(16384, 1024, 4096, 8, 2, _cabi.BF16)
    # perm + y (N*k*d) and h (N*k*f) dominate
    assert n > 2 * 16384 * (2 * 1024 + 4096) * 2
    lay = _cabi.workspace_layout(16384, 1024, 4096, 8, 2, _cabi.BF16)
    assert list(lay) == list(_cabi.WS_NAMES)
    offs = list(lay.values())
    assert offs == sorted(offs) and all(o % 1024 == 0 for o in offs)
    assert lib.moe_b200_plan_bytes(8) >= 4 * 8 * 8 + 2 * 8 * 128
    assert lib.moe_b200_router_blocks(65) == 2
    assert lib.moe_b200_decode_splits(4096) == 8 and lib.moe_b200_decode_splits(128) == 1
    assert lib.moe_b200_decode_max_rows() == 256
    assert lib.moe_b200_dispatch_scratch_bytes(1000, 8, 2) > 0


def test_bad_shapes_are_rejected_on_the_host():
    assert lib.moe_b200_workspace_bytes(16, 1020, 4096, 8, 2, _cabi.BF16) == 0   # d % 8
    assert lib.moe_b200_workspace_bytes(16, 1024, 4096, 300, 2, _cabi.BF16) == 0  # E > 256
    assert lib.moe_b200_workspace_bytes(16, 1024, 4096, 8, 9, _cabi.BF16) == 0    # k > 8
    assert lib.moe_b200_workspace_bytes(16, 1024, 4096, 2, 3, _cabi.BF16) == 0    # k > E
    assert lib.moe_b200_workspace_bytes(16, 1024, 4096, 8, 2, 7) == 0             # dtype
    assert b"dtype" in lib.moe_b200_last_error_string()
    # NULL workspace: error code, nothing launched
    rc = lib.moe_b200_forward(None, None, None, None, None, 16, 1024, 4096, 8, 2, _cabi.BF16, 0,
                              None, 0, None, None)
    assert rc == -1
    # misaligned workspace
    rc = lib.moe_b200_forward(None, None, None, None, None, 16, 1024, 4096, 8, 2, _cabi.BF16, 0,
                              8, 1 << 40, None, None)
    assert rc == -3
