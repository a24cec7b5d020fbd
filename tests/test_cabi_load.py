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
    assert lib.moe_b200_version() == _cabi.ABI_VERSION
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
    rc = lib.moe_b200_forward(None, None, None, None, None, None, None, 0.0, 16, 1024, 4096, 8, 2, _cabi.BF16, 0,
                              None, 0, None, None)
    assert rc == -1
    # misaligned workspace
    rc = lib.moe_b200_forward(None, None, None, None, None, None, None, 0.0, 16, 1024, 4096, 8, 2, _cabi.BF16, 0,
                              8, 1 << 40, None, None)
    assert rc == -3


def test_small_and_mid_size_entry_points_check_their_arguments():
    """The weight-streaming entry points reject what they cannot run before any launch."""
    a = 1 << 20     # any non-NULL, 16-byte aligned address: nothing is dereferenced on these paths
    # routing-independent kernel: N <= 128, E <= 32
    rc = lib.moe_b200_experts_decode_spec(a, a, a, a, 129, 2, 1024, 4096, 8, a, a, a, a, None)
    assert rc == -7 and b"128" in lib.moe_b200_last_error_string()
    rc = lib.moe_b200_experts_decode_spec(a, a, a, a, 64, 2, 1024, 4096, 33, a, a, a, a, None)
    assert rc == -7
    rc = lib.moe_b200_experts_decode_spec(a, None, a, a, 64, 2, 1024, 4096, 8, a, a, a, a, None)
    assert rc == -1
    # sorted-rows kernel: K ranges within [1, 8] and not more than there are 64-wide K blocks
    assert lib.moe_b200_experts_rows(a, a, a, 512, 1024, 4096, 8, 9, a, a, a, a, None) == -2
    assert lib.moe_b200_experts_rows(a, a, a, 512, 1024, 64, 8, 2, a, a, a, a, None) == -2
    assert lib.moe_b200_experts_rows(a, a, a, 512, 1024, 4096, 8, 4, a, a, None, a, None) == -1
    assert lib.moe_b200_experts_rows(a + 8, a, a, 512, 1024, 4096, 8, 4, a, a, a, a, None) == -3
    # one counter per row block: far too many rows
    assert lib.moe_b200_experts_rows(a, a, a, 1 << 20, 1024, 4096, 8, 4, a, a, a, a, None) == -7
    # sizes the forward uses
    assert lib.moe_b200_decode_spec_rows(1) == 16 and lib.moe_b200_decode_spec_rows(65) == 128
    assert lib.moe_b200_rows_splits(1024, 1024, 4096, 8) == 4
    assert 1 <= lib.moe_b200_rows_splits(1024, 4096, 256, 8) <= 4 // 8 + 1
    # shared-work front: token limit
    assert lib.moe_b200_front_small_split(a, a, a, 2049, 1024, 8, 2, _cabi.BF16, *([a] * 12), None) == -7
    assert lib.moe_b200_front_exchange_ints(512, 8, 2) == 32 * 2 * 8 + 32 * 8
    # the single-launch kernels' fused entry point: row limit
    assert lib.moe_b200_experts_decode_fused(a, a, a, 257, 1024, 4096, 8, a, a, a, a, None) == -2
    # the one-launch block: one to eight tokens, at most 32 experts, no NULL output, aligned rows
    tiny = lambda N, d, f, E, k, x=a, out=a: lib.moe_b200_decode_tiny(
        x, a, a, a, None, N, d, f, E, k, a, a, a, a, a, a, a, a, a, a, out, a, None)
    assert tiny(9, 1024, 4096, 8, 2) == -7 and b"N <= 8" in lib.moe_b200_last_error_string()
    assert tiny(4, 1024, 4096, 33, 2) == -7
    assert tiny(4, 1024, 4096, 8, 2, out=None) == -1
    assert tiny(4, 1024, 4096, 8, 2, x=a + 8) == -3
