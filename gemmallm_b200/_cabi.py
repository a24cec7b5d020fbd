"""ctypes binding of libmoe_b200.so (include/moe_b200.h).

The library is the only implementation: if it has not been built there is no
fallback and importing this module raises. Build it with
``python -m gemmallm_b200.build``.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libmoe_b200.so"
ABI_VERSION = 2

F32, BF16 = 0, 1
FLAG_DEFAULT, FLAG_WS_CLEAN = 0, 1
READY_OFFSET, READY_INTS = 64, 320
DEV_OK, DEV_TIMEOUT, DEV_BAD_INDEX = 0, 1, 2

WS_NAMES = (
    "status", "logits", "idx", "w", "psum_part", "psum", "aux", "scratch",
    "cnt_slot", "offsets", "row_of", "perm", "h", "y", "part", "norm_w", "norm_c", "stats", "xn",
)
WS_NUM = len(WS_NAMES)

_vp, _i, _i64, _sz, _f = C.c_void_p, C.c_int, C.c_int64, C.c_size_t, C.c_float

# name -> (restype, argtypes); every symbol include/moe_b200.h declares
SIGNATURES = {
    "moe_b200_version": (_i, []),
    "moe_b200_last_error_string": (C.c_char_p, []),
    "moe_b200_workspace_bytes": (_sz, [_i64, _i, _i, _i, _i, _i]),
    "moe_b200_workspace_layout": (_i, [_i64, _i, _i, _i, _i, _i, C.POINTER(_sz)]),
    "moe_b200_plan_bytes": (_sz, [_i]),
    "moe_b200_plan_build": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _sz, _vp]),
    "moe_b200_lora_merge": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i, _i, _i, _vp, _vp, _vp]),
    "moe_b200_router": (_i, [_vp, _vp, _vp, _i64, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "moe_b200_router_blocks": (_i64, [_i64]),
    "moe_b200_dispatch": (_i, [_vp, _vp, _i64, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                               _vp, _vp, _vp]),
    "moe_b200_dispatch_scratch_bytes": (_sz, [_i64, _i, _i]),
    "moe_b200_dispatch_static": (_i, [_vp, _vp, _i64, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp,
                                      _vp, _vp, _vp]),
    "moe_b200_experts": (_i, [_vp, _vp, _vp, _i64, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "moe_b200_front_small": (_i, [_vp, _vp, _vp, _i64, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp,
                                  _vp, _vp, _vp, _vp]),
    "moe_b200_decode_tiny": (_i, [_vp] * 5 + [_i64, _i, _i, _i, _i] + [_vp] * 13),
    "moe_b200_front_small_split": (_i, [_vp, _vp, _vp, _i64, _i, _i, _i, _i] + [_vp] * 12 + [_vp]),
    "moe_b200_front_exchange_ints": (_i64, [_i64, _i, _i]),
    "moe_b200_experts_rows": (_i, [_vp, _vp, _vp, _i64, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "moe_b200_rows_splits": (_i, [_i64, _i, _i, _i]),
    "moe_b200_experts_decode_spec": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "moe_b200_decode_spec_rows": (_i, [_i64]),
    "moe_b200_experts_decode_fused": (_i, [_vp, _vp, _vp, _i64, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "moe_b200_experts_gemv": (_i, [_vp, _vp, _vp, _i64, _i, _i, _i, _vp, _vp, _vp]),
    "moe_b200_decode_splits": (_i, [_i]),
    "moe_b200_decode_max_rows": (_i64, []),
    "moe_b200_combine_decode": (_i, [_vp, _i, _i64, _vp, _vp, _vp, _vp, _i, _vp, _i64, _i, _i, _vp,
                                     _vp]),
    "moe_b200_combine": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i, _i, _vp, _vp]),
    "moe_b200_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i64, _i, _i, _i, _i, _i, _i, _vp,
                              _sz, _vp, _vp]),
    "moe_b200_norm_fold": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "moe_b200_router_norm": (_i, [_vp, _vp, _vp, _f, _i64, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp,
                                  _vp]),
    "moe_b200_dispatch_norm": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _vp, _vp, _vp, _vp,
                                    _vp, _vp, _vp, _vp, _vp, _vp]),
    "moe_b200_layernorm": (_i, [_vp, _vp, _vp, _f, _i64, _i, _i, _vp, _vp]),
    "moe_b200_attention": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _f, _vp, _vp]),
    "moe_b200_train_workspace_bytes": (_sz, [_i64, _i, _i, _i, _i, _i]),
    "moe_b200_train_workspace_layout": (_i, [_i64, _i, _i, _i, _i, _i, C.POINTER(_sz)]),
    "moe_b200_train_setup": (_i, [_i64, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "moe_b200_forward_train": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _i, _f, C.c_uint64,
                                    _vp, _sz, _vp, _sz, _vp, _vp]),
    "moe_b200_backward": (_i, [_vp, _vp, _vp, _vp, _f, _i64, _i, _i, _i, _i, _i, _f, C.c_uint64,
                               _vp, _sz, _vp, _sz, _vp, _vp]),
    "moe_b200_experts_train": (_i, [_vp, _vp, _vp, _i64, _i, _i, _i, _f, C.c_uint64, _vp, _sz, _vp, _vp,
                                    _vp, _vp]),
    "moe_b200_experts_backward": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _f, C.c_uint64, _vp, _sz,
                                       _vp, _vp, _vp]),
    "moe_b200_ep_symm_bytes": (_sz, [_i64, _i, _i, _i, _i]),
    "moe_b200_ep_symm_layout": (_i, [_i64, _i, _i, _i, _i, C.POINTER(_sz)]),
    "moe_b200_ep_workspace_bytes": (_sz, [_i64, _i, _i, _i, _i, _i]),
    "moe_b200_ep_workspace_layout": (_i, [_i64, _i, _i, _i, _i, _i, C.POINTER(_sz)]),
    "moe_b200_ep_setup": (_i, [_vp, _vp, _i64, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "moe_b200_ep_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _i, _i, _i, _i,
                                 _i, _i, _vp, _vp, _sz, _vp, _vp, _vp]),
    "moe_b200_read_status": (_i, [_vp, C.POINTER(C.c_int32), _vp]),
}


class MoeB200Error(RuntimeError):
    pass


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise MoeB200Error(
            f"{LIB_PATH} is missing. This package has no fallback path: build the CUDA "
            "library first with `python -m gemmallm_b200.build`.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    if lib.moe_b200_version() != ABI_VERSION:
        raise MoeB200Error("libmoe_b200.so ABI version mismatch; rebuild it")
    return lib


lib = _load()


def check(rc: int, what: str = "") -> None:
    """Raise on a non-zero return code of a library call."""
    if rc != 0:
        msg = lib.moe_b200_last_error_string().decode()
        raise MoeB200Error(f"{what or 'libmoe_b200'} failed with code {rc}: {msg}")


def workspace_bytes(N: int, d: int, f: int, E: int, k: int, dtype: int) -> int:
    n = lib.moe_b200_workspace_bytes(N, d, f, E, k, dtype)
    if n == 0:
        raise MoeB200Error(
            f"unsupported shape N={N} d={d} f={f} E={E} k={k} dtype={dtype}: "
            + lib.moe_b200_last_error_string().decode())
    return n


def workspace_layout(N: int, d: int, f: int, E: int, k: int, dtype: int) -> dict[str, int]:
    arr = (_sz * WS_NUM)()
    check(lib.moe_b200_workspace_layout(N, d, f, E, k, dtype, arr), "workspace_layout")
    return {name: int(arr[i]) for i, name in enumerate(WS_NAMES)}


TWS_NAMES = ("gu", "pair_of", "koff", "dy", "dh", "dxs", "w1t", "w2t", "tmaps", "xt", "ht", "dyt", "dgut",
             "dl", "dw", "ones", "dwg_f32", "dxr", "g_wg", "g_bg", "g_w1", "g_b1", "g_w2", "g_b2")


def train_workspace_layout(N: int, d: int, f: int, E: int, k: int, dtype: int) -> dict[str, int]:
    arr = (_sz * len(TWS_NAMES))()
    check(lib.moe_b200_train_workspace_layout(N, d, f, E, k, dtype, arr), "train_workspace_layout")
    return {name: int(arr[i]) for i, name in enumerate(TWS_NAMES)}


EP_STAGES = ("router", "dispatch", "experts", "combine")
EP_SYMM_NAMES = ("flags", "cnt_all", "recv_meta", "recv_x", "ret_y")
EP_WS_NAMES = ("status", "logits", "idx", "w", "psum_part", "psum", "aux", "scratch", "cnt_slot0",
               "offsets_local", "owner", "h")


def ep_symm_layout(N_local: int, d: int, E: int, k: int, world: int) -> dict[str, int]:
    arr = (_sz * len(EP_SYMM_NAMES))()
    check(lib.moe_b200_ep_symm_layout(N_local, d, E, k, world, arr), "ep_symm_layout")
    return {name: int(arr[i]) for i, name in enumerate(EP_SYMM_NAMES)}


def ep_workspace_layout(N_local: int, d: int, f: int, E: int, k: int, world: int) -> dict[str, int]:
    arr = (_sz * len(EP_WS_NAMES))()
    check(lib.moe_b200_ep_workspace_layout(N_local, d, f, E, k, world, arr), "ep_workspace_layout")
    return {name: int(arr[i]) for i, name in enumerate(EP_WS_NAMES)}


def ptr_array(ptrs) -> C.Array:
    return (C.c_void_p * len(ptrs))(*ptrs)


def read_status(status_ptr: int, stream: int) -> list[int]:
    out = (C.c_int32 * 16)()
    lib.moe_b200_read_status(status_ptr, out, stream)
    return list(out)
