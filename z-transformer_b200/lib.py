"""ctypes binding of libztattn.so, the C ABI declared in include/zt_attn.h.

Loading fails loudly when the shared library has not been built: there is no
Python or CPU stand-in for any entry point.
"""
from __future__ import annotations

import ctypes as C
import os

from ._build import LIB_PATH

_vp, _i, _sz, _d = C.c_void_p, C.c_int, C.c_size_t, C.c_double

_SIGNATURES = {
    # name: (restype, argtypes)      -- the reference's six
    "zt_attn_dim_ok": (_i, [_i]),
    "zt_attn_forward_shmem": (_sz, [_i, _i, _i]),
    "zt_attn_bwd_dq_shmem": (_sz, [_i, _i]),
    "zt_attn_bwd_dkdv_shmem": (_sz, [_i]),
    "zt_attn_forward": (_i, [_vp] * 4 + [_i] * 8 + [_vp]),
    "zt_attn_backward": (_i, [_vp] * 10 + [_i] * 5 + [_vp]),
    # extensions
    "zt_attn_last_error": (C.c_char_p, []),
    "zt_attn_last_path": (C.c_char_p, []),
    "zt_attn_set_verbose": (None, [_i]),
    "zt_attn_set_path": (_i, [_i]),
    "zt_attn_launch_count": (C.c_ulonglong, []),
    "zt_attn_tc_status": (_i, [C.POINTER(_i)]),
    "zt_attn_profile": (None, [_i]),
    "zt_attn_profile_read": (_i, [C.c_char_p, _sz]),
    "zt_attn_forward_batched": (_i, [_vp] * 5 + [_i] * 5 + [_vp]),
    "zt_attn_backward_batched": (_i, [_vp] * 11 + [_sz] + [_i] * 5 + [_vp]),
    "zt_attn_backward_workspace_bytes": (_sz, [_i] * 5),
    "zt_attn_forward_batched_keep": (_i, [_vp] * 6 + [_sz] + [_i] * 5 + [_vp, C.POINTER(C.c_ulonglong)]),
    "zt_attn_backward_batched_kept": (_i, [_vp] * 11 + [_sz] + [_i] * 5 + [_vp, C.c_ulonglong]),
    "zt_attn_forward_batched_keep_peers": (_i, [_vp] * 6 + [_sz] + [_i] * 5 + [_vp, C.POINTER(C.c_ulonglong),
                                                 C.POINTER(_vp), _i]),
    "zt_attn_backward_batched_kept_peers": (_i, [_vp] * 11 + [_sz] + [_i] * 5 + [_vp, C.c_ulonglong, C.POINTER(_vp), _i]),
    "zt_attn_reserve": (_i, [_i] * 5),
    "zt_attn_arena_bytes": (_sz, []),
    "zt_attn_tc_saturated": (_i, [C.POINTER(C.c_uint)]),
    "zt_attn_rope_workspace_bytes": (_sz, [_i] * 5),
    "zt_attn_forward_rope_batched": (_i, [_vp] * 6 + [_sz] + [_i] * 6 + [_d, _vp, C.POINTER(C.c_ulonglong)]),
    "zt_attn_backward_rope_batched": (_i, [_vp] * 11 + [_sz] + [_i] * 6 + [_d, _vp, C.c_ulonglong]),
    "zt_proj_workspace_bytes": (_sz, [_i] * 4),
    "zt_proj_forward": (_i, [_vp] * 4 + [_sz] + [_i] * 4 + [_vp]),
    "zt_proj_backward": (_i, [_vp] * 6 + [_sz] + [_i] * 4 + [_vp]),
    "zt_attn_block_forward": (_i, [_vp] * 8 + [_sz, _vp, _sz] + [_i] * 7 + [_d, _vp, C.POINTER(C.c_ulonglong)]),
    "zt_attn_decode": (_i, [_vp] * 7 + [_sz] + [_i] * 5 + [_vp]),
    "zt_attn_decode_workspace_bytes": (_sz, [_i] * 5),
    "zt_attn_decode_static": (_i, [_vp] * 6 + [_i] * 5 + [_vp]),
    "zt_attn_decode_static_capacity": (_sz, []),
    "zt_attn_decode_status": (_i, [_vp, C.POINTER(_i)]),
    "zt_kv_append": (_i, [_vp] * 6 + [_i] * 4 + [_vp]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def load():
    """The loaded library; raises with the build command when it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -c \"import __graft_entry__ as g; "
                "g.build()\"` (nvcc, sm_100a). There is no fallback implementation.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means the library is stale
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().zt_attn_last_error().decode()


def last_path() -> str:
    return load().zt_attn_last_path().decode()


def profile(on: bool) -> None:
    load().zt_attn_profile(1 if on else 0)


def profile_read() -> dict:
    """{kernel name: (launches, total device ms)} since the last read."""
    buf = C.create_string_buffer(8192)
    load().zt_attn_profile_read(buf, len(buf))
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms = line.split()
        out[name] = (int(n), float(ms))
    return out


def tc_status() -> int:
    """0 unless a tensor-core kernel gave up on a bounded wait (synchronise first)."""
    v = C.c_int(0)
    if load().zt_attn_tc_status(C.byref(v)) != 0:
        raise RuntimeError(last_error())
    return v.value


def tc_saturated() -> int:
    """Backward thread blocks that met the bound on dS since the last call (synchronise first); 0 in a correct run."""
    v = C.c_uint(0)
    if load().zt_attn_tc_saturated(C.byref(v)) != 0:
        raise RuntimeError(last_error())
    return v.value


def launch_count() -> int:
    return int(load().zt_attn_launch_count())
