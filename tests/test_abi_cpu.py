"""CPU-only checks of the C ABI: the library loads, exports what include/zt_attn.h declares,
answers its pure functions like the reference, and refuses loudly without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "zt_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(zt_[a-z_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(zt):
    lib = zt.lib.load()
    names = declared_symbols()
    assert len(names) >= 17
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/zt_attn.h but not exported"
    assert set(zt.lib.EXPORTED_SYMBOLS) == set(names)


def test_dim_ok_is_even_and_32_to_256(zt):
    """src/cuda/attn_kernels.cu:648-659"""
    ok = zt.lib.load().zt_attn_dim_ok
    for d in (32, 34, 64, 80, 96, 128, 192, 256):
        assert ok(d) == 1
    for d in (0, -2, 2, 30, 31, 33, 127, 255, 257, 258, 1024):
        assert ok(d) == 0


def test_shmem_queries_keep_the_reference_formulas(zt):
    """Byte counts the reference's own run prints (outputs/bench/run-attn.log:49-59)."""
    L = zt.lib.load()
    assert (L.zt_attn_forward_shmem(32, 32, 1), L.zt_attn_bwd_dq_shmem(32, 32)) == (8704, 8960)
    assert (L.zt_attn_forward_shmem(128, 64, 1), L.zt_attn_bwd_dq_shmem(128, 64)) == (66816, 67584)
    assert (L.zt_attn_forward_shmem(96, 64, 1), L.zt_attn_bwd_dq_shmem(96, 64)) == (50304, 50944)
    assert (L.zt_attn_forward_shmem(192, 64, 1), L.zt_attn_bwd_dq_shmem(192, 64)) == (99840, 100864)
    assert (L.zt_attn_forward_shmem(256, 48, 1), L.zt_attn_bwd_dq_shmem(256, 48)) == (99904, 101120)
    assert L.zt_attn_bwd_dkdv_shmem(256) == 2048
    # group_q adds (dim + tile) floats per extra query (src/cuda/attn_kernels.cu:697-700)
    assert L.zt_attn_forward_shmem(32, 32, 4) == 8704 + 3 * 64 * 4


FWD_REFUSALS = [
    # (T, H, Hkv, D, group_q, max_tile, q_offset, n_keys), fragment of the reason -- in the
    # reference's order (src/cuda/attn_kernels.cu:843-906)
    ((0, 4, 2, 32, 1, 64, 0, 1), "T 0"),
    ((-1, 4, 2, 32, 1, 64, 0, 1), "T -1"),
    ((4, 4, 2, 33, 1, 64, 0, 4), "head_dim 33"),
    ((4, 4, 2, 30, 1, 64, 0, 4), "head_dim 30"),
    ((4, 4, 2, 258, 1, 64, 0, 4), "head_dim 258"),
    ((4, 3, 2, 32, 1, 64, 0, 4), "not a group"),
    ((4, 4, 0, 32, 1, 64, 0, 4), "not a group"),
    ((4, 65536, 32768, 32, 1, 64, 0, 4), "65535"),
    ((4, 4, 2, 32, 0, 64, 0, 4), "group_q 0"),
    ((4, 4, 2, 32, 65, 64, 0, 4), "group_q 65"),
    ((4, 4, 2, 256, 8, 64, 0, 4), "group_q 8"),
    ((1, 4, 2, 32, 1, 64, -1, 4), "q_offset -1"),
    ((1, 4, 2, 32, 1, 64, 0, 0), "n_keys 0"),
    ((4, 4, 2, 32, 1, 64, 1, 4), "q_offset 1"),
    ((1, 4, 2, 32, 1, 64, 2 ** 31 - 1, 1), "q_offset 2147483647"),
    ((4, 4, 2, 32, 1, 0, 0, 4), "max_tile 0"),
]


@pytest.mark.parametrize("args,fragment", FWD_REFUSALS)
def test_forward_refusals_in_the_reference_order(zt, args, fragment):
    L = zt.lib.load()
    L.zt_attn_set_verbose(0)
    one = ctypes.c_void_p(16)  # never dereferenced: every case is refused before any launch
    T, H, Hkv, D, gq, mt, qo, nk = args
    assert L.zt_attn_forward(one, one, one, one, T, H, Hkv, D, gq, mt, qo, nk, None) == 1
    assert fragment in zt.lib.last_error()
    L.zt_attn_set_verbose(1)


def test_backward_and_extension_refusals(zt):
    """src/cuda/attn_kernels.cu:962-990 for the backward's order."""
    L = zt.lib.load()
    L.zt_attn_set_verbose(0)
    p = ctypes.c_void_p(16)
    ten = [p] * 10
    assert L.zt_attn_backward(*ten, 0, 4, 2, 32, 64, None) == 1 and "T 0" in zt.lib.last_error()
    assert L.zt_attn_backward(*ten, 4, 4, 2, 31, 64, None) == 1 and "head_dim" in zt.lib.last_error()
    assert L.zt_attn_backward(*ten, 4, 5, 2, 32, 64, None) == 1 and "group" in zt.lib.last_error()
    assert L.zt_attn_backward(*ten, 4, 4, 2, 32, 0, None) == 1 and "max_tile" in zt.lib.last_error()
    assert L.zt_attn_forward_batched(p, p, p, p, None, 0, 4, 4, 2, 32, None) == 1
    assert "batch 0" in zt.lib.last_error()
    assert L.zt_attn_decode(p, p, p, p, p, None, p, 0, 2, 16, 4, 2, 32, None) == 1
    assert "workspace" in zt.lib.last_error()
    assert L.zt_attn_decode_workspace_bytes(2, 16, 3, 2, 32) == 0
    assert L.zt_attn_decode_workspace_bytes(64, 8192, 32, 8, 128) > 0
    L.zt_attn_set_verbose(1)


def test_newer_extension_refusals(zt):
    """Refusals that are decided on the host, before any device is looked at: peer lists, the projection's shapes and
    workspace, a stale token's form, the reserve call's geometry."""
    L = zt.lib.load()
    L.zt_attn_set_verbose(0)
    p = ctypes.c_void_p(256)
    tok = ctypes.c_ulonglong(7)
    peers = (ctypes.c_void_p * 8)(*([256] * 8))
    # more than seven peer copies; a null list; a misaligned peer
    assert L.zt_attn_forward_batched_keep_peers(p, p, p, p, p, p, 1 << 30, 1, 128, 4, 2, 64, None, ctypes.byref(tok),
                                                peers, 8) == 1
    assert "peer copies" in zt.lib.last_error() and tok.value == 7  # refused before the token was touched
    assert L.zt_attn_forward_batched_keep_peers(p, p, p, p, p, p, 1 << 30, 1, 128, 4, 2, 64, None, None, None, 2) == 1
    assert "null list" in zt.lib.last_error()
    bad = (ctypes.c_void_p * 2)(256, 260)
    assert L.zt_attn_backward_batched_kept_peers(*([p] * 11), 1 << 30, 1, 128, 4, 2, 64, None, 0, bad, 2) == 1
    assert "16-byte aligned" in zt.lib.last_error()
    # the projection: extents that are not multiples of 64, a missing workspace
    assert L.zt_proj_forward(p, p, p, p, 1 << 30, 1, 8, 100, 64, None) == 1 and "multiples of 64" in zt.lib.last_error()
    assert L.zt_proj_backward(p, p, p, p, p, None, 0, 1, 8, 64, 64, None) == 1 and "workspace" in zt.lib.last_error()
    assert L.zt_proj_workspace_bytes(2, 100, 128, 64) > 2 * (2 * 100 * 128 + 128 * 64 + 2 * 100 * 64)
    assert L.zt_proj_workspace_bytes(0, 100, 128, 64) == 0
    # reserve: the geometry checks of every launching call
    assert L.zt_attn_reserve(1, 0, 4, 2, 64) == 1 and "T 0" in zt.lib.last_error()
    assert L.zt_attn_reserve(1, 128, 5, 2, 64) == 1 and "group" in zt.lib.last_error()
    assert L.zt_attn_arena_bytes() >= 0
    L.zt_attn_set_verbose(1)


def test_no_cpu_fallback_without_a_device(zt):
    """A well-formed call on a machine without a GPU is refused, never computed on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    L = zt.lib.load()
    L.zt_attn_set_verbose(0)
    p = ctypes.c_void_p(16)
    assert L.zt_attn_forward(p, p, p, p, 4, 4, 2, 32, 1, 64, 0, 4, None) == 1
    assert "no usable CUDA device" in zt.lib.last_error()
    with pytest.raises(RuntimeError):
        zt.attention_forward(torch.zeros(4, 128), torch.zeros(4, 64), torch.zeros(4, 64), 4, 2, 32)
    L.zt_attn_set_verbose(1)
