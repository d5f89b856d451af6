"""The C++ mirror of src/cuda/device.zig (csrc/host/zt_host.{hpp,cpp}, libzthost.so) through its C shim:
the reference's own host tests (device.zig:502-645) on the pure functions, the holder's refusals before it
allocates, and -- on a GPU -- a forward and a backward through the holder against the oracle."""
import ctypes as C
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST_LIB = os.path.join(ROOT, "z-transformer_b200", "libzthost.so")
OK, DEGENERATE, TOO_LARGE, REFUSED, ALLOC_FAILED, TRANSFER_FAILED = range(6)
QUERY, KV, PER_ROW = 0, 1, 2
U64 = C.c_uint64


@pytest.fixture(scope="module")
def host(zt):  # zt: libztattn.so is built and loadable (libzthost.so links against it)
    assert os.path.exists(HOST_LIB), "build first: python -c 'import __graft_entry__ as g; g.build()'"
    L = C.CDLL(HOST_LIB)
    L.zth_bytes_for.argtypes = [C.c_int, U64, U64, U64, U64, C.POINTER(U64)]
    L.zth_to_c_int.argtypes = [U64, C.POINTER(C.c_int)]
    L.zth_forward_bounds.argtypes = [C.c_int] * 4
    L.zth_attn_init.argtypes = [U64, U64, U64, U64, C.POINTER(C.c_void_p)]
    L.zth_attn_deinit.argtypes = [C.c_void_p]
    L.zth_attn_total_bytes.argtypes = [C.c_void_p]
    L.zth_attn_total_bytes.restype = U64
    L.zth_attn_field.argtypes = [C.c_void_p, C.c_int]
    L.zth_attn_field.restype = C.c_void_p
    L.zth_attn_forward.argtypes = [C.c_void_p, C.c_int, C.c_int]
    L.zth_attn_forward_at.argtypes = [C.c_void_p] + [C.c_int] * 5
    L.zth_attn_backward.argtypes = [C.c_void_p, C.c_int]
    L.zth_attn_upload.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, U64]
    L.zth_attn_download.argtypes = [C.c_void_p, C.c_void_p, U64, C.c_void_p]
    return L


def bytes_for(L, kind, t, h, kv, d):
    out = U64(0)
    return L.zth_bytes_for(kind, t, h, kv, d, C.byref(out)), out.value


def test_sizes_and_refusals_of_the_pure_functions(host):
    assert bytes_for(host, QUERY, 256, 4, 2, 32) == (OK, 256 * 4 * 32 * 4)          # device.zig:502-507
    assert bytes_for(host, KV, 256, 4, 2, 32) == (OK, 256 * 2 * 32 * 4)
    assert bytes_for(host, PER_ROW, 256, 4, 2, 32) == (OK, 256 * 4 * 4)
    assert 2 * 4 * bytes_for(host, KV, 256, 4, 2, 32)[1] == 524288                   # device.zig:509-530
    for args in ((QUERY, 0, 4, 2, 32), (QUERY, 256, 0, 2, 32), (QUERY, 256, 4, 2, 0), (PER_ROW, 256, 4, 0, 32)):
        assert bytes_for(host, *args)[0] == DEGENERATE                               # device.zig:582-590
    for args in ((QUERY, 2 ** 64 - 1, 4, 2, 32), (QUERY, 1 << 40, 1 << 40, 1, 1), (KV, 2 ** 64 - 1, 4, 2, 32)):
        assert bytes_for(host, *args)[0] == TOO_LARGE                                # device.zig:592-598
    out = C.c_int(0)
    assert host.zth_to_c_int(1 << 31, C.byref(out)) == TOO_LARGE                     # device.zig:600-606
    assert host.zth_to_c_int(2 ** 31 - 1, C.byref(out)) == OK and out.value == 2 ** 31 - 1


def test_forward_bounds_agrees_with_the_python_mirror(host, zt):
    c_t, imax = 256, 2 ** 31 - 1                                                     # device.zig:612-645
    for args in ((c_t, 0, c_t, c_t), (c_t, 5, 6, 1), (c_t, c_t - 1, c_t, 1)):
        assert host.zth_forward_bounds(*args) == OK
    for args in ((c_t, 0, c_t + 1, 1), (c_t, 0, 0, 1), (c_t, 0, 1, c_t + 1), (c_t, 0, 1, 0), (c_t, c_t, c_t, 1),
                 (c_t, -1, c_t, 1), (c_t, imax, 1, 1), (c_t, imax - 1, 1, 2), (c_t, c_t + 1, c_t, 1)):
        assert host.zth_forward_bounds(*args) == TOO_LARGE
    for q_off in (-1, 0, 3, 7, 8):
        for n_keys in (0, 1, 4, 8, 9):
            for t in (0, 1, 2, 8, 9):
                try:
                    zt.forward_bounds(8, q_off, n_keys, t)
                    want = OK
                except zt.device.ShapeTooLarge:
                    want = TOO_LARGE
                assert host.zth_forward_bounds(8, q_off, n_keys, t) == want


def test_init_refuses_before_allocating(host):
    """device.zig:227-241: these never reach cudaMalloc, so they read the same with or without a GPU."""
    h = C.c_void_p()
    for args, want in (((8, 4, 2, 33), REFUSED), ((8, 5, 2, 32), REFUSED), ((1, 65536, 32768, 32), REFUSED),
                       ((1 << 31, 4, 2, 32), TOO_LARGE), ((0, 4, 2, 32), DEGENERATE)):
        assert host.zth_attn_init(*args, C.byref(h)) == want, args
        assert not h.value


@pytest.mark.gpu
def test_holder_forward_and_backward_against_the_oracle(host, oracle):
    T, H, Hkv, D = 200, 8, 2, 64
    q = oracle.fill_normal((T, H * D), 81, 0)
    k = oracle.fill_normal((T, Hkv * D), 81, 1)
    v = oracle.fill_normal((T, Hkv * D), 81, 2)
    do = oracle.fill_normal((T, H * D), 81, 3)
    h = C.c_void_p()
    assert host.zth_attn_init(T, H, Hkv, D, C.byref(h)) == OK
    try:
        assert host.zth_attn_total_bytes(h) == 4 * q.nbytes + 4 * k.nbytes + 3 * T * H * 4
        F = {n: host.zth_attn_field(h, i) for i, n in enumerate(
            ("q", "k", "v", "out", "dout", "dq", "dk", "dv", "row_max", "row_den", "row_del"))}
        for name, arr in (("q", q), ("k", k), ("v", v), ("dout", do)):
            assert host.zth_attn_upload(h, F[name], arr.ctypes.data, arr.size) == OK
        assert host.zth_attn_upload(h, F["k"], q.ctypes.data, q.size) == TOO_LARGE       # more than the buffer holds
        assert host.zth_attn_upload(h, q.ctypes.data, q.ctypes.data, 1) == TOO_LARGE     # not one of the holder's buffers
        assert host.zth_attn_forward(h, 1, 64) == OK
        out = np.empty_like(q)
        assert host.zth_attn_download(h, out.ctypes.data, out.size, F["out"]) == OK
        assert host.zth_attn_backward(h, 64) == OK
        dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
        for arr, name in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
            assert host.zth_attn_download(h, arr.ctypes.data, arr.size, F[name]) == OK
        assert host.zth_attn_forward_at(h, 1, 64, 0, T + 1, T) == TOO_LARGE              # forwardBounds first
        assert host.zth_attn_forward(h, 0, 64) == REFUSED                                # group_q 0: the C side refuses
    finally:
        host.zth_attn_deinit(h)
    ro = oracle.attention_forward(q, k, v, H, Hkv, D, threads=4)
    rdq, rdk, rdv = oracle.attention_backward(q, k, v, do, H, Hkv, D, threads=4)
    for got, ref in ((out, ro), (dq, rdq), (dk, rdk), (dv, rdv)):
        assert np.all(np.abs(got.astype(np.float64) - ref) <= 1e-5 + 1e-4 * np.abs(ref))


@pytest.mark.gpu
def test_cpp_pipeline_matches_the_batched_calls(host, zt):
    """zt::device::AttnPipeline (three streams, two slots, more sequences than slots) against the batched entry
    points on the same sequences, bit for bit."""
    import torch
    host.zth_pipeline_init.argtypes = [U64, U64, U64, U64, C.c_int, C.POINTER(C.c_void_p)]
    host.zth_pipeline_deinit.argtypes = [C.c_void_p]
    host.zth_pipeline_step.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 9
    B, T, H, Hkv, D = 5, 256, 8, 2, 64
    g = torch.Generator().manual_seed(91)
    hq, hdo = (torch.randn((B, T, H * D), generator=g).pin_memory() for _ in range(2))
    hk, hv = (torch.randn((B, T, Hkv * D), generator=g).pin_memory() for _ in range(2))
    hout, hdq = (torch.full((B, T, H * D), float("nan")).pin_memory() for _ in range(2))
    hdk, hdv = (torch.full((B, T, Hkv * D), float("nan")).pin_memory() for _ in range(2))
    hlse = torch.full((B, T, H), float("nan")).pin_memory()
    h = C.c_void_p()
    assert host.zth_pipeline_init(T, H, Hkv, D, 0, C.byref(h)) == DEGENERATE
    assert host.zth_pipeline_init(T, 5, 2, D, 2, C.byref(h)) == REFUSED
    assert host.zth_pipeline_init(T, H, Hkv, D, 2, C.byref(h)) == OK
    try:
        for _ in range(2):
            rc = host.zth_pipeline_step(h, B, hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), hdo.data_ptr(), hout.data_ptr(),
                                        hdq.data_ptr(), hdk.data_ptr(), hdv.data_ptr(), hlse.data_ptr())
            assert rc == OK
    finally:
        host.zth_pipeline_deinit(h)
    dev = torch.device("cuda:0")
    q, k, v, do = (x.to(dev) for x in (hq, hk, hv, hdo))
    out, lse = zt.attention_forward(q, k, v, H, Hkv, D, want_lse=True)
    dq, dk, dv = zt.attention_backward(q, k, v, out, lse, do, H, Hkv, D)
    for name, got, want in (("out", hout, out), ("lse", hlse, lse), ("dq", hdq, dq), ("dk", hdk, dk), ("dv", hdv, dv)):
        if name == "dq":  # (a sum over key tiles made in memory by the fused backward: equal run to run to rounding)
            assert bool(((got - want.cpu()).abs() <= 2e-6 + 2e-5 * want.cpu().abs()).all())
        else:
            assert torch.equal(got, want.cpu()), name
