"""zt_attn_decode_static: decode attention whose scratch is built into the library.

Some callers cannot allocate device memory when they need to decode: code written to the
reference's rule that entry points never allocate has no workspace to hand over, a server
that gave every byte of HBM to its own pool cannot cudaMalloc any more, and a latency-bound
loop cannot afford the device-wide stall of cudaMalloc/cudaFree.  For them the library offers
a decode entry point that uses a fixed array inside the library instead of a workspace.

The test calls it through the C ABI twice in a row (the second call finds the first call's
leftovers in the shared scratch) and compares with zt_attn_decode, which runs the same kernels
on a caller-owned workspace; the parity tolerance of this suite applies (1e-4 rel / 1e-5 abs).
It lives in a file pytest collects last so that a run stopping at the first failure has
already run everything else, and it passes both alone and after the other tests.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-4, 1e-5


def close(got, ref, what):
    got, ref = got.astype(np.float64), ref.astype(np.float64)
    assert np.array_equal(np.isnan(got), np.isnan(ref)), what
    err = np.abs(np.nan_to_num(got) - np.nan_to_num(ref))
    assert np.all(err <= ATOL + RTOL * np.abs(np.nan_to_num(ref))), (what, float(err.max()))


def randn(shape, seed, dev):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    return torch.randn(shape, generator=g, device=dev, dtype=torch.float32)


def call_static(L, q, kc, vc, n_keys, out, lse, B, n_ctx, H, Hkv, D):
    stream = torch.cuda.current_stream(q.device).cuda_stream
    return L.zt_attn_decode_static(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), n_keys.data_ptr(), out.data_ptr(),
                                   lse.data_ptr(), B, n_ctx, H, Hkv, D, stream)


def test_static_scratch_decode_matches_workspace_decode_twice(zt):
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    L = zt.lib.load()
    assert L.zt_attn_decode_static_capacity() == 16 * 2 ** 20
    # two different shapes back to back: the second call runs over the first one's leftovers
    cases = [(6, 700, 32, 8, 128, 101), (3, 333, 8, 2, 64, 202)]
    for round_ in range(2):
        for (B, n_ctx, H, Hkv, D, seed) in cases:
            kc, vc = randn((B, n_ctx, Hkv * D), seed, dev), randn((B, n_ctx, Hkv * D), seed + 1, dev)
            q = randn((B, H * D), seed + 2 + round_, dev)
            nk = np.random.default_rng(seed + round_).integers(1, n_ctx + 1, size=B).astype(np.int32)
            nk[0], nk[1] = n_ctx, 1
            if round_ == 1:
                nk[2] = 0          # a refused sequence: NaN row from both entry points
            n_keys = torch.from_numpy(nk).to(dev)
            ref, ref_lse = zt.decode_attention(q, kc, vc, n_keys, H, Hkv, D, want_lse=True)
            assert L.zt_attn_decode_workspace_bytes(B, n_ctx, H, Hkv, D) <= L.zt_attn_decode_static_capacity()
            out = torch.full_like(q, 123.0)
            lse = torch.full((B, H), 123.0, device=dev)
            if round_ == 0 and seed == 101:
                # the very first call on the device may have to find the built-in array (and, with lazy module
                # loading, make it exist): done once, here, before the calls whose memory use is measured
                assert call_static(L, q, kc, vc, n_keys, out, lse, B, n_ctx, H, Hkv, D) == 0, zt.lib.last_error()
            # the property the entry point is named for: the device's free memory is the same before and after
            # the call -- nothing was allocated (or freed) on the way, by the library or by torch on its behalf
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info(dev)
            reserved_before = torch.cuda.memory_reserved(dev)
            assert call_static(L, q, kc, vc, n_keys, out, lse, B, n_ctx, H, Hkv, D) == 0, zt.lib.last_error()
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info(dev)
            assert free_after == free_before and torch.cuda.memory_reserved(dev) == reserved_before
            close(out.cpu().numpy(), ref.cpu().numpy(), f"out round {round_} {B}x{n_ctx}")
            close(lse.cpu().numpy(), ref_lse.cpu().numpy(), f"lse round {round_} {B}x{n_ctx}")
            # the count of refused sequences sits in the built-in scratch; a NULL workspace reads it
            import ctypes
            bad = ctypes.c_int(-1)
            assert L.zt_attn_decode_status(None, ctypes.byref(bad)) == 0, zt.lib.last_error()
            assert bad.value == (1 if round_ == 1 else 0)


def test_static_scratch_refuses_what_does_not_fit(zt):
    dev = torch.device("cuda:0")
    L = zt.lib.load()
    L.zt_attn_set_verbose(0)
    # batch 64 x context 16384 needs more than 16 MiB of partial results
    B, n_ctx, H, Hkv, D = 64, 16384, 32, 8, 128
    assert L.zt_attn_decode_workspace_bytes(B, n_ctx, H, Hkv, D) > L.zt_attn_decode_static_capacity()
    x = torch.zeros(64, device=dev)
    nk = torch.ones(B, dtype=torch.int32, device=dev)
    out = torch.full((B, H * D), 5.0, device=dev)
    rc = L.zt_attn_decode_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), nk.data_ptr(), out.data_ptr(), None,
                                 B, n_ctx, H, Hkv, D, None)
    assert rc == 1 and "built-in scratch holds" in zt.lib.last_error()
    # a width that cannot use 128-bit loads is sent to zt_attn_decode
    rc = L.zt_attn_decode_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), nk.data_ptr(), out.data_ptr(), None,
                                 2, 16, 4, 2, 34, None)
    assert rc == 1 and "zt_attn_decode" in zt.lib.last_error()
    torch.cuda.synchronize()
    assert bool(torch.all(out == 5.0))
    L.zt_attn_set_verbose(1)
