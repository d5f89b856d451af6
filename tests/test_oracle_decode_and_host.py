"""Oracle pins for decode.attnStep, kv_cache.Layer and device.zig's host arithmetic."""
import numpy as np
import pytest

TINY = dict(n_heads=4, n_kv_heads=2, head_dim=32, n_ctx=32)  # src/decode_test.zig:12-20


def hashed(oracle, n, base=0):
    return np.array([oracle.fill_hash(base + i) for i in range(n)], dtype=np.float32)


def test_attn_step_refuses_instead_of_answering_zeros(oracle):
    """src/decode_test.zig:160-220"""
    H, Hkv, D = TINY["n_heads"], TINY["n_kv_heads"], TINY["head_dim"]
    q = hashed(oracle, H * D).reshape(1, -1)
    layer = oracle.Layer(TINY["n_ctx"], Hkv * D)
    with pytest.raises(oracle.DimensionMismatch):       # empty prefix
        oracle.attn_step(q, layer, H, Hkv, D)
    with pytest.raises(oracle.InvalidHeadConfig):
        oracle.attn_step(q, layer, H, 0, D)
    with pytest.raises(oracle.InvalidHeadConfig):
        oracle.attn_step(q, layer, 3, Hkv, D)
    with pytest.raises(oracle.DimensionMismatch):
        oracle.attn_step(q[:, :-1], layer, H, Hkv, D)
    layer.append(q[0, :Hkv * D], q[0, Hkv * D:2 * Hkv * D])
    out = oracle.attn_step(q, layer, H, Hkv, D)
    assert out.shape == (1, H * D)
    assert np.all(np.isfinite(out)) and np.any(out != 0)


def test_attn_step_equals_the_forward_row_at_every_position(oracle):
    """decode semantics q_offset = pos, n_keys = pos + 1 (src/decode_test.zig:222-319
    checks the CUDA arm the same way, at every position of a filling cache)."""
    H, Hkv, D, n_ctx = 4, 2, 32, 24
    q = hashed(oracle, n_ctx * H * D, 1000).reshape(n_ctx, -1)
    k = hashed(oracle, n_ctx * Hkv * D, 50000).reshape(n_ctx, -1)
    v = hashed(oracle, n_ctx * Hkv * D, 90000).reshape(n_ctx, -1)
    full, full_lse = oracle.attention_forward(q, k, v, H, Hkv, D, want_lse=True)
    layer = oracle.Layer(n_ctx, Hkv * D)
    for pos in range(n_ctx):
        layer.append(k[pos], v[pos])       # append before attend, src/decode.zig:259
        out, lse = oracle.attn_step(q[pos:pos + 1], layer, H, Hkv, D, want_lse=True)
        assert np.array_equal(out[0].view(np.uint32), full[pos].view(np.uint32))
        assert np.array_equal(lse[0], full_lse[pos])
        at = oracle.attention_forward_at(q[pos:pos + 1], layer.k, layer.v, H, Hkv, D, pos, pos + 1)
        assert np.array_equal(at[0].view(np.uint32), full[pos].view(np.uint32))
    with pytest.raises(oracle.Full):
        layer.append(k[0], v[0])


def test_forward_at_training_shape_is_the_forward(oracle):
    T, H, Hkv, D = 19, 4, 2, 8
    q = oracle.fill_normal((T, H * D), 7, 0)
    k = oracle.fill_normal((T, Hkv * D), 7, 1)
    v = oracle.fill_normal((T, Hkv * D), 7, 2)
    a = oracle.attention_forward(q, k, v, H, Hkv, D)
    b = oracle.attention_forward_at(q, k, v, H, Hkv, D, 0, T, threads=3)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    h, t0, t1 = 3, 5, 12
    rows, _ = oracle.attention_forward_rows(q, k, v, H, Hkv, D, h, t0, t1)
    assert np.array_equal(rows, a[t0:t1, h * D:(h + 1) * D])


def test_layer_sizes_and_refusals(oracle):
    """src/kv_cache.zig:233-290 (sizes, Full, wrong width leaves the cache untouched)."""
    layers = [oracle.Layer(256, 2 * 32) for _ in range(4)]
    assert sum(l.bytes() for l in layers) == 524288
    l = oracle.Layer(3, 8)
    with pytest.raises(oracle.DimensionMismatch):
        l.append(np.zeros(8), np.zeros(4))
    with pytest.raises(oracle.DimensionMismatch):
        l.append(np.zeros(4), np.zeros(8))
    assert l.visible() == 0
    for i in range(3):
        l.append(np.full(8, i), np.full(8, -i))
    assert l.visible() == 3
    with pytest.raises(oracle.Full):
        l.append(np.zeros(8), np.zeros(8))
    assert l.visible() == 3 and l.k[2, 0] == 2 and l.v[2, 0] == -2
    with pytest.raises(oracle.DimensionMismatch):
        oracle.Layer(0, 8)
    assert oracle.Layer(16, 5).bytes() * 3 == 3 * 16 * 5 * 2 * 4


def test_bytes_for_matches_device_zig(oracle):
    """src/cuda/device.zig:502-606"""
    Q, KV, PR = oracle.KIND_QUERY_HEADED, oracle.KIND_KV_HEADED, oracle.KIND_PER_ROW
    assert oracle.bytes_for(Q, 256, 4, 2, 32) == 256 * 4 * 32 * 4
    assert oracle.bytes_for(KV, 256, 4, 2, 32) == 256 * 2 * 32 * 4
    assert oracle.bytes_for(PR, 256, 4, 2, 32) == 256 * 4 * 4
    assert 2 * 4 * oracle.bytes_for(KV, 256, 4, 2, 32) == 524288
    total = 4 * oracle.bytes_for(Q, 256, 4, 2, 32) + 4 * oracle.bytes_for(KV, 256, 4, 2, 32) \
        + 3 * oracle.bytes_for(PR, 256, 4, 2, 32)
    assert total == 798720
    for args in ((Q, 0, 4, 2, 32), (Q, 256, 0, 2, 32), (Q, 256, 4, 2, 0), (PR, 256, 4, 0, 32)):
        with pytest.raises(oracle.DegenerateShape):
            oracle.bytes_for(*args)
    for args in ((Q, 2 ** 64 - 1, 4, 2, 32), (Q, 1 << 40, 1 << 40, 1, 1), (KV, 2 ** 64 - 1, 4, 2, 32)):
        with pytest.raises(oracle.ShapeTooLarge):
            oracle.bytes_for(*args)


def test_forward_bounds_accept_refuse_table(oracle):
    """src/cuda/device.zig:612-645"""
    c_t, imax = 256, 2 ** 31 - 1
    oracle.forward_bounds(c_t, 0, c_t, c_t)
    oracle.forward_bounds(c_t, 5, 6, 1)
    oracle.forward_bounds(c_t, c_t - 1, c_t, 1)
    for args in ((c_t, 0, c_t + 1, 1), (c_t, 0, 0, 1), (c_t, 0, 1, c_t + 1), (c_t, 0, 1, 0),
                 (c_t, c_t, c_t, 1), (c_t, -1, c_t, 1), (c_t, imax, 1, 1), (c_t, imax - 1, 1, 2),
                 (c_t, c_t + 1, c_t, 1)):
        with pytest.raises(oracle.ShapeTooLarge):
            oracle.forward_bounds(*args)


def test_lcg_fill_is_the_twin_generator(oracle):
    """src/cuda/attn_twin.zig:283-289, first values worked by hand from the recurrence."""
    x = 0xBEEF
    want = []
    for _ in range(5):
        x = (x * 1664525 + 1013904223) & 0xFFFFFFFF
        want.append(np.float32(np.float32(x >> 8) / np.float32(16777216.0)) - np.float32(0.5))
    got = oracle.fill_lcg(5, 0xBEEF)
    assert np.array_equal(got, np.array(want, dtype=np.float32))
    assert np.all(got >= -0.5) and np.all(got < 0.5)


def test_normal_fill_is_sliceable_and_standard(oracle):
    a = oracle.fill_normal((100001,), 0, 1)
    b = oracle.fill_normal((1000,), 0, 1, first=4097)
    assert np.array_equal(a[4097:5097], b)
    assert abs(float(a.mean())) < 0.02 and abs(float(a.std()) - 1.0) < 0.02
    assert not np.array_equal(a[:100], oracle.fill_normal((100,), 0, 2))
