"""The holder's pure host arithmetic, as src/cuda/device.zig:502-645 tests it (no GPU needed)."""
import pytest


def test_shipped_shape_sizes(zt):
    """device.zig:502-507"""
    K = zt.Kind
    assert zt.bytes_for(K.query_headed, 256, 4, 2, 32) == 256 * 4 * 32 * 4
    assert zt.bytes_for(K.kv_headed, 256, 4, 2, 32) == 256 * 2 * 32 * 4
    assert zt.bytes_for(K.per_row, 256, 4, 2, 32) == 256 * 4 * 4


def test_dk_dv_equal_the_kv_cache_term(zt):
    """device.zig:509-530"""
    assert 2 * 4 * zt.bytes_for(zt.Kind.kv_headed, 256, 4, 2, 32) == 524288


def test_eleven_buffers_total_798720(zt):
    """device.zig:532-580"""
    assert zt.device.total_bytes(256, 4, 2, 32) == 798720
    assert zt.device.total_bytes(256, 4, 2, 32) < 1024 * 1024


def test_degenerate_shape_is_refused_by_name(zt):
    """device.zig:582-590"""
    K, E = zt.Kind, zt.device.DegenerateShape
    for args in ((K.query_headed, 0, 4, 2, 32), (K.query_headed, 256, 0, 2, 32),
                 (K.query_headed, 256, 4, 2, 0), (K.per_row, 256, 4, 0, 32)):
        with pytest.raises(E):
            zt.bytes_for(*args)


def test_overflow_is_refused_not_truncated(zt):
    """device.zig:592-598"""
    K, E = zt.Kind, zt.device.ShapeTooLarge
    for args in ((K.query_headed, 2 ** 64 - 1, 4, 2, 32), (K.query_headed, 1 << 40, 1 << 40, 1, 1),
                 (K.kv_headed, 2 ** 64 - 1, 4, 2, 32)):
        with pytest.raises(E):
            zt.bytes_for(*args)


def test_to_c_int(zt):
    """device.zig:600-606"""
    with pytest.raises(zt.device.ShapeTooLarge):
        zt.to_c_int(1 << 31)
    assert zt.to_c_int(256) == 256
    assert zt.to_c_int(2 ** 31 - 1) == 2 ** 31 - 1


def test_forward_bounds_table(zt, oracle):
    """device.zig:612-645, and the mirror agrees with the oracle's restatement on a grid."""
    c_t, imax, E = 256, 2 ** 31 - 1, zt.device.ShapeTooLarge
    zt.forward_bounds(c_t, 0, c_t, c_t)
    zt.forward_bounds(c_t, 5, 6, 1)
    zt.forward_bounds(c_t, c_t - 1, c_t, 1)
    for args in ((c_t, 0, c_t + 1, 1), (c_t, 0, 0, 1), (c_t, 0, 1, c_t + 1), (c_t, 0, 1, 0),
                 (c_t, c_t, c_t, 1), (c_t, -1, c_t, 1), (c_t, imax, 1, 1), (c_t, imax - 1, 1, 2),
                 (c_t, c_t + 1, c_t, 1)):
        with pytest.raises(E):
            zt.forward_bounds(*args)
    for q_off in (-1, 0, 3, 7, 8):
        for n_keys in (0, 1, 4, 8, 9):
            for t in (0, 1, 2, 8, 9):
                try:
                    zt.forward_bounds(8, q_off, n_keys, t)
                    mine = True
                except E:
                    mine = False
                try:
                    oracle.forward_bounds(8, q_off, n_keys, t)
                    theirs = True
                except oracle.ShapeTooLarge:
                    theirs = False
                assert mine == theirs, (q_off, n_keys, t)


def test_attn_init_refuses_before_allocating(zt):
    """device.zig:227-241: head_dim 33, 5 heads over 2, 65536 heads are refused up front."""
    R = zt.device.ConfigRefused
    for args in ((8, 4, 2, 33), (8, 5, 2, 32), (1, 65536, 32768, 32)):
        with pytest.raises(R):
            zt.Attn(*args, device="cpu")
    with pytest.raises(zt.device.ShapeTooLarge):
        zt.Attn(1 << 31, 4, 2, 32, device="cpu")
