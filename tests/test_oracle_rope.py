"""The oracle's RoPE against the known-answer tests of src/rope_test.zig (values cited, not copied as code)."""
import numpy as np
import pytest


def f32(*v):
    return np.array(v, dtype=np.float32)


def test_position_zero_is_the_identity_bit_for_bit(oracle):
    x = f32(1, -2, 0.5, -0.25, 3, -4, 0.125, 7).reshape(1, 8)           # rope_test.zig:48-64
    y = oracle.rope_forward(x, 0, 8)
    assert y.tobytes() == x.tobytes()


def test_one_pair_one_radian(oracle):
    y = oracle.rope_forward(f32(3, 4).reshape(1, 2), 1, 2)               # rope_test.zig:66-79
    np.testing.assert_allclose(y[0], [-1.7449770216271669, 4.6856221778962484], atol=1e-6, rtol=0)


def test_both_halves_of_the_split_turn(oracle):
    y = oracle.rope_forward(f32(1, 2, 3, 4).reshape(1, 4), 1, 4)         # rope_test.zig:81-100
    np.testing.assert_allclose(y[0], [-1.9841106485555498, 1.9943411476361261, 2.4623779024123157,
                                      4.0028244261821879], atol=1e-6, rtol=0)


def test_half_split_layout_not_interleaved(oracle):
    y = oracle.rope_forward(f32(1, 0, 0, 0).reshape(1, 4), 1, 4)         # rope_test.zig:102-118
    np.testing.assert_allclose(y[0], [0.5403023058681397, 0, 0.8414709848078965, 0], atol=1e-6, rtol=0)


def test_each_head_block_rotates_on_its_own(oracle):
    y = oracle.rope_forward(f32(1, 2, 3, 4, 5, 6, 7, 8).reshape(1, 8), 1, 4)   # rope_test.zig:120-157
    want = [-1.9841106485555497, 1.9943411476364587, 2.4623779024123159, 4.0028244261826036,
            -3.1887853643145765, 5.9886802952732506, 7.9894710651164611, 8.0084772785471445]
    np.testing.assert_allclose(y[0], want, atol=1e-6, rtol=0)


def test_rotation_preserves_the_norm(oracle):
    x = f32(1, -2, 3, -4, 5, -6).reshape(1, 6)                            # rope_test.zig:159-172
    y = oracle.rope_forward(x, 3, 6)
    assert abs(np.linalg.norm(x.astype(np.float64)) - 9.5393920142) < 1e-5
    assert abs(np.linalg.norm(y.astype(np.float64)) - 9.5393920142) < 1e-5


def test_refusals(oracle):
    x = f32(1, 2, 3).reshape(1, 3)                                        # rope_test.zig:174-192
    with pytest.raises(oracle.OddHeadDim):
        oracle.rope_forward(x, 0, 3)
    with pytest.raises(oracle.OddHeadDim):
        oracle.rope_forward(x, 0, 0)
    with pytest.raises(oracle.DimensionMismatch):
        oracle.rope_forward(f32(1, 2, 3, 4, 5, 6).reshape(1, 6), 0, 4)


def test_row_r_sits_at_pos_plus_r(oracle):
    x = f32(1, 2, 3, 4, 0.5, -0.5, 1, -1, 1, -1, 0, 0).reshape(3, 4)     # rope_test.zig:194-229
    y = oracle.rope_forward(x, 2, 4)
    want = [[-3.1440391170241875, 1.9886783065859592, -0.3391430828157455, 4.0056408467070337],
            [-0.6361162563600899, -0.4957528720475413, -0.9194324925705119, -1.0021123139931044],
            [-0.6536436208636119, -0.9999840000426667, -0.7568024953079283, -0.0056568240796513]]
    np.testing.assert_allclose(y, want, atol=1e-6, rtol=0)


def test_backward_is_the_transpose(oracle):
    """ropeBackward (autograd.zig:851-874) is R^T: <R x, g> == <x, R^T g> to f32 rounding, and R^T R x == x."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((7, 3 * 16)).astype(np.float32)
    g = rng.standard_normal((7, 3 * 16)).astype(np.float32)
    y = oracle.rope_forward(x, 11, 16)
    gt = oracle.rope_backward(g, 11, 16)
    assert abs(np.vdot(y.astype(np.float64), g) - np.vdot(x.astype(np.float64), gt)) < 1e-4
    np.testing.assert_allclose(oracle.rope_backward(y, 11, 16), x, atol=2e-6, rtol=0)
