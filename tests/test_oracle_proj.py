"""The oracle's projection (tensor.matmul, inputGrad, weightGrad) against the reference's own literals.

src/tensor_test.zig:97-156 hold hand-computed products; :185-273 pins that the reduction is carried in f32, not
f64, by a divergence bracket ((k - 1) eps64 < worst < (k - 1) eps32 relative to sum |terms|).  The gradients have
no literals in the reference (they are pinned by whole-model finite differences); they are checked against the
products they are by definition.
"""
import numpy as np
import pytest


def test_matmul_1x1(oracle):
    """src/tensor_test.zig:97-111"""
    assert oracle.matmul([[3.0]], [[4.0]]).tolist() == [[12.0]]


def test_matmul_2x3_by_3x2(oracle):
    """src/tensor_test.zig:113-135"""
    got = oracle.matmul([[1, 2, 3], [4, 5, 6]], [[7, 8], [9, 10], [11, 12]])
    assert got.tolist() == [[58.0, 64.0], [139.0, 154.0]]


def test_matmul_3x2_by_2x2_writes_every_element(oracle):
    """src/tensor_test.zig:137-156"""
    got = oracle.matmul([[1, 2], [3, 4], [5, 6]], [[2, 0], [0, 3]])
    assert got.ravel().tolist() == [2.0, 6.0, 6.0, 12.0, 10.0, 18.0]


def test_matmul_zero_sized_and_mismatch(oracle):
    """src/tensor_test.zig:158-183,275-: a zero-deep contraction gives zeros; a mismatch is refused."""
    got = oracle.matmul(np.zeros((2, 0), np.float32), np.zeros((0, 3), np.float32))
    assert got.shape == (2, 3) and not got.any()
    with pytest.raises(oracle.DimensionMismatch):
        oracle.matmul(np.zeros((2, 3), np.float32), np.zeros((2, 3), np.float32))


def test_matmul_reduces_in_f32_not_f64(oracle):
    """src/tensor_test.zig:185-273: m 256, k 512, n 128, entries (u - 0.5) * 0.04; the worst divergence from the
    exactly rounded f64 sum, relative to sum |terms|, lies above what an f64 reduction could leave and below what
    an f32 one may."""
    m, k, n = 256, 512, 128
    rng = np.random.default_rng(7)
    a = ((rng.random((m, k), dtype=np.float32) - 0.5) * 0.04).astype(np.float32)
    b = ((rng.random((k, n), dtype=np.float32) - 0.5) * 0.04).astype(np.float32)
    got = oracle.matmul(a, b, threads=4).astype(np.float64)
    exact = a.astype(np.float64) @ b.astype(np.float64)
    abs_sum = np.abs(a.astype(np.float64)) @ np.abs(b.astype(np.float64))
    worst = float((np.abs(got - exact.astype(np.float32).astype(np.float64)) / abs_sum).max())
    assert (k - 1) * np.finfo(np.float64).eps < worst < (k - 1) * np.finfo(np.float32).eps


def test_gradients_are_the_products_they_are_defined_as(oracle):
    """inputGrad: dctx = dy . w^T added to out; weightGrad: dw += ctx^T . dy (src/autograd.zig:553-557)."""
    rng = np.random.default_rng(1)
    ctx = rng.standard_normal((40, 24)).astype(np.float32)
    w = rng.standard_normal((24, 16)).astype(np.float32)
    dy = rng.standard_normal((40, 16)).astype(np.float32)
    dctx = oracle.input_grad(dy, w)
    assert np.allclose(dctx, dy.astype(np.float64) @ w.astype(np.float64).T, rtol=1e-5, atol=1e-5)
    twice = oracle.input_grad(dy, w, out=dctx.copy())
    assert np.allclose(twice, 2 * dctx, rtol=1e-6)
    dw = np.full((24, 16), 0.5, dtype=np.float32)
    oracle.weight_grad(dw, ctx, dy)
    assert np.allclose(dw, 0.5 + ctx.astype(np.float64).T @ dy.astype(np.float64), rtol=1e-5, atol=1e-5)
