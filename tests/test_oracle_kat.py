"""The reference's known-answer tests for attention.forward, run on the oracle.

Each test restates one `test` block of src/attention_test.zig (line ranges in
the docstrings) with the same inputs and the same expectation, so the CPU
restatement in oracle/zt_oracle.c is pinned by the reference's own vectors.
"""
import math

import numpy as np
import pytest


def filled(rows, cols, vals):
    a = np.array(vals, dtype=np.float32)
    assert a.size == rows * cols
    return a.reshape(rows, cols)


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_one_head_one_token_returns_v_exactly(oracle):
    """src/attention_test.zig:15-28"""
    q, k, v = filled(1, 2, [1, 2]), filled(1, 2, [3, 4]), filled(1, 2, [5, 6])
    out = oracle.attention_forward(q, k, v, 1, 1, 2)
    assert np.array_equal(bits(out), bits(v))


def test_two_tokens_one_head_hand_computed(oracle):
    """src/attention_test.zig:30-44"""
    q = filled(2, 2, [1, 0, 0, 0])
    k = filled(2, 2, [1, 0, 0, 0])
    v = filled(2, 2, [1, 0, 3, 4])
    out = oracle.attention_forward(q, k, v, 1, 1, 2)
    assert np.array_equal(out.ravel(), np.array([1, 0, 2, 2], dtype=np.float32))


def test_ignores_keys_and_values_after_the_query(oracle):
    """src/attention_test.zig:46-72"""
    q = filled(3, 4, [1, 0, 0, 1, 1, 1, 1, 0, 0, 1, 1, -1])
    k = filled(3, 2, [1, 0, 0, 1, 1, 1])
    v = filled(3, 2, [1, 2, 3, 4, 5, 6])
    before = oracle.attention_forward(q, k, v, 2, 1, 2)
    k[1] = [99, 98]
    v[1] = [97, 96]
    after = oracle.attention_forward(q, k, v, 2, 1, 2)
    assert np.array_equal(bits(before[0]), bits(after[0]))
    assert after[1, 0] != before[1, 0]


def test_groups_query_heads_onto_their_kv_head(oracle):
    """src/attention_test.zig:74-95"""
    q = filled(2, 8, [1, 0, 1, 0, 0, 1, 0, 1, 0, 1, 0, 1, 1, 0, 1, 0])
    k = filled(2, 4, [1, 0, 2, 0, 0, 1, 0, 2])
    v = filled(2, 4, [1, 2, 3, 4, 5, 6, 7, 8])
    out = oracle.attention_forward(q, k, v, 4, 2, 2)
    assert np.array_equal(out[0, 0:2], np.array([1, 2], dtype=np.float32))
    assert np.array_equal(out[0, 4:6], np.array([3, 4], dtype=np.float32))
    for t in range(2):
        assert np.array_equal(out[t, 0:2], out[t, 2:4])
        assert out[t, 0] != out[t, 4]


def test_softmax_weights_sum_to_one(oracle):
    """src/attention_test.zig:97-111"""
    q = filled(4, 2, [1, 0, 0, 1, 1, 1, 0, -1])
    k = filled(4, 2, [1, 1, 0, 1, -1, 0, 2, 1])
    v = filled(4, 2, [1] * 8)
    out = oracle.attention_forward(q, k, v, 1, 1, 2)
    assert np.all(np.abs(out - 1.0) <= 1e-5)


def test_averages_exactly_the_causal_prefix(oracle):
    """src/attention_test.zig:113-128"""
    q = filled(4, 2, [1, 0, 1, 0, 1, 0, 1, 0])
    k = filled(4, 2, [0] * 8)
    v = filled(4, 2, [1, 2, 3, 4, 5, 6, 7, 8])
    out = oracle.attention_forward(q, k, v, 1, 1, 2)
    want = np.array([1, 2, 2, 3, 3, 4, 4, 5], dtype=np.float32)
    assert np.all(np.abs(out.ravel() - want) <= 1e-6)


def test_scales_scores_by_inverse_sqrt_head_dim(oracle):
    """src/attention_test.zig:130-147"""
    q = filled(2, 4, [1, 0, 0, 0, 0, 1, 0, 0])
    k = filled(2, 4, [2, 0, 0, 0, 0, 4, 0, 0])
    v = filled(2, 4, [1, 0, 0, 0, 0, 1, 0, 0])
    out = oracle.attention_forward(q, k, v, 1, 1, 4)
    want = np.array([1, 0, 0, 0, 0.11920292202211755, 0.88079707797788245, 0, 0])
    assert np.all(np.abs(out.ravel().astype(np.float64) - want) <= 1e-6)


def test_survives_scores_that_would_overflow_exp(oracle):
    """src/attention_test.zig:149-164"""
    q = filled(2, 2, [100, 0, 100, 0])
    k = filled(2, 2, [100, 0, 0, 0])
    v = filled(2, 2, [3, 5, 7, 9])
    out = oracle.attention_forward(q, k, v, 1, 1, 2)
    assert np.array_equal(out.ravel(), np.array([3, 5, 3, 5], dtype=np.float32))


def test_rejects_head_config_with_no_valid_group_split(oracle):
    """src/attention_test.zig:166-179"""
    q, k, v = filled(1, 2, [1, 2]), filled(1, 2, [3, 4]), filled(1, 2, [5, 6])
    for heads, kv, dim in ((1, 0, 2), (1, 1, 0), (3, 2, 2)):
        with pytest.raises(oracle.InvalidHeadConfig):
            oracle.attention_forward(q, k, v, heads, kv, dim)


def test_rejects_k_and_v_with_different_shapes(oracle):
    """src/attention_test.zig:181-195"""
    q = filled(2, 2, [1, 0, 0, 1])
    wide = filled(2, 2, [1, 0, 0, 1])
    wide_v = filled(2, 4, [1, 2, 3, 4, 5, 6, 7, 8])
    one = filled(1, 2, [1, 0])
    for kk, vv in ((wide, wide_v), (one, wide), (one, one)):
        with pytest.raises(oracle.DimensionMismatch):
            oracle.attention_forward(q, kk, vv, 1, 1, 2)


def test_rejects_a_kv_width_the_config_disagrees_with(oracle):
    """src/attention_test.zig:197-212"""
    q, kv, v = filled(1, 2, [1, 0]), filled(1, 2, [3, 4]), filled(1, 2, [5, 6])
    fat_q, fat_kv = filled(1, 3, [1, 2, 3]), filled(1, 3, [3, 4, 5])
    with pytest.raises(oracle.DimensionMismatch):
        oracle.attention_forward(fat_q, kv, v, 2, 1, 2)
    with pytest.raises(oracle.DimensionMismatch):
        oracle.attention_forward(q, fat_kv, v, 1, 1, 2)


def test_zero_tokens_returns_an_empty_output(oracle):
    """src/attention_test.zig:214-228"""
    e = np.zeros((0, 2), dtype=np.float32)
    out = oracle.attention_forward(e, e, e, 1, 1, 2)
    assert out.shape == (0, 2) and out.size == 0


def test_keeps_an_f64_accumulator_over_512_tokens(oracle):
    """src/attention_test.zig:230-295: 1/3 and 1/7 fill, T=512, D=8, rel 1e-6."""
    T, D = 512, 8
    tj = np.add.outer(np.arange(T), np.arange(D))
    x = np.where(tj % 2 == 0, np.float32(1.0) / np.float32(3.0),
                 np.float32(1.0) / np.float32(7.0)).astype(np.float32)
    out = oracle.attention_forward(x, x, x, 1, 1, D).astype(np.float64)
    xd = x.astype(np.float64)
    scale = 1.0 / math.sqrt(D)
    for t in range(T):
        s = (xd[: t + 1] @ xd[t]) * scale
        p = np.exp(s - s.max())
        # the reference sums ascending in s; np.cumsum keeps that order
        denom = np.cumsum(p)[-1]
        p = p / denom
        acc = np.zeros(D)
        for si in range(t + 1):
            acc += p[si] * xd[si]
        assert np.all(np.abs(acc - out[t]) <= 1e-6 * np.abs(acc))


def test_is_bit_reproducible_run_to_run(oracle):
    """src/attention_test.zig:297-318"""
    q = filled(3, 16, [round(0.1 * i, 1) for i in range(1, 49)])
    k = filled(3, 8, [0.5, 0.25, 0.125, 0.0625] * 2 + [1, 0.5, 0.25, 0.125] * 2 + [2, 1, 0.5, 0.25] * 2)
    v = filled(3, 8, list(range(1, 25)))
    a = oracle.attention_forward(q, k, v, 4, 2, 4)
    b = oracle.attention_forward(q, k, v, 4, 2, 4)
    c = oracle.attention_forward(q, k, v, 4, 2, 4, threads=4)
    assert np.array_equal(bits(a), bits(b))
    assert np.array_equal(bits(a), bits(c))
