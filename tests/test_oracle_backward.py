"""Pins for the oracle's attentionBackward (src/autograd.zig:636-842).

The reference holds no literal vectors for dq/dk/dv: its own tests pin the
backward by finite differences through the model (src/autograd_test.zig:834-859)
and by refusals (src/autograd_test.zig:879-999).  The same three kinds of check
are restated here for the C restatement: refusals, central differences against
the oracle's own forward, and an independent float64 autograd.
"""
import numpy as np
import pytest
import torch


def ramped(rows, cols, phase):
    """src/autograd_test.zig:869-877"""
    i = np.arange(rows * cols)
    return (np.float32(phase) * ((i % 7).astype(np.float32) - np.float32(3.0)) / np.float32(8.0)
            ).astype(np.float32).reshape(rows, cols)


def test_backward_refuses_what_the_reference_refuses(oracle):
    """src/autograd_test.zig:879-999"""
    T, wide = 4, 8
    q, k, v, dout = ramped(T, wide, 0.5), ramped(T, wide, 0.25), ramped(T, wide, -0.25), ramped(T, wide, 1.0)
    for heads, kv, dim in ((2, 0, 4), (2, 2, 0), (3, 2, 4)):
        with pytest.raises(oracle.InvalidHeadConfig):
            oracle.attention_backward(q, k, v, dout, heads, kv, dim)
    with pytest.raises(oracle.DimensionMismatch):
        oracle.attention_backward(q, ramped(T - 1, wide, 0.25), v, dout, 2, 2, 4)
    with pytest.raises(oracle.DimensionMismatch):
        oracle.attention_backward(q, k, v, ramped(T, wide - 1, 1.0), 2, 2, 4)
    with pytest.raises(oracle.DimensionMismatch):
        oracle.attention_backward(q, k, v, ramped(T, wide + 1, 1.0), 2, 2, 4)
    dq, dk, dv = oracle.attention_backward(q, k, v, dout, 2, 2, 4)
    assert not np.array_equal(dq, dk)


def sdpa_f64(q, k, v, H, Hkv, D):
    T = q.shape[0]
    g = H // Hkv
    qh = q.view(T, H, D).transpose(0, 1)
    kh = k.view(T, Hkv, D).transpose(0, 1).repeat_interleave(g, dim=0)
    vh = v.view(T, Hkv, D).transpose(0, 1).repeat_interleave(g, dim=0)
    s = qh @ kh.transpose(1, 2) / (D ** 0.5)
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    lse = torch.logsumexp(s, dim=-1)
    return (p @ vh).transpose(0, 1).reshape(T, H * D), lse.transpose(0, 1)


@pytest.mark.parametrize("T,H,Hkv,D,seed", [(17, 4, 2, 8, 1), (64, 8, 2, 32, 2), (33, 3, 3, 6, 3),
                                            (40, 6, 1, 16, 4)])
def test_backward_agrees_with_float64_autograd(oracle, T, H, Hkv, D, seed):
    q = oracle.fill_normal((T, H * D), seed, 0)
    k = oracle.fill_normal((T, Hkv * D), seed, 1)
    v = oracle.fill_normal((T, Hkv * D), seed, 2)
    do = oracle.fill_normal((T, H * D), seed, 3)
    out, lse = oracle.attention_forward(q, k, v, H, Hkv, D, want_lse=True)
    dq, dk, dv = oracle.attention_backward(q, k, v, do, H, Hkv, D)
    tq, tk, tv = (torch.tensor(x, dtype=torch.float64, requires_grad=True) for x in (q, k, v))
    o64, lse64 = sdpa_f64(tq, tk, tv, H, Hkv, D)
    o64.backward(torch.tensor(do, dtype=torch.float64))
    assert np.allclose(out, o64.detach().numpy(), rtol=2e-6, atol=1e-7)
    assert np.allclose(lse, lse64.detach().numpy(), rtol=2e-6, atol=1e-6)
    assert np.allclose(dq, tq.grad.numpy(), rtol=1e-5, atol=1e-6)
    # dk/dv carry the reference's per-term f32 roundings, hence the wider bound
    assert np.allclose(dk, tk.grad.numpy(), rtol=1e-4, atol=2e-6)
    assert np.allclose(dv, tv.grad.numpy(), rtol=1e-4, atol=2e-6)


def test_backward_matches_central_differences_of_the_forward(oracle):
    """The reference's own way of pinning it (src/autograd_test.zig:834-859), in f64."""
    T, H, Hkv, D = 6, 4, 2, 4
    rng = np.random.default_rng(0)
    q = rng.standard_normal((T, H * D)).astype(np.float32)
    k = rng.standard_normal((T, Hkv * D)).astype(np.float32)
    v = rng.standard_normal((T, Hkv * D)).astype(np.float32)
    do = rng.standard_normal((T, H * D)).astype(np.float32)
    dq, dk, dv = oracle.attention_backward(q, k, v, do, H, Hkv, D)

    def loss(qq, kk, vv):
        o, _ = sdpa_f64(torch.tensor(qq, dtype=torch.float64), torch.tensor(kk, dtype=torch.float64),
                        torch.tensor(vv, dtype=torch.float64), H, Hkv, D)
        return float((o * torch.tensor(do, dtype=torch.float64)).sum())

    eps = 1e-5
    for name, base, grad in (("q", q, dq), ("k", k, dk), ("v", v, dv)):
        b64 = base.astype(np.float64)
        for idx in [(0, 0), (T - 1, 1), (2, base.shape[1] - 1), (T // 2, 3)]:
            hi, lo = b64.copy(), b64.copy()
            hi[idx] += eps
            lo[idx] -= eps
            args_hi = {"q": (hi, k, v), "k": (q, hi, v), "v": (q, k, hi)}[name]
            args_lo = {"q": (lo, k, v), "k": (q, lo, v), "v": (q, k, lo)}[name]
            fd = (loss(*args_hi) - loss(*args_lo)) / (2 * eps)
            assert abs(fd - grad[idx]) <= 1e-5 + 1e-4 * abs(fd), (name, idx, fd, grad[idx])


def test_backward_is_causal(oracle):
    """A change of dout at the last row leaves dk/dv/dq of nothing but what that row reads
    (src/autograd_test.zig:526-598 checks the same property through the model)."""
    T, H, Hkv, D = 9, 2, 1, 4
    q = oracle.fill_normal((T, H * D), 5, 0)
    k = oracle.fill_normal((T, Hkv * D), 5, 1)
    v = oracle.fill_normal((T, Hkv * D), 5, 2)
    do = oracle.fill_normal((T, H * D), 5, 3)
    a = oracle.attention_backward(q, k, v, do, H, Hkv, D)
    do2 = do.copy()
    do2[0] += 1.0  # row 0 reads key 0 only
    b = oracle.attention_backward(q, k, v, do2, H, Hkv, D)
    assert np.array_equal(a[0][1:], b[0][1:])      # dq of later rows untouched
    assert np.array_equal(a[1][1:], b[1][1:])      # dk of later keys untouched
    assert np.array_equal(a[2][1:], b[2][1:])
    assert not np.array_equal(a[2][0], b[2][0])


def test_backward_threads_and_group_split_change_no_bit(oracle):
    T, H, Hkv, D = 48, 8, 4, 16
    q = oracle.fill_lcg(T * H * D, 0xBEEF).reshape(T, -1)
    k = oracle.fill_lcg(T * Hkv * D, 0x1234).reshape(T, -1)
    v = oracle.fill_lcg(T * Hkv * D, 0x5678).reshape(T, -1)
    do = oracle.fill_lcg(T * H * D, 0x9ABC).reshape(T, -1)
    one = oracle.attention_backward(q, k, v, do, H, Hkv, D, threads=1)
    many = oracle.attention_backward(q, k, v, do, H, Hkv, D, threads=4)
    for a, b in zip(one, many):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    g = H // Hkv
    for kv in range(Hkv):
        dq, dk, dv = oracle.attention_backward_kv_group(q, k, v, do, H, Hkv, D, kv)
        assert np.array_equal(dq[:, kv * g * D:(kv + 1) * g * D], one[0][:, kv * g * D:(kv + 1) * g * D])
        assert np.array_equal(dk[:, kv * D:(kv + 1) * D], one[1][:, kv * D:(kv + 1) * D])
        assert np.array_equal(dv[:, kv * D:(kv + 1) * D], one[2][:, kv * D:(kv + 1) * D])


def test_sampled_step_rows_are_the_full_pass_rows(oracle):
    """The benchmark's CPU sample computes a subset of rows with the full pass's arithmetic."""
    B, T, H, Hkv, D = 2, 21, 4, 2, 8
    q = oracle.fill_normal((B, T, H * D), 9, 0)
    k = oracle.fill_normal((B, T, Hkv * D), 9, 1)
    v = oracle.fill_normal((B, T, Hkv * D), 9, 2)
    do = oracle.fill_normal((B, T, H * D), 9, 3)
    flops, out, dq, dk, dv = oracle.sampled_step(q, k, v, do, H, Hkv, D, 4, 3, threads=3)
    rows = list(range(3, T, 4))
    assert flops == sum(14.0 * D * (t + 1) for t in rows) * B * H
    for b in range(B):
        fo = oracle.attention_forward(q[b], k[b], v[b], H, Hkv, D)
        fdq, _, _ = oracle.attention_backward(q[b], k[b], v[b], do[b], H, Hkv, D)
        assert np.array_equal(out[b][rows], fo[rows]) and np.array_equal(dq[b][rows], fdq[rows])
        others = [t for t in range(T) if t not in rows]
        assert not out[b][others].any()
    # with stride 1 it is the whole pass, dk/dv included
    flops1, out1, dq1, dk1, dv1 = oracle.sampled_step(q, k, v, do, H, Hkv, D, 1, 0, threads=2)
    for b in range(B):
        _, fdk, fdv = oracle.attention_backward(q[b], k[b], v[b], do[b], H, Hkv, D)
        assert np.array_equal(dk1[b], fdk) and np.array_equal(dv1[b], fdv)
    assert flops1 == 3.5 * 2 * B * H * D * T * (T + 1)
