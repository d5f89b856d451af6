"""Which of the three terms of the f16 hi/lo split the parity bar needs, product by product.

The tensor-core kernels issue every product a.b as ah.bh + ah.bl + al.bh on f16 pieces of power-of-two-scaled
operands; a term is a third of a product's tensor time, so a term the tolerance could spare would be worth
dropping.  This emulates the arithmetic of one KV group in numpy (float64 sums of exactly representable f16
products, so what differs from the float64 reference is the split alone) on the benchmark's kind of data, N(0,1),
and counts the elements of dq, dk, dv (and of P) that leave the bar |got - ref| <= 1e-5 + 1e-4 |ref| when one
term of one product is left out.  No GPU, no library: arithmetic only.
"""
import numpy as np
import pytest

T, H, D = 512, 4, 128
ATOL, RTOL = 1e-5, 1e-4


def _mult(x):
    return 2.0 ** (14 - np.floor(np.log2(np.abs(x).max())))


def _split(x):
    h = x.astype(np.float16)
    low = (x - h.astype(np.float64)).astype(np.float16)
    return h.astype(np.float64), low.astype(np.float64)


def _prod(a, b, drop=None):
    """a [M, K] . b [N, K]^T with the split's terms; drop: None, "hl" (a hi . b lo) or "lh" (a lo . b hi)."""
    ah, al = _split(a)
    bh, bl = _split(b)
    out = ah @ bh.T
    if drop != "hl":
        out = out + ah @ bl.T
    if drop != "lh":
        out = out + al @ bh.T
    return out


def _backward(q, k, v, do, drop_in=None, drop=None):
    """dq [T, H D], dk, dv [T, D] of one KV group with H query heads; `drop` applied to the product named drop_in."""
    scale = 1.0 / np.sqrt(D)
    mask = np.tril(np.ones((T, T), bool))
    mq, mk, mv, mdo = _mult(q), _mult(k), _mult(v), _mult(do)
    dq, dk, dv = np.zeros((T, H * D)), np.zeros((T, D)), np.zeros((T, D))
    p_bad = 0
    sel = lambda name: drop if drop_in == name else None  # noqa: E731
    for h in range(H):
        qh, doh = q[:, h * D:(h + 1) * D], do[:, h * D:(h + 1) * D]
        s_true = qh @ k.T * scale
        s_true[~mask] = -np.inf
        lse = np.log(np.exp(s_true - s_true.max(1, keepdims=True)).sum(1)) + s_true.max(1)
        p_true = np.exp(s_true - lse[:, None])
        delta = (p_true * (doh @ v.T)).sum(1)
        s = _prod(qh * mq, k * mk, sel("S")) / (mq * mk) * scale
        p = np.exp(s - lse[:, None])
        p[~mask] = 0.0
        p_bad += int((~(np.abs(p - p_true) <= ATOL + RTOL * p_true)).sum())
        dp = _prod(doh * mdo, v * mv, sel("dP")) / (mdo * mv)
        ds = p * (dp - delta[:, None])
        # dS leaves scaled per query row (a power of two that puts the row's bound under 2^14), as in the kernels
        rnorm = np.sqrt((doh * doh).sum(1))
        vnmax = np.sqrt((v * v).sum(1)).max()
        cq = 2.0 ** (13 - np.floor(np.log2(np.maximum(2.02 * rnorm * vnmax, 1e-300))))[:, None]
        dq[:, h * D:(h + 1) * D] = _prod(ds * cq, (k * mk).T, sel("dQ")) * scale / (cq * mk)
        rel = cq.min() / cq                                    # the row factor moved onto Q for dK
        dk += _prod((ds * cq).T, (qh * mq * rel).T, sel("dK")) * scale / (cq.min() * mq)
        dv += _prod((p * 1024.0).T, (doh * mdo).T, sel("dV")) / (1024.0 * mdo)
    return dq, dk, dv, p_bad


def _reference(q, k, v, do):
    scale = 1.0 / np.sqrt(D)
    mask = np.tril(np.ones((T, T), bool))
    dq, dk, dv = np.zeros((T, H * D)), np.zeros((T, D)), np.zeros((T, D))
    for h in range(H):
        qh, doh = q[:, h * D:(h + 1) * D], do[:, h * D:(h + 1) * D]
        s = qh @ k.T * scale
        s[~mask] = -np.inf
        p = np.exp(s - s.max(1, keepdims=True))
        p /= p.sum(1, keepdims=True)
        dp = doh @ v.T
        ds = p * (dp - (p * dp).sum(1, keepdims=True))
        dq[:, h * D:(h + 1) * D] = ds @ k * scale
        dk += ds.T @ qh * scale
        dv += p.T @ doh
    return dq, dk, dv


def _violations(got, ref):
    return int((~(np.abs(got - ref) <= ATOL + RTOL * np.abs(ref))).sum())


@pytest.fixture(scope="module")
def data():
    rng = np.random.default_rng(3)
    q, do = (rng.standard_normal((T, H * D)).astype(np.float32).astype(np.float64) for _ in range(2))
    k, v = (rng.standard_normal((T, D)).astype(np.float32).astype(np.float64) for _ in range(2))
    return q, k, v, do, _reference(q, k, v, do)


def test_three_terms_meet_the_bar(data):
    q, k, v, do, ref = data
    dq, dk, dv, p_bad = _backward(q, k, v, do)
    assert p_bad == 0
    assert [_violations(g, r) for g, r in zip((dq, dk, dv), ref)] == [0, 0, 0]


@pytest.mark.parametrize("drop", ["hl", "lh"], ids=["without-hi.lo", "without-lo.hi"])
@pytest.mark.parametrize("product", ["S", "dP", "dV", "dK", "dQ"])
def test_no_product_can_spare_a_term(data, product, drop):
    """Every two-term variant of every product leaves the bar: an 11-bit piece is wrong by up to 2^-12 of its value,
    and a sum of T such terms with random signs keeps that relative error (about 1.4e-4 rms against a bar of 1e-4).
    The counts (of 262144 dq, 65536 dk, 65536 dv elements; P: of the 525312 causal entries of four heads) are what
    section "Where the step stands" of the design notes quotes."""
    q, k, v, do, ref = data
    dq, dk, dv, p_bad = _backward(q, k, v, do, product, drop)
    bad = {"P": p_bad, "dq": _violations(dq, ref[0]), "dk": _violations(dk, ref[1]), "dv": _violations(dv, ref[2])}
    print(product, drop, bad)
    hit = {"S": ("dq", "dk", "dv"), "dP": ("dq", "dk"), "dV": ("dv",), "dK": ("dk",), "dQ": ("dq",)}[product]
    sizes = {"dq": dq.size, "dk": dk.size, "dv": dv.size}
    for name in hit:
        assert bad[name] > sizes[name] // 100, (product, drop, bad)   # more than 1 % of the elements miss the bar
