"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle.

Tolerance everywhere (the stated bar for this path): |got - ref| <= 1e-5 + 1e-4 |ref|,
element-wise, NaN counted as a failure -- for out, log-sum-exp, dq, dk and dv.
"""
import ctypes
import importlib.util
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
RTOL, ATOL = 1e-4, 1e-5


def close(got, ref, what=""):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    err = np.abs(got - ref)
    bad = ~(err <= ATOL + RTOL * np.abs(ref))
    if bad.any():
        i = int(np.argmax(np.where(np.isnan(err), np.inf, err)))
        raise AssertionError(f"{what}: {int(bad.sum())}/{err.size} outside tolerance; worst at flat "
                             f"index {i}: got {got.ravel()[i]!r} want {ref.ravel()[i]!r}")


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


def cu(x, dev):
    return torch.from_numpy(np.ascontiguousarray(x)).to(dev)


def same_gradients(got, want, D):
    """dq, dk, dv of two runs on the same inputs.  Bit for bit, except dq at head_dim 32, 64, 96, 128 (the fused
    backward: every key tile's CTA adds its share of dq in memory, in no fixed order) and all three at 192 and 256
    (the unfused one): those agree to rounding."""
    for name, a, b in zip(("dq", "dk", "dv"), got, want):
        if D in (192, 256) or (D in (32, 64, 96, 128) and name == "dq"):
            assert bool(((a - b).abs() <= 2e-6 + 2e-5 * b.abs()).all()), name
        else:
            assert torch.equal(a, b), name


def lcg_inputs(oracle, T, H, Hkv, D):
    q = oracle.fill_lcg(T * H * D, 0xBEEF).reshape(T, H * D)
    k = oracle.fill_lcg(T * Hkv * D, 0x1234).reshape(T, Hkv * D)
    v = oracle.fill_lcg(T * Hkv * D, 0x5678).reshape(T, Hkv * D)
    do = oracle.fill_lcg(T * H * D, 0x9ABC).reshape(T, H * D)
    return q, k, v, do


def normal_inputs(oracle, T, H, Hkv, D, seed):
    return (oracle.fill_normal((T, H * D), seed, 0), oracle.fill_normal((T, Hkv * D), seed, 1),
            oracle.fill_normal((T, Hkv * D), seed, 2), oracle.fill_normal((T, H * D), seed, 3))


def run_fwd_bwd(zt, dev, q, k, v, do, H, Hkv, D):
    tq, tk, tv, tdo = (cu(x, dev) for x in (q, k, v, do))
    o, lse = zt.attention_forward(tq, tk, tv, H, Hkv, D, want_lse=True)
    dq, dk, dv = zt.attention_backward(tq, tk, tv, o, lse, tdo, H, Hkv, D)
    torch.cuda.synchronize()
    return [x.cpu().numpy() for x in (o, lse, dq, dk, dv)]


# ---- the reference's known-answer tests, through the C ABI ------------------------------------
# The C ABI admits head_dim >= 32 only (src/cuda/attn_kernels.cu:147-148), so the literals of
# src/attention_test.zig (head_dim 2) are embedded in the first columns of a 32-wide head with
# zeros behind them; every expectation used below does not depend on the 1/sqrt(D) scale.

def pad(a, H, d_small, D=32):
    a = np.asarray(a, dtype=np.float32).reshape(-1, H, d_small)
    out = np.zeros((a.shape[0], H, D), dtype=np.float32)
    out[:, :, :d_small] = a
    return out.reshape(a.shape[0], H * D)


def abi_forward(zt, dev, q, k, v, H, Hkv, D):
    holder = zt.Attn(q.shape[0], H, Hkv, D, device=dev)
    holder.upload(holder.q, q)
    holder.upload(holder.k, k)
    holder.upload(holder.v, v)
    holder.forward(1, 64)
    return holder.download(q.size, holder.out).reshape(q.shape)


def test_kat_one_token_returns_v_exactly(zt, dev):
    """src/attention_test.zig:15-28"""
    out = abi_forward(zt, dev, pad([1, 2], 1, 2), pad([3, 4], 1, 2), pad([5, 6], 1, 2), 1, 1, 32)
    assert np.array_equal(out, pad([5, 6], 1, 2))


def test_kat_two_tokens_hand_computed(zt, dev):
    """src/attention_test.zig:30-44"""
    out = abi_forward(zt, dev, pad([1, 0, 0, 0], 1, 2), pad([1, 0, 0, 0], 1, 2), pad([1, 0, 3, 4], 1, 2),
                      1, 1, 32)
    close(out, pad([1, 0, 2, 2], 1, 2), "two tokens")


def test_kat_causality_bit_equality(zt, dev):
    """src/attention_test.zig:46-72"""
    q = pad([1, 0, 0, 1, 1, 1, 1, 0, 0, 1, 1, -1], 2, 2)
    k = pad([1, 0, 0, 1, 1, 1], 1, 2)
    v = pad([1, 2, 3, 4, 5, 6], 1, 2)
    before = abi_forward(zt, dev, q, k, v, 2, 1, 32)
    k2, v2 = k.copy(), v.copy()
    k2[1, :2] = [99, 98]
    v2[1, :2] = [97, 96]
    after = abi_forward(zt, dev, q, k2, v2, 2, 1, 32)
    assert np.array_equal(before[0].view(np.uint32), after[0].view(np.uint32))
    assert after[1, 0] != before[1, 0]


def test_kat_gqa_head_mapping(zt, dev):
    """src/attention_test.zig:74-95"""
    q = pad([1, 0, 1, 0, 0, 1, 0, 1, 0, 1, 0, 1, 1, 0, 1, 0], 4, 2)
    k = pad([1, 0, 2, 0, 0, 1, 0, 2], 2, 2)
    v = pad([1, 2, 3, 4, 5, 6, 7, 8], 2, 2)
    out = abi_forward(zt, dev, q, k, v, 4, 2, 32).reshape(2, 4, 32)
    assert np.array_equal(out[0, 0, :2], [1, 2]) and np.array_equal(out[0, 2, :2], [3, 4])
    for t in range(2):
        assert np.array_equal(out[t, 0], out[t, 1])
        assert out[t, 0, 0] != out[t, 2, 0]


def test_kat_weights_sum_to_one_and_prefix_means(zt, dev):
    """src/attention_test.zig:97-128"""
    out = abi_forward(zt, dev, pad([1, 0, 0, 1, 1, 1, 0, -1], 1, 2), pad([1, 1, 0, 1, -1, 0, 2, 1], 1, 2),
                      pad([1] * 8, 1, 2), 1, 1, 32)
    assert np.all(np.abs(out[:, :2] - 1.0) <= 1e-5)
    out = abi_forward(zt, dev, pad([1, 0] * 4, 1, 2), pad([0] * 8, 1, 2), pad([1, 2, 3, 4, 5, 6, 7, 8], 1, 2),
                      1, 1, 32)
    assert np.all(np.abs(out[:, :2].ravel() - np.array([1, 2, 2, 3, 3, 4, 4, 5])) <= 1e-6)


def test_kat_survives_exp_overflow(zt, dev):
    """src/attention_test.zig:149-164: 100*100/sqrt(32) = 1768 would overflow an unshifted exp."""
    out = abi_forward(zt, dev, pad([100, 0, 100, 0], 1, 2), pad([100, 0, 0, 0], 1, 2),
                      pad([3, 5, 7, 9], 1, 2), 1, 1, 32)
    assert np.array_equal(out[:, :2].ravel(), np.array([3, 5, 3, 5], dtype=np.float32))


def test_kat_f64_accumulator_case(zt, dev, oracle):
    """src/attention_test.zig:230-295 at head_dim 32: 1/3 and 1/7 fill, T = 512."""
    T, D = 512, 32
    tj = np.add.outer(np.arange(T), np.arange(D))
    x = np.where(tj % 2 == 0, np.float32(1) / np.float32(3), np.float32(1) / np.float32(7)).astype(np.float32)
    ref = oracle.attention_forward(x, x, x, 1, 1, D)
    close(abi_forward(zt, dev, x, x, x, 1, 1, D), ref, "1/3 1/7 fill")


def test_bit_reproducible_run_to_run(zt, dev, oracle):
    """src/attention_test.zig:297-318"""
    q, k, v, do = normal_inputs(oracle, 130, 4, 2, 32, 11)
    a = run_fwd_bwd(zt, dev, q, k, v, do, 4, 2, 32)
    b = run_fwd_bwd(zt, dev, q, k, v, do, 4, 2, 32)
    for name, x, y in zip(("out", "lse", "dq", "dk", "dv"), a, b):
        if name == "dq":  # a sum over key tiles made in memory: equal to rounding (bit for bit on path 8, below)
            assert np.all(np.abs(x - y) <= 2e-6 + 2e-5 * np.abs(y))
        else:
            assert np.array_equal(x.view(np.uint32), y.view(np.uint32)), name
    zt.lib.load().zt_attn_set_path(8)
    try:
        a = run_fwd_bwd(zt, dev, q, k, v, do, 4, 2, 32)
        b = run_fwd_bwd(zt, dev, q, k, v, do, 4, 2, 32)
    finally:
        zt.lib.load().zt_attn_set_path(0)
    for x, y in zip(a, b):
        assert np.array_equal(x.view(np.uint32), y.view(np.uint32))


# ---- golden vectors and the twin's geometries -----------------------------------------------

spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)


@pytest.mark.parametrize("tag,T,H,Hkv,D", make_golden.CASES)
def test_golden_vectors(zt, dev, tag, T, H, Hkv, D):
    g = np.load(os.path.join(HERE, "golden", f"{tag}.npz"))
    q, k, v, do = make_golden.inputs(T, H, Hkv, D)
    o, lse, dq, dk, dv = run_fwd_bwd(zt, dev, q, k, v, do, H, Hkv, D)
    for name, got in (("y", o), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
        close(got, g[name], f"{tag} {name}")


TWIN_SHAPES = [  # src/cuda/attn_twin.zig:82-111, the rows that finish in seconds on the CPU
    ("ctx256", 256, 4, 2, 32), ("ctx512", 512, 4, 2, 32), ("llama3-T256", 256, 32, 8, 128),
    ("gqa-96-T256", 256, 32, 8, 96), ("mha-192-T256", 256, 16, 16, 192), ("gqa-256-T256", 256, 8, 4, 256),
]


@pytest.mark.parametrize("tag,T,H,Hkv,D", TWIN_SHAPES)
def test_twin_shapes_forward_backward(zt, dev, oracle, tag, T, H, Hkv, D):
    q, k, v, do = lcg_inputs(oracle, T, H, Hkv, D)
    ref_o, ref_lse = oracle.attention_forward(q, k, v, H, Hkv, D, want_lse=True, threads=8)
    ref = [ref_o, ref_lse, *oracle.attention_backward(q, k, v, do, H, Hkv, D, threads=8)]
    got = run_fwd_bwd(zt, dev, q, k, v, do, H, Hkv, D)
    for name, g, r in zip(("out", "lse", "dq", "dk", "dv"), got, ref):
        close(g, r, f"{tag} {name}")
    # the reference's own gates, for comparison (src/cuda/attn.cu:51,114): absolute 1e-4 / 1e-5
    assert np.max(np.abs(got[0] - ref[0])) <= 1e-4
    for g, r in zip(got[2:], ref[2:]):
        assert np.max(np.abs(g - r)) <= 1e-5


@pytest.mark.parametrize("T", [1, 2, 3, 17, 31, 32, 33, 64, 127, 129, 200])
@pytest.mark.parametrize("H,Hkv,D", [(4, 2, 32), (6, 2, 64), (2, 1, 34)])
def test_ragged_lengths_and_tails(zt, dev, oracle, T, H, Hkv, D):
    q, k, v, do = normal_inputs(oracle, T, H, Hkv, D, seed=T)
    ref_o, ref_lse = oracle.attention_forward(q, k, v, H, Hkv, D, want_lse=True, threads=4)
    ref = [ref_o, ref_lse, *oracle.attention_backward(q, k, v, do, H, Hkv, D, threads=4)]
    got = run_fwd_bwd(zt, dev, q, k, v, do, H, Hkv, D)
    for name, g, r in zip(("out", "lse", "dq", "dk", "dv"), got, ref):
        close(g, r, f"T={T} {name}")


@pytest.mark.parametrize("B,T,H,Hkv,D", [(3, 70, 4, 2, 32), (2, 129, 8, 2, 128), (5, 33, 2, 2, 64)])
def test_batched_items_are_independent(zt, dev, oracle, B, T, H, Hkv, D):
    q = oracle.fill_normal((B, T, H * D), 21, 0)
    k = oracle.fill_normal((B, T, Hkv * D), 21, 1)
    v = oracle.fill_normal((B, T, Hkv * D), 21, 2)
    do = oracle.fill_normal((B, T, H * D), 21, 3)
    tq, tk, tv, tdo = (cu(x, dev) for x in (q, k, v, do))
    o, lse = zt.attention_forward(tq, tk, tv, H, Hkv, D, want_lse=True)
    dq, dk, dv = zt.attention_backward(tq, tk, tv, o, lse, tdo, H, Hkv, D)
    for b in range(B):
        ro, rl = oracle.attention_forward(q[b], k[b], v[b], H, Hkv, D, want_lse=True, threads=4)
        rdq, rdk, rdv = oracle.attention_backward(q[b], k[b], v[b], do[b], H, Hkv, D, threads=4)
        for name, g, r in (("out", o, ro), ("lse", lse, rl), ("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
            close(g[b].cpu().numpy(), r, f"item {b} {name}")


def test_reference_abi_backward(zt, dev, oracle):
    """zt_attn_backward as device.Attn.backward calls it (src/cuda/device.zig:403-406): no out,
    no lse, caller scratch for the three per-row buffers, outputs assigned over garbage."""
    T, H, Hkv, D = 150, 8, 4, 64
    q, k, v, do = lcg_inputs(oracle, T, H, Hkv, D)
    holder = zt.Attn(T, H, Hkv, D, device=dev)
    for name, x in (("q", q), ("k", k), ("v", v), ("dout", do)):
        holder.upload(getattr(holder, name), x)
    for name in ("dq", "dk", "dv"):
        getattr(holder, name).fill_(float("nan"))   # assigned, not accumulated into
    holder.forward(1, 64)
    holder.backward(64)
    ref_o, ref_lse = oracle.attention_forward(q, k, v, H, Hkv, D, want_lse=True, threads=8)
    rdq, rdk, rdv = oracle.attention_backward(q, k, v, do, H, Hkv, D, threads=8)
    close(holder.download(q.size, holder.out).reshape(q.shape), ref_o, "out")
    close(holder.download(q.size, holder.dq).reshape(q.shape), rdq, "dq")
    close(holder.download(k.size, holder.dk).reshape(k.shape), rdk, "dk")
    close(holder.download(k.size, holder.dv).reshape(k.shape), rdv, "dv")
    close(holder.download(T * H, holder.row_max).reshape(T, H), ref_lse, "row_max = lse")
    assert np.all(holder.download(T * H, holder.row_den) == 1.0)
    delta = (ref_o.astype(np.float64) * do).reshape(T, H, D).sum(-1)
    close(holder.download(T * H, holder.row_del).reshape(T, H), delta, "row_del")
    assert holder.total_bytes() == 4 * q.nbytes + 4 * k.nbytes + 3 * T * H * 4


def test_forward_at_offsets_and_key_counts(zt, dev, oracle):
    """q_offset / n_keys semantics (src/cuda/attn_kernels.cu:276-321) away from the two usual shapes."""
    H, Hkv, D, c_t = 4, 2, 32, 96
    q, k, v, _ = normal_inputs(oracle, c_t, H, Hkv, D, 31)
    holder = zt.Attn(c_t, H, Hkv, D, device=dev)
    for (t, q_off, n_keys) in ((5, 7, 12), (5, 7, 40), (33, 0, 96), (1, 0, 1), (1, 50, 96), (40, 56, 96)):
        holder.upload(holder.q, q[:t])
        holder.upload(holder.k, k[:n_keys])
        holder.upload(holder.v, v[:n_keys])
        holder.forward_at(1, 64, q_off, n_keys, t)
        got = holder.download(t * H * D, holder.out).reshape(t, H * D)
        ref = oracle.attention_forward_at(q[:t], k[:n_keys], v[:n_keys], H, Hkv, D, q_off, n_keys)
        close(got, ref, f"t={t} q_offset={q_off} n_keys={n_keys}")
    with pytest.raises(zt.device.ShapeTooLarge):
        holder.forward_at(1, 64, 0, c_t + 1, 1)
    with pytest.raises(zt.device.ShapeTooLarge):
        holder.forward_at(1, 64, c_t, c_t, 1)


def test_decode_step_at_every_position_of_a_filling_cache(zt, dev, oracle):
    """src/decode_test.zig:222-319: the CUDA decode step against attnStep at every position,
    per-row distinct hashed data, through the reference ABI (T = 1, q_offset = n_keys - 1)."""
    H, Hkv, D, n_ctx = 4, 2, 32, 32  # src/decode_test.zig:12-20
    kdata = np.array([oracle.fill_hash(7000 + i) for i in range(n_ctx * Hkv * D)], dtype=np.float32).reshape(n_ctx, -1)
    vdata = np.array([oracle.fill_hash(90000 + i) for i in range(n_ctx * Hkv * D)], dtype=np.float32).reshape(n_ctx, -1)
    qdata = np.array([oracle.fill_hash(300000 + i) for i in range(n_ctx * H * D)], dtype=np.float32).reshape(n_ctx, -1)
    holder = zt.Attn(n_ctx, H, Hkv, D, device=dev)
    layer = oracle.Layer(n_ctx, Hkv * D)
    dlayer = zt.kv_cache.Layer(n_ctx, Hkv * D, batch=1, device=dev)
    for pos in range(n_ctx):
        layer.append(kdata[pos], vdata[pos])
        dlayer.append(cu(kdata[pos:pos + 1], dev), cu(vdata[pos:pos + 1], dev))
        n_keys = layer.visible()
        ref = oracle.attn_step(qdata[pos:pos + 1], layer, H, Hkv, D)
        holder.upload(holder.q, qdata[pos])
        holder.upload(holder.k, layer.k[:n_keys])
        holder.upload(holder.v, layer.v[:n_keys])
        holder.forward_at(1, 64, n_keys - 1, n_keys, 1)
        got = holder.download(H * D, holder.out)
        # the reference's gate is relative to the largest reference value (src/decode_test.zig:330)
        assert np.max(np.abs(got - ref[0])) <= 1e-4 * np.max(np.abs(ref))
        close(got, ref[0], f"pos {pos} (reference ABI)")
        got2 = zt.kv_cache.attn_step(cu(qdata[pos:pos + 1], dev), dlayer, H, Hkv, D)
        close(got2[0].cpu().numpy(), ref[0], f"pos {pos} (resident cache)")
    assert int(dlayer.visible()[0]) == n_ctx
    with pytest.raises(zt.kv_cache.Full):
        dlayer.append(cu(kdata[:1], dev), cu(vdata[:1], dev))
    assert np.array_equal(dlayer.k[0].cpu().numpy(), layer.k)


DECODE_SHAPES = [  # B, n_ctx, H, Hkv, D
    (5, 300, 32, 8, 128), (4, 257, 4, 2, 32), (3, 200, 8, 8, 64), (3, 130, 16, 2, 64),
    (2, 150, 12, 4, 96), (2, 90, 8, 4, 256), (3, 70, 6, 2, 192), (2, 64, 4, 2, 34), (2, 1500, 32, 8, 128),
    (2, 100, 5, 1, 80),
]


@pytest.mark.parametrize("B,n_ctx,H,Hkv,D", DECODE_SHAPES)
def test_batched_ragged_decode(zt, dev, oracle, B, n_ctx, H, Hkv, D):
    rng = np.random.default_rng(B * 1000 + n_ctx)
    n_keys = rng.integers(1, n_ctx + 1, size=B).astype(np.int32)
    n_keys[0], n_keys[-1] = n_ctx, 1          # the two extremes always present
    kc = oracle.fill_normal((B, n_ctx, Hkv * D), 41, 1)
    vc = oracle.fill_normal((B, n_ctx, Hkv * D), 41, 2)
    q = oracle.fill_normal((B, H * D), 41, 0)
    ws = zt.DecodeWorkspace(B, n_ctx, H, Hkv, D, dev)
    out, lse = zt.decode_attention(cu(q, dev), cu(kc, dev), cu(vc, dev), cu(n_keys, dev), H, Hkv, D,
                                   workspace=ws, want_lse=True)
    torch.cuda.synchronize()
    assert ws.bad_sequences() == 0
    for b in range(B):
        ro, rl = oracle.attn_step_raw(q[b], kc[b], vc[b], int(n_keys[b]), H, Hkv, D, threads=4)
        close(out[b].cpu().numpy(), ro, f"sequence {b} out (n_keys {n_keys[b]})")
        close(lse[b].cpu().numpy(), rl, f"sequence {b} lse")


def test_decode_refuses_an_empty_or_overlong_prefix(zt, dev, oracle):
    """decode.attnStep refuses n_keys < 1 (src/decode.zig:350); on the device the refusal is a NaN
    row and a count, and the other sequences are still computed."""
    B, n_ctx, H, Hkv, D = 4, 64, 8, 2, 64
    kc = oracle.fill_normal((B, n_ctx, Hkv * D), 43, 1)
    vc = oracle.fill_normal((B, n_ctx, Hkv * D), 43, 2)
    q = oracle.fill_normal((B, H * D), 43, 0)
    n_keys = np.array([0, 64, 65, 10], dtype=np.int32)
    ws = zt.DecodeWorkspace(B, n_ctx, H, Hkv, D, dev)
    out = zt.decode_attention(cu(q, dev), cu(kc, dev), cu(vc, dev), cu(n_keys, dev), H, Hkv, D, workspace=ws)
    torch.cuda.synchronize()
    assert ws.bad_sequences() == 2
    out = out.cpu().numpy()
    assert np.all(np.isnan(out[0])) and np.all(np.isnan(out[2]))
    for b in (1, 3):
        ro, _ = oracle.attn_step_raw(q[b], kc[b], vc[b], int(n_keys[b]), H, Hkv, D)
        close(out[b], ro, f"sequence {b}")
    with pytest.raises(oracle.DimensionMismatch):
        oracle.attn_step_raw(q[0], kc[0], vc[0], 0, H, Hkv, D)


def test_kv_append_semantics(zt, dev, oracle):
    """src/kv_cache.zig:88-95 and its tests :239-290, for a batch of resident caches."""
    with pytest.raises(zt.ops.DimensionMismatch):
        zt.kv_cache.Layer(0, 8, device=dev)
    layer = zt.kv_cache.Layer(3, 8, batch=2, device=dev)
    assert layer.bytes() == 2 * 2 * 3 * 8 * 4
    with pytest.raises(zt.ops.DimensionMismatch):
        layer.append(torch.zeros(2, 8, device=dev), torch.zeros(2, 4, device=dev))
    assert layer.visible().tolist() == [0, 0]
    for i in range(3):
        layer.append(torch.full((2, 8), float(i), device=dev), torch.full((2, 8), float(-i), device=dev))
    assert layer.visible().tolist() == [3, 3]
    with pytest.raises(zt.kv_cache.Full):
        layer.append(torch.zeros(2, 8, device=dev), torch.zeros(2, 8, device=dev))
    assert layer.visible().tolist() == [3, 3] and float(layer.k[1, 2, 0]) == 2.0 and float(layer.v[0, 1, 7]) == -1.0
    # the C entry point itself: a full sequence is skipped and counted, the other one advances
    n_keys = torch.tensor([3, 1], dtype=torch.int32, device=dev)
    full = torch.zeros(1, dtype=torch.int32, device=dev)
    k_new, v_new = torch.full((2, 8), 9.0, device=dev), torch.full((2, 8), 8.0, device=dev)
    torch.cuda.synchronize()
    rc = zt.lib.load().zt_kv_append(layer.k.data_ptr(), layer.v.data_ptr(), n_keys.data_ptr(),
                                    k_new.data_ptr(), v_new.data_ptr(), full.data_ptr(), 2, 3, 1, 8, None)
    torch.cuda.synchronize()
    assert rc == 0 and n_keys.tolist() == [3, 2] and int(full) == 1
    assert float(layer.k[1, 1, 0]) == 9.0 and float(layer.k[0, 2, 0]) == 2.0


def test_library_is_the_thing_that_ran(zt, dev, oracle):
    before = zt.lib.launch_count()
    q, k, v, do = normal_inputs(oracle, 40, 4, 2, 32, 2)
    run_fwd_bwd(zt, dev, q, k, v, do, 4, 2, 32)
    assert zt.lib.launch_count() - before >= 4
    assert zt.lib.last_path() != "none"


def test_refused_call_touches_nothing(zt, dev):
    L = zt.lib.load()
    L.zt_attn_set_verbose(0)
    out = torch.full((4, 128), 7.0, device=dev)
    x = torch.zeros((4, 128), device=dev)
    rc = L.zt_attn_forward(x.data_ptr(), x.data_ptr(), x.data_ptr(), out.data_ptr(), 4, 4, 2, 33, 1, 64, 0, 4, None)
    torch.cuda.synchronize()
    L.zt_attn_set_verbose(1)
    assert rc == 1 and torch.all(out == 7.0)


# ---- tensor-core (tcgen05) forward ---------------------------------------------------------------

TC_SHAPES = [  # B, T, H, Hkv, D -- multiples of the tiles, tails, one tile, several key tiles
    (1, 128, 4, 2, 32), (2, 129, 4, 2, 64), (1, 200, 8, 2, 128), (2, 256, 4, 4, 128), (1, 321, 6, 3, 64),
    (1, 384, 4, 1, 32), (1, 640, 8, 8, 128), (2, 513, 4, 2, 128), (1, 200, 8, 2, 96), (2, 384, 4, 4, 96),
    # head_dim 256, and 192 zero-padded to it: one head per CTA, K fetched block by block (forward only)
    (1, 128, 2, 1, 256), (2, 200, 4, 2, 192), (1, 513, 4, 1, 256), (1, 320, 3, 3, 192), (2, 704, 4, 2, 256),
]


@pytest.mark.parametrize("path", [0, 7, 6, 2], ids=["f16split-auto", "f16split-2heads", "f16split-1head", "3xtf32"])
@pytest.mark.parametrize("B,T,H,Hkv,D", TC_SHAPES)
def test_tensor_core_forward_matches_oracle(zt, dev, oracle, B, T, H, Hkv, D, path):
    """The tensor-core forwards: the f16-split kernel (key tiles of 64; path 0 takes two heads of a KV group per CTA
    where the group is even and the launch is large enough, path 7 wherever the group is even, path 6 never), head_dim
    32 and 96 zero-padded to their 64- and 128-wide tiles, and the 3xTF32 kernel (path 2)."""
    q = oracle.fill_normal((B, T, H * D), 51, 0)
    k = oracle.fill_normal((B, T, Hkv * D), 51, 1)
    v = oracle.fill_normal((B, T, Hkv * D), 51, 2)
    zt.lib.load().zt_attn_set_path(path)
    try:
        o, lse = zt.attention_forward(cu(q, dev), cu(k, dev), cu(v, dev), H, Hkv, D, want_lse=True)
    finally:
        zt.lib.load().zt_attn_set_path(0)
    torch.cuda.synchronize()
    # (the 3xTF32 kernel has no padded-head form: head_dim 96 goes to the CUDA cores when it is asked for)
    assert zt.lib.last_path() == ("simt" if (path == 2 and D in (96, 192, 256)) else "tcgen05")
    assert zt.lib.tc_status() == 0
    for b in range(B):
        ro, rl = oracle.attention_forward(q[b], k[b], v[b], H, Hkv, D, want_lse=True, threads=8)
        close(o[b].cpu().numpy(), ro, f"item {b} out")
        close(lse[b].cpu().numpy(), rl, f"item {b} lse")


def test_tensor_core_and_simt_paths_agree(zt, dev, oracle):
    B, T, H, Hkv, D = 2, 700, 8, 2, 128
    q = cu(oracle.fill_normal((B, T, H * D), 52, 0), dev)
    k = cu(oracle.fill_normal((B, T, Hkv * D), 52, 1), dev)
    v = cu(oracle.fill_normal((B, T, Hkv * D), 52, 2), dev)
    L = zt.lib.load()
    L.zt_attn_set_path(1)
    o_simt = zt.attention_forward(q, k, v, H, Hkv, D)
    assert zt.lib.last_path() == "simt"
    L.zt_attn_set_path(0)
    o_tc = zt.attention_forward(q, k, v, H, Hkv, D)
    assert zt.lib.last_path() == "tcgen05"
    L.zt_attn_set_path(2)
    o_tf32 = zt.attention_forward(q, k, v, H, Hkv, D)
    L.zt_attn_set_path(0)
    torch.cuda.synchronize()
    assert zt.lib.tc_status() == 0
    close(o_tc.cpu().numpy(), o_simt.cpu().numpy(), "tcgen05 f16-split vs simt")
    close(o_tf32.cpu().numpy(), o_simt.cpu().numpy(), "tcgen05 3xTF32 vs simt")


def test_tensor_core_large_magnitudes_and_peaked_rows(zt, dev, oracle):
    """Scores far apart (a few dominant keys per row, maxima that keep growing past the lazy
    rescale threshold): the hi/lo split of P and the lazily moved maximum must still land
    inside the tolerance.  (Scores are kept below ~2^5: every f32-accumulating
    kernel loses |score| * 2^-23 per accumulation, which the exponential turns into a relative
    error of P.)"""
    T, H, Hkv, D = 300, 4, 2, 64
    q = oracle.fill_normal((T, H * D), 53, 0) * np.float32(2.5)
    k = oracle.fill_normal((T, Hkv * D), 53, 1) * np.float32(2.5)
    v = oracle.fill_normal((T, Hkv * D), 53, 2)
    o, lse = zt.attention_forward(cu(q, dev), cu(k, dev), cu(v, dev), H, Hkv, D, want_lse=True)
    torch.cuda.synchronize()
    assert zt.lib.last_path() == "tcgen05" and zt.lib.tc_status() == 0
    ro, rl = oracle.attention_forward(q, k, v, H, Hkv, D, want_lse=True, threads=8)
    close(o.cpu().numpy(), ro, "peaked out")
    close(lse.cpu().numpy(), rl, "peaked lse")


# ---- tensor-core (tcgen05) backward ---------------------------------------------------------------

TC_BWD_SHAPES = [  # B, T, H, Hkv, D
    (1, 128, 4, 2, 64), (2, 129, 4, 2, 128), (1, 200, 8, 2, 128), (1, 256, 4, 4, 64), (1, 321, 6, 3, 128),
    (2, 513, 4, 1, 128), (1, 640, 8, 8, 64),
    # a last key tile with a single query tile: every step of its walk is a flush, handed between the two
    # row-warp sets (a hand-off that once raced)
    (1, 150, 8, 4, 64), (1, 160, 16, 4, 64), (1, 150, 8, 4, 128), (3, 133, 8, 8, 64),
    # head_dim 32 on the 64-wide tiles (heads zero-padded in the operand planes, outputs 32 wide)
    (1, 128, 4, 2, 32), (2, 200, 8, 2, 32), (1, 384, 4, 1, 32), (1, 513, 6, 6, 32),
    # head_dim 96 on the 128-wide tiles
    (1, 200, 8, 2, 96), (2, 384, 4, 4, 96), (1, 150, 8, 4, 96),
]


@pytest.mark.parametrize("B,T,H,Hkv,D", TC_BWD_SHAPES)
def test_tensor_core_backward_matches_oracle(zt, dev, oracle, B, T, H, Hkv, D):
    q = oracle.fill_normal((B, T, H * D), 61, 0)
    k = oracle.fill_normal((B, T, Hkv * D), 61, 1)
    v = oracle.fill_normal((B, T, Hkv * D), 61, 2)
    do = oracle.fill_normal((B, T, H * D), 61, 3)
    zt.lib.load().zt_attn_set_path(0)
    tq, tk, tv, tdo = (cu(x, dev) for x in (q, k, v, do))
    o, lse = zt.attention_forward(tq, tk, tv, H, Hkv, D, want_lse=True)
    dq, dk, dv = zt.attention_backward(tq, tk, tv, o, lse, tdo, H, Hkv, D)
    torch.cuda.synchronize()
    assert zt.lib.last_path() == "tcgen05"
    assert zt.lib.tc_status() == 0
    for b in range(B):
        rdq, rdk, rdv = oracle.attention_backward(q[b], k[b], v[b], do[b], H, Hkv, D, threads=8)
        close(dq[b].cpu().numpy(), rdq, f"item {b} dq")
        close(dk[b].cpu().numpy(), rdk, f"item {b} dk")
        close(dv[b].cpu().numpy(), rdv, f"item {b} dv")


TC_BWD_WIDE_SHAPES = [  # B, T, H, Hkv, D, keep -- head_dim 256, and 192 zero-padded to it: the unfused form
    (1, 128, 2, 1, 256, False), (2, 200, 4, 2, 192, False), (1, 513, 4, 1, 256, True), (1, 320, 3, 3, 192, True),
    (2, 704, 4, 2, 256, False),
    # contractions longer than one piece of 1024: several CTAs add into one output tile
    (1, 1300, 4, 2, 256, True), (1, 2304, 4, 1, 192, False),
]


@pytest.mark.parametrize("B,T,H,Hkv,D,keep", TC_BWD_WIDE_SHAPES)
def test_wide_head_backward_matches_oracle(zt, dev, oracle, B, T, H, Hkv, D, keep):
    """head_dim 192 and 256: P and dS go through memory as operand planes (bwd_wide_scores), dQ, dK, dV are three
    products over them (gemm_tri).  With and without the planes of q, k, v that the forward leaves in the workspace."""
    q = oracle.fill_normal((B, T, H * D), 61, 0)
    k = oracle.fill_normal((B, T, Hkv * D), 61, 1)
    v = oracle.fill_normal((B, T, Hkv * D), 61, 2)
    do = oracle.fill_normal((B, T, H * D), 61, 3)
    zt.lib.load().zt_attn_set_path(0)
    tq, tk, tv, tdo = (cu(x, dev) for x in (q, k, v, do))
    ws = zt.BackwardWorkspace(B, T, H, Hkv, D, dev)
    assert ws.nbytes > 0
    o, lse = zt.attention_forward(tq, tk, tv, H, Hkv, D, want_lse=True, keep=ws if keep else None)
    assert (ws.token != 0) == keep
    dq, dk, dv = zt.attention_backward(tq, tk, tv, o, lse, tdo, H, Hkv, D, workspace=ws, kept=keep)
    torch.cuda.synchronize()
    assert zt.lib.last_path() == "tcgen05"
    assert zt.lib.tc_status() == 0 and zt.lib.tc_saturated() == 0
    for b in range(B):
        rdq, rdk, rdv = oracle.attention_backward(q[b], k[b], v[b], do[b], H, Hkv, D, threads=8)
        close(dq[b].cpu().numpy(), rdq, f"item {b} dq")
        close(dk[b].cpu().numpy(), rdk, f"item {b} dk")
        close(dv[b].cpu().numpy(), rdv, f"item {b} dv")


@pytest.mark.parametrize("B,T,H,Hkv,D", [(2, 513, 4, 2, 128), (1, 321, 6, 3, 96), (1, 704, 4, 2, 256), (2, 200, 4, 2, 192),
                                         (1, 400, 8, 2, 64), (1, 200, 4, 1, 32)])
def test_backward_forms_of_path_8_match_oracle(zt, dev, oracle, B, T, H, Hkv, D):
    """zt_attn_set_path(8): up to head_dim 128 the two-kernel backward (dQ's kernel first, then dK/dV's: dq, dk, dv
    bit-reproducible, the form that can also store dq into peers' memory); at 192 and 256 the scores kernel that
    loads every operand per tile.  Both against the oracle, and against the default forms to rounding."""
    q = oracle.fill_normal((B, T, H * D), 67, 0)
    k = oracle.fill_normal((B, T, Hkv * D), 67, 1)
    v = oracle.fill_normal((B, T, Hkv * D), 67, 2)
    do = oracle.fill_normal((B, T, H * D), 67, 3)
    tq, tk, tv, tdo = (cu(x, dev) for x in (q, k, v, do))
    o, lse = zt.attention_forward(tq, tk, tv, H, Hkv, D, want_lse=True)
    default = zt.attention_backward(tq, tk, tv, o, lse, tdo, H, Hkv, D)
    zt.lib.load().zt_attn_set_path(8)
    try:
        got = zt.attention_backward(tq, tk, tv, o, lse, tdo, H, Hkv, D)
        again = zt.attention_backward(tq, tk, tv, o, lse, tdo, H, Hkv, D)
    finally:
        zt.lib.load().zt_attn_set_path(0)
    torch.cuda.synchronize()
    assert zt.lib.last_path() == "tcgen05" and zt.lib.tc_status() == 0 and zt.lib.tc_saturated() == 0
    for a, b_, c in zip(got, again, default):
        if D <= 128:
            assert torch.equal(a, b_)
        assert bool(((a - c).abs() <= 4e-6 + 4e-5 * c.abs()).all())
    for b in range(B):
        rdq, rdk, rdv = oracle.attention_backward(q[b], k[b], v[b], do[b], H, Hkv, D, threads=8)
        close(got[0][b].cpu().numpy(), rdq, f"item {b} dq")
        close(got[1][b].cpu().numpy(), rdk, f"item {b} dk")
        close(got[2][b].cpu().numpy(), rdv, f"item {b} dv")


def test_backward_forms_agree_on_random_shapes(zt, dev):
    """Thirty shapes drawn with a fixed seed (every tensor-core width, sequence lengths with every kind of tail, one
    to three sequences, groups of one to four heads): the default backward (fused kernel; unfused at 192/256), the
    forms of path 8 and the CUDA-core kernels agree to rounding, and no kernel gives up a wait or clamps a dS."""
    rng = np.random.default_rng(20261126)
    L = zt.lib.load()
    for case in range(30):
        D = int(rng.choice([32, 64, 96, 128, 192, 256]))
        group = int(rng.choice([1, 2, 3, 4]))
        Hkv = int(rng.choice([1, 2, 3]))
        H = Hkv * group
        B = int(rng.choice([1, 2, 3]))
        T = int(rng.integers(128, 1100 if D <= 128 else 700))
        g = torch.Generator(device=dev).manual_seed(1000 + case)
        q, do = (torch.randn((B, T, H * D), generator=g, device=dev) for _ in range(2))
        k, v = (torch.randn((B, T, Hkv * D), generator=g, device=dev) for _ in range(2))
        do *= float(rng.choice([1e-3, 1.0, 30.0]))
        o, lse = zt.attention_forward(q, k, v, H, Hkv, D, want_lse=True)
        res = {}
        for path in (0, 8, 1):
            L.zt_attn_set_path(path)
            try:
                res[path] = zt.attention_backward(q, k, v, o, lse, do, H, Hkv, D)
            finally:
                L.zt_attn_set_path(0)
            assert zt.lib.last_path() == ("simt" if path == 1 else "tcgen05"), (case, path)
        torch.cuda.synchronize()
        assert zt.lib.tc_status() == 0 and zt.lib.tc_saturated() == 0, case
        for name, a, b_, c in zip(("dq", "dk", "dv"), res[0], res[8], res[1]):
            top = float(c.abs().max())
            assert float((a - c).abs().max()) <= 3e-5 * top, (case, (B, T, H, Hkv, D), name, "default vs CUDA cores")
            assert float((b_ - c).abs().max()) <= 3e-5 * top, (case, (B, T, H, Hkv, D), name, "path 8 vs CUDA cores")


def test_wide_head_backward_rows_of_very_different_size(zt, dev, oracle):
    """The wide-head backward scales dS per query row and moves the row's factor onto a second copy of Q for dK (whose
    contraction runs across rows).  Rows of dout from 1e-4 to 1e2 times the rest -- 2^20, beyond the 2^12 the factor
    may span, and inside what the planes of dout hold (one scale per KV group: rows 2^25 below the largest are
    lost to the f16 split whatever dS does) -- and an all-zero row: every KV group against its own largest gradient,
    and each row of dq against its own size."""
    T, H, Hkv, D = 384, 4, 2, 256
    q, k, v, do = normal_inputs(oracle, T, H, Hkv, D, 64)
    fac = np.ones(T, np.float32)
    fac[5::7] = 1e-2
    fac[6::11] = 1e2
    fac[3::13] = 1e-4
    do *= fac[:, None]
    do[17] = 0.0
    o, lse, dq, dk, dv = run_fwd_bwd(zt, dev, q, k, v, do, H, Hkv, D)
    assert zt.lib.last_path() == "tcgen05" and zt.lib.tc_status() == 0 and zt.lib.tc_saturated() == 0
    rdq, rdk, rdv = oracle.attention_backward(q, k, v, do, H, Hkv, D, threads=8)
    g = H // Hkv
    for name, got, ref, w in (("dk", dk, rdk, D), ("dv", dv, rdv, D)):
        for kv in range(Hkv):
            a, r = got[:, kv * w:(kv + 1) * w].astype(np.float64), ref[:, kv * w:(kv + 1) * w].astype(np.float64)
            assert np.max(np.abs(a - r)) <= 1e-4 * np.max(np.abs(r)), (name, kv)
    # dq row by row: a row's gradient scales with that row of dout, and so does the bar (its absolute part covers
    # rows whose gradient cancels, like row 0, where dS = p (dp - delta) is zero in exact arithmetic)
    a, r = dq.astype(np.float64), rdq.astype(np.float64)
    row_top = np.max(np.abs(r), axis=1)
    assert np.all(np.max(np.abs(a - r), axis=1) <= 1e-4 * row_top + 1e-5 * fac), "dq"
    assert np.all(a[17] == 0.0)


def test_tensor_core_backward_uneven_magnitudes(zt, dev, oracle):
    """Heads and tensors of very different scale: the per-(sequence, KV group) power-of-two scaling of
    the 16-bit split must keep every group inside the tolerance."""
    T, H, Hkv, D = 260, 8, 4, 128
    q = oracle.fill_normal((T, H * D), 62, 0)
    k = oracle.fill_normal((T, Hkv * D), 62, 1)
    v = oracle.fill_normal((T, Hkv * D), 62, 2)
    do = oracle.fill_normal((T, H * D), 62, 3)
    for g, f in enumerate((1e-3, 1.0, 37.0, 2.5e3)):
        v[:, g * D:(g + 1) * D] *= np.float32(f)
        do[:, 2 * g * D:(2 * g + 2) * D] *= np.float32(1.0 / f)
    q[:, :2 * D] *= np.float32(0.05)
    k[:, D:2 * D] *= np.float32(3.0)
    tq, tk, tv, tdo = (cu(x, dev) for x in (q, k, v, do))
    o, lse = zt.attention_forward(tq, tk, tv, H, Hkv, D, want_lse=True)
    dq, dk, dv = zt.attention_backward(tq, tk, tv, o, lse, tdo, H, Hkv, D)
    torch.cuda.synchronize()
    assert zt.lib.last_path() == "tcgen05" and zt.lib.tc_status() == 0
    rdq, rdk, rdv = oracle.attention_backward(q, k, v, do, H, Hkv, D, threads=8)
    # Gradients of a group scale with that group's inputs, so the gate is relative to each KV
    # group's own largest gradient (the reference's scale-relative gate, src/cuda/attn.cu:103-113).
    g = H // Hkv
    for name, got, ref, w in (("dq", dq, rdq, g * D), ("dk", dk, rdk, D), ("dv", dv, rdv, D)):
        got = got.cpu().numpy()
        for kv in range(Hkv):
            a, r = got[:, kv * w:(kv + 1) * w].astype(np.float64), ref[:, kv * w:(kv + 1) * w].astype(np.float64)
            assert np.max(np.abs(a - r)) <= 1e-4 * np.max(np.abs(r)), (name, kv)


def test_attn_pipeline_matches_batched_calls(zt, dev):
    """AttnPipeline (copies and kernels of consecutive sequences overlapped on three streams, two buffer
    slots) returns exactly what the batched entry points return for the same sequences: more sequences
    than slots, so every slot is reused."""
    B, T, H, Hkv, D = 5, 256, 8, 2, 64
    g = torch.Generator().manual_seed(77)
    hq, hdo = (torch.randn((B, T, H * D), generator=g).pin_memory() for _ in range(2))
    hk, hv = (torch.randn((B, T, Hkv * D), generator=g).pin_memory() for _ in range(2))
    hout, hdq = (torch.full((B, T, H * D), float("nan")).pin_memory() for _ in range(2))
    hdk, hdv = (torch.full((B, T, Hkv * D), float("nan")).pin_memory() for _ in range(2))
    hlse = torch.full((B, T, H), float("nan")).pin_memory()
    pipe = zt.AttnPipeline(T, H, Hkv, D, slots=2, device=dev)
    for _ in range(2):  # a second step reuses the slots' events
        pipe.step(hq, hk, hv, hdo, hout, hdq, hdk, hdv, hlse)
    q, k, v, do = (x.to(dev) for x in (hq, hk, hv, hdo))
    out, lse = zt.attention_forward(q, k, v, H, Hkv, D, want_lse=True)
    dq, dk, dv = zt.attention_backward(q, k, v, out, lse, do, H, Hkv, D)
    for name, got, want in (("out", hout, out), ("lse", hlse, lse), ("dq", hdq, dq), ("dk", hdk, dk), ("dv", hdv, dv)):
        if name == "dq":  # (summed in memory by the fused backward: equal to rounding)
            assert bool(((got - want.cpu()).abs() <= 2e-6 + 2e-5 * want.cpu().abs()).all())
        else:
            assert torch.equal(got, want.cpu()), name


ROPE_SHAPES = [  # B, T, H, Hkv, D, pos -- tensor-core shapes (the rotation rides in the pre-pass) and CUDA-core ones
    (1, 256, 8, 2, 128, 0), (2, 200, 4, 2, 64, 37), (1, 384, 4, 1, 32, 5), (1, 150, 6, 3, 128, 1000),
    (1, 96, 4, 2, 64, 3), (1, 160, 8, 2, 96, 11),
    # head_dim 256 and 192: rotated copies, then the unfused tensor-core backward
    (1, 200, 4, 2, 256, 9), (2, 320, 4, 1, 192, 0),
]


@pytest.mark.parametrize("B,T,H,Hkv,D,pos", ROPE_SHAPES)
def test_rope_fused_forward_backward_matches_oracle(zt, dev, oracle, B, T, H, Hkv, D, pos):
    """attention over rope(q), rope(k) with q, k handed over unrotated, and the gradients of the unrotated q, k:
    against rope.forward -> attention.forward and attentionBackward -> ropeBackward on the CPU
    (src/model.zig:372-375, src/autograd.zig:559-569)."""
    q = oracle.fill_normal((B, T, H * D), 71, 0)
    k = oracle.fill_normal((B, T, Hkv * D), 71, 1)
    v = oracle.fill_normal((B, T, Hkv * D), 71, 2)
    do = oracle.fill_normal((B, T, H * D), 71, 3)
    zt.lib.load().zt_attn_set_path(0)
    tq, tk, tv, tdo = (cu(x, dev) for x in (q, k, v, do))
    ws = zt.RopeWorkspace(B, T, H, Hkv, D, dev)
    o, lse = zt.attention_forward_rope(tq, tk, tv, H, Hkv, D, pos=pos, workspace=ws, want_lse=True)
    dq, dk, dv = zt.attention_backward_rope(tq, tk, tv, o, lse, tdo, H, Hkv, D, pos=pos, workspace=ws, kept=True)
    # the first backward used the planes the forward left in the workspace; a second one converts q, k, v itself
    again = zt.attention_backward_rope(tq, tk, tv, o, lse, tdo, H, Hkv, D, pos=pos, workspace=ws)
    torch.cuda.synchronize()
    assert zt.lib.tc_status() == 0
    same_gradients((dq, dk, dv), again, D)
    for b in range(B):
        qr, kr = oracle.rope_forward(q[b], pos, D), oracle.rope_forward(k[b], pos, D)
        ro, rl = oracle.attention_forward(qr, kr, v[b], H, Hkv, D, want_lse=True, threads=4)
        rdq, rdk, rdv = oracle.attention_backward(qr, kr, v[b], do[b], H, Hkv, D, threads=4)
        rdq, rdk = oracle.rope_backward(rdq, pos, D), oracle.rope_backward(rdk, pos, D)
        close(o[b].cpu().numpy(), ro, f"out[{b}]")
        close(lse[b].cpu().numpy(), rl, f"lse[{b}]")
        close(dq[b].cpu().numpy(), rdq, f"dq[{b}]")
        close(dk[b].cpu().numpy(), rdk, f"dk[{b}]")
        close(dv[b].cpu().numpy(), rdv, f"dv[{b}]")


def test_rope_calls_refuse_bad_arguments(zt, dev):
    B, T, H, Hkv, D = 1, 128, 4, 2, 64
    q = torch.zeros((B, T, H * D), device=dev)
    k = torch.zeros((B, T, Hkv * D), device=dev)
    ws = zt.RopeWorkspace(B, T, H, Hkv, D, dev)
    with pytest.raises(zt.device.ConfigRefused, match="negative"):
        zt.attention_forward_rope(q, k, k, H, Hkv, D, pos=-1, workspace=ws)
    with pytest.raises(zt.device.ConfigRefused, match="rotary base"):
        zt.attention_forward_rope(q, k, k, H, Hkv, D, theta=0.0, workspace=ws)
    L = zt.lib.load()
    rc = L.zt_attn_forward_rope_batched(q.data_ptr(), k.data_ptr(), k.data_ptr(), q.data_ptr(), None,
                                        ws.buf.data_ptr(), 16, B, T, H, Hkv, D, 0, 500000.0, None, None)
    assert rc == 1 and "workspace" in zt.lib.last_error()


@pytest.mark.parametrize("path", [0, 7, 6], ids=["auto", "2heads", "1head"])
def test_forward_keep_hands_its_planes_to_the_backward(zt, dev, path):
    """zt_attn_forward_batched_keep + zt_attn_backward_batched_kept (same workspace, the forward's token) give what the
    unpaired calls give (bit for bit, dq to rounding: see same_gradients).  Reuse happens only on the caller's word: a plain backward with that
    workspace converts everything again, whatever the pointers are; a spent or stale token is refused."""
    B, T, H, Hkv, D = 2, 300, 8, 2, 128
    g = torch.Generator(device=dev).manual_seed(9)
    q, do = (torch.randn((B, T, H * D), generator=g, device=dev) for _ in range(2))
    k, v = (torch.randn((B, T, Hkv * D), generator=g, device=dev) for _ in range(2))
    zt.lib.load().zt_attn_set_path(path)
    try:
        o0, l0 = zt.attention_forward(q, k, v, H, Hkv, D, want_lse=True)
        ref = zt.attention_backward(q, k, v, o0, l0, do, H, Hkv, D)
        ws = zt.BackwardWorkspace(B, T, H, Hkv, D, dev)
        for _ in range(2):  # twice: a token is good for one backward, the second round gets a new one
            o1, l1 = zt.attention_forward(q, k, v, H, Hkv, D, want_lse=True, keep=ws)
            assert ws.token != 0
            got = zt.attention_backward(q, k, v, o1, l1, do, H, Hkv, D, workspace=ws, kept=True)
            assert ws.token == 0
            assert torch.equal(o1, o0) and torch.equal(l1, l0)
            same_gradients(got, ref, D)
        # q is rewritten IN PLACE between the keep and a plain backward (same pointers, same workspace): the
        # plain backward never looks at kept planes, so the gradients are those of the new q
        qm = q.clone()
        zt.attention_forward(qm, k, v, H, Hkv, D, want_lse=True, keep=ws)
        qm.mul_(0.5)
        o2, l2 = zt.attention_forward(qm, k, v, H, Hkv, D, want_lse=True)
        want2 = zt.attention_backward(qm, k, v, o2, l2, do, H, Hkv, D)
        got2 = zt.attention_backward(qm, k, v, o2, l2, do, H, Hkv, D, workspace=ws)
        same_gradients(got2, want2, D)
        # that backward rewrote the workspace: the token of the keep before it is stale now, and is refused
        stale = ws.token
        assert stale != 0
        zt.lib.load().zt_attn_set_verbose(0)
        with pytest.raises(zt.device.ConfigRefused):
            zt.attention_backward(qm, k, v, o2, l2, do, H, Hkv, D, workspace=ws, kept=True)
        zt.lib.load().zt_attn_set_verbose(1)
        # and without a token the original tensors give the original gradients
        got3 = zt.attention_backward(q, k, v, o0, l0, do, H, Hkv, D, workspace=ws)
        same_gradients(got3, ref, D)
    finally:
        zt.lib.load().zt_attn_set_path(0)
        zt.lib.load().zt_attn_set_verbose(1)
    assert zt.lib.tc_status() == 0 and zt.lib.tc_saturated() == 0


def test_forward_forms_agree(zt, dev):
    """One head per CTA and two heads per CTA: a head's key tiles go through one softmax state instead of two
    merged ones, so rounding differs; the two agree far inside the forward's parity bound, at shapes with tails
    and a padded head."""
    for (B, T, H, Hkv, D) in [(2, 1000, 8, 2, 128), (1, 777, 8, 4, 64), (1, 500, 4, 1, 96)]:
        g = torch.Generator(device=dev).manual_seed(21)
        q = torch.randn((B, T, H * D), generator=g, device=dev)
        k, v = (torch.randn((B, T, Hkv * D), generator=g, device=dev) for _ in range(2))
        res = []
        for path in (6, 7):
            zt.lib.load().zt_attn_set_path(path)
            try:
                res.append(zt.attention_forward(q, k, v, H, Hkv, D, want_lse=True))
            finally:
                zt.lib.load().zt_attn_set_path(0)
            assert zt.lib.last_path() == "tcgen05"
        torch.cuda.synchronize()
        err = (res[0][0] - res[1][0]).abs()
        assert bool((err <= 2e-6 + 2e-5 * res[0][0].abs()).all())
    assert zt.lib.tc_status() == 0


def test_training_pair_is_capturable_in_a_cuda_graph(zt, dev):
    """zt_attn_forward_batched_keep + zt_attn_backward_batched_kept take all their scratch from the caller's workspace and
    only enqueue on the caller's stream, so a step can be captured once and replayed: short sequences are bound by
    the eight launches of a step, not by the kernels."""
    B, T, H, Hkv, D = 2, 512, 8, 2, 128
    g = torch.Generator(device=dev).manual_seed(13)
    q, do = (torch.randn((B, T, H * D), generator=g, device=dev) for _ in range(2))
    k, v = (torch.randn((B, T, Hkv * D), generator=g, device=dev) for _ in range(2))
    L = zt.lib.load()
    L.zt_attn_set_path(0)
    ws = zt.BackwardWorkspace(B, T, H, Hkv, D, dev)
    out, dq = torch.empty_like(q), torch.empty_like(q)
    dk, dv = torch.empty_like(k), torch.empty_like(v)
    lse, delta = (torch.empty((B, T, H), device=dev) for _ in range(2))

    def step(stream):
        token = ctypes.c_ulonglong(0)
        rc = L.zt_attn_forward_batched_keep(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                            ws.buf.data_ptr(), ws.nbytes, B, T, H, Hkv, D, stream, ctypes.byref(token))
        assert rc == 0 and token.value != 0, zt.lib.last_error()
        rc = L.zt_attn_backward_batched_kept(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                             do.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr(),
                                             ws.buf.data_ptr(), ws.nbytes, B, T, H, Hkv, D, stream, token.value)
        assert rc == 0, zt.lib.last_error()

    step(torch.cuda.current_stream(dev).cuda_stream)  # eager: also sets the kernels' shared-memory attributes
    torch.cuda.synchronize()
    want = [x.clone() for x in (out, lse, dq, dk, dv)]
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            step(torch.cuda.current_stream(dev).cuda_stream)
    for x in (out, lse, dq, dk, dv):
        x.fill_(float("nan"))
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want[0]) and torch.equal(lse, want[1])
    same_gradients((dq, dk, dv), want[2:], D)
    assert zt.lib.tc_status() == 0


# ---- dynamic range inside one (sequence, KV group) -------------------------------------------------------------

def _outlier_inputs(T, H, Hkv, D, which, mag, frac=1e-3, seed=5):
    """N(0,1) everywhere, with a fraction `frac` of the elements of the tensors named in `which` multiplied by mag."""
    rng = np.random.default_rng(seed)
    ts = {}
    for name, w in (("q", H * D), ("k", Hkv * D), ("v", Hkv * D), ("do", H * D)):
        x = rng.standard_normal((T, w)).astype(np.float32)
        if name in which:
            x[rng.random((T, w)) < frac] *= np.float32(mag)
        ts[name] = x
    return ts["q"], ts["k"], ts["v"], ts["do"]


def _violations(got, ref):
    g, r = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return int((~(np.abs(g - r) <= ATOL + RTOL * np.abs(r))).sum())


@pytest.mark.parametrize("which,mag", [(("do",), 1e2), (("v",), 1e2), (("v", "do"), 1e2), (("v",), 1e3), (("do",), 1e3),
                                       (("v", "do"), 1e3)],
                         ids=["dout-x100", "v-x100", "v+dout-x100", "v-x1000", "dout-x1000", "v+dout-x1000"])
@pytest.mark.parametrize("D", [128, 256])
def test_tensor_core_backward_outliers_inside_a_kv_group(zt, dev, oracle, which, mag, D):
    """The operand planes carry one power-of-two scale per (sequence, KV group), so what stresses the f16 split is a
    wide range INSIDE a group: here one element in a thousand of v and/or dout is 100 or 1000 times the rest (all
    in one KV group).  dS is scaled per query row in the dQ kernel and from the group's measured maximum in the
    dK/dV kernel, so the bulk rows keep their precision.  At a hundred times the bulk everything meets the stated
    bar (a handful of dk elements apart, as on the CUDA-core path, whose f32 sums meet the same rounding); at a
    thousand times, a few elements in ten thousand miss it (counts pinned below, a regression guard: before the
    per-row scale a quarter of dq and a third of dk missed it at a HUNDRED times).  Outliers in q and k are a
    different matter: scores of 10^3 and more lose |score| 2^-23 in any f32 accumulation, on the CUDA-core path
    and in the reference's own kernels alike, and are not this library's to fix."""
    T, H, Hkv = 512, 4, 1
    q, k, v, do = _outlier_inputs(T, H, Hkv, D, which, mag)
    ref_o, ref_lse = oracle.attention_forward(q, k, v, H, Hkv, D, want_lse=True, threads=8)
    ref = dict(zip(("dq", "dk", "dv"), oracle.attention_backward(q, k, v, do, H, Hkv, D, threads=8)))
    counts = {}
    for path in (0, 1):
        zt.lib.load().zt_attn_set_path(path)
        try:
            o, lse, dq, dk, dv = run_fwd_bwd(zt, dev, q, k, v, do, H, Hkv, D)
        finally:
            zt.lib.load().zt_attn_set_path(0)
        assert zt.lib.last_path() == ("tcgen05" if path == 0 else "simt")
        if D <= 128 or mag <= 1e2:
            close(o, ref_o, "out")
        else:  # (v a thousand times the bulk at 256 columns: 3 of 524288 elements of out miss the bar, near zeros)
            assert _violations(o, ref_o) <= 8
        close(lse, ref_lse, "lse")
        counts[path] = {n: _violations(x, ref[n]) for n, x in (("dq", dq), ("dk", dk), ("dv", dv))}
    assert zt.lib.tc_status() == 0 and zt.lib.tc_saturated() == 0
    n_q, n_k = T * H * D, T * Hkv * D
    if D == 256:
        # the unfused form, twice the terms per sum.  Measured at a hundred times: dq 0..156 of 524288 (CUDA cores
        # 0..53), dk <= 4, dv 0; at a thousand: dq <= 317 (7), dk <= 134 (8), dv <= 6 (0)
        lim = (2000, 16384, 65536) if mag <= 1e2 else (1000, 100, 1000)
        assert counts[0]["dq"] <= n_q // lim[0] and counts[0]["dk"] <= n_k // lim[1] and counts[0]["dv"] <= n_k // lim[2], counts
    elif mag <= 1e2:
        assert counts[0]["dq"] == 0 and counts[0]["dv"] <= 2 and counts[0]["dk"] <= 8, counts
    else:
        # measured: dq 1..64, dk 40..335, dv 0..33 of 262144 / 65536 elements (CUDA cores: 0..2, 6..33, 0)
        assert counts[0]["dq"] <= n_q // 2000 and counts[0]["dk"] <= n_k // 100 and counts[0]["dv"] <= n_k // 1000, counts


@pytest.mark.parametrize("scale_qk", [1.0, 3.0], ids=["N(0,1)", "scores-x9"])
@pytest.mark.parametrize("B,T,H,Hkv,D", [(1, 512, 8, 2, 128), (2, 384, 4, 2, 64)])
def test_f16_split_forward_is_no_less_accurate_than_3xtf32(zt, dev, oracle, B, T, H, Hkv, D, scale_qk):
    """The benchmark definition names 3xTF32 (every product as hi.hi + hi.lo + lo.hi on kind::tf32, 21 mantissa bits
    of each operand); the default kernels run the same three terms on f16 pieces of a power-of-two-scaled operand
    (22 bits).  Both forwards exist (path 2 is the 3xTF32 one), so the claim that the departure costs no accuracy is
    measured: against the oracle the f16-split forward's error is not larger than the 3xTF32 forward's, in rms and
    in the worst element, on plain inputs and on inputs whose scores are nine times wider."""
    q = oracle.fill_normal((B, T, H * D), 91, 0) * np.float32(scale_qk)
    k = oracle.fill_normal((B, T, Hkv * D), 91, 1) * np.float32(scale_qk)
    v = oracle.fill_normal((B, T, Hkv * D), 91, 2)
    ref = np.stack([oracle.attention_forward(q[b], k[b], v[b], H, Hkv, D, threads=8) for b in range(B)]).astype(np.float64)
    err = {}
    for path in (0, 2):
        zt.lib.load().zt_attn_set_path(path)
        try:
            o = zt.attention_forward(cu(q, dev), cu(k, dev), cu(v, dev), H, Hkv, D)
        finally:
            zt.lib.load().zt_attn_set_path(0)
        torch.cuda.synchronize()
        assert zt.lib.last_path() == "tcgen05"
        d = o.cpu().numpy().astype(np.float64) - ref
        err[path] = (float(np.sqrt((d * d).mean())), float(np.abs(d).max()))
    assert zt.lib.tc_status() == 0
    assert err[0][0] <= 1.1 * err[2][0] and err[0][1] <= 1.5 * err[2][1], err
