"""GPU checks at the benchmark configurations' full sizes.

The oracle is O(H T^2 D) scalar f64, so at these sizes it checks SAMPLED units exactly
(rows of a head, one KV group of the backward, whole sequences of a decode batch) and the
rest is covered by identities that hold for any input:
  * sum_s dv[s, kv, :] = sum_{h in group} sum_t dout[t, h, :]        (each softmax row sums to 1)
  * sum_t dq[t, h in group] . q[t, h]  =  sum_s dk[s, kv] . k[s, kv]  (both are sum ds * score)
  * decode: the log-sum-exp combine of any split equals the unsplit result (checked through the
    oracle on sampled sequences of every length class).
Inputs are i.i.d. N(0,1) generated on the device from a fixed seed; the sampled units are copied
back so the oracle sees the same bytes.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-4, 1e-5


def close(got, ref, what=""):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    err = np.abs(got - ref)
    bad = ~(err <= ATOL + RTOL * np.abs(ref))
    if bad.any():
        i = int(np.argmax(np.where(np.isnan(err), np.inf, err)))
        raise AssertionError(f"{what}: {int(bad.sum())}/{err.size} outside tolerance; worst at {i}: "
                             f"got {got.ravel()[i]!r} want {ref.ravel()[i]!r}")


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


def randn(shape, seed, dev):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    return torch.randn(shape, generator=g, device=dev, dtype=torch.float32)


@pytest.mark.parametrize("B,T,H,Hkv,D", [(8, 2048, 32, 8, 128), (8, 4096, 32, 8, 32), (8, 512, 32, 8, 256),
                                         (8, 1024, 32, 8, 64),
                                         (8, 4096, 32, 8, 128),     # the headline point of the sweep
                                         (1, 32768, 32, 8, 128)])   # the long-context prefill
def test_prefill_sweep_point(zt, dev, oracle, B, T, H, Hkv, D):
    q, k, v, do = (randn((B, T, n * D), s, dev) for n, s in ((H, 1), (Hkv, 2), (Hkv, 3), (H, 4)))
    o, lse = zt.attention_forward(q, k, v, H, Hkv, D, want_lse=True)
    dq, dk, dv = zt.attention_backward(q, k, v, o, lse, do, H, Hkv, D)
    torch.cuda.synchronize()
    for x in (o, lse, dq, dk, dv):
        assert bool(torch.isfinite(x).all())
    group = H // Hkv
    # identities, in float64 on the device
    dv_sum = dv.double().view(B, T, Hkv, D).sum(1)
    do_sum = do.double().view(B, T, Hkv, group, D).sum(3).sum(1)
    assert torch.allclose(dv_sum, do_sum, rtol=1e-4, atol=1e-3 * float(do_sum.abs().max()))
    dq_q = (dq.double() * q.double()).view(B, T, Hkv, group * D).sum((1, 3))
    dk_k = (dk.double() * k.double()).view(B, T, Hkv, D).sum((1, 3))
    assert torch.allclose(dq_q, dk_k, rtol=1e-4, atol=1e-4 * float(dk_k.abs().max()) + 1e-3)
    # sampled rows of the forward against the oracle: first, middle, last rows of three heads
    for (b, h) in ((0, 0), (B // 2, H // 2 + 1), (B - 1, H - 1)):
        qh, kh, vh = (x[b].cpu().numpy() for x in (q, k, v))
        for t0 in (0, T // 2 - 3, T - 4):
            ro, rl = oracle.attention_forward_rows(qh, kh, vh, H, Hkv, D, h, t0, t0 + 4)
            close(o[b, t0:t0 + 4, h * D:(h + 1) * D].cpu().numpy(), ro, f"out b{b} h{h} rows {t0}..")
            close(lse[b, t0:t0 + 4, h].cpu().numpy(), rl, f"lse b{b} h{h} rows {t0}..")


def test_prefill_backward_one_kv_group_exact(zt, dev, oracle):
    """One KV group of one item of a sweep point, every row, against the oracle."""
    B, T, H, Hkv, D = 2, 1024, 32, 8, 128
    q, k, v, do = (randn((B, T, n * D), s, dev) for n, s in ((H, 5), (Hkv, 6), (Hkv, 7), (H, 8)))
    o, lse = zt.attention_forward(q, k, v, H, Hkv, D, want_lse=True)
    dq, dk, dv = zt.attention_backward(q, k, v, o, lse, do, H, Hkv, D)
    b, kv, g = 1, 5, H // Hkv
    rdq, rdk, rdv = oracle.attention_backward_kv_group(*(x[b].cpu().numpy() for x in (q, k, v, do)), H, Hkv, D, kv)
    cols_q = slice(kv * g * D, (kv + 1) * g * D)
    cols_k = slice(kv * D, (kv + 1) * D)
    close(dq[b, :, cols_q].cpu().numpy(), rdq[:, cols_q], "dq group")
    close(dk[b, :, cols_k].cpu().numpy(), rdk[:, cols_k], "dk group")
    close(dv[b, :, cols_k].cpu().numpy(), rdv[:, cols_k], "dv group")


def _host_threads():
    import os
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def test_headline_backward_one_kv_group_every_element(zt, dev, oracle):
    """The benchmark's own point (batch 8, T 4096, 32/8 heads, head_dim 128): every element of dq (four heads)
    and of dk, dv of one KV group of one sequence against the oracle, element-wise at the stated bar.  The dK/dV
    kernel's accumulators take terms from all 4 x 64 query tiles here, the walk and the flush schedule that keep
    the tensor core's truncating accumulation in check are exercised at their full depth, and a tile flushed to
    the wrong rows could not hide behind a sum."""
    B, T, H, Hkv, D = 8, 4096, 32, 8, 128
    q, k, v, do = (randn((B, T, n * D), s, dev) for n, s in ((H, 21), (Hkv, 22), (Hkv, 23), (H, 24)))
    o, lse = zt.attention_forward(q, k, v, H, Hkv, D, want_lse=True)
    dq, dk, dv = zt.attention_backward(q, k, v, o, lse, do, H, Hkv, D)
    torch.cuda.synchronize()
    assert zt.lib.last_path() == "tcgen05" and zt.lib.tc_status() == 0 and zt.lib.tc_saturated() == 0
    b, kv, g = 5, 3, H // Hkv
    rdq, rdk, rdv = oracle.backward_window(*(x[b].cpu().numpy() for x in (q, k, v, do)), H, Hkv, D, kv,
                                           list(range(T)), T, threads=_host_threads())
    close(dq[b].view(T, H, D)[:, kv * g:(kv + 1) * g].cpu().numpy(), rdq, "dq of the group")
    close(dk[b, :, kv * D:(kv + 1) * D].cpu().numpy(), rdk, "dk of the group")
    close(dv[b, :, kv * D:(kv + 1) * D].cpu().numpy(), rdv, "dv of the group")


def test_long_context_backward_sampled_rows_and_last_keys(zt, dev, oracle):
    """T 32768 (the long-context prefill): dq of sampled query rows of one KV group and dk, dv of its last 2048
    keys (a key needs only the query rows at or after it, so the tail is what the oracle can afford), element-wise
    at the stated bar.  The earliest key tiles, whose accumulators see all 512 query tiles, are covered by the
    identities of test_prefill_sweep_point and, exactly, at T 4096 above."""
    B, T, H, Hkv, D = 1, 32768, 32, 8, 128
    q, k, v, do = (randn((B, T, n * D), s, dev) for n, s in ((H, 31), (Hkv, 32), (Hkv, 33), (H, 34)))
    o, lse = zt.attention_forward(q, k, v, H, Hkv, D, want_lse=True)
    dq, dk, dv = zt.attention_backward(q, k, v, o, lse, do, H, Hkv, D)
    torch.cuda.synchronize()
    assert zt.lib.last_path() == "tcgen05" and zt.lib.tc_status() == 0 and zt.lib.tc_saturated() == 0
    kv, g, window = 6, H // Hkv, 2048
    rows = [0, 1, 127, 128, 4095, 16383, 16384, 30000, 32767]
    rdq, rdk, rdv = oracle.backward_window(*(x[0].cpu().numpy() for x in (q, k, v, do)), H, Hkv, D, kv, rows, window,
                                           threads=_host_threads())
    close(dq[0].view(T, H, D)[rows][:, kv * g:(kv + 1) * g].cpu().numpy(), rdq, "dq of sampled rows")
    close(dk[0, T - window:, kv * D:(kv + 1) * D].cpu().numpy(), rdk, "dk of the last keys")
    close(dv[0, T - window:, kv * D:(kv + 1) * D].cpu().numpy(), rdv, "dv of the last keys")


def test_llama3_decode_full_size(zt, dev, oracle):
    """B 64, context 8192 (the new token's row included), 32/8 heads, head_dim 128: 4 GiB of cache."""
    B, n_ctx, H, Hkv, D = 64, 8192, 32, 8, 128
    kc, vc = randn((B, n_ctx, Hkv * D), 11, dev), randn((B, n_ctx, Hkv * D), 12, dev)
    q = randn((B, H * D), 13, dev)
    n_keys = torch.full((B,), n_ctx, dtype=torch.int32, device=dev)
    ws = zt.DecodeWorkspace(B, n_ctx, H, Hkv, D, dev)
    out, lse = zt.decode_attention(q, kc, vc, n_keys, H, Hkv, D, workspace=ws, want_lse=True)
    torch.cuda.synchronize()
    assert ws.bad_sequences() == 0 and bool(torch.isfinite(out).all())
    for b in (0, 31, 63):
        ro, rl = oracle.attn_step_raw(q[b].cpu().numpy(), kc[b].cpu().numpy(), vc[b].cpu().numpy(), n_ctx,
                                      H, Hkv, D, threads=8)
        close(out[b].cpu().numpy(), ro, f"sequence {b}")
        close(lse[b].cpu().numpy(), rl, f"sequence {b} lse")


def test_ragged_decode_full_size(zt, dev, oracle):
    """B 256, per-sequence context uniform in [1, 16384]: 32 GiB of padded cache."""
    B, n_ctx, H, Hkv, D = 256, 16384, 32, 8, 128
    free, _ = torch.cuda.mem_get_info(dev)
    if free < 40 * 2 ** 30:
        pytest.skip("needs 40 GiB of free device memory")
    kc = torch.empty((B, n_ctx, Hkv * D), dtype=torch.float32, device=dev)
    vc = torch.empty_like(kc)
    for i in range(0, B, 32):  # filled in slices to bound the generator's temporary
        kc[i:i + 32] = randn((32, n_ctx, Hkv * D), 100 + i, dev)
        vc[i:i + 32] = randn((32, n_ctx, Hkv * D), 500 + i, dev)
    q = randn((B, H * D), 14, dev)
    rng = np.random.default_rng(0)
    nk = rng.integers(1, n_ctx + 1, size=B).astype(np.int32)
    nk[3], nk[200] = 1, n_ctx
    n_keys = torch.from_numpy(nk).to(dev)
    ws = zt.DecodeWorkspace(B, n_ctx, H, Hkv, D, dev)
    out = zt.decode_attention(q, kc, vc, n_keys, H, Hkv, D, workspace=ws)
    torch.cuda.synchronize()
    assert ws.bad_sequences() == 0 and bool(torch.isfinite(out).all())
    for b in (3, 200, int(np.argsort(nk)[B // 2]), 255):
        n = int(nk[b])
        ro, _ = oracle.attn_step_raw(q[b].cpu().numpy(), kc[b, :n].cpu().numpy(), vc[b, :n].cpu().numpy(), n,
                                     H, Hkv, D, threads=8)
        close(out[b].cpu().numpy(), ro, f"sequence {b} (n_keys {n})")
