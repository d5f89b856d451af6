"""The N > 1 host logic on CPU: two gloo ranks shard the work, compute their units with the
oracle (the CUDA library needs a GPU), gather, and must reproduce the unsharded result bit for
bit -- units are independent, so sharding may not change a single value."""
import importlib
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import zt_oracle as oracle
    zt = importlib.import_module("z-transformer_b200")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sh = zt.sharding
        if case == "kv_heads":
            T, H, Hkv, D = 24, 8, 4, 16
            q = oracle.fill_normal((T, H * D), 3, 0)
            k = oracle.fill_normal((T, Hkv * D), 3, 1)
            v = oracle.fill_normal((T, Hkv * D), 3, 2)
            do = oracle.fill_normal((T, H * D), 3, 3)
            s = sh.shard_kv_heads(H, Hkv, world, rank)
            ql, dol = (sh.slice_heads(torch.from_numpy(x), s.h0, s.h1, D).numpy() for x in (q, do))
            kl, vl = (sh.slice_heads(torch.from_numpy(x), s.kv0, s.kv1, D).numpy() for x in (k, v))
            o, lse = oracle.attention_forward(ql, kl, vl, s.n_heads, s.n_kv_heads, D, want_lse=True)
            dq, dk, dv = oracle.attention_backward(ql, kl, vl, dol, s.n_heads, s.n_kv_heads, D)
            got = [sh.gather_heads(torch.from_numpy(x), world).numpy() for x in (o, lse, dq, dk, dv)]
            fo, flse = oracle.attention_forward(q, k, v, H, Hkv, D, want_lse=True)
            want = [fo, flse, *oracle.attention_backward(q, k, v, do, H, Hkv, D)]
        elif case == "batch":
            B, T, H, Hkv, D = 4, 9, 4, 2, 8
            q = oracle.fill_normal((B, T, H * D), 4, 0)
            k = oracle.fill_normal((B, T, Hkv * D), 4, 1)
            v = oracle.fill_normal((B, T, Hkv * D), 4, 2)
            mine = sh.shard_batch(B, world, rank)
            local = np.stack([oracle.attention_forward(q[b], k[b], v[b], H, Hkv, D) for b in mine])
            got = [sh.gather_batch(torch.from_numpy(local), world).numpy()]
            want = [np.stack([oracle.attention_forward(q[b], k[b], v[b], H, Hkv, D) for b in range(B)])]
        else:  # ragged decode
            B, n_ctx, H, Hkv, D = 6, 40, 4, 2, 8
            rng = np.random.default_rng(5)
            n_keys = rng.integers(1, n_ctx + 1, size=B)
            kc = oracle.fill_normal((B, n_ctx, Hkv * D), 5, 1)
            vc = oracle.fill_normal((B, n_ctx, Hkv * D), 5, 2)
            q = oracle.fill_normal((B, H * D), 5, 0)
            assignment, inverse = sh.balance_sequences(n_keys, world)
            local = np.stack([oracle.attn_step_raw(q[b], kc[b], vc[b], int(n_keys[b]), H, Hkv, D)[0]
                              for b in assignment[rank]])
            got = [sh.gather_sequences(torch.from_numpy(local), inverse, world).numpy()]
            want = [np.stack([oracle.attn_step_raw(q[b], kc[b], vc[b], int(n_keys[b]), H, Hkv, D)[0]
                              for b in range(B)])]
        ok = all(np.array_equal(g.view(np.uint32), w.view(np.uint32)) for g, w in zip(got, want))
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", ["kv_heads", "batch", "ragged_decode"])
def test_two_ranks_reproduce_the_unsharded_result(case):
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), case, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}


def test_shard_plans(zt):
    sh = zt.sharding
    s = sh.shard_kv_heads(32, 8, 4, 3)
    assert (s.kv0, s.kv1, s.h0, s.h1) == (6, 8, 24, 32)
    assert list(sh.shard_batch(8, 4, 1)) == [2, 3]
    with pytest.raises(ValueError):
        sh.shard_kv_heads(32, 8, 3, 0)
    with pytest.raises(ValueError):
        sh.shard_batch(7, 2, 0)
    n_keys = [100, 1, 50, 49, 99, 2, 3, 98]
    assignment, inverse = sh.balance_sequences(n_keys, 2)
    assert sorted(assignment[0] + assignment[1]) == list(range(8))
    assert len(assignment[0]) == len(assignment[1]) == 4
    loads = [sum(n_keys[i] for i in a) for a in assignment]
    assert abs(loads[0] - loads[1]) <= 2
    flat = assignment[0] + assignment[1]
    assert [flat[inverse[i]] for i in range(8)] == list(range(8))
