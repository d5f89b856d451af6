"""Two ranks on two GPUs: the training pair whose kernels write out and dq straight into every rank's gathered copy
(zt_attn_forward_batched_keep_peers / zt_attn_backward_batched_kept_peers), against the unsharded computation.
Needs two CUDA devices; skipped elsewhere.  Each rank is a child process (NCCL, 127.0.0.1)."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, results):
    import importlib
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    zt = importlib.import_module("z-transformer_b200")
    B, T, H, Hkv, D = 4, 384, 8, 2, 128
    g = torch.Generator(device=dev).manual_seed(77)           # the same full tensors on every rank
    q, do = (torch.randn((B, T, H * D), generator=g, device=dev) for _ in range(2))
    k, v = (torch.randn((B, T, Hkv * D), generator=g, device=dev) for _ in range(2))
    # the unsharded answer
    o_ref, lse_ref = zt.attention_forward(q, k, v, H, Hkv, D, want_lse=True)
    dq_ref, dk_ref, dv_ref = zt.attention_backward(q, k, v, o_ref, lse_ref, do, H, Hkv, D)
    # this rank's sequences
    mine = zt.sharding.shard_batch(B, world, rank)
    sl = slice(mine.start, mine.stop)
    Bs = len(mine)
    qs, ks, vs, dos = (x[sl].contiguous() for x in (q, k, v, do))
    g_out = zt.sharding.GatheredOutput((Bs, T, H * D), world, rank, dev)
    g_dq = zt.sharding.GatheredOutput((Bs, T, H * D), world, rank, dev)
    ok = True
    for round_ in range(2):                                     # twice: the buffers are reused step after step
        g_out.gathered.fill_(float("nan")), g_dq.gathered.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()                                          # nobody writes into a buffer a peer is still clearing
        ws = zt.BackwardWorkspace(Bs, T, H, Hkv, D, dev)
        lse = torch.empty((Bs, T, H), device=dev)
        delta = torch.empty_like(lse)
        dk, dv = torch.empty_like(ks), torch.empty_like(vs)
        token = zt.sharding.forward_keep_gathered(qs, ks, vs, g_out, lse, ws, H, Hkv, D)
        assert token != 0
        zt.sharding.backward_kept_gathered(qs, ks, vs, g_out.local, lse, dos, g_dq, dk, dv, delta, ws, token, H, Hkv, D)
        dk_all = zt.sharding.gather_batch(dk, world)            # ordered after the kernels: when it is done on a rank,
        dv_all = zt.sharding.gather_batch(dv, world)            # every peer's kernels have finished writing to it
        torch.cuda.synchronize()
        ok &= torch.equal(g_out.gathered.view(B, T, H * D), o_ref)
        # (the references come from the fused backward; the call that also stores dq into the peers runs the
        # two-kernel form, whose dS is scaled differently: equal to rounding, not bit for bit)
        def near(a, b):
            return bool(((a - b).abs() <= 2e-6 + 2e-5 * b.abs()).all())
        ok &= near(g_dq.gathered.view(B, T, H * D), dq_ref)
        ok &= near(dk_all, dk_ref) and near(dv_all, dv_ref)
    ok &= zt.lib.tc_status() == 0
    results[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_outputs_written_into_every_ranks_gathered_copy():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, 29577, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():   # a rank that never finished: end exactly the processes this test started
            p.terminate()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert dict(results) == {0: True, 1: True}
