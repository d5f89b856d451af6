"""The per-device arena behind the entry points that take no workspace (zt_attn_forward, zt_attn_backward,
zt_attn_forward_batched): it may allocate, so it must never do so inside a stream capture, and a caller can size
it up front with zt_attn_reserve.  (This file sorts before the full-size tests so that the arena is still small
when it runs; it also works after them.)"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


def test_reference_abi_refuses_to_grow_its_arena_inside_a_capture(zt, dev):
    """zt_attn_forward takes its operand planes from the per-device arena.  Growing the arena means cudaMalloc,
    which must not happen while the caller's stream is being captured: the call is refused (return 1, nothing
    launched, the capture intact) and works once zt_attn_reserve has sized the arena beforehand."""
    L = zt.lib.load()
    H, Hkv, D = 8, 2, 128
    # a sequence whose operand planes (T x (8 + 2 + 2) x 128 x 4 bytes) need more than the arena holds now
    T = max(9000, int(L.zt_attn_arena_bytes() * 1.25) // ((H + 2 * Hkv) * D * 4))
    g = torch.Generator(device=dev).manual_seed(3)
    q = torch.randn((T, H * D), generator=g, device=dev)
    k, v = (torch.randn((T, Hkv * D), generator=g, device=dev) for _ in range(2))
    out = torch.full_like(q, 7.0)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    L.zt_attn_set_verbose(0)
    rcs = []
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            st = torch.cuda.current_stream(dev).cuda_stream
            rcs.append(L.zt_attn_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), T, H, Hkv, D, 1, 64, 0, T, st))
    L.zt_attn_set_verbose(1)
    assert rcs == [1] and "zt_attn_reserve" in zt.lib.last_error()
    graph.replay()  # an empty graph: the refused call enqueued nothing and did not break the capture
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())
    assert L.zt_attn_reserve(1, T, H, Hkv, D) == 0
    graph2 = torch.cuda.CUDAGraph()
    # eager once (sets the kernels' shared-memory attributes), then captured
    assert L.zt_attn_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), T, H, Hkv, D, 1, 64, 0, T,
                             torch.cuda.current_stream(dev).cuda_stream) == 0
    torch.cuda.synchronize()
    want = out.clone()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph2, stream=side):
            st = torch.cuda.current_stream(dev).cuda_stream
            assert L.zt_attn_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), T, H, Hkv, D, 1, 64, 0, T, st) == 0
    out.fill_(float("nan"))
    graph2.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want) and zt.lib.tc_status() == 0
