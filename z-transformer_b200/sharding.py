"""Multi-GPU sharding of the attention path: independent units, one gather at the end.

The unit of independence is (sequence, KV head together with its group of query
heads): the forward rows, dq, and dk/dv of a KV head depend only on that head's
K, V and on its group's Q and dO (src/attention.zig:111-112,
src/autograd.zig:723-724,821-838).  So ranks never exchange anything on the data
path; an all-gather only returns the sharded outputs to every rank.  One process
per GPU; `torch.distributed` (NCCL on GPUs, gloo in CPU tests) does the plumbing.
Every tensor a collective touches lives in the calling rank's own memory.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class HeadShard:
    """KV heads [kv0, kv1) and their query heads [h0, h1) owned by one rank."""
    kv0: int
    kv1: int
    h0: int
    h1: int

    @property
    def n_kv_heads(self) -> int:
        return self.kv1 - self.kv0

    @property
    def n_heads(self) -> int:
        return self.h1 - self.h0


def shard_kv_heads(n_heads: int, n_kv_heads: int, world: int, rank: int) -> HeadShard:
    """Contiguous, equal split of the KV heads; a group never straddles two ranks."""
    if n_kv_heads <= 0 or n_heads % n_kv_heads != 0:
        raise ValueError(f"{n_heads} heads over {n_kv_heads} kv heads is not a group")
    if world < 1 or not 0 <= rank < world or n_kv_heads % world != 0:
        raise ValueError(f"{n_kv_heads} kv heads do not split over {world} ranks")
    group = n_heads // n_kv_heads
    per = n_kv_heads // world
    return HeadShard(rank * per, (rank + 1) * per, rank * per * group, (rank + 1) * per * group)


def shard_batch(batch: int, world: int, rank: int) -> range:
    """Contiguous, equal split of independent sequences."""
    if world < 1 or not 0 <= rank < world or batch % world != 0:
        raise ValueError(f"{batch} sequences do not split over {world} ranks")
    per = batch // world
    return range(rank * per, (rank + 1) * per)


def balance_sequences(n_keys, world: int):
    """Assign ragged sequences to ranks: longest first, each to the least-loaded rank that
    still has room, with equal counts per rank so the final all-gather is uniform.

    Returns (assignment, inverse): assignment[r] lists the sequence indices rank r owns,
    and inverse[i] is the position of sequence i in the concatenation of all ranks' lists.
    """
    n = len(n_keys)
    if world < 1 or n % world != 0:
        raise ValueError(f"{n} sequences do not split over {world} ranks")
    per = n // world
    order = sorted(range(n), key=lambda i: (-int(n_keys[i]), i))
    load = [0] * world
    assignment = [[] for _ in range(world)]
    for i in order:
        r = min((r for r in range(world) if len(assignment[r]) < per), key=lambda r: (load[r], r))
        assignment[r].append(i)
        load[r] += int(n_keys[i])
    inverse = [0] * n
    pos = 0
    for r in range(world):
        for i in assignment[r]:
            inverse[i] = pos
            pos += 1
    return assignment, inverse


def slice_heads(x, h0: int, h1: int, head_dim: int):
    """Columns of heads [h0, h1) of a [..., H*D] tensor as a contiguous [..., Hs*D] copy."""
    return x[..., h0 * head_dim:h1 * head_dim].contiguous()


def _all_gather(local, world: int, group=None):
    import torch
    import torch.distributed as dist
    local = local.contiguous()
    # the concatenated form ([world * n0, ...]) is the one every backend accepts
    flat = torch.empty((world * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype,
                       device=local.device)
    dist.all_gather_into_tensor(flat, local, group=group)
    return flat.view((world,) + tuple(local.shape))


def gather_heads(local, world: int, group=None):
    """[..., T, Hs*D] per rank -> [..., T, H*D] on every rank (rank r's heads at columns r*Hs*D)."""
    if world == 1:
        return local
    g = _all_gather(local, world, group)          # [G, ..., T, Hs*D]
    g = g.movedim(0, -2)                          # [..., T, G, Hs*D]
    return g.reshape(*g.shape[:-2], g.shape[-2] * g.shape[-1]).contiguous()


def gather_batch(local, world: int, group=None):
    """[Bs, ...] per rank -> [B, ...] on every rank (rank r's sequences at rows r*Bs)."""
    if world == 1:
        return local
    g = _all_gather(local, world, group)
    return g.reshape((g.shape[0] * g.shape[1],) + tuple(g.shape[2:]))


def gather_sequences(local, inverse, world: int, group=None):
    """Undo balance_sequences: [Bs, ...] per rank -> [B, ...] in the caller's original order."""
    import torch
    g = gather_batch(local, world, group)
    idx = torch.as_tensor(inverse, dtype=torch.long, device=g.device)
    return g.index_select(0, idx)


class GatheredOutput:
    """An output tensor that every rank's kernels fill in place on every rank: [world, *shard_shape] floats in
    symmetric memory (one allocation per rank, all mapped into each other's address space).  Rank r's kernels are
    given `local` (its shard's place in its own copy) as their output and `peer_pointers()` (the same place in every
    other rank's copy) as peer copies; once all ranks' kernels have finished -- any collective or barrier ordered
    after them tells -- `gathered` holds every shard on every rank, with no all-gather of this tensor.

    Needs NCCL-initialised torch.distributed, one rank per GPU on one node (torch symmetric memory maps the peers'
    buffers through CUDA virtual-memory handles)."""

    def __init__(self, shard_shape, world: int, rank: int, device, group=None):
        import math

        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.world, self.rank = world, rank
        self.shard_shape = tuple(int(x) for x in shard_shape)
        self.gathered = symm_mem.empty((world,) + self.shard_shape, dtype=torch.float32, device=device)
        self.handle = symm_mem.rendezvous(self.gathered, group if group is not None else dist.group.WORLD)
        shard_bytes = 4 * math.prod(self.shard_shape)
        self.local = self.gathered[rank]
        self._peers = [int(self.handle.buffer_ptrs[r]) + rank * shard_bytes for r in range(world) if r != rank]

    def peer_tensors(self):
        """This rank's shard's place in every OTHER rank's copy, as tensors: `t.copy_(self.local)` on a side stream
        is a device-to-device copy over NVLink by the copy engines (no SM is involved), the way to push a shard that
        was written locally when the kernels' own epilogues should not carry the peer stores (a step whose kernels
        are about as short as the transfer: the stores would hold the SMs)."""
        import torch
        if not hasattr(self, "_peer_tensors"):
            full = (self.world,) + self.shard_shape
            self._peer_tensors = [self.handle.get_buffer(r, full, torch.float32)[self.rank]
                                  for r in range(self.world) if r != self.rank]
        return self._peer_tensors

    def peer_pointers(self):
        """(ctypes array of the peers' device pointers, count) for the *_peers entry points."""
        import ctypes
        arr = (ctypes.c_void_p * max(1, len(self._peers)))(*self._peers)
        return arr, len(self._peers)


def forward_keep_gathered(q, k, v, out: GatheredOutput, lse, workspace, n_heads, n_kv_heads, head_dim):
    """zt_attn_forward_batched_keep_peers on this rank's shard: out lands in out.local and in every peer's copy.
    Returns the token for the kept planes (0 when the shape left the tensor-core path: the call is then refused)."""
    import ctypes

    import torch

    from . import lib as _lib
    from .device import ConfigRefused
    B, T = q.shape[0], q.shape[1]
    peers, n = out.peer_pointers()
    token = ctypes.c_ulonglong(0)
    with torch.cuda.device(q.device):
        rc = _lib.load().zt_attn_forward_batched_keep_peers(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.local.data_ptr(), lse.data_ptr(), workspace.buf.data_ptr(),
            workspace.nbytes, B, T, n_heads, n_kv_heads, head_dim, torch.cuda.current_stream(q.device).cuda_stream,
            ctypes.byref(token), peers, n)
    if rc != 0:
        raise ConfigRefused(_lib.last_error())
    return token.value


def backward_kept_gathered(q, k, v, out_local, lse, dout, dq: GatheredOutput, dk, dv, delta, workspace, token, n_heads,
                           n_kv_heads, head_dim):
    """zt_attn_backward_batched_kept_peers: dq lands in dq.local and in every peer's copy; dk, dv stay local (they are
    a quarter of dq's bytes and are flushed many times per CTA: gather them with gather_batch / gather_heads)."""
    import torch

    from . import lib as _lib
    from .device import ConfigRefused
    B, T = q.shape[0], q.shape[1]
    peers, n = dq.peer_pointers()
    with torch.cuda.device(q.device):
        rc = _lib.load().zt_attn_backward_batched_kept_peers(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out_local.data_ptr(), lse.data_ptr(), dout.data_ptr(),
            dq.local.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr(), workspace.buf.data_ptr(),
            workspace.nbytes, B, T, n_heads, n_kv_heads, head_dim, torch.cuda.current_stream(q.device).cuda_stream,
            token, peers, n)
    if rc != 0:
        raise ConfigRefused(_lib.last_error())
