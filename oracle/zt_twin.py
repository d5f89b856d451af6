"""Writes the directory the reference's twin program writes (src/cuda/attn_twin.zig:150-269), from the oracle.

TEST INFRASTRUCTURE, like the rest of oracle/: only tests/ and the harness check use it.  The
reference's twin runs attention.forward and autograd.attentionBackward on the CPU for a table of shapes
and leaves, per shape, `<tag>.{q,k,v,y,dout,dq,dk,dv}.bin` (raw little-endian f32) and one row of
`manifest.tsv`: `tag T n_heads n_kv_heads head_dim iters cpu_us`.  Zig is not available here, so this
module produces the same files from the C restatement of those two functions: same shapes
(attn_twin.zig:73-112), same fill (the LCG of attn_twin.zig:283-289 with seeds 0xbeef, 0x1234, 0x5678,
0x9abc for q, k, v, dout), same layout.  `cpu_us` is the oracle's own forward time (minimum of three
calls), not the Zig program's.
"""
from __future__ import annotations

import os
import time

import numpy as np

import zt_oracle as oracle

# tag, T, n_heads, n_kv_heads, head_dim, iters  (attn_twin.zig:81-112)
TWIN_SHAPES = (
    ("ctx256", 256, 4, 2, 32, 2000),
    ("ctx512", 512, 4, 2, 32, 1000),
    ("ctx1024", 1024, 4, 2, 32, 300),
    ("ctx2048", 2048, 4, 2, 32, 80),
    ("ctx4096", 4096, 4, 2, 32, 20),
    ("llama3-T256", 256, 32, 8, 128, 50),
    ("llama3-T512", 512, 32, 8, 128, 10),
    ("gqa-96-T256", 256, 32, 8, 96, 50),
    ("gqa-96-T512", 512, 32, 8, 96, 10),
    ("mha-192-T256", 256, 16, 16, 192, 50),
    ("gqa-256-T256", 256, 8, 4, 256, 50),
)

SEEDS = {"q": 0xBEEF, "k": 0x1234, "v": 0x5678, "dout": 0x9ABC}


def rising_scores(q, k, v, dout, head_dim):
    """A transform for write_twin_dir: every score grows with the key's position, by more than 2^8 from one
    64-key tile to the next (q shifted to positive values, k[s] raised in proportion to s).  A forward that
    moves its running maximum lazily moves it in every tile on such data, which is what a negative control for
    the maximum's correction needs; on the reference's own fill the maximum settles in the first tile."""
    step = 12.0 / (64.0 * head_dim ** 0.5 * 1.4427)  # per key: 12 in log2 units per 64 keys at mean(q) = 1
    rise = (np.arange(k.shape[0], dtype=np.float32) * np.float32(step))[:, None]
    return q + np.float32(1.0), k + rise, v, dout


def write_twin_dir(path: str, shapes=TWIN_SHAPES, threads: int = 0, transform=None) -> list[str]:
    """Writes manifest.tsv and the eight blobs of every shape into `path`; returns the tags.
    transform(q, k, v, dout, head_dim) -> (q, k, v, dout), when given, reshapes the reference's fill."""
    os.makedirs(path, exist_ok=True)
    threads = threads or max(1, len(os.sched_getaffinity(0)))
    rows = []
    for tag, T, H, Hkv, D, iters in shapes:
        q = oracle.fill_lcg(T * H * D, SEEDS["q"]).reshape(T, H * D)
        k = oracle.fill_lcg(T * Hkv * D, SEEDS["k"]).reshape(T, Hkv * D)
        v = oracle.fill_lcg(T * Hkv * D, SEEDS["v"]).reshape(T, Hkv * D)
        dout = oracle.fill_lcg(T * H * D, SEEDS["dout"]).reshape(T, H * D)
        if transform is not None:
            q, k, v, dout = (np.ascontiguousarray(x, dtype=np.float32) for x in transform(q, k, v, dout, D))
        best = float("inf")
        y = None
        for _ in range(3):
            t0 = time.perf_counter()
            y = oracle.attention_forward(q, k, v, H, Hkv, D, threads=threads)
            best = min(best, time.perf_counter() - t0)
        dq, dk, dv = oracle.attention_backward(q, k, v, dout, H, Hkv, D, threads=threads)
        for name, arr in (("q", q), ("k", k), ("v", v), ("y", y), ("dout", dout), ("dq", dq), ("dk", dk), ("dv", dv)):
            np.ascontiguousarray(arr, dtype="<f4").tofile(os.path.join(path, f"{tag}.{name}.bin"))
        rows.append(f"{tag} {T} {H} {Hkv} {D} {iters} {best * 1e6:.6f}\n")
    with open(os.path.join(path, "manifest.tsv"), "w") as f:
        f.writelines(rows)
    return [s[0] for s in shapes]


if __name__ == "__main__":
    import sys
    print(write_twin_dir(sys.argv[1]))
