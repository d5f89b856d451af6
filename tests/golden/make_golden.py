"""Writes tests/golden/*.npz from the CPU oracle (oracle/zt_oracle.c).

The reference is Zig and cannot run beside this script, so these vectors are the
oracle's own outputs on the reference's fixture generator (32-bit LCG, seeds
0xbeef/0x1234/0x5678/0x9abc, src/cuda/attn_twin.zig:162-164,211,283-289).  They
freeze the oracle (tests/test_golden.py re-derives them) and give the GPU tests a
target that needs no CPU recomputation.  Run:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import zt_oracle as oracle  # noqa: E402

# tag, T, n_heads, n_kv_heads, head_dim: the twin's geometries (attn_twin.zig:82-111) at a T that
# keeps each file small.
CASES = [
    ("ctx256", 256, 4, 2, 32),      # the GPT-mini shape itself, full size
    ("llama3-T32", 32, 32, 8, 128),
    ("gqa-96-T24", 24, 32, 8, 96),
    ("mha-192-T24", 24, 16, 16, 192),
    ("gqa-256-T17", 17, 8, 4, 256),
]


def inputs(T, H, Hkv, D):
    q = oracle.fill_lcg(T * H * D, 0xBEEF).reshape(T, H * D)
    k = oracle.fill_lcg(T * Hkv * D, 0x1234).reshape(T, Hkv * D)
    v = oracle.fill_lcg(T * Hkv * D, 0x5678).reshape(T, Hkv * D)
    do = oracle.fill_lcg(T * H * D, 0x9ABC).reshape(T, H * D)
    return q, k, v, do


def main():
    for tag, T, H, Hkv, D in CASES:
        q, k, v, do = inputs(T, H, Hkv, D)
        y, lse = oracle.attention_forward(q, k, v, H, Hkv, D, want_lse=True)
        dq, dk, dv = oracle.attention_backward(q, k, v, do, H, Hkv, D)
        np.savez_compressed(os.path.join(HERE, f"{tag}.npz"), shape=np.array([T, H, Hkv, D]),
                            y=y, lse=lse, dq=dq, dk=dk, dv=dv)
        print(tag, "written")


if __name__ == "__main__":
    main()
