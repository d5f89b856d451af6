"""The committed golden vectors still are what the oracle computes (CPU only)."""
import glob
import importlib.util
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)


@pytest.mark.parametrize("tag,T,H,Hkv,D", make_golden.CASES)
def test_golden_vectors_match_the_oracle(oracle, tag, T, H, Hkv, D):
    g = np.load(os.path.join(HERE, "golden", f"{tag}.npz"))
    assert list(g["shape"]) == [T, H, Hkv, D]
    q, k, v, do = make_golden.inputs(T, H, Hkv, D)
    y, lse = oracle.attention_forward(q, k, v, H, Hkv, D, want_lse=True, threads=4)
    dq, dk, dv = oracle.attention_backward(q, k, v, do, H, Hkv, D, threads=4)
    for name, got in (("y", y), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
        assert np.array_equal(g[name].view(np.uint32), got.view(np.uint32)), name


def test_every_golden_file_has_a_case():
    files = {os.path.basename(f)[:-4] for f in glob.glob(os.path.join(HERE, "golden", "*.npz"))}
    assert files == {c[0] for c in make_golden.CASES}
