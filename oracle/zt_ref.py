"""The reference's own CUDA attention library, compiled from where it lies.  TEST INFRASTRUCTURE ONLY.

What this is for: the reference holds no literal vectors for dq, dk, dv (its backward is pinned by
whole-model finite differences and by its GPU harness against the Zig CPU code).  Its CUDA kernels
(src/cuda/attn_kernels.cu:197-634) WERE graded by the reference against the real
attention.forward / autograd.attentionBackward, at <= 8.4e-7 (outputs/bench/run-attn.log:36-46),
and they compile here although the Zig code does not.  Outputs of those kernels are therefore
vectors the reference itself made, and the CPU restatement in zt_oracle.c is pinned against them.

build():  nvcc on the reference's two source files in place -> oracle/_ref/ (never copied into
          this repository; oracle/_ref/ is ignored by git and travels to the GPU machine as built
          files).  Needs the reference tree; a no-op without it.
Ref:      ctypes binding of the six `zt_attn_*` symbols of oracle/_ref/libattn_ref.so, called with
          torch device pointers.  Used by tests/golden/make_ref_fixtures.py only.
"""
from __future__ import annotations

import ctypes as C
import os
import shutil
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref")
REF_LIB = os.path.join(REF_DIR, "libattn_ref.so")
REF_HARNESS = os.path.join(REF_DIR, "attn_ref")
REFERENCE_ROOT = os.environ.get("ZT_REFERENCE_ROOT", "/root/reference")


def _nvcc() -> str | None:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def build(force: bool = False) -> bool:
    """Compile the reference's library object and its harness program into oracle/_ref/.

    libattn_ref.so: src/cuda/attn_kernels.cu as a shared library (its `extern "C"` block, :641-1038).
    attn_ref:       src/cuda/attn.cu, the reference's harness `main` (:683), which #includes the kernels.
    Returns True when both exist afterwards."""
    src_dir = os.path.join(REFERENCE_ROOT, "src", "cuda")
    kern, harness = os.path.join(src_dir, "attn_kernels.cu"), os.path.join(src_dir, "attn.cu")
    nvcc = _nvcc()
    if nvcc and os.path.exists(kern) and os.path.exists(harness):
        os.makedirs(REF_DIR, exist_ok=True)
        if force or not os.path.exists(REF_LIB):
            subprocess.check_call([nvcc, "-arch=sm_100", "-O2", "-shared", "-Xcompiler", "-fPIC", "-o", REF_LIB, kern])
        if force or not os.path.exists(REF_HARNESS):
            subprocess.check_call([nvcc, "-arch=sm_100", "-O2", "-o", REF_HARNESS, harness])
    return os.path.exists(REF_LIB) and os.path.exists(REF_HARNESS)


class Ref:
    """The reference library's entry points (signatures: src/cuda/device.zig:58-105)."""

    def __init__(self):
        if not os.path.exists(REF_LIB):
            raise FileNotFoundError(f"{REF_LIB}: build it where the reference tree is (zt_ref.build())")
        self.lib = C.CDLL(REF_LIB)
        vp, ci = C.c_void_p, C.c_int
        self.lib.zt_attn_forward.argtypes = [vp] * 4 + [ci] * 8 + [vp]
        self.lib.zt_attn_backward.argtypes = [vp] * 10 + [ci] * 5 + [vp]

    def forward(self, q, k, v, n_heads, n_kv_heads, dim, q_offset=0, n_keys=None, group_q=1, max_tile=64):
        """zt_attn_forward on torch CUDA tensors q [T, H*D], k, v [>= n_keys, Hkv*D]; returns out."""
        import torch
        T = q.shape[0]
        n_keys = k.shape[0] if n_keys is None else n_keys
        out = torch.empty_like(q)
        rc = self.lib.zt_attn_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), T, n_heads, n_kv_heads,
                                      dim, group_q, max_tile, q_offset, n_keys, None)
        torch.cuda.synchronize()
        if rc != 0:
            raise RuntimeError("the reference's zt_attn_forward refused the call")
        return out

    def backward(self, q, k, v, dout, n_heads, n_kv_heads, dim, max_tile=64):
        """zt_attn_backward; returns dq, dk, dv."""
        import torch
        T = q.shape[0]
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        rows = [torch.empty(T * n_heads, dtype=torch.float32, device=q.device) for _ in range(3)]
        rc = self.lib.zt_attn_backward(q.data_ptr(), k.data_ptr(), v.data_ptr(), dout.data_ptr(), dq.data_ptr(),
                                       dk.data_ptr(), dv.data_ptr(), rows[0].data_ptr(), rows[1].data_ptr(),
                                       rows[2].data_ptr(), T, n_heads, n_kv_heads, dim, max_tile, None)
        torch.cuda.synchronize()
        if rc != 0:
            raise RuntimeError("the reference's zt_attn_backward refused the call")
        return dq, dk, dv


if __name__ == "__main__":
    print("built" if build(force=True) else "reference tree or nvcc missing: nothing built")
