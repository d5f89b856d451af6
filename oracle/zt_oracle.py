"""ctypes binding of the CPU oracle (oracle/zt_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
module; the shipped library never does.  Arrays are numpy float32, C-contiguous.
The functions mirror the reference's Zig API closely enough that the tests read
like the reference's own: errors come back as exceptions named after the Zig
error values (src/attention.zig:71-79, src/kv_cache.zig Error, src/cuda/device.zig Error).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libzt_oracle.so")


class InvalidHeadConfig(Exception):
    pass


class DimensionMismatch(Exception):
    pass


class Full(Exception):
    pass


class ShapeTooLarge(Exception):
    pass


class DegenerateShape(Exception):
    pass


class OddHeadDim(Exception):
    """error.OddHeadDim (src/rope.zig:28)."""


_ERR = {1: InvalidHeadConfig, 2: DimensionMismatch, 3: MemoryError, 4: Full, 5: ShapeTooLarge,
        6: DegenerateShape, 7: OddHeadDim}


def build(force: bool = False) -> str:
    """Compile the oracle with gcc if the shared object is missing or stale."""
    src = os.path.join(_HERE, "zt_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(
            ["gcc", "-O3", "-fno-fast-math", "-ffp-contract=off", "-fopenmp", "-fPIC", "-Wall",
             "-Wextra", "-std=c11", "-shared", "-o", _SO, src, "-lm"])
    return _SO


_lib = None
_fp = C.POINTER(C.c_float)
_sz = C.c_size_t


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.zto_attention_forward.argtypes = [_fp, _sz, _sz, _fp, _sz, _sz, _fp, _sz, _sz, _sz, _sz,
                                               _sz, _fp, _fp, C.c_int]
        _lib.zto_attention_forward_at.argtypes = [_fp, _fp, _fp, _fp, _fp, _sz, _sz, _sz, _sz, _sz,
                                                  _sz, C.c_int]
        _lib.zto_attn_step.argtypes = [_fp, _sz, _fp, _fp, _sz, _sz, _sz, _sz, _sz, _sz, _fp, _fp,
                                       C.c_int]
        _lib.zto_attention_backward.argtypes = [_fp, _sz, _sz, _fp, _sz, _sz, _fp, _sz, _sz, _fp, _sz,
                                                _sz, _sz, _sz, _sz, _fp, _fp, _fp, C.c_int]
        _lib.zto_attention_backward_kv_group.argtypes = [_fp, _fp, _fp, _fp, _sz, _sz, _sz, _sz, _sz,
                                                         _fp, _fp, _fp]
        _lib.zto_backward_window.argtypes = [_fp, _fp, _fp, _fp, _sz, _sz, _sz, _sz, _sz, C.POINTER(_sz), _sz, _sz,
                                             _fp, _fp, _fp, C.c_int]
        _lib.zto_matmul.argtypes = [_fp, _sz, _sz, _fp, _sz, _sz, _fp, C.c_int]
        _lib.zto_input_grad.argtypes = [_fp, _fp, _sz, _sz, _fp, _sz, _sz, C.c_int]
        _lib.zto_weight_grad.argtypes = [_fp, _fp, _sz, _sz, _fp, _sz, C.c_int]
        _lib.zto_attention_forward_rows.argtypes = [_fp, _fp, _fp, _fp, _fp, _sz, _sz, _sz, _sz, _sz,
                                                    _sz, _sz]
        _lib.zto_sampled_step.argtypes = [_fp] * 8 + [_sz] * 7 + [C.c_int, C.c_int,
                                                               C.POINTER(C.c_double)]
        _lib.zto_bytes_for.argtypes = [C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64,
                                       C.POINTER(C.c_uint64)]
        _lib.zto_forward_bounds.argtypes = [C.c_int] * 4
        _lib.zto_fill_lcg.argtypes = [_fp, _sz, C.c_uint32]
        _lib.zto_fill_lcg.restype = None
        _lib.zto_fill_hash.argtypes = [C.c_uint64]
        _lib.zto_fill_hash.restype = C.c_float
        _lib.zto_fill_normal.argtypes = [_fp, _sz, C.c_uint64, C.c_uint64, C.c_uint64]
        _lib.zto_fill_normal.restype = None
        _lib.zto_rope_forward.argtypes = [_fp, _sz, _sz, _sz, C.c_double, _sz, _fp]
        _lib.zto_rope_backward.argtypes = [_fp, _sz, _sz, _sz, C.c_double, _sz, _fp]
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise _ERR.get(rc, RuntimeError)(f"oracle error {rc}")


def _f32(a) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def _p(a: np.ndarray):
    return a.ctypes.data_as(_fp)


def _2d(a):
    a = _f32(a)
    if a.ndim != 2:
        raise ValueError("expected a [rows, cols] array")
    return a


def attention_forward(q, k, v, n_heads: int, n_kv_heads: int, head_dim: int, *, want_lse=False,
                      threads: int = 1):
    """attention.forward (src/attention.zig:36-153). Returns out, or (out, lse)."""
    q, k, v = _2d(q), _2d(k), _2d(v)
    out = np.zeros((q.shape[0], n_heads * head_dim), dtype=np.float32)
    lse = np.zeros((q.shape[0], n_heads), dtype=np.float32) if want_lse else None
    _check(lib().zto_attention_forward(_p(q), q.shape[0], q.shape[1], _p(k), k.shape[0], k.shape[1],
                                       _p(v), v.shape[0], v.shape[1], n_heads, n_kv_heads, head_dim,
                                       _p(out), _p(lse) if want_lse else None, threads))
    return (out, lse) if want_lse else out


def attention_forward_at(q, k, v, n_heads, n_kv_heads, head_dim, q_offset, n_keys, *,
                         want_lse=False, threads=1):
    """The C ABI's q_offset/n_keys forward on the CPU (src/cuda/attn_kernels.cu:276-321)."""
    q, k, v = _2d(q), _2d(k), _2d(v)
    T = q.shape[0]
    assert q.shape[1] == n_heads * head_dim and k.shape[1] == n_kv_heads * head_dim
    assert k.shape[0] >= n_keys and v.shape[0] >= n_keys
    out = np.zeros((T, n_heads * head_dim), dtype=np.float32)
    lse = np.zeros((T, n_heads), dtype=np.float32) if want_lse else None
    _check(lib().zto_attention_forward_at(_p(q), _p(k), _p(v), _p(out),
                                          _p(lse) if want_lse else None, T, n_heads, n_kv_heads,
                                          head_dim, q_offset, n_keys, threads))
    return (out, lse) if want_lse else out


def attention_backward(q, k, v, dout, n_heads, n_kv_heads, head_dim, *, threads=1):
    """autograd.attentionBackward (src/autograd.zig:636-842). Returns dq, dk, dv."""
    q, k, v, dout = _2d(q), _2d(k), _2d(v), _2d(dout)
    dq = np.zeros_like(q)
    dk = np.zeros_like(k)
    dv = np.zeros_like(v)
    _check(lib().zto_attention_backward(_p(q), q.shape[0], q.shape[1], _p(k), k.shape[0], k.shape[1],
                                        _p(v), v.shape[0], v.shape[1], _p(dout), dout.shape[0],
                                        dout.shape[1], n_heads, n_kv_heads, head_dim, _p(dq), _p(dk),
                                        _p(dv), threads))
    return dq, dk, dv


def attention_backward_kv_group(q, k, v, dout, n_heads, n_kv_heads, head_dim, kv):
    """One KV head's share of attentionBackward; other columns come back as zeros."""
    q, k, v, dout = _2d(q), _2d(k), _2d(v), _2d(dout)
    dq, dk, dv = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
    _check(lib().zto_attention_backward_kv_group(_p(q), _p(k), _p(v), _p(dout), q.shape[0], n_heads,
                                                 n_kv_heads, head_dim, kv, _p(dq), _p(dk), _p(dv)))
    return dq, dk, dv


def backward_window(q, k, v, dout, n_heads, n_kv_heads, head_dim, kv, rows, window, *, threads=1):
    """attentionBackward of KV head `kv` where a long sequence can afford it: dq of the query rows in
    `rows` for the group's heads ([len(rows), group, D]) and dk, dv of the last `window` keys
    ([window, D] each), in the reference's arithmetic and accumulation order."""
    q, k, v, dout = _2d(q), _2d(k), _2d(v), _2d(dout)
    group = n_heads // n_kv_heads
    rows_a = (_sz * len(rows))(*[int(r) for r in rows])
    dq_rows = np.zeros((len(rows), group, head_dim), dtype=np.float32)
    dk_win = np.zeros((window, head_dim), dtype=np.float32)
    dv_win = np.zeros((window, head_dim), dtype=np.float32)
    _check(lib().zto_backward_window(_p(q), _p(k), _p(v), _p(dout), q.shape[0], n_heads, n_kv_heads, head_dim, kv,
                                     rows_a, len(rows), window, _p(dq_rows), _p(dk_win), _p(dv_win), threads))
    return dq_rows, dk_win, dv_win


def attention_forward_rows(q, k, v, n_heads, n_kv_heads, head_dim, h, t0, t1):
    """Rows [t0, t1) of head h of attention.forward; returns ([t1-t0, D], [t1-t0])."""
    q, k, v = _2d(q), _2d(k), _2d(v)
    out = np.zeros_like(q)
    lse = np.zeros((q.shape[0], n_heads), dtype=np.float32)
    _check(lib().zto_attention_forward_rows(_p(q), _p(k), _p(v), _p(out), _p(lse), q.shape[0],
                                            n_heads, n_kv_heads, head_dim, h, t0, t1))
    return out[t0:t1, h * head_dim:(h + 1) * head_dim].copy(), lse[t0:t1, h].copy()


def sampled_step(q, k, v, dout, n_heads, n_kv_heads, head_dim, row_stride, row_phase, *,
                 backward=True, threads=1):
    """Every row_stride-th query row of a [B, T, ...] forward(+backward) pass; returns the
    reference's operation count for the rows computed and the partially filled outputs."""
    q, k, v, dout = (_f32(x) for x in (q, k, v, dout))
    B, T = q.shape[0], q.shape[1]
    out, dq, dk, dv = np.zeros_like(q), np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
    flops = C.c_double(0.0)
    _check(lib().zto_sampled_step(_p(q), _p(k), _p(v), _p(dout), _p(out), _p(dq), _p(dk), _p(dv), B, T,
                                  n_heads, n_kv_heads, head_dim, row_stride, row_phase,
                                  1 if backward else 0, threads, C.byref(flops)))
    return flops.value, out, dq, dk, dv


class Layer:
    """kv_cache.Layer (src/kv_cache.zig:60-135): k, v [n_ctx, width] and a fill count."""

    def __init__(self, n_ctx: int, width: int):
        if n_ctx == 0 or width == 0:
            raise DimensionMismatch("kv_cache.Layer.init")
        self.k = np.zeros((n_ctx, width), dtype=np.float32)
        self.v = np.zeros((n_ctx, width), dtype=np.float32)
        self.len = 0

    def append(self, k_row, v_row) -> None:
        k_row, v_row = _f32(k_row).ravel(), _f32(v_row).ravel()
        if k_row.size != self.k.shape[1] or v_row.size != self.v.shape[1]:
            raise DimensionMismatch("kv_cache.Layer.append")
        if self.len >= self.k.shape[0]:
            raise Full("kv_cache.Layer.append")
        self.k[self.len] = k_row
        self.v[self.len] = v_row
        self.len += 1

    def visible(self) -> int:
        return self.len

    def bytes(self) -> int:
        return (self.k.size + self.v.size) * 4


def attn_step(q, layer: Layer, n_heads, n_kv_heads, head_dim, *, want_lse=False, threads=1):
    """decode.attnStep (src/decode.zig:326-392): q is [1, n_heads*head_dim]."""
    q = _2d(q)
    out = np.zeros((1, n_heads * head_dim), dtype=np.float32)
    lse = np.zeros((1, n_heads), dtype=np.float32) if want_lse else None
    _check(lib().zto_attn_step(_p(q), q.shape[1], _p(layer.k), _p(layer.v), layer.k.shape[1],
                               layer.v.shape[1], layer.visible(), n_heads, n_kv_heads, head_dim,
                               _p(out), _p(lse) if want_lse else None, threads))
    return (out, lse) if want_lse else out


def attn_step_raw(q, k_cache, v_cache, n_keys, n_heads, n_kv_heads, head_dim, *, threads=1):
    """attnStep over bare cache arrays [n_ctx, n_kv_heads*head_dim]; returns (out[H*D], lse[H])."""
    q = _f32(q).reshape(1, -1)
    k_cache, v_cache = _2d(k_cache), _2d(v_cache)
    out = np.zeros((n_heads * head_dim,), dtype=np.float32)
    lse = np.zeros((n_heads,), dtype=np.float32)
    _check(lib().zto_attn_step(_p(q), q.shape[1], _p(k_cache), _p(v_cache), k_cache.shape[1],
                               v_cache.shape[1], n_keys, n_heads, n_kv_heads, head_dim, _p(out),
                               _p(lse), threads))
    return out, lse


def matmul(a, b, *, threads=1) -> np.ndarray:
    """tensor.matmul (src/tensor.zig:78-106): f32 accumulation over ascending k."""
    a, b = _2d(a), _2d(b)
    out = np.zeros((a.shape[0], b.shape[1]), dtype=np.float32)
    _check(lib().zto_matmul(_p(a), a.shape[0], a.shape[1], _p(b), b.shape[0], b.shape[1], _p(out), threads))
    return out


def input_grad(dout, w, *, out=None, threads=1) -> np.ndarray:
    """inputGrad (src/autograd.zig:999-1022): out += dout . w^T; a fresh zero tensor when out is None."""
    dout, w = _2d(dout), _2d(w)
    if out is None:
        out = np.zeros((dout.shape[0], w.shape[0]), dtype=np.float32)
    _check(lib().zto_input_grad(_p(out), _p(dout), dout.shape[0], dout.shape[1], _p(w), w.shape[0], w.shape[1], threads))
    return out


def weight_grad(w_grad, inp, dout, *, threads=1) -> np.ndarray:
    """weightGrad (src/autograd.zig:958-972): w_grad += inp^T . dout, in place, rows in ascending order."""
    inp, dout = _2d(inp), _2d(dout)
    assert w_grad.dtype == np.float32 and w_grad.flags.c_contiguous and w_grad.shape == (inp.shape[1], dout.shape[1])
    _check(lib().zto_weight_grad(_p(w_grad), _p(inp), inp.shape[0], inp.shape[1], _p(dout), dout.shape[1], threads))
    return w_grad


KIND_QUERY_HEADED, KIND_KV_HEADED, KIND_PER_ROW = 0, 1, 2


def bytes_for(kind: int, t: int, n_heads: int, n_kv_heads: int, dim: int) -> int:
    """device.bytesFor (src/cuda/device.zig:162-171)."""
    out = C.c_uint64(0)
    _check(lib().zto_bytes_for(kind, t, n_heads, n_kv_heads, dim, C.byref(out)))
    return out.value


def forward_bounds(c_t: int, q_offset: int, n_keys: int, t: int) -> None:
    """device.forwardBounds (src/cuda/device.zig:489-501); raises ShapeTooLarge."""
    _check(lib().zto_forward_bounds(c_t, q_offset, n_keys, t))


def fill_lcg(n: int, seed: int) -> np.ndarray:
    """attn_twin.zig's fixture generator (src/cuda/attn_twin.zig:283-289)."""
    a = np.empty(n, dtype=np.float32)
    lib().zto_fill_lcg(_p(a), n, seed)
    return a


def fill_hash(i: int) -> float:
    """decode_test.zig's index hash (src/decode_test.zig:35-42)."""
    return float(lib().zto_fill_hash(i))


def fill_normal(shape, seed: int, stream: int, first: int = 0, out: np.ndarray | None = None):
    """i.i.d. N(0,1) f32: element i of a stream depends only on (seed, stream, first+i).

    Streams by convention: 0 q, 1 k, 2 v, 3 dout.
    """
    n = int(np.prod(shape))
    a = out if out is not None else np.empty(n, dtype=np.float32)
    lib().zto_fill_normal(a.ctypes.data_as(_fp), n, seed, stream, first)
    return a.reshape(shape)


ROPE_THETA = 500000.0  # model.rope_theta (src/model.zig:23)


def rope_forward(x, pos: int, head_dim: int, theta: float = ROPE_THETA) -> np.ndarray:
    """rope.forward (src/rope.zig:21-55): row r of x [rows, heads * head_dim] rotated to position pos + r."""
    x = _2d(x)
    out = np.empty_like(x)
    _check(lib().zto_rope_forward(_p(x), x.shape[0], x.shape[1], pos, theta, head_dim, _p(out)))
    return out


def rope_backward(dout, pos: int, head_dim: int, theta: float = ROPE_THETA) -> np.ndarray:
    """ropeBackward (src/autograd.zig:851-874): the gradient of rope_forward's input from that of its output."""
    dout = _2d(dout)
    din = np.empty_like(dout)
    _check(lib().zto_rope_backward(_p(dout), dout.shape[0], dout.shape[1], pos, theta, head_dim, _p(din)))
    return din
