"""Thin wrappers that hand torch CUDA tensors to the C ABI (include/zt_attn.h).

Each function checks shapes the way the reference's CPU functions do
(src/attention.zig:71-79, src/autograd.zig:659-685, src/decode.zig:338-350) and
raises the mirror of the Zig error; the arithmetic happens only in libztattn.
"""
from __future__ import annotations

from . import lib as _lib
from .device import ConfigRefused


class InvalidHeadConfig(Exception):
    """error.InvalidHeadConfig (src/attention.zig:71-73)."""


class DimensionMismatch(Exception):
    """error.DimensionMismatch (src/attention.zig:74-79)."""


def _stream(t):
    import torch
    return torch.cuda.current_stream(t.device).cuda_stream


def _need_cuda_f32(*tensors):
    import torch
    for x in tensors:
        if x is None:
            continue
        if not x.is_cuda:
            raise RuntimeError("libztattn has no CPU path: tensors must live on a CUDA device")
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise DimensionMismatch("tensors must be contiguous float32")


def _head_config(n_heads, n_kv_heads, head_dim):
    if n_kv_heads == 0 or head_dim == 0 or n_heads % n_kv_heads != 0:
        raise InvalidHeadConfig(f"{n_heads}/{n_kv_heads} heads, head_dim {head_dim}")


class BackwardWorkspace:
    """Caller-owned scratch of the batched backward for one (batch, T, heads, dim) shape.  Handed to
    attention_forward as `keep`, it also carries the forward's operand planes of q, k, v over to the backward."""

    def __init__(self, batch, t, n_heads, n_kv_heads, head_dim, device="cuda"):
        import torch
        self.shape = (batch, t, n_heads, n_kv_heads, head_dim)
        self.nbytes = int(_lib.load().zt_attn_backward_workspace_bytes(*self.shape))
        self.buf = torch.empty(max(self.nbytes, 16), dtype=torch.uint8, device=device)
        self.token = 0  # of the planes the last forward(keep=self) left here; 0: none


def attention_forward(q, k, v, n_heads, n_kv_heads, head_dim, *, want_lse=False, keep=None):
    """Batched attention.forward.  q [B, T, H*D] (or [T, H*D]); returns out (and lse [B, T, H]).
    keep: a BackwardWorkspace of this shape; the forward's operand planes of q, k, v are left in it, and a
    backward given it with kept=True (the caller's word that q, k, v were not written in between) skips
    converting them again."""
    import torch
    _head_config(n_heads, n_kv_heads, head_dim)
    squeeze = q.dim() == 2
    if squeeze:
        q, k, v = q[None], k[None], v[None]
    _need_cuda_f32(q, k, v)
    B, T = q.shape[0], q.shape[1]
    if (k.shape[0] != B or v.shape[0] != B or k.shape[1] != T or v.shape[1] != T
            or k.shape[2] != n_kv_heads * head_dim or v.shape[2] != k.shape[2]
            or q.shape[2] != n_heads * head_dim):
        raise DimensionMismatch("q/k/v shapes disagree with the head configuration")
    out = torch.empty_like(q)
    lse = torch.empty((B, T, n_heads), dtype=torch.float32, device=q.device) if want_lse else None
    if T == 0:
        return (out[0] if squeeze else out, lse) if want_lse else (out[0] if squeeze else out)
    if keep is not None and keep.shape != (B, T, n_heads, n_kv_heads, head_dim):
        raise DimensionMismatch("the workspace was sized for another shape")
    with torch.cuda.device(q.device):
        if keep is not None:
            import ctypes
            token = ctypes.c_ulonglong(0)
            rc = _lib.load().zt_attn_forward_batched_keep(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr() if want_lse else None,
                keep.buf.data_ptr() if keep.nbytes else None, keep.nbytes, B, T, n_heads, n_kv_heads, head_dim,
                _stream(q), ctypes.byref(token))
            keep.token = token.value
        else:
            rc = _lib.load().zt_attn_forward_batched(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                lse.data_ptr() if want_lse else None, B, T, n_heads, n_kv_heads, head_dim, _stream(q))
    if rc != 0:
        raise ConfigRefused(_lib.last_error())
    if squeeze:
        out = out[0]
        lse = lse[0] if want_lse else None
    return (out, lse) if want_lse else out


def attention_backward(q, k, v, out, lse, dout, n_heads, n_kv_heads, head_dim, *, workspace=None, kept=False):
    """Batched autograd.attentionBackward from the forward's out and lse; returns dq, dk, dv.
    workspace: a BackwardWorkspace of this shape (one is allocated per call otherwise).
    kept: the workspace was the `keep` of the forward of these very q, k, v and they have not been written
    since: the backward then uses the planes the forward left there (refused if they are gone)."""
    import torch
    _head_config(n_heads, n_kv_heads, head_dim)
    squeeze = q.dim() == 2
    if squeeze:
        q, k, v, out, lse, dout = q[None], k[None], v[None], out[None], lse[None], dout[None]
    _need_cuda_f32(q, k, v, out, lse, dout)
    B, T = q.shape[0], q.shape[1]
    if (k.shape[0] != B or v.shape[0] != B or k.shape[1] != T or v.shape[1] != T
            or k.shape[2] != n_kv_heads * head_dim or v.shape[2] != k.shape[2] or q.shape[2] != n_heads * head_dim):
        raise DimensionMismatch("q/k/v shapes disagree with the head configuration")
    if dout.shape != q.shape or out.shape != q.shape or lse.shape != (B, T, n_heads):
        raise DimensionMismatch("dout/out/lse shapes disagree with q")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    delta = torch.empty_like(lse)
    L = _lib.load()
    if workspace is not None:
        if workspace.shape != (B, T, n_heads, n_kv_heads, head_dim):
            raise DimensionMismatch("the workspace was sized for another shape")
        ws_bytes, ws = workspace.nbytes, (workspace.buf if workspace.nbytes else None)
    else:
        ws_bytes = L.zt_attn_backward_workspace_bytes(B, T, n_heads, n_kv_heads, head_dim)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=q.device) if ws_bytes else None
    token = 0
    if kept:
        if workspace is None:
            raise DimensionMismatch("kept=True needs the workspace the forward kept its planes in")
        token, workspace.token = workspace.token, 0
    with torch.cuda.device(q.device):
        rc = L.zt_attn_backward_batched_kept(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), dout.data_ptr(),
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr(),
            ws.data_ptr() if ws is not None else None, ws_bytes, B, T, n_heads, n_kv_heads, head_dim,
            _stream(q), token)
    if rc != 0:
        raise ConfigRefused(_lib.last_error())
    if squeeze:
        return dq[0], dk[0], dv[0]
    return dq, dk, dv


ROPE_THETA = 500000.0  # model.rope_theta (src/model.zig:23)


class RopeWorkspace:
    """Caller-owned scratch of the rope calls for one (batch, T, heads, dim) shape."""

    def __init__(self, batch, t, n_heads, n_kv_heads, head_dim, device="cuda"):
        import torch
        self.shape = (batch, t, n_heads, n_kv_heads, head_dim)
        self.nbytes = int(_lib.load().zt_attn_rope_workspace_bytes(*self.shape))
        if self.nbytes == 0:
            raise ConfigRefused("the shape is not admissible")
        self.buf = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.token = 0  # of the planes the last rope forward left here; 0: none


def _rope_args(q, k, v, n_heads, n_kv_heads, head_dim, workspace):
    _head_config(n_heads, n_kv_heads, head_dim)
    _need_cuda_f32(q, k, v)
    if q.dim() != 3:
        raise DimensionMismatch("the rope calls take [B, T, width] tensors")
    B, T = q.shape[0], q.shape[1]
    if (k.shape[:2] != (B, T) or v.shape != k.shape or k.shape[2] != n_kv_heads * head_dim
            or q.shape[2] != n_heads * head_dim):
        raise DimensionMismatch("q/k/v shapes disagree with the head configuration")
    if workspace is None:
        workspace = RopeWorkspace(B, T, n_heads, n_kv_heads, head_dim, q.device)
    elif workspace.shape != (B, T, n_heads, n_kv_heads, head_dim):
        raise DimensionMismatch("the workspace was sized for another shape")
    return B, T, workspace


def attention_forward_rope(q, k, v, n_heads, n_kv_heads, head_dim, *, pos=0, theta=ROPE_THETA, workspace=None,
                           want_lse=False):
    """attention.forward over rope.forward(q), rope.forward(k) (src/model.zig:372-375): q, k are the
    unrotated projections [B, T, width]; row r sits at position pos + r."""
    import torch
    B, T, workspace = _rope_args(q, k, v, n_heads, n_kv_heads, head_dim, workspace)
    out = torch.empty_like(q)
    lse = torch.empty((B, T, n_heads), dtype=torch.float32, device=q.device) if want_lse else None
    import ctypes
    token = ctypes.c_ulonglong(0)
    with torch.cuda.device(q.device):
        rc = _lib.load().zt_attn_forward_rope_batched(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr() if want_lse else None,
            workspace.buf.data_ptr(), workspace.nbytes, B, T, n_heads, n_kv_heads, head_dim, pos, theta, _stream(q),
            ctypes.byref(token))
    workspace.token = token.value
    if rc != 0:
        raise ConfigRefused(_lib.last_error())
    return (out, lse) if want_lse else out


def attention_backward_rope(q, k, v, out, lse, dout, n_heads, n_kv_heads, head_dim, *, pos=0, theta=ROPE_THETA,
                            workspace=None, kept=False):
    """Gradients of the unrotated q and k (and of v): autograd.attentionBackward followed by
    ropeBackward (src/autograd.zig:559-569,851-874).  kept: as in attention_backward, for the workspace of the
    rope forward of these q, k, v at this pos and theta."""
    import torch
    B, T, workspace = _rope_args(q, k, v, n_heads, n_kv_heads, head_dim, workspace)
    _need_cuda_f32(out, lse, dout)
    if dout.shape != q.shape or out.shape != q.shape or lse.shape != (B, T, n_heads):
        raise DimensionMismatch("dout/out/lse shapes disagree with q")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    delta = torch.empty_like(lse)
    token = 0
    if kept:
        token, workspace.token = workspace.token, 0
    with torch.cuda.device(q.device):
        rc = _lib.load().zt_attn_backward_rope_batched(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), dout.data_ptr(),
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr(), workspace.buf.data_ptr(), workspace.nbytes,
            B, T, n_heads, n_kv_heads, head_dim, pos, theta, _stream(q), token)
    if rc != 0:
        raise ConfigRefused(_lib.last_error())
    return dq, dk, dv


class ProjWorkspace:
    """Caller-owned scratch of the projection calls for one (batch, T, k, n) shape."""

    def __init__(self, batch, t, k, n, device="cuda"):
        import torch
        self.shape = (batch, t, k, n)
        self.nbytes = int(_lib.load().zt_proj_workspace_bytes(batch, t, k, n))
        self.buf = torch.empty(max(self.nbytes, 16), dtype=torch.uint8, device=device)


def _proj_args(ctx, wo, workspace):
    _need_cuda_f32(ctx, wo)
    if ctx.dim() != 3 or wo.dim() != 2 or ctx.shape[2] != wo.shape[0] or wo.device != ctx.device:
        raise DimensionMismatch("the projection takes ctx [B, T, k] and wo [k, n] on one device")
    B, T, k = ctx.shape
    n = wo.shape[1]
    if workspace is None:
        workspace = ProjWorkspace(B, T, k, n, ctx.device)
    elif workspace.shape != (B, T, k, n):
        raise DimensionMismatch("the workspace was sized for another shape")
    return B, T, k, n, workspace


def proj_forward(ctx, wo, *, workspace=None):
    """tensor.matmul(ctx, l.wo) (src/model.zig:396) for a batch: ctx [B, T, k], wo [k, n] -> y [B, T, n]."""
    import torch
    B, T, k, n, workspace = _proj_args(ctx, wo, workspace)
    y = torch.empty((B, T, n), dtype=torch.float32, device=ctx.device)
    with torch.cuda.device(ctx.device):
        rc = _lib.load().zt_proj_forward(ctx.data_ptr(), wo.data_ptr(), y.data_ptr(), workspace.buf.data_ptr(),
                                         workspace.nbytes, B, T, k, n, _stream(ctx))
    if rc != 0:
        raise ConfigRefused(_lib.last_error())
    return y


def proj_backward(ctx, wo, dy, dwo, *, workspace=None):
    """The projection's gradients (src/autograd.zig:553-557): returns dctx = dy . wo^T and ADDS ctx^T . dy into the
    caller's dwo [k, n] (weightGrad accumulates into the layer's gradient)."""
    import torch
    B, T, k, n, workspace = _proj_args(ctx, wo, workspace)
    _need_cuda_f32(dy, dwo)
    if tuple(dy.shape) != (B, T, n) or tuple(dwo.shape) != (k, n) or dy.device != ctx.device or dwo.device != ctx.device:
        raise DimensionMismatch("dy must be [B, T, n] and dwo [k, n] on ctx's device")
    dctx = torch.empty_like(ctx)
    with torch.cuda.device(ctx.device):
        rc = _lib.load().zt_proj_backward(ctx.data_ptr(), wo.data_ptr(), dy.data_ptr(), dctx.data_ptr(), dwo.data_ptr(),
                                          workspace.buf.data_ptr(), workspace.nbytes, B, T, k, n, _stream(ctx))
    if rc != 0:
        raise ConfigRefused(_lib.last_error())
    return dctx


class AttentionBlock:
    """The attention part of a transformer block as a training step runs it, device-resident, over the C ABI:

        forward   ctx = attention(rope(q), rope(k), v)      (src/model.zig:372-393)
                  y   = ctx . wo                            (src/model.zig:396)
        backward  dctx = dy . wo^T, dwo += ctx^T . dy       (src/autograd.zig:553-557)
                  dq, dk, dv = ropeBackward(attentionBackward(...))   (src/autograd.zig:559-569)

    q, k are the projections before rope.forward; row r sits at position pos + r.  The reference's trainer calls
    attentionBackward at src/autograd.zig:559 on the CPU only (its CUDA backward has no call site); this is that
    call site for the device path.  All scratch is sized once, here; a step allocates only its outputs."""

    def __init__(self, batch, t, n_heads, n_kv_heads, head_dim, d_model, *, theta=ROPE_THETA, device="cuda"):
        _head_config(n_heads, n_kv_heads, head_dim)
        self.shape = (batch, t, n_heads, n_kv_heads, head_dim)
        self.d_model, self.theta = d_model, theta
        self.rope_ws = RopeWorkspace(batch, t, n_heads, n_kv_heads, head_dim, device)
        self.proj_ws = ProjWorkspace(batch, t, n_heads * head_dim, d_model, device)
        self.saved = None

    def forward(self, q, k, v, wo, *, pos=0, fused=True):
        """y = (attention(rope(q), rope(k), v)) . wo.  fused: one call of zt_attn_block_forward (the attention
        kernel's epilogue leaves ctx as the projection's operand planes); otherwise the two calls one after the
        other -- same numbers, one more pass over ctx."""
        import ctypes
        import torch
        B, T, H, Hkv, D = self.shape
        if not fused:
            ctx, lse = attention_forward_rope(q, k, v, H, Hkv, D, pos=pos, theta=self.theta, workspace=self.rope_ws,
                                              want_lse=True)
            y = proj_forward(ctx, wo, workspace=self.proj_ws)
        else:
            _, _, _ = _rope_args(q, k, v, H, Hkv, D, self.rope_ws)
            _need_cuda_f32(wo)
            if tuple(wo.shape) != (H * D, self.d_model) or wo.device != q.device:
                raise DimensionMismatch("wo must be [n_heads * head_dim, d_model] on q's device")
            ctx = torch.empty_like(q)
            lse = torch.empty((B, T, H), dtype=torch.float32, device=q.device)
            y = torch.empty((B, T, self.d_model), dtype=torch.float32, device=q.device)
            token = ctypes.c_ulonglong(0)
            with torch.cuda.device(q.device):
                rc = _lib.load().zt_attn_block_forward(
                    q.data_ptr(), k.data_ptr(), v.data_ptr(), wo.data_ptr(), ctx.data_ptr(), lse.data_ptr(), y.data_ptr(),
                    self.rope_ws.buf.data_ptr(), self.rope_ws.nbytes, self.proj_ws.buf.data_ptr(), self.proj_ws.nbytes,
                    B, T, H, Hkv, D, self.d_model, pos, self.theta, _stream(q), ctypes.byref(token))
            self.rope_ws.token = token.value
            if rc != 0:
                raise ConfigRefused(_lib.last_error())
        self.saved = (q, k, v, wo, ctx, lse, pos)
        return y

    def backward(self, dy, dwo):
        """Returns dq, dk, dv (of the unrotated q, k) and adds the projection's weight gradient into dwo.  The
        caller's word, as with kept=True elsewhere: q, k, v have not been written since forward()."""
        if self.saved is None:
            raise DimensionMismatch("backward() needs the forward() of the same step")
        q, k, v, wo, ctx, lse, pos = self.saved
        self.saved = None
        B, T, H, Hkv, D = self.shape
        dctx = proj_backward(ctx, wo, dy, dwo, workspace=self.proj_ws)
        return attention_backward_rope(q, k, v, ctx, lse, dctx, H, Hkv, D, pos=pos, theta=self.theta,
                                       workspace=self.rope_ws, kept=self.rope_ws.token != 0)


class DecodeWorkspace:
    """Caller-owned scratch of zt_attn_decode for one (batch, n_ctx, heads, dim) shape."""

    def __init__(self, batch, n_ctx, n_heads, n_kv_heads, head_dim, device="cuda"):
        import torch
        self.shape = (batch, n_ctx, n_heads, n_kv_heads, head_dim)
        self.nbytes = int(_lib.load().zt_attn_decode_workspace_bytes(*self.shape))
        if self.nbytes == 0:
            raise ConfigRefused("the decode shape is not admissible")
        self.buf = torch.empty(self.nbytes, dtype=torch.uint8, device=device)

    def bad_sequences(self) -> int:
        import ctypes
        n = ctypes.c_int(0)
        if _lib.load().zt_attn_decode_status(self.buf.data_ptr(), ctypes.byref(n)) != 0:
            raise RuntimeError(_lib.last_error())
        return n.value


def decode_attention(q, k_cache, v_cache, n_keys, n_heads, n_kv_heads, head_dim, *, workspace=None,
                     want_lse=False, out=None):
    """decode.attnStep for a batch: q [B, H*D], caches [B, n_ctx, Hkv*D], n_keys int32 [B]."""
    import torch
    _head_config(n_heads, n_kv_heads, head_dim)
    _need_cuda_f32(q, k_cache, v_cache)
    B, n_ctx = k_cache.shape[0], k_cache.shape[1]
    if (q.shape != (B, n_heads * head_dim) or k_cache.shape[2] != n_kv_heads * head_dim
            or v_cache.shape != k_cache.shape):
        raise DimensionMismatch("q/cache shapes disagree with the head configuration")
    if n_keys.dtype != torch.int32 or n_keys.shape != (B,) or not n_keys.is_cuda:
        raise DimensionMismatch("n_keys must be an int32 CUDA tensor of one count per sequence")
    if workspace is None:
        workspace = DecodeWorkspace(B, n_ctx, n_heads, n_kv_heads, head_dim, q.device)
    if out is None:
        out = torch.empty_like(q)
    else:
        _need_cuda_f32(out)
        if out.shape != q.shape or out.device != q.device:
            raise DimensionMismatch("out must be a [B, H*D] tensor on q's device")
    if k_cache.device != q.device or v_cache.device != q.device or n_keys.device != q.device:
        raise DimensionMismatch("q, the caches and n_keys must live on one device")
    lse = torch.empty((B, n_heads), dtype=torch.float32, device=q.device) if want_lse else None
    with torch.cuda.device(q.device):
        rc = _lib.load().zt_attn_decode(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), n_keys.data_ptr(), out.data_ptr(),
            lse.data_ptr() if want_lse else None, workspace.buf.data_ptr(), workspace.nbytes, B, n_ctx,
            n_heads, n_kv_heads, head_dim, _stream(q))
    if rc != 0:
        raise ConfigRefused(_lib.last_error())
    return (out, lse) if want_lse else out


class AttnPipeline:
    """Forward + backward of a run of equally shaped sequences whose tensors live in host memory.

    The reference's trainer drives device.Attn one sequence at a time: upload q, k, v (and dout),
    launch, download (src/model.zig:481-514), each step waiting for the one before.  On a PCIe
    link the copies take longer than the kernels, so this class runs the three stages on streams
    of their own over `slots` sets of device buffers: while sequence b is in the kernels, b+1 is
    on its way up and b-1 on its way down.  It calls the batched entry points (batch 1), which
    take the forward's out and log-sum-exp, so nothing is recomputed in the backward.

    Host tensors must be pinned for the copies to overlap; results are complete when step()
    returns.
    """

    def __init__(self, t, n_heads, n_kv_heads, head_dim, slots=2, device="cuda"):
        import torch
        _head_config(n_heads, n_kv_heads, head_dim)
        if slots < 1:
            raise DimensionMismatch("slots must be at least 1")
        self.shape = (t, n_heads, n_kv_heads, head_dim)
        self.device = torch.device(device)
        self.slots = slots
        L = _lib.load()
        self.ws_bytes = int(L.zt_attn_backward_workspace_bytes(1, t, n_heads, n_kv_heads, head_dim))
        wq, wkv = n_heads * head_dim, n_kv_heads * head_dim
        f32 = dict(dtype=torch.float32, device=self.device)
        self.buf = []
        for _ in range(slots):
            b = {name: torch.empty((t, wq), **f32) for name in ("q", "dout", "out", "dq")}
            b.update({name: torch.empty((t, wkv), **f32) for name in ("k", "v", "dk", "dv")})
            b["lse"] = torch.empty((t, n_heads), **f32)
            b["delta"] = torch.empty((t, n_heads), **f32)
            b["ws"] = torch.empty(max(self.ws_bytes, 16), dtype=torch.uint8, device=self.device)
            self.buf.append(b)
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        ev = lambda: [torch.cuda.Event() for _ in range(slots)]
        self.ready_f, self.ready_b = ev(), ev()  # q, k, v of the slot are on the device; dout is
        self.done_f, self.done = ev(), ev()      # the slot's forward has finished; its backward has
        self.free = ev()                         # the slot's outputs are on the host

    def step(self, q, k, v, dout, out, dq, dk, dv, lse=None):
        """q, dout, out, dq: host [B, T, H*D]; k, v, dk, dv: host [B, T, Hkv*D]; lse: host [B, T, H] or
        None.  Reads q, k, v, dout and fills out, dq, dk, dv (and lse)."""
        import ctypes
        import torch
        t, n_heads, n_kv_heads, head_dim = self.shape
        B = q.shape[0]
        wq, wkv = n_heads * head_dim, n_kv_heads * head_dim
        for x, w in ((q, wq), (dout, wq), (out, wq), (dq, wq), (k, wkv), (v, wkv), (dk, wkv), (dv, wkv)):
            if x.is_cuda or x.dtype != torch.float32 or tuple(x.shape) != (B, t, w) or not x.is_contiguous():
                raise DimensionMismatch("host tensors must be contiguous float32 [B, T, width]")
        if lse is not None and tuple(lse.shape) != (B, t, n_heads):
            raise DimensionMismatch("lse must be [B, T, H]")
        L = _lib.load()
        start = torch.cuda.Event()
        start.record(torch.cuda.current_stream(self.device))
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(start)
        with torch.cuda.device(self.device):
            for b in range(B):
                sl = b % self.slots
                d = self.buf[sl]
                # The forward needs q, k, v only and its output can leave while the backward runs, so dout goes
                # up behind them and out goes down ahead of the gradients: less of the first upload and of
                # the last download is left outside the overlap.
                with torch.cuda.stream(self.s_in):
                    if b >= self.slots:
                        self.s_in.wait_event(self.done[sl])  # the slot's inputs have been consumed
                    d["q"].copy_(q[b], non_blocking=True)
                    d["k"].copy_(k[b], non_blocking=True)
                    d["v"].copy_(v[b], non_blocking=True)
                    self.ready_f[sl].record(self.s_in)
                    d["dout"].copy_(dout[b], non_blocking=True)
                    self.ready_b[sl].record(self.s_in)
                with torch.cuda.stream(self.s_run):
                    self.s_run.wait_event(self.ready_f[sl])
                    if b >= self.slots:
                        self.s_run.wait_event(self.free[sl])  # the slot's outputs have been read
                    st = self.s_run.cuda_stream
                    token = ctypes.c_ulonglong(0)  # the slot's q, k, v stay untouched until its backward
                    rc = L.zt_attn_forward_batched_keep(d["q"].data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(),
                                                        d["out"].data_ptr(), d["lse"].data_ptr(),
                                                        d["ws"].data_ptr() if self.ws_bytes else None, self.ws_bytes,
                                                        1, t, n_heads, n_kv_heads, head_dim, st, ctypes.byref(token))
                    self.done_f[sl].record(self.s_run)
                    self.s_run.wait_event(self.ready_b[sl])
                    if rc == 0:
                        rc = L.zt_attn_backward_batched_kept(
                            d["q"].data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(), d["out"].data_ptr(),
                            d["lse"].data_ptr(), d["dout"].data_ptr(), d["dq"].data_ptr(), d["dk"].data_ptr(),
                            d["dv"].data_ptr(), d["delta"].data_ptr(),
                            d["ws"].data_ptr() if self.ws_bytes else None, self.ws_bytes, 1, t, n_heads,
                            n_kv_heads, head_dim, st, token.value)
                    if rc != 0:
                        torch.cuda.synchronize(self.device)
                        raise ConfigRefused(_lib.last_error())
                    self.done[sl].record(self.s_run)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(self.done_f[sl])
                    out[b].copy_(d["out"], non_blocking=True)
                    if lse is not None:
                        lse[b].copy_(d["lse"], non_blocking=True)
                    self.s_out.wait_event(self.done[sl])
                    dq[b].copy_(d["dq"], non_blocking=True)
                    dk[b].copy_(d["dk"], non_blocking=True)
                    dv[b].copy_(d["dv"], non_blocking=True)
                    self.free[sl].record(self.s_out)
        self.s_out.synchronize()
        self.s_run.synchronize()
