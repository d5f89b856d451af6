"""Device-resident KV cache with the reference's kv_cache semantics (src/kv_cache.zig).

The reference keeps the cache on the host and re-uploads the whole filled prefix
on every decode step (src/decode.zig:435-437); here the cache lives in HBM, one
[batch, n_ctx, n_kv_heads*head_dim] pair per layer, rows are appended by a kernel
and the decode kernel reads them in place.
"""
from __future__ import annotations

from . import lib as _lib
from .device import ConfigRefused
from .ops import DecodeWorkspace, DimensionMismatch, decode_attention


class Full(Exception):
    """kv_cache Error.Full (src/kv_cache.zig:88-95)."""


class Layer:
    """kv_cache.Layer for `batch` sequences: k, v [batch, n_ctx, width] and per-sequence len."""

    def __init__(self, n_ctx: int, width: int, batch: int = 1, device="cuda"):
        import torch
        if n_ctx == 0 or width == 0:
            raise DimensionMismatch("kv_cache.Layer.init")  # src/kv_cache.zig:66
        self.n_ctx, self.width, self.batch = n_ctx, width, batch
        self.k = torch.zeros((batch, n_ctx, width), dtype=torch.float32, device=device)
        self.v = torch.zeros_like(self.k)
        self.len = torch.zeros((batch,), dtype=torch.int32, device=device)
        self._full = torch.zeros((1,), dtype=torch.int32, device=device)

    def append(self, k_rows, v_rows) -> None:
        """One new row per sequence ([batch, width]); refuses, writing nothing, when any
        sequence is full or a width is wrong (src/kv_cache.zig:88-95)."""
        import torch
        if k_rows.shape != (self.batch, self.width) or v_rows.shape != (self.batch, self.width):
            raise DimensionMismatch("kv_cache.Layer.append")
        if int(self.len.max().item()) >= self.n_ctx:
            raise Full("kv_cache.Layer.append")
        self._full.zero_()
        with torch.cuda.device(self.k.device):
            rc = _lib.load().zt_kv_append(
                self.k.data_ptr(), self.v.data_ptr(), self.len.data_ptr(), k_rows.contiguous().data_ptr(),
                v_rows.contiguous().data_ptr(), self._full.data_ptr(), self.batch, self.n_ctx, 1,
                self.width, torch.cuda.current_stream(self.k.device).cuda_stream)
        if rc != 0:
            raise ConfigRefused(_lib.last_error())

    def visible(self):
        """Per-sequence filled row counts (src/kv_cache.zig:133-135)."""
        return self.len

    def bytes(self) -> int:
        return 2 * self.batch * self.n_ctx * self.width * 4


def attn_step(q, layer: Layer, n_heads, n_kv_heads, head_dim, *, workspace: DecodeWorkspace | None = None,
              want_lse=False):
    """decode.cudaAttnStep (src/decode.zig:405-473) without the per-step upload: q [batch, H*D]."""
    if layer.width != n_kv_heads * head_dim:
        raise DimensionMismatch("cache width disagrees with the head configuration")
    return decode_attention(q, layer.k, layer.v, layer.len, n_heads, n_kv_heads, head_dim,
                            workspace=workspace, want_lse=want_lse)
