"""Device-resident KV cache with the reference's kv_cache semantics (src/kv_cache.zig).

The reference keeps the cache on the host and re-uploads the whole filled prefix
on every decode step (src/decode.zig:435-437); here the cache lives in HBM, one
[batch, n_ctx, n_kv_heads*head_dim] pair per layer, rows are appended by a kernel
and the decode kernel reads them in place.

A decode loop must not wait for the GPU between steps, so the refusals the reference
makes from a layer's `len` (Error.Full, src/kv_cache.zig:88-95,196) are made here from a
count kept on the host: every append advances every sequence of a layer by one row, so
the host knows an upper bound of the fill counts without reading them back.  Only when
that bound says a sequence MAY be full (lens that were set ragged by hand) are the device
counts read to decide exactly.
"""
from __future__ import annotations

from . import lib as _lib
from .device import ConfigRefused
from .ops import DecodeWorkspace, DimensionMismatch, _need_cuda_f32, decode_attention


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
        self._len_bound = 0  # no sequence of the layer holds more rows than this

    def set_lens(self, lens) -> None:
        """Start from given per-sequence fill counts (a ragged batch whose rows were written directly)."""
        import torch
        lens = torch.as_tensor(lens, dtype=torch.int32)
        if lens.shape != (self.batch,) or int(lens.min()) < 0 or int(lens.max()) > self.n_ctx:
            raise DimensionMismatch("kv_cache.Layer.set_lens")
        self._len_bound = int(lens.max())
        self.len.copy_(lens.to(self.len.device))

    def check_append(self, k_rows, v_rows) -> None:
        """Every refusal of append, made without writing anything: widths, placement, and Full."""
        if tuple(k_rows.shape) != (self.batch, self.width) or tuple(v_rows.shape) != (self.batch, self.width):
            raise DimensionMismatch("kv_cache.Layer.append")
        _need_cuda_f32(k_rows, v_rows)
        if k_rows.device != self.k.device or v_rows.device != self.k.device:
            raise DimensionMismatch("the new rows must live on the cache's device")
        if self._len_bound >= self.n_ctx:
            # possibly full: the device counts decide (this read waits for the GPU; it happens only at the
            # very end of a cache's life, or on caches whose lens were set ragged)
            if int(self.len.max().item()) >= self.n_ctx:
                raise Full("kv_cache.Layer.append")

    def append(self, k_rows, v_rows) -> None:
        """One new row per sequence ([batch, width]); refuses, writing nothing, when any
        sequence is full or a width is wrong (src/kv_cache.zig:88-95)."""
        self.check_append(k_rows, v_rows)
        self._append_unchecked(k_rows, v_rows)

    def _append_unchecked(self, k_rows, v_rows) -> None:
        import torch
        with torch.cuda.device(self.k.device):
            rc = _lib.load().zt_kv_append(
                self.k.data_ptr(), self.v.data_ptr(), self.len.data_ptr(), k_rows.data_ptr(), v_rows.data_ptr(),
                self._full.data_ptr(), self.batch, self.n_ctx, 1, self.width,
                torch.cuda.current_stream(self.k.device).cuda_stream)
        if rc != 0:
            raise ConfigRefused(_lib.last_error())
        self._len_bound = min(self._len_bound + 1, self.n_ctx)

    def skipped_full(self) -> int:
        """Sequences the append kernel has left untouched because they were full, over the layer's life (reads
        the device: waits for the GPU).  Zero unless a caller bypassed check_append."""
        return int(self._full.item())

    def visible(self):
        """Per-sequence filled row counts (src/kv_cache.zig:133-135)."""
        return self.len

    def bytes(self) -> int:
        return 2 * self.batch * self.n_ctx * self.width * 4


class Cache:
    """kv_cache.Cache (src/kv_cache.zig:140-225): one Layer per transformer layer, advanced together."""

    def __init__(self, n_layers: int, n_ctx: int, width: int, batch: int = 1, device="cuda"):
        if n_layers == 0:
            raise DimensionMismatch("kv_cache.Cache.init")  # src/kv_cache.zig:154
        self.layers = [Layer(n_ctx, width, batch, device) for _ in range(n_layers)]
        self.len = 0

    def append_all(self, ks, vs) -> None:
        """One position for every layer, all or nothing (src/kv_cache.zig:180-200): EVERY layer is checked
        (count of tensors, widths, room) before ANY of them is written."""
        if len(ks) != len(self.layers) or len(vs) != len(self.layers):
            raise DimensionMismatch("kv_cache.Cache.appendAll")
        for layer, k_rows, v_rows in zip(self.layers, ks, vs):
            layer.check_append(k_rows, v_rows)
        for layer, k_rows, v_rows in zip(self.layers, ks, vs):
            layer._append_unchecked(k_rows, v_rows)
        self.len += 1

    def full(self) -> bool:
        """Whether another position would not fit (src/kv_cache.zig:211-214)."""
        if not self.layers:
            return True
        return self.len >= self.layers[0].n_ctx

    def bytes(self) -> int:
        """src/kv_cache.zig:220-224."""
        return sum(layer.bytes() for layer in self.layers)


def attn_step(q, layer: Layer, n_heads, n_kv_heads, head_dim, *, workspace: DecodeWorkspace | None = None,
              want_lse=False):
    """decode.cudaAttnStep (src/decode.zig:405-473) without the per-step upload: q [batch, H*D]."""
    if layer.width != n_kv_heads * head_dim:
        raise DimensionMismatch("cache width disagrees with the head configuration")
    return decode_attention(q, layer.k, layer.v, layer.len, n_heads, n_kv_heads, head_dim,
                            workspace=workspace, want_lse=want_lse)
