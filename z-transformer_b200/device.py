"""Host-side mirror of the reference's Zig holder, src/cuda/device.zig.

Same names, argument meaning and error behaviour: `bytes_for`, `to_c_int`,
`forward_bounds` are pure functions (tested without a GPU, as device.zig:502-645
tests them); `Attn` owns the eleven device buffers of one (t, n_heads,
n_kv_heads, dim) shape and drives the C ABI.  torch supplies device memory and
the stream, nothing else.
"""
from __future__ import annotations

import enum

from . import lib as _lib

USIZE_MAX = 2 ** 64 - 1
C_INT_MAX = 2 ** 31 - 1


class Error(Exception):
    """Base of the holder's errors (device.zig:119-141)."""


class DegenerateShape(Error):
    pass


class ShapeTooLarge(Error):
    pass


class ConfigRefused(Error):
    pass


class DeviceAllocFailed(Error):
    pass


class DeviceTransferFailed(Error):
    pass


class Kind(enum.Enum):
    """Which buffer a size is for (device.zig:145-152)."""
    query_headed = 0  # [T, n_heads * dim]   q, out, dout, dq
    kv_headed = 1     # [T, n_kv_heads * dim] k, v, dk, dv
    per_row = 2       # [T, n_heads]          row_max, row_den, row_del


def _mul(a: int, b: int) -> int:
    r = a * b
    if r > USIZE_MAX:
        raise ShapeTooLarge(f"{a} * {b} overflows usize")
    return r


def bytes_for(kind: Kind, t: int, n_heads: int, n_kv_heads: int, dim: int) -> int:
    """device.bytesFor (device.zig:162-171): checked, never truncated."""
    if t == 0 or dim == 0 or n_heads == 0 or n_kv_heads == 0:
        raise DegenerateShape("a zero dimension")
    if kind is Kind.query_headed:
        cols = _mul(n_heads, dim)
    elif kind is Kind.kv_headed:
        cols = _mul(n_kv_heads, dim)
    else:
        cols = n_heads
    return _mul(_mul(t, cols), 4)


def to_c_int(x: int) -> int:
    """device.toCInt (device.zig:179-182)."""
    if x > C_INT_MAX:
        raise ShapeTooLarge(f"{x} does not fit a C int")
    return int(x)


def forward_bounds(c_t: int, q_offset: int, n_keys: int, t: int) -> None:
    """device.forwardBounds (device.zig:489-501); raises ShapeTooLarge instead of returning it."""
    if n_keys < 1 or n_keys > c_t:
        raise ShapeTooLarge("n_keys outside the k/v buffers")
    if t < 1 or t > c_t:
        raise ShapeTooLarge("t outside the q/out buffers")
    if q_offset < 0 or q_offset > c_t or t > c_t - q_offset:
        raise ShapeTooLarge("q_offset outside the sequence")
    if q_offset + t > n_keys:
        raise ShapeTooLarge("the last query row has no key of its own")


_NAMES = ("q", "k", "v", "out", "dout", "dq", "dk", "dv", "row_max", "row_den", "row_del")
_KINDS = (Kind.query_headed, Kind.kv_headed, Kind.kv_headed, Kind.query_headed, Kind.query_headed,
          Kind.query_headed, Kind.kv_headed, Kind.kv_headed, Kind.per_row, Kind.per_row, Kind.per_row)


class Attn:
    """Eleven device buffers sized once for a fixed shape (device.zig:185-432)."""

    N_BUFFERS = 11

    def __init__(self, t: int, n_heads: int, n_kv_heads: int, dim: int, device="cuda"):
        import torch

        self.c_t = to_c_int(t)
        self.c_heads = to_c_int(n_heads)
        self.c_kv_heads = to_c_int(n_kv_heads)
        self.c_dim = to_c_int(dim)
        L = _lib.load()
        # Ask the C side before allocating anything (device.zig:227-241).
        if L.zt_attn_dim_ok(self.c_dim) == 0:
            raise ConfigRefused(f"head_dim {dim}")
        if self.c_heads <= 0 or self.c_kv_heads <= 0 or self.c_heads % self.c_kv_heads != 0:
            raise ConfigRefused(f"{n_heads} heads over {n_kv_heads} kv heads")
        if n_heads > 65535:
            raise ConfigRefused(f"{n_heads} heads")
        self.t, self.n_heads, self.n_kv_heads, self.dim = t, n_heads, n_kv_heads, dim
        self.device = torch.device(device)
        self._buf = {}
        try:
            for name, kind in zip(_NAMES, _KINDS):
                nbytes = bytes_for(kind, t, n_heads, n_kv_heads, dim)
                self._buf[name] = torch.empty(nbytes // 4, dtype=torch.float32, device=self.device)
        except RuntimeError as e:  # torch's allocator failing is cudaMalloc failing
            self._buf.clear()
            raise DeviceAllocFailed(str(e)) from e
        # the library's own scratch for this shape is sized with the holder's buffers, so that forward() and
        # backward() never allocate (the one line a maintainer adds to device.Attn.init)
        if self.device.type == "cuda":
            with torch.cuda.device(self.device):
                if L.zt_attn_reserve(1, self.c_t, self.c_heads, self.c_kv_heads, self.c_dim) != 0:
                    self._buf.clear()
                    raise DeviceAllocFailed(_lib.last_error())

    def __getattr__(self, name):
        buf = self.__dict__.get("_buf", {})
        if name in buf:
            return buf[name]
        raise AttributeError(name)

    def deinit(self) -> None:
        self._buf.clear()

    def total_bytes(self) -> int:
        """device.zig:355-360: four query-headed, four kv-headed, three per-row."""
        return total_bytes(self.t, self.n_heads, self.n_kv_heads, self.dim)

    def _stream(self):
        import torch
        return torch.cuda.current_stream(self.device).cuda_stream

    def forward(self, group_q: int = 1, max_tile: int = 64) -> None:
        """The training shape: q_offset 0, n_keys = t = c_t (device.zig:381-383)."""
        self.forward_at(group_q, max_tile, 0, self.c_t, self.c_t)

    def forward_at(self, group_q: int, max_tile: int, q_offset: int, n_keys: int, t: int) -> None:
        """device.zig:387-398."""
        import torch
        forward_bounds(self.c_t, q_offset, n_keys, t)
        b = self._buf
        with torch.cuda.device(self.device):
            rc = _lib.load().zt_attn_forward(b["q"].data_ptr(), b["k"].data_ptr(), b["v"].data_ptr(),
                                             b["out"].data_ptr(), t, self.c_heads, self.c_kv_heads,
                                             self.c_dim, group_q, max_tile, q_offset, n_keys,
                                             self._stream())
        if rc != 0:
            raise ConfigRefused(_lib.last_error())

    def backward(self, max_tile: int = 64) -> None:
        """device.zig:403-406."""
        import torch
        b = self._buf
        with torch.cuda.device(self.device):
            rc = _lib.load().zt_attn_backward(
                b["q"].data_ptr(), b["k"].data_ptr(), b["v"].data_ptr(), b["dout"].data_ptr(),
                b["dq"].data_ptr(), b["dk"].data_ptr(), b["dv"].data_ptr(), b["row_max"].data_ptr(),
                b["row_den"].data_ptr(), b["row_del"].data_ptr(), self.c_t, self.c_heads,
                self.c_kv_heads, self.c_dim, max_tile, self._stream())
        if rc != 0:
            raise ConfigRefused(_lib.last_error())

    def upload(self, dst, src) -> None:
        """Host to device (device.zig:412-419); src is a numpy float32 array."""
        import numpy as np
        import torch
        src = np.ascontiguousarray(src, dtype=np.float32).ravel()
        if src.size * 4 > dst.numel() * 4:
            raise ShapeTooLarge("source larger than the device buffer")
        try:
            dst[: src.size].copy_(torch.from_numpy(src))
        except RuntimeError as e:
            raise DeviceTransferFailed(str(e)) from e

    def download(self, n: int, src):
        """Device to host (device.zig:426-431): the first n floats of `src`; this copy is
        also the synchronisation point, as in the reference's callers."""
        if n * 4 > src.numel() * 4:
            raise ShapeTooLarge("destination larger than the device buffer")
        try:
            return src[:n].cpu().numpy()
        except RuntimeError as e:
            raise DeviceTransferFailed(str(e)) from e


def total_bytes(t: int, n_heads: int, n_kv_heads: int, dim: int) -> int:
    qh = bytes_for(Kind.query_headed, t, n_heads, n_kv_heads, dim)
    kvh = bytes_for(Kind.kv_headed, t, n_heads, n_kv_heads, dim)
    pr = bytes_for(Kind.per_row, t, n_heads, n_kv_heads, dim)
    return 4 * qh + 4 * kvh + 3 * pr
