"""B200-native attention hot path for Z-TRANSFORMER: ctypes host layer over libztattn.so.

The directory name has a hyphen; import it with
``importlib.import_module("z-transformer_b200")``.
"""
from . import device, kv_cache, lib, ops, sharding  # noqa: F401
from ._build import build_library  # noqa: F401
from .device import Attn, Kind, bytes_for, forward_bounds, to_c_int  # noqa: F401
from .ops import (AttnPipeline, DecodeWorkspace, attention_backward, attention_forward,  # noqa: F401
                  decode_attention)
