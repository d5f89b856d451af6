"""B200-native attention hot path for Z-TRANSFORMER: ctypes host layer over libztattn.so.

The directory name has a hyphen; import it with
``importlib.import_module("z-transformer_b200")``.
"""
from . import device, kv_cache, lib, ops, sharding  # noqa: F401
from ._build import build_library  # noqa: F401
from .device import Attn, Kind, bytes_for, forward_bounds, to_c_int  # noqa: F401
from .ops import (AttentionBlock, AttnPipeline, BackwardWorkspace, DecodeWorkspace, ProjWorkspace,  # noqa: F401
                  RopeWorkspace, attention_backward, attention_backward_rope, attention_forward,
                  attention_forward_rope, decode_attention, proj_backward, proj_forward)
