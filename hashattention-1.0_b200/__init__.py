"""B200-native (sm_100a) sparse-decode path of HashAttention behind the reference's Python API.

The directory name is not a Python identifier; load it under the module name
``hashattention_b200`` (``__graft_entry__.load_package()`` does that), after which
``from hashattention_b200 import load_usa, convert_usa`` mirrors
``from hashattention.hashattention_llama import load_usa, convert_usa``.
"""
from . import _lib, partition
from .cache import PagedHashKVCache
from .ops import Budget, ChunkRows, HostStepBuffers, SparseDecodeContext, decode_step_host, set_nvtx
from .torch_ops import decode_step_op
from .usa import USA, PackedHashWeights

__all__ = [
    "USA", "PackedHashWeights", "PagedHashKVCache", "Budget", "ChunkRows", "SparseDecodeContext", "HostStepBuffers",
    "decode_step_host", "decode_step_op", "set_nvtx", "_lib", "partition",
]
