"""infer_b200 - sm_100a implementation of the paged KV-cache path of Graylatzhou/Infer.

Host side (this package): the reference's Python interfaces for the path - Sequence,
BlockManager, step metadata, Context, Attention, the ``infer_ops``-style op module - over
``libinfer_b200.so`` (csrc/, C ABI in include/infer_b200.h)."""
from .block_manager import BlockManager
from .context import Context, get_context, reset_context, set_context
from .sequence import Sequence

__all__ = ["BlockManager", "Context", "get_context", "set_context", "reset_context",
           "Sequence"]
__version__ = "0.1.0"
