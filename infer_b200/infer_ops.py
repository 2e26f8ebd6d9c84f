"""Module with the attribute names of the reference's ``infer_ops`` package
(infer_ops/__init__.py:17-43) for the ops of the paged KV-cache path: importing it loads
the shared library, registers ``torch.ops._C.*`` and re-exports the ops."""
import torch

from . import _lib, ops

_lib.load()
ops.register_torch_ops()

flash_attn_prefill = torch.ops._C.flash_attn_prefill
store_kvcache = torch.ops._C.store_kvcache
paged_attn_decode = torch.ops._C.paged_attn_decode
paged_attn_prefill = torch.ops._C.paged_attn_prefill

__all__ = ["flash_attn_prefill", "store_kvcache", "paged_attn_decode", "paged_attn_prefill"]
