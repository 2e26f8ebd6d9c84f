"""Step staging: all host inputs of one step in ONE pinned arena, one host->device copy.

The reference uploads every step's metadata as separate pinned tensors
(`torch.tensor(..., pin_memory=True).cuda(non_blocking=True)`, four to six copies per step,
infer/engine/model_runner.py:103-124).  Each small copy costs a few microseconds of launch
latency, which is a visible fraction of a ~200 us decode step.  ``StepStaging`` lays the
tensors out back to back (256-byte aligned) in a pinned host buffer and a device buffer of
the same size; ``upload()`` moves everything with a single asynchronous copy.
"""
from __future__ import annotations

import math

import torch


class StepStaging:
    def __init__(self, spec: dict, device):
        """spec: name -> (shape, dtype).  Creates ``self.host[name]`` (pinned views to fill)
        and ``self.dev[name]`` (device views to pass to the ops)."""
        offsets, at = {}, 0
        for name, (shape, dtype) in spec.items():
            nbytes = math.prod(shape) * torch.empty(0, dtype=dtype).element_size()
            offsets[name] = (at, nbytes, tuple(shape), dtype)
            at = (at + nbytes + 255) // 256 * 256
        self.nbytes = max(at, 256)
        self._host = torch.empty(self.nbytes, dtype=torch.uint8)
        if torch.device(device).type == "cuda":
            self._host = self._host.pin_memory()
        self._dev = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.host, self.dev = {}, {}
        for name, (off, nbytes, shape, dtype) in offsets.items():
            self.host[name] = self._host[off:off + nbytes].view(dtype).view(shape)
            self.dev[name] = self._dev[off:off + nbytes].view(dtype).view(shape)

    def upload(self):
        self._dev.copy_(self._host, non_blocking=True)
