"""Activation offload: tensors saved for backward inside the wrapped region live in pinned host memory and come back
on demand (reference: siirl/utils/model_utils/activation_offload.py, enabled by ``enable_activation_offload``).
Built on ``torch.autograd.graph.saved_tensors_hooks``; copies run on a side stream so the device->host transfer of
layer i overlaps the forward of layer i+1.  Small tensors (below ``min_bytes``) stay on the device."""
from __future__ import annotations

import contextlib

import torch


class ActivationOffload:
    def __init__(self, min_bytes: int = 1 << 20, enabled: bool = True):
        self.min_bytes, self.enabled = min_bytes, enabled
        self.stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self.bytes_offloaded = 0

    def _pack(self, t: torch.Tensor):
        if not t.is_cuda or t.numel() * t.element_size() < self.min_bytes or isinstance(t, torch.nn.Parameter):
            return t
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            host.copy_(t, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        t.record_stream(self.stream)
        self.bytes_offloaded += host.numel() * host.element_size()
        return (host, t.device, ev)

    def _unpack(self, packed):
        if isinstance(packed, torch.Tensor):
            return packed
        host, dev, ev = packed
        ev.synchronize()
        return host.to(dev, non_blocking=True)

    @contextlib.contextmanager
    def region(self):
        if not self.enabled or self.stream is None:
            yield
            return
        with torch.autograd.graph.saved_tensors_hooks(self._pack, self._unpack):
            yield
