"""Pinned host staging for the host-to-device copies of ``format_data``.

Upstream's ``format_data`` (qml_lightning/models/kernel.py:601-722) builds every tensor on the host and copies it with a
blocking ``.cuda()`` from pageable memory.  Here the padded arrays of a batch are written straight into one grow-only
page-locked buffer and copied with ``non_blocking=True`` on the current stream, so the host returns at once and can
format the next batch while the device works on this one.  The buffer is reused: before it is written again the event
recorded after the previous batch's copies is waited for (the copies only, not the kernels that follow them).
One stage belongs to one model and one host thread.
"""
import numpy as np
import torch

_TORCH_DTYPE = {np.dtype(np.float32): torch.float32, np.dtype(np.float64): torch.float64, np.dtype(np.int32): torch.int32,
                np.dtype(np.int64): torch.int64}
_ALIGN = 256


class PinnedStage:

    def __init__(self):
        self.buffer = None
        self.copied = None

    def arrays(self, specs):
        """Zero-filled numpy arrays (and the tensors that alias them) of the given ``(shape, dtype)`` list, carved out
        of the pinned buffer."""
        sizes = [int(np.prod(shape)) * np.dtype(dt).itemsize for shape, dt in specs]
        total = sum((n + _ALIGN - 1) // _ALIGN * _ALIGN for n in sizes) + _ALIGN
        if self.copied is not None:
            self.copied.synchronize()
            self.copied = None
        if self.buffer is None or self.buffer.numel() < total:
            self.buffer = torch.empty(total + total // 2, dtype=torch.uint8, pin_memory=True)
        tensors, off = [], 0
        for (shape, dt), n in zip(specs, sizes):
            t = self.buffer[off:off + n].view(_TORCH_DTYPE[np.dtype(dt)]).view(*shape)
            t.zero_()
            tensors.append(t)
            off += (n + _ALIGN - 1) // _ALIGN * _ALIGN
        return [t.numpy() for t in tensors], tensors

    def upload(self, tensors, device):
        """Device copies of the staged tensors, enqueued on the current stream of ``device`` without waiting."""
        out = [torch.empty(t.shape, dtype=t.dtype, device=device).copy_(t, non_blocking=True) for t in tensors]
        self.copied = torch.cuda.Event()
        self.copied.record(torch.cuda.current_stream(device))
        return out
