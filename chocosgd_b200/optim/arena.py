"""FlatArena: one flat fp32 buffer per quantity; model tensors are views of it.

The reference copies all parameters into a fresh flat ``TensorBuffer`` and back several
times per step (``dl_code/pcode/optim/utils.py:50-62``, ``dl_code/pcode/utils/tensor_buffer.py:11-40``).
Here ``p.data`` and ``p.grad`` of every parameter alias slices of two persistent flat
tensors ``x`` and ``g`` for the whole run, so the optimizers and the gossip kernels see
the model as one vector without any packing, and one kernel launch covers all tensors.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Tuple

import torch

from ..compress.segments import Segments


class FlatArena:
    def __init__(self, named_params: Iterable[Tuple[str, torch.nn.Parameter]], device=None):
        named = [(n, p) for n, p in named_params if p.requires_grad]
        if not named:
            raise ValueError("no trainable parameters")
        self.names: List[str] = [n for n, _ in named]
        self.params: List[torch.nn.Parameter] = [p for _, p in named]
        device = device if device is not None else self.params[0].device
        self.device = torch.device(device)
        self.seg = Segments.from_sizes([p.numel() for p in self.params], self.names)
        self.x = torch.zeros(self.seg.total, dtype=torch.float32, device=self.device)
        self.g = torch.zeros(self.seg.total, dtype=torch.float32, device=self.device)
        # 4-d tensors that arrive in channels_last (NHWC / KRSC) format keep that memory order
        # inside their segment: the flat slice is viewed [K, R, S, C] and permuted back to the
        # logical [K, C, R, S] shape, so state_dict() values and shapes are unchanged.
        self.channels_last = [
            p.dim() == 4 and p.is_contiguous(memory_format=torch.channels_last) and not p.is_contiguous()
            for p in self.params
        ]
        for p, sl, cl in zip(self.params, self.seg.slices(), self.channels_last):
            self._view(self.x[sl], p.shape, cl).copy_(p.data.to(torch.float32))
        self.rebind()

    @staticmethod
    def _view(flat, shape, channels_last):
        if not channels_last:
            return flat.view(shape)
        k, c, r, s = shape
        return flat.view(k, r, s, c).permute(0, 3, 1, 2)

    def rebind(self):
        """(Re-)point ``p.data`` / ``p.grad`` at the flat buffers."""
        for p, sl, cl in zip(self.params, self.seg.slices(), self.channels_last):
            p.data = self._view(self.x[sl], p.shape, cl)
            p.grad = self._view(self.g[sl], p.shape, cl)

    def adopt_x(self, new_x: torch.Tensor):
        """Replace the parameter storage (e.g. by a peer-mapped allocation)."""
        new_x.copy_(self.x)
        self.x = new_x
        self.rebind()

    def zero_grad(self):
        self.g.zero_()

    def check_bound(self) -> bool:
        """True while every parameter and gradient still aliases the arena (something
        like ``model.to()`` or ``zero_grad(set_to_none=True)`` silently breaks it)."""
        base_x, base_g = self.x.data_ptr(), self.g.data_ptr()
        for p, off in zip(self.params, self.seg.offsets):
            if p.data.data_ptr() != base_x + 4 * off:
                return False
            if p.grad is None or p.grad.data_ptr() != base_g + 4 * off:
                return False
        return True

    def per_element(self, per_segment_values) -> torch.Tensor:
        out = torch.zeros(self.seg.total, dtype=torch.float32, device=self.device)
        for sl, v in zip(self.seg.slices(), per_segment_values):
            out[sl] = float(v)
        return out

    def valid_mask(self) -> torch.Tensor:
        return torch.from_numpy(self.seg.valid_mask()).to(self.device)
