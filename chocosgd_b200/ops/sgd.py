"""Fused local optimizer ops on flat arenas (``csrc/sgd.cu``)."""
from __future__ import annotations

import torch

from . import _lib


def grad_clip_(engine, max_norm: float, stream=None) -> torch.Tensor:
    """Global gradient-norm clipping that does not rewrite the gradient: one kernel computes
    ||g||_2 over the engine's gradient (flat or per-tensor pointers) and stores
    ``min(1, max_norm / (norm + 1e-6))`` into the device-resident gradient scale, which the
    following update kernel multiplies in.  Returns the norm (one entry per logical rank)
    (``torch.nn.utils.clip_grad_norm_`` semantics, ``dl_code/pcode/distributed_running_nlp.py:94-97``)."""
    if getattr(engine, "_clip_norm", None) is None:
        engine._clip_norm = torch.zeros(engine.n_local, dtype=torch.float32, device=engine.device)
    lib = _lib.load()
    _lib.check(
        lib.grad_clip_coef(engine._pp, engine.tables.n_chunks, engine.n_local, float(max_norm),
                           _lib.ptr(engine._clip_norm), _lib.stream_ptr(stream)),
        "grad_clip_coef",
    )
    return engine._clip_norm
