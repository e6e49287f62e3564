"""Intra-node data parallelism for ``--n_sub_process k``: one graph node drives ``k`` local
GPUs and its batch is split across them (the reference wraps the model in
``torch.nn.DataParallel``, ``dl_code/main.py:79-81,167-169``; its hand-written
``AllReduceDataParallel`` is dead code).  The wrapper keeps ``state_dict`` keys of the
wrapped module, so checkpoints are interchangeable with single-GPU nodes."""
from __future__ import annotations

import torch


class LocalDataParallel(torch.nn.DataParallel):
    def __init__(self, module, device_ids):
        ids = [int(d) % max(torch.cuda.device_count(), 1) for d in device_ids]
        super().__init__(module, device_ids=sorted(set(ids)))

    def state_dict(self, *args, **kwargs):
        return self.module.state_dict(*args, **kwargs)

    def load_state_dict(self, state_dict, *args, **kwargs):
        return self.module.load_state_dict(state_dict, *args, **kwargs)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)
