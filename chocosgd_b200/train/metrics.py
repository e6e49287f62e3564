"""Evaluation metrics: top-1 / top-5 accuracy (top-5 only with >= 5 classes) for
classification, perplexity for language models (``dl_code/pcode/create_metrics.py:17-51``).
Results stay on the device as 0-d tensors; nothing here forces a host sync."""
from __future__ import annotations

import torch


class Metrics:
    def __init__(self, model, task="classification"):
        self.task = task
        self.model = model
        if task == "classification":
            n_cls = getattr(model, "num_classes", None)
            if n_cls is None and hasattr(model, "module"):
                n_cls = getattr(model.module, "num_classes", None)
            self.topks = (1, 5) if (n_cls is None or n_cls >= 5) else (1,)
            self.metric_names = ["top{}".format(k) for k in self.topks]
        elif task == "language_modeling":
            self.metric_names = ["ppl"]
        else:
            raise NotImplementedError(task)

    @property
    def primary(self):
        return self.metric_names[0]

    @torch.no_grad()
    def evaluate(self, loss, output, target):
        if self.task == "classification":
            return accuracy(output, target, self.topks)
        return [torch.exp(loss.detach())]


@torch.no_grad()
def accuracy(output, target, topk=(1,)):
    """Percentage of samples whose label is among the k highest scores."""
    maxk = max(topk)
    batch = target.size(0)
    _, pred = output.topk(maxk, 1, True, True)
    correct = pred.t().eq(target.view(1, -1).expand(maxk, batch))
    return [correct[:k].reshape(-1).float().sum() * (100.0 / batch) for k in topk]
