"""Model-distance helpers (``dl_code/pcode/utils/auxiliary.py:18-77``)."""
from datetime import datetime

import torch


def get_model_difference(model1, model2) -> float:
    """L2 norm of the parameter difference, accumulated in float64."""
    acc = torch.zeros((), dtype=torch.float64)
    for w1, w2 in zip(model1.parameters(), model2.parameters()):
        d = (w2.detach().double() - w1.detach().double()).reshape(-1)
        acc = acc + (d * d).sum().cpu()
    return float(acc.sqrt())


def flat_difference_norm(x1: torch.Tensor, x2: torch.Tensor) -> float:
    d = x2.double() - x1.double()
    return float((d * d).sum().sqrt())


def str2time(string, pattern):
    return datetime.strptime(string, pattern)


def get_fullname(o):
    return "%s.%s" % (o.__module__, o.__class__.__name__)


def is_float(value) -> bool:
    try:
        float(value)
        return True
    except (TypeError, ValueError):
        return False


class dict2obj:
    def __init__(self, d):
        for a, b in d.items():
            if isinstance(b, (list, tuple)):
                setattr(self, a, [dict2obj(x) if isinstance(x, dict) else x for x in b])
            else:
                setattr(self, a, dict2obj(b) if isinstance(b, dict) else b)
