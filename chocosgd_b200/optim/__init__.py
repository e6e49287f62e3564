"""The eight distributed algorithms selectable with ``--optimizer``
(``dl_code/pcode/create_optimizer.py:27-44``)."""
from .arena import FlatArena
from .base import DistributedOptimizer, build_param_groups
from .choco import ChocoSGD
from .dcd_psgd import DCD_PSGD
from .deep_squeeze import DeepSqueeze
from .dgc import DGC
from .ecd_psgd import ECD_PSGD
from .ef_sign_sgd import EF_SignSGD
from .sgd import SGD

_REGISTRY = {
    "sgd": SGD,
    "dgc": DGC,
    "dcd_psgd": DCD_PSGD,
    "ecd_psgd": ECD_PSGD,
    "parallel_choco": ChocoSGD,
    "parallel_choco_v": ChocoSGD,
    "ef_sign_sgd": EF_SignSGD,
    "deep_squeeze": DeepSqueeze,
}


def define_optimizer(conf, model, graph, group=None, **kw):
    try:
        cls = _REGISTRY[conf.optimizer]
    except KeyError:
        raise NotImplementedError(conf.optimizer) from None
    return cls(model, conf, graph, group, **kw)
