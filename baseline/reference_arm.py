"""Reference arm of the benchmark: the UNMODIFIED reference code installed under
``baseline/_ref`` (its ``pcode`` package), driven through its own public classes.

What runs: ``pcode.models.resnet`` (ResNet-20 / ResNet-50) or ``pcode.models.RNNLM``,
``pcode.create_optimizer.define_optimizer``
with ``--optimizer parallel_choco_v``, the reference compressors / aggregators / topology,
and the body of its training iteration (``dl_code/pcode/distributed_running_cv.py:42-62``:
host->device copy, zero_grad, forward, loss, metrics with their ``.item()`` reads, backward,
``optimizer.step(timer=..., scheduler=...)``).  Nothing from ``chocosgd_b200`` is imported.

Harness glue that is not reference code (each item is a documented deviation):
* ``bit2byte`` (an external C++ extension the reference imports, not in its tree) is
  replaced by a pure-PyTorch module with the same two functions;
* ``dl_code/main.py`` cannot run offline (torchtext / spacy / datasets), so the loop body
  is driven directly with synthetic CIFAR-shaped batches;
* ``parallel_choco_v`` instead of ``parallel_choco`` (the latter hard-codes an MPI group);
* ring needs n > 2 in the reference: n = 1, 2 use its ``complete`` graph, whose matrix
  equals the ring rule there ([1] and 1/2 everywhere);
* ``track_time`` off (its timer synchronises the device around every scope);
* top-5 accuracy: ``.view(-1)`` of a transposed tensor raises on torch >= 1.7; the metric
  function is re-bound once to the same operations with ``.reshape(-1)``;
* unbatched NCCL ``isend`` + ``irecv`` on both ends of an edge block each other (observed
  here: the 2-GPU run sat until the process-group timeout), so the module-level ``dist``
  name of ``pcode.utils.communication`` is proxied to issue the same messages as one
  ``batch_isend_irecv``; the reference source files are untouched.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def install_bit2byte_shim():
    b = types.ModuleType("bit2byte")

    def packing(src):  # int32 [32, M] of signs -> int32 [M]
        out = torch.zeros(src.shape[1], dtype=torch.int64, device=src.device)
        for i in range(32):
            out |= (src[i] < 0).to(torch.int64) << i
        out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
        return out.to(torch.int32)

    def unpacking(src, dst):  # int32 [M] -> values {0, 2} in dst [32, M]
        s = src.to(torch.int64) & 0xFFFFFFFF
        for i in range(32):
            dst[i] = (2 * ((s >> i) & 1)).to(torch.int32)
        return dst

    b.packing, b.unpacking = packing, unpacking
    sys.modules["bit2byte"] = b


class _LazyReq:
    def __init__(self, batch):
        self.batch, self.req = batch, None

    def wait(self):
        self.batch.flush()
        for r in self.req or ():
            r.wait()


class BatchedP2P:
    """Stand-in for the ``dist`` name inside the reference's communication module.

    The reference posts ``dist.isend`` then ``dist.irecv`` per neighbour
    (``dl_code/pcode/utils/communication.py:259-262``).  With NCCL both ends of an edge
    enqueue their send first and block each other.  This proxy forwards everything to
    ``torch.distributed`` but queues those two calls and issues the SAME sends / receives
    as one ``batch_isend_irecv`` when the first request is waited on."""

    def __init__(self, real):
        self._real, self._ops, self._reqs = real, [], []

    def __getattr__(self, name):
        return getattr(self._real, name)

    def isend(self, tensor, dst, **kw):
        return self._queue(self._real.isend, tensor, dst)

    def irecv(self, tensor, src=None, **kw):
        return self._queue(self._real.irecv, tensor, src)

    def _queue(self, op, tensor, peer):
        r = _LazyReq(self)
        self._ops.append(self._real.P2POp(op, tensor, peer))
        self._reqs.append(r)
        return r

    def flush(self):
        if not self._ops:
            return
        ops, lazy = self._ops, self._reqs
        self._ops, self._reqs = [], []
        works = list(self._real.batch_isend_irecv(ops))  # NCCL returns one coalesced work
        for l in lazy:
            l.req = works


def available():
    return os.path.isdir(os.path.join(REF, "pcode"))


def build(rank, world, comm_op, batch_size, device, consensus_stepsize=0.5, model_name="resnet20", init_state=None):
    """Reference model + optimizer + metrics for one of the benchmark workloads:
    ``resnet20`` (CIFAR shapes, fp32), ``resnet50`` (ImageNet shapes; the caller runs it under bf16
    autocast) or ``lstm`` (2 x 650 tied-weight language model, vocabulary 33 278, clip 0.4)."""
    if REF not in sys.path:
        sys.path.insert(0, REF)
    install_bit2byte_shim()
    import pcode.create_metrics as create_metrics
    import pcode.create_optimizer as create_optimizer
    import pcode.models as models
    import pcode.utils.communication as communication
    import pcode.utils.topology as topology
    from pcode.utils.timer import Timer

    if not isinstance(communication.dist, BatchedP2P):
        communication.dist = BatchedP2P(dist)

    topo = "ring" if world > 2 else "complete"
    is_lm = model_name == "lstm"
    conf = argparse.Namespace(
        arch={"resnet20": "resnet20", "resnet50": "resnet50", "lstm": "rnn_lm"}[model_name],
        data="imagenet" if model_name == "resnet50" else "cifar10", optimizer="parallel_choco_v", comm_op=comm_op,
        compress_ratio=0.99, quantize_level=4, is_biased=True, backend="nccl", use_ipc=False,
        consensus_stepsize=consensus_stepsize, comm_device="cuda",
        weight_decay=0.0 if is_lm else 1e-4, lr=2.5 if is_lm else 0.1, momentum_factor=0.0 if is_lm else 0.9,
        use_nesterov=not is_lm, epoch_=0.5, local_index=0, distributed=True, graph_topology=topo,
        n_mpi_process=world, n_sub_process=1, on_cuda=True, batch_size=batch_size,
        rnn_clip=0.4, n_tokens=33278,
    )
    conf.graph = topology.define_graph_topology(
        topo, world=",".join(["0"] * world), n_mpi_process=world, n_sub_process=1, comm_device="cuda",
        on_cuda=True, rank=rank,
    )
    torch.manual_seed(6)
    if is_lm:
        model = models.RNNLM(ntoken=conf.n_tokens, ninp=650, nhid=650, nlayers=2, tie_weights=True, dropout=0.4,
                             weight_norm=False).to(device)
    else:
        model = models.resnet(conf).to(device)
    if init_state is not None:   # trajectory comparison: start from a given set of weights (a state dict file)
        model.load_state_dict(torch.load(init_state, map_location=device))
    optimizer = create_optimizer.define_optimizer(conf, model)
    metrics = create_metrics.Metrics(model, task="language_modeling" if is_lm else "classification")
    if not is_lm:
        metrics.metrics_fn = _accuracy_with_reshape(metrics)
    timer = Timer(verbosity_level=0, on_cuda=True)
    criterion = torch.nn.CrossEntropyLoss(reduction="mean")
    return conf, model, optimizer, metrics, timer, criterion


def _accuracy_with_reshape(metrics):
    """The reference's ``Metrics._accuracy`` (``dl_code/pcode/create_metrics.py:31-48``) flattens a
    transposed tensor with ``.view(-1)``, which torch >= 1.7 rejects for top-5.  This is the same
    sequence of operations (one ``topk``, one ``eq``, one ``.item()`` per k) with ``.reshape(-1)``,
    bound once at build time so that no exception is raised inside the timed loop."""
    topks = metrics.topks

    def accuracy(loss, output, target):
        _, pred = output.topk(max(topks), 1, True, True)
        pred = pred.t()
        correct = pred.eq(target.view(1, -1).expand_as(pred))
        return [correct[:k].reshape(-1).float().sum(0, keepdim=True).mul_(100.0 / target.size(0)).item()
                for k in topks]

    return accuracy


def finish(state):
    """Join the reference's helper thread so no exchange is in flight at teardown."""
    optimizer = state[2]
    thread = getattr(optimizer, "helper_thread", None)
    if thread is not None:
        thread.join()
    torch.cuda.synchronize()


def train_iteration(conf, model, optimizer, metrics, timer, criterion, inp_host, tgt_host, step, amp_dtype=None):
    """One iteration of the reference's CV loop (``amp_dtype``: forward under autocast, which the
    reference, written for PyTorch 1.3, does not have; used for the bf16 ResNet-50 workload so that
    both arms compute in the same precision)."""
    model.train()
    conf.local_index = step + 1
    conf.epoch_ = (step + 1) / 391.0
    _input, _target = inp_host.cuda(non_blocking=True), tgt_host.cuda(non_blocking=True)
    optimizer.zero_grad()
    if amp_dtype is not None:
        with torch.autocast("cuda", dtype=amp_dtype):
            output = model(_input)
        output = output.float()
    else:
        output = model(_input)
    loss = criterion(output, _target)
    perf = metrics.evaluate(loss, output, _target)  # .item() per metric, as in the reference
    loss_v = loss.item()
    loss.backward()
    optimizer.step(timer=timer, scheduler=None)
    return loss_v, perf


def train_iteration_lm(conf, model, optimizer, metrics, timer, criterion, inp_host, tgt_host, step, hidden):
    """One iteration of the reference's language-model loop
    (``dl_code/pcode/distributed_running_nlp.py:41-97,132-139``): detach the carried hidden state,
    host->device copy, zero_grad, forward, loss over the flattened logits, perplexity metric and
    ``loss.item()`` (host synchronisations, as there), backward, ``clip_grad_norm_``, ``optimizer.step``.
    Returns ``(loss value, new hidden state)``."""
    model.train()
    conf.local_index = step + 1
    conf.epoch_ = (step + 1) / 100.0
    hidden = model.repackage_hidden(hidden)
    _input, _target = inp_host.cuda(non_blocking=True), tgt_host.cuda(non_blocking=True)
    optimizer.zero_grad()
    output, hidden = model(_input, hidden)
    loss = criterion(output.view(-1, conf.n_tokens), _target.contiguous().view(-1))
    metrics.evaluate(loss, output, _target)   # exp(loss): reads the loss on the host
    loss_v = loss.item()
    loss.backward()
    torch.nn.utils.clip_grad_norm_(model.parameters(), conf.rnn_clip)
    optimizer.step(timer=timer)
    return loss_v, hidden
