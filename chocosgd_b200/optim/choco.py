"""CHOCO-SGD (memory-efficient form), the algorithm this framework is built around.

State per rank: ``x_hat`` (own public copy) and ``s = sum_j w_ij x_hat_j``, both zero at
start.  One step (``dl_code/pcode/optim/parallel_choco_v.py:104-155``)::

    x   <- x - lr d'                           local momentum-SGD step
    (the exchange of the previous step must have been applied to x_hat, s)
    x   <- x + gamma (s - x_hat)               consensus
    q_i  = Q(x - x_hat)                        per-tensor compression
    exchange q with the graph neighbours
    x_hat <- x_hat + q_i ;  s <- s + sum_j w_ij q_j     (j runs over neighbours and self)

``step()`` returns the bits of the *previous* exchange (``:113,155``).

Two execution paths share this class:

* ``impl="torch"`` - flat PyTorch ops + ``torch.distributed`` send/recv.  Runs on CPU/Gloo,
  is the ``--gossip_impl nccl`` baseline on GPUs, and the readable statement of the math.
* ``impl="fused"`` - the hand-written sm_100a kernels (``ops/gossip.py``): SGD, consensus,
  compression and the NVLink push to the neighbours' mailboxes happen inside the kernels;
  no ``torch.distributed`` call and no separate elementwise kernel is on that path.

Both the reference's ``parallel_choco`` (gossip in a helper *process*) and
``parallel_choco_v`` (helper *thread*) select this class: the overlap they implement on
the host is expressed here with CUDA streams / deferred completion instead.
"""
from __future__ import annotations

import torch

from .base import DistributedOptimizer


class ChocoSGD(DistributedOptimizer):
    timer_labels = (
        "sync.apply_grad",
        "sync.finish_sync",
        "sync.recover_hat_params",
        "sync.update_flatten_params",
        "sync.update_local_model",
        "sync.start_sync",
    )

    def __init__(self, model, conf, graph, group=None, impl="auto", engine=None):
        super().__init__(model, conf, graph, group)
        self.consensus_stepsize = float(conf.consensus_stepsize)
        self.codec = self.make_codec()
        self.x_hat = torch.zeros_like(self.arena.x)
        self.s = torch.zeros_like(self.arena.x)
        self.gossip_step = 0  # index of the next exchange
        self._pending = None  # (pending exchange, step index, own payload)
        self._pending_bits = 0
        self.overlap = bool(getattr(conf, "overlap_gossip", True))
        want = getattr(conf, "gossip_impl", "auto") if impl == "auto" else impl
        if want == "auto":
            want = "fused" if (self.device.type == "cuda" and engine is not False) else "torch"
        if want == "nccl" or self.identity_quantizer():
            want = "torch"  # --quantize_level 32 is the identity codec: no packed format applies
        self.impl = want
        self.engine = None
        if self.impl == "fused":
            if engine is None or engine is False:
                from ..ops.gossip import ChocoEngine

                engine = ChocoEngine.for_optimizer(self, group)
            self.engine = engine

    # ---- torch path ----------------------------------------------------------------------
    def _finish_sync(self):
        if self._pending is None:
            return
        pending, step = self._pending
        received = pending.wait()
        for rank, weight in self.neighbors_info.items():
            payload = received[rank]
            if self.codec.is_sparse:
                pos, val = self.codec.sparse(payload, step, rank)
                if rank == self.rank:
                    self.x_hat.index_add_(0, pos, val)
                self.s.index_add_(0, pos, val, alpha=weight)
            else:
                q = self.codec.decompress(payload, step, rank)
                if rank == self.rank:
                    self.x_hat.add_(q)
                self.s.add_(q, alpha=weight)
        self._pending = None
        self.n_bits = self._pending_bits

    def _step_torch(self, timer, ep):
        a = self.arena
        with timer("sync.apply_grad", epoch=ep):
            a.x.add_(self.local_direction(), alpha=-self.lr)
        with timer("sync.finish_sync", epoch=ep):
            self._finish_sync()
        with timer("sync.update_flatten_params", epoch=ep):
            a.x.add_(self.s - self.x_hat, alpha=self.consensus_stepsize)
        with timer("sync.start_sync", epoch=ep):
            payload = self.codec.compress(a.x - self.x_hat, self.gossip_step, self.rank)
            self._pending = (self.neighbor_exchange().start(payload), self.gossip_step)
            self._pending_bits = self.codec.n_bits()
            self.gossip_step += 1
            if not self.overlap:
                self._finish_sync()
        return self.n_bits

    # ---- fused path: host part / device part (the latter is what a CUDA graph captures) -------
    @property
    def capturable(self) -> bool:
        return self.impl == "fused"

    def prepare_step(self):
        """Host side of a fused step: refresh the device-resident hyper-parameters, account bits."""
        self.local_index += 1
        self.engine.set_hyper(self.lr, self.momentum, self.consensus_stepsize, self.nesterov)
        bits, self.n_bits = self.n_bits, self.codec.n_bits()
        self.gossip_step += 1
        return bits

    def launch(self, stream=None):
        """Device side of a fused step: the gossip kernels, nothing else."""
        if self._buckets_fired is not None:
            self._finish_buckets(stream)
            return
        self.engine.launch_step(stream)

    # ---- the step bucket by bucket, overlapped with the backward pass ---------------------------------
    # With per-tensor compression (sign + L1 norm of each tensor) the step of one tensor depends on that
    # tensor's gradient only.  Tensors are grouped, in arena order, into buckets of about ``bucket_bytes``;
    # a post-accumulate-grad hook launches a bucket's part of the step on a side stream as soon as the
    # last gradient of the bucket exists, while the backward pass of the earlier layers still runs
    # (the reference overlaps the exchange of step t with the computation of step t + 1 from a helper
    # thread: dl_code/pcode/optim/parallel_choco_v.py:111-113, 144-154).  ``launch()`` then only joins.
    _buckets_fired = None

    def bucket_plan(self, bucket_bytes: int):
        """``[(param indices, first chunk, chunk count)]`` in arena order (cached: the chunk table lives on the
        device and must not be read while a graph is being captured)."""
        cache = self.__dict__.setdefault("_bucket_plans", {})
        if bucket_bytes in cache:
            return cache[bucket_bytes]
        cache[bucket_bytes] = plan = self._make_bucket_plan(bucket_bytes)
        return plan

    def _make_bucket_plan(self, bucket_bytes: int):
        sizes = [int(n) * 4 for n in self.seg.sizes]
        plan, cur, acc = [], [], 0
        for i, b in enumerate(sizes):
            cur.append(i)
            acc += b
            if acc >= bucket_bytes:
                plan.append(cur)
                cur, acc = [], 0
        if cur:
            plan.append(cur)
        return [(idx,) + self.engine.segment_chunk_range(idx[0], idx[-1]) for idx in plan]

    def supports_buckets(self) -> bool:
        return self.impl == "fused" and self.engine.codec == 3 and type(self.engine).__name__ == "ChocoEngine"

    def arm_buckets(self, bucket_bytes: int, side_stream, extra_streams=()):
        """Install the hooks for ONE backward pass (call before it; ``launch()`` disarms).  ``extra_streams``:
        streams on which gradients may be produced besides the current one (weight-gradient stream)."""
        plan = self.bucket_plan(bucket_bytes)
        params = self.arena.params
        self._buckets_fired = [False] * len(plan)
        self._bucket_plan, self._bucket_stream = plan, side_stream
        left = [len(idx) for idx, _, _ in plan]
        self._bucket_handles = []
        self.engine._n_launch = 0

        def make_hook(b):
            def hook(_p):
                left[b] -= 1
                if left[b] == 0:
                    self._fire_bucket(b, extra_streams)
            return hook

        for b, (idx, _, _) in enumerate(plan):
            for i in idx:
                self._bucket_handles.append(params[i].register_post_accumulate_grad_hook(make_hook(b)))

    def _fire_bucket(self, b, extra_streams=()):
        side = self._bucket_stream
        side.wait_stream(torch.cuda.current_stream(self.device))
        capturing = torch.cuda.is_current_stream_capturing()
        for st in extra_streams:
            with torch.cuda.stream(st):
                joined = torch.cuda.is_current_stream_capturing()
            if joined or not capturing:   # (a stream outside the running capture has no work of this step)
                side.wait_stream(st)
        _, c0, nc = self._bucket_plan[b]
        self.engine.launch_step_range(c0, nc, stream=side)
        self._buckets_fired[b] = True

    def _finish_buckets(self, stream=None):
        main = stream if stream is not None else torch.cuda.current_stream(self.device)
        for h in self._bucket_handles:
            h.remove()
        # tensors whose gradient never arrived through a hook (unused parameters): their buckets go now
        for b, fired in enumerate(self._buckets_fired):
            if not fired:
                self._fire_bucket(b)
        main.wait_stream(self._bucket_stream)
        self.engine._steps += 1
        self.engine.launches_per_step = self.engine._n_launch
        self._buckets_fired = None

    # ---- public ------------------------------------------------------------------------------
    def step(self, closure=None, **kargs):
        timer, ep = self.timer_of(kargs), self.epoch_of(kargs)
        if self.impl == "fused":
            with timer("sync.gossip_fused", epoch=ep):
                bits = self.prepare_step()
                self.launch()
            return bits
        self.local_index += 1
        return self._step_torch(timer, ep)

    def reset_consensus_state(self):
        """Zero x_hat and s (all survivors do this together after the graph changed)."""
        self.finalize()
        self.x_hat.zero_()
        self.s.zero_()

    def finalize(self):
        if self.impl == "fused":
            self.engine.flush(self)
        else:
            self._finish_sync()

    def algo_state(self):
        self.finalize()
        return {"x_hat": self.x_hat, "s": self.s, "gossip_step": self.gossip_step}

    def load_algo_state(self, st):
        if "x_hat" in st:
            self.x_hat.copy_(st["x_hat"])
            self.s.copy_(st["s"])
            self.gossip_step = int(st.get("gossip_step", 0))
            if self.engine is not None:
                self.engine.reset_step(self.gossip_step)
