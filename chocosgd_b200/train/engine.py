"""One training step as a replayable unit.

``TrainStep`` is the public call a user makes per batch::

    step = TrainStep(model, criterion, optimizer, example_input, example_target)
    loss = step(input_from_pinned_host_memory, target)        # device 0-d tensor

With a capturable (fused) optimizer on CUDA the whole step - forward, loss, backward,
gradient clipping, the fused SGD/gossip kernels, metric accumulation - is captured once in a
CUDA graph and replayed; the host only copies the batch into static buffers, refreshes the
device-resident learning rate when it changes, and launches the graph.  Gradients are not
packed: the update kernels read each tensor's gradient where autograd produced it, through a
pointer table.  On CPU, or with an optimizer that communicates through ``torch.distributed``,
the same object runs eagerly.

The reference's loop does this on the host every step with per-tensor launches and three
``.item()`` synchronisations (``dl_code/pcode/distributed_running_cv.py:42-62,154-161``).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops.ce import criterion_is_plain_ce, cross_entropy as fused_cross_entropy, supported as ce_supported
from ..ops.sgd import grad_clip_


class TrainStep:
    def __init__(
        self,
        model,
        criterion,
        optimizer,
        example_input: torch.Tensor,
        example_target: torch.Tensor,
        metrics=None,
        use_cuda_graph: bool = True,
        clip_grad_norm: Optional[float] = None,
        hidden=None,
        amp_dtype: Optional[torch.dtype] = None,
        warmup_iters: int = 3,
        channels_last: Optional[bool] = None,
        gossip_bucket_mb: float = 0.0,
    ):
        self.model, self.criterion, self.opt, self.metrics = model, criterion, optimizer, metrics
        self.device = optimizer.device
        self.clip = clip_grad_norm
        self.amp_dtype = amp_dtype
        if channels_last is None:
            channels_last = any(optimizer.arena.channels_last)
        self.channels_last = channels_last
        self.is_cuda = self.device.type == "cuda"
        self.fused = bool(getattr(optimizer, "capturable", False))
        self.use_graph = bool(use_cuda_graph and self.is_cuda and self.fused)
        self.static_input = torch.zeros(example_input.shape, dtype=example_input.dtype, device=self.device)
        if channels_last and self.static_input.dim() == 4:
            self.static_input = self.static_input.contiguous(memory_format=torch.channels_last)
        self.static_target = torch.zeros(example_target.shape, dtype=example_target.dtype, device=self.device)
        self.hidden = hidden  # tuple of static tensors for recurrent models
        self.loss = torch.zeros((), dtype=torch.float32, device=self.device)
        n_perf = len(metrics.metric_names) if metrics is not None else 0
        self.perf = torch.zeros(n_perf, dtype=torch.float32, device=self.device)
        self.graph = None
        self.h2d_bytes = example_input.numel() * example_input.element_size() + (
            example_target.numel() * example_target.element_size())
        self._warm = 0
        self._warmup_iters = warmup_iters
        self.kernel_launches_per_step = None
        self.flips = None
        self.bn_counters = None
        self._fused_ce = False
        self._copy_stream = None
        # gossip bucket by bucket from gradient hooks, overlapped with the rest of the backward pass
        # (captured step, per-tensor codec, no global-norm clipping, at least two buckets)
        self._bucket_bytes = 0
        if (gossip_bucket_mb and self.use_graph and clip_grad_norm is None
                and getattr(optimizer, "supports_buckets", lambda: False)()):
            nbytes = int(gossip_bucket_mb * (1 << 20))
            if len(optimizer.bucket_plan(nbytes)) >= 2:
                self._bucket_bytes = nbytes
                self._gossip_stream = torch.cuda.Stream(device=self.device)
        if self.is_cuda:
            from ..ops import nn as native_nn

            self._fused_ce = native_nn.native_enabled("ce") and criterion_is_plain_ce(criterion)

            if native_nn.native_enabled("bn"):
                from ..ops.bn import BnCounters

                self.bn_counters = BnCounters(model)

            if native_nn.native_enabled("conv"):
                from ..ops.conv import FlippedWeights

                self.flips = FlippedWeights(model)

    # ---- the step body (captured or eager) ------------------------------------------------------
    def _forward_backward(self):
        params = self.opt.arena.params
        if self.flips is not None:
            from ..ops.conv import set_active_flips

            self.flips.refresh()  # one kernel: flipped filters of every native convolution
            set_active_flips(self.flips)
        if self.flips is not None:
            from ..ops.conv import FUSION

            FUSION.clear()   # hand-over tables between layers are per step
        if self.bn_counters is not None and self.model.training:
            self.bn_counters.tick()  # one add for all batch-norm step counters
        if self.fused:
            for p in params:
                p.grad = None  # autograd then hands over its own gradient tensors (no accumulate kernels)
        ctx = torch.autocast("cuda", dtype=self.amp_dtype) if self.amp_dtype is not None else _null()
        stats = None
        with ctx:
            if self.hidden is not None:
                h = tuple(t.detach() for t in self.hidden)
                out, new_h = self.model(self.static_input, h)
                logits, tgt = out.reshape(-1, out.size(-1)), self.static_target.reshape(-1)
            else:
                fused_head = None
                if self._fused_ce and self.amp_dtype is None and hasattr(self.model, "head_loss"):
                    feat = self.model.forward_features(self.static_input)
                    fused_head = self.model.head_loss(feat, self.static_target)
                    out = None if fused_head is not None else self.model.classify(feat)
                else:
                    out = self.model(self.static_input)
                logits, tgt = out, self.static_target
            if self.hidden is None and fused_head is not None:
                loss, stats = fused_head          # pooling + classifier + loss + accuracies: one kernel
            elif self._fused_ce and logits.dim() == 2 and ce_supported(logits, tgt):
                loss, stats = fused_cross_entropy(logits, tgt, True)  # loss, gradient, accuracies: one kernel
            else:
                loss = self.criterion(logits, tgt)
        loss.backward()
        if self.flips is not None:
            self.flips.valid = False
        with torch.no_grad():
            if self.hidden is not None:
                for dst, src in zip(self.hidden, new_h):
                    dst.copy_(src.detach())
            self.loss.copy_(loss.detach().float())
            if self.metrics is not None:
                if stats is not None and self.metrics.task == "classification":
                    self.perf.copy_(stats[1:1 + len(self.metrics.metric_names)])
                else:
                    perf = self.metrics.evaluate(loss, logits.float(), tgt)
                    self.perf.copy_(torch.stack([p.float() for p in perf]))
        return loss

    # ---- side-effect-free warm-up --------------------------------------------------------------
    def _snapshot(self):
        """Everything the warm-up steps change: parameters, momentum, the algorithm's state tensors,
        module buffers (batch-norm statistics and counters), the recurrent state, host counters."""
        opt = self.opt
        algo = {k: v.clone() for k, v in opt.algo_state().items() if torch.is_tensor(v)}
        return {
            "x": opt.arena.x.clone(),
            "m": None if opt.momentum_buf is None else opt.momentum_buf.clone(),
            "algo": algo,
            "buffers": [b.clone() for b in self.model.buffers()],
            "hidden": None if self.hidden is None else [h.clone() for h in self.hidden],
            "local_index": opt.local_index, "n_bits": opt.n_bits,
            "mom_flags": opt.engine.momentum_flags(),
        }

    def _restore(self, snap):
        opt = self.opt
        opt.finalize()                       # apply the exchange still in flight, then roll back
        live = opt.algo_state()
        with torch.no_grad():
            opt.arena.x.copy_(snap["x"])
            if snap["m"] is not None:
                opt.momentum_buf.copy_(snap["m"])
            elif opt.momentum_buf is not None:
                opt.momentum_buf.zero_()
            for k, v in snap["algo"].items():
                live[k].copy_(v)
            for b, v in zip(self.model.buffers(), snap["buffers"]):
                b.copy_(v)
            if snap["hidden"] is not None:
                for h, v in zip(self.hidden, snap["hidden"]):
                    h.copy_(v)
        opt.local_index, opt.n_bits = snap["local_index"], snap["n_bits"]
        opt.engine.set_momentum_flags(snap["mom_flags"])
        opt.engine.rebase_time()

    def prime(self):
        """Build the CUDA graph.  The warm-up iterations that capture needs run as real steps on
        the data currently in the static buffers, then every effect of theirs is rolled back
        (parameters, momentum, x_hat / s / memories, batch-norm statistics, recurrent state), so
        that the captured step replayed next is the first update of this batch: the graph path
        and the eager path follow the same trajectory.  Only the device-resident exchange
        counter keeps counting (it pairs with the mailbox flags of the neighbours, which ran the
        same warm-up).  Returns 1, the number of training steps the call amounts to."""
        if not self.use_graph or self.graph is not None:
            return 0
        snap = self._snapshot()
        # the table must exist (with its final address) before capture: create it from
        # placeholder gradients, capture, then point it at the captured gradients
        eng = self.opt.engine
        eng.set_grad_pointers(self.opt.rank, [torch.zeros_like(p) for p in self.opt.arena.params])
        table = eng._grad_tables[self.opt.rank][0]
        self._grad_ptrs_dirty = True
        self._capture_with_table(table)
        self._restore(snap)
        self.opt.prepare_step()
        self.graph.replay()              # the first real step on this batch
        return 1

    def _capture_with_table(self, table):
        eng = self.opt.engine
        # the step runs on a high-priority stream: kernels forked to side streams (weight
        # gradients) then fill the SMs that the critical path leaves idle instead of delaying it
        s = torch.cuda.Stream(priority=-1)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(self._warmup_iters):
                self.opt.prepare_step()
                self._forward_backward()
                self._fill_table(table)
                if self.clip is not None:
                    grad_clip_(eng, self.clip)
                self.opt.launch()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        for p in self.opt.arena.params:
            p.grad = None
        self.graph = torch.cuda.CUDAGraph()
        from ..ops import _lib

        n0 = _lib.LAUNCHES[0]
        with torch.cuda.graph(self.graph, stream=s):
            if self._bucket_bytes:
                from ..ops.conv import wgrad_side_stream

                ws = wgrad_side_stream(self.device)
                self.opt.arm_buckets(self._bucket_bytes, self._gossip_stream, (ws,) if ws is not None else ())
            self._forward_backward()
            if self.clip is not None:
                grad_clip_(eng, self.clip)
            self.opt.launch()
        # kernels of the native library inside one replay (library kernels are not counted)
        self.kernel_launches_per_step = _lib.LAUNCHES[0] - n0
        self._captured_grads = [p.grad for p in self.opt.arena.params]
        self._fill_table(table)
        torch.cuda.synchronize()
        return self._warmup_iters

    def _fill_table(self, table):
        grads = [p.grad for p in self.opt.arena.params]
        for gt, p in zip(grads, self.opt.arena.params):
            # same memory order as the parameter's segment (dense, same strides)
            assert gt is not None and gt.data_ptr() % 16 == 0
            assert all(a == b for a, b, n in zip(gt.stride(), p.stride(), p.shape) if n > 1), (gt.stride(), p.stride())
        host = torch.tensor([gt.data_ptr() for gt in grads], dtype=torch.int64)
        table.copy_(host)
        self._table_keepalive = grads

    # ---- public call -----------------------------------------------------------------------------
    def load_batch(self, inp: torch.Tensor, tgt: torch.Tensor):
        """Host batch -> static device buffers.  On CUDA the host-to-device copy runs on its own
        stream into a staging buffer, so the copy of batch i overlaps the (asynchronously running)
        step i-1; the step's stream then only does a device-to-device copy (which also converts to
        channels_last)."""
        if not self.is_cuda or inp.is_cuda:
            self.static_input.copy_(inp, non_blocking=True)
            self.static_target.copy_(tgt, non_blocking=True)
            return
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
            self._stage_in = torch.empty(inp.shape, dtype=self.static_input.dtype, device=self.device)
            self._stage_tgt = torch.empty(tgt.shape, dtype=self.static_target.dtype, device=self.device)
            self._ready, self._consumed = torch.cuda.Event(), torch.cuda.Event()
            self._consumed.record(torch.cuda.current_stream(self.device))
        cs, main = self._copy_stream, torch.cuda.current_stream(self.device)
        cs.wait_event(self._consumed)  # the staging buffers are free once the previous batch was taken over
        with torch.cuda.stream(cs):
            self._stage_in.copy_(inp, non_blocking=True)
            self._stage_tgt.copy_(tgt, non_blocking=True)
            self._ready.record(cs)
        main.wait_event(self._ready)
        self.static_input.copy_(self._stage_in)
        self.static_target.copy_(self._stage_tgt)
        self._consumed.record(main)

    def __call__(self, inp: Optional[torch.Tensor] = None, tgt: Optional[torch.Tensor] = None, **step_kw):
        """Run one training step; returns the loss as a 0-d device tensor (no host sync)."""
        if inp is not None:
            self.load_batch(inp, tgt)
        if self.use_graph:
            if self.graph is None:
                self.prime()
                return self.loss
            self.opt.prepare_step()
            self.graph.replay()
            return self.loss
        if self.fused:
            eng = self.opt.engine
            self.opt.prepare_step()
            self._forward_backward()
            if getattr(self, "_eager_table", None) is None:
                eng.set_grad_pointers(self.opt.rank, [p.grad for p in self.opt.arena.params])
                self._eager_table = eng._grad_tables[self.opt.rank][0]
            else:
                self._fill_table(self._eager_table)
            if self.clip is not None:
                grad_clip_(eng, self.clip)
            self.opt.launch()
            return self.loss
        # eager path with a torch.distributed / CPU optimizer: gradients alias the flat arena
        self.opt.arena.rebind() if self.opt.arena.params[0].grad is None else None
        self._forward_backward()
        if self.clip is not None:
            g = self.opt.arena.g
            norm = g.norm()
            g.mul_(torch.clamp(self.clip / (norm + 1e-6), max=1.0))
        self.opt.step(**step_kw)
        return self.loss

    @property
    def n_bits(self):
        return self.opt.n_bits


class _null:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False
