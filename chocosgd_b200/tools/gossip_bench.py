"""Gossip micro-benchmark: one CHOCO gossip step on a flat fp32 buffer (no model, zero gradient).

    python -m chocosgd_b200.tools.gossip_bench --sizes 1048576,16777216 --topology ring
    python -m torch.distributed.run --nproc-per-node 8 -m chocosgd_b200.tools.gossip_bench ...

For every (size, codec) it prints one JSON line: microseconds per step (CUDA events, max over
ranks), achieved local memory bandwidth, and the fraction of the roofline
``max(local bytes / HBM bandwidth, neighbour payload bytes / NVLink bandwidth)``.
``--impl torch`` times this framework's torch.distributed path (the same algorithm with
library send/recv and PyTorch ops).  ``--impl reference`` times the reference's own gossip step:
its ``ParallelCHOCO_V`` optimizer (``dl_code/pcode/optim/parallel_choco_v.py:104-155``: its
compressors, its ``DecentralizedAggregation`` send / recv, its helper thread) from the install
under ``baseline/_ref``, on a "model" that is one flat parameter of the same size with a zero
gradient, so a step is its local update plus one full gossip exchange.

Byte model of the roofline (what an ideal implementation must move per element, momentum off):
x, g, x_hat, s read and x, x_hat, s written and g cleared (32 B); sign adds its payload bits;
QSGD, top-k and random-k add one write and one read of the difference (the norm / the selection
threshold must be known before the payload can be produced), QSGD also its payload bits."""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..compress.reference import make_codec
from ..compress.segments import Segments
from ..parallel.topology import Graph

HBM_GBS_DEFAULT, NVLINK_GBS = 6560.3, 770.0


def measured_hbm():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def local_bytes_per_elem(comm_op, deg, nbits):
    """Algorithmic HBM traffic of one step per element (momentum off): x, g, x_hat, s read and
    x, x_hat, s written, the gradient cleared, plus scratch / payload traffic of the codec."""
    base = 4 * 4 + 4 * 4
    if comm_op == "sign":
        return base + (deg + 2) / 8.0
    if comm_op == "quantize_qsgd":
        return base + 8 + (nbits + 1) * (deg + 2) / 8.0
    if comm_op == "compress_top_k":
        return base + 8      # one write + one re-read of the difference; 1 % payloads are negligible
    return base + 8


def reference_step(rank, world, topology, comm_op, n, dev):
    """One gossip step of the reference's own ``ParallelCHOCO_V`` on a flat parameter of ``n``
    elements.  Harness glue as in ``baseline/reference_arm.py`` (pure-PyTorch ``bit2byte``, batched
    NCCL send / recv, its ``complete`` graph where its ring refuses n <= 2)."""
    import argparse as _ap
    import sys

    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, os.path.join(root, "baseline"))
    import reference_arm as ref

    if not ref.available():
        raise SystemExit(json.dumps({"bench": "gossip", "impl": "reference",
                                     "unavailable": "reference not installed under baseline/_ref"}))
    if "compress" in comm_op and n > (1 << 24):
        # The reference ships sparse indices inside an fp32 message (exact only below 2^24); above that
        # an index can round up to n, and its scatter then trips a device-side assert (seen once at
        # 2^27 elements with random-k).  Such inputs are not given to it.
        return None, None, 0, 0
    if ref.REF not in sys.path:
        sys.path.insert(0, ref.REF)
    ref.install_bit2byte_shim()
    import pcode.create_optimizer as create_optimizer
    import pcode.utils.communication as communication
    import pcode.utils.topology as topo_mod
    from pcode.optim.utils import join_thread
    from pcode.utils.timer import Timer

    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29517")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    if not isinstance(communication.dist, ref.BatchedP2P):
        communication.dist = ref.BatchedP2P(dist)
    topo = topology if (world > 2 or topology == "complete") else "complete"
    conf = _ap.Namespace(
        arch="flat", optimizer="parallel_choco_v", comm_op=comm_op, compress_ratio=0.99, quantize_level=4,
        is_biased=True, backend="nccl", use_ipc=False, consensus_stepsize=0.5, comm_device="cuda", weight_decay=0.0,
        lr=0.0, momentum_factor=0.0, use_nesterov=False, epoch_=0.5, local_index=0, distributed=True,
        graph_topology=topo, n_mpi_process=world, n_sub_process=1, on_cuda=True)
    conf.graph = topo_mod.define_graph_topology(topo, world=",".join(["0"] * world), n_mpi_process=world,
                                                n_sub_process=1, comm_device="cuda", on_cuda=True, rank=rank)

    class Flat(torch.nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(rank)
            self.weight = torch.nn.Parameter(torch.randn(n, device=dev))

    model = Flat()
    opt = create_optimizer.define_optimizer(conf, model)
    timer = Timer(verbosity_level=0, on_cuda=True)
    model.weight.grad = torch.zeros_like(model.weight)

    def step():
        opt.step(timer=timer, scheduler=None)

    def join():
        th = getattr(opt, "helper_thread", None)
        if th is not None:
            join_thread(th)
        torch.cuda.synchronize()

    k = max(1, int(n * 0.01))
    payload = {"sign": 4 * ((n + 31) // 32 + 1), "quantize_qsgd": 4 * n, "compress_top_k": 8 * k,
               "compress_random_k": 8 * k}[comm_op]
    return step, {"join": join, "opt": opt, "model": model}, 4, payload


def run(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    hbm, hbm_src = measured_hbm()
    graph = Graph(args.topology, world, rank)
    deg = len(graph.neighbors())
    for n in [int(s) for s in args.sizes.split(",")]:
        for comm_op in args.comm_ops.split(","):
            seg = Segments.from_sizes([n])
            kw = dict(compress_ratio=0.99 if "compress" in comm_op else None,
                      qsgd_levels=16 if comm_op == "quantize_qsgd" else None)
            torch.manual_seed(rank)
            x = torch.randn(seg.total, device=dev)
            mk = lambda: torch.zeros(seg.total, device=dev)
            ref_state = None
            if args.impl == "reference":
                step, ref_state, nbits, payload_bytes = reference_step(rank, world, args.topology, comm_op, n, dev)
                launches = None
                del x
                x = None
                if step is None:
                    if rank == 0:
                        print(json.dumps({"bench": "gossip", "impl": "reference", "n_gpus": world, "elements": n,
                                          "topology": args.topology, "comm_op": comm_op,
                                          "unavailable": "the reference sends sparse indices as fp32 (exact below 2^24 "
                                                         "only); beyond that its scatter can index out of range"}),
                              flush=True)
                    continue
            elif args.impl == "fused":
                from ..ops.gossip import ChocoEngine, RankBuffers
                from ..parallel.symm import DistributedMailbox, LoopbackMailbox

                bufs = {rank: RankBuffers(x, mk(), mk(), mk(), mk())}
                mb = (lambda pw: DistributedMailbox(graph, pw, dev)) if world > 1 else (
                    lambda pw: LoopbackMailbox({rank: []}, pw, dev))
                coop = None if args.coop == "auto" else args.coop == "on"
                eng = ChocoEngine([rank], bufs, {rank: graph.get_neighborhood()}, seg, [0.0], comm_op, mb, dev, coop=coop,
                                  **kw)
                eng.set_hyper(0.0, 0.0, 0.5, False)
                step = eng.launch_step
                nbits, payload_bytes, launches = eng.nbits, 4 * eng.payload_words, None
            else:
                codec = make_codec(seg, comm_op, kw["compress_ratio"], None, kw["qsgd_levels"])
                from ..parallel.comm import DecentralizedAggregation

                agg = DecentralizedAggregation(rank, graph.get_neighborhood())
                x_hat, s, state = mk(), mk(), {"t": 0}
                nb = graph.get_neighborhood()

                def step():
                    x.add_(s - x_hat, alpha=0.5)
                    payload = codec.compress(x - x_hat, state["t"], rank)
                    got = agg._agg(payload, op="get_raw_sync_data")
                    for r, w in nb.items():
                        q = codec.decompress(got[r], state["t"], r)
                        if r == rank:
                            x_hat.add_(q)
                        s.add_(q, alpha=w)
                    state["t"] += 1

                nbits, payload_bytes, launches = getattr(codec, "nbits", 0), 4 * codec.payload_words(), None
            for _ in range(args.warmup):
                step()
            torch.cuda.synchronize()
            cg = None
            if args.impl == "fused" and args.graph:
                # replay the step from a CUDA graph, as the training loop does: the number is
                # device time per step, not host launch overhead
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    step()
                torch.cuda.current_stream().wait_stream(side)
                cg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(cg):
                    step()
                step = cg.replay
                step()
                torch.cuda.synchronize()
            if ref_state is not None:
                ref_state["join"]()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                step()
            if ref_state is not None:
                ref_state["join"]()   # the exchange of the last step completes inside the timed region
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if world > 1:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t)
            if args.impl == "fused":
                eng.flush()
                launches = eng.launches_per_step
            us = 1e3 * ms / args.steps
            lb = local_bytes_per_elem(comm_op, deg, nbits) * n
            t_hbm, t_link = lb / (hbm * 1e9), deg * payload_bytes / (NVLINK_GBS * 1e9)
            roof = max(t_hbm, t_link)
            if rank == 0:
                print(json.dumps({
                    "bench": "gossip", "impl": args.impl, "n_gpus": world, "topology": args.topology, "elements": n,
                    "comm_op": comm_op, "us_per_step": round(us, 2), "payload_bytes_per_peer": payload_bytes,
                    "achieved_local_GBps": round(lb / (us * 1e-6) / 1e9, 1),
                    "roofline_us": round(roof * 1e6, 2), "bound": "hbm" if t_hbm >= t_link else "nvlink",
                    "roofline_frac": round(roof / (us * 1e-6), 3), "hbm_peak": f"{hbm} GB/s ({hbm_src})",
                    "kernels_per_step": launches, "cuda_graph": bool(args.impl == "fused" and args.graph), "inputs": "buffers >> L2 for n >= 16M; no flush below"}), flush=True)
            if args.impl == "fused":
                if world > 1:
                    dist.barrier()
                eng.close()
            del x, step, ref_state
            torch.cuda.empty_cache()
    if world > 1:
        dist.destroy_process_group()


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--sizes", default="1048576,16777216,134217728")
    p.add_argument("--comm_ops", default="sign,compress_top_k,compress_random_k,quantize_qsgd")
    p.add_argument("--topology", default="ring")
    p.add_argument("--impl", default="fused", choices=("fused", "torch", "reference"))
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--graph", type=int, default=1)
    p.add_argument("--coop", default="auto", choices=("auto", "on", "off"),
                   help="top-k / random-k step as one cooperative kernel (auto: the engine's default, the kernel chain)")
    run(p.parse_args(argv))


if __name__ == "__main__":
    main()
