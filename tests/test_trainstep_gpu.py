"""TrainStep on a GPU: CUDA-graph replay, eager fused and the torch-path optimizer agree."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(arch, comm_op, impl, extra=()):
    from chocosgd_b200.config import get_args
    from chocosgd_b200.models import define_model
    from chocosgd_b200.optim import define_optimizer
    from chocosgd_b200.parallel.topology import Graph

    argv = ["--arch", arch, "--optimizer", "parallel_choco_v", "--comm_op", comm_op, "--graph_topology", "ring",
            "--lr", "0.05", "--momentum_factor", "0.9", "--use_nesterov", "True", "--weight_decay", "1e-4",
            "--consensus_stepsize", "0.3", "--gossip_impl", impl, "--drop_rate", "0.0"] + list(extra)
    if "compress" in comm_op:
        argv += ["--compress_ratio", "0.9"]
    if comm_op == "quantize_qsgd":
        argv += ["--quantize_level", "4"]
    conf = get_args(argv)
    graph = Graph("ring", 1, 0)
    torch.manual_seed(0)
    dl = {"n_tokens": 500} if arch == "rnn_lm" else None
    model = define_model(conf, graph, data_loader=dl, device=torch.device("cuda"), consistent=False, verbose=False)
    return conf, model, define_optimizer(conf, model, graph)


def _run_cv(impl, use_graph, comm_op, steps=6):
    from chocosgd_b200.train.engine import TrainStep
    from chocosgd_b200.train.metrics import Metrics

    conf, model, opt = _build("resnet20", comm_op, impl)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(16, 3, 32, 32, generator=g).pin_memory()
    y = torch.randint(0, 10, (16,), generator=g).pin_memory()
    step = TrainStep(model, torch.nn.CrossEntropyLoss(), opt, x, y, metrics=Metrics(model), use_cuda_graph=use_graph,
                     warmup_iters=1)
    model.train()
    losses = []
    n_calls = steps  # the warm-up steps of the graph capture are rolled back: every call is one step
    torch.backends.cudnn.benchmark = False
    torch.backends.cudnn.deterministic = True
    for _ in range(n_calls):
        losses.append(float(step(x, y)))
    opt.finalize()
    if opt.engine is not None:
        opt.engine.check()
    return losses, opt.arena.x.clone(), opt.local_index


@pytest.mark.parametrize("comm_op", ["sign", "compress_top_k"])
def test_graph_replay_equals_eager_fused(comm_op):
    # two steps: differences can only come from kernel-selection noise, not from amplification
    _, x_e2, n_e2 = _run_cv("fused", False, comm_op, steps=2)
    _, x_g2, n_g2 = _run_cv("fused", True, comm_op, steps=2)
    assert n_e2 == n_g2 == 2
    assert (x_e2 - x_g2).abs().max() < 2e-3 * x_e2.abs().max()
    # six steps of a tiny-batch ResNet amplify rounding noise: compare the loss only
    l_e, x_e, n_e = _run_cv("fused", False, comm_op)
    l_g, x_g, n_g = _run_cv("fused", True, comm_op)
    assert n_e == n_g == 6
    assert abs(l_e[-1] - l_g[-1]) < 5e-2 * abs(l_e[-1]) + 1e-3
    assert l_e[-1] < l_e[0]


def test_fused_kernels_equal_torch_path_in_training():
    _, x_f, _ = _run_cv("fused", False, "sign", steps=2)
    _, x_t, _ = _run_cv("nccl", False, "sign", steps=2)
    assert (x_f - x_t).abs().max() < 2e-3 * x_t.abs().max()
    l_f, _, _ = _run_cv("fused", False, "sign")
    l_t, _, _ = _run_cv("nccl", False, "sign")
    assert abs(l_f[-1] - l_t[-1]) < 5e-2 * abs(l_t[-1]) + 1e-3


def test_lstm_step_with_clipping_in_a_graph():
    from chocosgd_b200.train.engine import TrainStep
    from chocosgd_b200.train.metrics import Metrics

    outs = {}
    for use_graph in (False, True):
        conf, model, opt = _build("rnn_lm", "quantize_qsgd", "fused",
                                  ["--rnn_n_hidden", "64", "--rnn_n_layers", "2", "--rnn_clip", "0.4"])
        g = torch.Generator().manual_seed(2)
        x = torch.randint(0, 500, (8, 4), generator=g).pin_memory()
        y = torch.randint(0, 500, (8, 4), generator=g).pin_memory()
        hidden = tuple(h.cuda() for h in model.init_hidden(4))
        step = TrainStep(model, torch.nn.CrossEntropyLoss(), opt, x, y, metrics=Metrics(model, "language_modeling"),
                         use_cuda_graph=use_graph, clip_grad_norm=0.4, hidden=hidden, warmup_iters=1)
        model.train()
        n_calls = 6  # graph capture leaves no trace: every call is one step
        losses = [float(step(x, y)) for _ in range(n_calls)]
        opt.finalize()
        opt.engine.check()
        outs[use_graph] = (losses, opt.arena.x.clone(), float(step.perf[0]))
    assert outs[False][0][-1] < outs[False][0][0]
    assert abs(outs[True][0][-1] - outs[False][0][-1]) < 3e-2 * outs[False][0][-1]
    assert outs[True][2] > 1.0  # perplexity


def test_native_layers_in_a_step_count_batches_and_join_the_side_stream():
    """All native layer kinds inside TrainStep: every batch-norm counter advances once per step
    (one fused add); the weight gradients computed on the side stream reach the update, eagerly
    and from the CUDA graph (same kernels: parameters agree after two steps); against the library
    ops the first loss agrees and training makes progress."""
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.train.engine import TrainStep

    def run(native, use_graph, steps):
        nnn.configure_native("all" if native else "off")
        try:
            conf, model, opt = _build("resnet20", "sign", "fused")
            g = torch.Generator().manual_seed(1)
            x = torch.randn(32, 3, 32, 32, generator=g).pin_memory()
            y = torch.randint(0, 10, (32,), generator=g).pin_memory()
            step = TrainStep(model, torch.nn.CrossEntropyLoss(), opt, x, y, use_cuda_graph=use_graph, warmup_iters=1)
            model.train()
            n_calls = steps  # graph capture leaves no trace: every call is one step
            losses = [float(step(x, y)) for _ in range(n_calls)]
            opt.finalize()
            opt.engine.check()
            counters = [int(m.num_batches_tracked) for m in model.modules() if isinstance(m, torch.nn.BatchNorm2d)]
            return losses, counters, opt.local_index, opt.arena.x.clone()
        finally:
            nnn.configure_native("off")

    _, c_e, n_e, x_e = run(True, False, 2)
    _, c_g, n_g, x_g = run(True, True, 2)
    assert n_e == n_g == 2 and set(c_e) == set(c_g) == {2}
    assert (x_e - x_g).abs().max() < 2e-3 * x_e.abs().max()
    l_n, c_n, n_n, _ = run(True, True, 6)
    l_r, c_r, n_r, _ = run(False, False, 6)
    assert n_n == n_r == 6 and c_n == c_r and set(c_n) == {6}
    assert abs(l_n[0] - l_r[0]) < 0.02 * abs(l_r[0])  # same first step: the capture's warm-up left no trace
    assert l_n[-1] < l_n[0] and l_r[-1] < l_r[0]


def test_gossip_issued_bucket_by_bucket_during_backward_equals_one_launch():
    """Sign codec: the step launched per bucket of tensors from gradient hooks (side stream, inside the
    captured graph) gives the same parameters as the single launch after the backward pass."""
    from chocosgd_b200.train.engine import TrainStep
    from chocosgd_b200.train.metrics import Metrics

    def run(bucket_mb):
        conf, model, opt = _build("resnet20", "sign", "fused")
        g = torch.Generator().manual_seed(1)
        x = torch.randn(16, 3, 32, 32, generator=g).pin_memory()
        y = torch.randint(0, 10, (16,), generator=g).pin_memory()
        step = TrainStep(model, torch.nn.CrossEntropyLoss(), opt, x, y, metrics=Metrics(model), use_cuda_graph=True,
                         warmup_iters=1, gossip_bucket_mb=bucket_mb)
        model.train()
        torch.backends.cudnn.benchmark = False
        torch.backends.cudnn.deterministic = True
        for _ in range(3):
            step(x, y)
        opt.finalize()
        opt.engine.check()
        assert opt.engine.step_index() >= 3
        return opt.arena.x.clone(), opt.x_hat.clone(), step.kernel_launches_per_step, bool(step._bucket_bytes)

    x1, h1, n1, b1 = run(0.0)
    x2, h2, n2, b2 = run(0.2)      # 1.1 MB of parameters -> 6 buckets
    assert not b1 and b2 and n2 > n1
    assert (x1 - x2).abs().max() <= 2e-3 * x1.abs().max()
    assert (h1 - h2).abs().max() <= 2e-3 * h1.abs().max() + 1e-6
