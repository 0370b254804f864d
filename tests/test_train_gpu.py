"""End-to-end checks on a GPU: the bf16 kernel path against the fp32 CPU model,
and the CUDA-graph trainer against the eager trainer."""

import copy
import tempfile

import pytest
import torch

import speculators_b200 as sb
from speculators_b200.train import Trainer, TrainerConfig
from speculators_b200.train.synthetic import SyntheticLoader

from conftest import make_tiny_batch, make_tiny_eagle3

pytestmark = pytest.mark.gpu


def _trainer(model, batch, graph):
    kwargs, _ = sb.Eagle3DraftModel.get_trainer_kwargs(loss_fn="kl_div", ttt_steps=3, ttt_step_loss_decay=1.0)
    return Trainer(model, TrainerConfig(lr=1e-3, num_epochs=1, save_path=tempfile.mkdtemp(), train_call_kwargs=kwargs,
                                        scheduler_type="none", log_freq=10**9, use_cuda_graph=graph, device="cuda:0"),
                   SyntheticLoader([batch], 4))


def test_gpu_loss_matches_cpu_fp32(tiny_verifier_dir, tiny_vocab_maps):
    model = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps, num_layers=2)
    batch = make_tiny_batch(T=40)
    kwargs, _ = sb.Eagle3DraftModel.get_trainer_kwargs(loss_fn="kl_div", ttt_steps=3, ttt_step_loss_decay=1.0)
    _, loss_cpu, m_cpu = model(**batch, **kwargs)
    gpu = copy.deepcopy(model).to("cuda", torch.bfloat16)
    _, loss_gpu, m_gpu = gpu(**{k: v.cuda() for k, v in batch.items()}, **kwargs)
    assert abs(float(loss_gpu) - float(loss_cpu)) < 0.05 * abs(float(loss_cpu)) + 0.05
    loss_gpu.backward()
    assert all(torch.isfinite(p.grad).all() for p in gpu.parameters() if p.requires_grad)


def test_graph_and_eager_trainers_agree_and_learn(tiny_verifier_dir, tiny_vocab_maps):
    base = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps)
    batch = make_tiny_batch(T=64, docs=(20, 30, 10), pad=4)
    t_eager = _trainer(copy.deepcopy(base), batch, graph=False)
    t_graph = _trainer(copy.deepcopy(base), batch, graph=True)
    le = [float(t_eager.train_step(batch)[0].item()) for _ in range(5)]
    lg = [float(t_graph.train_step(batch)[0].item()) for _ in range(5)]
    assert le[-1] < le[0] and lg[-1] < lg[0]
    for a, b in zip(le, lg):
        assert abs(a - b) < 2e-2 * abs(a) + 1e-3, (le, lg)
    assert t_graph._graphed is not None and len(t_graph._graphed.cache) == 1


def test_async_step_returns_every_loss_through_pinned_handles(tiny_verifier_dir, tiny_vocab_maps):
    """``train_step_async``: the loss of step n is read after step n + 1 was enqueued and is
    the value a synchronous ``train_step`` on an identical trainer reports for step n."""
    base = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps)
    batch = make_tiny_batch(T=64, docs=(20, 30, 10), pad=4)
    sync, lagged = _trainer(copy.deepcopy(base), batch, graph=True), _trainer(copy.deepcopy(base), batch, graph=True)
    want = [float(sync.train_step(batch)[0].item()) for _ in range(6)]
    got, pending = [], None
    for _ in range(6):
        handle = lagged.train_step_async(batch, batch)
        if pending is not None:
            got.append(pending.value())
        pending = handle
    got.append(pending.value())
    assert got == pytest.approx(want, rel=1e-5, abs=1e-6)


def test_fused_step_tail_matches_op_by_op_metrics():
    """One-launch tail (masked mean, decay, accuracy counters, prev_correct update) against
    the same quantities computed with separate torch ops, forward and backward."""
    from speculators_b200.models.eagle3 import metrics as em

    torch.manual_seed(0)
    T, V = 300, 512
    targets = (torch.randn(1, T, V, device="cuda") * 2).to(torch.bfloat16)
    mask = torch.rand(1, T, device="cuda") > 0.4
    results = {}
    for fused in (True, False):
        em.USE_FUSED_TAIL = fused
        logits = (torch.randn(1, T, V, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)) * 2).to(torch.bfloat16).requires_grad_()
        prev = mask.clone()
        total, log = torch.zeros((), device="cuda"), {}
        for step in range(3):
            # make some predictions right so that the conditional counters are not trivial
            with torch.no_grad():
                lg = logits.detach().clone()
                hit_rows = torch.arange(0, T - step, 3, device="cuda")
                lg[0, hit_rows, targets[0, hit_rows + step].argmax(-1)] = 50.0
            lg.requires_grad_()
            loss, m = em.compute_metrics(lg, targets, mask, prev, step, 0.8)
            loss.backward()
            total = total + loss.detach()
            log.update({k: float(v) for k, v in m.items()})
            log[f"grad_{step}"] = lg.grad.float().abs().sum().item()
        results[fused] = (float(total), log, prev.clone())
    em.USE_FUSED_TAIL = True
    (lf, mf, pf), (lo, mo, po) = results[True], results[False]
    assert abs(lf - lo) <= 1e-4 * abs(lo) + 1e-6 and torch.equal(pf, po)
    assert set(mf) == set(mo)
    for key in mo:
        assert abs(mf[key] - mo[key]) <= 1e-4 * abs(mo[key]) + 1e-5, (key, mf[key], mo[key])
    assert mo["cond_acc_1_total"] < mo["cond_acc_0_total"] and mo["full_acc_0_sum"] > 0


@pytest.mark.parametrize("graph", [True, False])
def test_prefetched_inputs_give_the_same_steps(tiny_verifier_dir, tiny_vocab_maps, graph):
    """``train_step(batch, next_batch)`` stages the next batch on a side stream (graph replay: one staging set
    copied into the graph's inputs; eager steps: two alternating sets, since a step reads its inputs until its
    backward pass ends); the losses must equal those of the plain call sequence, also when the announced batch
    is not the one that arrives."""
    base = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps)
    seq = [{k: v.pin_memory() for k, v in make_tiny_batch(T=64, docs=(20, 30, 10), pad=4, seed=s).items()} for s in (0, 1, 2)]
    order = [0, 1, 2, 1, 0, 2, 2, 1]
    plain = _trainer(copy.deepcopy(base), seq[0], graph=graph)
    ahead = _trainer(copy.deepcopy(base), seq[0], graph=graph)
    want = [float(plain.train_step(seq[i])[0].item()) for i in order]
    got = []
    for n, i in enumerate(order):
        nxt = seq[order[n + 1]] if n + 1 < len(order) else None
        if n == 2:
            nxt = seq[0]  # a wrong announcement: the staged copy must be ignored at the next call
        got.append(float(ahead.train_step(seq[i], nxt)[0].item()))
    assert got == want


def test_engine_flat_gradients_match_plain_autograd(tiny_verifier_dir, tiny_vocab_maps):
    """Weight gradients accumulated in place into the flat buffer by ``ops.linear``
    equal the gradients plain autograd produces for the same bf16 model."""
    from speculators_b200.parallel import EngineConfig, TrainEngine

    base = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps, num_layers=2)
    batch = {k: v.cuda() for k, v in make_tiny_batch(T=64, docs=(20, 30, 10), pad=4).items()}
    kwargs, _ = sb.Eagle3DraftModel.get_trainer_kwargs(loss_fn="kl_div", ttt_steps=3, ttt_step_loss_decay=1.0)
    plain = copy.deepcopy(base).to("cuda", torch.bfloat16)
    plain(**batch, **kwargs)[1].backward()
    flat_model = copy.deepcopy(base)
    engine = TrainEngine(flat_model, EngineConfig(compute_dtype=torch.bfloat16), device="cuda")
    engine.zero_grad()
    flat_model(**batch, **kwargs)[1].backward()
    ref = dict(plain.named_parameters())
    for name, p in flat_model.named_parameters():
        if not p.requires_grad:
            continue
        a, b = p.grad.float(), ref[name].grad.float()
        assert float((a - b).abs().max()) <= 0.03 * float(b.abs().max()) + 1e-3, name
    # zero_grad leaves the matrices uncleared and flags them: a second backward without it
    # accumulates, one after it starts over, and a weight no backward touched is cleared
    # by the optimizer step
    first = engine.flat_g.float().clone()
    flat_model(**batch, **kwargs)[1].backward()
    twice = engine.flat_g.float()
    assert float((twice - 2 * first).abs().max()) <= 0.03 * float(first.abs().max()) + 1e-3
    engine.zero_grad()
    flat_model(**batch, **kwargs)[1].backward()
    assert float((engine.flat_g.float() - first).abs().max()) <= 0.03 * float(first.abs().max()) + 1e-3
    engine.zero_grad()
    before = engine.flat_w.float().clone()
    engine.step(lr=0.0)  # nothing was back-propagated: every gradient must read as zero
    assert float(engine.flat_g.float().abs().max()) == 0.0
    assert float(engine.grad_norm()) == 0.0 and torch.equal(engine.flat_w.float(), before)


def test_bf16_gradient_pipeline_tracks_an_fp32_run_for_200_steps(tiny_verifier_dir, tiny_vocab_maps):
    """Gradients here are bf16 end to end (weight gradients accumulate in bf16 over the TTT
    passes, the optimizer reads bf16), where the reference keeps fp32 ``.grad``.  Pin what that
    costs: the GPU trainer (bf16 weights, activations and gradients, fp32 master weights) and
    an all-fp32 CPU trainer start from the same weights and see the same eight batches for 200
    steps; the loss curves must stay together and end at the same level."""
    base = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps)
    batches = [make_tiny_batch(T=64, docs=(20, 30, 10), pad=4, seed=s) for s in range(8)]
    kwargs, _ = sb.Eagle3DraftModel.get_trainer_kwargs(loss_fn="kl_div", ttt_steps=3, ttt_step_loss_decay=1.0)

    def make(device, graph):
        return Trainer(copy.deepcopy(base), TrainerConfig(lr=2e-3, num_epochs=1, save_path=tempfile.mkdtemp(), train_call_kwargs=kwargs,
                                                          scheduler_type="none", log_freq=10**9, use_cuda_graph=graph, device=device),
                       SyntheticLoader(batches, 200))

    gpu, cpu = make("cuda:0", True), make("cpu", False)
    lg, lc = [], []
    for step in range(200):
        b = batches[step % len(batches)]
        lg.append(gpu.train_step(b)[0].detach().float().reshape(1).clone())
        lc.append(float(cpu.train_step(b)[0]))
    lg = torch.cat(lg).cpu().tolist()
    assert lc[-1] < 0.7 * lc[0] and lg[-1] < 0.7 * lg[0]  # both learn
    gaps = [abs(a - b) / max(abs(b), 1e-3) for a, b in zip(lg, lc)]
    assert max(gaps[:20]) < 0.03, max(gaps[:20])  # same trajectory at the start ...
    tail_g, tail_c = sum(lg[-16:]) / 16, sum(lc[-16:]) / 16
    assert abs(tail_g - tail_c) < 0.08 * tail_c + 0.01, (tail_g, tail_c)  # ... and the same level after 200 steps
    assert sum(gaps) / len(gaps) < 0.15, sum(gaps) / len(gaps)  # step-by-step the two runs drift apart (measured: 0.07), the level stays


def test_muon_on_gpu_tracks_the_fp32_engine():
    """Muon with the iteration on the package's GEMM and the two element-wise kernels (bf16
    weights on a GPU) against the same engine in fp32 on the CPU, from the same init."""
    from torch import nn

    from speculators_b200.models.layers import Linear
    from speculators_b200.parallel.engine import EngineConfig, TrainEngine

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(0)
            self.a, self.b, self.c = Linear(256, 512), Linear(512, 128), Linear(128, 384)
            self.gain = nn.Parameter(torch.ones(384))

        def forward(self, x):
            return self.c(torch.tanh(self.b(torch.tanh(self.a(x))))) * self.gain

    cfg = dict(lr=1e-3, optimizer="muon", muon_lr=0.02, max_grad_norm=1.0)
    cpu_net = Net()
    gpu_net = copy.deepcopy(cpu_net)
    e_cpu = TrainEngine(cpu_net, EngineConfig(**cfg, compute_dtype=torch.float32), device="cpu")
    e_gpu = TrainEngine(gpu_net, EngineConfig(**cfg, compute_dtype=torch.bfloat16), device="cuda:0")
    from speculators_b200 import ops

    before = ops.native().launch_count()
    for step in range(5):
        g = torch.Generator().manual_seed(step)
        x, y = torch.randn(96, 256, generator=g), torch.randn(96, 384, generator=g)
        for net, eng, dev, dt in ((cpu_net, e_cpu, "cpu", torch.float32), (gpu_net, e_gpu, "cuda:0", torch.bfloat16)):
            eng.zero_grad()
            ((net(x.to(dev, dt)).float() - y.to(dev)) ** 2).mean().backward()
            eng.step()
    torch.cuda.synchronize()
    ops.check_gemm_status()
    assert ops.native().launch_count() - before > 5 * 3 * (2 + 3 * 5)  # momentum, apply and the iteration's GEMMs ran natively
    want, got = e_cpu.master_state_dict(), e_gpu.master_state_dict()
    for name in want:
        w, g_ = want[name], got[name].cpu()
        moved = (w - dict(Net().named_parameters())[name].detach()).abs().max()
        assert moved > 0
        # matrices: Newton-Schulz in bf16 against fp32; vectors (AdamW): the first steps are sign-like, bf16 gradients flip a few
        tol = 0.15 if w.ndim == 2 else 0.4
        assert (w - g_).abs().max() < tol * moved + 1e-4, (name, float((w - g_).abs().max()), float(moved))
