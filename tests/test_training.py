"""Training utilities on CPU: LoRA, optimizers against torch.optim, schedules, losses, trainer, gradient checkpointing."""
import math

import pytest
import torch

from oxibonsai_b200 import training as TR
from oxibonsai_b200.core import Qwen3Config


def test_lora_adapter_is_a_noop_until_trained_and_merges_exactly():
    cfg = TR.LoraConfig(rank=4, alpha=8.0)
    a = TR.LoraAdapter(16, 12, cfg, seed=1)
    x, w = torch.randn(5, 16), torch.randn(12, 16)
    base = x @ w.T
    assert torch.equal(a(x, base), base) and a.param_count() == 4 * (16 + 12) and cfg.scale == 2.0
    with torch.no_grad():
        a.B.normal_()
    merged = a.merge_into_weights(w)
    assert torch.allclose(x @ merged.T, a(x, base), atol=1e-5) and a.memory_bytes() == a.param_count() * 4
    reg = TR.LoraRegistry(cfg)
    reg.add("blk.0.attn_q", 16, 12)
    assert torch.equal(reg.apply_adapter("missing", x, base), base) and reg.adapter_count() == 1 and reg.module_names() == ["blk.0.attn_q"]
    assert TR.LoraRegistry.estimate_adapters_for_budget(1 << 20, 4096, 4096, 8) == (1 << 20) // (8 * 8192 * 4)
    s = TR.BonsaiLoraSet(Qwen3Config(hidden=256, inter=512, layers=2, heads=4, kv_heads=2, head_dim=64), cfg).add_attention_adapters().add_mlp_adapters()
    assert s.registry.adapter_count() == 8 and 0 < s.efficiency_ratio(10_000_000) < 0.01
    assert s.total_trainable_params() == 2 * 4 * ((256 + 256) + (256 + 128) + (256 + 512) + (512 + 256))


@pytest.mark.parametrize("ours,theirs,kw", [
    (TR.Sgd, torch.optim.SGD, dict(lr=0.1, momentum=0.9, weight_decay=0.01)),
    (TR.Sgd, torch.optim.SGD, dict(lr=0.1, momentum=0.9, nesterov=True)),
    (TR.Adam, torch.optim.Adam, dict(lr=0.01, weight_decay=0.01)),
    (TR.AdamW, torch.optim.AdamW, dict(lr=0.01, weight_decay=0.1)),
])
def test_optimizers_match_torch(ours, theirs, kw):
    torch.manual_seed(0)
    w0 = torch.randn(6, 4)
    a, b = w0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
    oa, ob = ours([a], **kw), theirs([b], **kw)
    x, y = torch.randn(10, 4), torch.randn(10, 6)
    for _ in range(5):
        for p, o in ((a, oa), (b, ob)):
            o.zero_grad()
            ((x @ p.T - y) ** 2).mean().backward()
            o.step()
    assert torch.allclose(a, b, atol=1e-6)


def test_grad_clipping_and_schedules():
    p = torch.ones(4, requires_grad=True)
    (p * torch.tensor([3.0, 4.0, 0.0, 0.0])).sum().backward()
    assert TR.grad_norm([p]) == pytest.approx(5.0) and TR.clip_grad_norm([p], 1.0) == pytest.approx(5.0) and TR.grad_norm([p]) == pytest.approx(1.0, rel=1e-4)
    assert TR.ConstantLr(0.1).at(99) == 0.1 and TR.WarmupConstantLr(1.0, 10).at(4) == 0.5 and TR.WarmupConstantLr(1.0, 10).at(50) == 1.0
    c = TR.CosineAnnealingLr(1.0, 100, 0.1)
    assert c.at(0) == 1.0 and c.at(50) == pytest.approx(0.55) and c.at(100) == pytest.approx(0.1) and c.at(500) == pytest.approx(0.1)
    w = TR.LinearWarmupCosineDecay(1.0, 10, 110)
    assert w.at(4) == 0.5 and w.at(10) == pytest.approx(1.0) and w.at(60) == pytest.approx(0.5) and w.at(110) == pytest.approx(0.0, abs=1e-9)
    assert TR.PolynomialDecay(1.0, 100, 0.0, 2.0).at(50) == 0.25
    o = TR.OneCycleLr(1.0, 100, 0.3)
    assert o.at(0) == pytest.approx(0.04) and o.at(30) == pytest.approx(1.0) and o.at(100) == pytest.approx(0.0, abs=1e-9) and o.progress(50) == 0.5
    cy = TR.CyclicLr(0.1, 1.0, 10)
    assert cy.at(0) == pytest.approx(0.1) and cy.at(10) == pytest.approx(1.0) and cy.at(20) == pytest.approx(0.1) and cy.at(15) == pytest.approx(0.55)
    r = TR.ReduceOnPlateau(1.0, patience=1, factor=0.5, min_lr=0.3)
    lrs = [r.step(m) for m in (1.0, 0.9, 0.95, 0.95, 0.95, 0.95, 0.95, 0.95)]
    assert lrs[:3] == [1.0, 1.0, 1.0] and lrs[3] == 0.5 and lrs[-1] == 0.3 and r.times_reduced() == 2


def test_losses():
    torch.manual_seed(1)
    lg, t = torch.randn(6, 5), torch.tensor([0, 1, 2, 3, 4, 0])
    assert torch.allclose(TR.cross_entropy(lg, t), torch.nn.functional.cross_entropy(lg, t))
    assert torch.allclose(TR.label_smoothed_cross_entropy(lg, t, 0.1), torch.nn.functional.cross_entropy(lg, t, label_smoothing=0.1), atol=1e-6)
    assert torch.allclose(TR.label_smoothed_cross_entropy(lg, t, 0.0), TR.cross_entropy(lg, t)) and torch.allclose(TR.focal_loss(lg, t, 0.0), TR.cross_entropy(lg, t))
    assert TR.focal_loss(lg, t, 2.0) < TR.cross_entropy(lg, t)
    assert TR.kl_divergence(lg, lg) == pytest.approx(0.0, abs=1e-7) and TR.kl_divergence(lg, torch.randn(6, 5)) > 0
    assert torch.allclose(TR.distillation_loss(lg, lg, t, 2.0, 0.0), TR.cross_entropy(lg, t))
    a, b = torch.tensor([0.0, 3.0]), torch.tensor([0.5, 0.0])
    assert TR.mse(a, b) == pytest.approx((0.25 + 9) / 2) and TR.huber_loss(a, b, 1.0) == pytest.approx((0.125 + 2.5) / 2)
    e = torch.nn.functional.normalize(torch.randn(4, 8), dim=-1)
    assert TR.contrastive_loss(e, e) < TR.contrastive_loss(e, e.flip(0))
    lg2 = lg.clone().requires_grad_(True)
    TR.cross_entropy(lg2, t).backward()
    assert torch.allclose(lg2.grad, TR.cross_entropy_grad(lg, t), atol=1e-6)
    perfect = torch.full((4, 5), -30.0)
    toks = torch.tensor([0, 1, 2, 3])
    perfect[torch.arange(3), toks[1:]] = 30.0
    assert TR.sequence_perplexity(perfect, toks) == pytest.approx(1.0, abs=1e-5) and TR.ntp_loss(perfect, toks) < 1e-5


def test_lora_trainer_fits_a_low_rank_update():
    torch.manual_seed(0)
    w = torch.randn(12, 16)
    target_delta = torch.randn(12, 2) @ torch.randn(2, 16) * 0.3
    x = torch.randn(64, 16)
    y = x @ (w + target_delta).T
    reg = TR.LoraRegistry(TR.LoraConfig(rank=4, alpha=4.0))
    reg.add("lin", 16, 12, seed=3)
    tr = TR.LoraTrainer(reg, TR.LoraTrainingConfig(lr=0.05, total_steps=300, warmup_steps=10, max_grad_norm=10.0))
    while not tr.is_complete():
        s = tr.step(lambda: TR.mse(reg.apply_adapter("lin", x, x @ w.T), y))
    assert tr.total_steps() == 300 and tr.history[0].loss > 0.5 and tr.average_loss(10) < 0.02 and tr.convergence_rate() > 0.95
    assert s.lr < 0.05 and tr.last_step() is s and tr.history[4].lr == pytest.approx(0.025)


def test_gradient_checkpointing_gives_identical_gradients():
    torch.manual_seed(0)
    def make():
        torch.manual_seed(5)
        return [torch.nn.Sequential(torch.nn.Linear(8, 32), torch.nn.GELU(), torch.nn.Linear(32, 8)) for _ in range(3)]
    plain, ck = torch.nn.Sequential(*make()), TR.CheckpointedPipeline(make())
    x = torch.randn(4, 8)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    plain(xa).pow(2).sum().backward()
    ck(xb).pow(2).sum().backward()
    assert torch.allclose(xa.grad, xb.grad, atol=1e-6)
    for p, q in zip(plain.parameters(), ck.parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-6)
    with torch.no_grad():
        assert torch.allclose(ck(x), plain(x))
    est = ck.memory_estimate(4, 8, inner_activations_per_segment=3)
    assert est["savings"] == pytest.approx(0.75) and ck.num_segments() == 3
    b = TR.CheckpointBudget(100)
    assert b.allocate(60) and not b.allocate(50) and b.remaining() == 40 and b.utilization() == 0.6
    b.free(60)
    assert b.can_allocate(100)
