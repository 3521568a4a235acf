import torch

from agentgarten_b200.infra.config import LazyCall
from agentgarten_b200.infra.optim import FusedAdam
from agentgarten_b200.models.dmd import DMDModel, GANConfig, PhaseClock
from agentgarten_b200.models.exact_regularization import exact_penalties
from agentgarten_b200.networks.discriminator import DiscriminatorHead

from helpers import synthetic_batch, tiny_conditioner, tiny_config, tiny_network


def test_phase_clock():
    clock = PhaseClock(fake_score_updates_per_student=2, warmup_updates=3)
    roles = ["w" if clock.is_warmup(i) else "s" if clock.is_student(i) else "f" for i in range(10)]
    assert roles == ["w", "w", "w", "s", "f", "f", "s", "f", "f", "s"]
    assert clock.role_updates(9) == {"student": 2, "fake_score": 4}
    assert clock.is_cadence_due(9, 2) and not clock.is_cadence_due(8, 2) and not clock.is_cadence_due(9, 3)


def _model(gan=None, regularization="finite_difference"):
    cfg = tiny_config()
    disc = gan_cfg = None
    if gan:
        disc = DiscriminatorHead(hidden_size=256, feature_layers=(0, 1), num_heads=4, mlp_ratio=2.0)
        gan_cfg = GANConfig(regularization=regularization, warmup_updates=1)
    model = DMDModel(student=tiny_network(cfg, seed=0), real_score=tiny_network(cfg, seed=1),
                     fake_score=tiny_network(cfg, seed=2), conditioner=tiny_conditioner(cfg),
                     discriminator=disc, gan=gan_cfg, fake_score_updates_per_student=1,
                     real_score_guidance=1.0, seed=3)
    model.parallelize("cpu")
    optim = {name: LazyCall(FusedAdam)(lr=1e-4, betas=(0.0, 0.999)) for name in
             ("student", "fake_score", "discriminator")}
    sched = LazyCall(torch.optim.lr_scheduler.LambdaLR)(lr_lambda=LazyCall(
        __import__("agentgarten_b200.infra.optim", fromlist=["LinearWarmup"]).LinearWarmup)(warmup_steps=2))
    model.init_optimizer_scheduler(optim, sched)
    return model


def test_dmd_student_replay_is_bitwise_and_roles_alternate():
    model = _model()
    batch = model.prepare_data_batch(synthetic_batch(frames=9))
    assert model.get_optimizer_names(0) == ("student",) and model.get_optimizer_names(1) == ("fake_score",)
    torch.manual_seed(0)
    out, loss = model.training_step(batch, 0)
    assert float(out["metrics/student/sgf_recovery_max_abs"]) == 0.0
    loss.backward()
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in model.student.parameters())
    assert all(p.grad is None for p in model.real_score.parameters())
    model.zero_grad(set_to_none=True)
    out, loss = model.training_step(batch, 1)
    loss.backward()
    assert "metrics/fake_score/loss" in out
    assert any(p.grad is not None for p in model.fake_score.parameters())
    assert all(p.grad is None for p in model.student.parameters())


def test_dmd_gan_finite_difference_and_exact():
    for kind in ("finite_difference", "exact"):
        model = _model(gan=True, regularization=kind)
        batch = model.prepare_data_batch(synthetic_batch(frames=5))
        assert model.get_optimizer_names(0) == ("discriminator",)
        torch.manual_seed(1)
        out, loss = model.training_step(batch, 0)      # warm-up: discriminator only
        loss.backward()
        assert all(p.grad is None for p in model.fake_score.parameters())
        assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in model.discriminator.parameters())
        assert "metrics/discriminator/r1" in out
        model.zero_grad(set_to_none=True)
        out, loss = model.training_step(batch, 1)      # student with generator gradient
        loss.backward()
        assert "metrics/student/gan_loss" in out


def test_exact_penalty_gradient_matches_double_backward():
    torch.manual_seed(0)
    backbone = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.Tanh(), torch.nn.Linear(8, 8)).double()
    backbone.requires_grad_(False)

    class Head(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.net = torch.nn.Sequential(torch.nn.Linear(8, 5), torch.nn.Tanh(), torch.nn.Linear(5, 1)).double()

        def forward(self, groups):
            return torch.cat([self.net(g[0]) for g in groups]).reshape(-1)

    head = Head()
    rows = torch.randn(4, 6, dtype=torch.float64)
    result = exact_penalties(lambda x: (backbone(x),), head, rows)
    (result.penalty.sum() + result.surrogate.sum()).backward()
    fast = [torch.zeros_like(p) if p.grad is None else p.grad.clone() for p in head.parameters()]
    head.zero_grad()
    x = rows.clone().requires_grad_(True)
    (gx,) = torch.autograd.grad(head([(backbone(x),)]).sum(), x, create_graph=True)
    penalty = gx.square().flatten(1).sum(1)
    penalty.sum().backward()
    assert torch.allclose(result.penalty, penalty.detach())
    for a, p in zip(fast, head.parameters()):
        assert torch.allclose(a, torch.zeros_like(p) if p.grad is None else p.grad, atol=1e-10)
