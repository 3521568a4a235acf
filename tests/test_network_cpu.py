import torch

from agentgarten_b200.models.diffusion import DiffusionModel
from agentgarten_b200.models.flow import FlowUniPC, RectifiedFlowSchedule, invariant_randn, rf_interpolate, rf_x0
from agentgarten_b200.networks.cosmos3.attention import block_causal_plan
from agentgarten_b200.networks.cosmos3.network import patchify, unpatchify
from agentgarten_b200.protocols import HistoryWindow
from agentgarten_b200.infra.optim import FusedAdam

from helpers import synthetic_batch, tiny_conditioner, tiny_config, tiny_network


def test_patchify_roundtrip():
    x = torch.randn(2, 6, 3, 4, 8)
    p = patchify(x, 2)
    assert p.shape == (2, 3, 8, 24)
    assert torch.equal(unpatchify(p, channels=6, grid=(2, 4), patch_size=2), x)


def test_flow_pointwise_and_schedule():
    x0, noise = torch.randn(2, 4, 3, 2, 2), torch.randn(2, 4, 3, 2, 2)
    s = torch.tensor([0.25, 1.0])
    xt = rf_interpolate(x0, noise, s)
    assert torch.allclose(rf_x0(xt, s, noise - x0), x0, atol=1e-6)
    per_frame = torch.rand(2, 3)
    xt = rf_interpolate(x0, noise, per_frame)
    assert torch.allclose(xt[1, :, 2], (1 - per_frame[1, 2]) * x0[1, :, 2] + per_frame[1, 2] * noise[1, :, 2])
    for kind in ("uniform", "logitnormal", "waver"):
        sig = RectifiedFlowSchedule(shift=5.0, train_distribution=kind).sample(1000, device=torch.device("cpu"))
        assert sig.min() >= 0 and sig.max() <= 1 and sig.mean() > 0.5


def test_invariant_randn_is_batching_invariant():
    ref = torch.zeros(3, 2, 2)
    a = invariant_randn(ref, [5, 6, 7])
    b = invariant_randn(ref[:1], [6])
    assert torch.equal(a[1:2], b)
    assert not torch.equal(invariant_randn(ref, [5, 6, 7], stream=1), a)


def test_unipc_integrates_linear_flow_exactly():
    # velocity of the straight path between fixed noise and data is constant: noise - x0
    x0, noise = torch.randn(1, 2, 2, 2, 2), torch.randn(1, 2, 2, 2, 2)
    solver = FlowUniPC(8, shift=3.0)
    start = (1 - solver.sigmas[0]) * x0 + solver.sigmas[0] * noise
    out = solver.run(start, lambda x, s: noise - x0)
    assert torch.allclose(out, x0, atol=1e-4)


def test_block_causal_plan_and_window():
    assert block_causal_plan(4, False, HistoryWindow()) == [[0], [0, 1], [0, 1, 2], [0, 1, 2, 3]]
    tf = block_causal_plan(5, True, HistoryWindow())
    assert tf == [[0], [0, 1], [0, 2], [0, 2, 3], [0, 2, 4]]
    windowed = block_causal_plan(5, False, HistoryWindow(sink_blocks=1, recent_blocks=1))
    assert windowed[4] == [0, 1, 3, 4]


def test_bidirectional_training_step_decreases_loss():
    cfg = tiny_config()
    model = DiffusionModel(net=tiny_network(cfg), conditioner=tiny_conditioner(cfg), text_dropout=0.0)
    model.parallelize("cpu")
    opt = FusedAdam(model._group_trainable_parameters(), lr=2e-3, use_te_capturable_kernel=True,
                    master_weights=True)
    batch = model.prepare_data_batch(synthetic_batch())
    losses = []
    for it in range(8):
        g = torch.Generator().manual_seed(0)
        _, loss = model._objective(batch, g, None)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(float(loss))
    assert losses[-1] < losses[0] * 0.9


def test_forward_ar_replays_cached_rollout_bitwise():
    cfg = tiny_config()
    net = tiny_network(cfg).eval()
    cond = tiny_conditioner(cfg)
    batch = cond.encode(synthetic_batch(frames=9), training=False)
    condition = cond.condition(batch)
    latent = batch["latent"]
    anchor, target = latent[:, :, :1], latent[:, :, 1:]
    sigma = torch.tensor([[0.7] * 4 + [0.3] * 4])
    noisy = rf_interpolate(target, torch.randn_like(target), sigma)
    with torch.no_grad():
        full = net.forward_ar(anchor, noisy, sigma, condition, block_frames=4, clean=target)
        cache = net.prefill(anchor, condition)
        outs = []
        for b in range(2):
            sl = slice(4 * b, 4 * b + 4)
            outs.append(net.denoise(cache, noisy[:, :, sl], sigma[:, sl]))
            cache = net.commit(cache, target[:, :, sl])
        rolled = torch.cat(outs, dim=2)
    assert torch.equal(full, rolled)
    assert cache.frames_committed == 8


def test_fused_adam_matches_torch_adamw():
    torch.manual_seed(0)
    a = torch.nn.Parameter(torch.randn(5, 4))
    b = torch.nn.Parameter(a.detach().clone())
    mine = FusedAdam([a], lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
    ref = torch.optim.AdamW([b], lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
    for _ in range(4):
        g = torch.randn(5, 4)
        a.grad, b.grad = g.clone(), g.clone()
        mine.step()
        ref.step()
    assert torch.allclose(a, b, atol=1e-6)
    zero = torch.nn.Parameter(torch.randn(3))
    no_moment = FusedAdam([zero], lr=1e-2, betas=(0.0, 0.999))
    zero.grad = torch.ones(3)
    no_moment.step()
    assert "exp_avg" not in no_moment.state[zero]


def test_adaln_operators_fall_back_to_the_operator_sequence():
    """Off the GPU (and whenever gradients are wanted) the AdaLN helpers are the plain expressions."""
    import torch

    from agentgarten_b200 import ops

    torch.manual_seed(0)
    x, y = torch.randn(2, 5, 16), torch.randn(2, 5, 16)
    weight = torch.rand(16) + 0.5
    shift, scale, gate = (0.3 * torch.randn(2, 5, 48)).chunk(3, dim=-1)
    want = ops.rms_norm(x, weight, 1e-6) * (1 + scale) + shift
    assert torch.equal(ops.norm_modulate(x, weight, scale, shift, 1e-6), want)
    assert torch.equal(ops.gated_residual(x, gate, y), x + gate * y)
    x.requires_grad_()
    ops.norm_modulate(x, weight, scale, shift, 1e-6).sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()


def test_one_pass_backward_work_lists_cover_every_reader_once_and_number_the_turns():
    """Every (key tile, visible query row) appears in exactly one block entry, blocks are aligned
    to 128 rows, and the turns of a block count up from zero in tile order."""
    import collections

    from agentgarten_b200.ops.attention import build_schedule

    sizes = [300, 200, 390]
    plan = [[0], [0, 1], [0, 2]]
    schedule = build_schedule(sizes, sizes, plan, 130, torch.device("cpu"))
    tiles, blocks = schedule.fused_tiles.tolist(), schedule.fused_blocks.tolist()
    starts = [0, 300, 500, 890]
    turns = collections.defaultdict(list)
    for k_row, rows, first, count, source in tiles:
        seen = set()
        for q_block, lo, hi, turn in blocks[first:first + count]:
            assert q_block % 128 == 0 and 0 <= lo < hi <= 128
            turns[q_block].append(turn)
            rows_seen = set(range(q_block + lo, q_block + hi))
            assert not (rows_seen & seen)
            seen |= rows_seen
        if source == 0:
            want = set(range(890))
        else:
            chunk = max(j for j in range(3) if starts[j] <= k_row)
            want = {r for c, visible in enumerate(plan) if chunk in visible
                    for r in range(starts[c], starts[c + 1])}
        assert seen == want, (k_row, source)
    assert [t[4] for t in tiles[:2]] == [0, 0] and all(t[4] == 1 for t in tiles[2:])
    for q_block, taken in turns.items():
        assert taken == list(range(len(taken))), q_block
    assert build_schedule([200], [200], [[0]], 0, torch.device("cpu"), causal=True).fused_tiles is None


def test_adjoined_weights_form_one_view_and_keep_their_values():
    """``adjoin`` lays 2-D parameters out back to back without changing them, ``joined`` then finds
    one matrix over them; parameters in separate storages (or in another order) are not joined, and
    the joint GEMM never applies on the CPU."""
    from agentgarten_b200 import ops

    torch.manual_seed(0)
    q, k, v = (torch.nn.Linear(16, n, bias=False) for n in (32, 8, 8))
    before = [m.weight.detach().clone() for m in (q, k, v)]
    assert ops.joined([m.weight for m in (q, k, v)]) is None
    ops.adjoin([m.weight for m in (q, k, v)])
    whole = ops.joined([m.weight for m in (q, k, v)])
    assert whole is not None and whole.shape == (48, 16)
    assert torch.equal(whole, torch.cat(before))
    for module, old in zip((q, k, v), before):
        assert torch.equal(module.weight, old)
    assert ops.joined([k.weight, q.weight, v.weight]) is None
    ops.adjoin([m.weight for m in (q, k, v)])            # already adjacent: nothing moves
    assert ops.joined([m.weight for m in (q, k, v)]).data_ptr() == whole.data_ptr()
    assert ops.joint_linear(torch.randn(3, 16), (q, k, v)) is None
