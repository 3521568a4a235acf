"""End-to-end checks of the CUDA path: fused layer vs op-by-op vs fp32, optimizer engine."""

import copy
import os

import pytest
import torch

from agentgarten_b200.infra.optim import FusedAdam
from agentgarten_b200.models.diffusion import DiffusionModel
from agentgarten_b200.ops import native

from helpers import synthetic_batch, tiny_conditioner, tiny_config, tiny_network

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _config():
    return tiny_config(hidden_size=512, intermediate_size=1024, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=128, mrope_section=(24, 20, 20))


def _model(device, dtype, config):
    net = tiny_network(config, device="cpu", dtype=torch.float32, seed=0)
    cond = tiny_conditioner(config, device="cpu", dtype=torch.float32, seed=1)
    model = DiffusionModel(net=net, conditioner=cond, text_dropout=0.0)
    model.to(device=device, dtype=dtype)
    return model


def _loss_and_grads(model, batch, seed=0):
    torch.manual_seed(seed)
    model.zero_grad(set_to_none=True)
    _, loss = model.training_step(model.prepare_data_batch(batch), 0)
    loss.backward()
    grads = {n: p.grad.detach().float().cpu() for n, p in model.net.named_parameters()
             if p.grad is not None}
    return float(loss), grads


def test_fused_layer_matches_op_path_and_fp32(monkeypatch):
    config = _config()
    batch_cpu = synthetic_batch(frames=3, height=8, width=12, text=9, seed=3)
    batch = {k: v.to(DEV) for k, v in batch_cpu.items()}
    reference = _model("cpu", torch.float32, config)
    # identical noise on both devices: draw on CPU, patch randn/rand through a fixed generator
    model = _model(DEV, torch.bfloat16, config)

    def run(m, b, device):
        g = torch.Generator(device=device).manual_seed(7)
        m.zero_grad(set_to_none=True)
        out, loss = m._objective(m.prepare_data_batch(b), g, None)
        loss.backward()
        return float(loss), {n: p.grad.detach().float().cpu() for n, p in m.net.named_parameters()
                             if p.grad is not None}

    # CPU and CUDA generators differ, so compare the two CUDA paths exactly in distribution
    # and the fp32 model on the same device for values.
    ref_gpu = _model(DEV, torch.float32, config)
    loss_ref, grads_ref = run(ref_gpu, batch, DEV)
    before = native.launches()
    loss_fused, grads_fused = run(model, batch, DEV)
    assert native.launches() > before
    monkeypatch.setenv("AGB200_DISABLE_FUSED_LAYER", "1")
    loss_ops, grads_ops = run(model, batch, DEV)
    monkeypatch.delenv("AGB200_DISABLE_FUSED_LAYER")
    torch.cuda.synchronize()
    assert int(native.ext().status(0).item()) == 0
    assert abs(loss_fused - loss_ref) < 2e-2 * abs(loss_ref)
    assert abs(loss_ops - loss_ref) < 2e-2 * abs(loss_ref)
    for name, ref in grads_ref.items():
        if ref.norm() < 1e-8:
            continue
        for label, grads in (("fused", grads_fused), ("ops", grads_ops)):
            rel = float((grads[name] - ref).norm() / ref.norm())
            assert rel < 8e-2, (label, name, rel)
    del reference


def test_joint_projection_gemms_match_one_gemm_per_weight():
    """With the optimizer engine's flat buffer q|k|v and gate|up are adjacent in memory, so each
    group runs as one GEMM forward and two backward (strided head norm, dv written into the joint
    gradient).  Forward values are bit for bit those of one GEMM per weight; gradients agree to
    bf16 rounding (the joint input gradient is summed in fp32 over all of q|k|v)."""
    from agentgarten_b200.ops import fused_layer

    config = _config()
    batch = {k: v.to(DEV) for k, v in synthetic_batch(frames=3, height=16, width=16, text=9, seed=8).items()}
    model = _model(DEV, torch.bfloat16, config)
    loss_separate, separate = _loss_and_grads(model, batch, seed=5)
    FusedAdam([p for p in model.net.parameters() if p.requires_grad], lr=1e-4,
              use_te_capturable_kernel=True, master_weights=True)
    blocks = [m for m in model.net.modules() if hasattr(m, "mlp_moe_gen")]
    q, k, v = (m.weight for m in blocks[0].self_attn.parts()[:3])
    assert fused_layer._joined((q, k, v)) is not None and fused_layer._joined((q.grad, k.grad, v.grad)) is not None
    mlp = blocks[0].mlp_moe_gen
    assert fused_layer._joined((mlp.gate_proj.weight, mlp.up_proj.weight)) is not None
    torch.manual_seed(5)
    for p in model.net.parameters():
        if p.grad is not None:
            p.grad.zero_()
    _, loss = model.training_step(model.prepare_data_batch(batch), 0)
    loss.backward()
    torch.cuda.synchronize()
    assert int(native.ext().status(0).item()) == 0
    assert float(loss) == loss_separate
    for name, p in model.net.named_parameters():
        if name in separate and separate[name].norm() > 1e-8:
            rel = float((p.grad.float().cpu() - separate[name]).norm() / separate[name].norm())
            assert rel < 2e-2, (name, rel)


def test_flat_adam_matches_foreach():
    torch.manual_seed(0)
    shapes = [(64, 32), (7, 24), (130,), (3, 5, 8)]
    params_a = [torch.nn.Parameter(torch.randn(s, device=DEV).to(torch.bfloat16)) for s in shapes]
    params_b = [torch.nn.Parameter(p.detach().clone()) for p in params_a]
    flat = FusedAdam(params_a, lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.01,
                     use_te_capturable_kernel=True, master_weights=True)
    plain = FusedAdam(params_b, lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.01,
                      use_te_capturable_kernel=True, master_weights=True, flat=False)
    assert flat.engine is not None and plain.engine is None
    for step in range(3):
        grads = [torch.randn(s, device=DEV).to(torch.bfloat16) for s in shapes]
        for p, q, g in zip(params_a, params_b, grads):
            p.grad.copy_(g)
            q.grad = g.clone()
        expected_norm = torch.stack([g.float().square().sum() for g in grads]).sum()
        assert torch.allclose(flat.grad_norm_sq(), expected_norm, rtol=1e-4)
        flat.step()
        plain.step()
        flat.zero_grad()
        plain.zero_grad()
        for p, q in zip(params_a, params_b):
            assert torch.allclose(p.float(), q.float(), atol=1e-2, rtol=1e-2)
    flat.engine.publish_state()
    for p, q in zip(params_a, params_b):
        assert torch.allclose(flat.state[p]["master_param"], plain.state[q]["master_param"], atol=1e-5)
        assert torch.allclose(flat.state[p]["exp_avg"], plain.state[q]["exp_avg"], atol=1e-6)


def test_nonfinite_gradient_skips_update():
    p = torch.nn.Parameter(torch.ones(64, 8, device=DEV, dtype=torch.bfloat16))
    opt = FusedAdam([p], lr=1e-1, use_te_capturable_kernel=True, master_weights=True)
    p.grad.fill_(float("inf"))
    opt.step()
    assert float(opt.found_nonfinite()) == 1.0
    assert torch.equal(p.detach(), torch.ones_like(p))


def test_smoke_entry():
    import __graft_entry__

    __graft_entry__.smoke()


def test_stream_graph_replay_matches_eager():
    from agentgarten_b200.inference.serving import prepare_serving
    from agentgarten_b200.networks.cosmos3.network import Cosmos3Condition
    from agentgarten_b200.networks.cosmos3.streaming import Cosmos3Stream, StreamPolicy

    config = _config()
    net = tiny_network(config, device="cpu", seed=0).to(DEV, torch.bfloat16).eval()
    cond = tiny_conditioner(config, device="cpu", seed=1).to(DEV, torch.bfloat16)
    batch = {k: v.to(DEV) for k, v in synthetic_batch(frames=21, height=8, width=12, text=9, seed=5).items()}
    encoded = cond.encode(batch, training=False)
    condition = cond.condition(encoded)
    latent = encoded["latent"]

    def block(lo, hi):
        return Cosmos3Condition(text=condition.text, depth=condition.depth[:, :, lo:hi],
                                normal=condition.normal[:, :, lo:hi], fps=condition.fps)

    policy = StreamPolicy(block_frames=4, sink_frames=1, history_frames=8, rope="top_aligned",
                          train_frames=13)
    outputs = {}
    for graphs in (False, True):
        prepare_serving(net, cuda_graphs=graphs)
        stream = Cosmos3Stream(net, policy)
        stream.start(latent[:, :, :1], block(0, 1))
        outs = []
        gen = torch.Generator(device=DEV).manual_seed(3)
        for b in range(5):
            lo, hi = 1 + 4 * b, 5 + 4 * b
            noisy = torch.randn(latent[:, :, lo:hi].shape, device=DEV, generator=gen)
            for sigma in (1.0, 0.5):
                outs.append(stream.denoise(noisy, torch.tensor([sigma], device=DEV), block(lo, hi)))
            stream.commit(latent[:, :, lo:hi], block(lo, hi))
        outputs[graphs] = outs
        assert stream.layers[0].frames == policy.capacity
    torch.cuda.synchronize()
    assert int(native.ext().status(0).item()) == 0
    for eager, replayed in zip(outputs[False], outputs[True]):
        assert torch.isfinite(eager).all()
        assert torch.equal(eager, replayed)


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def _stream_outputs(net, condition, latent, policy, **serving):
    from agentgarten_b200.inference.serving import prepare_serving
    from agentgarten_b200.networks.cosmos3.network import Cosmos3Condition
    from agentgarten_b200.networks.cosmos3.streaming import Cosmos3Stream

    def block(lo, hi):
        return Cosmos3Condition(text=condition.text, depth=condition.depth[:, :, lo:hi],
                                normal=condition.normal[:, :, lo:hi], fps=condition.fps)

    prepare_serving(net, **serving)
    stream = Cosmos3Stream(net, policy)
    stream.start(latent[:, :, :1], block(0, 1))
    outs = []
    gen = torch.Generator(device=DEV).manual_seed(3)
    for b in range(4):
        lo, hi = 1 + 4 * b, 5 + 4 * b
        noisy = torch.randn(latent[:, :, lo:hi].shape, device=DEV, generator=gen)
        for sigma in (1.0, 0.5):
            outs.append(stream.denoise(noisy, torch.tensor([sigma], device=DEV), block(lo, hi)))
        stream.commit(latent[:, :, lo:hi], block(lo, hi))
    torch.cuda.synchronize()
    return outs


@pytest.mark.parametrize("reduce_rows", [1, 4])
@pytest.mark.parametrize("tokens", [101, 130, 387])
def test_tensor_parallel_run_with_ragged_row_counts(tokens, reduce_rows):
    """Row counts that fill neither a tile of 128 nor a group of four rows: the tensor-parallel
    kernels (one rank) against the layer-by-layer path on the same tokens."""
    from agentgarten_b200 import ops
    from agentgarten_b200.parallel.tensor_parallel import TensorParallelServing

    torch.manual_seed(tokens)
    config = _config()
    net = tiny_network(config, device="cpu", seed=0).to(DEV, torch.bfloat16).eval()
    plan = TensorParallelServing(net, None, max_tokens=512)
    plan.reduce_rows = reduce_rows  # both forms of the reduce kernel
    hidden = torch.randn(1, tokens, config.hidden_size, device=DEV).bfloat16()
    positions = torch.stack((torch.arange(tokens) // 24, (torch.arange(tokens) // 6) % 4, torch.arange(tokens) % 6),
                            dim=-1).unsqueeze(0).to(DEV)
    rope = net.rotary_emb(positions, torch.bfloat16)

    def attend(index, queries, keys, values):
        return [ops.attention(queries[0], keys[0].contiguous(), values[0].contiguous())]

    with torch.no_grad():
        want = hidden
        for index, layer in enumerate(net.layers):
            (want,) = layer([want], [rope], attend, index)
        want = net.proj_out(net.norm_moe_gen(want))
        for _ in range(2):  # the second call reuses the counters of the first
            got = plan.run(hidden, rope, attend)
    torch.cuda.synchronize()
    assert int(native.ext().status(0).item()) == 0
    assert got.shape == want.shape and rel(got, want) < 2e-2, rel(got, want)


def test_tensor_parallel_kernels_on_one_rank_match_the_layer_path(monkeypatch):
    """Runs with the peer-written buffers poisoned (NaN until a producer stores into them): the
    outputs stay finite and equal to the layer path, so no consumer reads a row before it was
    pushed."""
    from agentgarten_b200.networks.cosmos3.streaming import StreamPolicy

    monkeypatch.setenv("AGB200_POISON", "1")

    config = _config()
    net = tiny_network(config, device="cpu", seed=0).to(DEV, torch.bfloat16).eval()
    cond = tiny_conditioner(config, device="cpu", seed=1).to(DEV, torch.bfloat16)
    batch = {k: v.to(DEV) for k, v in synthetic_batch(frames=17, height=8, width=12, text=9, seed=5).items()}
    encoded = cond.encode(batch, training=False)
    condition, latent = cond.condition(encoded), encoded["latent"]
    policy = StreamPolicy(block_frames=4, sink_frames=1, history_frames=8, rope="top_aligned", train_frames=13)
    plain = _stream_outputs(net, condition, latent, policy, cuda_graphs=False)
    eager = _stream_outputs(net, condition, latent, policy, cuda_graphs=False, tensor_parallel=True, max_tokens=1024)
    replay = _stream_outputs(net, condition, latent, policy, cuda_graphs=True, tensor_parallel=True, max_tokens=1024)
    assert int(native.ext().status(0).item()) == 0
    for a, b, c in zip(plain, eager, replay):
        assert torch.isfinite(b).all()
        assert rel(b, a) < 2e-2, rel(b, a)
        assert torch.equal(b, c)
    from agentgarten_b200.inference.serving import release_serving
    release_serving(net)


def test_forward_ar_replays_cached_rollout_bitwise_on_the_kernels():
    """Teacher-forced training and the cached rollout must give identical bits: key tiles
    never straddle segments, so both accumulate a row over the same tile partition."""
    from agentgarten_b200.models.flow import rf_interpolate

    config = _config()
    net = tiny_network(config, device="cpu", seed=0).to(DEV, torch.bfloat16).eval()
    cond = tiny_conditioner(config, device="cpu", seed=1).to(DEV, torch.bfloat16)
    batch = {k: v.to(DEV) for k, v in synthetic_batch(frames=9, height=16, width=16, text=9, seed=2).items()}
    encoded = cond.encode(batch, training=False)
    condition, latent = cond.condition(encoded), encoded["latent"]
    anchor, target = latent[:, :, :1], latent[:, :, 1:]
    sigma = torch.tensor([[0.7] * 4 + [0.3] * 4], device=DEV)
    noisy = rf_interpolate(target, torch.randn_like(target), sigma)
    before = native.launches()
    with torch.no_grad():
        full = net.forward_ar(anchor, noisy, sigma, condition, block_frames=4, clean=target)
        cache = net.prefill(anchor, condition)
        outs = []
        for b in range(2):
            sl = slice(4 * b, 4 * b + 4)
            outs.append(net.denoise(cache, noisy[:, :, sl], sigma[:, sl]))
            cache = net.commit(cache, target[:, :, sl])
    assert native.launches() > before
    assert torch.isfinite(full).all()
    assert torch.equal(full, torch.cat(outs, dim=2))
    assert int(native.ext().status(0).item()) == 0


@pytest.mark.parametrize("regularization", ["finite_difference", "exact"])
def test_dmd_gan_step_runs_on_the_kernels(regularization):
    """Student / fake-score / discriminator updates on bf16 CUDA towers; the exact penalties
    differentiate the frozen backbone in forward mode, i.e. through the tangent kernel."""
    from agentgarten_b200.infra.config import LazyCall
    from agentgarten_b200.infra.optim import LinearWarmup
    from agentgarten_b200.models.dmd import DMDModel, GANConfig
    from agentgarten_b200.networks.discriminator import DiscriminatorHead
    from agentgarten_b200.parallel.engine import ParallelConfig

    config = _config()
    parallel = ParallelConfig(parameter_dtype="bfloat16", fully_shard=False, activation_checkpointing="none")
    head = DiscriminatorHead(hidden_size=config.hidden_size, feature_layers=(0, 1), num_heads=4, mlp_ratio=2.0)
    model = DMDModel(student=tiny_network(config, seed=0), real_score=tiny_network(config, seed=1),
                     fake_score=tiny_network(config, seed=2), conditioner=tiny_conditioner(config),
                     discriminator=head, gan=GANConfig(regularization=regularization, warmup_updates=1),
                     fake_score_updates_per_student=1, real_score_guidance=1.0, seed=3,
                     student_parallel=parallel, score_parallel=parallel, real_score_parallel=parallel,
                     conditioner_parallel=parallel)
    model.parallelize(torch.device(DEV))
    optim = {name: LazyCall(FusedAdam)(lr=1e-4, betas=(0.0, 0.999)) for name in
             ("student", "fake_score", "discriminator")}
    sched = LazyCall(torch.optim.lr_scheduler.LambdaLR)(lr_lambda=LazyCall(LinearWarmup)(warmup_steps=2))
    model.init_optimizer_scheduler(optim, sched)
    batch = {k: v.to(DEV) for k, v in synthetic_batch(frames=5, height=16, width=16, text=9, seed=4).items()}
    batch = model.prepare_data_batch(batch)
    before = native.launches()
    for iteration in range(3):  # discriminator warm-up, student, fake score
        torch.manual_seed(iteration)
        out, loss = model.training_step(batch, iteration)
        assert torch.isfinite(loss), (iteration, float(loss))
        loss.backward()
        model.zero_grad(set_to_none=True)
    assert native.launches() > before
    torch.cuda.synchronize()
    assert int(native.ext().status(0).item()) == 0


def test_training_step_is_bitwise_reproducible():
    """Same seed, same inputs: identical loss and gradients (no atomics anywhere in backward)."""
    config = _config()
    model = _model(DEV, torch.bfloat16, config)
    batch = {k: v.to(DEV) for k, v in synthetic_batch(frames=5, height=16, width=16, text=9, seed=6).items()}
    first_loss, first = _loss_and_grads(model, batch, seed=4)
    second_loss, second = _loss_and_grads(model, batch, seed=4)
    assert first_loss == second_loss
    assert first.keys() == second.keys() and all(torch.equal(first[k], second[k]) for k in first)


def test_sampling_paths_run_on_the_kernels():
    """UniPC sampling with guidance (bidirectional) and the block-by-block cached rollout
    (autoregressive), both decoded by the VAE in bf16 on the device."""
    from agentgarten_b200.codecs import Wan22VAECodec
    from agentgarten_b200.models.autoregressive import AutoregressiveModel

    config = _config()
    codec = Wan22VAECodec(None, dtype="bfloat16", architecture=dict(dim=16, dec_dim=16, z_dim=48))
    batch = {k: v.to(DEV) for k, v in synthetic_batch(frames=5, height=8, width=8, text=9, seed=8).items()}
    before = native.launches()
    for kind in ("bidirectional", "autoregressive"):
        net = tiny_network(config, device="cpu", seed=0)
        cond = tiny_conditioner(config, device="cpu", seed=1)
        cond.codec, cond.empty_prompt_ids = codec, (3, 4, 1)
        if kind == "bidirectional":
            model = DiffusionModel(net=net, conditioner=cond, text_dropout=0.0)
        else:
            model = AutoregressiveModel(net=net, conditioner=cond, mode="diffusion_forcing", block_frames=4)
        model.to(device=DEV, dtype=torch.bfloat16).eval()
        encoded = model.prepare_data_batch(dict(batch))
        out = model.sample(encoded, num_steps=3, guidance=2.0, seed=1)
        assert set(out) >= {"ground_truth", "sample"}
        assert out["sample"].shape == (1, 3, 17, 128, 128) and torch.isfinite(out["sample"]).all()
    assert native.launches() > before
    torch.cuda.synchronize()
    assert int(native.ext().status(0).item()) == 0
