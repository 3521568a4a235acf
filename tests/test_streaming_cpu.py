import pytest
import torch

from agentgarten_b200.models.flow import rf_interpolate
from agentgarten_b200.networks.cosmos3.network import Cosmos3Condition
from agentgarten_b200.networks.cosmos3.streaming import Cosmos3Stream, StreamPolicy, StreamRoPE
from agentgarten_b200.ops import reference
from agentgarten_b200.ops.kernels.stream_cache import relocate

from helpers import synthetic_batch, tiny_conditioner, tiny_config, tiny_network


def _block_condition(condition, lo, hi):
    return Cosmos3Condition(text=condition.text, depth=condition.depth[:, :, lo:hi],
                            normal=condition.normal[:, :, lo:hi], fps=condition.fps)


def test_policy_positions():
    p = StreamPolicy(block_frames=4, sink_frames=5, history_frames=8, rope="top_aligned", train_frames=21)
    assert p.capacity == 13
    assert p.positions((0, 1, 2, 3, 4, 9, 10), 17) == (0, 1, 2, 3, 4, 9, 10)
    assert p.positions((0, 4, 9, 20), 21) == (0, 4, 5, 16)
    c = StreamPolicy(block_frames=4, sink_frames=1, history_frames=8, rope="contiguous")
    assert c.positions((0, 5, 12), 13) == (0, 1, 8)
    with pytest.raises(ValueError):
        StreamPolicy(sink_frames=3)
    with pytest.raises(ValueError):
        StreamPolicy(history_frames=None, rope="top_aligned")


def test_stream_matches_cached_rollout_with_absolute_positions():
    cfg = tiny_config()
    net = tiny_network(cfg).eval()
    cond = tiny_conditioner(cfg)
    batch = cond.encode(synthetic_batch(frames=9), training=False)
    condition = cond.condition(batch)
    latent = batch["latent"]
    anchor = latent[:, :, :1]
    stream = Cosmos3Stream(net, StreamPolicy(block_frames=4, sink_frames=1, history_frames=None,
                                             rope=StreamRoPE.ABSOLUTE))
    stream.start(anchor, _block_condition(condition, 0, 1))
    with torch.no_grad():
        cache = net.prefill(anchor, condition)
    for b in range(2):
        lo, hi = 1 + 4 * b, 5 + 4 * b
        clean = latent[:, :, lo:hi]
        sigma = torch.tensor([0.6])
        noisy = rf_interpolate(clean, torch.randn_like(clean), sigma)
        block = _block_condition(condition, lo, hi)
        with torch.no_grad():
            expected = net.denoise(cache, noisy, sigma)
            cache = net.commit(cache, clean)
        got = stream.denoise(noisy, sigma, block)
        assert torch.allclose(got, expected, atol=2e-5)
        stream.commit(clean, block)
    assert stream.frame_ids == tuple(range(9)) and stream.layers[0].frames == 9


def test_bounded_stream_evicts_and_relocates():
    cfg = tiny_config()
    net = tiny_network(cfg).eval()
    cond = tiny_conditioner(cfg)
    batch = cond.encode(synthetic_batch(frames=21), training=False)
    condition = cond.condition(batch)
    latent = batch["latent"]
    policy = StreamPolicy(block_frames=4, sink_frames=1, history_frames=8, rope="top_aligned",
                          train_frames=13)
    stream = Cosmos3Stream(net, policy)
    stream.start(latent[:, :, :1], _block_condition(condition, 0, 1))
    for b in range(5):
        lo, hi = 1 + 4 * b, 5 + 4 * b
        block = _block_condition(condition, lo, hi)
        out = stream.denoise(torch.randn_like(latent[:, :, lo:hi]), torch.tensor([0.9]), block)
        assert torch.isfinite(out).all() and out.shape == latent[:, :, lo:hi].shape
        stream.commit(latent[:, :, lo:hi], block)
        assert len(stream.frame_ids) <= policy.capacity
    assert stream.frame_ids == (0, *range(13, 21))
    assert stream.layers[0].frames == policy.capacity
    # the block that follows sits at the top of the training range
    assert policy.positions((21,), 21) == (9,)


def test_relocate_matches_reference_rows():
    torch.manual_seed(0)
    rows = torch.randn(1, 12, 2, 8)
    ang = torch.randn(1, 9, 4)
    cos, sin = torch.cat((ang, ang), -1).cos(), torch.cat((ang, ang), -1).sin()
    out = torch.zeros(1, 12, 2, 8)
    relocate(rows, out, 2, 3, (cos, sin))
    assert torch.equal(out[0, :2], rows[0, :2])
    moved = rows[0, 5:12]
    expect = moved * cos[0, 2:9, None] + reference.rotate_half(moved) * sin[0, 2:9, None]
    assert torch.allclose(out[0, 2:9], expect, atol=1e-6)


def test_reference_images_condition_a_block_without_touching_the_cache():
    from agentgarten_b200.networks.cosmos3.reference import denoise_with_references

    cfg = tiny_config()
    net = tiny_network(cfg).eval()
    cond = tiny_conditioner(cfg)
    batch = cond.encode(synthetic_batch(frames=5), training=False)
    condition = cond.condition(batch)
    latent = batch["latent"]
    stream = Cosmos3Stream(net, StreamPolicy(block_frames=4, sink_frames=1, history_frames=None,
                                             rope=StreamRoPE.ABSOLUTE))
    block = _block_condition(condition, 1, 5)
    sigma = torch.tensor([0.7])
    noisy = rf_interpolate(latent[:, :, 1:5], torch.randn_like(latent[:, :, 1:5]), sigma)
    with pytest.raises(RuntimeError):
        denoise_with_references(stream, noisy, sigma, block, [latent[:, :, :1]])
    stream.start(latent[:, :, :1], _block_condition(condition, 0, 1))
    plain = stream.denoise(noisy, sigma, block)
    assert torch.equal(denoise_with_references(stream, noisy, sigma, block, []), plain)
    before = [(layer.frames, layer.key.clone()) for layer in stream.layers]
    image = torch.randn(1, 48, 1, 8, 8)
    guided = denoise_with_references(stream, noisy, sigma, block, [image, image * 0.5])
    assert guided.shape == plain.shape and torch.isfinite(guided).all()
    assert not torch.allclose(guided, plain, atol=1e-4)
    for layer, (frames, key) in zip(stream.layers, before):
        end = layer.text_tokens + frames * layer.frame_tokens
        assert layer.frames == frames and torch.equal(layer.key[:, :end], key[:, :end])
    assert torch.allclose(stream.denoise(noisy, sigma, block), plain, atol=1e-6)
    with pytest.raises(ValueError):
        denoise_with_references(stream, noisy, sigma, block, [torch.randn(1, 48, 2, 8, 8)])


def test_reset_keeps_the_arenas_and_a_restarted_stream_repeats_its_outputs():
    """A bounded stream that is reset and started again on the same prompt replays the same
    velocities from the kept arenas; ``release=True`` and a changed geometry drop them."""
    cfg = tiny_config()
    net = tiny_network(cfg).eval()
    cond = tiny_conditioner(cfg)
    batch = cond.encode(synthetic_batch(frames=17), training=False)
    condition = cond.condition(batch)
    latent = batch["latent"]
    policy = StreamPolicy(block_frames=4, sink_frames=1, history_frames=8, rope="top_aligned",
                          train_frames=13)
    stream = Cosmos3Stream(net, policy)
    torch.manual_seed(3)
    noise = torch.randn_like(latent)

    def run():
        stream.start(latent[:, :, :1], _block_condition(condition, 0, 1))
        outs = []
        for b in range(4):  # the last two commits evict (an odd number of arena swaps)
            lo, hi = 1 + 4 * b, 5 + 4 * b
            block = _block_condition(condition, lo, hi)
            outs.append(stream.denoise(noise[:, :, lo:hi], torch.tensor([0.8]), block))
            stream.commit(latent[:, :, lo:hi], block)
        return outs

    first = run()
    arenas = [layer.key.data_ptr() for layer in stream.layers]
    stream.reset()
    assert stream.next_frame == 0 and stream.frame_ids == () and stream.text is None
    assert all(layer.frames == 0 for layer in stream.layers) and len(stream.layers) == len(net.layers)
    second = run()
    assert [layer.key.data_ptr() for layer in stream.layers] == arenas
    for a, b in zip(first, second):
        assert torch.equal(a, b)
    stream.reset(release=True)
    assert stream.layers == []
    run()
    stream.reset()
    # another frame geometry cannot reuse the arenas: they are rebuilt on start
    small = cond.condition(cond.encode(synthetic_batch(frames=5, height=4, width=4), training=False))
    stream.start(torch.randn(1, 48, 1, 4, 4), _block_condition(small, 0, 1))
    assert stream.layers[0].frames == 1 and stream.grid == (2, 2)
