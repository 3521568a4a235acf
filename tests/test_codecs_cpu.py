"""Wan 2.2 VAE and the tiny recurrent decoder: shapes, chunk invariance, streaming equivalence."""

import pytest
import torch

from agentgarten_b200.codecs import TAEW22SuperDecoder, Wan22VAECodec
from agentgarten_b200.codecs._taehv.taehv import TAEHV, StreamingTAEHV
from agentgarten_b200.codecs.wan22 import (CausalConv3d, CausalState, Wan22VAE, pixel_fold, pixel_unfold,
                                           random_vae)

ARCH = dict(dim=8, dec_dim=8, z_dim=4)


def test_pixel_fold_layout_and_inverse():
    x = torch.arange(2 * 3 * 2 * 4 * 6, dtype=torch.float32).reshape(2, 3, 2, 4, 6)
    folded = pixel_fold(x)
    assert folded.shape == (2, 12, 2, 2, 3)
    # channel index = (c, column offset, row offset)
    assert torch.equal(folded[:, 0 * 4 + 1 * 2 + 0], x[:, 0, :, 0::2, 1::2])
    assert torch.equal(folded[:, 2 * 4 + 0 * 2 + 1], x[:, 2, :, 1::2, 0::2])
    assert torch.equal(pixel_unfold(folded), x)


def test_causal_conv_chunks_equal_whole_clip():
    torch.manual_seed(0)
    conv = CausalConv3d(3, 5, 3, padding=1)
    x = torch.randn(1, 3, 7, 6, 6)
    whole = conv(x)
    state = CausalState()
    pieces = [conv(x[:, :, a:b], state) for a, b in ((0, 1), (1, 2), (2, 5), (5, 7))]
    assert torch.allclose(torch.cat(pieces, 2), whole, atol=1e-6)
    # nothing from later frames leaks backwards
    y = x.clone()
    y[:, :, 4:] += 1.0
    assert torch.equal(conv(y)[:, :, :4], whole[:, :, :4])


def test_vae_shapes_and_window_invariance():
    codec = Wan22VAECodec(None, dtype="float32", architecture=ARCH)
    video = torch.rand(1, 3, 9, 32, 48) * 2 - 1
    latent = codec.encode(video)
    assert latent.shape == (1, 4, codec.latent_frames(9), 2, 3)
    assert codec.pixel_frames(latent.shape[2]) == 9
    assert codec.decode(latent).shape == video.shape
    vae, scale = codec.stream_components("cpu")
    a = vae.encode(video, scale, temporal_window=4)
    b = vae.encode(video, scale, temporal_window=8)
    assert torch.allclose(a, b, atol=1e-5)
    one = vae.decode(latent, scale, frames_per_pass=1)
    two = vae.decode(latent, scale, frames_per_pass=2)
    assert torch.allclose(one, two, atol=1e-5)


def test_vae_rejects_bad_lengths():
    vae = random_vae(**ARCH)
    scale = (0.0, 1.0)
    with pytest.raises(ValueError):
        vae.encode(torch.zeros(1, 3, 6, 16, 16), scale, temporal_window=4)
    with pytest.raises(ValueError):
        vae.encode(torch.zeros(1, 3, 5, 16, 16), scale, temporal_window=6)
    with pytest.raises(ValueError):
        vae.encode(torch.zeros(3, 5, 16, 16), scale, temporal_window=4)


def test_vae_stream_matches_clip():
    codec = Wan22VAECodec(None, dtype="float32", architecture=ARCH)
    video = torch.rand(1, 3, 13, 16, 16) * 2 - 1
    latent = codec.encode(video)
    stream = codec.stream("cpu")
    online = torch.cat([stream.encode(video[:, :, :5]), stream.encode(video[:, :, 5:])], dim=2)
    assert torch.allclose(online, latent, atol=1e-5)
    pixels = torch.cat([stream.decode(latent[:, :, :2]), stream.decode(latent[:, :, 2:])], dim=2)
    assert torch.allclose(pixels, codec.decode(latent), atol=1e-5)
    stream.reset()
    assert stream.decode(latent[:, :, :1]).shape[2] == 1


def test_vae_state_dict_names_follow_the_released_checkpoint():
    names = set(Wan22VAE(**ARCH).state_dict())
    for key in ("encoder.conv1.weight", "encoder.downsamples.0.downsamples.0.residual.0.gamma",
                "encoder.downsamples.1.downsamples.0.shortcut.weight",
                "encoder.downsamples.1.downsamples.2.time_conv.weight",
                "encoder.downsamples.0.downsamples.2.resample.1.weight",
                "encoder.middle.1.to_qkv.weight", "encoder.head.2.bias", "conv1.weight", "conv2.bias",
                "decoder.upsamples.0.upsamples.3.time_conv.weight",
                "decoder.upsamples.2.upsamples.3.resample.1.bias", "decoder.middle.1.norm.gamma",
                "decoder.head.0.gamma"):
        assert key in names, key


@pytest.mark.parametrize("arch", ["taew2_2_super", "taew2_2"])
def test_tiny_decoder_modes_agree(arch):
    torch.manual_seed(0)
    model = TAEHV(None, arch_name=arch).eval()
    assert (model.patch_size, model.latent_channels, model.t_upscale, model.frames_to_trim) == (2, 48, 4, 3)
    latent = torch.randn(1, 3, 48, 2, 2)
    with torch.no_grad():
        together = model.decode_video(latent, parallel=True)
        serial = model.decode_video(latent, parallel=False)
        assert together.shape == (1, 9, 3, 32, 32)
        assert torch.allclose(together, serial, atol=1e-5)
        stream = StreamingTAEHV(model)
        chunks = torch.cat([stream.decode_chunk(latent[:, :1]), stream.decode_chunk(latent[:, 1:])], dim=1)
        assert torch.allclose(chunks, together, atol=1e-5)
        video = torch.rand(1, 6, 3, 32, 32)
        assert torch.allclose(model.encode_video(video), model.encode_video(video, parallel=False), atol=1e-5)


def test_super_decoder_surface():
    decoder = TAEW22SuperDecoder(None, frames_per_pass=2)
    latent = torch.randn(1, 48, 3, 2, 2)
    video = decoder.decode(latent)
    assert video.shape == (1, 3, 9, 32, 32) and video.min() >= -1 and video.max() <= 1
    stream = decoder.stream("cpu")
    first, rest = stream.decode(latent[:, :, :1]), stream.decode(latent[:, :, 1:])
    assert first.shape[2] == 1 and rest.shape[2] == 8
    assert torch.allclose(torch.cat([first, rest], 2), video, atol=1e-5)
    with pytest.raises(ValueError):
        stream.decode(torch.randn(1, 48, 1, 4, 4))  # shape change without reset
    with pytest.raises(ValueError):
        decoder.decode(torch.randn(1, 16, 1, 2, 2))
    codec = Wan22VAECodec(None, dtype="float32", decoder=decoder)
    assert torch.equal(codec.decode(latent), video)


def test_convolution_helpers_fall_back_to_the_library_definition():
    """Off the GPU the convolution helpers are the plain convolutions with the epilogue applied."""
    from agentgarten_b200.ops.conv import conv_frames, conv_volume, depthwise_frames, eligible, packed_weight

    torch.manual_seed(0)
    conv = torch.nn.Conv3d(8, 16, 3, padding=(0, 1, 1))
    x = torch.randn(1, 8, 4, 6, 7)
    residual = torch.randn(1, 16, 2, 6, 7)
    assert not eligible(conv, x)
    with torch.no_grad():
        want = torch.relu(conv(x) + residual)
        assert torch.equal(conv_volume(conv, x, residual, relu=True), want)
        frames = torch.nn.Conv2d(8, 12, 3, padding=1)
        y = torch.randn(2, 8, 5, 5)
        assert torch.equal(conv_frames(frames, y), frames(y))
        deep = torch.nn.Conv2d(8, 8, 7, padding=3, groups=8, bias=False)
        assert torch.equal(depthwise_frames(deep, y), deep(y))
    # the kernel layout of a weight: [Cout rounded up to 8, taps, Cin], taps in (t, h, w) order
    packed, bias = packed_weight(frames, torch.float32)
    assert packed.shape == (16, 9, 8) and bias.shape == (16,)
    assert torch.equal(packed[:12, 4], frames.weight[:, :, 1, 1]) and not packed[12:].any()


def test_channels_last_forms_of_the_shortcuts_match_the_planar_forms():
    """The parameter-free shortcuts and the temporal interleave have a path for channels-last
    volumes (what the convolution kernels produce); it computes the same values and keeps the layout."""
    from agentgarten_b200.codecs.wan22 import AverageDown, CausalState, DuplicateUp, Resample, _channels_last

    torch.manual_seed(0)
    for cin, cout, ft in ((16, 16, 2), (16, 8, 2), (32, 8, 1), (16, 16, 1)):
        up = DuplicateUp(cin, cout, ft, 2)
        x = torch.randn(2, cin, 3, 4, 5)
        packed = x.contiguous(memory_format=torch.channels_last_3d)
        for first in (False, True):
            got = up(packed, first=first)
            assert torch.equal(got, up(x, first=first))
        assert _channels_last(up(packed))
    for cin, cout, ft, frames in ((8, 16, 2, 4), (8, 8, 1, 3), (16, 16, 2, 3), (8, 32, 2, 2)):
        down = AverageDown(cin, cout, ft, 2)
        x = torch.randn(2, cin, frames, 4, 6)
        got = down(x.contiguous(memory_format=torch.channels_last_3d))
        assert _channels_last(got) and torch.allclose(got, down(x), atol=1e-6)
    resample = Resample(8, "upsample3d")
    x = torch.randn(1, 8, 3, 4, 5)
    outputs = []
    for value in (x, x.contiguous(memory_format=torch.channels_last_3d)):
        state = CausalState()
        state.advance()  # past the first chunk: the temporal doubling is active
        outputs.append(resample(value, state))
    assert outputs[0].shape == (1, 8, 6, 8, 10) and torch.allclose(outputs[0], outputs[1], atol=1e-6)
