"""Per-kernel timings against the measured roofline.

``python -m agentgarten_b200.ops.microbench [--op conv gemm attention ...] [--tokens N] [--json]``

Each case is timed with CUDA events on the launching stream after three warm-up launches;
between timed launches a 256 MB buffer is rewritten so nothing is served from the 126 MB
L2. Throughput is reported in absolute units and, when ``MEASURED_PEAKS.json`` sits at the
repository root, as a fraction of the measured cuBLAS bf16 rate (tensor-core kernels) or of
the measured copy bandwidth (memory-bound kernels).  ``--launches N`` limits the timed
launches (useful under a profiler, which wants few, small launches).
"""

from __future__ import annotations

import argparse
import json
import statistics
from pathlib import Path

import torch

from agentgarten_b200 import ops
from agentgarten_b200.ops import native

_FLUSH = None


def _flush_l2() -> None:
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.fill_(1)


def _time(fn, launches: int) -> float:
    """Median milliseconds of ``fn`` over ``launches`` timed calls."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    samples = []
    for _ in range(launches):
        _flush_l2()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        samples.append(start.elapsed_time(stop))
    return statistics.median(samples)


def _peaks() -> dict:
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return {"tflops": float(data.get("bf16_tflops", 0) or 0), "gbs": float(data.get("hbm_gbs", 0) or 0),
                "source": "measured"}
    return {"tflops": 1590.0, "gbs": 6650.0, "source": "fallback"}


def bench_gemm(tokens: int, launches: int) -> list[dict]:
    out = []
    for name, (n, k) in {"qkv 4096->6144": (6144, 4096), "mlp up 4096->12288": (12288, 4096),
                         "mlp down 12288->4096": (4096, 12288)}.items():
        a = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
        ms = _time(lambda: ops.linear(a, w), launches)
        out.append({"kernel": "gemm_kernel", "case": f"{name}, {tokens} rows", "ms": ms,
                    "tflops": 2.0 * tokens * n * k / ms / 1e9})
    return out


def bench_attention(tokens: int, launches: int, heads: int = 32, kv_heads: int = 8) -> list[dict]:
    from agentgarten_b200.ops import attention_native

    q = torch.randn(1, tokens, heads, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(1, tokens, kv_heads, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(1, tokens, kv_heads, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    flops = 4.0 * tokens * tokens * heads * 128
    with torch.no_grad():
        fwd = _time(lambda: attention_native.dense(q, k, v), launches)
    result = attention_native.dense(q, k, v)
    grad = torch.randn_like(result)

    def backward():
        torch.autograd.grad(result, (q, k, v), grad, retain_graph=True)

    bwd = _time(backward, launches)
    case = f"{tokens} tokens, {heads}/{kv_heads} heads x 128, dense"
    return [{"kernel": "attn_fwd_kernel", "case": case, "ms": fwd, "tflops": flops / fwd / 1e9},
            {"kernel": "attn_delta + attn_dq + attn_dkv", "case": case, "ms": bwd,
             "tflops": 2.5 * flops / bwd / 1e9}]


def bench_jvp(tokens: int, launches: int, heads: int = 32, kv_heads: int = 8) -> list[dict]:
    from agentgarten_b200.ops.attention import attention_jvp

    q, tq = (torch.randn(1, tokens, heads, 128, device="cuda", dtype=torch.bfloat16) for _ in range(2))
    k, v, tk, tv = (torch.randn(1, tokens, kv_heads, 128, device="cuda", dtype=torch.bfloat16)
                    for _ in range(4))
    ms = _time(lambda: attention_jvp(q, k, v, tq, tk, tv), launches)
    flops = 3.0 * 4.0 * tokens * tokens * heads * 128  # six products against the forward's two
    return [{"kernel": "attn_jvp_kernel", "case": f"{tokens} tokens, {heads}/{kv_heads} heads x 128, dense",
             "ms": ms, "tflops": flops / ms / 1e9}]


def bench_pointwise(tokens: int, launches: int) -> list[dict]:
    out = []
    x = torch.randn(tokens, 4096, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(4096, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: ops.rms_norm(x, w, 1e-6), launches)
    out.append({"kernel": "rms_norm_fwd", "case": f"{tokens} x 4096", "ms": ms,
                "gbs": 2 * x.numel() * 2 / ms / 1e6})
    gate = torch.randn(tokens, 12288, device="cuda", dtype=torch.bfloat16)
    up = torch.randn_like(gate)
    ms = _time(lambda: ops.silu_mul(gate, up), launches)
    out.append({"kernel": "silu_mul_fwd", "case": f"{tokens} x 12288", "ms": ms,
                "gbs": 3 * gate.numel() * 2 / ms / 1e6})
    return out


def bench_conv(tokens: int, launches: int) -> list[dict]:
    """3x3x3 convolutions at the shapes of the Wan 2.2 decoder levels, against cuDNN on the same input."""
    out = []
    for channels, frames, height, width in ((256, 4, 240, 416), (512, 4, 120, 208), (1024, 2, 60, 104)):
        x = torch.randn(1, frames + 2, height, width, channels, device="cuda", dtype=torch.bfloat16)
        weight = torch.randn(channels, channels, 3, 3, 3, device="cuda", dtype=torch.bfloat16) * 0.01
        packed = weight.permute(0, 2, 3, 4, 1).reshape(channels, 27, channels).contiguous()
        ms = _time(lambda: native.ext().conv3d(x, packed, None, None, 3, 3, 3, False, None, False), launches)
        logical = x.permute(0, 4, 1, 2, 3)
        cl_weight = weight.contiguous(memory_format=torch.channels_last_3d)
        library = _time(lambda: torch.nn.functional.conv3d(logical, cl_weight, padding=(0, 1, 1)), launches)
        flops = 2.0 * frames * height * width * 27 * channels * channels
        out.append({"kernel": "conv3d_kernel", "case": f"{channels} ch, {frames} frames {height}x{width}, 3x3x3",
                    "ms": ms, "tflops": flops / ms / 1e9, "cudnn_ms": library})
    return out


def bench_depthwise(tokens: int, launches: int) -> list[dict]:
    """7x7 depthwise convolutions of the wide TAEHV decoder (fp16), against cuDNN / ATen."""
    out = []
    for channels, frames, height, width in ((256, 4, 240, 416), (512, 4, 120, 208), (1024, 4, 60, 104)):
        conv = torch.nn.Conv2d(channels, channels, 7, padding=3, groups=channels, bias=False)
        conv = conv.to("cuda", torch.float16).to(memory_format=torch.channels_last)
        x = torch.randn(frames, channels, height, width, device="cuda", dtype=torch.float16)
        x = x.contiguous(memory_format=torch.channels_last)
        from agentgarten_b200.ops.conv import depthwise_frames

        with torch.no_grad():
            ms = _time(lambda: depthwise_frames(conv, x), launches)
            library = _time(lambda: conv(x), launches)
        out.append({"kernel": "depthwise_kernel", "case": f"{channels} ch, {frames} x {height}x{width}, 7x7 fp16",
                    "ms": ms, "gbs": 2 * x.numel() * 2 / ms / 1e6, "cudnn_ms": library})
    return out


def bench_codec(tokens: int, launches: int) -> list[dict]:
    """Whole decoders on random weights: Wan 2.2 VAE (bf16) and the TAEHV decoders (fp16) on three
    latent frames of 30x52 (nine 480x832 pixel frames), with this package's convolution kernels
    and with the library convolutions (``AGB200_LIBRARY_CONV=1``)."""
    import os

    from agentgarten_b200.codecs._taehv.taehv import TAEHV
    from agentgarten_b200.codecs.wan22 import random_vae, to_channels_last

    out = []
    latent = torch.randn(1, 48, 3, 30, 52, device="cuda")

    def both(name, fn):
        row = {"kernel": "conv3d_kernel + pointwise", "case": name}
        for key, flag in (("ms", "0"), ("cudnn_ms", "1")):
            os.environ["AGB200_LIBRARY_CONV"] = flag
            with torch.no_grad():
                row[key] = _time(fn, max(2, launches // 2))
        os.environ.pop("AGB200_LIBRARY_CONV", None)
        row["frames_per_s"] = 9 / row["ms"] * 1e3
        out.append(row)

    vae = to_channels_last(random_vae(seed=0).to("cuda", torch.bfloat16)).eval()
    z = latent.bfloat16()
    both("Wan 2.2 VAE decoder, 3 latent frames 30x52", lambda: vae.decode(z, (0.0, 1.0), frames_per_pass=2))
    for name in ("taew2_2", "taew2_2_super"):
        tiny = TAEHV(checkpoint_path=None, arch_name=name).eval()
        tiny = tiny.to("cuda", torch.float16).to(memory_format=torch.channels_last)
        frames = latent.transpose(1, 2).half()
        both(f"TAEHV {name} decoder, 3 latent frames 30x52",
             lambda: tiny.decode_video(frames, parallel=True, show_progress_bar=False))
    return out


def bench_mma_rate(tokens: int, launches: int) -> list[dict]:
    """Cycles per tcgen05.mma instruction (M 128, K 16) issued back to back: the figure the
    attention kernels' tile shapes are chosen from.  ``tflops`` is what that rate gives on all SMs
    at the maximum SM clock."""
    out = []
    C = native.ext()
    mhz = 1965.0   # the part's maximum SM clock; under the power cap a long kernel sees 1.5-1.7 GHz
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for columns, from_tmem in ((64, False), (128, False), (256, False), (64, True), (128, True)):
        C.mma_issue_rate(columns, from_tmem, 16)
        cycles = C.mma_issue_rate(columns, from_tmem, 256)
        flops_per_cycle = 2.0 * 128 * columns * 16 / cycles
        out.append({"kernel": "tcgen05.mma issue rate", "ms": cycles,
                    "case": f"M128 N{columns} K16, A from {'TMEM' if from_tmem else 'smem'}: cycles per instruction in the ms column",
                    "tflops": flops_per_cycle * sms * mhz * 1e6 / 1e12})
    return out


CASES = {"mma_rate": bench_mma_rate, "codec": bench_codec, "conv": bench_conv, "depthwise": bench_depthwise, "gemm": bench_gemm, "attention": bench_attention, "jvp": bench_jvp, "pointwise": bench_pointwise}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--op", nargs="*", default=[c for c in CASES if c not in ("codec", "mma_rate")], choices=list(CASES))
    parser.add_argument("--tokens", type=int, default=8192)
    parser.add_argument("--launches", type=int, default=10)
    parser.add_argument("--json", action="store_true")
    args = parser.parse_args(argv)
    native.require()
    peaks = _peaks()
    rows = []
    for name in args.op:
        rows += CASES[name](args.tokens, args.launches)
    for row in rows:
        if "tflops" in row and peaks["tflops"]:
            row["fraction"] = row["tflops"] / peaks["tflops"]
        if "gbs" in row and peaks["gbs"]:
            row["fraction"] = row["gbs"] / peaks["gbs"]
        row["of"] = f"of {peaks['source']}"
    if args.json:
        print(json.dumps({"peaks": peaks, "rows": rows, "launches": native.launches()}))
    else:
        for row in rows:
            if "frames_per_s" in row:
                rate = f"{row['frames_per_s']:8.1f} frames/s"
            elif "tflops" in row:
                rate = f"{row['tflops']:8.1f} TFLOP/s"
            else:
                rate = f"{row['gbs']:8.1f} GB/s   "
            extra = f"  (cuDNN {row['cudnn_ms']:.3f} ms)" if "cudnn_ms" in row else ""
            print(f"{row['kernel']:34s} {row['case']:46s} {row['ms']:8.3f} ms {rate} "
                  f"{row.get('fraction', 0):5.2f} {row['of']}{extra}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
