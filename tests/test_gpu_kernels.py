"""sm_100a kernels against plain PyTorch fp32 references of the same operators."""

import pytest
import torch

from agentgarten_b200 import ops
from agentgarten_b200.ops import native, reference
from agentgarten_b200.ops.linear import gemm

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _status_ok():
    torch.cuda.synchronize()
    assert int(native.ext().status(torch.cuda.current_device()).item()) == 0


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 520, 192), (1000, 1024, 4096), (514, 192, 4096)])
@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False), (True, True)])
def test_gemm_layouts(m, n, k, trans_a, trans_b):
    torch.manual_seed(0)
    if trans_a and m % 8:
        m = (m + 7) // 8 * 8
    a = torch.randn((k, m) if trans_a else (m, k), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((n, k) if trans_b else (k, n), device=DEV, dtype=torch.bfloat16)
    out = gemm(a, b, trans_a=trans_a, trans_b=trans_b)
    ref = (a.float().t() if trans_a else a.float()) @ (b.float().t() if trans_b else b.float())
    _status_ok()
    assert out.shape == ref.shape
    assert _rel(out, ref) < 4e-3


def test_gemm_epilogues():
    torch.manual_seed(1)
    m, n, k = 333, 384, 256
    a = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(n, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(m, n, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ w.float().t()
    out = gemm(a, w, bias=bias, residual=res)
    assert _rel(out, ref + bias.float() + res.float()) < 4e-3
    acc = torch.randn(m, n, device=DEV, dtype=torch.float32)
    expect = acc + ref
    gemm(a, w, out=acc, accumulate=True)
    assert _rel(acc, expect) < 1e-3
    accb = torch.randn(m, n, device=DEV, dtype=torch.bfloat16)
    expect = accb.float() + ref
    gemm(a, w, out=accb, accumulate=True)
    assert _rel(accb, expect) < 4e-3
    _status_ok()


def test_gemm_row_invariance():
    torch.manual_seed(2)
    a = torch.randn(700, 512, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(768, 512, device=DEV, dtype=torch.bfloat16)
    whole = gemm(a, w)
    part = gemm(a[130:391].contiguous(), w)
    assert torch.equal(whole[130:391], part)


@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False)])
def test_gemm_on_cta_pairs_matches_single_cta_tiles(trans_a, trans_b, monkeypatch):
    """Enough 256 x 256 tiles for one per pair of SMs sends a product to the two-SM kernel
    (tcgen05 cta_group::2): ragged edges, both operand layouts and every epilogue give bit for
    bit what the single-CTA kernel gives, and both agree with an fp32 product."""
    torch.manual_seed(21)
    m, n, k = 2312, 2328, 320          # 10 x 10 tiles with ragged last rows and columns
    a = torch.randn((k, m) if trans_a else (m, k), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((n, k) if trans_b else (k, n), device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(n, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(m, n, device=DEV, dtype=torch.bfloat16)
    start32 = torch.randn(m, n, device=DEV, dtype=torch.float32)
    start16 = torch.randn(m, n, device=DEV, dtype=torch.bfloat16)

    def run():
        plain = gemm(a, b, trans_a=trans_a, trans_b=trans_b)
        fused = gemm(a, b, trans_a=trans_a, trans_b=trans_b, bias=bias, residual=res)
        acc32, acc16 = start32.clone(), start16.clone()
        gemm(a, b, trans_a=trans_a, trans_b=trans_b, out=acc32, accumulate=True)
        gemm(a, b, trans_a=trans_a, trans_b=trans_b, out=acc16, accumulate=True)
        torch.cuda.synchronize()
        return plain, fused, acc32, acc16

    monkeypatch.setenv("AGB200_GEMM_PAIRS", "1")
    pairs = run()
    monkeypatch.setenv("AGB200_GEMM_PAIRS", "0")
    single = run()
    _status_ok()
    ref = (a.float().t() if trans_a else a.float()) @ (b.float().t() if trans_b else b.float())
    assert _rel(pairs[0], ref) < 4e-3
    assert _rel(pairs[1], ref + bias.float() + res.float()) < 4e-3
    assert _rel(pairs[2], start32 + ref) < 1e-3
    assert _rel(pairs[3], start16.float() + ref) < 4e-3
    for got, want in zip(pairs, single):
        assert torch.equal(got, want)


def test_linear_autograd():
    torch.manual_seed(3)
    x = torch.randn(2, 100, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(512, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = ops.linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    assert _rel(y, yr) < 4e-3
    assert _rel(x.grad, xr.grad) < 4e-3
    assert _rel(w.grad, wr.grad) < 4e-3
    assert _rel(b.grad, br.grad) < 1e-2
    _status_ok()


@pytest.mark.parametrize("rows,width", [(37, 256), (1000, 4096)])
def test_rms_norm(rows, width):
    torch.manual_seed(4)
    x = torch.randn(rows, width, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(width, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    y = ops.rms_norm(x, w, 1e-6)
    assert torch.equal(y, reference.rms_norm(x.detach(), w.detach(), 1e-6))
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = (t.detach().float().requires_grad_(True) for t in (x, w))
    reference.rms_norm(xr, wr, 1e-6).backward(g.float())
    assert _rel(x.grad, xr.grad) < 1e-2
    assert _rel(w.grad, wr.grad) < 1e-2
    total, normed = ops.rms_norm_add(x.detach(), g, w.detach(), 1e-6)
    tr, nr = reference.rms_norm_add(x.detach(), g, w.detach(), 1e-6)
    assert torch.equal(total, tr) and torch.equal(normed, nr)


def test_head_norm_rope():
    torch.manual_seed(5)
    b, n, h = 2, 77, 4
    x = torch.randn(b, n, h, 128, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(128, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    ang = torch.randn(b, n, 64, device=DEV) * 3
    cos = torch.cat((ang, ang), -1).cos().to(torch.bfloat16)
    sin = torch.cat((ang, ang), -1).sin().to(torch.bfloat16)
    y = ops.head_norm_rope(x, w, cos, sin, 1e-6)
    yr = reference.head_norm_rope(x.detach(), w.detach(), cos, sin, 1e-6)
    assert (y.float() - yr.float()).abs().max() <= 2 * 2 ** -8 * yr.float().abs().max()
    assert _rel(y, yr) < 3e-3
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = (t.detach().float().requires_grad_(True) for t in (x, w))
    reference.head_norm_rope(xr, wr, cos.float(), sin.float(), 1e-6).backward(g.float())
    assert _rel(x.grad, xr.grad) < 1e-2
    assert _rel(w.grad, wr.grad) < 1e-2


def test_silu_mul():
    torch.manual_seed(6)
    a = torch.randn(123, 1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(123, 1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = ops.silu_mul(a, b)
    yr = reference.silu_mul(a.detach(), b.detach())
    assert _rel(y, yr) < 3e-3
    g = torch.randn_like(y)
    y.backward(g)
    ar, br = (t.detach().float().requires_grad_(True) for t in (a, b))
    reference.silu_mul(ar, br).backward(g.float())
    assert _rel(a.grad, ar.grad) < 1e-2 and _rel(b.grad, br.grad) < 1e-2


def test_rf_combine():
    torch.manual_seed(7)
    x0 = torch.randn(2, 48, 5, 6, 8, device=DEV)
    noise = torch.randn_like(x0)
    for sigma in (torch.rand(2, device=DEV), torch.rand(2, 5, device=DEV)):
        with torch.no_grad():
            assert torch.allclose(ops.rf_interpolate(x0, noise, sigma),
                                  reference.rf_interpolate(x0, noise, sigma), atol=1e-6)
            assert torch.allclose(ops.rf_x0(x0, sigma, noise), reference.rf_x0(x0, sigma, noise), atol=1e-6)


def _attention_inputs(b, nq, nk, hq, hkv, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    q = torch.randn(b, nq, hq, 128, device=DEV, dtype=torch.bfloat16, generator=g)
    k = torch.randn(b, nk, hkv, 128, device=DEV, dtype=torch.bfloat16, generator=g)
    v = torch.randn(b, nk, hkv, 128, device=DEV, dtype=torch.bfloat16, generator=g)
    return q, k, v


@pytest.mark.parametrize("nq,nk", [(128, 128), (200, 333), (517, 1100)])
@pytest.mark.parametrize("causal", [False, True])
def test_attention_dense_forward(nq, nk, causal):
    if causal:
        nk = nq
    q, k, v = _attention_inputs(2, nq, nk, 4, 2, 10)
    with torch.no_grad():
        out = ops.attention(q, k, v, causal=causal)
        ref = reference.attention(q.float(), k.float(), v.float(), causal=causal)
    _status_ok()
    assert _rel(out, ref) < 6e-3
    assert (out.float() - ref).abs().max() < 3e-2


def test_attention_planned_forward_with_text():
    torch.manual_seed(11)
    b, hq, hkv = 2, 4, 2
    sizes = [130, 260, 260, 96]
    g = torch.Generator(device=DEV).manual_seed(12)
    mk = lambda n, h: torch.randn(b, n, h, 128, device=DEV, dtype=torch.bfloat16, generator=g)
    queries = [mk(n, hq) for n in sizes]
    keys = [mk(n, hkv) for n in sizes]
    values = [mk(n, hkv) for n in sizes]
    text_k, text_v = mk(48, hkv), mk(48, hkv)
    valid = torch.tensor([17, 48], device=DEV)
    plan = [[0], [0, 1], [0, 1, 2], [0, 2, 3]]
    with torch.no_grad():
        outs = ops.planned_attention(queries, keys, values, plan, text_keys=text_k,
                                     text_values=text_v, text_valid=valid)
    _status_ok()
    for i, visible in enumerate(plan):
        kk = torch.cat([text_k, *[keys[j] for j in visible]], 1).float()
        vv = torch.cat([text_v, *[values[j] for j in visible]], 1).float()
        mask = torch.ones(b, kk.shape[1], dtype=torch.bool, device=DEV)
        mask[:, :48] = torch.arange(48, device=DEV)[None] < valid[:, None]
        ref = reference.attention(queries[i].float(), kk, vv, mask)
        assert _rel(outs[i], ref) < 6e-3, i


def test_attention_chunk_invariance():
    """A query chunk gives bitwise the same output alone or next to other chunks."""
    b, hq, hkv = 1, 4, 2
    g = torch.Generator(device=DEV).manual_seed(13)
    mk = lambda n, h: torch.randn(b, n, h, 128, device=DEV, dtype=torch.bfloat16, generator=g)
    queries = [mk(150, hq), mk(300, hq)]
    keys = [mk(150, hkv), mk(300, hkv)]
    values = [mk(150, hkv), mk(300, hkv)]
    with torch.no_grad():
        both = ops.planned_attention(queries, keys, values, [[0], [0, 1]])
        alone = ops.planned_attention([queries[1]], keys, values, [[0, 1]])
    assert torch.equal(both[1], alone[0])


@pytest.fixture(params=["fused", "split"])
def backward_form(request, monkeypatch):
    """Both forms of the attention backward: one pass over the scores, or the dQ and dK/dV kernels."""
    monkeypatch.setenv("AGB200_ATTN_BWD", request.param)
    return request.param


def test_one_pass_backward_is_bit_reproducible_and_matches_the_two_kernel_form(monkeypatch):
    """Many key tiles add to every query block (the order is fixed by the turn counters): two runs
    agree bit for bit, and the result agrees with the two-kernel form to bf16 rounding."""
    q, k, v = _attention_inputs(2, 1000, 1210, 8, 2, 31)
    q, k, v = (t.requires_grad_(True) for t in (q, k, v))
    grad = torch.randn(2, 1000, 8, 128, device=DEV, dtype=torch.bfloat16)

    def run(form):
        monkeypatch.setenv("AGB200_ATTN_BWD", form)
        out = ops.attention(q, k, v)
        return torch.autograd.grad(out, (q, k, v), grad)

    first, second, split = run("fused"), run("fused"), run("split")
    _status_ok()
    for a, b in zip(first, second):
        assert torch.equal(a, b)
    for a, b in zip(first, split):
        assert _rel(a, b) < 1e-2


def test_attention_backward_dense(backward_form):
    q, k, v = _attention_inputs(2, 300, 420, 4, 2, 20)
    q, k, v = (t.requires_grad_(True) for t in (q, k, v))
    out = ops.attention(q, k, v)
    g = torch.randn_like(out)
    out.backward(g)
    _status_ok()
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    reference.attention(qr, kr, vr).backward(g.float())
    assert _rel(q.grad, qr.grad) < 2e-2
    assert _rel(k.grad, kr.grad) < 2e-2
    assert _rel(v.grad, vr.grad) < 2e-2


def test_attention_backward_planned_with_text(backward_form):
    b, hq, hkv = 2, 4, 2
    sizes = [130, 260, 96]
    g = torch.Generator(device=DEV).manual_seed(21)
    mk = lambda n, h: torch.randn(b, n, h, 128, device=DEV, dtype=torch.bfloat16, generator=g)
    queries = [mk(n, hq).requires_grad_(True) for n in sizes]
    keys = [mk(n, hkv).requires_grad_(True) for n in sizes]
    values = [mk(n, hkv).requires_grad_(True) for n in sizes]
    text_k, text_v = mk(48, hkv), mk(48, hkv)
    valid = torch.tensor([17, 48], device=DEV)
    plan = [[0], [0, 1], [0, 2]]
    outs = ops.planned_attention(queries, keys, values, plan, text_keys=text_k,
                                 text_values=text_v, text_valid=valid)
    grads = [torch.randn_like(o) for o in outs]
    torch.autograd.backward(outs, grads)
    _status_ok()
    qs = [t.detach().float().requires_grad_(True) for t in queries]
    ks = [t.detach().float().requires_grad_(True) for t in keys]
    vs = [t.detach().float().requires_grad_(True) for t in values]
    for i, visible in enumerate(plan):
        kk = torch.cat([text_k.float(), *[ks[j] for j in visible]], 1)
        vv = torch.cat([text_v.float(), *[vs[j] for j in visible]], 1)
        mask = torch.ones(b, kk.shape[1], dtype=torch.bool, device=DEV)
        mask[:, :48] = torch.arange(48, device=DEV)[None] < valid[:, None]
        reference.attention(qs[i], kk, vv, mask).backward(grads[i].float())
    for mine, ref in zip([*queries, *keys, *values], [*qs, *ks, *vs]):
        assert _rel(mine.grad, ref.grad) < 2e-2


@pytest.mark.parametrize("nq,nk,text_len,valid", [(256, 320, 0, None), (200, 450, 0, None),
                                                   (130, 300, 96, (96, 17)), (64, 64, 64, (5, 64))])
def test_attention_jvp_kernel_matches_fp64(nq, nk, text_len, valid):
    from agentgarten_b200.ops import reference
    from agentgarten_b200.ops.attention import attention_jvp

    torch.manual_seed(nq + nk)
    batch, hq, hkv = 2, 4, 2
    q, tq = (torch.randn(batch, nq, hq, 128, device=DEV).bfloat16() for _ in range(2))
    k, v, tk, tv = (torch.randn(batch, nk, hkv, 128, device=DEV).bfloat16() for _ in range(4))
    mask, prefix = None, None
    if valid is not None:
        lengths = torch.tensor(valid, device=DEV)
        mask = torch.ones(batch, nk, dtype=torch.bool, device=DEV)
        mask[:, :text_len] = torch.arange(text_len, device=DEV)[None] < lengths[:, None]
        prefix = (text_len, lengths)
    out, tangent = attention_jvp(q, k, v, tq, tk, tv, key_mask=mask, prefix=prefix)
    want, want_tangent = reference.attention_jvp(q, k, v, tq, tk, tv, mask)
    assert out.dtype == torch.float32 and tangent.dtype == torch.float32
    assert _rel(out, want) < 1e-2, _rel(out, want)
    assert _rel(tangent, want_tangent) < 2e-2, _rel(tangent, want_tangent)
    assert int(native.ext().status(0).item()) == 0


def test_forward_mode_through_the_attention_op_uses_the_kernel():
    import torch.autograd.forward_ad as fwAD

    from agentgarten_b200 import ops
    from agentgarten_b200.ops import reference

    torch.manual_seed(0)
    q, tq = (torch.randn(1, 192, 4, 128, device=DEV).bfloat16() for _ in range(2))
    k, v, tk, tv = (torch.randn(1, 256, 2, 128, device=DEV).bfloat16() for _ in range(4))
    before = native.launches()
    with fwAD.dual_level():
        out = ops.attention(fwAD.make_dual(q, tq), fwAD.make_dual(k, tk), fwAD.make_dual(v, tv))
        primal, tangent = fwAD.unpack_dual(out)
    assert native.launches() > before
    want, want_tangent = reference.attention_jvp(q, k, v, tq, tk, tv)
    assert _rel(primal, want) < 2e-2 and _rel(tangent, want_tangent) < 3e-2


def test_linear_forward_mode_runs_on_the_gemm_kernel():
    """A dual input (and a dual weight) go through the tcgen05 GEMM: tangent = dx W^T + x dW^T."""
    import torch.autograd.forward_ad as fwAD

    from agentgarten_b200.ops.linear import linear

    g = torch.Generator(device=DEV).manual_seed(4)
    x, dx = (torch.randn(3, 50, 256, device=DEV, generator=g).bfloat16() for _ in range(2))
    w, dw = (torch.randn(384, 256, device=DEV, generator=g).bfloat16() * 0.1 for _ in range(2))
    b = torch.randn(384, device=DEV, generator=g).bfloat16()
    before = native.launches()
    with torch.no_grad(), fwAD.dual_level():
        out = linear(fwAD.make_dual(x, dx), fwAD.make_dual(w, dw), b)
        primal, tangent = fwAD.unpack_dual(out)
    assert native.launches() - before >= 3
    want = x.float() @ w.float().t() + b.float()
    want_tangent = dx.float() @ w.float().t() + x.float() @ dw.float().t()
    assert _rel(primal, want) < 1e-2 and _rel(tangent, want_tangent) < 2e-2
    with torch.no_grad(), fwAD.dual_level():
        only_x = fwAD.unpack_dual(linear(fwAD.make_dual(x, dx), w, None)).tangent
    assert _rel(only_x, dx.float() @ w.float().t()) < 1e-2


def test_a_peer_that_never_arrives_ends_the_wait_with_a_status():
    """A gather-GEMM whose input rows are never announced gives up after its bounded wait,
    records the peer-timeout code and leaves the context usable."""
    C = native.ext()
    torch.cuda.synchronize()
    status = C.status(0)
    status.zero_()
    a = torch.randn(256, 256, device=DEV).bfloat16()
    w = torch.randn(512, 256, device=DEV).bfloat16()
    out = torch.empty(256, 512, device=DEV, dtype=torch.bfloat16)
    ready = torch.zeros(2, dtype=torch.int32, device=DEV)   # nothing ever advances these
    seen = torch.zeros(2, dtype=torch.int32, device=DEV)
    ticket = torch.zeros(1, dtype=torch.int32, device=DEV)
    C.tp_gemm(a, w, out, 0, 1, ready, seen, ticket, [], [], 0)
    torch.cuda.synchronize()
    assert int(status.item()) == 5  # kTimeoutPeer
    # the production readers see it: the update consensus and the checkpoint guard raise
    from agentgarten_b200.infra.nonfinite import synchronize_found_nonfinite
    from agentgarten_b200.ops import kernel_status

    weight = torch.nn.Parameter(torch.ones(4, device=DEV))
    weight.grad = torch.ones(4, device=DEV)
    with pytest.raises(kernel_status.KernelStatusError, match="kTimeoutPeer"):
        synchronize_found_nonfinite(None, (torch.optim.SGD([weight], lr=0.1),), fallback_device=DEV)
    assert kernel_status.read(DEV) == 5
    status.zero_()
    # the same call completes once the rows are announced, and ordinary kernels still run
    ready.fill_(128)
    seen.zero_()
    ticket.zero_()
    C.tp_gemm(a, w, out, 0, 1, ready, seen, ticket, [], [], 0)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert _rel(out, a.float() @ w.float().t()) < 1e-2
    assert seen.tolist() == [128, 128]


def test_a_work_list_entry_outside_its_tensor_is_refused_by_the_kernel():
    """The attention kernels check the entries of their host-built work lists against the
    extents of their tensors before the first access: a key segment that reaches past the keys
    makes the CTAs record kBadIndex and skip their work (no access through the bad entry); the
    context stays usable and the same call with a sound list runs."""
    from agentgarten_b200.ops.attention import build_schedule

    C = native.ext()
    torch.cuda.synchronize()
    status = C.status(0)
    status.zero_()
    q, k, v = _attention_inputs(1, 256, 256, 2, 1, 40)
    schedule = build_schedule([256], [256], [[0]], 0, q.device)
    entries = schedule.entries.clone()
    entries[0, 2] = 384              # 384 keys claimed, 256 exist (a tiled load past them would read zeros)
    C.attn_fwd(q, k, v, None, None, None, schedule.q_tiles, entries, 128 ** -0.5, 1)
    torch.cuda.synchronize()
    assert int(status.item()) == 7   # kBadIndex
    status.zero_()
    out, _ = C.attn_fwd(q, k, v, None, None, None, schedule.q_tiles, schedule.entries, 128 ** -0.5, 1)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert _rel(out, reference.attention(q.float(), k.float(), v.float())) < 1e-2


@pytest.mark.parametrize("nq,nk,hq,hkv", [(300, 5000, 4, 1), (128, 12000, 8, 2), (3120, 20000, 4, 1)])
def test_split_key_attention_matches_reference(nq, nk, hq, hkv):
    from agentgarten_b200.ops import attention_native

    torch.manual_seed(nq)
    q = torch.randn(1, nq, hq, 128, device=DEV).bfloat16()
    k = torch.randn(1, nk, hkv, 128, device=DEV).bfloat16()
    v = torch.randn(1, nk, hkv, 128, device=DEV).bfloat16()
    assert attention_native._key_splits(1, nq, nk, hq, hkv, q.device) > 1
    with torch.no_grad():
        out = attention_native.dense(q, k, v)
    want = reference.attention(q.float(), k.float(), v.float(), None)
    assert _rel(out, want) < 1e-2, _rel(out, want)
    _status_ok()


@pytest.mark.parametrize("channels,silu", [(160, True), (1024, False), (8, True), (640, True)])
def test_channel_norm_kernel(channels, silu):
    torch.manual_seed(channels)
    x = torch.randn(2, 3, 5, 7, channels, device=DEV).bfloat16()
    gamma = torch.rand(channels, device=DEV) + 0.5
    out = native.ext().channel_norm(x, gamma, silu)
    wide = x.float()
    want = wide / wide.norm(dim=-1, keepdim=True).clamp_min(1e-12) * channels ** 0.5 * gamma
    if silu:
        want = torch.nn.functional.silu(want)
    assert _rel(out, want) < 5e-3, _rel(out, want)
    _status_ok()


@pytest.mark.parametrize("cin,cout,kernel,frames,height,width,extras", [
    (64, 64, (3, 3, 3), 5, 16, 24, False),
    (160, 320, (3, 3, 3), 4, 30, 52, True),     # ragged channel block, two column tiles, ragged patches
    (32, 48, (1, 3, 3), 3, 8, 8, True),         # frames smaller than a patch
    (96, 200, (1, 1, 1), 2, 9, 130, False),     # pointwise; output channels padded to the tile
    (64, 128, (3, 1, 1), 6, 12, 20, True),      # temporal kernel only
    (256, 256, (3, 3, 3), 3, 24, 40, True),
])
@pytest.mark.parametrize("dtype,relu", [(torch.bfloat16, False), (torch.float16, True)])
def test_conv_kernel_matches_fp32_convolution(cin, cout, kernel, frames, height, width, extras, dtype, relu):
    torch.manual_seed(cin + cout)
    kt, kh, kw = kernel
    x = torch.randn(2, frames, height, width, cin, device=DEV).to(dtype)
    weight = (torch.randn(cout, cin, kt, kh, kw, device=DEV) / (cin * kt * kh * kw) ** 0.5).to(dtype)
    bias = torch.randn(cout, device=DEV).to(dtype) if extras else None
    packed = weight.permute(0, 2, 3, 4, 1).reshape(cout, -1, cin).contiguous()
    residual = torch.randn(2, frames - kt + 1, height, width, cout, device=DEV).to(dtype) if extras else None
    out = native.ext().conv3d(x, packed, bias, residual, kt, kh, kw, relu, None, False)
    _status_ok()
    want = torch.nn.functional.conv3d(x.float().permute(0, 4, 1, 2, 3), weight.float(),
                                      None if bias is None else bias.float(), padding=(0, kh // 2, kw // 2))
    want = want.permute(0, 2, 3, 4, 1)
    if residual is not None:
        want = want + residual.float()
    if relu:
        want = want.relu()
    assert out.shape == want.shape and out.dtype == dtype
    assert _rel(out, want) < 6e-3, _rel(out, want)
    assert (out.float() - want).abs().max() < 0.06


@pytest.mark.parametrize("history_frames", [0, 1, 2])
def test_causal_conv_reads_history_in_place(history_frames):
    """The causal form (zeros, then history, then the chunk, none of them joined) against the
    convolution of the joined volume."""
    torch.manual_seed(history_frames)
    cin, cout, frames, height, width = 64, 96, 3, 10, 18
    x = torch.randn(2, frames, height, width, cin, device=DEV).bfloat16()
    history = torch.randn(2, history_frames, height, width, cin, device=DEV).bfloat16() if history_frames else None
    weight = (torch.randn(cout, cin, 3, 3, 3, device=DEV) / (27 * cin) ** 0.5).bfloat16()
    packed = weight.permute(0, 2, 3, 4, 1).reshape(cout, -1, cin).contiguous()
    out = native.ext().conv3d(x, packed, None, None, 3, 3, 3, False, history, True)
    _status_ok()
    pieces = [torch.zeros(2, 2 - history_frames, height, width, cin, device=DEV).bfloat16()]
    pieces += [history] if history is not None else []
    joined = torch.cat(pieces + [x], dim=1)
    want = native.ext().conv3d(joined, packed, None, None, 3, 3, 3, False, None, False)
    assert out.shape == want.shape == (2, frames, height, width, cout)
    assert torch.equal(out, want)


def test_conv_modules_use_the_kernel_and_match():
    from agentgarten_b200.ops.conv import conv_frames, conv_volume

    torch.manual_seed(5)
    conv = torch.nn.Conv3d(64, 96, 3, padding=(0, 1, 1)).to(DEV, torch.bfloat16)
    x = torch.randn(1, 64, 5, 20, 28, device=DEV).bfloat16().contiguous(memory_format=torch.channels_last_3d)
    residual = torch.randn(1, 96, 3, 20, 28, device=DEV).bfloat16()
    before = native.launches()
    with torch.no_grad():
        got = conv_volume(conv, x, residual)
        want = conv(x).float() + residual.float()
    assert native.launches() == before + 1
    assert got.shape == want.shape and _rel(got, want) < 1e-2
    frames = torch.nn.Conv2d(32, 32, 3, padding=1).to(DEV, torch.bfloat16)
    y = torch.randn(3, 32, 18, 22, device=DEV).bfloat16()
    with torch.no_grad():
        assert _rel(conv_frames(frames, y), frames(y).float()) < 1e-2
    # output channels that are not a multiple of 8 are padded for the kernel and cut again
    odd = torch.nn.Conv2d(64, 12, 3, padding=1).to(DEV, torch.float16)
    y = torch.randn(2, 64, 16, 40, device=DEV).half()
    with torch.no_grad():
        got = conv_frames(odd, y, relu=True)
        assert got.shape == (2, 12, 16, 40) and _rel(got, odd(y).float().relu()) < 1e-2
    # a convolution that wants gradients stays on the differentiable path
    z = conv_volume(conv, x)
    assert z.requires_grad
    _status_ok()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("kernel,channels,height,width", [(7, 64, 13, 22), (7, 256, 9, 7), (3, 32, 6, 5), (5, 8, 8, 33)])
def test_depthwise_kernel_matches_fp32_convolution(dtype, kernel, channels, height, width):
    from agentgarten_b200.ops.conv import depthwise_frames

    torch.manual_seed(kernel * channels)
    conv = torch.nn.Conv2d(channels, channels, kernel, padding=kernel // 2, groups=channels,
                           bias=kernel == 3).to(DEV, dtype)
    x = torch.randn(3, channels, height, width, device=DEV).to(dtype)
    before = native.launches()
    with torch.no_grad():
        got = depthwise_frames(conv, x)
        want = torch.nn.functional.conv2d(x.float(), conv.weight.float(),
                                          None if conv.bias is None else conv.bias.float(),
                                          padding=kernel // 2, groups=channels)
    assert native.launches() == before + 1
    assert got.shape == want.shape and got.dtype == dtype
    assert _rel(got, want) < (4e-3 if dtype == torch.float16 else 8e-3), _rel(got, want)


@pytest.mark.parametrize("name", ["taew2_2", "taew2_2_super"])
def test_taehv_decoder_on_gpu_matches_cpu_fp32(name):
    from agentgarten_b200.codecs._taehv.taehv import TAEHV

    torch.manual_seed(2)
    cpu = TAEHV(checkpoint_path=None, arch_name=name).eval()
    gpu = TAEHV(checkpoint_path=None, arch_name=name).eval()
    gpu.load_state_dict(cpu.state_dict())
    gpu = gpu.to(DEV, torch.float16).to(memory_format=torch.channels_last)
    latent = torch.randn(1, 3, 48, 6, 10)
    before = native.launches()
    with torch.no_grad():
        want = cpu.decode_video(latent, parallel=True, show_progress_bar=False)
        got = gpu.decode_video(latent.to(DEV, torch.float16), parallel=True, show_progress_bar=False)
    assert native.launches() > before + 10  # the convolutions ran in the kernel
    assert got.shape == want.shape and _rel(got, want.to(DEV)) < 3e-2, _rel(got, want.to(DEV))
    _status_ok()


def test_vae_on_gpu_matches_cpu_fp32():
    from agentgarten_b200.codecs.wan22 import random_vae, to_channels_last

    arch = dict(dim=16, dec_dim=16, z_dim=8)
    cpu = random_vae(seed=3, **arch)
    gpu = to_channels_last(random_vae(seed=3, **arch).to(DEV, torch.bfloat16))
    scale = (0.0, 1.0)
    video = torch.rand(1, 3, 9, 32, 48) * 2 - 1
    before = native.launches()
    with torch.no_grad():
        want = cpu.encode(video, scale, temporal_window=4)
        got = gpu.encode(video.to(DEV, torch.bfloat16), scale, temporal_window=4)
        assert native.launches() > before  # the fused norm kernel ran
        assert _rel(got, want.to(DEV)) < 5e-2, _rel(got, want.to(DEV))
        pixels = cpu.decode(want, scale, frames_per_pass=2)
        got_pixels = gpu.decode(want.to(DEV, torch.bfloat16), scale, frames_per_pass=2)
        assert got_pixels.shape == pixels.shape and _rel(got_pixels, pixels.to(DEV)) < 8e-2


def test_silu_mul_pair():
    torch.manual_seed(0)
    both = torch.randn(37, 2 * 48, device=DEV).bfloat16()
    out = native.ext().silu_mul_pair(both)
    want = ops.silu_mul(both[:, :48].contiguous(), both[:, 48:].contiguous())
    assert torch.equal(out, want)


def test_head_norm_rope_reads_a_column_block_in_place():
    torch.manual_seed(0)
    rows, heads = 70, 3
    wide = torch.randn(rows, (heads + 2) * 128, device=DEV).bfloat16()
    weight = (torch.rand(128, device=DEV) + 0.5).bfloat16()
    cos = torch.randn(1, rows, 128, device=DEV).bfloat16()
    sin = torch.randn(1, rows, 128, device=DEV).bfloat16()
    block = wide[:, 128:128 + heads * 128].view(1, rows, heads, 128)
    assert not block.is_contiguous()
    out, _ = native.ext().head_norm_rope_fwd(block, weight, cos, sin, 1e-6)
    want, _ = native.ext().head_norm_rope_fwd(block.contiguous(), weight, cos, sin, 1e-6)
    assert out.is_contiguous() and torch.equal(out, want)


@pytest.mark.parametrize("hq,hkv", [(3, 3), (6, 2), (2, 1)])
def test_attention_forward_backward_with_odd_and_even_head_groups(hq, hkv, backward_form):
    """An odd number of query heads per KV head runs one head per forward CTA, an even one two."""
    torch.manual_seed(hq * 10 + hkv)
    q = torch.randn(2, 200, hq, 128, device=DEV).bfloat16().requires_grad_()
    k = torch.randn(2, 330, hkv, 128, device=DEV).bfloat16().requires_grad_()
    v = torch.randn(2, 330, hkv, 128, device=DEV).bfloat16().requires_grad_()
    out = ops.attention(q, k, v)
    grad = torch.randn_like(out)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), grad)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    want = reference.attention(qf, kf, vf, None)
    wq, wk, wv = torch.autograd.grad(want, (qf, kf, vf), grad.float())
    assert _rel(out, want) < 1e-2
    assert _rel(dq, wq) < 2e-2 and _rel(dk, wk) < 2e-2 and _rel(dv, wv) < 2e-2
    _status_ok()


def test_adaln_kernels_match_the_eager_sequence():
    """norm + modulate and the gated residual read their terms in place from the six-way
    modulation projection and reproduce the operator-by-operator bf16 result."""
    torch.manual_seed(4)
    rows, width = 77, 512
    x = torch.randn(2, rows, width, device=DEV).bfloat16()
    y = torch.randn(2, rows, width, device=DEV).bfloat16()
    weight = (torch.rand(width, device=DEV) + 0.5).bfloat16()
    terms = (0.3 * torch.randn(2, rows, 6 * width, device=DEV)).bfloat16().chunk(6, dim=-1)
    shift, scale, gate = terms[0], terms[1], terms[2]
    before = native.launches()
    with torch.no_grad():
        got = ops.norm_modulate(x, weight, scale, shift, 1e-6)
        want = ops.rms_norm(x, weight, 1e-6) * (1 + scale) + shift
        assert native.launches() >= before + 2
        assert (got.float() - want.float()).abs().max() <= 2e-2 and _rel(got, want) < 3e-3
        fp32 = reference.rms_norm(x.float(), weight.float(), 1e-6) * (1 + scale.float()) + shift.float()
        assert _rel(got, fp32) < 8e-3
        mixed = ops.gated_residual(x, gate, y)
        assert torch.equal(mixed, x + gate * y)
    # with gradients wanted the differentiable path runs
    xg = x.clone().requires_grad_()
    assert ops.norm_modulate(xg, weight, scale, shift, 1e-6).requires_grad


def test_geometry_kernels_match_the_operator_sequence(monkeypatch):
    from agentgarten_b200.networks.cosmos3 import geometry

    torch.manual_seed(9)
    depth = torch.rand(2, 1, 3, 17, 23, device=DEV) * 30
    depth[0, 0, 0, :3] = 0.0
    depth[1, 0, 1, 5, :4] = float("nan")
    depth[1, 0, 2, 7, :4] = float("inf")
    scale = torch.tensor([0.7, 1.9], device=DEV)
    normal = torch.randint(0, 256, (2, 3, 3, 17, 23), device=DEV, dtype=torch.uint8)
    normal[0, :, 0, 0, :5] = 127  # (almost) zero vectors stay finite
    before = native.launches()
    got_rgb, got_n = geometry.colorize_depth(depth, scale), geometry.prepare_normal(normal)
    assert native.launches() == before + 2
    monkeypatch.setattr(geometry, "_fused_kernels", lambda tensor: None)
    want_rgb, want_n = geometry.colorize_depth(depth, scale), geometry.prepare_normal(normal)
    assert got_rgb.shape == want_rgb.shape and (got_rgb - want_rgb).abs().max() < 1e-5
    assert got_n.shape == want_n.shape and (got_n - want_n).abs().max() < 1e-5
    single = geometry.colorize_depth(depth, scale[:1])
    monkeypatch.undo()
    assert (single - geometry.colorize_depth(depth, scale[:1])).abs().max() < 1e-5


def test_rope_table_kernel_matches_the_definition():
    """cos / sin tables from one kernel against the PyTorch definition (FP32 angle, then cosine
    and sine): equal after rounding to bf16 except where the FP32 results differ in the last
    place and straddle a bf16 boundary; FP32 tables within 2e-7."""
    from agentgarten_b200.networks.cosmos3 import Cosmos3Config
    from agentgarten_b200.networks.cosmos3.layers import Cosmos3RotaryEmbedding

    rope = Cosmos3RotaryEmbedding(Cosmos3Config(num_hidden_layers=1))
    g = torch.Generator(device=DEV).manual_seed(2)
    positions = torch.rand(2, 777, 3, device=DEV, generator=g) * 600
    before = native.launches()
    cos32, sin32 = rope(positions, torch.float32)
    cos16, sin16 = rope(positions, torch.bfloat16)
    assert native.launches() == before + 2
    angle = rope.angles(positions)
    full = torch.cat((angle, angle), dim=-1)
    assert (cos32 - full.cos()).abs().max() < 2e-7 and (sin32 - full.sin()).abs().max() < 2e-7
    for got, want in ((cos16, full.cos().bfloat16()), (sin16, full.sin().bfloat16())):
        assert got.shape == want.shape and (got != want).float().mean() < 1e-3
        assert (got.float() - want.float()).abs().max() < 1e-2


@pytest.mark.parametrize("src,dst", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32),
                                     (torch.float32, torch.float32)])
def test_patch_layout_kernels_match_the_rearrangement(src, dst):
    from einops import rearrange

    from agentgarten_b200.networks.cosmos3.network import patchify, unpatchify

    g = torch.Generator(device=DEV).manual_seed(3)
    latent = torch.randn(2, 12, 3, 6, 10, device=DEV, generator=g).to(src).requires_grad_()
    before = native.launches()
    patches = patchify(latent, 2, dst)
    assert native.launches() == before + 1
    want = rearrange(latent.detach().to(dst), "b c t (h p) (w q) -> b t (h w) (p q c)", p=2, q=2)
    assert patches.dtype == dst and torch.equal(patches, want)
    grad = torch.randn(patches.shape, device=DEV, generator=g).to(dst)
    patches.backward(grad)
    back = rearrange(grad.to(src), "b t (h w) (p q c) -> b c t (h p) (w q)", h=3, w=5, p=2, q=2, c=12)
    assert torch.equal(latent.grad, back)
    again = unpatchify(patches.detach(), channels=12, grid=(3, 5), patch_size=2, dtype=src)
    assert torch.equal(again, latent.detach().to(dst).to(src))


def test_geometry_pool_blur_and_warp_kernels_match_the_library_formulation(monkeypatch):
    """The three frame kernels against avg_pool2d / padded depthwise conv2d / grid_sample: the
    same functions of ``networks/cosmos3/geometry.py`` run once on the kernels and once with them
    switched off, with the same random draws."""
    from agentgarten_b200.networks.cosmos3 import geometry

    g = torch.Generator(device=DEV).manual_seed(11)
    depth = torch.randn(2, 3, 5, 36, 52, device=DEV, generator=g)
    depth[0, 0, 0, 0, 0] = float("nan")
    depth[1, 2, 3, 5, 7] = float("inf")
    normal = torch.randn(2, 3, 5, 36, 52, device=DEV, generator=g)
    config = geometry.GeometryAugmentationConfig(spatial_probability=1.0, spatial_max_scale=1.3,
                                                 spatial_max_shift_fraction=0.1, spatial_max_shear=0.1,
                                                 spatial_max_perspective=0.1)

    def run():
        torch.manual_seed(5)
        pooled = geometry.downsample_geometry({"depth": depth, "normal": normal}, factor=4)
        blurred = geometry._gaussian(normal[0].permute(1, 0, 2, 3).contiguous(), 1.7)
        warped = geometry._warp_from_first_frame({"depth": normal, "normal": normal * 2}, config=config)
        return pooled, blurred, warped

    before = native.launches()
    mine = run()
    assert native.launches() >= before + 4
    monkeypatch.setattr(geometry, "_fused_kernels", lambda tensor: None)
    want = run()
    for name in ("depth", "normal"):
        assert mine[0][name].shape == want[0][name].shape
        assert torch.allclose(mine[0][name], want[0][name], atol=1e-5)
        assert torch.allclose(mine[2][name], want[2][name], atol=2e-4), float((mine[2][name] - want[2][name]).abs().max())
        assert torch.equal(mine[2][name][:, :, -1], want[2][name][:, :, -1])   # the last frame is untouched
    assert torch.allclose(mine[1], want[1], atol=1e-5)


def test_geometry_resize_and_stretch_kernels_match_the_library_formulation(monkeypatch):
    """Texture suppression (area down, bilinear up) and the quadrant stretch against
    ``F.interpolate``: the same functions of ``networks/cosmos3/geometry.py`` with the kernels on
    and off, with the same random draws; extents that divide neither way."""
    from agentgarten_b200.networks.cosmos3 import geometry

    g = torch.Generator(device=DEV).manual_seed(13)
    depth = torch.randn(3, 3, 4, 37, 53, device=DEV, generator=g)
    normal = torch.randn(3, 3, 4, 37, 53, device=DEV, generator=g)
    config = geometry.GeometryAugmentationConfig(texture_suppression_probability=1.0,
                                                 texture_downsample_min=1.5, texture_downsample_max=3.7)

    def run(training):
        torch.manual_seed(9)
        smooth = geometry._suppress_texture({"depth": depth, "normal": normal}, data_batch={}, config=config)
        grown = geometry.stretch_geometry({"depth": depth, "normal": normal}, training=training, divisor=16)
        return smooth, grown

    for training in (True, False):
        with monkeypatch.context() as patch:
            before = native.launches()
            mine = run(training)
            assert native.launches() >= before + 3 * 2 + 1   # per sample the blur and the resizes; one stretch
            patch.setattr(geometry, "_fused_kernels", lambda tensor: None)
            want = run(training)
        for name in ("depth", "normal"):
            assert mine[1][name].shape == want[1][name].shape == (3, 3, 4, 48, 64)
            for part in (0, 1):
                error = float((mine[part][name] - want[part][name]).abs().max())
                assert error < 2e-5, (training, part, name, error)


def test_dmd_target_kernel_matches_the_fp64_expression():
    """Target and step size of the distribution-matching loss: two launches against the chain of
    FP64 tensor expressions, one sample with a spread below the floor."""
    g = torch.Generator(device=DEV).manual_seed(17)
    estimate = torch.randn(3, 16, 5, 12, 20, device=DEV, generator=g)
    fake = estimate + 0.3 * torch.randn(estimate.shape, device=DEV, generator=g)
    teacher = estimate + 0.2 * torch.randn(estimate.shape, device=DEV, generator=g)
    teacher[2] = estimate[2] + 1e-7          # spread clamps to 1e-5
    before = native.launches()
    with torch.no_grad():
        target, rms = ops.dmd_target(estimate, fake, teacher)
    assert native.launches() == before + 2 and target.dtype == torch.float64
    wide, far = estimate.double(), teacher.double()
    spread = (wide - far).abs().flatten(1).mean(1).clamp_min(1e-5)
    step = (fake.double() - far) / spread.view(-1, 1, 1, 1, 1)
    assert torch.allclose(target, wide - step, rtol=1e-12, atol=1e-12)
    assert float(rms) == pytest.approx(float(step.float().square().mean().sqrt()), rel=1e-5)
    again, _ = ops.dmd_target(estimate, fake, teacher)   # gradients on: the tensor expressions
    assert torch.allclose(again, target, rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rows_linear_matches_fp32_linear_and_its_gradients(dtype):
    """The timestep embedder's FP32 linears on their own kernels: values and all three gradients
    against ``F.linear`` on the upcast weights."""
    g = torch.Generator(device=DEV).manual_seed(6)
    x = torch.randn(13, 256, device=DEV, generator=g, requires_grad=True)
    w = (torch.randn(384, 256, device=DEV, generator=g) * 0.1).to(dtype).requires_grad_()
    b = torch.randn(384, device=DEV, generator=g).to(dtype).requires_grad_()
    before = native.launches()
    y = ops.rows_linear(x, w, b)
    grad = torch.randn(y.shape, device=DEV, generator=g)
    y.backward(grad)
    assert native.launches() == before + 3 and y.dtype == torch.float32
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    want = torch.nn.functional.linear(xr, wr, br)
    want.backward(grad)
    assert torch.allclose(y, want, atol=1e-4, rtol=1e-5)
    assert torch.allclose(x.grad, xr.grad, atol=1e-4, rtol=1e-5)
    tolerance = 1e-4 if dtype == torch.float32 else 4e-2
    assert torch.allclose(w.grad.float(), wr.grad, atol=tolerance, rtol=1e-2)
    assert torch.allclose(b.grad.float(), br.grad, atol=tolerance, rtol=1e-2)
