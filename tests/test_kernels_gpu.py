"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ext():
    from visionrl_b200.ops import _ext

    return _ext.load()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


# ---------------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (1000, 1536, 1536),
                                   (77, 264, 200), (4096, 6144, 1536), (16, 9216, 1536)])
def test_gemm_nt_matches_fp32(ext, m, n, k):
    torch.manual_seed(0)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    out = ext.gemm_bf16(a, b, None, None, None, 0, 0, False, False, False)
    assert ext.gemm_last_status() == 0
    ref = a.float() @ b.float().t()
    assert _rel(out, ref) < 5e-3


def test_gemm_fp32_output_and_epilogues(ext):
    torch.manual_seed(1)
    bsz, s, k, n = 3, 160, 512, 768
    a = torch.randn(bsz * s, k, device="cuda", dtype=torch.bfloat16) * 0.5
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    gate = torch.randn(bsz, n, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(bsz * s, n, device="cuda", dtype=torch.bfloat16)
    base = a.float() @ w.float().t() + bias.float()
    out32 = ext.gemm_bf16(a, w, bias, None, None, 0, 0, False, False, True)
    assert out32.dtype == torch.float32 and _rel(out32, base) < 2e-3
    gelu = ext.gemm_bf16(a, w, bias, None, None, 1, 0, False, False, False)
    assert _rel(gelu, torch.nn.functional.gelu(base, approximate="tanh")) < 1e-2
    silu = ext.gemm_bf16(a, w, bias, None, None, 2, 0, False, False, False)
    assert _rel(silu, torch.nn.functional.silu(base)) < 1e-2
    gated = ext.gemm_bf16(a, w, bias, gate, res, 0, s, False, False, False)
    ref = res.float() + gate.float().repeat_interleave(s, 0) * base
    assert _rel(gated, ref) < 1e-2
    assert ext.gemm_last_status() == 0


@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (1184, 1536, 4608), (296, 520, 136)])
def test_gemm_transposed_operands(ext, m, n, k):
    """dX = dY @ W (B stored [K, N]) and dW = dY^T @ X (both operands stored [K, *])."""
    torch.manual_seed(2)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b_kn = torch.randn(k, n, device="cuda", dtype=torch.bfloat16)
    out = ext.gemm_bf16(a, b_kn, None, None, None, 0, 0, False, True, False)
    assert _rel(out, a.float() @ b_kn.float()) < 5e-3
    a_km = torch.randn(k, m, device="cuda", dtype=torch.bfloat16)
    out2 = ext.gemm_bf16(a_km, b_kn, None, None, None, 0, 0, True, True, False)
    assert _rel(out2, a_km.float().t() @ b_kn.float()) < 5e-3
    assert ext.gemm_last_status() == 0


def test_gemm_rejects_unaligned_pitch(ext):
    a = torch.randn(64, 300, device="cuda", dtype=torch.bfloat16)      # stored [K, M], M % 8 != 0
    b = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="pitch"):
        ext.gemm_bf16(a, b, None, None, None, 0, 0, True, True, False)
    ok = ext.gemm_bf16(a[:, :296].contiguous(), b, None, None, None, 0, 0, True, True, False)
    assert ok.shape == (296, 256)


def test_linear_autograd_matches_fp32():
    from visionrl_b200.ops.linear import linear

    torch.manual_seed(3)
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(512, 256, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_()
    b = torch.randn(512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf, bf = (t.detach().float().requires_grad_() for t in (x, w, b))
    yf = torch.nn.functional.linear(xf, wf, bf)
    yf.backward(g.float())
    assert _rel(y, yf) < 5e-3 and _rel(x.grad, xf.grad) < 1e-2
    assert _rel(w.grad, wf.grad) < 1e-2 and _rel(b.grad, bf.grad) < 1e-2


# ------------------------------------------------------------------------------ SDE step
@pytest.mark.parametrize("gaussian", [True, False])
@pytest.mark.parametrize("shape", [(3, 16, 64, 64), (2, 16, 3, 20, 28), (5, 7)])
def test_sde_step_matches_reference(ext, gaussian, shape):
    from visionrl_b200.ops.sde import sde_step, sde_step_reference

    torch.manual_seed(4)
    b = shape[0]
    v, x, noise = (torch.randn(shape, device="cuda") for _ in range(3))
    a = 1 + 0.1 * torch.randn(b, device="cuda")
    bb = -0.1 + 0.02 * torch.randn(b, device="cuda")
    scale = 0.05 + 0.1 * torch.rand(b, device="cuda")
    dt = -0.1 * torch.ones(b, device="cuda")
    got = sde_step(v, x, a, bb, scale, dt, noise=noise, gaussian=gaussian)
    ref = sde_step_reference(v, x, a, bb, scale, dt, noise=noise, gaussian=gaussian)
    for g, r in zip(got, ref):
        assert torch.allclose(g, r, rtol=2e-4, atol=2e-4)
    # replay with the recorded sample reproduces the rollout log-prob bit for bit
    again = sde_step(v, x, a, bb, scale, dt, prev_sample=got[0], gaussian=gaussian)
    assert torch.equal(again[1], got[1])
    det = sde_step(v, x, a, bb, scale, dt, noise=noise, deterministic=True, gaussian=gaussian)
    assert torch.allclose(det[0], x + dt.view(-1, *([1] * (len(shape) - 1))) * v, atol=1e-5)


def test_sde_step_backward(ext):
    from visionrl_b200.ops.sde import sde_step, sde_step_reference

    torch.manual_seed(5)
    shape = (3, 4, 8, 8)
    x, prev = torch.randn(shape, device="cuda"), torch.randn(shape, device="cuda")
    a = torch.full((3,), 0.97, device="cuda")
    b = torch.full((3,), -0.08, device="cuda")
    scale = torch.full((3,), 0.2, device="cuda")
    dt = torch.full((3,), -0.1, device="cuda")
    w_lp, w_mu = torch.randn(3, device="cuda"), torch.randn(shape, device="cuda")
    grads = []
    for fn in (sde_step, sde_step_reference):
        v = torch.randn(shape, device="cuda", generator=torch.Generator("cuda").manual_seed(9),
                        requires_grad=True)
        _, lp, mu = fn(v, x, a, b, scale, dt, prev_sample=prev)
        ((lp * w_lp).sum() + (mu * w_mu).sum()).backward()
        grads.append(v.grad)
    assert torch.allclose(grads[0], grads[1], rtol=1e-4, atol=1e-5)


# --------------------------------------------------------------------------------- losses
def test_token_loss_matches_reference(ext):
    from visionrl_b200.ops.losses import token_grpo_loss, token_grpo_loss_reference

    torch.manual_seed(6)
    bsz, length = 6, 97
    old = torch.randn(bsz, length, device="cuda") * 0.1
    ref = old + 0.05 * torch.randn_like(old)
    adv = torch.randn(bsz, device="cuda")
    mask = (torch.rand(bsz, length, device="cuda") > 0.2).float()
    for kl in ("k3", "k1"):
        outs = []
        for fn in (token_grpo_loss, token_grpo_loss_reference):
            lp = (old + 0.02 * torch.randn(bsz, length, device="cuda",
                                           generator=torch.Generator("cuda").manual_seed(1))
                  ).requires_grad_()
            pol, klv, clip, akl = fn(lp, old, adv, mask, ref, 0.01, kl)
            (pol + 0.3 * klv).backward()
            outs.append((pol, klv, clip, akl, lp.grad))
        for g, r in zip(*outs):
            assert torch.allclose(g, r, rtol=1e-4, atol=1e-6)


def test_grpo_sample_loss_matches_reference(ext):
    from visionrl_b200.ops.losses import grpo_clipped_loss, grpo_clipped_loss_reference

    torch.manual_seed(7)
    old = torch.randn(16, device="cuda")
    adv = torch.randn(16, device="cuda")
    res = []
    for fn in (grpo_clipped_loss, grpo_clipped_loss_reference):
        lp = (old + 1e-4 * torch.arange(16, device="cuda").float() - 5e-4).requires_grad_()
        loss, clip, akl = fn(lp, old, adv, 1e-4)
        loss.backward()
        res.append((loss, clip, akl, lp.grad))
    for g, r in zip(*res):
        assert torch.allclose(g, r, rtol=1e-4, atol=1e-7)


def test_per_sample_mse_and_sum_squares(ext):
    torch.manual_seed(8)
    for dtype in (torch.float32, torch.bfloat16):
        p = torch.randn(5, 16, 9, 20, 26, device="cuda", dtype=dtype)
        t = torch.randn_like(p)
        got = ext.per_sample_mse(p, t)
        ref = (p.float() - t.float()).pow(2).mean(dim=(1, 2, 3, 4))
        assert torch.allclose(got, ref, rtol=1e-4)
        flat = torch.randn(1_000_003 if dtype == torch.float32 else 1_000_008, device="cuda",
                           dtype=dtype)
        assert torch.allclose(ext.sum_squares(flat), flat.float().pow(2).sum(), rtol=1e-4)


def test_fused_adamw_matches_torch(ext):
    import copy

    from visionrl_b200.ops.optim import FusedAdamW

    torch.manual_seed(9)
    net = torch.nn.Sequential(torch.nn.Linear(64, 96), torch.nn.Linear(96, 32)).cuda()
    ref = copy.deepcopy(net)
    ours = FusedAdamW(net.parameters(), lr=1e-2, weight_decay=0.05)
    theirs = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.05)
    for _ in range(5):
        x = torch.randn(8, 64, device="cuda")
        for m, o in ((net, ours), (ref, theirs)):
            o.zero_grad()
            m(x).pow(2).mean().backward()
            o.step()
    for a, b in zip(net.parameters(), ref.parameters()):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-6)
    assert torch.allclose(ours.grad_norm(), torch.sqrt(sum(p.grad.pow(2).sum()
                                                         for p in net.parameters())), rtol=1e-4)


# ---------------------------------------------------------------------------------- norms
@pytest.mark.parametrize("d", [64, 1536, 5120])
def test_adaln_forward_backward(ext, d):
    from visionrl_b200.ops.norm import adaln_layernorm, adaln_layernorm_reference

    torch.manual_seed(10)
    b, s = 2, 37
    res = []
    for fn in (adaln_layernorm, adaln_layernorm_reference):
        gen = torch.Generator("cuda").manual_seed(3)
        x = torch.randn(b, s, d, device="cuda", generator=gen).bfloat16().requires_grad_()
        sh = (0.1 * torch.randn(b, d, device="cuda", generator=gen)).bfloat16().requires_grad_()
        sc = (0.1 * torch.randn(b, d, device="cuda", generator=gen)).bfloat16().requires_grad_()
        y = fn(x, sh, sc)
        y.backward(torch.randn(y.shape, device="cuda", generator=gen).bfloat16())
        res.append((y, x.grad, sh.grad, sc.grad))
    for g, r in zip(*res):
        assert _rel(g, r) < 2e-2


@pytest.mark.parametrize("d", [128, 2048])
def test_rmsnorm_forward_backward(ext, d):
    from visionrl_b200.ops.norm import rmsnorm, rmsnorm_reference

    res = []
    for fn in (rmsnorm, rmsnorm_reference):
        gen = torch.Generator("cuda").manual_seed(4)
        x = torch.randn(3, 19, d, device="cuda", generator=gen).bfloat16().requires_grad_()
        w = (1 + 0.1 * torch.randn(d, device="cuda", generator=gen)).bfloat16().requires_grad_()
        y = fn(x, w)
        y.backward(torch.randn(y.shape, device="cuda", generator=gen).bfloat16())
        res.append((y, x.grad, w.grad))
    for g, r in zip(*res):
        assert _rel(g, r) < 2e-2


@pytest.mark.parametrize("heads,dh,across,use_rope", [(24, 64, False, False), (12, 128, True, True),
                                                      (4, 64, False, True), (40, 128, True, True)])
def test_qkv_prepare_forward_backward(ext, heads, dh, across, use_rope):
    from visionrl_b200.ops.qkv import qkv_prepare, qkv_prepare_reference

    b, s, d = 2, 21, heads * dh
    wn = d if across else dh
    rope = None
    if use_rope:
        ang = torch.rand(s, dh // 2, device="cuda") * 6.28
        rope = (torch.cos(ang), torch.sin(ang))
    res = []
    for fn in (qkv_prepare, qkv_prepare_reference):
        gen = torch.Generator("cuda").manual_seed(5)
        qkv = torch.randn(b, s, 3 * d, device="cuda", generator=gen).bfloat16().requires_grad_()
        qw = (1 + 0.1 * torch.randn(wn, device="cuda", generator=gen)).bfloat16().requires_grad_()
        kw = (1 + 0.1 * torch.randn(wn, device="cuda", generator=gen)).bfloat16().requires_grad_()
        q, k, v = fn(qkv, heads, qw, kw, rope=rope)
        gq, gk, gv = (torch.randn(q.shape, device="cuda", generator=gen).bfloat16() for _ in range(3))
        torch.autograd.backward([q, k, v], [gq, gk, gv])
        res.append((q, k, v, qkv.grad, qw.grad, kw.grad))
    for g, r in zip(*res):
        assert _rel(g, r) < 3e-2


# ------------------------------------------------------------------------- model-level parity
def test_mmdit_forward_backward_kernels_vs_torch_ops():
    from visionrl_b200.models.nn.mmdit import MMDiT, MMDiTConfig
    from visionrl_b200.ops import _ext

    torch.manual_seed(11)
    cfg = MMDiTConfig(num_layers=2, hidden_size=256, num_heads=4, in_channels=16, context_dim=128,
                      pooled_dim=64, max_grid=32)
    net = MMDiT(cfg).cuda().bfloat16()
    lat = torch.randn(2, 16, 16, 16, device="cuda")
    t = torch.tensor([800.0, 300.0], device="cuda")
    ctx = torch.randn(2, 24, 128, device="cuda")
    pooled = torch.randn(2, 64, device="cuda")
    outs = []
    for flag in (True, False):
        _ext.set_kernels_enabled(flag)
        try:
            net.zero_grad()
            y = net(lat, t, ctx, pooled)
            y.float().pow(2).mean().backward()
            outs.append((y.detach().clone(), net.blocks[0].attn_x.qkv.weight.grad.clone()))
        finally:
            _ext.set_kernels_enabled(True)
    assert _rel(outs[0][0], outs[1][0]) < 3e-2
    assert _rel(outs[0][1], outs[1][1]) < 6e-2
    assert _ext.load().gemm_last_status() == 0


@pytest.mark.gpu
def test_colsum_matches_fp32():
    from visionrl_b200.ops import _ext

    x = torch.randn(4712, 1536, device="cuda", dtype=torch.bfloat16)
    got = _ext.load().colsum(x)
    ref = x.float().sum(0)
    assert torch.allclose(got, ref, atol=2e-2, rtol=1e-3)
    x = torch.randn(37, 72, device="cuda", dtype=torch.bfloat16)
    assert torch.allclose(_ext.load().colsum(x), x.float().sum(0), atol=1e-3, rtol=1e-3)


@pytest.mark.gpu
def test_adaln_accepts_strided_modulation_views():
    from visionrl_b200.ops.norm import adaln_layernorm

    b, s, d = 3, 77, 256
    x = torch.randn(b, s, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    mod = torch.randn(b, 6 * d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    shift, scale = mod[:, d:2 * d], mod[:, 3 * d:4 * d]
    y = adaln_layernorm(x, shift, scale, 1e-6)
    xf, mf = x.detach().float().requires_grad_(), mod.detach().float().requires_grad_()
    ref = torch.nn.functional.layer_norm(xf, (d,), eps=1e-6) * (1 + mf[:, None, 3 * d:4 * d]) \
        + mf[:, None, d:2 * d]
    assert torch.allclose(y.float(), ref, atol=3e-2, rtol=3e-2)
    g = torch.randn_like(y)
    y.backward(g)
    ref.backward(g.float())
    assert torch.allclose(x.grad.float(), xf.grad, atol=5e-2, rtol=5e-2)
    assert torch.allclose(mod.grad.float(), mf.grad, atol=0.15, rtol=5e-2)


# ----------------------------------------------------------------------------- AR-path kernels
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_token_logprob_fwd_bwd(dtype):
    from visionrl_b200.ops.logprob import token_log_probs, token_log_probs_reference

    torch.manual_seed(0)
    logits = (torch.randn(37, 16384, device="cuda") * 3).to(dtype).requires_grad_()
    ids = torch.randint(0, 16384, (37,), device="cuda")
    lp = token_log_probs(logits, ids, 0.7)
    ref_in = logits.detach().float().requires_grad_()
    ref = token_log_probs_reference(ref_in, ids, 0.7)
    assert torch.allclose(lp, ref, atol=2e-4, rtol=1e-4)
    g = torch.randn_like(lp)
    lp.backward(g)
    ref.backward(g)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert torch.allclose(logits.grad.float(), ref_in.grad, atol=tol, rtol=tol)


@pytest.mark.gpu
@pytest.mark.parametrize("form,rows,vocab,temp", [
    ("epilogue", 300, 4096 + 1024, 1.0),
    ("epilogue", 37, 2048 + 8 * 13, 0.7),        # row tail, vocabulary not a multiple of 64
    ("chunked", 300, 4096 + 1024, 1.0),
])
def test_fused_head_log_probs_matches_reference(monkeypatch, form, rows, vocab, temp):
    from visionrl_b200.ops import logprob as LP
    from visionrl_b200.ops.logprob import fused_head_log_probs, fused_head_log_probs_reference

    monkeypatch.setattr(LP, "_CHUNKED_FOLD", form == "chunked")
    torch.manual_seed(1)
    hid = 256
    h = (torch.randn(rows, hid, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(vocab, hid, device="cuda") * 0.05).bfloat16().requires_grad_()
    b = (torch.randn(vocab, device="cuda") * 0.1).bfloat16().requires_grad_()
    ids = torch.randint(0, vocab, (rows,), device="cuda")
    ids[0], ids[-1] = 0, vocab - 1                  # first and last column as targets
    lp = fused_head_log_probs(h, w, b, ids, temp, chunk=2048)
    hf, wf, bf = (t.detach().float().requires_grad_() for t in (h, w, b))
    ref = fused_head_log_probs_reference(hf, wf, bf, ids, temp)
    assert torch.allclose(lp, ref, atol=5e-3, rtol=1e-3)
    g = torch.randn_like(lp)
    lp.backward(g)
    ref.backward(g)
    assert torch.allclose(h.grad.float(), hf.grad, atol=2e-2, rtol=5e-2)
    assert torch.allclose(w.grad.float(), wf.grad, atol=2e-2, rtol=5e-2)
    assert torch.allclose(b.grad.float(), bf.grad, atol=2e-2, rtol=5e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_sample_tokens_inverse_cdf(dtype):
    from visionrl_b200.ops.sampling import sample_cfg_tokens

    torch.manual_seed(2)
    rows, vocab, w, t = 32, 16384, 5.0, 0.9
    cond = (torch.randn(rows, vocab, device="cuda") * 2).to(dtype)
    uncond = (torch.randn(rows, vocab, device="cuda") * 2).to(dtype)
    u = torch.rand(rows, device="cuda")
    tokens, logp = sample_cfg_tokens(cond, uncond, u, w, t)
    tokens2, logp2 = sample_cfg_tokens(cond, uncond, u, w, t)
    assert torch.equal(tokens, tokens2) and torch.equal(logp, logp2)
    guided = uncond.double() + w * (cond.double() - uncond.double())
    cdf = torch.softmax(guided / t, dim=-1).cumsum(-1)
    hi = cdf.gather(-1, tokens[:, None])[:, 0]
    lo = torch.where(tokens > 0, cdf.gather(-1, (tokens - 1).clamp_min(0)[:, None])[:, 0],
                     torch.zeros_like(hi))
    target = u.double()
    assert bool(((target >= lo - 1e-4) & (target <= hi + 1e-4)).all())
    ref_lp = torch.log_softmax(cond.float() / t, dim=-1).gather(-1, tokens[:, None])[:, 0]
    assert torch.allclose(logp, ref_lp, atol=2e-4, rtol=1e-4)


@pytest.mark.gpu
def test_decode_attention_matches_reference():
    from visionrl_b200.ops.attention import decode_attention, decode_attention_reference

    torch.manual_seed(3)
    rows, heads, max_len, d, length = 6, 16, 96, 128, 77
    cache = torch.randn(2, rows, heads, max_len, d, device="cuda").bfloat16()
    q = torch.randn(rows, heads, 1, d, device="cuda").bfloat16()
    valid = torch.rand(rows, max_len, device="cuda") > 0.2
    valid[:, 0] = True
    got = decode_attention(q, cache[0], cache[1], valid, length)
    ref = decode_attention_reference(q.float(), cache[0].float(), cache[1].float(), valid, length)
    assert torch.allclose(got.float(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("global_std", [False, True])
def test_group_advantages_kernel(global_std):
    from visionrl_b200.algorithms.grpo import (group_normalized_advantages,
                                                group_normalized_advantages_reference)

    torch.manual_seed(4)
    rewards = torch.randn(67, device="cuda")
    gids = torch.randint(0, 9, (67,), device="cuda") * 7 + 3
    gids[-1] = 1000          # singleton group
    got = group_normalized_advantages(rewards, gids, 1e-8, 5.0, global_std)
    ref = group_normalized_advantages_reference(rewards.cpu(), gids.cpu(), 1e-8, 5.0, global_std)
    assert torch.allclose(got.cpu(), ref, atol=1e-5, rtol=1e-5)
    assert got[-1].item() == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("m", [1, 16, 32])
def test_int4_gemv_matches_dequantised_matmul(m):
    from visionrl_b200.ops.quant import int4_linear, int4_linear_reference, quantize_int4

    torch.manual_seed(5)
    n, k = 2048 + 24, 2048
    w = torch.randn(n, k, device="cuda") * 0.05
    packed, scales = quantize_int4(w)
    x = torch.randn(m, k, device="cuda").bfloat16()
    bias = torch.randn(n, device="cuda").bfloat16()
    got = int4_linear(x, packed, scales, bias)
    ref = int4_linear_reference(x.float(), packed, scales, bias)
    assert torch.allclose(got.float(), ref, atol=3e-2, rtol=2e-2)


@pytest.mark.gpu
def test_moe_routing_kernels_and_block():
    from visionrl_b200.ops import moe

    torch.manual_seed(6)
    tokens, experts, k, dim = 1000, 8, 2, 256
    logits = torch.randn(tokens, experts, device="cuda")
    w, idx = moe.route(logits, k)
    rw, ridx = moe.route_reference(logits, k)
    assert torch.equal(idx, ridx) and torch.allclose(w, rw, atol=1e-5)
    perm, inv, offsets = moe.permute(idx, experts)
    rperm, rinv, roff = moe.permute_reference(idx, experts)
    assert torch.equal(perm, rperm) and torch.equal(inv, rinv) and torch.equal(offsets, roff)
    block = moe.MoEFFN(dim, 512, experts, k).cuda().bfloat16()
    x = torch.randn(4, 250, dim, device="cuda").bfloat16()
    with torch.no_grad():
        got = block(x)
        ref = moe.moe_ffn_reference(block, x)
    assert torch.allclose(got.float(), ref.float(), atol=6e-2, rtol=6e-2)
    xg = x.clone().requires_grad_()
    block(xg).float().pow(2).mean().backward()
    assert xg.grad is not None and torch.isfinite(xg.grad.float()).all()
    assert block.w1.grad is not None and block.gate.weight.grad is not None


@pytest.mark.gpu
def test_moe_grouped_path_matches_fp32_oracle_forward_and_backward():
    """Padded permutation + grouped tcgen05 products (device-scheduled, one launch per layer) against
    the dense fp32 per-expert loop, gradients of inputs, expert weights, biases and the gate included;
    one expert receives no token at all, and the token count is not a multiple of the tile height."""
    import copy

    from visionrl_b200.ops import moe

    torch.manual_seed(16)
    tokens, experts, k, dim, hidden = 777, 6, 2, 128, 320
    logits = torch.randn(tokens, experts, device="cuda")
    logits[:, 4] = -50.0                                  # expert 4 is never chosen
    _, idx = moe.route(logits, k)
    got = moe.permute_padded(idx, experts)
    want = moe.permute_padded_reference(idx, experts)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert int(got[2][5] - got[2][4]) == 0                # the empty expert owns no tile

    block = moe.MoEFFN(dim, hidden, experts, k).cuda().bfloat16()
    with torch.no_grad():
        block.gate.weight[4].fill_(0.0)
        block.gate.weight.mul_(4.0)
        block.b1.normal_(std=0.1)
        block.b2.normal_(std=0.1)
    x = (torch.randn(3, 259, dim, device="cuda") * 0.7).bfloat16()
    x[..., 0] = 1.0
    with torch.no_grad():
        block.gate.weight[4, 0] = -50.0                   # ... so expert 4 is never routed to here either
    assert block._grouped_ok(x.reshape(-1, dim))
    ref_block = copy.deepcopy(block).float()
    xa = x.clone().requires_grad_()
    xb = x.float().clone().requires_grad_()
    ya = block(xa)
    tokens_f = xb.reshape(-1, dim)
    with torch.no_grad():                                 # the oracle follows the block's own routing choice
        _, ex = moe.route(block.gate(x.reshape(-1, dim)), k)
    assert not bool((ex == 4).any())
    probs = torch.softmax(ref_block.gate(tokens_f), dim=-1).gather(-1, ex.long())
    w = probs / probs.sum(-1, keepdim=True)
    yb = torch.zeros_like(tokens_f)
    for e in range(experts):
        h = torch.nn.functional.gelu(tokens_f @ ref_block.w1[e].t() + ref_block.b1[e], approximate="tanh")
        ye = h @ ref_block.w2[e].t() + ref_block.b2[e]
        yb = yb + ye * ((ex == e).float() * w).sum(-1, keepdim=True)
    yb = yb.view(x.shape)
    assert _rel(ya, yb) < 2e-2
    g = torch.randn_like(yb)
    ya.backward(g.bfloat16())
    yb.backward(g)
    assert _rel(xa.grad, xb.grad) < 3e-2
    for name in ("w1", "b1", "w2", "b2"):
        ga, gb = getattr(block, name).grad, getattr(ref_block, name).grad
        assert torch.isfinite(ga.float()).all()
        assert _rel(ga, gb) < 3e-2, name
        assert float(ga[4].float().abs().max()) == 0.0    # the empty expert's gradients are exact zeros
    assert _rel(block.gate.weight.grad, ref_block.gate.weight.grad) < 5e-2


@pytest.mark.gpu
def test_gemm_tma_store_epilogue_tails_with_gate_residual():
    from visionrl_b200.ops import _ext

    torch.manual_seed(7)
    ext = _ext.load()
    batch, seq, k, n = 3, 77, 192, 200          # M = 231 (not a multiple of 32), N % 64 != 0
    m = batch * seq
    a = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(n, device="cuda").bfloat16()
    mod = torch.randn(batch, 3 * n, device="cuda").bfloat16()
    gate = mod[:, n:2 * n]                       # strided view
    res = torch.randn(m, n, device="cuda").bfloat16()
    poison = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    del poison
    got = ext.gemm_bf16(a, w, bias, gate, res, 0, seq, False, False, False)
    lin = a.float() @ w.float().t() + bias.float()
    ref = res.float() + gate.float().repeat_interleave(seq, 0) * lin
    assert ext.gemm_last_status() == 0
    assert torch.isfinite(got.float()).all()
    assert torch.allclose(got.float(), ref, atol=6e-2, rtol=3e-2)
    got2 = ext.gemm_bf16(a, w, bias, None, res, 1, 1, False, False, False)
    ref2 = torch.nn.functional.gelu(lin, approximate="tanh") + res.float()
    assert torch.allclose(got2.float(), ref2, atol=6e-2, rtol=3e-2)


# ------------------------------------------------------------------------ tcgen05 attention
@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(2, 3, 1178, 1178, 64), (1, 2, 300, 512, 128), (2, 2, 128, 77, 64),
                                   (1, 4, 515, 515, 128)])
def test_flash_attention_forward_matches_fp32(shape):
    from visionrl_b200.ops import _ext
    from visionrl_b200.ops.attention import attention_reference, flash_attention_forward

    b, h, sq, skv, d = shape
    torch.manual_seed(8)
    q = torch.randn(b, h, sq, d, device="cuda").bfloat16()
    k = torch.randn(b, h, skv, d, device="cuda").bfloat16()
    v = torch.randn(b, h, skv, d, device="cuda").bfloat16()
    out, lse = flash_attention_forward(q, k, v, d ** -0.5)
    torch.cuda.synchronize()
    assert _ext.load().flash_attn_last_status() == 0
    ref = attention_reference(q.float(), k.float(), v.float())
    assert out.shape == ref.shape
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    scores = torch.matmul(q.float(), k.float().transpose(-1, -2)) * d ** -0.5
    assert torch.allclose(lse, torch.logsumexp(scores, dim=-1), atol=2e-3, rtol=1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("shape", [(2, 3, 1178, 1178, 64), (1, 2, 300, 512, 128), (2, 2, 128, 77, 64),
                                   (1, 2, 515, 515, 128)])
def test_flash_attention_forward_variants_agree_with_fp32(shape, variant):
    """Both forward kernels (register-accumulating, lazy-rescale) against the fp32 oracle; the
    lazy one is also checked on scores with a large dynamic range, where its running maximum
    grows past the rescale threshold several times."""
    from visionrl_b200.ops import _ext
    from visionrl_b200.ops.attention import attention_reference, flash_attention_forward

    b, h, sq, skv, d = shape
    torch.manual_seed(8)
    for spread in (1.0, 6.0):
        q = (torch.randn(b, h, sq, d, device="cuda") * spread).bfloat16()
        k = torch.randn(b, h, skv, d, device="cuda").bfloat16()
        # keys grow along the sequence so later tiles raise the maximum
        k = (k.float() * torch.linspace(0.2, 1.5, skv, device="cuda")[None, None, :, None]).bfloat16()
        v = torch.randn(b, h, skv, d, device="cuda").bfloat16()
        out, lse = flash_attention_forward(q, k, v, d ** -0.5, False, variant)
        torch.cuda.synchronize()
        assert _ext.load().flash_attn_last_status() == 0
        ref = attention_reference(q.float(), k.float(), v.float())
        assert torch.allclose(out.float(), ref, atol=3e-2, rtol=3e-2)
        scores = torch.matmul(q.float(), k.float().transpose(-1, -2)) * d ** -0.5
        assert torch.allclose(lse, torch.logsumexp(scores, dim=-1), atol=5e-3, rtol=2e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(2, 3, 640, 640, 128), (1, 2, 300, 300, 64), (2, 2, 130, 515, 128),
                                   (1, 4, 77, 77, 64), (1, 2, 1, 200, 128)])
def test_flash_attention_causal_forward_backward_match_fp32(shape):
    """Causal attention (Sq <= Skv, last query aligned with the last key), tails included."""
    from visionrl_b200.ops import _ext
    from visionrl_b200.ops.attention import (attention_reference, flash_attention_backward,
                                             flash_attention_forward)

    b, h, sq, skv, d = shape
    torch.manual_seed(28)
    q = torch.randn(b, h, sq, d, device="cuda").bfloat16()
    k = torch.randn(b, h, skv, d, device="cuda").bfloat16()
    v = torch.randn(b, h, skv, d, device="cuda").bfloat16()
    dout = torch.randn(b, h, sq, d, device="cuda").bfloat16()
    out, lse = flash_attention_forward(q, k, v, d ** -0.5, True)
    dq, dk, dv = flash_attention_backward(dout, q, k, v, out, lse, d ** -0.5, True)
    torch.cuda.synchronize()
    assert _ext.load().flash_attn_last_status() == 0
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref_out = attention_reference(qf, kf, vf, causal=True)
    assert torch.allclose(out.float(), ref_out, atol=2e-2, rtol=2e-2)
    ref = torch.autograd.grad(ref_out, (qf, kf, vf), dout.float())
    for got, want in zip((dq, dk, dv), ref):
        err = (got.float() - want).abs().max().item()
        assert err <= 2e-2 * max(1.0, want.abs().max().item()), err


@pytest.mark.gpu
def test_causal_attention_dispatch_trains_through_own_kernels():
    from visionrl_b200.ops import _ext
    from visionrl_b200.ops import attention as A

    torch.manual_seed(29)
    b, h, s, d = 2, 4, 200, 128
    q, k, v = (torch.randn(b, h, s, d, device="cuda").bfloat16().requires_grad_(True) for _ in range(3))
    before = _ext.launch_count
    out = A.attention(q, k, v, causal=True)
    out.float().pow(2).sum().backward()
    assert _ext.launch_count - before >= 4          # forward + three backward launches
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = A.attention_reference(qf, kf, vf, causal=True)
    ref.pow(2).sum().backward()
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    for got, want in ((q, qf), (k, kf), (v, vf)):
        assert (got.grad.float() - want.grad).abs().max().item() <= 3e-2 * max(1.0, want.grad.abs().max().item())


@pytest.mark.gpu
def test_flash_attention_token_major_views_and_dispatch():
    from visionrl_b200.ops.attention import attention, attention_reference

    torch.manual_seed(9)
    b, s, h, d = 2, 333, 4, 64
    bufs = [torch.randn(b, s, h, d, device="cuda").bfloat16() for _ in range(3)]
    q, k, v = (t.transpose(1, 2) for t in bufs)            # [B, H, S, D] views, token-major storage
    with torch.no_grad():
        out = attention(q, k, v)
    ref = attention_reference(q.float(), k.float(), v.float())
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    merged = out.transpose(1, 2).reshape(b, s, h * d)
    assert merged.data_ptr() == out.data_ptr()              # merging heads is a view, not a copy


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(1, 1, 64, 64, 64), (2, 2, 130, 77, 64), (1, 2, 300, 512, 128),
                                   (1, 4, 515, 515, 128), (2, 3, 1178, 1178, 64)])
def test_flash_attention_backward_matches_fp32_autograd(shape):
    from visionrl_b200.ops import _ext
    from visionrl_b200.ops.attention import (attention_reference, flash_attention_backward,
                                             flash_attention_forward)

    b, h, sq, skv, d = shape
    torch.manual_seed(18)
    q = torch.randn(b, h, sq, d, device="cuda").bfloat16()
    k = torch.randn(b, h, skv, d, device="cuda").bfloat16()
    v = torch.randn(b, h, skv, d, device="cuda").bfloat16()
    dout = torch.randn(b, h, sq, d, device="cuda").bfloat16()
    out, lse = flash_attention_forward(q, k, v, d ** -0.5)
    dq, dk, dv = flash_attention_backward(dout, q, k, v, out, lse, d ** -0.5)
    torch.cuda.synchronize()
    assert _ext.load().flash_attn_last_status() == 0
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = torch.autograd.grad(attention_reference(qf, kf, vf), (qf, kf, vf), dout.float())
    for got, want in zip((dq, dk, dv), ref):
        assert got.shape == want.shape
        err = (got.float() - want).abs().max().item()
        assert err <= 2e-2 * max(1.0, want.abs().max().item()), err
    # same inputs, same bits: no atomics anywhere in the backward
    again = flash_attention_backward(dout, q, k, v, out, lse, d ** -0.5)
    assert all(torch.equal(a, b_) for a, b_ in zip(again, (dq, dk, dv)))


@pytest.mark.gpu
def test_differentiable_attention_runs_own_kernels_on_token_major_views():
    from visionrl_b200.ops import attention as A

    torch.manual_seed(19)
    b, s, h, d = 2, 333, 4, 64
    bufs = [torch.randn(b, s, h, d, device="cuda").bfloat16().requires_grad_(True) for _ in range(3)]
    w = torch.randn(b, h, s, d, device="cuda").bfloat16()
    grads = {}
    for impl in ("own", "library"):
        A.set_backward_impl(impl)
        try:
            q, k, v = (t.transpose(1, 2) for t in bufs)
            out = A.attention(q, k, v)
            grads[impl] = torch.autograd.grad((out.float() * w.float()).sum(), bufs)
            if impl == "own":
                assert type(out.grad_fn).__name__ == "_FlashAttnFnBackward"
        finally:
            A.set_backward_impl("own")
    for a, b_ in zip(grads["own"], grads["library"]):
        assert torch.allclose(a.float(), b_.float(), atol=3e-2, rtol=3e-2)


@pytest.mark.gpu
def test_backward_phase_counters_and_mma_issue_probe():
    from visionrl_b200.ops import _ext
    from visionrl_b200.ops.attention import flash_attention_backward, flash_attention_forward

    ext = _ext.load()
    torch.manual_seed(20)
    q, k, v, do = (torch.randn(1, 2, 300, 64, device="cuda").bfloat16() for _ in range(4))
    out, lse = flash_attention_forward(q, k, v, 0.125)
    plain = flash_attention_backward(do, q, k, v, out, lse, 0.125)
    ext.flash_attn_bwd_timing(True)
    timed = flash_attention_backward(do, q, k, v, out, lse, 0.125)
    counters = ext.flash_attn_bwd_timing(False)
    assert counters.shape == (2, 16)
    # 2 heads x ceil(300 / 128) owned tiles per pass, ceil(300 / 64) steps each
    assert counters[:, 0].tolist() == [6, 6] and counters[:, 14].tolist() == [30, 30]
    assert (counters[:, 1] > 0).all()
    assert all(torch.equal(a, b) for a, b in zip(plain, timed))          # counters do not change results
    assert ext.flash_attn_last_status() == 0
    issue, complete, ok = ext.mma_issue_probe(128, 32, 8, True, 1, False).tolist()
    assert ok == 1 and 0 < issue <= complete < 32 * 8 * 2000


@pytest.mark.gpu
def test_joint_qkv_prepare_matches_concatenated_reference():
    from visionrl_b200.ops.qkv import joint_qkv_prepare, qkv_prepare_reference

    torch.manual_seed(10)
    b, sa, sb, heads, dh = 2, 40, 13, 4, 64
    d = heads * dh
    res = []
    for use_kernel in (True, False):
        gen = torch.Generator("cuda").manual_seed(3)
        xa = torch.randn(b, sa, 3 * d, device="cuda", generator=gen).bfloat16().requires_grad_()
        xb = torch.randn(b, sb, 3 * d, device="cuda", generator=gen).bfloat16().requires_grad_()
        ws = [(1 + 0.1 * torch.randn(dh, device="cuda", generator=gen)).bfloat16().requires_grad_()
              for _ in range(4)]
        if use_kernel:
            q, k, v = joint_qkv_prepare(xa, xb, heads, (ws[0], ws[1]), (ws[2], ws[3]))
        else:
            qa, ka, va = qkv_prepare_reference(xa, heads, ws[0], ws[1])
            qb, kb, vb = qkv_prepare_reference(xb, heads, ws[2], ws[3])
            q, k, v = torch.cat([qa, qb], 2), torch.cat([ka, kb], 2), torch.cat([va, vb], 2)
        grads = [torch.randn(q.shape, device="cuda", generator=gen).bfloat16() for _ in range(3)]
        torch.autograd.backward([q, k, v], grads)
        res.append((q, k, v, xa.grad, xb.grad, *[w.grad for w in ws]))
    for got, ref in zip(*res):
        assert _rel(got, ref) < 3e-2


@pytest.mark.gpu
def test_gate_residual_fused_forward_backward():
    from visionrl_b200.ops.linear import gate_residual

    torch.manual_seed(12)
    b, s, d = 3, 77, 256
    res = []
    for fused in (True, False):
        gen = torch.Generator("cuda").manual_seed(1)
        y = torch.randn(b, s, d, device="cuda", generator=gen).bfloat16().requires_grad_()
        mod = torch.randn(b, 3 * d, device="cuda", generator=gen).bfloat16().requires_grad_()
        r = torch.randn(b, s, d, device="cuda", generator=gen).bfloat16().requires_grad_()
        gate = mod[:, d:2 * d]
        if fused:
            out = gate_residual(y, gate, r)
        else:
            out = (r.float() + gate.float().unsqueeze(1) * y.float())
        g = torch.randn(b, s, d, device="cuda", generator=gen).bfloat16()
        out.backward(g.to(out.dtype))
        res.append((out, y.grad, mod.grad, r.grad))
    for got, ref in zip(*res):
        assert _rel(got, ref) < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(2, 128, 64, 48), (1, 256, 33, 17), (2, 512, 16, 16)])
@pytest.mark.parametrize("apply_silu", [True, False])
def test_groupnorm_nhwc_matches_fp32(shape, apply_silu):
    from visionrl_b200.ops.norm import group_norm_silu

    torch.manual_seed(13)
    n, c, h, w = shape
    norm = torch.nn.GroupNorm(32, c, eps=1e-6).cuda().bfloat16()
    with torch.no_grad():
        norm.weight.copy_(1 + 0.2 * torch.randn(c))
        norm.bias.copy_(0.1 * torch.randn(c))
    x = (torch.randn(n, c, h, w, device="cuda") * 2 + 0.5).bfloat16().contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        got = group_norm_silu(x, norm, apply_silu)
    ref = torch.nn.functional.group_norm(x.float(), 32, norm.weight.float(), norm.bias.float(), 1e-6)
    if apply_silu:
        ref = torch.nn.functional.silu(ref)
    assert got.is_contiguous(memory_format=torch.channels_last)
    assert torch.allclose(got.float(), ref, atol=3e-2, rtol=3e-2)


@pytest.mark.gpu
def test_gelu_mlp_fused_epilogues_match_fp32():
    from visionrl_b200.ops.linear import gelu_mlp

    torch.manual_seed(14)
    m, d, hid = 333, 256, 1024
    res = []
    for fused in (True, False):
        gen = torch.Generator("cuda").manual_seed(2)
        dt = torch.bfloat16 if fused else torch.float32
        x = torch.randn(3, m // 3, d, device="cuda", generator=gen).to(dt).requires_grad_()
        w1 = (torch.randn(hid, d, device="cuda", generator=gen) * 0.05).to(dt).requires_grad_()
        b1 = (torch.randn(hid, device="cuda", generator=gen) * 0.1).to(dt).requires_grad_()
        w2 = (torch.randn(d, hid, device="cuda", generator=gen) * 0.05).to(dt).requires_grad_()
        b2 = (torch.randn(d, device="cuda", generator=gen) * 0.1).to(dt).requires_grad_()
        if fused:
            y = gelu_mlp(x, w1, b1, w2, b2)
        else:
            hpre = torch.nn.functional.linear(x, w1, b1)
            y = torch.nn.functional.linear(torch.nn.functional.gelu(hpre, approximate="tanh"), w2, b2)
        g = torch.randn(y.shape, device="cuda", generator=gen).to(dt)
        y.backward(g)
        res.append((y, x.grad, w1.grad, b1.grad, w2.grad, b2.grad))
    for got, ref in zip(*res):
        assert _rel(got, ref) < 3e-2


@pytest.mark.gpu
def test_gemm_dual_output_returns_pre_and_post_activation():
    from visionrl_b200.ops import _ext

    torch.manual_seed(15)
    a = torch.randn(300, 192, device="cuda").bfloat16()
    w = (torch.randn(200, 192, device="cuda") * 0.1).bfloat16()
    b = torch.randn(200, device="cuda").bfloat16()
    post, pre = _ext.load().gemm_bf16_dual(a, w, b, 1)
    ref = a.float() @ w.float().t() + b.float()
    assert torch.allclose(pre.float(), ref, atol=5e-2, rtol=2e-2)
    assert torch.allclose(post.float(), torch.nn.functional.gelu(ref, approximate="tanh"), atol=5e-2, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("int4", [False, True])
def test_janus_graph_decode_matches_eager_decode(int4):
    from visionrl_b200.models.families.janus_pro.policy import JanusProConfig, JanusProPolicy

    arch = {"num_layers": 2, "hidden_size": 256, "num_heads": 2, "ffn_dim": 512, "vocab_size": 512,
            "image_vocab_size": 1024, "codebook_dim": 8, "vq_base": 32, "vq_mults": (1, 2), "vq_blocks": 1}
    cfg = JanusProConfig(model_path="", dtype="bfloat16", use_lora=True, lora_rank=4, lora_alpha=8,
                         image_token_num=16, image_size=64, patch_size=16, random_init=True,
                         int4_decode=int4, arch=arch)
    policy = JanusProPolicy(cfg, device="cuda")
    b, l_text = 3, 8
    ids = torch.randint(0, 512, (2 * b, l_text), device="cuda")
    mask = torch.ones(2 * b, l_text, dtype=torch.long, device="cuda")
    mask[0, -2:] = 0
    emb = policy.embed_text(ids)
    outs = []
    for graph in (True, False):
        policy.decode_graph = graph
        gen = torch.Generator(device="cpu").manual_seed(5)
        tokens, logp = policy.sample_image_tokens(emb[:b], emb[b:], mask[:b], mask[b:], cfg_weight=3.0,
                                                  temperature=0.9, image_token_num=16, generator=gen)
        outs.append((tokens.clone(), logp.clone()))
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1], outs[1][1])
    assert outs[0][0].min() >= 0 and outs[0][0].max() < 1024 and torch.isfinite(outs[0][1]).all()


@pytest.mark.gpu
@pytest.mark.parametrize("m", [1, 20, 32, 64])
@pytest.mark.parametrize("nk", [(2048 + 24, 2048), (512, 5632), (6144, 256)])
def test_int4_tensor_core_gemm_matches_dequantised_matmul(m, nk):
    from visionrl_b200.ops import _ext
    from visionrl_b200.ops.quant import int4_linear_reference, quantize_int4

    torch.manual_seed(16)
    n, k = nk
    w = torch.randn(n, k, device="cuda") * 0.05
    packed, scales = quantize_int4(w)
    x = torch.randn(m, k, device="cuda").bfloat16()
    bias = torch.randn(n, device="cuda").bfloat16()
    ext = _ext.load()
    got = ext.int4_gemm(x, packed, scales, bias, 128)
    torch.cuda.synchronize()
    assert ext.int4_gemm_last_status() == 0
    ref = int4_linear_reference(x.float(), packed, scales, bias)
    assert torch.allclose(got.float(), ref, atol=4e-2, rtol=2e-2)
    again = ext.int4_gemm(x, packed, scales, None, 128)
    assert torch.allclose(again.float(), ref - bias.float(), atol=4e-2, rtol=2e-2)


@pytest.mark.gpu
def test_weight_gradients_accumulate_in_place_across_backward_calls():
    from visionrl_b200.ops.linear import accumulate_weight_grads_in_place, gelu_mlp, linear

    torch.manual_seed(17)
    d, hid = 256, 512
    w = (torch.randn(d, d, device="cuda") * 0.05).bfloat16().requires_grad_()
    w1 = (torch.randn(hid, d, device="cuda") * 0.05).bfloat16().requires_grad_()
    w2 = (torch.randn(d, hid, device="cuda") * 0.05).bfloat16().requires_grad_()
    params = [w, w1, w2]
    for p in params:
        p.grad = torch.zeros_like(p)
    buffers = [p.grad.data_ptr() for p in params]
    ref = [torch.zeros_like(p, dtype=torch.float32) for p in params]
    for step in range(3):
        x = torch.randn(4, 100, d, device="cuda").bfloat16()
        with accumulate_weight_grads_in_place():
            (gelu_mlp(linear(x, w), w1, None, w2, None).float().pow(2).mean() * 50).backward()
        xf = x.float()
        pf = [p.detach().float().requires_grad_() for p in params]
        h = torch.nn.functional.linear(xf, pf[0])
        y = torch.nn.functional.linear(torch.nn.functional.gelu(torch.nn.functional.linear(h, pf[1]),
                                                                approximate="tanh"), pf[2])
        (y.pow(2).mean() * 50).backward()
        for r, q in zip(ref, pf):
            r += q.grad
    for p, ptr, r in zip(params, buffers, ref):
        assert p.grad.data_ptr() == ptr                      # still the same buffer
        assert _rel(p.grad, r) < 4e-2


@pytest.mark.gpu
def test_flag_signal_wait_and_bounded_expiry_single_device():
    """Flag kernels on one device: a signalled slot satisfies the wait; a slot nobody sets makes
    the wait give up after its limit and report, leaving the stream usable."""
    import time

    from visionrl_b200.ops import _ext

    ext = _ext.load()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    peers = torch.tensor([flags.data_ptr()], dtype=torch.int64)       # a group of one: this device
    ext.flag_signal(peers, flags, 9, 1, 5)
    ext.flag_wait(flags, 9, 1, 5, 1.0, status)
    torch.cuda.synchronize()
    assert int(flags[9]) == 5 and status.tolist() == [0, 0, 0, 0]
    t0 = time.time()
    ext.flag_wait(flags, 20, 2, 3, 0.3, status)                        # slots 20, 21 stay at zero
    after = torch.ones(4, device="cuda").sum()
    torch.cuda.synchronize()
    assert 0.25 < time.time() - t0 < 3.0
    code, slot, seen, expected = status.tolist()
    assert code == 1 and slot in (20, 21) and seen == 0 and expected == 3
    assert float(after) == 4.0
    # barrier of a one-rank group returns at once
    status.zero_()
    ext.flag_barrier(peers, flags, 0, 1, 0, 1, 1.0, status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0] and int(flags[0]) == 1


@pytest.mark.gpu
def test_wrappers_refuse_cpu_operands():
    """Every tensor operand is checked, not only the first: a CPU tensor is a Python error."""
    from visionrl_b200.ops import _ext

    ext = _ext.load()
    n = 1024
    p = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    g = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    master = torch.zeros(n, device="cuda")
    m_cpu = torch.zeros(n)
    v = torch.zeros(n, device="cuda")
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ext.adamw_flat(p, g, master, m_cpu, v, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, None)
    r = torch.zeros(8, device="cuda")
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ext.group_advantages(r, torch.zeros(8, dtype=torch.int64), 1e-6, 5.0, False)
    x = torch.zeros(2, 64, device="cuda")
    ab = torch.ones(2, device="cuda")
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ext.sde_step_fwd(x, x.clone(), ab, ab, torch.ones(2), ab, None, x.clone(), False, True)
    lp = torch.zeros(2, 8, device="cuda")
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ext.token_loss_fwd(lp, torch.zeros(2, 8), torch.zeros(2, device="cuda"), None, None, 0.2, True)


@pytest.mark.gpu
@pytest.mark.parametrize("has_cfg,dtype", [(True, torch.bfloat16), (False, torch.float32)])
@pytest.mark.parametrize("sde_type", ["sde", "cps"])
def test_fused_rollout_step_matches_the_separate_ops(has_cfg, dtype, sde_type):
    """Guidance combine + SDE step + log-density + trajectory write in one kernel against the
    separate tensor ops, with the noise given; the replay of what it wrote reproduces the
    recorded log-probability bit for bit; with Philox noise the step is a pure function of the seed."""
    from visionrl_b200.algorithms.flow_matching import step_coefficients
    from visionrl_b200.ops import _ext
    from visionrl_b200.ops.sde import sde_step

    ext = _ext.load()
    torch.manual_seed(31)
    b, steps, shape, g = 3, 4, (16, 12, 20), 4.5
    n = 16 * 12 * 20
    path = torch.zeros(b, steps + 1, *shape, device="cuda")
    path[:, 1] = torch.randn(b, *shape, device="cuda")
    pred = torch.randn((2 if has_cfg else 1) * b, *shape, device="cuda").to(dtype)
    sigmas = torch.linspace(1.0, 0.0, steps + 1, device="cuda")
    index = torch.full((b,), 1, dtype=torch.long, device="cuda")
    a, bb, _std, scale, _sq, dt = step_coefficients(sigmas, index, 0.7, sde_type)
    noise = torch.randn(b, n, device="cuda")
    logp = torch.zeros(b, steps, device="cuda")
    ext.sde_rollout_step(pred, has_cfg, g, 0, path, 1, a.contiguous(), bb.contiguous(), scale.contiguous(),
                         dt.contiguous(), noise, 0, 0, logp, False, sde_type == "sde")
    if has_cfg:
        u, c = pred.float().chunk(2, dim=0)
        v = u + g * (c - u)
    else:
        v = pred.float()
    want_next, want_lp, _ = sde_step(v, path[:, 1].contiguous(), a, bb, scale, dt, None, noise.view(b, *shape),
                                     False, sde_type == "sde")
    assert torch.allclose(path[:, 2], want_next, atol=1e-6, rtol=1e-6)
    assert torch.allclose(logp[:, 1], want_lp, atol=1e-5, rtol=1e-5)
    # replay: the recorded next latent given back reproduces the recorded log-probability exactly
    _, replay_lp, _ = sde_step(v, path[:, 1].contiguous(), a, bb, scale, dt, path[:, 2].contiguous(), None,
                               False, sde_type == "sde")
    assert torch.equal(replay_lp, logp[:, 1])
    # Philox noise: same seed and offset -> same bits, another seed -> other bits, sane moments
    outs = []
    for seed in (7, 7, 8):
        p2, lp2 = path.clone(), torch.zeros_like(logp)
        ext.sde_rollout_step(pred, has_cfg, g, 0, p2, 1, a.contiguous(), bb.contiguous(), scale.contiguous(),
                             dt.contiguous(), None, seed, 4, lp2, False, sde_type == "sde")
        outs.append(p2[:, 2].clone())
    assert torch.equal(outs[0], outs[1]) and not torch.equal(outs[0], outs[2])
    mean = a.view(-1, 1, 1, 1) * path[:, 1] + bb.view(-1, 1, 1, 1) * v
    eps = (outs[0] - mean) / scale.view(-1, 1, 1, 1)
    assert abs(float(eps.mean())) < 0.05 and abs(float(eps.std()) - 1.0) < 0.05
    # deterministic steps ignore the noise
    p3, lp3 = path.clone(), torch.zeros_like(logp)
    ext.sde_rollout_step(pred, has_cfg, g, 0, p3, 1, a.contiguous(), bb.contiguous(), scale.contiguous(),
                         dt.contiguous(), None, 1, 0, lp3, True, sde_type == "sde")
    assert torch.allclose(p3[:, 2], path[:, 1] + dt.view(-1, 1, 1, 1) * v, atol=1e-6)


@pytest.mark.gpu
def test_fused_decode_step_matches_the_tensor_op_layer_path(monkeypatch):
    """The decode step with fused glue kernels (add + RMSNorm, RoPE + cache append, SwiGLU) against
    the same step written with tensor ops: hidden state and cache contents, three positions."""
    from visionrl_b200.models.nn.llama import LlamaConfig, LlamaDecoder

    torch.manual_seed(41)
    cfg = LlamaConfig(num_layers=3, hidden_size=512, num_heads=4, ffn_dim=1024, vocab_size=128)
    net = LlamaDecoder(cfg).to("cuda", torch.bfloat16).eval()
    rows, max_len = 6, 16
    outs, caches = [], []
    for fused in (True, False):
        if not fused:
            monkeypatch.setattr(LlamaDecoder, "_fused_decode_ok", lambda self, e: False)
        cache = net.new_cache(rows, max_len, torch.device("cuda"), torch.bfloat16)
        gen = torch.Generator(device="cuda").manual_seed(5)
        hidden = []
        with torch.no_grad():
            for p in range(3):
                emb = torch.randn(rows, cfg.hidden_size, device="cuda", generator=gen).bfloat16()
                hidden.append(net.decode_step_at(emb, cache, torch.tensor([p], device="cuda")))
        outs.append(torch.stack(hidden))
        caches.append(cache.data.clone())
    assert torch.allclose(outs[0].float(), outs[1].float(), atol=6e-2, rtol=6e-2)
    assert torch.allclose(caches[0].float(), caches[1].float(), atol=3e-2, rtol=3e-2)
    assert float(caches[0][:, :, :, :, 3:].abs().max()) == 0.0           # nothing written past position 2


@pytest.mark.gpu
@pytest.mark.parametrize("rows,k,n,rank", [(32, 2048, 6144, 32), (5, 256, 264, 8), (64, 1024, 2048, 64), (32, 2048, 2048, 128), (9, 512, 520, 40)])
def test_lora_apply_rows_matches_fp32_reference(rows, k, n, rank):
    """The decode-sized low-rank update y += s (x A^T) B^T against fp32 tensor math, row and column tails
    included, and the layer-level path it serves (LoRALinear without autograd, a few rows)."""
    from visionrl_b200.models.nn.layers import LoRALinear
    from visionrl_b200.ops import _ext

    torch.manual_seed(41)
    x = torch.randn(rows, k, device="cuda").bfloat16()
    a = (torch.randn(rank, k, device="cuda") / rank).bfloat16()
    b = (torch.randn(n, rank, device="cuda") * 0.1).bfloat16()
    y0 = torch.randn(rows, n, device="cuda").bfloat16()
    y = y0.clone()
    _ext.load().lora_apply_rows(y, x, a, b, 0.5)
    want = y0.float() + 0.5 * (x.float() @ a.float().t()) @ b.float().t()
    assert torch.allclose(y.float(), want, atol=2e-2, rtol=2e-2)
    layer = LoRALinear(k, n, bias=True).cuda().bfloat16()
    layer.add_adapter(rank, 2.0 * rank)
    with torch.no_grad():
        layer.lora_B.normal_(std=0.05)
        small = layer(x)                                    # kernel path (rows <= 64, no autograd)
    big = layer(torch.cat([x] * (65 // rows + 1))[:65 + rows])[:rows]     # > 64 rows: the tensor-op path
    assert _rel(small, big) < 2e-2


@pytest.mark.gpu
def test_decode_attention_skips_unwritten_slots_and_matches_reference():
    """Runs of eight keys per pass: masked keys (including NaN-filled, never written cache slots) have no
    influence, lengths that are not a multiple of the run are handled, fully masked rows give zeros."""
    from visionrl_b200.ops import _ext

    torch.manual_seed(43)
    rows, heads, length, d = 6, 4, 77, 128
    q = torch.randn(rows, heads, d, device="cuda").bfloat16()
    kc = torch.randn(rows, heads, length, d, device="cuda").bfloat16()
    vc = torch.randn(rows, heads, length, d, device="cuda").bfloat16()
    valid = torch.rand(rows, length, device="cuda") < 0.6
    valid[1] = False
    valid[2, :] = True
    kc[~valid.unsqueeze(1).expand(-1, heads, -1)] = float("nan")
    vc[~valid.unsqueeze(1).expand(-1, heads, -1)] = float("nan")
    out = _ext.load().decode_attention(q.view(rows, heads, 1, d), kc, vc, valid, length, d ** -0.5).view(rows, heads, d)
    scores = torch.einsum("rhd,rhld->rhl", q.float(), torch.nan_to_num(kc.float())) * d ** -0.5
    scores = scores.masked_fill(~valid.unsqueeze(1), float("-inf"))
    probs = torch.nan_to_num(torch.softmax(scores, dim=-1))
    want = torch.einsum("rhl,rhld->rhd", probs, torch.nan_to_num(vc.float()))
    assert torch.isfinite(out.float()).all()
    assert torch.allclose(out.float(), want, atol=2e-2, rtol=2e-2)
    assert float(out[1].float().abs().max()) == 0.0
