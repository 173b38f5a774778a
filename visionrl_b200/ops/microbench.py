"""Per-kernel micro-benchmarks: ``python -m visionrl_b200.ops.microbench <kernel> [options]``.

Every case times the sm_100a kernel with CUDA events on the launching stream (warm-up first,
synchronise on both sides, a buffer larger than L2 rewritten between iterations) and prints one
JSON line with the achieved throughput, the same figure for the library / eager counterpart,
and the fraction of the roofline denominator passed with ``--peak-tflops`` / ``--peak-gbs``.
The same entry points are what the profiler captures are taken from (``--iters 1 --warmup 1``).
"""

from __future__ import annotations

import argparse
import json
import sys

import torch

_L2_FLUSH_BYTES = 256 << 20


def _time(fn, iters: int, warmup: int, flush: torch.Tensor | None) -> float:
    """Median milliseconds of ``fn`` over ``iters`` runs."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    samples = []
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        # keep the device busy for ~0.1 ms while the host enqueues the work: the events then bracket
        # device execution only, not the launch latency of the first kernel (which would dominate a
        # kernel of a few microseconds)
        torch.cuda._sleep(200_000)
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        samples.append(start.elapsed_time(stop))
    samples.sort()
    return samples[len(samples) // 2]


def _flush_buffer(enabled: bool) -> torch.Tensor | None:
    return torch.zeros(_L2_FLUSH_BYTES // 4, device="cuda", dtype=torch.int32) if enabled else None


def bench_gemm(args) -> dict:
    from visionrl_b200.ops import _ext

    ext = _ext.load()
    m, n, k = args.m, args.n, args.k
    flush = _flush_buffer(not args.no_flush)
    act = {"none": 0, "gelu": 1, "silu": 2}[args.act]
    if args.layout != "nt":
        # the two backward forms of a linear layer: nn = dX = dY[M,K] @ W[K,N] (B row-major),
        # tn = dW = dY[K,M].T @ X[K,N] (both operands row-major over the contraction)
        a = torch.randn((m, k) if args.layout == "nn" else (k, m), device="cuda", dtype=torch.bfloat16)
        b = torch.randn(k, n, device="cuda", dtype=torch.bfloat16) * 0.02
        a_mn = args.layout == "tn"

        def own_b():
            return ext.gemm_bf16(a, b, None, None, None, 0, 0, a_mn, True, False)

        def lib_b():
            return (a.t() if a_mn else a) @ b

        flops = 2.0 * m * n * k
        t_lib = _time(lib_b, args.iters, args.warmup, flush)
        t_own = _time(own_b, args.iters, args.warmup, flush)
        err = (own_b().float() - lib_b().float()).abs().max().item() / max(lib_b().float().abs().max().item(), 1e-6)
        out = {"kernel": "gemm_bf16", "layout": args.layout, "m": m, "n": n, "k": k,
               "cublas_ms": round(t_lib, 4), "cublas_tflops": round(flops / t_lib / 1e9, 1),
               "ms": round(t_own, 4), "tflops": round(flops / t_own / 1e9, 1),
               "max_rel_diff_vs_cublas": round(err, 5), "status": int(ext.gemm_last_status())}
        if args.peak_tflops:
            out["frac_of_measured_peak"] = round(out["tflops"] / args.peak_tflops, 3)
        return out
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16) * 0.02
    bias = torch.randn(n, device="cuda", dtype=torch.bfloat16) if args.bias else None

    def own():
        return ext.gemm_bf16(a, w, bias, None, None, act, 1, False, False, False)

    def lib():
        return torch.nn.functional.linear(a, w, bias)

    out = {"kernel": "gemm_bf16", "m": m, "n": n, "k": k, "act": args.act, "bias": bool(args.bias)}
    flops = 2.0 * m * n * k
    if not args.skip_lib:
        t_lib = _time(lib, args.iters, args.warmup, flush)
        out["cublas_ms"] = round(t_lib, 4)
        out["cublas_tflops"] = round(flops / t_lib / 1e9, 1)
    t_own = _time(own, args.iters, args.warmup, flush)
    out["ms"] = round(t_own, 4)
    out["tflops"] = round(flops / t_own / 1e9, 1)
    if args.peak_tflops:
        out["frac_of_measured_peak"] = round(out["tflops"] / args.peak_tflops, 3)
    status = ext.gemm_last_status() if hasattr(ext, "gemm_last_status") else 0
    out["status"] = int(status)
    if not args.skip_check:
        ref = torch.nn.functional.linear(a.float(), w.float(), bias.float() if bias is not None else None)
        if act == 1:
            ref = torch.nn.functional.gelu(ref, approximate="tanh")
        elif act == 2:
            ref = torch.nn.functional.silu(ref)
        err = (own().float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
        out["max_rel_err"] = round(err, 5)
    return out


def bench_sde(args) -> dict:
    from visionrl_b200.ops import _ext

    ext = _ext.load()
    b, n = args.batch, args.elems
    v = torch.randn(b, n, device="cuda")
    x = torch.randn(b, n, device="cuda")
    noise = torch.randn(b, n, device="cuda")
    a, bb, scale, dt = (torch.rand(b, device="cuda") + 0.1 for _ in range(4))
    flush = _flush_buffer(not args.no_flush)

    def own():
        return ext.sde_step_fwd(v, x, a, bb, scale, dt, None, noise, False, True)

    t = _time(own, args.iters, args.warmup, flush)
    moved = b * n * 4 * 5   # velocity, sample, noise in; next sample, mean out
    out = {"kernel": "sde_step_fwd", "batch": b, "elems": n, "ms": round(t, 4),
           "gbs": round(moved / t / 1e6, 1)}
    if args.peak_gbs:
        out["frac_of_measured_peak"] = round(out["gbs"] / args.peak_gbs, 3)
    return out


def bench_adaln(args) -> dict:
    from visionrl_b200.ops.norm import adaln_layernorm

    b, s, d = args.batch, args.seq, args.dim
    x = torch.randn(b, s, d, device="cuda", dtype=torch.bfloat16)
    mod = torch.randn(b, 2 * d, device="cuda", dtype=torch.bfloat16)
    shift, scale = mod[:, :d], mod[:, d:]
    flush = _flush_buffer(not args.no_flush)
    t = _time(lambda: adaln_layernorm(x, shift, scale, 1e-6), args.iters, args.warmup, flush)
    moved = 2 * x.numel() * 2
    out = {"kernel": "adaln_fwd", "batch": b, "seq": s, "dim": d, "ms": round(t, 4),
           "gbs": round(moved / t / 1e6, 1)}
    if args.peak_gbs:
        out["frac_of_measured_peak"] = round(out["gbs"] / args.peak_gbs, 3)
    return out


def bench_rowwise(args) -> dict:
    """The bandwidth-bound row kernels of a transformer block at one shape: adaLN forward/backward,
    QKV post-processing forward/backward (per-head RMS norm), gated-residual backward.  GB/s counts
    the tensors each kernel must read and write once."""
    from visionrl_b200.ops import _ext

    ext = _ext.load()
    b, s, d, heads = args.batch, args.seq, args.dim, args.heads
    dh = d // heads
    dev, bf = "cuda", torch.bfloat16
    x = torch.randn(b, s, d, device=dev, dtype=bf)
    gy = torch.randn(b, s, d, device=dev, dtype=bf)
    mod = torch.randn(b, 3 * d, device=dev, dtype=bf) * 0.1
    shift, scale, gate = mod[:, :d], mod[:, d:2 * d], mod[:, 2 * d:]
    qkv = torch.randn(b, s, 3 * d, device=dev, dtype=bf)
    qw = torch.ones(dh, device=dev, dtype=bf)
    kw = torch.ones(dh, device=dev, dtype=bf)
    flush = _flush_buffer(not args.no_flush)
    _, mean, rstd = ext.adaln_fwd(x, shift, scale, 1e-6)
    q, k, v, qr = ext.qkv_prepare_fwd(qkv, qw, kw, None, None, heads, 1e-6, None, None, None, 0)
    gq, gk, gv = (torch.randn_like(q).permute(0, 2, 1, 3) for _ in range(3))      # [B, H, S, Dh] views
    row = x.numel() * 2
    cases = {
        "adaln_fwd": (lambda: ext.adaln_fwd(x, shift, scale, 1e-6), 2 * row),
        "adaln_bwd": (lambda: ext.adaln_bwd(gy, x, scale, mean, rstd), 3 * row),
        "qkv_prepare_fwd": (lambda: ext.qkv_prepare_fwd(qkv, qw, kw, None, None, heads, 1e-6, None, None, None, 0),
                            6 * row),
        "qkv_prepare_bwd": (lambda: ext.qkv_prepare_bwd(gq, gk, gv, qkv, qw, kw, None, None, qr, heads, 0),
                            8 * row),          # g (3), q and k inputs (2), d(qkv) (3)
        "gate_residual_bwd": (lambda: ext.gate_residual_bwd(gy, x, gate), 3 * row),
    }
    out = {"kernel": "rowwise", "batch": b, "seq": s, "dim": d, "heads": heads}
    for name, (fn, moved) in cases.items():
        t = _time(fn, args.iters, args.warmup, flush)
        out[name] = {"ms": round(t, 4), "gbs": round(moved / t / 1e6, 1)}
        if args.peak_gbs:
            out[name]["frac_of_measured_peak"] = round(moved / t / 1e6 / args.peak_gbs, 3)
    return out


def bench_decode(args) -> dict:
    """The three kernels a decode step of the LLaMA trunk spends its time in, at decode size: the int4
    weight-only GEMM (per projection), decode attention over a half-filled cache, and the low-rank
    update.  GB/s counts the bytes each must read once."""
    from visionrl_b200.ops import _ext
    from visionrl_b200.ops.quant import quantize_int4

    ext = _ext.load()
    rows, d, heads, ffn, length, rank = args.rows, args.dim, args.heads, args.ffn, args.length, args.rank
    dev, bf = "cuda", torch.bfloat16
    flush = _flush_buffer(not args.no_flush)
    out = {"kernel": "decode", "rows": rows, "dim": d, "heads": heads, "ffn": ffn, "cache_len": length}
    x = torch.randn(rows, d, device=dev, dtype=bf)
    for name, (n, k) in {"int4_qkv": (3 * d, d), "int4_out": (d, d), "int4_gate_up": (2 * ffn, d),
                         "int4_down": (d, ffn)}.items():
        w = torch.randn(n, k, device=dev) * 0.02
        packed, scales = quantize_int4(w, 128)
        xin = x if k == d else torch.randn(rows, k, device=dev, dtype=bf)
        t = _time(lambda: ext.int4_gemm(xin, packed, scales, None, 128), args.iters, args.warmup, flush)
        out[name] = {"ms": round(t, 4), "gbs": round(n * k / 2 / t / 1e6, 1)}
    dh = d // heads
    q = torch.randn(rows, heads, 1, dh, device=dev, dtype=bf)
    kc = torch.randn(rows, heads, length, dh, device=dev, dtype=bf)
    vc = torch.randn(rows, heads, length, dh, device=dev, dtype=bf)
    valid = torch.zeros(rows, length, device=dev, dtype=torch.bool)
    valid[:, :length // 2] = True
    t = _time(lambda: ext.decode_attention(q, kc, vc, valid, length, dh ** -0.5), args.iters, args.warmup, flush)
    out["decode_attention"] = {"ms": round(t, 4),
                               "gbs": round(2 * rows * heads * (length // 2) * dh * 2 / t / 1e6, 1)}
    a = torch.randn(rank, d, device=dev, dtype=bf)
    b = torch.randn(3 * d, rank, device=dev, dtype=bf)
    y = torch.zeros(rows, 3 * d, device=dev, dtype=bf)
    t = _time(lambda: ext.lora_apply_rows(y, x, a, b, 1.0), args.iters, args.warmup, flush)
    out["lora_apply_rows"] = {"ms": round(t, 4)}
    return out


def bench_attention(args) -> dict:
    from visionrl_b200.ops.attention import flash_attention_forward

    b, h, s, d = args.batch, args.heads, args.seq, args.head_dim
    causal, variant = bool(args.causal), int(args.variant)
    q, k, v = (torch.randn(b, h, s, d, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    flush = _flush_buffer(not args.no_flush)
    flops = 4.0 * b * h * s * s * d * (0.5 if causal else 1.0)
    out = {"kernel": "attention_fwd", "batch": b, "heads": h, "seq": s, "head_dim": d,
           "causal": causal, "variant": variant}
    sdpa = torch.nn.functional.scaled_dot_product_attention
    own = lambda: flash_attention_forward(q, k, v, d ** -0.5, causal, variant)[0]  # noqa: E731
    with torch.no_grad():
        t_lib = _time(lambda: sdpa(q, k, v, is_causal=causal), args.iters, args.warmup, flush)
        t = _time(own, args.iters, args.warmup, flush)
        ref = sdpa(q.float(), k.float(), v.float(), is_causal=causal)
        out["max_abs_err"] = round((own().float() - ref).abs().max().item(), 5)
    out.update({"sdpa_ms": round(t_lib, 4), "sdpa_tflops": round(flops / t_lib / 1e9, 1),
                "ms": round(t, 4), "tflops": round(flops / t / 1e9, 1)})
    if args.peak_tflops:
        out["frac_of_measured_peak"] = round(out["tflops"] / args.peak_tflops, 3)
    if args.backward:
        from visionrl_b200.ops.attention import flash_attention_backward, flash_attention_forward

        scale = d ** -0.5
        dout = torch.randn_like(q)
        o, lse = flash_attention_forward(q, k, v, scale, causal, variant)
        t_b = _time(lambda: flash_attention_backward(dout, q, k, v, o, lse, scale, causal), args.iters,
                    args.warmup, flush)
        ql, kl, vl = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
        ol = torch.nn.functional.scaled_dot_product_attention(ql, kl, vl, is_causal=causal)
        t_lb = _time(lambda: torch.autograd.grad(ol, (ql, kl, vl), dout, retain_graph=True),
                     args.iters, args.warmup, flush)
        qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
        ref = torch.autograd.grad(torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=causal),
                                  (qf, kf, vf), dout.float())
        got = flash_attention_backward(dout, q, k, v, o, lse, scale, causal)
        out.update({"bwd_ms": round(t_b, 4), "bwd_tflops": round(2.5 * flops / t_b / 1e9, 1),
                    "sdpa_bwd_ms": round(t_lb, 4), "sdpa_bwd_tflops": round(2.5 * flops / t_lb / 1e9, 1),
                    "bwd_max_abs_err": [round((g.float() - r).abs().max().item(), 5) for g, r in zip(got, ref)]})
    return out


def bench_mma_issue(args) -> dict:
    """Cycles one issuing thread spends per tcgen05.mma, per commit and per (complete) mbarrier wait."""
    from visionrl_b200.ops import _ext

    ext = _ext.load()
    rows = []
    for n in (64, 128, 256):
        # wait: 0 none, 1 bounded try_wait loop, 2 one non-blocking test_wait
        for group, commit, wait, tmem_a in ((8, False, 0, False), (8, True, 0, False), (8, True, 1, False),
                                            (8, True, 2, False), (4, True, 1, False), (8, False, 0, True)):
            if n == 256 and (tmem_a or group != 8):
                continue
            ext.mma_issue_probe(n, 8, group, commit, wait, tmem_a)                    # warm-up
            issue, complete, ok = ext.mma_issue_probe(n, args.groups, group, commit, wait, tmem_a).tolist()
            rows.append({"n": n, "group": group, "commit_each_group": commit, "wait_each_group": wait,
                         "a_in_tmem": tmem_a, "issue_cycles_per_group": round(issue / args.groups, 1),
                         "complete_cycles_per_group": round(complete / args.groups, 1), "ok": bool(ok)})
    return {"kernel": "mma_issue_probe", "groups": args.groups, "rows": rows}


def bench_attention_phases(args) -> dict:
    """Per-step cycle counters of the two backward passes (see ``flash_attn_bwd_timing``)."""
    from visionrl_b200.ops import _ext
    from visionrl_b200.ops.attention import flash_attention_backward, flash_attention_forward

    ext = _ext.load()
    names = ["ctas", "cta_cycles", "issuerA_wait_own", "issuerA_wait_tiles", "issuerA_wait_elementwise",
             "elementwise_wait_S", "elementwise_tmem_load", "issuerB_waits", "elementwise_compute",
             "elementwise_fence_arrive", "issuerB_issue", "elementwise_epilogue", "producer_wait_stage",
             "producer_vectors", "steps", "issuerA_issue"]
    b, h, s, d = args.batch, args.heads, args.seq, args.head_dim
    q, k, v, do = (torch.randn(b, h, s, d, device="cuda", dtype=torch.bfloat16) for _ in range(4))
    o, lse = flash_attention_forward(q, k, v, d ** -0.5)
    for _ in range(2):
        flash_attention_backward(do, q, k, v, o, lse, d ** -0.5)
    torch.cuda.synchronize()
    ext.flash_attn_bwd_timing(True)
    flash_attention_backward(do, q, k, v, o, lse, d ** -0.5)
    t = ext.flash_attn_bwd_timing(False).tolist()
    out = {"kernel": "attention_bwd_phases", "batch": b, "heads": h, "seq": s, "head_dim": d}
    for row, name in zip(t, ("dkv_pass", "dq_pass")):
        steps = max(row[14], 1)
        out[name] = {"cycles_per_step": round(row[1] / steps, 1),
                     **{n: round(row[i] / steps, 1) for i, n in enumerate(names) if i not in (0, 1, 14)}}
    return out


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="visionrl_b200.ops.microbench")
    parser.add_argument("--iters", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--no-flush", action="store_true")
    parser.add_argument("--peak-tflops", type=float, default=0.0)
    parser.add_argument("--peak-gbs", type=float, default=0.0)
    sub = parser.add_subparsers(dest="kernel", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=9424)
    g.add_argument("--n", type=int, default=6144)
    g.add_argument("--k", type=int, default=1536)
    g.add_argument("--act", default="none", choices=["none", "gelu", "silu"])
    g.add_argument("--bias", action="store_true")
    g.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"],
                   help="nt: x @ W.T (forward); nn: dY @ W (input gradient); tn: dY.T @ X (weight gradient)")
    g.add_argument("--skip-lib", action="store_true")
    g.add_argument("--skip-check", action="store_true")
    g.set_defaults(fn=bench_gemm)
    s = sub.add_parser("sde")
    s.add_argument("--batch", type=int, default=64)
    s.add_argument("--elems", type=int, default=898560)
    s.set_defaults(fn=bench_sde)
    n = sub.add_parser("adaln")
    n.add_argument("--batch", type=int, default=16)
    n.add_argument("--seq", type=int, default=1024)
    n.add_argument("--dim", type=int, default=1536)
    n.set_defaults(fn=bench_adaln)
    rw = sub.add_parser("rowwise")
    rw.add_argument("--batch", type=int, default=8)
    rw.add_argument("--seq", type=int, default=1024)
    rw.add_argument("--dim", type=int, default=1536)
    rw.add_argument("--heads", type=int, default=24)
    rw.set_defaults(fn=bench_rowwise)
    dc = sub.add_parser("decode")
    dc.add_argument("--rows", type=int, default=32)
    dc.add_argument("--dim", type=int, default=2048)
    dc.add_argument("--heads", type=int, default=16)
    dc.add_argument("--ffn", type=int, default=5632)
    dc.add_argument("--length", type=int, default=640)
    dc.add_argument("--rank", type=int, default=32)
    dc.set_defaults(fn=bench_decode)
    t = sub.add_parser("attention")
    t.add_argument("--batch", type=int, default=16)
    t.add_argument("--heads", type=int, default=24)
    t.add_argument("--seq", type=int, default=1178)
    t.add_argument("--head-dim", type=int, default=64)
    t.add_argument("--backward", action="store_true")
    t.add_argument("--causal", action="store_true")
    t.add_argument("--variant", type=int, default=0,
                   help="forward kernel: 0 default for the shape, 1 register-accumulating, 2 lazy-rescale")
    t.set_defaults(fn=bench_attention)
    tp = sub.add_parser("attention_phases")
    tp.add_argument("--batch", type=int, default=16)
    tp.add_argument("--heads", type=int, default=24)
    tp.add_argument("--seq", type=int, default=1178)
    tp.add_argument("--head-dim", type=int, default=64)
    tp.set_defaults(fn=bench_attention_phases)
    mp = sub.add_parser("mma_issue")
    mp.add_argument("--groups", type=int, default=256)
    mp.set_defaults(fn=bench_mma_issue)
    args = parser.parse_args(argv)
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    print(json.dumps(args.fn(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
