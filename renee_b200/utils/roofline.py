"""``python -m renee_b200.utils.roofline [--peaks MEASURED_PEAKS.json] [--repeats 20] [--only SUBSTRING]``:
per-kernel roofline report on one GPU.  ``--case NAME --launches N`` instead launches one case N times and
exits (a small, self-ending workload to put under a profiler); ``--list`` prints the case names.

Times every hand-written kernel of the training step in isolation at the headline benchmark's shapes
(encoder: 8192 tokens = 256 sequences x 32 — and 1024 tokens, one rank's share at 8 GPUs — H = 768, F = 3072,
12 heads; classifier: B = 256, D = 768, one 16384-label chunk, and B = 512 with the 163840-label shard of the
1.3 M-label configuration; AdamW over 66.4 M parameters; top-100 of 16384 logits x 256 rows) with CUDA events, after
warm-up, rotating through enough buffer sets that consecutive launches never find their inputs in L2, and
prints for each: microseconds, achieved GB/s and TFLOP/s from the ALGORITHMIC bytes and FLOPs (every operand
counted once), and the fraction of the roofline max(bytes / copy bandwidth, FLOPs / GEMM rate) built from the
measured peaks file (``hbm_gbs``, ``bf16_tflops`` burst: the kernels are timed in isolation).  Without the file
the fallback 6650 GB/s / 1590 TFLOP/s is used and the header says so.

The reference has no profiling tooling (a commented-out profiler import, main.py:13).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def _time_us(fn, n_sets: int, repeats: int) -> float:
    for i in range(max(3, n_sets)):
        fn(i % n_sets)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(repeats):
        fn(i % n_sets)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / repeats * 1e3


def _cases(dev, dt, NS):
    """Yields ``(name, make)``; ``make()`` allocates the case's buffers and returns ``(fn(i), n_sets, bytes, flops)``."""
    from renee_b200 import ops
    from renee_b200.ops import cuda as cu
    from renee_b200.optim.hparams import HP, HyperParams

    T, H, F, nh = 8192, 768, 3072, 12
    rng = ops.StepRNG(1, torch.tensor([1], dtype=torch.int32, device=dev))
    rn = lambda *s, n=NS, sc=1.0: [(torch.randn(*s, device=dev) * sc).to(dt) for _ in range(n)]
    em = lambda *s, n=NS: [torch.empty(*s, device=dev, dtype=dt) for _ in range(n)]
    vec = lambda n, v=0.0: torch.full((n,), v, device=dev, dtype=dt)

    # ---- encoder GEMMs (tcgen05, fused epilogues) at T = 8192 and at the 8-GPU share T = 1024
    def gemm_fwd(Tn, K, N, epi):
        def make():
            x, W, out = rn(Tn, K), rn(N, K, n=1, sc=0.05)[0], em(Tn, N)
            extra = 0
            if epi == "store":
                fn = lambda i: cu.linear_fwd(x[i], W, out[i])
            elif epi == "bias_gelu":
                pre = em(Tn, N)
                extra = Tn * N * 2
                b = vec(N)
                fn = lambda i: cu.linear_fwd(x[i], W, out[i], "bias_gelu", bias=b, pre_out=pre[i])
            else:
                res, b = rn(Tn, N), vec(N)
                extra = Tn * N * 2
                fn = lambda i: cu.linear_fwd(x[i], W, out[i], "bias_dropout_resid", bias=b, resid=res[i], p=0.1, rng=rng,
                                             stream=3)
            return fn, NS, (Tn * K + N * K + Tn * N) * 2 + extra, 2.0 * Tn * K * N
        return make

    def gemm_dgrad(Tn, N, K, epi):
        def make():
            dy, W, out = rn(Tn, N), rn(N, K, n=1, sc=0.05)[0], em(Tn, K)
            extra = 0
            if epi == "store":
                fn = lambda i: cu.linear_dgrad(dy[i], W, out[i])
            elif epi == "add":
                res = rn(Tn, K)
                extra = Tn * K * 2
                fn = lambda i: cu.linear_dgrad(dy[i], W, out[i], "add", resid=res[i])
            else:
                f, db = rn(Tn, K), vec(K)
                extra = Tn * K * 2
                # as in the engine's backward pass: the bias-gradient column sums only accumulate here, one launch
                # at the end of the pass converts all of them
                plan = cu.DeferredColumns(dev, dt)

                def fn(i):
                    with cu.deferred_columns(plan):
                        cu.linear_dgrad(dy[i], W, out[i], "gelu_bwd", pre=f[i], dbias=db)
            return fn, NS, (Tn * N + N * K + Tn * K) * 2 + extra, 2.0 * Tn * K * N
        return make

    def gemm_wgrad(Tn, N, K):
        def make():
            dy, x, dW = rn(Tn, N, sc=0.1), rn(Tn, K), em(N, K)
            return (lambda i: cu.linear_wgrad(dy[i], x[i], dW[i])), NS, (Tn * N + Tn * K + N * K) * 2, 2.0 * Tn * K * N
        return make

    def lib_mm(Tn, K, N):
        def make():
            x, W, out = rn(Tn, K), rn(N, K, n=1, sc=0.05)[0], em(Tn, N)
            return (lambda i: torch.mm(x[i], W.t(), out=out[i])), NS, (Tn * K + N * K + Tn * N) * 2, 2.0 * Tn * K * N
        return make

    for Tn in (8192, 1024):
        yield f"gemm fwd qkv store T={Tn}", gemm_fwd(Tn, H, 3 * H, "store")
        yield f"gemm fwd out-proj bias+dropout+resid T={Tn}", gemm_fwd(Tn, H, H, "bdr")
        yield f"gemm fwd ffn1 bias+gelu T={Tn}", gemm_fwd(Tn, H, F, "bias_gelu")
        yield f"gemm fwd ffn2 bias+dropout+resid T={Tn}", gemm_fwd(Tn, F, H, "bdr")
        yield f"gemm dgrad ffn2 gelu_bwd+colsum T={Tn}", gemm_dgrad(Tn, H, F, "gelu_bwd")
        yield f"gemm dgrad ffn1 add T={Tn}", gemm_dgrad(Tn, F, H, "add")
        yield f"gemm dgrad out-proj store T={Tn}", gemm_dgrad(Tn, H, H, "store")
        yield f"gemm dgrad qkv add T={Tn}", gemm_dgrad(Tn, 3 * H, H, "add")
        yield f"gemm wgrad ffn2 [768x3072] T={Tn}", gemm_wgrad(Tn, H, F)
        yield f"gemm wgrad ffn1 [3072x768] T={Tn}", gemm_wgrad(Tn, F, H)
        yield f"gemm wgrad out-proj [768x768] T={Tn}", gemm_wgrad(Tn, H, H)
        yield f"gemm wgrad qkv [2304x768] T={Tn}", gemm_wgrad(Tn, 3 * H, H)
        yield f"library mm qkv (cuBLAS, for comparison) T={Tn}", lib_mm(Tn, H, 3 * H)
        yield f"library mm ffn2 (cuBLAS, for comparison) T={Tn}", lib_mm(Tn, F, H)

    # ---- encoder element-wise kernels
    def ln_fwd_only():
        pre, y = rn(T, H), em(T, H)
        mean, rstd = torch.zeros(T, device=dev), torch.ones(T, device=dev)
        g, b = vec(H, 1.0), vec(H)
        return (lambda i: cu.ln_fwd(pre[i], g, b, 1e-12, y[i], mean, rstd)), NS, 2 * T * H * 2, 0.0
    yield "ln_fwd (LayerNorm of a stored input)", ln_fwd_only

    def ln_fwd():
        x, res, pre, y = rn(T, H), rn(T, H), em(T, H), em(T, H)
        mean, rstd = torch.zeros(T, device=dev), torch.ones(T, device=dev)
        g, b, bias = vec(H, 1.0), vec(H), vec(H)
        return (lambda i: ops.bias_dropout_add_ln_fwd(x[i], bias, res[i], g, b, 1e-12, 0.1, rng, 3, y[i], pre[i], mean,
                                                      rstd)), NS, 4 * T * H * 2, 0.0
    yield "bias_dropout_add_ln_fwd", ln_fwd

    def ln_bwd():
        x, res, pre, y = rn(T, H), rn(T, H), em(T, H), em(T, H)
        mean, rstd = torch.zeros(T, device=dev), torch.ones(T, device=dev)
        g = vec(H, 1.0)
        dg, db, dbi = vec(H), vec(H), vec(H)
        return (lambda i: ops.bias_dropout_add_ln_bwd(x[i], res[i], g, mean, rstd, 0.1, rng, 3, dg, db, dbi, pre[i],
                                                      y[i])), NS, 4 * T * H * 2, 0.0
    yield "bias_dropout_add_ln_bwd", ln_bwd

    def gelu_fwd():
        xf, of = rn(T, F, n=4), em(T, F, n=4)
        bF = vec(F)
        return (lambda i: ops.bias_gelu_fwd(xf[i], bF, of[i])), 4, 2 * T * F * 2, 0.0
    yield "bias_gelu_fwd", gelu_fwd

    def gelu_bwd():
        xf, da, of = rn(T, F, n=4), rn(T, F, n=4), em(T, F, n=4)
        bF, dbF = vec(F), vec(F)
        return (lambda i: ops.bias_gelu_bwd(da[i], xf[i], bF, dbF, of[i])), 4, 3 * T * F * 2, 0.0
    yield "bias_gelu_bwd", gelu_bwd

    # ---- attention, 256 x 32 tokens and 64 x 128 tokens
    for b_, S_ in ((256, 32), (64, 128)):
        def att(direction, b_=b_, S_=S_):
            def make():
                qkv, ctx, dqkv = rn(T, 3 * H), em(T, H), em(T, 3 * H)
                bq, dbq = vec(3 * H), vec(3 * H)
                mask = torch.ones(b_, S_, dtype=torch.int32, device=dev)
                ws = [ops.attention_workspace(b_, S_, nh, dev, dt) for _ in range(NS)]
                pbytes = b_ * nh * S_ * S_ * 2
                fl = 4.0 * b_ * nh * S_ * S_ * (H // nh)
                fwd = lambda i: ops.attention_fwd(qkv[i], bq, mask, nh, 0.1, rng, 4, ctx[i], ws[i])
                if direction == "fwd":
                    return fwd, NS, T * 3 * H * 2 + T * H * 2 + pbytes, fl
                for i in range(NS):
                    fwd(i)
                return (lambda i: ops.attention_bwd(ctx[i], qkv[i], bq, mask, nh, 0.1, rng, 4, ws[i], dqkv[i], dbq)), \
                    NS, 2 * T * 3 * H * 2 + T * H * 2 + pbytes, 2.5 * fl
            return make
        yield f"attention_fwd S={S_}", att("fwd")
        yield f"attention_bwd S={S_}", att("bwd")

    # ---- classifier: one 16384-label chunk at B = 256 and the 163840-label shard of the 1.3 M config at B = 512
    for B, L in ((256, 16384), (512, 163840)):
        D = 768
        ns = NS if L < 100000 else 1          # the large shard exceeds L2 by itself (W alone is 252 MB)
        gemm = 2.0 * B * L * D

        def xfc(kind, B=B, L=L, ns=ns, gemm=gemm):
            def make():
                X = (torch.randn(B, D, device=dev) * 0.5).half()
                W = [(torch.randn(L, D, device=dev) * 0.05).half() for _ in range(ns)]
                Gt = [torch.zeros(L, B, dtype=torch.float16, device=dev) for _ in range(ns)]
                hp = HyperParams(dev)
                hp.buf[HP.LR_XFC] = 1e-3
                zero = torch.zeros(1, dtype=torch.int32, device=dev)
                if kind == "logits":
                    return (lambda i: cu.xfc_logits_grad(W[i], X, Gt[i], B, zero, zero, zero, 0)), ns, \
                        L * D * 2 + L * B * 2 + B * D * 2, gemm
                if kind == "logits2":
                    return (lambda i: cu.xfc_logits_grad_v2(W[i], X, Gt[i], B, zero, zero, zero, 0)), ns, \
                        L * D * 2 + L * B * 2 + B * D * 2, gemm
                if kind == "dx2":
                    dX = torch.zeros(B, D, device=dev)
                    return (lambda i: cu.xfc_dx_v2(Gt[i], B, W[i], B, dX, hp.buf)), ns, \
                        L * D * 2 + L * B * 2 + B * D * 4, gemm
                if kind == "dx":
                    dX = torch.zeros(B, D, device=dev)
                    splits = cu.dx_splits(B, D, L)
                    return (lambda i: cu.xfc_dx(Gt[i], B, W[i], B, dX, hp.buf, splits)), ns, \
                        L * D * 2 + L * B * 2 + B * D * 4, gemm
                if kind in ("dw", "dw2"):
                    M = [torch.zeros(L, D, device=dev, dtype=torch.float16) for _ in range(ns)]
                    v2 = kind == "dw2"
                    return (lambda i: cu.xfc_dw_sgd(Gt[i], B, X, W[i], M[i], hp.buf, 0.9, 1e-4, v2=v2)), ns, \
                        4 * L * D * 2 + L * B * 2 + B * D * 2, gemm
                raise KeyError(kind)
            return make
        yield f"xfc_logits_grad (one tile per CTA) B={B} L={L}", xfc("logits")
        yield f"xfc_logits_grad (persistent CTA pairs) B={B} L={L}", xfc("logits2")
        yield f"xfc_dx (one tile per CTA) B={B} L={L}", xfc("dx")
        yield f"xfc_dx (persistent CTA pairs) B={B} L={L}", xfc("dx2")
        yield f"xfc_dw_sgd (one tile per CTA) B={B} L={L}", xfc("dw")
        yield f"xfc_dw_sgd (persistent CTA pairs) B={B} L={L}", xfc("dw2")

    def topk():
        B, L = 256, 16384
        Zt = [torch.randn(B, L, device=dev) for _ in range(NS)]
        ov, oi = torch.empty(B, 100, device=dev), torch.empty(B, 100, dtype=torch.int32, device=dev)
        return (lambda i: cu.topk_rows(Zt[i], L, 100, 0, ov, oi)), NS, B * L * 4, 0.0
    yield "topk_rows k=100", topk

    def topk_fused():
        # prediction with k = 5 over a 131072-label shard: W is read once, no logits are written
        B, L, D = 256, 131072, 768
        X = torch.randn(B, D, device=dev).half()
        W = [(torch.randn(L, D, device=dev) * 0.05).half() for _ in range(2)]
        return (lambda i: cu.xfc_topk8(W[i % 2], X, 5)), 2, L * D * 2 + B * D * 2, 2.0 * B * L * D
    yield "xfc_topk k=5 fused into the logits GEMM (B=256, L=131072; all its launches)", topk_fused

    def adamw():
        n = 66_400_000 // 1024 * 1024
        p32, am, av = torch.zeros(n, device=dev), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        g, p16 = torch.zeros(n, device=dev, dtype=dt), torch.zeros(n, device=dev, dtype=dt)
        hp = HyperParams(dev)
        hp.buf[HP.LR_ENC] = 1e-5
        return (lambda i: ops.adamw_step(p32, am, av, g, p16, hp, 0.9, 0.999, 1e-6, 0.01, n // 2)), 1, n * 28, 0.0
    yield "adamw (66.4 M parameters)", adamw


def main(argv=None) -> None:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, root)
    from renee_b200.ops import cuda as cu

    ap = argparse.ArgumentParser()
    ap.add_argument("--peaks", default=os.path.join(root, "MEASURED_PEAKS.json"))
    ap.add_argument("--repeats", type=int, default=20)
    ap.add_argument("--only", default="", help="substring: time only the cases whose name contains it")
    ap.add_argument("--case", default="", help="profiling mode: launch the one case with this exact name --launches "
                                               "times (after one warm-up launch) and exit; no timing")
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--list", action="store_true", help="print the case names and exit")
    a = ap.parse_args(argv)
    if os.path.exists(a.peaks):
        pk = json.load(open(a.peaks))
        hbm, tf, src = float(pk["hbm_gbs"]), float(pk["bf16_tflops"]), "measured"
    else:
        hbm, tf, src = 6650.0, 1590.0, "fallback"
    dev = torch.device("cuda", 0)
    dt = torch.bfloat16
    NS = 6                                    # buffer sets: 6 x (>= 12 MB per operand) exceeds the 126 MB L2
    if a.list:
        for name, _ in _cases(dev, dt, NS):
            print(name)
        return
    rows = []
    for name, make in _cases(dev, dt, NS):
        if a.case:
            if name != a.case:
                continue
            fn, ns, _, _ = make()
            fn(0)
            torch.cuda.synchronize()
            for i in range(a.launches):
                fn((i + 1) % ns)
            torch.cuda.synchronize()
            cu.check_status()
            print(f"launched {name!r} {a.launches} times")
            return
        if a.only and a.only not in name:
            continue
        fn, ns, nbytes, flops = make()
        us = _time_us(fn, ns, a.repeats)
        floor = max(nbytes / (hbm * 1e9), flops / (tf * 1e12)) * 1e6
        rows.append(dict(kernel=name, us=round(us, 2), gbs=round(nbytes / us / 1e3, 1),
                         tflops=round(flops / us / 1e6, 1), roofline_us=round(floor, 2),
                         fraction=round(floor / us, 3)))
        del fn
        torch.cuda.empty_cache()
    if a.case:
        raise SystemExit(f"no case named {a.case!r}; see --list")
    cu.check_status()
    print(json.dumps({"peaks": {"source": src, "hbm_gbs": hbm, "bf16_tflops": tf}, "kernels": rows}))
    print(f"| kernel | µs | GB/s | TFLOP/s | roofline µs | fraction of {src} |\n|---|---|---|---|---|---|")
    for r in rows:
        print(f"| {r['kernel']} | {r['us']} | {r['gbs']} | {r['tflops']} | {r['roofline_us']} | {r['fraction']} |")


if __name__ == "__main__":
    main()
