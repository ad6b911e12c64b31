"""``python -m renee_b200.utils.roofline [--peaks MEASURED_PEAKS.json] [--repeats 20]``: per-kernel roofline
report on one GPU.

Times every hand-written kernel of the training step in isolation at the headline benchmark's shapes
(encoder: 8192 tokens = 256 sequences x 32, H = 768, F = 3072, 12 heads; classifier: B = 256, D = 768, one
16384-label chunk; AdamW over 66.4 M parameters; top-100 of 16384 logits x 256 rows) with CUDA events, after
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


def main(argv=None) -> None:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, root)
    from renee_b200 import ops
    from renee_b200.ops import cuda as cu
    from renee_b200.optim.hparams import HP, HyperParams

    ap = argparse.ArgumentParser()
    ap.add_argument("--peaks", default=os.path.join(root, "MEASURED_PEAKS.json"))
    ap.add_argument("--repeats", type=int, default=20)
    a = ap.parse_args(argv)
    if os.path.exists(a.peaks):
        pk = json.load(open(a.peaks))
        hbm, tf, src = float(pk["hbm_gbs"]), float(pk["bf16_tflops"]), "measured"
    else:
        hbm, tf, src = 6650.0, 1590.0, "fallback"
    dev = torch.device("cuda", 0)
    dt = torch.bfloat16
    T, H, F, nh = 8192, 768, 3072, 12
    NS = 6                                    # buffer sets: 6 x (>= 25 MB per operand) exceeds the 126 MB L2
    rng = ops.StepRNG(1, torch.tensor([1], dtype=torch.int32, device=dev))
    rn = lambda *s, n=NS: [torch.randn(*s, device=dev).to(dt) for _ in range(n)]
    em = lambda *s, n=NS: [torch.empty(*s, device=dev, dtype=dt) for _ in range(n)]
    rows = []

    def add(name, us, nbytes, flops=0.0):
        floor = max(nbytes / (hbm * 1e9), flops / (tf * 1e12)) * 1e6
        rows.append(dict(kernel=name, us=round(us, 2), gbs=round(nbytes / us / 1e3, 1),
                         tflops=round(flops / us / 1e6, 1), roofline_us=round(floor, 2),
                         fraction=round(floor / us, 3)))

    # ---- encoder element-wise kernels
    x, res, pre, y = rn(T, H), rn(T, H), em(T, H), em(T, H)
    gam, bet, bias = (torch.ones(H, device=dev, dtype=dt), torch.zeros(H, device=dev, dtype=dt),
                      torch.zeros(H, device=dev, dtype=dt))
    mean, rstd = torch.zeros(T, device=dev), torch.ones(T, device=dev)
    dg, db, dbi = [torch.empty(H, device=dev, dtype=dt) for _ in range(3)]
    us = _time_us(lambda i: ops.bias_dropout_add_ln_fwd(x[i], bias, res[i], gam, bet, 1e-12, 0.1, rng, 3, y[i], pre[i],
                                                        mean, rstd), NS, a.repeats)
    add("bias_dropout_add_ln_fwd", us, 4 * T * H * 2)
    us = _time_us(lambda i: ops.bias_dropout_add_ln_bwd(x[i], res[i], gam, mean, rstd, 0.1, rng, 3, dg, db, dbi,
                                                        pre[i], y[i]), NS, a.repeats)
    add("bias_dropout_add_ln_bwd", us, 4 * T * H * 2)
    del x, res, pre, y
    xf, da, of = rn(T, F, n=4), rn(T, F, n=4), em(T, F, n=4)
    bF, dbF = torch.zeros(F, device=dev, dtype=dt), torch.empty(F, device=dev, dtype=dt)
    us = _time_us(lambda i: ops.bias_gelu_fwd(xf[i], bF, of[i]), 4, a.repeats)
    add("bias_gelu_fwd", us, 2 * T * F * 2)
    us = _time_us(lambda i: ops.bias_gelu_bwd(da[i], xf[i], bF, dbF, of[i]), 4, a.repeats)
    add("bias_gelu_bwd", us, 3 * T * F * 2)
    del xf, da, of
    # ---- attention, 256 x 32 tokens and 64 x 128 tokens
    qkv, ctx, dqkv = rn(T, 3 * H), em(T, H), em(T, 3 * H)
    bq, dbq = torch.zeros(3 * H, device=dev, dtype=dt), torch.empty(3 * H, device=dev, dtype=dt)
    for b_, S_ in ((256, 32), (64, 128)):
        mask = torch.ones(b_, S_, dtype=torch.int32, device=dev)
        ws = [ops.attention_workspace(b_, S_, nh, dev, dt) for _ in range(NS)]
        pbytes = b_ * nh * S_ * S_ * 2
        fl = 4.0 * b_ * nh * S_ * S_ * (H // nh)
        us = _time_us(lambda i: ops.attention_fwd(qkv[i], bq, mask, nh, 0.1, rng, 4, ctx[i], ws[i]), NS, a.repeats)
        add(f"attention_fwd S={S_}", us, T * 3 * H * 2 + T * H * 2 + pbytes, fl)
        us = _time_us(lambda i: ops.attention_bwd(ctx[i], qkv[i], bq, mask, nh, 0.1, rng, 4, ws[i], dqkv[i], dbq),
                      NS, a.repeats)
        add(f"attention_bwd S={S_}", us, 2 * T * 3 * H * 2 + T * H * 2 + pbytes, 2.5 * fl)
        del ws
    del qkv, ctx, dqkv
    # ---- classifier: one 16384-label chunk
    B, D, L = 256, 768, 16384
    X = (torch.randn(B, D, device=dev) * 0.5).half()
    W = [(torch.randn(L, D, device=dev) * 0.05).half() for _ in range(NS)]
    M = [torch.zeros(L, D, device=dev, dtype=torch.float16) for _ in range(NS)]
    Gt = [torch.zeros(L, B, dtype=torch.float16, device=dev) for _ in range(NS)]
    dX = torch.zeros(B, D, device=dev)
    hp = HyperParams(dev)
    hp.buf[HP.LR_XFC] = 1e-3
    hp.buf[HP.LR_ENC] = 1e-5
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    gemm = 2.0 * B * L * D
    us = _time_us(lambda i: cu.xfc_logits_grad(W[i], X, Gt[i], B, zero, zero, zero, 0), NS, a.repeats)
    add("xfc_logits_grad (tcgen05)", us, L * D * 2 + L * B * 2 + B * D * 2, gemm)
    splits = cu.dx_splits(B, D, L)
    us = _time_us(lambda i: cu.xfc_dx(Gt[i], B, W[i], B, dX, hp.buf, splits), NS, a.repeats)
    add("xfc_dx (tcgen05, split-K)", us, L * D * 2 + L * B * 2 + B * D * 4, gemm)
    us = _time_us(lambda i: cu.xfc_dw_sgd(Gt[i], B, X, W[i], M[i], hp.buf, 0.9, 1e-4), NS, a.repeats)
    add("xfc_dw_sgd (tcgen05 + TMA epilogue)", us, 4 * L * D * 2 + L * B * 2 + B * D * 2, gemm)
    Zt = [torch.empty(B, L, device=dev) for _ in range(NS)]
    ov, oi = torch.empty(B, 100, device=dev), torch.empty(B, 100, dtype=torch.int32, device=dev)
    us = _time_us(lambda i: cu.xfc_logits_grad(W[i], X, None, L, None, None, None, 0, raw_out=Zt[i]), NS, a.repeats)
    add("xfc_logits raw (tcgen05)", us, L * D * 2 + B * L * 4 + B * D * 2, gemm)
    for z in Zt:
        z.normal_()
    us = _time_us(lambda i: cu.topk_rows(Zt[i], L, 100, 0, ov, oi), NS, a.repeats)
    add("topk_rows k=100", us, B * L * 4)
    del W, M, Gt, Zt
    # ---- AdamW over the encoder's flat buffers (larger than L2 by itself)
    n = 66_400_000 // 1024 * 1024
    p32, am, av = torch.zeros(n, device=dev), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    g, p16 = torch.zeros(n, device=dev, dtype=dt), torch.zeros(n, device=dev, dtype=dt)
    us = _time_us(lambda i: ops.adamw_step(p32, am, av, g, p16, hp, 0.9, 0.999, 1e-6, 0.01, n // 2), 1, a.repeats)
    add("adamw (66.4 M parameters)", us, n * 28)
    cu.check_status()
    print(json.dumps({"peaks": {"source": src, "hbm_gbs": hbm, "bf16_tflops": tf}, "kernels": rows}))
    print(f"| kernel | µs | GB/s | TFLOP/s | roofline µs | fraction of {src} |\n|---|---|---|---|---|---|")
    for r in rows:
        print(f"| {r['kernel']} | {r['us']} | {r['gbs']} | {r['tflops']} | {r['roofline_us']} | {r['fraction']} |")


if __name__ == "__main__":
    main()
