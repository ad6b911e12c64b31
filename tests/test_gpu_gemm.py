"""The tcgen05 encoder GEMMs (``ops/csrc/gemm.cu``) against plain PyTorch fp32 math of the same op: every
layout (forward NT, data-gradient NN, split-K weight-gradient TN), every fused epilogue, ragged row counts,
all three N tiles; then the flat encoder engine on the own GEMMs against the same engine on library GEMMs."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

from renee_b200 import ops
from renee_b200.ops import reference as ref


def dev():
    return torch.device("cuda", 0)


def cu():
    from renee_b200.ops import cuda
    return cuda


def _rng(seed=4321):
    return ops.StepRNG(seed, torch.tensor([seed], dtype=torch.int32, device=dev()))


def _rel(got, want):
    """Largest error relative to the scale of the reference (a GEMM output's entries share one scale)."""
    return float((got.float() - want).abs().max() / want.abs().max().clamp_min(1e-6))


SHAPES = [(1024, 768, 2304), (8192, 768, 768), (1024, 768, 3072), (8192, 3072, 768), (1000, 768, 768), (77, 128, 512),
          (333, 512, 128), (129, 64, 64)]


NCTA = [0, 1, 2]       # 0: the library chooses; 1: one CTA per 128-row tile; 2: a CTA pair (cta_group::2) per 256-row tile


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,K,N", SHAPES)
@pytest.mark.parametrize("bn,ncta", [(0, 0), (64, 1), (128, 1), (256, 1), (128, 2), (256, 2)])
def test_linear_fwd_store(dt, T, K, N, bn, ncta):
    if bn and (T > 2000 or dt == torch.float16) and not (bn == 256 and N >= 768):
        pytest.skip("forced tile sizes are covered on the small shapes")
    torch.manual_seed(T + K)
    x = torch.randn(T, K, device=dev()).to(dt)
    W = (torch.randn(N, K, device=dev()) * 0.05).to(dt)
    out = torch.full((T, N), 7.0, device=dev(), dtype=dt)
    cu().linear_fwd(x, W, out, bn=bn, ncta=ncta)
    want = x.float() @ W.float().t()
    assert _rel(out, want) < 1e-2
    cu().check_status()


@pytest.mark.parametrize("ncta", NCTA)
@pytest.mark.parametrize("T,K,N", [(1024, 768, 3072), (8192, 768, 3072), (200, 128, 512)])
def test_linear_fwd_bias_gelu(T, K, N, ncta):
    dt = torch.bfloat16
    torch.manual_seed(1)
    x = torch.randn(T, K, device=dev()).to(dt)
    W = (torch.randn(N, K, device=dev()) * 0.05).to(dt)
    b = torch.randn(N, device=dev()).to(dt)
    act, pre = torch.empty(T, N, device=dev(), dtype=dt), torch.empty(T, N, device=dev(), dtype=dt)
    cu().linear_fwd(x, W, act, "bias_gelu", bias=b, pre_out=pre, ncta=ncta)
    f = x.float() @ W.float().t() + b.float()
    assert _rel(pre, f) < 1e-2
    want = torch.nn.functional.gelu(pre.float())          # GELU of the stored (rounded) pre-activation
    torch.testing.assert_close(act.float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("ncta", NCTA)
@pytest.mark.parametrize("p", [0.0, 0.1])
@pytest.mark.parametrize("T,K,N", [(1024, 768, 768), (8192, 3072, 768), (1000, 3072, 768), (90, 512, 128)])
def test_linear_fwd_bias_dropout_resid_then_ln(T, K, N, p, ncta):
    """The GEMM epilogue + the LayerNorm kernel equal the stand-alone bias+dropout+residual+LayerNorm op applied
    to the plain product, with the SAME dropout mask (the backward pass regenerates it from the element index)."""
    dt = torch.bfloat16
    torch.manual_seed(2)
    x = torch.randn(T, K, device=dev()).to(dt)
    W = (torch.randn(N, K, device=dev()) * 0.03).to(dt)
    b, gam, bet = [torch.randn(N, device=dev()).to(dt) for _ in range(3)]
    res = torch.randn(T, N, device=dev()).to(dt)
    rng = _rng()
    pre = torch.empty(T, N, device=dev(), dtype=dt)
    cu().linear_fwd(x, W, pre, "bias_dropout_resid", bias=b, resid=res, p=p, rng=rng, stream=11, ncta=ncta)
    prod = (x.float() @ W.float().t())
    yr, prer, mr, rr = ref.bias_dropout_add_ln_fwd(prod, b.float(), res.float(), gam.float(), bet.float(), 1e-12, p,
                                                   rng.seed, 11)
    torch.testing.assert_close(pre.float(), prer, rtol=2e-2, atol=3e-2)
    if p > 0:       # identical mask: dropped elements are exactly the residual
        dropped = ~ops.keep_mask(rng.seed, 11, (T, N), p, dev())
        assert torch.equal(pre[dropped], res[dropped])
    y = torch.empty_like(pre)
    mean, rstd = torch.empty(T, device=dev()), torch.empty(T, device=dev())
    cu().ln_fwd(pre, gam, bet, 1e-12, y, mean, rstd)
    pf = pre.float()
    mu = pf.mean(1)
    var = pf.var(1, unbiased=False)
    torch.testing.assert_close(mean, mu, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(rstd, (var + 1e-12).rsqrt(), rtol=1e-3, atol=1e-3)
    want = (pf - mu[:, None]) * (var + 1e-12).rsqrt()[:, None] * gam.float() + bet.float()
    torch.testing.assert_close(y.float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("ncta", NCTA)
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,N,K", [(1024, 768, 768), (8192, 2304, 768), (1000, 3072, 768), (8192, 768, 3072), (77, 512, 128)])
def test_linear_dgrad_store_and_add(dt, T, N, K, ncta):
    torch.manual_seed(3)
    dy = torch.randn(T, N, device=dev()).to(dt)
    W = (torch.randn(N, K, device=dev()) * 0.05).to(dt)
    res = torch.randn(T, K, device=dev()).to(dt)
    want = dy.float() @ W.float()
    out = torch.empty(T, K, device=dev(), dtype=dt)
    cu().linear_dgrad(dy, W, out, ncta=ncta)
    assert _rel(out, want) < 1e-2
    cu().linear_dgrad(dy, W, out, "add", resid=res, ncta=ncta)
    assert _rel(out, want + res.float()) < 1e-2


@pytest.mark.parametrize("ncta", NCTA)
@pytest.mark.parametrize("T,N,K", [(1024, 768, 3072), (8192, 768, 3072), (300, 128, 512)])
def test_linear_dgrad_gelu_bwd_with_bias_gradient(T, N, K, ncta):
    dt = torch.bfloat16
    torch.manual_seed(4)
    dy = torch.randn(T, N, device=dev()).to(dt)
    W = (torch.randn(N, K, device=dev()) * 0.05).to(dt)
    f = torch.randn(T, K, device=dev()).to(dt)
    out = torch.empty(T, K, device=dev(), dtype=dt)
    dbias = torch.full((K,), 9.0, device=dev(), dtype=dt)
    cu().linear_dgrad(dy, W, out, "gelu_bwd", pre=f, dbias=dbias, ncta=ncta)
    ff = f.float().requires_grad_(True)
    torch.nn.functional.gelu(ff).backward(dy.float() @ W.float())
    want = ff.grad
    assert _rel(out, want) < 1.5e-2
    torch.testing.assert_close(dbias.float(), out.float().sum(0), rtol=2e-2, atol=2e-2 * (T ** 0.5))
    # inside a deferred-column plan the sums land in the plan's accumulators and one finalize converts them
    plan = cu().DeferredColumns(dev(), dt)
    dbias2 = torch.zeros(K, device=dev(), dtype=dt)
    with cu().deferred_columns(plan):
        cu().linear_dgrad(dy, W, out, "gelu_bwd", pre=f, dbias=dbias2, ncta=ncta)
    plan.finalize()
    torch.testing.assert_close(dbias2.float(), dbias.float(), rtol=1e-2, atol=1e-2 * (T ** 0.5))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,N,K", [(1024, 768, 768), (8192, 768, 768), (8192, 2304, 768), (1024, 3072, 768), (8192, 768, 3072),
                                   (1000, 768, 3072), (77, 128, 512), (4096, 64, 64)])
@pytest.mark.parametrize("ncta", NCTA)
def test_linear_wgrad_split_k(dt, T, N, K, ncta):
    torch.manual_seed(5)
    dy = (torch.randn(T, N, device=dev()) * 0.1).to(dt)
    x = torch.randn(T, K, device=dev()).to(dt)
    dW = torch.full((N, K), 3.0, device=dev(), dtype=dt)
    want = dy.float().t() @ x.float()
    for _ in range(2):           # the scratch and the counters are left zero: a second call gives the same result
        cu().linear_wgrad(dy, x, dW, ncta=ncta)
        assert _rel(dW, want) < 1e-2
    sk = cu()._SK.get(0)
    if sk is not None and sk.buf is not None:
        assert float(sk.buf.abs().max()) == 0.0 and int(sk.counters.abs().max()) == 0
    cu().check_status()


def _engine(own: bool, S=32, b=24):
    from renee_b200.models.encoder import EncoderConfig
    from renee_b200.models.flat_encoder import FlatEncoder
    os.environ["RENEE_B200_OWN_GEMM"] = "1" if own else "0"
    try:
        enc = FlatEncoder(EncoderConfig(n_layers=2), dev(), torch.bfloat16, "cls", 0, seed=3)
    finally:
        os.environ.pop("RENEE_B200_OWN_GEMM", None)
    assert enc.own_gemm == own
    return enc


def test_flat_encoder_picks_the_gemm_path_by_token_count():
    """Default mode: library GEMMs below OWN_GEMM_MIN_TOKENS tokens per step, the own kernels from there on."""
    from renee_b200.models.encoder import EncoderConfig
    from renee_b200.models import flat_encoder as fe
    from renee_b200.ops import StepRNG
    os.environ.pop("RENEE_B200_OWN_GEMM", None)
    enc = fe.FlatEncoder(EncoderConfig(n_layers=1), dev(), torch.bfloat16, "cls", 0, seed=3)
    rng = StepRNG(1, torch.tensor([1], dtype=torch.int32, device=dev()))
    for b, S in ((8, 32), (fe.OWN_GEMM_MIN_TOKENS // 32, 32)):
        ids = torch.randint(1000, 30000, (b, S), device=dev(), dtype=torch.int32)
        mask = torch.ones(b, S, device=dev(), dtype=torch.int32)
        out = enc.forward(ids, mask, rng, train=False)
        assert enc.own_gemm == (b * S >= fe.OWN_GEMM_MIN_TOKENS)
        assert torch.isfinite(out).all()
    cu().check_status()


@pytest.mark.parametrize("S,b", [(32, 24), (20, 7)])
def test_flat_encoder_on_own_gemms_matches_library_gemms(S, b):
    """Same weights, same dropout seeds: forward output and every parameter gradient agree to 16-bit tolerance."""
    a, c = _engine(True), _engine(False)
    torch.manual_seed(0)
    ids = torch.randint(1000, 30000, (b, S), device=dev(), dtype=torch.int32)
    lens = torch.randint(3, S + 1, (b,), device=dev())
    mask = (torch.arange(S, device=dev())[None] < lens[:, None]).to(torch.int32)
    ids = ids * mask
    d_emb = torch.randn(b, 768, device=dev()) * 0.1
    outs, grads = [], []
    for enc in (a, c):
        rng = _rng(99)
        e = enc.forward(ids, mask, rng, train=True).clone()
        enc.backward(d_emb)
        outs.append(e)
        grads.append(enc.g.float().clone())
    torch.cuda.synchronize()
    cu().check_status()
    torch.testing.assert_close(outs[0], outs[1], rtol=3e-2, atol=3e-2)
    ga, gc = grads
    assert torch.isfinite(ga).all()
    # per-parameter comparison at the scale of each gradient
    for name, slot in a.slots.items():
        x, y = ga[slot.offset: slot.offset + slot.numel], gc[slot.offset: slot.offset + slot.numel]
        scale = float(y.abs().max().clamp_min(1e-4))
        err = float((x - y).abs().max())
        assert err <= 6e-2 * scale + 1e-3, f"{name}: max err {err} at scale {scale}"


@pytest.mark.parametrize("B,D,Ls,k", [(256, 768, 16384, 5), (100, 128, 40000, 8), (512, 768, 5003 * 8, 3), (33, 64, 1000, 5)])
def test_fused_topk8_equals_torch_topk(B, D, Ls, k):
    """The running top-8 in the GEMM epilogue (logits never written) against ``torch.topk`` of the fp32 product of
    the same fp16 operands: same values; same labels wherever the k-th value is not tied."""
    torch.manual_seed(B + Ls)
    X = (torch.randn(B, D, device=dev()) * 0.5).half()
    W = (torch.randn(Ls, D, device=dev()) * 0.05).half()
    v, i = cu().xfc_topk8(W, X, k)
    Z = X.float() @ W.float().t()
    vr, ir = torch.topk(Z, k, dim=1)
    torch.testing.assert_close(v, vr, rtol=2e-3, atol=2e-3)           # fp32 accumulation order differs
    assert int(i.max()) < Ls and int(i.min()) >= 0
    # the labels are the right ones: their exact logits equal the reference top-k values
    torch.testing.assert_close(torch.gather(Z, 1, i), vr, rtol=2e-3, atol=2e-3)
    assert (i == ir).float().mean() > 0.98
    cu().check_status()
