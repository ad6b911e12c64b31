"""Loss-skipping classifier step vs dense BCEWithLogits(sum) + autograd + torch SGD
(the oracle is the math of the reference's default path, dl_base.py:274-295)."""
import torch

from renee_b200.models.xfc import XFCClassifier
from renee_b200.optim.hparams import HP, HyperParams
from renee_b200.ops import reference as ref


def _problem(B=24, D=64, Ls=400, seed=0):
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(B, D, generator=g) * 0.5
    rows = torch.randint(0, B, (60,), generator=g)
    labels = torch.randint(0, Ls, (60,), generator=g)
    pairs = torch.unique(torch.stack([labels, rows], 1), dim=0)      # sorted by label, deduplicated
    return X, pairs[:, 1].int().contiguous(), pairs[:, 0].int().contiguous()


def _oracle(W0, X, rows, labels, lr, mo, wd, scale, steps=2):
    W = torch.nn.Parameter(W0.clone().double())
    opt = torch.optim.SGD([W], lr=lr, momentum=mo, weight_decay=wd)
    Xd = X.double().requires_grad_(True)
    out = None
    for _ in range(steps):
        opt.zero_grad(); Xd.grad = None
        Z = Xd @ W.t()
        Y = torch.zeros_like(Z); Y[rows.long(), labels.long()] = 1.0
        loss = torch.nn.functional.binary_cross_entropy_with_logits(Z, Y, reduction="sum")
        loss.backward()
        out = (loss.detach(), Xd.grad.clone() * scale)
        opt.step()
    return W.detach(), out


def test_step_matches_autograd_two_steps_with_chunks():
    X, rows, labels = _problem()
    xfc = XFCClassifier(400, 64, "cpu", fp16=False, seed=3, max_batch=24, accum=3)
    assert xfc.chunk < 400      # exercises label chunking (split accumulation)
    W0 = xfc.W.clone()
    hp = HyperParams("cpu", init_scale=4096.0)
    hp.buf[HP.LR_XFC] = 0.05
    dX = torch.zeros(24, 64)
    for _ in range(2):
        loss = xfc.step(X, rows, labels, rows.numel(), dX, hp, 0.9, 1e-2, want_loss=True)
    W_ref, (loss_ref, dX_ref) = _oracle(W0, X, rows, labels, 0.05, 0.9, 1e-2, 4096.0)
    torch.testing.assert_close(xfc.W.double(), W_ref, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(dX.double(), dX_ref, rtol=1e-4, atol=1e-2)
    torch.testing.assert_close(loss.double(), loss_ref, rtol=1e-5, atol=1e-3)


def test_duplicates_subtract_once_and_empty_positives():
    X, rows, labels = _problem()
    W = torch.randn(400, 64) * 0.02
    Gt, _ = ref.xfc_logit_grad(X, W, torch.cat([rows, rows[:5]]), torch.cat([labels, labels[:5]]))
    Gt1, _ = ref.xfc_logit_grad(X, W, rows, labels)
    torch.testing.assert_close(Gt, Gt1)
    Gt0, _ = ref.xfc_logit_grad(X, W, rows[:0], labels[:0])
    torch.testing.assert_close(Gt0, torch.sigmoid(W @ X.t()))


def test_fp16_storage_tracks_fp32_master():
    X, rows, labels = _problem()
    a = XFCClassifier(400, 64, "cpu", fp16=True, seed=3, max_batch=24)
    b = XFCClassifier(400, 64, "cpu", fp16=False, seed=3, max_batch=24)
    hp = HyperParams("cpu", init_scale=1.0)
    hp.buf[HP.LR_XFC] = 0.05
    dXa, dXb = torch.zeros(24, 64), torch.zeros(24, 64)
    for _ in range(3):
        a.step(X.half(), rows, labels, rows.numel(), dXa, hp, 0.9, 1e-4)
        b.step(X, rows, labels, rows.numel(), dXb, hp, 0.9, 1e-4)
    assert a.W.dtype == torch.float16 and a.M.dtype == torch.float16
    torch.testing.assert_close(a.W.float(), b.W, rtol=2e-2, atol=2e-3)
    torch.testing.assert_close(dXa, dXb, rtol=5e-2, atol=5e-2)


def test_weight_init_is_independent_of_world_size():
    full = XFCClassifier(256, 16, "cpu", fp16=False, rank=0, seed=9).W
    parts = [XFCClassifier(64, 16, "cpu", fp16=False, rank=r, seed=9).W for r in range(4)]
    torch.testing.assert_close(torch.cat(parts), full)


def test_topk_chunked_equals_full():
    X, _, _ = _problem()
    xfc = XFCClassifier(400, 64, "cpu", fp16=False, seed=3, max_batch=24, accum=3)
    v, i = xfc.topk(X, 7)
    vr, ir = torch.topk(X @ xfc.W.t(), 7, dim=1)
    torch.testing.assert_close(v, vr); assert torch.equal(i, ir)


def test_fp16_weight_storage_drift_against_fp32_masters_late_in_the_schedule():
    """fp16 storage of W and momentum vs the reference's fp32 masters (dl_base.py:185, 562) over 400 steps at
    a learning rate typical of the end of the cosine schedule, where an update lr*M is far below half an fp16
    ulp of W (|W| ~ 0.03: ulp 1.5e-5).  Round-to-nearest loses most of the update; stochastic rounding (the
    default, same arithmetic as the dW kernel's epilogue) follows the fp32 trajectory in expectation."""
    torch.manual_seed(0)
    Ls, D, B, steps = 256, 64, 32, 400
    lr, mo, wd = 2e-5, 0.9, 1e-4
    W0 = (torch.randn(Ls, D) * 0.03)
    W32, M32 = W0.clone(), torch.zeros(Ls, D)
    Wrn, Mrn = W0.half(), torch.zeros(Ls, D, dtype=torch.float16)
    Wsr, Msr = W0.half(), torch.zeros(Ls, D, dtype=torch.float16)
    start = Wrn.float().clone()
    for t in range(steps):
        X = torch.randn(B, D).abs() * 0.5                      # one-signed features: every weight drifts one way
        Gt = (torch.rand(Ls, B) * 0.02)                       # sigmoid(z) - y of mostly-negative labels: small, one-signed
        Gt[torch.randint(0, Ls, (8,)), torch.randint(0, B, (8,))] -= 1.0
        ref.xfc_dw_sgd(Gt, X, W32, M32, lr, mo, wd)
        ref.xfc_dw_sgd(Gt.half(), X.half(), Wrn, Mrn, lr, mo, wd)
        ref.xfc_dw_sgd(Gt.half(), X.half(), Wsr, Msr, lr, mo, wd, sr_seed=1000 + t)
    moved = (W32 - start).abs().mean()                        # how far fp32 masters travelled
    err_rn = (Wrn.float() - W32).abs().mean()
    err_sr = (Wsr.float() - W32).abs().mean()
    # stochastic rounding stays within rounding noise of the fp32 trajectory; round-to-nearest falls behind by a
    # large part of the distance travelled
    assert err_sr < 0.35 * moved, (float(err_sr), float(moved))
    assert err_rn > 1.3 * err_sr, (float(err_rn), float(err_sr))
    # and the MEAN displacement (what matters for tail labels) is kept by SR, largely lost by RN
    d32, drn, dsr = (W32 - start).mean(), (Wrn.float() - start).mean(), (Wsr.float() - start).mean()
    assert abs(dsr - d32) < 0.2 * abs(d32)
    assert abs(drn - d32) > 3.0 * abs(dsr - d32)
