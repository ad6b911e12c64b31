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
