"""Plain PyTorch implementations of every fused op of the package.

These are (a) the numerical oracles the CUDA kernels are tested against, computed in fp32, and
(b) the implementation used for CPU tensors (unit tests, the CPU plumbing configuration).  Each
function documents which sm_100a kernel replaces it on a GPU.

Shapes: ``T = b*S`` tokens, ``H`` hidden, ``F`` FFN width, ``nh`` heads, ``hd = H/nh``.
Dropout masks come from :mod:`renee_b200.ops.rng` so forward and backward (and the kernels) agree.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .rng import keep_mask


def _mask(seed, stream, shape, p, device):
    return keep_mask(seed, stream, shape, p, device=device)


# ----------------------------------------------------------------------------- embeddings + LN
def embed_ln_fwd(ids, word, pos, gamma, beta, eps, S, p, seed, stream, out_dtype):
    """word[ids] + pos[s] → LayerNorm → dropout.  Returns ``(y[T,H], mean[T], rstd[T])``."""
    T = ids.numel()
    x = word[ids.reshape(-1).long()].float() + pos[:S].float().repeat(T // S, 1)
    mean = x.mean(-1)
    var = x.var(-1, unbiased=False)
    rstd = torch.rsqrt(var + eps)
    y = (x - mean[:, None]) * rstd[:, None] * gamma.float() + beta.float()
    if p > 0:
        y = y * _mask(seed, stream, y.shape, p, y.device) / (1.0 - p)
    return y.to(out_dtype), mean, rstd


def _ln_bwd(dy, xhat, gamma, rstd):
    g = dy * gamma.float()
    H = dy.shape[-1]
    dx = (g - g.mean(-1, keepdim=True) - xhat * (g * xhat).mean(-1, keepdim=True)) * rstd[:, None]
    return dx, (dy * xhat).sum(0), dy.sum(0)


def embed_ln_bwd(dy, ids, word, pos, gamma, mean, rstd, S, p, seed, stream, pad_id,
                 dword, dpos, dgamma, dbeta):
    """Backward of :func:`embed_ln_fwd`; accumulates into ``dword/dpos`` and writes ``dgamma/dbeta``."""
    T = ids.numel()
    flat = ids.reshape(-1).long()
    dy = dy.float()
    if p > 0:
        dy = dy * _mask(seed, stream, dy.shape, p, dy.device) / (1.0 - p)
    x = word[flat].float() + pos[:S].float().repeat(T // S, 1)
    xhat = (x - mean[:, None]) * rstd[:, None]
    dx, dg, db = _ln_bwd(dy, xhat, gamma, rstd)
    dgamma.copy_(dg.to(dgamma.dtype))
    dbeta.copy_(db.to(dbeta.dtype))
    keep = (flat != pad_id)
    acc = torch.zeros(dword.shape, dtype=torch.float32, device=dword.device)
    acc.index_add_(0, flat[keep], dx[keep])
    dword.copy_(acc.to(dword.dtype))
    dp = torch.zeros(dpos.shape, dtype=torch.float32, device=dpos.device)
    dp[:S] = dx.view(T // S, S, -1).sum(0)
    dpos.copy_(dp.to(dpos.dtype))


# ----------------------------------------------------------------------------- attention
def attention_fwd(qkv, bqkv, mask, nh, p, seed, stream):
    """qkv[T,3H] (bias not yet added), mask[b,S] (1 = token).  Returns ``(ctx[T,H], probs)`` where
    probs[b,nh,S,S] are the post-softmax (pre-dropout) weights kept for the backward pass."""
    b, S = mask.shape
    H = qkv.shape[1] // 3
    hd = H // nh
    x = (qkv.float() + bqkv.float()).view(b, S, 3, nh, hd)
    q, k, v = x[:, :, 0].transpose(1, 2), x[:, :, 1].transpose(1, 2), x[:, :, 2].transpose(1, 2)
    s = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(hd)
    s = s.masked_fill(mask[:, None, None, :] == 0, -1e30)
    probs = torch.softmax(s, -1)
    w = probs
    if p > 0:
        w = probs * _mask(seed, stream, probs.shape, p, probs.device) / (1.0 - p)
    ctx = torch.matmul(w, v).transpose(1, 2).reshape(b * S, H)
    return ctx.to(qkv.dtype), probs


def attention_bwd(dctx, qkv, bqkv, mask, probs, nh, p, seed, stream):
    """Returns ``dqkv[T,3H]`` (gradient w.r.t. the biased projections)."""
    b, S = mask.shape
    H = qkv.shape[1] // 3
    hd = H // nh
    x = (qkv.float() + bqkv.float()).view(b, S, 3, nh, hd)
    q, k, v = x[:, :, 0].transpose(1, 2), x[:, :, 1].transpose(1, 2), x[:, :, 2].transpose(1, 2)
    do = dctx.float().view(b, S, nh, hd).transpose(1, 2)
    probs = probs.float()
    if p > 0:
        m = _mask(seed, stream, probs.shape, p, probs.device) / (1.0 - p)
        w = probs * m
    else:
        m, w = None, probs
    dv = torch.matmul(w.transpose(-1, -2), do)
    dw = torch.matmul(do, v.transpose(-1, -2))
    dp = dw * m if m is not None else dw
    ds = probs * (dp - (dp * probs).sum(-1, keepdim=True)) / math.sqrt(hd)
    dq = torch.matmul(ds, k)
    dk = torch.matmul(ds.transpose(-1, -2), q)
    out = torch.stack([dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)], dim=2)
    return out.reshape(b * S, 3 * H).to(qkv.dtype)


# ----------------------------------------------------------------------------- bias+dropout+residual+LN
def bias_dropout_add_ln_fwd(x, bias, resid, gamma, beta, eps, p, seed, stream):
    """``pre = resid + dropout(x + bias)``; ``y = LN(pre)``.  Returns ``(y, pre, mean, rstd)``."""
    t = x.float() + bias.float()
    if p > 0:
        t = t * _mask(seed, stream, t.shape, p, t.device) / (1.0 - p)
    pre = (resid.float() + t).to(x.dtype)
    pf = pre.float()
    mean = pf.mean(-1)
    rstd = torch.rsqrt(pf.var(-1, unbiased=False) + eps)
    y = (pf - mean[:, None]) * rstd[:, None] * gamma.float() + beta.float()
    return y.to(x.dtype), pre, mean, rstd


def bias_dropout_add_ln_bwd(dy, pre, gamma, mean, rstd, p, seed, stream, dgamma, dbeta, dbias):
    """Returns ``(d_pre, d_branch)``: gradient w.r.t. the LN input (= residual stream) and w.r.t. the
    pre-bias branch output ``x``.  Writes ``dgamma, dbeta, dbias``."""
    xhat = (pre.float() - mean[:, None]) * rstd[:, None]
    d_pre, dg, db = _ln_bwd(dy.float(), xhat, gamma, rstd)
    d_branch = d_pre
    if p > 0:
        d_branch = d_pre * _mask(seed, stream, d_pre.shape, p, d_pre.device) / (1.0 - p)
    dgamma.copy_(dg.to(dgamma.dtype))
    dbeta.copy_(db.to(dbeta.dtype))
    d_pre = d_pre.to(dy.dtype)
    d_branch = d_branch.to(dy.dtype)
    dbias.copy_(d_branch.float().sum(0).to(dbias.dtype))
    return d_pre, d_branch


# ----------------------------------------------------------------------------- bias + GELU
def bias_gelu_fwd(x, bias):
    return F.gelu(x.float() + bias.float()).to(x.dtype)


def bias_gelu_bwd(da, x, bias, dbias):
    z = x.float() + bias.float()
    cdf = 0.5 * (1.0 + torch.erf(z / math.sqrt(2.0)))
    pdf = torch.exp(-0.5 * z * z) / math.sqrt(2.0 * math.pi)
    dx = (da.float() * (cdf + z * pdf)).to(x.dtype)
    dbias.copy_(dx.float().sum(0).to(dbias.dtype))
    return dx


def colsum(x, out):
    out.copy_(x.float().sum(0).to(out.dtype))
    return out


# ----------------------------------------------------------------------------- pooling, embedding dropout
def pool_fwd(h, mask, mode):
    """h[b,S,H] → fp32 [b,H]: mask-weighted mean (reference dl_base.py:131-141) or CLS token."""
    if mode == "cls":
        return h[:, 0].float().contiguous()
    m = mask.unsqueeze(-1).float()
    return (h.float() * m).sum(1) / m.sum(1).clamp(min=1e-9)


def pool_bwd(de, mask, mode, S, out_dtype):
    b, H = de.shape
    if mode == "cls":
        dh = torch.zeros(b, S, H, dtype=torch.float32, device=de.device)
        dh[:, 0] = de.float()
        return dh.to(out_dtype)
    m = mask.unsqueeze(-1).float()
    return (de.float()[:, None, :] * m / m.sum(1, keepdim=True).clamp(min=1e-9)).to(out_dtype)


def dropout_cast_fwd(e, p, seed, stream, out_dtype):
    """Classifier-input dropout (reference main.py:149,151) + cast to the classifier dtype."""
    if p > 0:
        e = e.float() * _mask(seed, stream, e.shape, p, e.device) / (1.0 - p)
    return e.to(out_dtype)


def dropout_bwd(dx, p, seed, stream):
    if p > 0:
        return dx.float() * _mask(seed, stream, dx.shape, p, dx.device) / (1.0 - p)
    return dx.float()


# ----------------------------------------------------------------------------- classifier (XFC) step
def xfc_logit_grad(X, W, pos_rows, pos_labels, want_loss=False):
    """``Gt[Ls,B] = sigmoid(W Xᵀ)`` with 1 subtracted at the positives — the gradient of the
    sum-reduced BCE-with-logits w.r.t. the logits, computed without forming the loss
    (reference dl_base.py:590-594).  fp32 accumulation; the result is rounded to X's dtype.
    Optionally returns the sparse loss ``Σ max(z,0) − Σ z[pos] + Σ log(1+exp(−|z|))``
    (dl_base.py:579-583)."""
    Z = W.float() @ X.float().t()                       # [Ls, B]
    loss = None
    if want_loss:
        loss = Z.clamp(min=0).sum() + torch.log1p(torch.exp(-Z.abs())).sum()
        if pos_rows.numel():
            loss = loss - Z[pos_labels.long(), pos_rows.long()].sum()
    Gt = torch.sigmoid(Z)
    if pos_rows.numel():
        Gt[pos_labels.long(), pos_rows.long()] -= 1.0
    return Gt.to(X.dtype), loss


def xfc_dx(Gt, W, scale):
    """``dX[B,D] = scale · Gᵀᵀ · W`` in fp32 (reference dl_base.py:602-608)."""
    return scale * (Gt.float().t() @ W.float())


def xfc_dw_sgd(Gt, X, W, M, lr, mo, wd, dW_acc=None, sr_seed=None):
    """``dW = Gt · X`` then SGD with momentum and L2 weight decay applied in place on ``W``/``M``
    (torch/apex SGD semantics: ``g += wd·W; M = mo·M + g; W -= lr·M``; a zero-initialised ``M``
    makes the first step ``M = g``).  With ``dW_acc`` the gradient is only accumulated."""
    dW = Gt.float() @ X.float()
    if dW_acc is not None:
        dW_acc += dW
        return
    sgd_update(W, M, dW, lr, mo, wd, sr_seed)


def stochastic_round_fp16(x: torch.Tensor, seed: int, stream: int = 0x5152) -> torch.Tensor:
    """fp32 -> fp16 with stochastic rounding, the arithmetic of the dW kernel's epilogue (``sr_half``): add
    13 uniform random bits below the mantissa bits fp16 keeps, then truncate.  Unbiased in fp16's normal range.
    The random bits come from the counter-based hash of the element index."""
    from .rng import mix32
    idx = torch.arange(x.numel(), dtype=torch.int64, device=x.device)
    rnd = mix32(int(seed), stream, idx) & 0x1FFF
    bits = x.float().contiguous().view(torch.int32).view(-1).to(torch.int64) & 0xFFFFFFFF
    bits = ((bits + rnd) & 0xFFFFFFFF) & ~0x1FFF
    bits = torch.where(bits >= 2 ** 31, bits - 2 ** 32, bits).to(torch.int32)
    return bits.view(torch.float32).view(x.shape).to(torch.float16)      # exact: the dropped bits are zero


def sgd_update(W, M, dW, lr, mo, wd, sr_seed=None):
    """``sr_seed``: round the new fp16 weights stochastically (fp16 storage only) instead of to nearest."""
    g = dW.float() + wd * W.float()
    m = mo * M.float() + g
    M.copy_(m.to(M.dtype))
    w = W.float() - lr * M.float()
    if sr_seed is not None and W.dtype == torch.float16:
        W.copy_(stochastic_round_fp16(w, sr_seed))
    else:
        W.copy_(w.to(W.dtype))


def topk_logits(X, W, k):
    """Row-wise top-k of ``X Wᵀ`` → ``(values[B,k] fp32, indices[B,k] int64)``."""
    Z = X.float() @ W.float().t()
    v, i = torch.topk(Z, min(k, Z.shape[1]), dim=1)
    return v, i


# ----------------------------------------------------------------------------- optimizer
def adamw_step(p32, m, v, g, p16, lr, beta1, beta2, eps, wd, n_decay, step, inv_scale, found_inf):
    """Fused AdamW (decoupled decay) over flat buffers with gradient unscaling; skipped entirely when
    ``found_inf`` is set.  Weight decay ``wd`` applies to the first ``n_decay`` elements only (the
    flat buffer is laid out decayed-parameters-first).  ``p16`` receives the low-precision copy used
    by the next forward (may be ``None``)."""
    if float(found_inf) != 0.0:
        return
    gf = g.float() * inv_scale
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (v / bc2).sqrt_().add_(eps)
    p32[:n_decay].mul_(1 - lr * wd)
    p32.addcdiv_(m / bc1, denom, value=-lr)
    if p16 is not None:
        p16.copy_(p32.to(p16.dtype))
